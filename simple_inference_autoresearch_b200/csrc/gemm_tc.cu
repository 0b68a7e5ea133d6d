// bfloat16 matrix products C[M,N] = A[M,K] * W[N,K]^T on the 5th-generation tensor
// cores of sm_100a: operands staged in shared memory by TMA (128-byte swizzle),
// tcgen05.mma issued by one thread with the float32 accumulator in tensor memory,
// tcgen05.ld for the epilogue.  These are the products the reference sends to
// cuBLAS or to its Triton GEMMs (ops/attention.py:139-178,348; ops/mlp.py:179-214;
// ops/embedding.py:123-141).
//
// One kernel serves both orientations, because A and W are both K-major:
//   D[P x Q] = X[P,K] * Y[Q,K]^T,  X rows on the 128-wide MMA M axis, Y rows on N.
//   * many rows (prefill): X = A, Y = W, C[p][q] = D[p][q].
//   * few rows (decode, M <= 128): X = W, Y = A ("swap-AB": the weight fills the
//     128-row axis and the batch sits on the narrow N axis), C[q][p] = D[p][q].
// Few output tiles are cut along K (split-K): the parts of a tile run as one thread-block
// cluster; every block owns a share of the tile's outputs, receives the other blocks'
// float32 partials for them through distributed shared memory, and adds them in rank
// order.  No scratch in global memory, and one order of summation.
//
// Warp roles (192 threads): warp 0 issues TMA loads, warp 1 allocates tensor memory
// and issues the MMAs, warps 2..5 run the epilogue (warp w reads TMEM lanes
// 32*(w%4) .. 32*(w%4)+31).  Every wait on an mbarrier is bounded; when a wait
// expires the block raises a status flag, drains, frees its tensor memory and
// returns (the result of that launch is then invalid and the host raises).
#include "tcgen05.cuh"

#include <unordered_map>

namespace siar {

constexpr int kBM = 128;     // MMA M
constexpr int kBK = 64;      // one 128-byte swizzle row of bf16

// silu(g) * u in 32-bit, the reference's SwiGLU (kernels/swiglu_kernel.py:139-140), here applied to
// the float32 accumulators of the gate/up product before anything is rounded.
__device__ __forceinline__ float swiglu_f(float g, float u) { return g / (1.f + expf(-g)) * u; }


template <typename TOut> __device__ __forceinline__ void store_out(TOut* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

struct GemmParams {
  void* C;            // output, TOut
  int* status;
  int P, Q, K;        // D is P x Q
  int ldc;            // leading dimension of C
  int transpose_out;  // 0: C[p][q], 1: C[q][p]
  int kb_per_split;   // k-blocks of 64 per split
  int x_is_weight;    // X is written by no kernel (swap-AB): its tiles may load before pdl_wait()
  int swiglu;         // weight rows interleaved (gate_j, up_j): write silu(gate) * up, half as many outputs
  // The residual stream inside the products.  With r the float32 residual, w the weight of the
  // RMSNorm that follows and W the weight of the product after it,
  //     (r * rsqrt(mean(r^2) + eps) * w) W^T  =  rsqrt(mean(r^2) + eps) * ((r * w) W^T):
  // the norm's row factor can be applied to the product's rows afterwards.  So
  //  * a product that ends a sublayer (accumulate) adds itself into the residual, C (float32) += D,
  //    and, when rb_out is given, also writes rb_out = bf16(C_new * next_w) [rows, ldc] (the operand
  //    of the next product) and ss_out[row][part] = the sum of squares of C_new over this block's
  //    outputs of the row (ss_parts parts per row, every one written by exactly one block);
  //  * the product that follows (ss_in given) loads rb as an ordinary operand and multiplies each
  //    of its rows by rsqrt(sum(ss_in[row][0..ss_in_parts)) * inv_width + eps) on the accumulators,
  //    before the activation (SwiGLU epilogue) or the store.
  // No norm kernel runs between the two, and nothing but the bf16 operand is rounded.
  int accumulate;
  float* ss_out;
  int ss_parts;
  __nv_bfloat16* rb_out;
  const void* next_w;      // [outputs] norm weight, bfloat16 or (next_w_f32) float32
  int next_w_f32;
  const float* ss_in;
  int ss_in_parts;
  float inv_width;         // 1 / (width of the normed row) = 1 / K
  float eps;
#ifdef SIAR_TIMING
  unsigned long long* stamps;   // [blocks][16] globaltimer marks, for profiling builds only
#endif
};

#ifdef SIAR_TIMING
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Marks of the small kernel, one row of 16 per block: 0 block started, 1 first weight tiles asked for,
// 2 dependency wait returned, 3 first stage landed, 4 accumulator complete, 5 cluster past its first
// barrier, 7 hand-over complete, 10 owners' adding write-out done, 8 tile staged (no split), 9 write-out
// done, 6 block about to leave.
#define SIAR_STAMP(i) \
  if (prm.stamps) prm.stamps[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (i)] = gtime()
#else
#define SIAR_STAMP(i)
#endif

// ------------------------------------------------------------------ kernel
// A load that is issued where it stands: the old values of the outputs are asked for long before the
// sums they are added to exist, and a plain load may be moved down to its first use, where every
// group of outputs would wait a trip to L2 of its own.
__device__ __forceinline__ float ld_f32_here(const float* p) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_f32x4_here(const float* p) {
  float4 v;
  asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
// 32 bytes a thread and instruction (sm_100): a whole sector, where a float4 fills half of one
__device__ __forceinline__ void ld_f32x8_here(const float* p, float4& a, float4& b) {
  asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w), "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w) : "l"(p) : "memory");
}
__device__ __forceinline__ void st_f32x8(float* p, const float4& a, const float4& b) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w), "f"(b.x), "f"(b.y), "f"(b.z), "f"(b.w) : "memory");
}
__device__ __forceinline__ void st_b32x8(void* p, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}
__device__ __forceinline__ float load_norm_w_here(const void* w, int is_f32, long long i) {
  if (is_f32) return ld_f32_here(reinterpret_cast<const float*>(w) + i);
  unsigned short v;
  asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(reinterpret_cast<const __nv_bfloat16*>(w) + i) : "memory");
  return __bfloat162float(__ushort_as_bfloat16(v));
}
__device__ __forceinline__ float load_norm_w(const void* w, int is_f32, long long i) {
  return is_f32 ? reinterpret_cast<const float*>(w)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]);
}
// Eight consecutive norm weights from index i (a multiple of 8; w is 16-byte aligned).
__device__ __forceinline__ void load_norm_w8(const void* w, int is_f32, long long i, float (&out)[8]) {
  if (is_f32) {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
    const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(w) + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      out[2 * e] = f.x; out[2 * e + 1] = f.y;
    }
  }
}

// At most 112 registers per thread (three blocks' worth per SM): a block of this kernel then fits
// on an SM beside two blocks of the decode attention kernel, so it starts, sets up and asks for
// its first weight tiles while the attention in front of it is still running.
template <int BN, int STAGES, typename TOut>
__global__ void __launch_bounds__(192, 3)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY, const GemmParams prm) {
  constexpr uint32_t kXBytes = kBM * kBK * 2;
  constexpr uint32_t kYBytes = BN * kBK * 2;
  constexpr uint32_t kStageBytes = kXBytes + kYBytes;
  constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;
  constexpr int kSsSlots = 64;                     // most columns one block owns when it adds (see below)

  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float ss_red[4][kSsSlots];
  __shared__ float inv_s[BN < 128 ? BN : 128];     // row factors of the norm in front, by tile column (few rows)
  // 16-column tiles split along K: the partials of this block's outputs arrive here from the cluster's
  // blocks (float recv16[sender][owned output][128 tile rows]) and are counted on recv_bar
  __shared__ __align__(16) float recv16[BN == 16 ? 24 * kBM : 4];
  __shared__ __align__(8) uint64_t recv_bar;

  const uint32_t dyn = smem_u32(smem_dyn);
  unsigned char* tiles = smem_dyn + ((1024u - (dyn & 1023u)) & 1023u);   // 1024-byte aligned for the swizzle

  pdl_launch_dependents();
  SIAR_TRACE(10, 0);
  if (threadIdx.x == 0) { SIAR_STAMP(0); }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p0 = blockIdx.x * kBM, q0 = blockIdx.y * BN;
  const int num_kb_total = (prm.K + kBK - 1) / kBK;
  const int kb_begin = blockIdx.z * prm.kb_per_split;
  const int kb_end = min(num_kb_total, kb_begin + prm.kb_per_split);
  const int num_kb = kb_end - kb_begin;
  const int splits = gridDim.z;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    mbar_init(&recv_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // 16-column tiles in a cluster: every block's barrier exists before anyone sends to it (the wait that
  // belongs to this arrival comes just before the hand-over, long after)
  if (BN == 16 && splits > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  // A block that starts after another one has reported an expired wait does no work:
  // a broken launch then ends after one wave instead of one second per block.
  const bool dead = (*(volatile int*)prm.status & kStatusWaitExpired) != 0;
  constexpr int kChunks = (BN + 15) / 16;
  constexpr int LD = BN + 1;                       // padded row of the accumulator stage
  float* stage = reinterpret_cast<float*>(tiles);
  TOut* C = (TOut*)prm.C;
  bool acc_ok = false;      // epilogue threads: the accumulator in tensor memory is complete
  // Adding into C with the weight's rows on the tile's rows: the values of C this thread adds to and the
  // next norm's weights of its outputs (asked for at the start of the epilogue).
  float old_c[16];
  float nw4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 16; ++j) old_c[j] = 0.f;
  // As a cluster a block owns, of the tile's BN columns (rows of the activations), column jq when
  // jq % splits == rank (16-column tiles) or the groups of four columns gq with gq % splits == rank
  // (wider tiles).  owned_row(j, first) is the row of C behind the j-th owned column counted from
  // `first` (in columns, or in columns of whole groups), or -1 when there is none.
  auto owned_row = [&](int j, int first) -> int {
    const int rank = (int)blockIdx.z;
    int jq;
    if (BN == 16) {
      jq = (first + j) * splits + rank;
    } else {
      const int gq = (first / 4 + (j >> 2)) * splits + rank;
      jq = gq < BN / 4 ? 4 * gq + (j & 3) : BN;
    }
    return jq < BN && q0 + jq < prm.Q ? q0 + jq : -1;
  };
  // whole float4 / four-bfloat16 accesses along the outputs of one row of C
  const bool acc_vec = sizeof(TOut) == 4 && prm.ldc % 4 == 0 && (reinterpret_cast<uintptr_t>(C) % 16) == 0 &&
                       (reinterpret_cast<uintptr_t>(prm.rb_out) % 8) == 0 &&
                       p0 + 4 * ((int)(threadIdx.x & 31)) + 3 < prm.P;
  float inv_row = 1.f;      // the norm's factor of this thread's tile row (many rows on the tile's rows)
  const bool scaled = prm.ss_in != nullptr;

  {
  if (dead) {
    // fall through to the write-out barriers and the teardown
  } else if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmY) : "memory");
      int issued = 0;
      // Weights do not depend on earlier kernels: the first STAGES tiles of the weight operand
      // are requested before this grid waits for its predecessors.
      // x_is_weight: 1 the X operand is the weight, 2 the Y operand is (the many-row orientation)
      const int pre = prm.x_is_weight ? min(STAGES, num_kb) : 0;
      const bool y_first = prm.x_is_weight == 2;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], kStageBytes);
        if (y_first)
          tma_load_2d(tiles + (size_t)i * kStageBytes + kXBytes, &tmY, &full_bar[i], (kb_begin + i) * kBK, q0);
        else
          tma_load_2d(tiles + (size_t)i * kStageBytes, &tmX, &full_bar[i], (kb_begin + i) * kBK, p0);
      }
      SIAR_STAMP(1);
      pdl_wait();
      SIAR_TRACE(10, 2);
      SIAR_STAMP(2);
      if (y_first) {
        for (int i = 0; i < pre; ++i)
          tma_load_2d(tiles + (size_t)i * kStageBytes, &tmX, &full_bar[i], (kb_begin + i) * kBK, p0);
      } else {
        for (int i = 0; i < pre; ++i)
          tma_load_2d(tiles + (size_t)i * kStageBytes + kXBytes, &tmY, &full_bar[i], (kb_begin + i) * kBK, q0);
      }
      issued = pre;
      for (int i = pre; i < num_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1) || *(volatile int*)&abort_flag) {
          abort_flag = 1;
          atomicOr(prm.status, kStatusWaitExpired);
          break;
        }
        unsigned char* xs = tiles + (size_t)s * kStageBytes;
        mbar_expect_tx(&full_bar[s], kStageBytes);
        tma_load_2d(xs, &tmX, &full_bar[s], (kb_begin + i) * kBK, p0);
        tma_load_2d(xs + kXBytes, &tmY, &full_bar[s], (kb_begin + i) * kBK, q0);
        issued = i + 1;
      }
      if (*(volatile int*)&abort_flag) {
        // let the copies that are still in flight land before the block leaves
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(BN < 16 ? 16 : BN);
      bool ok = true;
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph) || *(volatile int*)&abort_flag) { ok = false; break; }
        if (i == 0) { SIAR_STAMP(3); }
        tc_fence_after();
        const uint32_t xs = smem_u32(tiles + (size_t)s * kStageBytes);
        const uint64_t da = smem_desc_sw128(xs), db = smem_desc_sw128(xs + kXBytes);
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          // advancing 16 elements along K inside the swizzled row = 32 bytes = 2 descriptor units
          umma_f16(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
      }
      if (!ok) {
        abort_flag = 1;
        atomicOr(prm.status, kStatusWaitExpired);
      }
      umma_commit(&tmem_full_bar);    // accumulator complete (or abandoned)
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> shared-memory stage
    const int quad = warp & 3;
    const int et = (int)threadIdx.x - 64;
    pdl_wait();   // C may still be read by an earlier kernel; ss_in is written by the product in front
    bool ok = true;
    if (scaled) {
      // the factors of the norm in front: one per row of the activations, which are the tile's
      // columns (few rows, transposed output) or its rows; the parts are added in their own order
      if (prm.transpose_out) {
        if (et < BN && et < 128) {
          const int q = q0 + et;
          float ss = 0.f;
          if (q < prm.Q)
            for (int t = 0; t < prm.ss_in_parts; ++t) ss += prm.ss_in[(size_t)q * prm.ss_in_parts + t];
          inv_s[et] = rsqrtf(ss * prm.inv_width + prm.eps);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      } else {
        const int pp = p0 + et;
        float ss = 0.f;
        if (pp < prm.P)
          for (int t = 0; t < prm.ss_in_parts; ++t) ss += prm.ss_in[(size_t)pp * prm.ss_in_parts + t];
        inv_row = rsqrtf(ss * prm.inv_width + prm.eps);
      }
    }
    if constexpr (sizeof(TOut) == 4) {
      // Adding into C with the weight's rows on the tile's rows: what the write-out adds to is asked for
      // now, long before the sums exist, and so is the next norm's weight.  Without a split a thread
      // writes tile row et of every column; as a cluster it writes tile rows 4 lane .. 4 lane + 3 of the
      // owned columns ew, ew + 4, ... (ew = its warp among the four), see the write-out.
      if (prm.accumulate && prm.transpose_out) {
        const float* Cf = reinterpret_cast<const float*>(C);
        if (splits == 1) {
          if constexpr (BN == 16) {
            const int pp = p0 + et;
            if (prm.rb_out != nullptr && pp < prm.P) nw4[0] = load_norm_w_here(prm.next_w, prm.next_w_f32, pp);
#pragma unroll
            for (int j = 0; j < 16; ++j)
              old_c[j] = (q0 + j < prm.Q && pp < prm.P) ? ld_f32_here(Cf + (long long)(q0 + j) * prm.ldc + pp) : 0.f;
          }
        } else {
          const int ew = et >> 5, pp4 = p0 + 4 * (et & 31);
          if (prm.rb_out != nullptr) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (pp4 + i < prm.P) nw4[i] = load_norm_w_here(prm.next_w, prm.next_w_f32, pp4 + i);
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int q = owned_row(ew + 4 * k, 0);
            if (q < 0) continue;
            const float* src = Cf + (long long)q * prm.ldc + pp4;
            if (acc_vec) {
              const float4 o = ld_f32x4_here(src);
              old_c[4 * k] = o.x; old_c[4 * k + 1] = o.y; old_c[4 * k + 2] = o.z; old_c[4 * k + 3] = o.w;
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (pp4 + i < prm.P) old_c[4 * k + i] = ld_f32_here(src + i);
            }
          }
        }
      }
    }
    if (num_kb > 0) {
      ok = mbar_wait(&tmem_full_bar, 0) && ok;
      if (!ok) { abort_flag = 1; atomicOr(prm.status, kStatusWaitExpired); }
    }
    tc_fence_after();
    if (threadIdx.x == 64) { SIAR_STAMP(4); }
    ok = ok && !*(volatile int*)&abort_flag;
    // Without split-K the accumulator tile goes to the (now idle) pipeline memory, one padded
    // float row per tile row, so that it can be written out in whole row segments.
    if (splits == 1) {
      const int tr = quad * 32 + lane;
#pragma unroll 1
      for (int ch = 0; ch < kChunks; ++ch) {
        uint32_t r[16];
        if (num_kb > 0 && ok) {
          SIAR_TMEM_LD_16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ch * 16), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0u;
        }
        if (scaled) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            r[j] = __float_as_uint(__uint_as_float(r[j]) * (prm.transpose_out ? inv_s[(ch * 16 + j) & 127] : inv_row));
        }
        if (BN >= 32 && prm.transpose_out) {
          // wide tiles are staged column by column (stage[column][tile row]): a warp writes 32
          // consecutive words, and the write-out reads four tile rows of a column as one float4
#pragma unroll
          for (int j = 0; j < 16; ++j) stage[(ch * 16 + j) * kBM + tr] = __uint_as_float(r[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) stage[tr * LD + ch * 16 + j] = __uint_as_float(r[j]);
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) { SIAR_STAMP(8); }
    }
    acc_ok = ok;
  }
  }  // roles

  // ---------------- write-out
  if (splits > 1) {
    // split-K: the blocks of a cluster hold partial tiles of the same outputs.  Output jq of
    // the tile belongs to the block of rank jq % splits.  Each block sends its partials to their owners
    // (remote shared-memory stores into slot [sender rank]); each owner adds them in rank order, so the
    // sum has one order, and stores.
    // Wide tiles receive in the pipeline's memory: barrier 1, every block's main loop is done and its
    // memory free; the stores; barrier 2, all partials have arrived.
    // 16-column tiles (the decode step's products) receive in a buffer of their own and count the
    // arriving bytes on an mbarrier (st.async), so no block waits for the slowest block's main loop
    // before it sends, nor for all hand-overs before it adds: the only cluster barrier left is the
    // one that keeps a block alive until nobody can send to it any more, and its wait comes last.
    // (Measured and not kept: the same for wide tiles, 16-byte st.async behind barrier 1 instead of plain
    // remote stores and barrier 2.  From barrier 1 to the last partial's arrival it took 3.9 us instead
    // of 2.3-3.5 us at 64 rows, and a decode step at batch 64 was 0.3% slower.)
    const int rank = (int)blockIdx.z;
    const int NL = (BN + splits - 1) / splits;          // outputs per owner
    const int et = threadIdx.x - 64;                    // epilogue thread = tile row p
    constexpr bool kAsync = BN == 16;
    if (kAsync) {
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");     // of the arrival at the start
      if (threadIdx.x == 64) {
        const int owned = (BN - rank + splits - 1) / splits;                     // outputs jq = rank, rank + splits, ...
        mbar_expect_tx(&recv_bar, (uint32_t)(owned * splits * kBM * 4));
      }
    } else {
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (threadIdx.x == 64) { SIAR_STAMP(5); }
    const uint32_t recv = kAsync ? smem_u32(recv16) : smem_u32(tiles);          // float recv[splits][NL][128]
    // Tiles of 32 and more columns hand over groups of four columns: group gq belongs to rank
    // gq % splits, and a thread sends a group as one 16-byte remote store
    // (float4 recv[sender][group slot][128 tile rows]).
    constexpr int kGroups = BN / 4;
    const int NLg = (kGroups + splits - 1) / splits;    // groups per owner
    if constexpr (BN >= 32) {
      if (warp >= 2) {
        const int quad = warp & 3;
        const int tr = quad * 32 + lane;
        int push_owner = 0, push_gl = 0;
#pragma unroll 1
        for (int ch = 0; ch < BN / 32; ++ch) {
          uint32_t r[32];
          if (num_kb > 0 && acc_ok) {
            SIAR_TMEM_LD_32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ch * 32), r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          if (scaled) {       // every block scales its own partials: the factor is the row's, not the split's
#pragma unroll
            for (int j = 0; j < 32; ++j)
              r[j] = __float_as_uint(__uint_as_float(r[j]) * (prm.transpose_out ? inv_s[(ch * 32 + j) & 127] : inv_row));
          }
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4) {
            const uint32_t local = recv + (uint32_t)(((rank * NLg + push_gl) * 128 + tr) * 16);
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(push_owner));
            asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "r"(r[4 * g4]),
                         "r"(r[4 * g4 + 1]), "r"(r[4 * g4 + 2]), "r"(r[4 * g4 + 3])
                         : "memory");
            if (++push_owner == splits) { push_owner = 0; ++push_gl; }
          }
        }
      }
    } else if (warp >= 2) {
      const int quad = warp & 3;
      const int tr = quad * 32 + lane;                  // the tile row this thread reads from TMEM
      int push_owner = 0, push_jl = 0;
#pragma unroll 1
      for (int ch = 0; ch < kChunks; ++ch) {
        uint32_t r[16];
        if (num_kb > 0 && acc_ok) {
          SIAR_TMEM_LD_16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ch * 16), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0u;
        }
        if (scaled) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            r[j] = __float_as_uint(__uint_as_float(r[j]) * (prm.transpose_out ? inv_s[(ch * 16 + j) & 127] : inv_row));
        }
        // output jq goes to rank jq % splits, slot jq / splits: both kept as running counters
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (ch * 16 + j < BN) {
            const uint32_t local = recv + (uint32_t)(((rank * NL + push_jl) * 128 + tr) * 4);
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(push_owner));
            if (kAsync) {
              uint32_t remote_bar;
              asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(smem_u32(&recv_bar)), "r"(push_owner));
              asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.u32 [%0], %1, [%2];"
                           ::"r"(remote), "r"(r[j]), "r"(remote_bar) : "memory");
            } else {
              asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(r[j]) : "memory");
            }
            if (++push_owner == splits) { push_owner = 0; ++push_jl; }
          }
        }
      }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    if (kAsync) {
      // this block's outputs are complete when all their bytes have been counted
      if (warp >= 2 && !dead && !mbar_wait(&recv_bar, 0)) {
        abort_flag = 1;
        atomicOr(prm.status, kStatusWaitExpired);
      }
    } else {
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (threadIdx.x == 64) { SIAR_STAMP(7); }
    if (warp >= 2 && !dead) {
      const int pp = p0 + et;
      const int ew = et >> 5;
      const float* mine = kAsync ? recv16 : reinterpret_cast<const float*>(tiles);
      bool stored = false;
      // Adding into C as a cluster, the weight's rows on the tile's rows.  Taken one output after the
      // other by the thread of its tile row (two narrow stores and a warp reduction each, four warps on
      // the SM and nothing else to issue meanwhile) the write-out of 16 outputs a thread took 6 us at 64
      // rows.  So the sums over the ranks go through shared memory once more, transposed
      // (sums[column][tile row]), and warp ew writes the owned columns ew, ew + 4, ...: a lane adds four
      // consecutive outputs of a row of C to their old values (asked for at the start of the epilogue),
      // stores them as one float4 and their bf16(r * w) as one 8-byte word, and the warp's sum of
      // squares is the column's whole share of this tile, which lane 0 writes.
      if constexpr (sizeof(TOut) == 4) {
        if (prm.accumulate && prm.transpose_out) {
          stored = true;
          float* Cf = reinterpret_cast<float*>(C);
          const int pp4 = p0 + 4 * lane;
          // `first`: the pass's first owned column; `sums`: [columns of the pass][128 tile rows]
          auto write_pass = [&](int first, const float* sums, const float (&old)[16]) {
            float ssq[4] = {0.f, 0.f, 0.f, 0.f};
            int qk[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              qk[k] = owned_row(ew + 4 * k, first);
              if (qk[k] < 0) continue;
              const float4 v = *reinterpret_cast<const float4*>(sums + (ew + 4 * k) * kBM + 4 * lane);
              const float r[4] = {old[4 * k] + v.x, old[4 * k + 1] + v.y, old[4 * k + 2] + v.z, old[4 * k + 3] + v.w};
              const long long at = (long long)qk[k] * prm.ldc + pp4;
              if (acc_vec) {
                *reinterpret_cast<float4*>(Cf + at) = make_float4(r[0], r[1], r[2], r[3]);
                if (prm.rb_out != nullptr) {
                  uint2 pk;
                  pk.x = pack_bf16x2(r[0] * nw4[0], r[1] * nw4[1]);
                  pk.y = pack_bf16x2(r[2] * nw4[2], r[3] * nw4[3]);
                  *reinterpret_cast<uint2*>(prm.rb_out + at) = pk;
                }
                ssq[k] = (r[0] * r[0] + r[1] * r[1]) + (r[2] * r[2] + r[3] * r[3]);
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  if (pp4 + i >= prm.P) break;
                  Cf[at + i] = r[i];
                  if (prm.rb_out != nullptr) prm.rb_out[at + i] = __float2bfloat16_rn(r[i] * nw4[i]);
                  ssq[k] += r[i] * r[i];
                }
              }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
              for (int k = 0; k < 4; ++k) ssq[k] += __shfl_xor_sync(0xffffffffu, ssq[k], o);
            }
            if (lane == 0 && prm.ss_out != nullptr) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                if (qk[k] >= 0) prm.ss_out[(size_t)qk[k] * prm.ss_parts + blockIdx.x] = ssq[k];
            }
          };
          if constexpr (BN == 16) {
            // NL <= 8 owned columns (16 over at least 2 ranks); the pipeline's memory is idle by now
            float* sums = reinterpret_cast<float*>(tiles);
            float r8[8];
#pragma unroll
            for (int jl = 0; jl < 8; ++jl) r8[jl] = 0.f;
            for (int z = 0; z < splits; ++z) {
#pragma unroll
              for (int jl = 0; jl < 8; ++jl)
                if (jl < NL) r8[jl] += mine[(z * NL + jl) * 128 + et];
            }
#pragma unroll
            for (int jl = 0; jl < 8; ++jl)
              if (jl < NL) sums[jl * kBM + et] = r8[jl];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            write_pass(0, sums, old_c);
          } else {
            // four owned groups (16 columns) a pass; the sums stand behind the ranks' partials
            const float4* mine4 = reinterpret_cast<const float4*>(tiles);
            float* sums = reinterpret_cast<float*>(tiles) + (size_t)splits * NLg * 128 * 4;
            static_assert((BN / 4 + 7) * 2048 + 16 * kBM * 4 <= STAGES * (int)kStageBytes, "partials and sums fit the pipeline's memory");
            for (int gl0 = 0; gl0 < NLg; gl0 += 4) {
              float old[16];
              if (gl0 > 0) {
                asm volatile("bar.sync 1, 128;" ::: "memory");       // the pass before has read its sums
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const int q = owned_row(ew + 4 * k, 4 * gl0);
#pragma unroll
                  for (int i = 0; i < 4; ++i)
                    old[4 * k + i] = (q >= 0 && pp4 + i < prm.P) ? ld_f32_here(Cf + (long long)q * prm.ldc + pp4 + i) : 0.f;
                }
              }
              float4 acc[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int z = 0; z < splits; ++z) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  if (gl0 + u >= NLg) continue;
                  const float4 v = mine4[(z * NLg + gl0 + u) * 128 + et];
                  acc[u].x += v.x; acc[u].y += v.y; acc[u].z += v.z; acc[u].w += v.w;
                }
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                if (gl0 + u >= NLg) continue;
                sums[(4 * u) * kBM + et] = acc[u].x;
                sums[(4 * u + 1) * kBM + et] = acc[u].y;
                sums[(4 * u + 2) * kBM + et] = acc[u].z;
                sums[(4 * u + 3) * kBM + et] = acc[u].w;
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (gl0 == 0) write_pass(0, sums, old_c); else write_pass(4 * gl0, sums, old);
            }
          }
        }
      }
      if (threadIdx.x == 64) { SIAR_STAMP(10); }
      if constexpr (BN >= 32) {
        const float4* mine4 = reinterpret_cast<const float4*>(tiles);
        // Adding into the residual in the plain orientation: the old values of four groups are asked
        // for at once (one trip to L2 for four groups instead of one trip each, in a row of them).
        bool batched = false;
        if constexpr (sizeof(TOut) == 4) {
          if (!stored && prm.accumulate && !prm.transpose_out && pp < prm.P && prm.ldc % 4 == 0 &&
              (reinterpret_cast<uintptr_t>(C) % 16) == 0) {
            batched = true;
            float* crow = reinterpret_cast<float*>(C) + (long long)pp * prm.ldc + q0;
            __nv_bfloat16* rbrow = prm.rb_out != nullptr ? prm.rb_out + (long long)pp * prm.ldc + q0 : nullptr;
            float ss_acc = 0.f;
            for (int gl0 = 0; gl0 < NLg; gl0 += 4) {
              float4 old[4];
              bool ok[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int gq = (gl0 + u) * splits + rank;
                ok[u] = gl0 + u < NLg && gq < kGroups && q0 + 4 * gq + 3 < prm.Q;
                if (ok[u]) old[u] = *reinterpret_cast<const float4*>(crow + 4 * gq);
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                if (!ok[u]) continue;
                const int gl = gl0 + u, gq = gl * splits + rank;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int z = 0; z < splits; ++z) {
                  const float4 v = mine4[(z * NLg + gl) * 128 + et];
                  acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                acc.x += old[u].x; acc.y += old[u].y; acc.z += old[u].z; acc.w += old[u].w;
                *reinterpret_cast<float4*>(crow + 4 * gq) = acc;
                ss_acc += (acc.x * acc.x + acc.y * acc.y) + (acc.z * acc.z + acc.w * acc.w);
                if (rbrow != nullptr) {
                  const long long f = q0 + 4 * gq;
                  uint2 pk;
                  pk.x = pack_bf16x2(acc.x * load_norm_w(prm.next_w, prm.next_w_f32, f),
                                     acc.y * load_norm_w(prm.next_w, prm.next_w_f32, f + 1));
                  pk.y = pack_bf16x2(acc.z * load_norm_w(prm.next_w, prm.next_w_f32, f + 2),
                                     acc.w * load_norm_w(prm.next_w, prm.next_w_f32, f + 3));
                  *reinterpret_cast<uint2*>(rbrow + 4 * gq) = pk;
                }
              }
            }
            // this block's share of the row's sum of squares (the launcher only asks for it when every
            // group is whole, so nothing is left to the loop below)
            if (prm.ss_out != nullptr) prm.ss_out[(size_t)pp * prm.ss_parts + blockIdx.y * splits + rank] = ss_acc;
          }
        }
        for (int gl = 0; gl < NLg && !stored; ++gl) {
          const int gq = gl * splits + rank;
          if (gq >= kGroups || q0 + 4 * gq >= prm.Q) break;
          if (batched && q0 + 4 * gq + 3 < prm.Q) continue;      // done above
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int z = 0; z < splits; ++z) {
            const float4 v = mine4[(z * NLg + gl) * 128 + et];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
          if (pp < prm.P && !prm.transpose_out) {
            // rows of A on the tile's rows (prompts of a few hundred tokens): the group is four
            // consecutive outputs of row pp; `accumulate` adds them into the float32 residual
            const int q = q0 + 4 * gq;
            TOut* dst = C + (long long)pp * prm.ldc + q;
            const bool whole = q + 3 < prm.Q && prm.ldc % 4 == 0 && (reinterpret_cast<uintptr_t>(C) % 16) == 0;
            if constexpr (sizeof(TOut) == 4) {
              if (prm.accumulate) {
                if (whole) {
                  const float4 o = *reinterpret_cast<const float4*>(dst);
                  acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
                } else {
                  acc.x += reinterpret_cast<const float*>(dst)[0];
                  if (q + 1 < prm.Q) acc.y += reinterpret_cast<const float*>(dst)[1];
                  if (q + 2 < prm.Q) acc.z += reinterpret_cast<const float*>(dst)[2];
                  if (q + 3 < prm.Q) acc.w += reinterpret_cast<const float*>(dst)[3];
                }
              }
              if (whole) *reinterpret_cast<float4*>(dst) = acc;
            } else {
              if (whole) {
                uint2 pk;
                pk.x = pack_bf16x2(acc.x, acc.y);
                pk.y = pack_bf16x2(acc.z, acc.w);
                *reinterpret_cast<uint2*>(dst) = pk;
              }
            }
            if (!whole) {
              store_out<TOut>(dst, acc.x);
              if (q + 1 < prm.Q) store_out<TOut>(dst + 1, acc.y);
              if (q + 2 < prm.Q) store_out<TOut>(dst + 2, acc.z);
              if (q + 3 < prm.Q) store_out<TOut>(dst + 3, acc.w);
            }
          } else if (pp < prm.P) {
            const int q = q0 + 4 * gq;
            TOut* dst = C + (long long)q * prm.ldc + pp;
            store_out<TOut>(dst, acc.x);
            if (q + 1 < prm.Q) store_out<TOut>(dst + prm.ldc, acc.y);
            if (q + 2 < prm.Q) store_out<TOut>(dst + 2 * (long long)prm.ldc, acc.z);
            if (q + 3 < prm.Q) store_out<TOut>(dst + 3 * (long long)prm.ldc, acc.w);
          }
        }
        stored = true;
      }
      for (int jl = 0; jl < NL && !stored; ++jl) {
        const int jq = jl * splits + rank;
        const int q = q0 + jq;
        if (jq >= BN || q >= prm.Q) break;
        float acc = 0.f;
        for (int z = 0; z < splits; ++z) acc += mine[(z * NL + jl) * 128 + et];
        if (pp < prm.P) store_out<TOut>(C + (long long)q * prm.ldc + pp, acc);
      }
    }
  } else if (warp >= 2 && !dead) {
    const int et = threadIdx.x - 64;          // 0..127
    const int ew = et >> 5;
    if (BN >= 32 && prm.transpose_out) {
      // wide tiles: warp ew takes columns ew, ew + 4, ...; a lane holds four consecutive tile rows
      // of the column, which are four (or, as two (gate, up) pairs, two) consecutive outputs
      const int cols = min(BN, prm.Q - q0);
      const int pp = p0 + 4 * lane;
      const bool vec_ok = prm.ldc % 4 == 0 && (reinterpret_cast<uintptr_t>(C) % 16) == 0 && pp + 3 < prm.P;
      for (int jq = ew; jq < cols; jq += 4) {
        const float4 v = *reinterpret_cast<const float4*>(stage + jq * kBM + 4 * lane);
        if (prm.swiglu) {
          TOut* dst = C + (long long)(q0 + jq) * prm.ldc + (pp >> 1);
          const float o0 = swiglu_f(v.x, v.y), o1 = swiglu_f(v.z, v.w);
          if (sizeof(TOut) == 2 && vec_ok) {
            *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(o0, o1);
          } else {
            if (pp + 1 < prm.P) store_out<TOut>(dst, o0);
            if (pp + 3 < prm.P) store_out<TOut>(dst + 1, o1);
          }
        } else {
          TOut* dst = C + (long long)(q0 + jq) * prm.ldc + pp;
          if (vec_ok) {
            if constexpr (sizeof(TOut) == 4) {
              *reinterpret_cast<float4*>(dst) = v;
            } else {
              uint2 pk;
              pk.x = pack_bf16x2(v.x, v.y);
              pk.y = pack_bf16x2(v.z, v.w);
              *reinterpret_cast<uint2*>(dst) = pk;
            }
          } else {
            if (pp < prm.P) store_out<TOut>(dst, v.x);
            if (pp + 1 < prm.P) store_out<TOut>(dst + 1, v.y);
            if (pp + 2 < prm.P) store_out<TOut>(dst + 2, v.z);
            if (pp + 3 < prm.P) store_out<TOut>(dst + 3, v.w);
          }
        }
      }
    } else if (prm.transpose_out && prm.swiglu) {
      // tile rows are weight rows (gate_j, up_j, gate_j+1, ...): even rows write silu(gate) * up
      const int pp = p0 + et;
      if ((et & 1) == 0 && pp + 1 < prm.P) {
        const int cols = min(BN, prm.Q - q0);
        for (int jq = 0; jq < cols; ++jq)
          store_out<TOut>(C + (long long)(q0 + jq) * prm.ldc + (pp >> 1),
                          swiglu_f(stage[et * LD + jq], stage[(et + 1) * LD + jq]));
      }
    } else if (prm.transpose_out) {
      // C[q][p]: for a fixed q the 128 tile rows are contiguous
      const int pp = p0 + et;
      const int cols = min(BN, prm.Q - q0);
      bool stored = false;
      if constexpr (BN == 16 && sizeof(TOut) == 4) {
        if (prm.accumulate) {
          const float nw = nw4[0];
#pragma unroll
          for (int jq = 0; jq < 16; ++jq) {
            if (jq >= cols) break;
            float r = 0.f;
            if (pp < prm.P) {
              r = old_c[jq] + stage[et * LD + jq];
              reinterpret_cast<float*>(C)[(long long)(q0 + jq) * prm.ldc + pp] = r;
              if (prm.rb_out != nullptr) prm.rb_out[(long long)(q0 + jq) * prm.ldc + pp] = __float2bfloat16_rn(r * nw);
            }
            const float v = warp_sum(r * r);
            if (lane == 0) ss_red[ew][jq] = v;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (prm.ss_out != nullptr && et < cols)
            prm.ss_out[(size_t)(q0 + et) * prm.ss_parts + blockIdx.x] =
                (ss_red[0][et] + ss_red[1][et]) + (ss_red[2][et] + ss_red[3][et]);
          stored = true;
        }
      }
      if (!stored && pp < prm.P) {
        for (int jq = 0; jq < cols; ++jq)
          store_out<TOut>(C + (long long)(q0 + jq) * prm.ldc + pp, stage[et * LD + jq]);
      }
    } else {
      const int cols = min(BN, prm.Q - q0);
      constexpr int VEC = 4;                    // elements per lane and pass
      const bool vec_ok = (prm.ldc % VEC == 0) && (cols % VEC == 0) &&
                          ((reinterpret_cast<uintptr_t>(C) % 16) == 0);
      for (int rr = ew; rr < kBM; rr += 4) {
        const int pp = p0 + rr;
        if (pp >= prm.P) break;
        const float* src = stage + rr * LD;
        TOut* dst = C + (long long)pp * prm.ldc + q0;
        if (vec_ok) {
          for (int c4 = lane * VEC; c4 < cols; c4 += 32 * VEC) {
            const float v0 = src[c4], v1 = src[c4 + 1], v2 = src[c4 + 2], v3 = src[c4 + 3];
            if constexpr (sizeof(TOut) == 4) {
              *reinterpret_cast<float4*>(dst + c4) = make_float4(v0, v1, v2, v3);
            } else {
              __nv_bfloat162 lo = __floats2bfloat162_rn(v0, v1), hi = __floats2bfloat162_rn(v2, v3);
              uint2 pk;
              pk.x = *reinterpret_cast<uint32_t*>(&lo);
              pk.y = *reinterpret_cast<uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(dst + c4) = pk;
            }
          }
        } else {
          for (int c1 = lane; c1 < cols; c1 += 32) store_out<TOut>(dst + c1, src[c1]);
        }
      }
    }
  }
  if (threadIdx.x == 64) { SIAR_STAMP(9); }
  // a block of 16-column tiles in a cluster stays until every block has sent what it had to send
  if (BN == 16 && splits > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  SIAR_TRACE(10, 1);
  if (threadIdx.x == 0) { SIAR_STAMP(6); }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}


// The factor of the norm in front of a product for row p of its activations (1 without such a norm):
// the parts of the row's sum of squares are added in their own order, whatever block wrote them.
__device__ __forceinline__ float norm_row_factor(const GemmParams& prm, int p) {
  if (prm.ss_in == nullptr || p >= prm.P) return 1.f;
  float ss = 0.f;
  for (int t = 0; t < prm.ss_in_parts; ++t) ss += prm.ss_in[(size_t)p * prm.ss_in_parts + t];
  return rsqrtf(ss * prm.inv_width + prm.eps);
}

// 32 consecutive accumulators of tile row p (columns q .. q + 31) to C: plain, added into C
// (accumulate), or as 16 silu(gate) * up values (swiglu).  With ss_in the accumulators are first
// multiplied by row_scale, the factor of the norm in front of this product for row p.  An
// accumulating product with rb_out also writes bf16(new C * next_w) to rbrow and returns the sum
// of squares of the new C values it stored (0 otherwise).
// What an accumulating chunk adds to and multiplies by, asked for one chunk ahead: the 32 old values of
// C and (for rb_out with bfloat16 norm weights) the 32 weights of the next norm.
struct ChunkAhead {
  float4 old[8];
  uint4 w[4];
  bool have;      // the values above are those of this chunk
};
template <typename TOut>
__device__ __forceinline__ void fetch_ahead(ChunkAhead& a, const TOut* crow, const __nv_bfloat16* rbrow, int p, int q,
                                            const GemmParams& prm, bool vec_ok) {
  a.have = false;
  if constexpr (sizeof(TOut) == 4) {
    if (prm.accumulate && !prm.swiglu && vec_ok && p < prm.P && q + 32 <= prm.Q) {
      a.have = true;
      const float* src = reinterpret_cast<const float*>(crow) + q;
      if ((reinterpret_cast<uintptr_t>(src) & 31) == 0) {
#pragma unroll
        for (int j = 0; j < 8; j += 2) ld_f32x8_here(src + 4 * j, a.old[j], a.old[j + 1]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) a.old[j] = ld_f32x4_here(src + 4 * j);
      }
      if (rbrow != nullptr && !prm.next_w_f32) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 v = ld_f32x4_here(reinterpret_cast<const float*>(reinterpret_cast<const __nv_bfloat16*>(prm.next_w) + q + 8 * j));
          a.w[j] = make_uint4(__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w));
        }
      }
    }
  }
}
template <typename TOut>
__device__ __forceinline__ float store_chunk(uint32_t (&r)[32], TOut* crow, __nv_bfloat16* rbrow, int p, int q,
                                             const GemmParams& prm, bool vec_ok, float row_scale,
                                             const ChunkAhead* ahead = nullptr) {
  float ss = 0.f;
  if (prm.ss_in != nullptr) {
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * row_scale);
  }
  if (prm.swiglu) {
    // columns are (gate_j, up_j) pairs: 16 outputs from these 32 accumulators
    if (p < prm.P && q < prm.Q) {
      TOut* orow = crow + (q >> 1);
      if (vec_ok && q + 32 <= prm.Q && sizeof(TOut) == 2) {
        const bool wide = (reinterpret_cast<uintptr_t>(orow) & 31) == 0;
        uint4 keep_pk = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int j = 0; j < 32; j += 16) {
          uint4 pk;
          pk.x = pack_bf16x2(swiglu_f(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                             swiglu_f(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])));
          pk.y = pack_bf16x2(swiglu_f(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])),
                             swiglu_f(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
          pk.z = pack_bf16x2(swiglu_f(__uint_as_float(r[j + 8]), __uint_as_float(r[j + 9])),
                             swiglu_f(__uint_as_float(r[j + 10]), __uint_as_float(r[j + 11])));
          pk.w = pack_bf16x2(swiglu_f(__uint_as_float(r[j + 12]), __uint_as_float(r[j + 13])),
                             swiglu_f(__uint_as_float(r[j + 14]), __uint_as_float(r[j + 15])));
          if (!wide) *reinterpret_cast<uint4*>(orow + (j >> 1)) = pk;
          else if (j) st_b32x8(orow, keep_pk, pk);
          keep_pk = pk;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          if (q + j + 1 < prm.Q)
            store_out<TOut>(orow + (j >> 1), swiglu_f(__uint_as_float(r[j]), __uint_as_float(r[j + 1])));
      }
    }
  } else if (p < prm.P && q < prm.Q) {
    if (vec_ok && q + 32 <= prm.Q) {
      if constexpr (sizeof(TOut) == 4) {
        if (prm.accumulate) {          // C += D: the product adds itself into the residual stream
          float4 old[8];
          const bool got = ahead != nullptr && ahead->have;
#pragma unroll
          for (int j = 0; j < 8; ++j) old[j] = got ? ahead->old[j] : *reinterpret_cast<const float4*>(crow + q + 4 * j);
          const bool wide = (reinterpret_cast<uintptr_t>(crow + q) & 31) == 0;
          float4 keep = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 v = make_float4(old[j].x + __uint_as_float(r[4 * j]), old[j].y + __uint_as_float(r[4 * j + 1]),
                                         old[j].z + __uint_as_float(r[4 * j + 2]), old[j].w + __uint_as_float(r[4 * j + 3]));
            if (!wide) *reinterpret_cast<float4*>(crow + q + 4 * j) = v;
            else if (j & 1) st_f32x8(reinterpret_cast<float*>(crow) + q + 4 * (j - 1), keep, v);
            keep = v;
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            r[4 * j] = __float_as_uint(v.x); r[4 * j + 1] = __float_as_uint(v.y);
            r[4 * j + 2] = __float_as_uint(v.z); r[4 * j + 3] = __float_as_uint(v.w);
          }
          if (rbrow != nullptr) {
            const bool wide_rb = (reinterpret_cast<uintptr_t>(rbrow + q) & 31) == 0;
            uint4 keep_pk = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float w[8];
              if (got && !prm.next_w_f32) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&ahead->w[j >> 3]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = __bfloat1622float2(h[e]);
                  w[2 * e] = f.x; w[2 * e + 1] = f.y;
                }
              } else {
                load_norm_w8(prm.next_w, prm.next_w_f32, q + j, w);
              }
              uint4 pk;
              pk.x = pack_bf16x2(__uint_as_float(r[j]) * w[0], __uint_as_float(r[j + 1]) * w[1]);
              pk.y = pack_bf16x2(__uint_as_float(r[j + 2]) * w[2], __uint_as_float(r[j + 3]) * w[3]);
              pk.z = pack_bf16x2(__uint_as_float(r[j + 4]) * w[4], __uint_as_float(r[j + 5]) * w[5]);
              pk.w = pack_bf16x2(__uint_as_float(r[j + 6]) * w[6], __uint_as_float(r[j + 7]) * w[7]);
              if (!wide_rb) *reinterpret_cast<uint4*>(rbrow + q + j) = pk;
              else if (j & 8) st_b32x8(rbrow + q + j - 8, keep_pk, pk);
              keep_pk = pk;
            }
          }
        } else {
          const bool wide = (reinterpret_cast<uintptr_t>(crow + q) & 31) == 0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const float4 a = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                         __uint_as_float(r[j + 3]));
            const float4 b = make_float4(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]), __uint_as_float(r[j + 6]),
                                         __uint_as_float(r[j + 7]));
            if (wide) {
              st_f32x8(reinterpret_cast<float*>(crow) + q + j, a, b);
            } else {
              *reinterpret_cast<float4*>(crow + q + j) = a;
              *reinterpret_cast<float4*>(crow + q + j + 4) = b;
            }
          }
        }
      } else {
        const bool wide = (reinterpret_cast<uintptr_t>(crow + q) & 31) == 0;
        uint4 keep_pk = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 pk;
          pk.x = pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
          pk.y = pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
          pk.z = pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
          pk.w = pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
          if (!wide) *reinterpret_cast<uint4*>(crow + q + j) = pk;
          else if (j & 8) st_b32x8(crow + q + j - 8, keep_pk, pk);
          keep_pk = pk;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (q + j < prm.Q) {
          float v = __uint_as_float(r[j]);
          if constexpr (sizeof(TOut) == 4) {
            if (prm.accumulate) {
              v += reinterpret_cast<const float*>(crow)[q + j];
              ss += v * v;
              if (rbrow != nullptr) rbrow[q + j] = __float2bfloat16_rn(v * load_norm_w(prm.next_w, prm.next_w_f32, q + j));
            }
          }
          store_out<TOut>(crow + q + j, v);
        }
    }
  }
  return ss;
}

// ------------------------------------------------------------------ persistent kernel (many rows)
// The prefill orientation (X = activations, C[p][q] = D[p][q]) as persistent blocks: one block
// per SM walks output tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (tile rows fastest, so
// that a wave of blocks shares weight tiles in L2).  Tensor memory holds TWO accumulators:
// while the epilogue warps drain tile i from one, the MMA thread already fills the other with
// tile i + 1, and the TMA thread runs ahead through the shared-memory ring.  The epilogue
// stores straight from registers: each thread owns one tile row and writes 32 consecutive
// outputs at a time with 16-byte stores.
// Tried and not kept: sharing out the k-blocks of the last, partial wave of tiles among all SMs
// ("stream-K": partial tiles through a float32 workspace, flags, the finishing block adding them in the
// order of their k-blocks).  At 2,048 rows of the Llama-3.1-8B products, where the last wave holds 88
// or 108 tiles for 148 SMs, it was slower, not faster: the query/key/value product 121 us against 95,
// the output product 112 against 80, the down product 226 against 208.  The blocks of a wave read the
// same operand tiles at about the same time (16 blocks share a weight tile, 9 or 10 an activation
// tile); with every block at another place in K that is lost, and the kernel is bound by what L2
// delivers (a wave's time goes as 128 + BN, the operand rows a tile loads per k-block).
template <int BN, int STAGES, typename TOut>
__global__ void __launch_bounds__(192, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                          const GemmParams prm) {
  constexpr uint32_t kXBytes = kBM * kBK * 2;
  constexpr uint32_t kYBytes = BN * kBK * 2;
  constexpr uint32_t kStageBytes = kXBytes + kYBytes;
  constexpr uint32_t kTmemCols = 2 * BN <= 256 ? 256 : 512;   // two accumulators (an allocation is a power of two)
  static_assert(BN % 32 == 0 && BN <= 256, "the epilogue stores 32 columns at a time");

  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  pdl_launch_dependents();
  const uint32_t dyn = smem_u32(smem_dyn);
  unsigned char* tiles = smem_dyn + ((1024u - (dyn & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_p = (prm.P + kBM - 1) / kBM, tiles_q = (prm.Q + BN - 1) / BN;
  const int n_tiles = tiles_p * tiles_q;
  const int num_kb = (prm.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 1);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const bool dead = (*(volatile int*)prm.status & kStatusWaitExpired) != 0;

  if (dead) {
    // nothing
  } else if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmY) : "memory");
      pdl_wait();
      int it = 0, issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const int p0 = (t % tiles_p) * kBM, q0 = (t / tiles_p) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1) || *(volatile int*)&abort_flag) { ok = false; break; }
          unsigned char* xs = tiles + (size_t)s * kStageBytes;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          tma_load_2d(xs, &tmX, &full_bar[s], kb * kBK, p0);
          tma_load_2d(xs + kXBytes, &tmY, &full_bar[s], kb * kBK, q0);
          issued = it + 1;
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicOr(prm.status, kStatusWaitExpired);
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(BN);
      int it = 0, i = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++i) {
        const int acc = i & 1;
        // the epilogue has drained this accumulator (passes at once for the first two tiles)
        if (!mbar_wait(&tempty_bar[acc], ((i >> 1) & 1) ^ 1) || *(volatile int*)&abort_flag) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph) || *(volatile int*)&abort_flag) { ok = false; break; }
          tc_fence_after();
          const uint32_t xs = smem_u32(tiles + (size_t)s * kStageBytes);
          const uint64_t da = smem_desc_sw128(xs), db = smem_desc_sw128(xs + kXBytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_f16(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tfull_bar[acc]);
      }
      if (!ok) {
        abort_flag = 1;
        atomicOr(prm.status, kStatusWaitExpired);
      }
    }
  } else {
    const int quad = warp & 3;
    TOut* C = (TOut*)prm.C;
    pdl_wait();
    // with the SwiGLU epilogue a 32-column chunk becomes 16 outputs: rows must stay 16-byte aligned
    const bool vec_ok = (prm.ldc % (prm.swiglu ? 16 : 8) == 0) && ((reinterpret_cast<uintptr_t>(C) % 16) == 0);
    int i = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++i) {
      const int acc = i & 1;
      const int p0 = (t % tiles_p) * kBM, q0 = (t / tiles_p) * BN;
      const int p = p0 + quad * 32 + lane;
      const float row_scale = norm_row_factor(prm, p);     // read while the tile's main loop still runs
      TOut* crow = C + (long long)p * prm.ldc;
      __nv_bfloat16* rbrow = prm.rb_out != nullptr ? prm.rb_out + (long long)p * prm.ldc : nullptr;
      ChunkAhead ahead;
      fetch_ahead<TOut>(ahead, crow, rbrow, p, q0, prm, vec_ok);      // nobody else writes this row's outputs
      if (!mbar_wait(&tfull_bar[acc], (i >> 1) & 1) || *(volatile int*)&abort_flag) {
        abort_flag = 1;
        atomicOr(prm.status, kStatusWaitExpired);
        break;
      }
      tc_fence_after();
      float ss = 0.f;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        // what this chunk adds to was asked for a chunk ago (the first chunk's before the tile was
        // complete); the next chunk's is asked for now, so that its trip to L2 runs under this chunk
        const ChunkAhead cur = ahead;
        fetch_ahead<TOut>(ahead, crow, rbrow, p, q0 + (ch + 1) * 32, prm, vec_ok && ch + 1 < BN / 32);
        uint32_t r[32];
        SIAR_TMEM_LD_32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + ch * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int q = q0 + ch * 32;
        ss += store_chunk<TOut>(r, crow, rbrow, p, q, prm, vec_ok, row_scale, &cur);
      }
      if (prm.ss_out != nullptr && p < prm.P) prm.ss_out[(size_t)p * prm.ss_parts + t / tiles_p] = ss;
      // this accumulator may be overwritten once all four epilogue warps have read it
      tc_fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) mbar_arrive(&tempty_bar[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ persistent kernel, two SMs per tile
// The same orientation with cta_group::2: a cluster of two blocks (two SMs) owns a 256 x 256 output
// tile.  Each block loads 128 of the tile's A rows and 128 of its B rows, so a block brings in
// (128 + 128) x 64 elements per k-block for its 128 x 256 outputs instead of (128 + 256) x 64: a
// third less traffic from L2, which is what bounds the one-SM kernel.  The even block's MMA thread
// issues M = 256, N = 256 MMAs that read both blocks' shared memory and write both blocks' tensor
// memory; both blocks' TMA loads count on the even block's barrier; tcgen05.commit arrives on both
// blocks' barriers at once; both blocks' epilogues release the accumulator on the even block's
// barrier.  Everything else (persistent walk over tiles, two accumulators, epilogues) is as above.
template <int STAGES, typename TOut>
__global__ void __launch_bounds__(192, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                    const GemmParams prm) {
  constexpr int BN = 256;                               // the MMA's N; a block holds BN / 2 rows of B
  constexpr uint32_t kXBytes = kBM * kBK * 2;
  constexpr uint32_t kYBytes = (BN / 2) * kBK * 2;
  constexpr uint32_t kStageBytes = kXBytes + kYBytes;
  constexpr uint32_t kTmemCols = 2 * BN;               // two accumulators

  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];    // used in the even block
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];       // used in the even block
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  pdl_launch_dependents();
  const uint32_t dyn = smem_u32(smem_dyn);
  unsigned char* tiles = smem_dyn + ((1024u - (dyn & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_rank();                 // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_p = (prm.P + 2 * kBM - 1) / (2 * kBM), tiles_q = (prm.Q + BN - 1) / BN;
  const int n_tiles = tiles_p * tiles_q;
  const int num_kb = (prm.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2);                     // one arrival from each block's epilogue
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(&tmem_base_slot, kTmemCols);
  tc_fence_before();
  cluster_sync_all();                                   // both blocks' barriers exist before either is signalled
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const bool dead = (*(volatile int*)prm.status & kStatusWaitExpired) != 0;

  if (dead) {
    // nothing
  } else if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmY) : "memory");
      pdl_wait();
      int it = 0;
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += n_pairs) {
        const int p0 = (t % tiles_p) * 2 * kBM + rank * kBM;        // this block's rows of A (and of the output)
        const int q0 = (t / tiles_p) * BN + rank * (BN / 2);        // this block's rows of B
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1) || *(volatile int*)&abort_flag) { ok = false; break; }
          unsigned char* xs = tiles + (size_t)s * kStageBytes;
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * kStageBytes);   // both blocks' bytes
          tma_load_2d_pair(xs, &tmX, &full_bar[s], kb * kBK, p0);
          tma_load_2d_pair(xs + kXBytes, &tmY, &full_bar[s], kb * kBK, q0);
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicOr(prm.status, kStatusWaitExpired);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instr_desc_bf16_pair(BN);
      int it = 0, i = 0;
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += n_pairs, ++i) {
        const int acc = i & 1;
        // both epilogues have drained this accumulator (passes at once for the first two tiles)
        if (!mbar_wait(&tempty_bar[acc], ((i >> 1) & 1) ^ 1) || *(volatile int*)&abort_flag) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph) || *(volatile int*)&abort_flag) { ok = false; break; }
          tc_fence_after();
          const uint32_t xs = smem_u32(tiles + (size_t)s * kStageBytes);
          const uint64_t da = smem_desc_sw128(xs), db = smem_desc_sw128(xs + kXBytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_f16_pair(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[s]);              // the stage is free in both blocks
        }
        if (ok) umma_commit_pair(&tfull_bar[acc]);      // both blocks' halves of the tile are complete
      }
      if (!ok) {
        abort_flag = 1;
        atomicOr(prm.status, kStatusWaitExpired);
      }
    }
  } else {
    const int quad = warp & 3;
    TOut* C = (TOut*)prm.C;
    pdl_wait();
    const bool vec_ok = (prm.ldc % (prm.swiglu ? 16 : 8) == 0) && ((reinterpret_cast<uintptr_t>(C) % 16) == 0);
    int i = 0;
    for (int t = pair; t < n_tiles; t += n_pairs, ++i) {
      const int acc = i & 1;
      const int p0 = (t % tiles_p) * 2 * kBM + rank * kBM, q0 = (t / tiles_p) * BN;
      const int p = p0 + quad * 32 + lane;
      const float row_scale = norm_row_factor(prm, p);     // read while the tile's main loop still runs
      TOut* crow = C + (long long)p * prm.ldc;
      __nv_bfloat16* rbrow = prm.rb_out != nullptr ? prm.rb_out + (long long)p * prm.ldc : nullptr;
      ChunkAhead ahead;
      fetch_ahead<TOut>(ahead, crow, rbrow, p, q0, prm, vec_ok);      // nobody else writes this row's outputs
      if (!mbar_wait(&tfull_bar[acc], (i >> 1) & 1) || *(volatile int*)&abort_flag) {
        abort_flag = 1;
        atomicOr(prm.status, kStatusWaitExpired);
        break;
      }
      tc_fence_after();
      float ss = 0.f;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        const ChunkAhead cur = ahead;              // asked for a chunk ago; the next chunk's is asked for now
        fetch_ahead<TOut>(ahead, crow, rbrow, p, q0 + (ch + 1) * 32, prm, vec_ok && ch + 1 < BN / 32);
        uint32_t r[32];
        SIAR_TMEM_LD_32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + ch * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        ss += store_chunk<TOut>(r, crow, rbrow, p, q0 + ch * 32, prm, vec_ok, row_scale, &cur);
      }
      if (prm.ss_out != nullptr && p < prm.P) prm.ss_out[(size_t)p * prm.ss_parts + t / tiles_p] = ss;
      tc_fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) mbar_arrive_even(&tempty_bar[acc]);
    }
  }
  // neither block leaves (or gives its tensor memory back) while the other may still touch it
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
struct MapKey {
  const void* ptr;
  int rows, K, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && K == o.K && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.K << 20) ^ (size_t)k.box_rows;
  }
};

// A [rows, K] bf16 matrix, K contiguous, seen in boxes of box_rows x 64 with the
// 128-byte swizzle; reads past rows or K give zeros.
static bool tensor_map(const void* ptr, int rows, int K, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, K, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  cuuint32_t estride[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

template <int BN, int STAGES, typename TOut>
static int launch(const CUtensorMap& tmX, const CUtensorMap& tmY, const GemmParams& prm, int splits, cudaStream_t s) {
  constexpr size_t smem = (size_t)STAGES * (kBM * kBK * 2 + BN * kBK * 2) + 1024;
  auto kern = gemm_tc_kernel<BN, STAGES, TOut>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((prm.P + kBM - 1) / kBM, (prm.Q + BN - 1) / BN, splits);
  // The `splits` blocks of an output tile form one thread-block cluster (along z).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = splits;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, kern, tmX, tmY, prm);
}

template <int BN, int STAGES, typename TOut>
static int launch_persistent(const CUtensorMap& tmX, const CUtensorMap& tmY, const GemmParams& prm, int sm_count,
                             cudaStream_t s) {
  constexpr size_t smem = (size_t)STAGES * (kBM * kBK * 2 + BN * kBK * 2) + 1024;
  auto kern = gemm_tc_persistent_kernel<BN, STAGES, TOut>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int n_tiles = ((prm.P + kBM - 1) / kBM) * ((prm.Q + BN - 1) / BN);
  const int blocks = n_tiles < sm_count ? n_tiles : sm_count;
  return (int)launch_kernel(kern, dim3(blocks), dim3(192), smem, s, tmX, tmY, prm);
}

template <int STAGES, typename TOut>
static int launch_pair(const CUtensorMap& tmX, const CUtensorMap& tmY, const GemmParams& prm, int sm_count,
                       cudaStream_t s) {
  constexpr size_t smem = (size_t)STAGES * (kBM * kBK * 2 + 128 * kBK * 2) + 1024;
  auto kern = gemm_tc_pair_kernel<STAGES, TOut>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int n_tiles = ((prm.P + 2 * kBM - 1) / (2 * kBM)) * ((prm.Q + 255) / 256);
  const int pairs = n_tiles < sm_count / 2 ? n_tiles : sm_count / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, kern, tmX, tmY, prm);
}

}  // namespace siar

using namespace siar;

SIAR_DEFINE_PDL_SWITCH()


#ifdef SIAR_TIMING
// profiling builds: every launch writes its marks to a region of its own, [launch % 64][block < 2048][16]
static unsigned long long* g_stamps = nullptr;
static int g_stamp_launch = 0;
extern "C" void siar_gemm_tc_set_stamps(unsigned long long* p) { g_stamps = p; g_stamp_launch = 0; }
#endif

// Products of many rows with at least 256 output columns: two SMs per 256 x 256 tile or one SM per
// 128 x 256 tile.  pair_mode 0 = never pairs, 2 = always, 1 = pairs from kPairRows rows on (measured on
// B200 with the Llama-3.1-8B products: at 8,192 rows pairs are 2% faster, at 2,048 rows 1.5% slower; both
// run near the clocks the power cap allows, so the third less traffic from L2 buys little).
constexpr int kPairRows = 4096;

// Products with fewer output tiles than SMs are split along K into about this many blocks per two SMs
// (three: 1.5 blocks an SM).  A block keeps five stages of 18 KB on their way; with one block an SM the
// 160 blocks of the o and down products hold 14 MB in flight where 7 TB/s times the loaded latency wants
// about 20.  Measured on the Llama-3.1-8B decode step: o and down cut 7 ways instead of 5 and qkv 5 ways
// instead of 4 take 0.5-1.2% off a step at batch 1 to 16; 8 ways for o and down or 6 for qkv are 2-3%
// slower, and so were two or three blocks an SM (4-6%).
#ifndef SIAR_SPLIT_HALVES
#define SIAR_SPLIT_HALVES 3
#endif
constexpr int kSplitHalves = SIAR_SPLIT_HALVES;

// How a product of these sizes runs: orientation, tile width, split along K and kernel.
struct GemmPlan {
  bool swap;          // few rows: the weight on the MMA's row axis, the output written transposed
  int P, Q, BN;
  int splits, kbps;   // small kernel: blocks per output tile along K, k-blocks of 64 per block
  int kernel;         // 0 small kernel, 1 small kernel as clusters in the plain orientation, 2 pairs of SMs, 3 persistent
  int ss_parts;       // parts of a row's sum of squares an accumulating launch writes (0: it cannot)
};

// Tile width of a many-row product on the persistent kernel: tiles are handed out in waves of one per
// SM, and the last wave is as long as the others however few tiles it holds, so a width that makes
// the waves come out even can beat the widest one.  A 128 x BN tile loads 128 + BN operand rows per
// k-block, and that traffic, not the arithmetic, sets its time (measured on B200 at 1,024 to 4,096 rows
// with the Llama-3.1-8B products: the time of a wave goes as 128 + BN to within a few per cent), so the
// estimate is waves * (128 + BN); a narrower tile is taken only when that is 3% below the widest
// one's.  At 2,048 rows the widest tile wins for all four products; at 1,024 rows 224 columns take
// 8% off the gate/up product (7 waves either way) and 192 columns 9% off the query/key/value product.
static int many_row_tile_width(int M, int N, int sm_count, int forced) {
  if (N < 256) return 128;
  if (forced == 256 || forced == 224 || forced == 192 || forced == 160 || forced == 128) return forced;
  const long long tiles_p = (M + kBM - 1) / kBM;
  auto cost = [&](int bn) {
    const long long tiles = tiles_p * ((N + bn - 1) / bn);
    return (double)((tiles + sm_count - 1) / sm_count) * (kBM + bn);
  };
  int best = 256;
  double best_cost = cost(256) * 0.97;
  for (int bn = 224; bn >= 128; bn -= 32) {
    const double c = cost(bn);
    if (c < best_cost) { best_cost = c; best = bn; }
  }
  return best;
}

static bool make_plan(int M, int N, int K, int epilogue, int max_splits, int sm_count, int pair_mode, int tile_n,
                      GemmPlan* out) {
  GemmPlan g;
  g.swap = M <= 128;
  g.P = g.swap ? N : M;
  g.Q = g.swap ? M : N;
  if (g.swap) g.BN = g.Q <= 16 ? 16 : g.Q <= 32 ? 32 : g.Q <= 64 ? 64 : 128;
  else g.BN = g.Q >= 256 ? 256 : 128;
  if (epilogue == 1) max_splits = 1;
  const int tiles = ((g.P + kBM - 1) / kBM) * ((g.Q + g.BN - 1) / g.BN);
  const int num_kb = (K + kBK - 1) / kBK;
  int splits = 1;
  if (g.swap && tiles < sm_count) {
    splits = (kSplitHalves * sm_count / 2 + tiles - 1) / tiles;
    // ... but slices of fewer than eight k-blocks (little more than the five stages a block asks for before
    // it has even waited for its input) only as far as it takes to give every SM a block (the 3,072-wide
    // o product of the 3B shape: 7 ways, not 8, is 1% of a decode step)
    const int by_length = num_kb / 8, one_each = (sm_count + tiles - 1) / tiles;
    const int longest_cut = by_length > one_each ? by_length : one_each;
    if (splits > longest_cut) splits = longest_cut;
    if (splits > 8) splits = 8;
    if (splits > max_splits) splits = max_splits;
    if (splits > num_kb / 4) splits = num_kb / 4;
    if (splits < 1) splits = 1;
  }
  g.kbps = (num_kb + splits - 1) / splits;
  g.splits = (num_kb + g.kbps - 1) / g.kbps;
  g.kernel = g.swap ? 0 : 3;
  g.ss_parts = 0;
  if (g.swap) {
    // 16-column tiles add with or without a split; wider ones only as clusters (the owner blocks add)
    if (g.BN == 16 || g.splits > 1) g.ss_parts = (N + kBM - 1) / kBM;
    else if (epilogue == 2) return false;
  } else {
    // Prompts of a few hundred tokens give the many-row orientation fewer tiles than there are SMs,
    // and a tile's block then streams its weight rows alone, at a single SM's share of the bandwidth.
    // Those products run on the small-batch kernel in this orientation instead: a cluster of blocks
    // per 128 x 256 tile, each with a slice of K, partial sums joined through distributed shared memory.
    if (g.BN == 256 && epilogue != 1 && tiles < sm_count) {
      int sp = sm_count / tiles;              // one block to an SM (192 KB of pipeline stages): one wave
      sp = sp >= 8 ? 8 : sp >= 4 ? 4 : sp >= 2 ? 2 : 1;      // clusters of 3, 5, 6 or 7 do not all find room at once
      if (sp > max_splits) sp = max_splits;
      if (sp > num_kb / 4) sp = num_kb / 4;
      if (sp >= 2) {
        const int per = (num_kb + sp - 1) / sp;
        sp = (num_kb + per - 1) / per;
        if (sp >= 2) {
          g.kernel = 1;
          g.splits = sp;
          g.kbps = per;
          g.ss_parts = N % 4 == 0 ? ((N + 255) / 256) * sp : 0;
        }
      }
    }
    if (g.kernel == 3) {
      if (g.BN == 256 && sm_count >= 2 && (pair_mode >= 2 || (pair_mode == 1 && g.P >= kPairRows))) g.kernel = 2;
      else g.BN = many_row_tile_width(M, N, sm_count, tile_n);
      g.ss_parts = (N + g.BN - 1) / g.BN;
    }
  }
  *out = g;
  return true;
}

// Returns 0 on launch, a cudaError_t on failure, and -1 when the shape is one this
// unit does not take (the caller then uses the CUDA-core kernel).
//   A [M,K], W [N,K] bf16 row-major; C [M,N] bf16 (out_f32 == 0) or float32.
//   max_splits caps the split along K (1 = never split; at most 8, the portable cluster size).
//   epilogue 1: W's rows are interleaved (gate_0, up_0, gate_1, up_1, ...) and C [M, N/2] bf16 receives
//   silu(gate) * up (never split along K).
//   epilogue 2: C [M,N] float32 += the product.  With rb_out [M,N] bf16, next_w [N] and ss_out
//   [M, ss_out_parts] it also leaves what the product after the next RMSNorm needs: bf16(new C * next_w)
//   and the rows' sums of squares in ss_out_parts parts (siar_gemm_tc_ss_parts says how many; refused when
//   that does not match).
//   ss_in != nullptr: A is such an rb; the rows of the product are multiplied by
//   rsqrt(sum(ss_in[row][0..ss_in_parts)) / K + eps) before the epilogue's activation and the store.
static int run_gemm(const void* A, const void* W, void* C, int M, int N, int K, int out_f32, int max_splits,
                    int epilogue, int* status, int sm_count, void* stream, const float* ss_in, int ss_in_parts,
                    float eps, float* ss_out, int ss_out_parts, void* rb_out, const void* next_w, int next_w_f32,
                    int pair_mode, int tile_n) {
  if (M <= 0 || N <= 0) return 0;
  if (epilogue < 0 || epilogue > 2) return -1;
  if (epilogue == 1 && (out_f32 || (N & 1))) return -1;
  if (epilogue == 2 && !out_f32) return -1;
  if (ss_in != nullptr && (epilogue == 2 || ss_in_parts <= 0)) return -1;
  if (epilogue != 2 && (ss_out != nullptr || rb_out != nullptr)) return -1;
  if ((ss_out != nullptr) != (rb_out != nullptr) || (rb_out != nullptr && next_w == nullptr)) return -1;
  if (K % 8 != 0 || K < 8) return -1;                       // TMA needs 16-byte row strides
  if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)rb_out) & 15) return -1;
  cudaStream_t s = (cudaStream_t)stream;
  GemmPlan g;
  if (!make_plan(M, N, K, epilogue, max_splits, sm_count, pair_mode, tile_n, &g)) return -1;
  if (ss_out != nullptr && (g.ss_parts == 0 || g.ss_parts != ss_out_parts || N % 8 != 0)) return -1;
  const bool swap = g.swap;
  const void* X = swap ? W : A;
  const void* Y = swap ? A : W;
  const int P = g.P, Q = g.Q, BN = g.BN;
  CUtensorMap tmX, tmY;
  if (!tensor_map(X, P, K, kBM, &tmX)) return -1;
  if (!tensor_map(Y, Q, K, BN, &tmY)) return -1;
  const int splits = g.splits;

  GemmParams prm;
  prm.C = C;
  prm.status = status;
  prm.P = P; prm.Q = Q; prm.K = K;
  prm.ldc = epilogue == 1 ? N / 2 : N;
  prm.swiglu = epilogue == 1 ? 1 : 0;
  prm.transpose_out = swap ? 1 : 0;
  prm.kb_per_split = g.kbps;
  prm.x_is_weight = swap ? 1 : 0;
  prm.accumulate = epilogue == 2 ? 1 : 0;
  prm.ss_out = ss_out;
  prm.ss_parts = ss_out_parts;
  prm.rb_out = (__nv_bfloat16*)rb_out;
  prm.next_w = next_w;
  prm.next_w_f32 = next_w_f32;
  prm.ss_in = ss_in;
  prm.ss_in_parts = ss_in_parts;
  prm.inv_width = 1.f / (float)K;
  prm.eps = eps;
#ifdef SIAR_TIMING
  prm.stamps = g_stamps ? g_stamps + (size_t)(g_stamp_launch++ % 64) * 2048 * 16 : nullptr;
#endif

  if (g.kernel == 1) {
    prm.x_is_weight = 2;
    return out_f32 ? launch<256, 4, float>(tmX, tmY, prm, splits, s) : launch<256, 4, __nv_bfloat16>(tmX, tmY, prm, splits, s);
  }
  if (g.kernel == 2) {
    CUtensorMap tmY2;
    if (tensor_map(Y, Q, K, 128, &tmY2))
      return out_f32 ? launch_pair<6, float>(tmX, tmY2, prm, sm_count, s)
                     : launch_pair<6, __nv_bfloat16>(tmX, tmY2, prm, sm_count, s);
  }
  if (!swap) {
#define SIAR_PERSISTENT(BN_, ST_)                                                                   \
  return out_f32 ? launch_persistent<BN_, ST_, float>(tmX, tmY, prm, sm_count, s)                   \
                 : launch_persistent<BN_, ST_, __nv_bfloat16>(tmX, tmY, prm, sm_count, s)
    switch (BN) {            // stages: what fits in shared memory
      case 256: SIAR_PERSISTENT(256, 4);
      case 224: SIAR_PERSISTENT(224, 5);
      case 192: SIAR_PERSISTENT(192, 5);
      case 160: SIAR_PERSISTENT(160, 6);
      default: SIAR_PERSISTENT(128, 6);
    }
#undef SIAR_PERSISTENT
  }
#define SIAR_GO(BN_, ST_)                                                                      \
  return out_f32 ? launch<BN_, ST_, float>(tmX, tmY, prm, splits, s)                           \
                 : launch<BN_, ST_, __nv_bfloat16>(tmX, tmY, prm, splits, s)
  switch (BN) {
    case 16: SIAR_GO(16, 5);
    case 32: SIAR_GO(32, 5);
    case 64: SIAR_GO(64, 4);
    case 128: SIAR_GO(128, 3);
    default: SIAR_GO(256, 4);
  }
#undef SIAR_GO
}

extern "C" int siar_gemm_tc_bf16(const void* A, const void* W, void* C, int M, int N, int K, int out_f32,
                                 int max_splits, int epilogue, int* status, int sm_count, void* stream,
                                 int pair_mode, int tile_n) {
  if (epilogue == 2) return -1;
  return run_gemm(A, W, C, M, N, K, out_f32, max_splits, epilogue, status, sm_count, stream, nullptr, 0, 0.f, nullptr,
                  0, nullptr, nullptr, 0, pair_mode, tile_n);
}

// Parts of a row's sum of squares that siar_gemm_tc_bf16_fused writes to ss_out for an accumulating
// product (epilogue 2) of these sizes; 0 when such a launch cannot leave them.
extern "C" int siar_gemm_tc_ss_parts(int M, int N, int K, int max_splits, int sm_count, int pair_mode, int tile_n) {
  GemmPlan g;
  if (M <= 0 || N <= 0 || K % 8 != 0 || K < 8 || N % 8 != 0) return 0;
  if (!make_plan(M, N, K, 2, max_splits, sm_count, pair_mode, tile_n, &g)) return 0;
  return g.ss_parts;
}

// The same product inside a float32 residual stream (see run_gemm and GemmParams).
extern "C" int siar_gemm_tc_bf16_fused(const void* A, const void* W, void* C, int M, int N, int K, int out_f32,
                                       int max_splits, int epilogue, int* status, int sm_count, void* stream,
                                       const float* ss_in, int ss_in_parts, float eps, float* ss_out,
                                       int ss_out_parts, void* rb_out, const void* next_w, int next_w_f32,
                                       int pair_mode, int tile_n) {
  return run_gemm(A, W, C, M, N, K, out_f32, max_splits, epilogue, status, sm_count, stream, ss_in, ss_in_parts, eps,
                  ss_out, ss_out_parts, rb_out, next_w, next_w_f32, pair_mode, tile_n);
}
