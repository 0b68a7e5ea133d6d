// Causal grouped-query attention for prompts (any mix of new-token counts per sequence) on the
// 5th-generation tensor cores: S = Q K^T and O += P V are tcgen05.mma instructions with S and O in
// tensor memory, Q / K / V tiles come by TMA (K and V straight from the pages of the cache), and
// the softmax runs on 256 threads, each owning one row.  bfloat16, head_dim 64 or 128, up to 128
// query heads per kv head; other sizes use the warp-level kernel of attention_mma.cu.  The rules are those
// of attention.cu (bottom-right causal, scale after the dot, running maximum, division at the end),
// cited there; as in the reference's flash kernel P is rounded to bfloat16 before P.V
// (kernels/attention_kernel.py:221).
//
// Rows of one (sequence, kv head) are (query position, head in group) pairs; a block takes two
// query tiles of 128 rows (the MMA's M), each holding floor(128 / G) whole tokens (a group size
// that does not divide 128 leaves the tile's last rows unused: they are masked like the rows past
// the end of a prompt), and walks the keys in tiles of 64 (one cache page), so every K / V tile
// that arrives is used by two query tiles:
//   TMA thread      Q once (a 3-D box: 64 dims x G heads x floor(128/G) tokens lands as packed rows),
//                   then K and V of each key tile into three-stage rings of their own (a K stage
//                   is free as soon as the scores that read it are done, a V stage a step later);
//   MMA thread      for each query tile S = Q K^T (8 MMAs of K = 16 over the two 64-dim halves),
//                   one key tile ahead of the softmax (S is double-buffered in tensor memory), and,
//                   once that tile's softmax threads have written P, O += P V (4 MMAs over 16 keys
//                   each; P is the A operand read from tensor memory, V an MN-major operand in
//                   shared memory: its 64-dim rows are the contiguous index);
//   softmax threads (one group of 128 per query tile) read their row of S from tensor memory, mask,
//                   exponentiate in the base-2 domain, write P (bf16 pairs) over the first 32
//                   columns of the S they read (shared memory carries only Q, K and V: P through
//                   shared memory cost a write and a read of 16 KiB per tile and step, measured 11%
//                   of the kernel's time at 8,192 tokens), and keep the row sum.  O stays in tensor memory;
//                   it is rescaled there only when a row's maximum has grown by more than 2^8 since
//                   the last rescale (the final division uses the same reference maximum, so the
//                   result is exact up to rounding), and read once at the end.
// Tensor memory: 2 x 2 x 64 columns of S and 2 x head_dim columns of O (512 columns allocated), one block per SM.
// Every mbarrier wait is bounded and reports through the status word.
#include "tcgen05.cuh"

#include <math.h>

#include <unordered_map>

namespace siar {

constexpr int kRows = 128;       // rows per query tile
constexpr int kQTiles = 2;       // query tiles per block
constexpr int kKeys = 64;        // keys per tile
constexpr int kStages = 3;       // K and V rings
constexpr int smem_bytes(int hd) { return kQTiles * kRows * hd * 2 + kStages * 2 * kKeys * hd * 2; }
constexpr uint32_t kTmemCols = 512;                 // S[q][buf]: 64 columns each from 0; O[q]: 128 each from 256
constexpr float kRescaleGap = 8.f;                  // log2 of the growth that forces a rescale
constexpr int kThreads = 128 + kQTiles * 128;   // TMA warp, one MMA warp per query tile, a spare, the softmax warps

struct AttnTcParams {
  __nv_bfloat16* out;
  const int* block_table;
  const int* slot_ids;
  const int* q_start;
  const int* base_len;
  int* status;
  int Hq, Hkv, page_tokens, max_pages;
  float scale;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#define SIAR_TMEM_ST_32(taddr, r)                                                                                  \
  asm volatile(                                                                                                    \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "                                                             \
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28," \
      "%29,%30,%31};" ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),    \
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),     \
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),   \
      "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)                           \
      : "memory")

template <int kHd>
__global__ void __launch_bounds__(kThreads)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const AttnTcParams prm) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t q_full;
  __shared__ __align__(8) uint64_t s_full[kQTiles][2], p_full[kQTiles][2], pv_full[kQTiles][2];
  // keys and values have rings of their own: a key stage is free again as soon as the scores that
  // read it are done, a value stage only after P.V, a step later, so each is asked for as early as it can be
  __shared__ __align__(8) uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  constexpr int kHalves = kHd / 64;                  // 64-dim (128-byte) column blocks of a row
  constexpr int kQBytes = kRows * kHd * 2;           // 16 KiB per half
  constexpr int kTileBytes = kKeys * kHd * 2;        // 8 KiB per half
  pdl_launch_dependents();
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = prm.Hq / prm.Hkv;
  const int tile_rows = (kRows / G) * G;             // rows of a query tile in use: whole tokens only
  const int t0 = prm.q_start[b];                 // batch description: written by no kernel of this step
  const int q_len = prm.q_start[b + 1] - t0;
  const int rows_total = q_len * G;
  // blocks with the most keys (the last rows) start first: the tail of the grid is made of short blocks
  const int row0 = (gridDim.x - 1 - blockIdx.x) * (kQTiles * tile_rows);
  if (row0 >= rows_total) return;
  const int base = prm.base_len[b];
  const int slot = prm.slot_ids[b];
  // per query tile: its rows and the key tiles it needs (later rows see more keys)
  int rows_q[kQTiles], nt[kQTiles];
  int n_q = 0;
#pragma unroll
  for (int g = 0; g < kQTiles; ++g) {
    rows_q[g] = max(0, min(tile_rows, rows_total - row0 - g * tile_rows));
    nt[g] = rows_q[g] > 0 ? (base + (row0 + g * tile_rows + rows_q[g] - 1) / G + 1 + kKeys - 1) / kKeys : 0;
    if (rows_q[g] > 0) n_q = g + 1;
  }
  // Both query tiles walk all the key tiles of the block (the first tile's last one may be masked
  // entirely): a stage of the ring is then released by as many MMA threads as there are tiles.
  const int nt_max = nt[n_q - 1];
#pragma unroll
  for (int g = 0; g < kQTiles; ++g)
    if (rows_q[g] > 0) nt[g] = nt_max;

  const uint32_t dyn = smem_u32(smem_dyn);
  unsigned char* sm = smem_dyn + ((1024u - (dyn & 1023u)) & 1023u);
  unsigned char* q_s = sm;                                   // [q tile][half][128 rows][64 dims]
  unsigned char* k_s = q_s + kQTiles * kQBytes;              // [stage][half][64 keys][64 dims]
  unsigned char* v_s = k_s + kStages * kTileBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int g = 0; g < kQTiles; ++g) {
      mbar_init(&s_full[g][0], 1);
      mbar_init(&s_full[g][1], 1);
      mbar_init(&p_full[g][0], 1);
      mbar_init(&p_full[g][1], 1);
      mbar_init(&pv_full[g][0], 1);
      mbar_init(&pv_full[g][1], 1);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], n_q);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], n_q);
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
  pdl_wait();

#define SIAR_FAIL()                                   \
  {                                                   \
    abort_flag = 1;                                   \
    atomicOr(prm.status, kStatusWaitExpired);         \
  }
#define SIAR_ABORTED() (*(volatile int*)&abort_flag != 0)

  if (dead) {
    // another block already reported an expired wait: do nothing
  } else if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmK) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmV) : "memory");
      mbar_expect_tx(&q_full, n_q * tile_rows * kHd * 2);      // a box is tile_rows packed rows (the rest of the tile stays as it was: masked rows)
      for (int g = 0; g < n_q; ++g) {
        const int tok = t0 + (row0 + g * tile_rows) / G;
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_3d(q_s + g * kQBytes + h * (kQBytes / kHalves), &tmQ, &q_full, 64 * h, kvh * G, tok);
      }
      const int* table = prm.block_table + (size_t)slot * prm.max_pages;
      int issued_k = 0, issued_v = 0;
      // A cell below zero means "no page": the sequence does not hold these positions.  It is read
      // as page 0 (never as a row in front of the pool) and reported through the status word.
      bool bad_page = false;
      int page = table[0];                       // read one tile ahead of its use
      if (page < 0) { bad_page = true; page = 0; }
      for (int i = 0; i < nt_max; ++i) {
        const int s = i % kStages;
        const uint32_t ph = ((i / kStages) & 1) ^ 1;
        const int j0 = i * kKeys;
        const int row = (page * prm.Hkv + kvh) * prm.page_tokens + (j0 % prm.page_tokens);
        if (i + 1 < nt_max) {
          page = table[(j0 + kKeys) / prm.page_tokens];
          if (page < 0) { bad_page = true; page = 0; }
        }
        if (!mbar_wait(&k_empty[s], ph) || SIAR_ABORTED()) { SIAR_FAIL(); break; }
        mbar_expect_tx(&k_full[s], kTileBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_2d(k_s + s * kTileBytes + h * (kTileBytes / kHalves), &tmK, &k_full[s], 64 * h, row);
        issued_k = i + 1;
        if (!mbar_wait(&v_empty[s], ph) || SIAR_ABORTED()) { SIAR_FAIL(); break; }
        mbar_expect_tx(&v_full[s], kTileBytes);
#pragma unroll
        for (int h = 0; h < kHalves; ++h)
          tma_load_2d(v_s + s * kTileBytes + h * (kTileBytes / kHalves), &tmV, &v_full[s], 64 * h, row);
        issued_v = i + 1;
      }
      if (bad_page) atomicOr(prm.status, kStatusBadPage);
      if (SIAR_ABORTED()) {    // let copies in flight land before the block leaves
        mbar_wait(&q_full, 0);
        for (int i = max(0, issued_k - kStages); i < issued_k; ++i) mbar_wait(&k_full[i % kStages], (i / kStages) & 1);
        for (int i = max(0, issued_v - kStages); i < issued_v; ++i) mbar_wait(&v_full[i % kStages], (i / kStages) & 1);
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------- MMA issue: one thread per query tile (the two tiles depend on nothing of
    // each other but the K / V stages, and two issuing warps sit on two schedulers)
    const int g = warp - 1;
    if (lane == 0 && g < n_q) {
      constexpr uint32_t idesc_qk = instr_desc_bf16(kKeys);
      constexpr uint32_t idesc_pv = instr_desc_bf16(kHd, true);
      // descriptors differ in their low word only (the address field, in units of 16 bytes)
      const uint32_t hi_k = (uint32_t)(smem_desc_sw128(0) >> 32);
      const uint32_t hi_v = (uint32_t)(smem_desc_sw128_mn(0, kTileBytes / kHalves) >> 32);
      const uint32_t q_lo = (uint32_t)smem_desc_sw128(smem_u32(q_s + g * kQBytes));
      const uint32_t k_lo = (uint32_t)smem_desc_sw128(smem_u32(k_s));
      const uint32_t v_lo = (uint32_t)smem_desc_sw128_mn(smem_u32(v_s), kTileBytes / kHalves);
      const uint32_t tmem_o = tmem_base + 256u + (uint32_t)(g * kHd);
      // S[g][i & 1] = Q_g K_i^T over the two 64-dim halves, 4 steps of 16 dims (32 bytes) in each
      auto issue_qk = [&](int i) {
        const uint32_t ks = k_lo + (uint32_t)((i % kStages) * (kTileBytes >> 4));
        const uint32_t tmem_s = tmem_base + (uint32_t)((g * 2 + (i & 1)) * kKeys);
#pragma unroll
        for (int kk = 0; kk < kHd / kUmmaK; ++kk)
          umma_f16_words(tmem_s, q_lo + (uint32_t)((kk / 4) * (kQBytes / kHalves >> 4) + (kk % 4) * 2), hi_k,
                         ks + (uint32_t)((kk / 4) * (kTileBytes / kHalves >> 4) + (kk % 4) * 2), hi_k, idesc_qk, kk > 0 ? 1u : 0u);
        umma_commit(&s_full[g][i & 1]);
        umma_commit(&k_empty[i % kStages]);       // the key stage is free once these scores are done
      };
      bool ok = mbar_wait(&q_full, 0) && mbar_wait(&k_full[0], 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int i = 0; i < nt_max && ok; ++i) {
        if (i + 1 < nt_max) {
          if (!mbar_wait(&k_full[(i + 1) % kStages], ((i + 1) / kStages) & 1) || SIAR_ABORTED()) { ok = false; break; }
          tc_fence_after();
          issue_qk(i + 1);
        }
        if (!mbar_wait(&p_full[g][i & 1], (i >> 1) & 1) || !mbar_wait(&v_full[i % kStages], (i / kStages) & 1) ||
            SIAR_ABORTED()) { ok = false; break; }
        tc_fence_after();
        // O_g += P_g V_i: 4 steps of 16 keys; V rows (keys) are 128 bytes of one dim half,
        // 8-row groups 1024 bytes apart, the two dim halves 8 KiB apart
        // P_i sits in tensor memory, in the first 32 columns of the scores it was made from
        const uint32_t tmem_p = tmem_base + (uint32_t)((g * 2 + (i & 1)) * kKeys);
        const uint32_t vs = v_lo + (uint32_t)((i % kStages) * (kTileBytes >> 4));
#pragma unroll
        for (int t = 0; t < kKeys / kUmmaK; ++t)
          umma_f16_tmem_a(tmem_o, tmem_p + (uint32_t)(t * 8), vs + (uint32_t)(t * (2048 >> 4)), hi_v, idesc_pv,
                          (i > 0 || t > 0) ? 1u : 0u);
        umma_commit(&pv_full[g][i & 1]);
        umma_commit(&v_empty[i % kStages]);
      }
      if (!ok) SIAR_FAIL();
    }
  } else if (warp >= 4 && (warp - 4) / 4 < n_q) {
    // ---------------- softmax: one thread per row, one group of four warps per query tile
    const int g = (warp - 4) / 4;
    const int quad = warp & 3;                 // the tensor-memory lanes this warp may touch
    const int row = quad * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const uint32_t tmem_o = tmem_base + 256u + (uint32_t)(g * kHd) + lane_base;
    const int rg = row0 + g * tile_rows + row;
    const int kv_end = row < rows_q[g] ? base + rg / G + 1 : 0;
    const float sl2 = prm.scale * 1.4426950408889634f;
    const int n_tiles = nt[g];
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      const int j0 = i * kKeys;
      if (!mbar_wait(&s_full[g][i & 1], (i >> 1) & 1) || SIAR_ABORTED()) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_s = tmem_base + (uint32_t)((g * 2 + (i & 1)) * kKeys) + lane_base;
      uint32_t sr[64];
      SIAR_TMEM_LD_32(tmem_s, sr);
      {
        uint32_t* hi = sr + 32;
        SIAR_TMEM_LD_32(tmem_s + 32, hi);
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (j0 + kKeys > kv_end) {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (j0 + j >= kv_end) sr[j] = 0xff800000u;      // -inf
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 64; j += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx[e] = fmaxf(mx[e], __uint_as_float(sr[j + e]));
      }
      const float raw = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      const float m_new = fmaxf(m_used, raw * sl2);
      const bool need = m_new > m_used + kRescaleGap;      // also true for the first finite maximum
      if (i > 0 && __any_sync(0xffffffffu, need)) {
        // O may be touched once the previous tile's P.V has completed
        if (!mbar_wait(&pv_full[g][(i - 1) & 1], ((i - 1) >> 1) & 1) || SIAR_ABORTED()) { ok = false; break; }
        tc_fence_after();
        const float alpha = need ? (m_used == -INFINITY ? 0.f : ex2(m_used - m_new)) : 1.f;
        l *= alpha;
#pragma unroll 1
        for (int ch = 0; ch < kHd / 32; ++ch) {
          uint32_t o[32];
          SIAR_TMEM_LD_32(tmem_o + ch * 32, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          SIAR_TMEM_ST_32(tmem_o + ch * 32, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      if (need) m_used = m_new;
      const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
      // P = 2^(s c - m) as bf16 pairs, written over the first 32 columns of the scores in tensor
      // memory (this thread holds its whole row in registers by now).  The next scores for this
      // buffer are issued after the P.V that reads P, and the tensor pipe keeps that order.
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pw[32];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2(fmaf(__uint_as_float(sr[c * 8 + 2 * e]), sl2, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(sr[c * 8 + 2 * e + 1]), sl2, neg_m));
          sum[e] += p0 + p1;
          pw[c * 4 + e] = pack_bf16x2(p0, p1);
        }
      }
      SIAR_TMEM_ST_32(tmem_s, pw);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
      tc_fence_before();
      if (g == 0)
        asm volatile("bar.sync 1, 128;" ::: "memory");
      else
        asm volatile("bar.sync 2, 128;" ::: "memory");
      if ((threadIdx.x & 127) == 0) mbar_arrive(&p_full[g][i & 1]);
    }
    if (ok) ok = mbar_wait(&pv_full[g][(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
    if (!ok) {
      SIAR_FAIL();
    } else {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = prm.out + (size_t)(t0 + rg / G) * prm.Hq * kHd + (size_t)(kvh * G + rg % G) * kHd;
#pragma unroll 1
      for (int ch = 0; ch < kHd / 32; ++ch) {
        uint32_t o[32];
        SIAR_TMEM_LD_32(tmem_o + ch * 32, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < rows_q[g]) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
            pk.y = pack_bf16x2(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
            pk.z = pack_bf16x2(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
            pk.w = pack_bf16x2(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + ch * 32 + j) = pk;
          }
        }
      }
    }
  }
#undef SIAR_FAIL
#undef SIAR_ABORTED
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base_slot, kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
struct PoolKey {
  const void* ptr;
  long long rows;
  int hd;
  bool operator==(const PoolKey& o) const { return ptr == o.ptr && rows == o.rows && hd == o.hd; }
};
struct PoolKeyHash {
  size_t operator()(const PoolKey& k) const { return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows ^ ((size_t)k.hd << 48); }
};

// The pool of one cache entry as a [rows, head_dim] matrix seen in boxes of 64 rows x 64 dims.
static bool pool_map(const void* ptr, long long rows, int kHd, CUtensorMap* out) {
  static std::unordered_map<PoolKey, CUtensorMap, PoolKeyHash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  PoolKey key{ptr, rows, kHd};
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)kHd, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)kHd * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)kKeys};
  cuuint32_t estride[2] = {1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 1024) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// The query part of the fused qkv rows as [tokens, Hq heads, head_dim], seen in boxes of
// floor(128/G) tokens x G heads x 64 dims: one box is the packed rows of a kv head's group that a
// query tile uses (all 128 when G divides 128).
static bool query_map(const void* qkv, int n_tokens, int Hq, int Hkv, int kHd, CUtensorMap* out) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const int G = Hq / Hkv;
  cuuint64_t gdim[3] = {(cuuint64_t)kHd, (cuuint64_t)Hq, (cuuint64_t)n_tokens};
  cuuint64_t gstride[2] = {(cuuint64_t)kHd * 2, (cuuint64_t)(Hq + 2 * Hkv) * kHd * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(kRows / G)};
  cuuint32_t estride[3] = {1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(qkv), gdim, gstride, box, estride,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace siar

using namespace siar;

SIAR_DEFINE_PDL_SWITCH()

// 1 when this unit takes the sizes: head_dim 64 or 128, at most 128 query heads per kv head, pages
// of 64 tokens (or a multiple).
extern "C" int siar_attn_tc_supported(int Hq, int Hkv, int D, int page_tokens) {
  if (Hkv <= 0 || Hq % Hkv != 0) return 0;
  const int G = Hq / Hkv;
  return (D == 64 || D == 128) && G <= 128 && page_tokens % kKeys == 0;
}

template <int HD>
static int launch_prefill(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnTcParams& prm,
                          dim3 grid, cudaStream_t s) {
  constexpr size_t smem = smem_bytes(HD) + 1024;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  return (int)launch_kernel(attn_prefill_tc_kernel<HD>, grid, dim3(kThreads), smem, s, tmQ, tmK, tmV, prm);
}

// qkv [N, (Hq + 2 Hkv) * D] bf16 with q already rotated and the new keys and values already in
// the cache; k_pool / v_pool [n_pages, Hkv, page_tokens, D]; out [N, Hq * D] bf16.
extern "C" int siar_attn_tc_prefill(const void* qkv, const void* k_pool, const void* v_pool, const int* block_table,
                                    const int* slot_ids, const int* q_start, const int* base_len, void* out, int N,
                                    int B, int Hq, int Hkv, int D, int page_tokens, int max_pages, int n_pages,
                                    int max_q_len, float scale, int* status, void* stream) {
  if (B == 0 || max_q_len == 0 || N == 0) return 0;
  if (!siar_attn_tc_supported(Hq, Hkv, D, page_tokens) || Hkv > 65535 || B > 65535) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) return (int)cudaErrorInvalidValue;
  CUtensorMap tmQ, tmK, tmV;
  const long long rows = (long long)n_pages * Hkv * page_tokens;
  if (!query_map(qkv, N, Hq, Hkv, D, &tmQ) || !pool_map(k_pool, rows, D, &tmK) || !pool_map(v_pool, rows, D, &tmV))
    return (int)cudaErrorInvalidValue;
  AttnTcParams prm;
  prm.out = (__nv_bfloat16*)out;
  prm.block_table = block_table;
  prm.slot_ids = slot_ids;
  prm.q_start = q_start;
  prm.base_len = base_len;
  prm.status = status;
  prm.Hq = Hq; prm.Hkv = Hkv; prm.page_tokens = page_tokens; prm.max_pages = max_pages;
  prm.scale = scale;
  const int G = Hq / Hkv;
  const int tile_rows = (kRows / G) * G;
  dim3 grid((max_q_len * G + kQTiles * tile_rows - 1) / (kQTiles * tile_rows), Hkv, B);
  return D == 64 ? launch_prefill<64>(tmQ, tmK, tmV, prm, grid, (cudaStream_t)stream)
                 : launch_prefill<128>(tmQ, tmK, tmV, prm, grid, (cudaStream_t)stream);
}
