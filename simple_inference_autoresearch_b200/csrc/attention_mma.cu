// bfloat16 causal grouped-query attention over the paged cache on the tensor cores
// (warp-level m16n8k16 MMA, float32 accumulation and float32 softmax state).  Same
// rules as the CUDA-core kernels in attention.cu, which stay the 32-bit path and the
// path for head sizes other than 64 and 128 (the formulas and their places in the
// reference are cited there).  As in the reference's flash kernel, P is rounded to
// bfloat16 before the P.V product (kernels/attention_kernel.py:221).
//
// The G query heads that share a kv head are packed on the MMA's row axis, so keys
// and values are read once per kv head, not once per query head:
//   * prefill: rows of one (sequence, kv head) are (query position, head in group)
//     pairs; a block takes 64 consecutive rows (16 per warp) and walks the keys in
//     tiles of 64 = one cache page, double-buffered with cp.async.
//   * decode: one new token, so the G heads are the only rows (padded to 16); a
//     block takes a chunk of 128 keys (32 per warp), joins its warps' partial
//     softmax states in shared memory and writes one partial per chunk to scratch;
//     the block of a (sequence, kv head) that finishes last joins the chunks in chunk
//     order.  A sequence of at most one chunk is finished by its only block.
// Key tiles start at multiples of the tile size, so a row's reduction order depends
// on its position only.
#include "attention_mma.cuh"

#include <math.h>

namespace siar {

constexpr int kPad = 8;             // bf16 elements of padding per shared-memory row (16 bytes)
constexpr int kMmaDecodeChunk = 128;   // granularity of a decode block's key range
// keys per warp and pipeline step in the decode kernel: 16 rows of 256 bytes at head_dim 128, 32 rows
// of 128 bytes at head_dim 64 (the same bytes on their way per warp; with 16 the smaller head streamed
// at little more than half the rate)
__host__ __device__ constexpr int decode_warp_keys(int d) { return d <= 64 ? 32 : 16; }
constexpr int kDecodeStages = 3;       // pipeline depth per warp
constexpr int kDecodeBlocksPerSM = 2;  // what shared memory allows with that depth
constexpr int kJoinPad = 8;            // floats of padding per row of the warps' join buffer (decode)
constexpr int kMmaPrefillRows = 64;
constexpr int kMmaKeyTile = 64;

#ifdef SIAR_TIMING
__device__ unsigned long long* g_attn_stamps = nullptr;   // profiling builds only: [blocks][8] globaltimer marks
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define SIAR_STAMP(i)                                                                                    \
  if (g_attn_stamps && threadIdx.x == 0)                                                                 \
  g_attn_stamps[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (i)] = gtime()
#else
#define SIAR_STAMP(i)
#endif

// Loads of what the kernel in front of this one wrote (the fused qkv rows), for code that runs after
// pdl_wait() in a kernel that has other work in front of the wait.  A load through a const
// __restrict__ pointer is an "invariant" load to the compiler (the location is promised not to change
// while the kernel lives), and invariant loads may be moved above any barrier, the dependency wait
// included: the query was then read while the product in front was still writing it.  A volatile asm
// with a memory clobber stays behind the wait.
__device__ __forceinline__ uint32_t ld_after_wait_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ __nv_bfloat16 ld_after_wait_bf16(const __nv_bfloat16* p) {
  unsigned short v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
  return __ushort_as_bfloat16(v);
}

// ------------------------------------------------------------------ decode
// grid (chunks, Hkv, B), 128 threads.  A block owns a run of consecutive keys of one
// (sequence, kv head); warp w walks keys [c0 + 64 it + 16 w, +16) for it = 0, 1, ... with a
// running (max, sum, output) per query head, its kDecodeStages shared-memory stages filled by
// cp.async kDecodeStages - 1 steps ahead (small stages, so that two blocks fit on an SM).
// The host chooses the number of chunks (chunk_keys, a multiple of 128, for the longest sequence the
// launch allows) so that the grid fills the GPU: one chunk per sequence when the batch alone gives
// enough blocks, 128-key chunks for a single sequence; the kernel shares a sequence's own tiles out
// evenly over that many blocks.
template <int D>
__global__ void __launch_bounds__(128)
attn_decode_mma_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ k_pool,
                       const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ block_table,
                       const int* __restrict__ slot_ids, const int* __restrict__ q_start,
                       const int* __restrict__ base_len, float* __restrict__ part_ml, float* __restrict__ part_acc,
                       int* __restrict__ counters, __nv_bfloat16* __restrict__ out, int Hq, int Hkv, int page_tokens,
                       int max_pages, int max_chunks, int chunk_keys, float scale, const float* __restrict__ inv_freq,
                       int fuse_rope, int write_kv, int* __restrict__ status) {
  // fuse_rope: the fused qkv rows are as the product left them; this kernel rotates q (in
  // registers) and the new token's k by the token's position, writes that k and v to the cache
  // (write_kv) and uses them from shared memory, so no separate rotate-and-write kernel runs.
  __shared__ float cs_s[D];                     // cos[D/2], sin[D/2] of the new token's position
  pdl_launch_dependents();
  SIAR_TRACE(20, 0);
  // What this kernel reads before its query: the batch description and the block table (written
  // before the step's first kernel, behind a copy that nothing overtakes) and the keys and values of
  // earlier positions.  When the kernel itself is the step's only writer of its cache entry
  // (fuse_rope && write_kv) those are final since earlier steps, so the whole prologue (lengths ->
  // block table -> first tiles, three dependent trips to L2, and the rotation angles) runs while the
  // product in front is still at work, and only the query waits.  A layer that reads the cache another
  // layer of this step writes (write_kv == 0), or whose new keys a separate kernel stores (no fuse_rope),
  // waits first.
  const bool early = fuse_rope && write_kv;
  if (!early) {
    pdl_wait();
    SIAR_TRACE(20, 2);
  }
  constexpr int RS = D + kPad;                 // row stride in elements
  constexpr int CPR = D / 8;                   // 16-byte pieces per row
  constexpr int WK = decode_warp_keys(D);      // keys per warp and step
  constexpr int kStageElems = 2 * 4 * WK * RS; // K and V tiles of the four warps
  __shared__ int is_last;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [kDecodeStages][K|V][4][WK][RS]

  const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  // The prologue is a chain of dependent reads (lengths -> table -> tiles; row -> query), each a
  // trip to L2: everything that has its address is asked for before anything is used.
  const int base_b = base_len[b], slot = slot_ids[b], row_b = q_start[b];
  // A sequence longer than the launch was sized for (a captured step replayed past its length
  // bucket): the keys beyond the grid are not read, the chunk count stays within the grid (so the
  // counters end at zero and the row is written), and the status word says so.
  const bool past_grid = base_b + 1 > max_chunks * chunk_keys;
  const int kv_len = past_grid ? max_chunks * chunk_keys : base_b + 1;
  const float sl2 = scale * 1.4426950408889634f;     // scores, maxima and the partials' maxima are in the base-2 domain
  // The grid has max_chunks blocks per (sequence, kv head), sized for the longest sequence the launch
  // allows (a captured step: its whole length bucket).  A sequence's key tiles (one pipeline step of the
  // four warps each) are shared out evenly over the chunks it uses, the first chunks taking the odd
  // ones, so that a sequence at the start of a bucket does not leave the last block a sliver and the
  // others a fifth more than their share (0.5-0.7% of a decode step at batch 4 to 16).  Tiles start at
  // multiples of the tile size whatever the cut.
  const int n_tiles = (kv_len + 4 * WK - 1) / (4 * WK);
  // all of the grid's blocks while the join reads their partials in one trip (eight at once), else as
  // many as chunk_keys-long chunks would take
  const int n_chunks = max_chunks <= 8 ? min(max_chunks, n_tiles) : (kv_len + chunk_keys - 1) / chunk_keys;
  if (c >= n_chunks) return;
  const int tiles_each = n_tiles / n_chunks, tiles_odd = n_tiles % n_chunks;
  const int my_tiles = tiles_each + (c < tiles_odd ? 1 : 0);
  SIAR_STAMP(0);
  const int c0 = (c * tiles_each + min(c, tiles_odd)) * 4 * WK;
  const int c_end = min(kv_len, c0 + my_tiles * 4 * WK);
  const int n_it = my_tiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int* table = block_table + (size_t)slot * max_pages;
  // The page of a tile is read from the block table one step before the tile is requested, so
  // that the (dependent) table read never sits in front of the loads it feeds.
  // A block-table cell below zero is a page the sequence does not hold: its keys are read from
  // page 0 (an address that exists), the new token's key and value are not stored, and the status
  // word says so, so that the host raises instead of using the result.
  bool absent_page = false;
  auto page_of = [&](int it) {
    const int w0 = c0 + it * 4 * WK + warp * WK;
    int page = w0 < c_end ? __ldg(table + w0 / page_tokens) : 0;
    if (page < 0) { absent_page = true; page = 0; }
    return page;
  };
  auto load_tile = [&](int it, int stage, int page) {
    const int w0 = c0 + it * 4 * WK + warp * WK;
    const int valid = min(WK, c_end - w0);
    if (valid <= 0) return;
    const size_t row0 = ((size_t)page * Hkv + kvh) * page_tokens + (w0 % page_tokens);
    const __nv_bfloat16* kg = k_pool + row0 * D;
    const __nv_bfloat16* vg = v_pool + row0 * D;
    __nv_bfloat16* kw = tiles + stage * kStageElems + warp * WK * RS;
    __nv_bfloat16* vw = kw + 4 * WK * RS;
#pragma unroll
    for (int i = 0; i < WK * CPR / 32; ++i) {
      const int id = i * 32 + lane;
      const int r = id / CPR, ch = id % CPR;
      const int ok = r < valid ? 16 : 0;
      const size_t goff = (size_t)(ok ? r : 0) * D + ch * 8;
      cp_async_16(smem_u32_generic(kw + r * RS + ch * 8), kg + goff, ok);
      cp_async_16(smem_u32_generic(vw + r * RS + ch * 8), vg + goff, ok);
    }
  };
  int pages[kDecodeStages];
#pragma unroll
  for (int pre = 0; pre < kDecodeStages; ++pre) pages[pre] = page_of(pre);
#pragma unroll
  for (int pre = 0; pre < kDecodeStages - 1; ++pre) {
    if (pre < n_it) load_tile(pre, pre, pages[pre]);
    cp_async_commit();
  }
  SIAR_STAMP(7);
  int page_ahead = pages[kDecodeStages - 1];      // page of tile it + kDecodeStages - 1 at step it
  static_assert(D / 2 <= 128, "one thread per rotation frequency");
  const int pos = base_b;                          // position of the new token
  if (fuse_rope) {
    if (threadIdx.x < D / 2) {
      float sn = 0.f, cs = 1.f;
      if (inv_freq != nullptr) sincosf((float)pos * __ldg(inv_freq + threadIdx.x), &sn, &cs);
      cs_s[threadIdx.x] = cs;
      cs_s[D / 2 + threadIdx.x] = sn;
    }
  }
  if (early) {
    pdl_wait();            // the fused qkv rows of this step are complete
    SIAR_TRACE(20, 2);
  }
  // query fragments straight from global memory: rows g and g + 8 of the (padded) group
  const size_t tok_row = (size_t)row_b * (Hq + 2 * Hkv) * D;
  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* qrow = qkv + tok_row + (size_t)kvh * G * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int col = kk * 16 + q * 2;
      qa[kk][0] = g < G ? ld_after_wait_u32(qrow + (size_t)g * D + col) : 0u;
      qa[kk][1] = g + 8 < G ? ld_after_wait_u32(qrow + (size_t)(g + 8) * D + col) : 0u;
      qa[kk][2] = g < G ? ld_after_wait_u32(qrow + (size_t)g * D + col + 8) : 0u;
      qa[kk][3] = g + 8 < G ? ld_after_wait_u32(qrow + (size_t)(g + 8) * D + col + 8) : 0u;
    }
  }

  if (fuse_rope) __syncthreads();                  // cos / sin are in shared memory
  {
    if (fuse_rope) {
      // columns c < D/2 pair with c + D/2: fragment kk pairs with fragment kk + D/32, same register
#pragma unroll
      for (int kk = 0; kk < D / 32; ++kk) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int col = kk * 16 + q * 2 + (r >= 2 ? 8 : 0);
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[kk][r]));
          const float2 c2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[kk + D / 32][r]));
          const float c0v = cs_s[col], c1v = cs_s[col + 1], s0v = cs_s[D / 2 + col], s1v = cs_s[D / 2 + col + 1];
          qa[kk][r] = pack_bf16(a.x * c0v - c2.x * s0v, a.y * c1v - c2.y * s1v);
          qa[kk + D / 32][r] = pack_bf16(c2.x * c0v + a.x * s0v, c2.y * c1v + a.y * s1v);
        }
      }
    }
  }
  SIAR_STAMP(1);

  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  for (int it = 0; it < n_it; ++it) {
    const int stage = it % kDecodeStages;
    if (it + kDecodeStages - 1 < n_it)
      load_tile(it + kDecodeStages - 1, (it + kDecodeStages - 1) % kDecodeStages, page_ahead);
    cp_async_commit();
    page_ahead = page_of(it + kDecodeStages);       // used at the next step
    cp_async_wait<kDecodeStages - 1>();
    __syncwarp();
    if (it == 0) { SIAR_STAMP(2); }
    const int w0 = c0 + it * 4 * WK + warp * WK;
    const int valid = min(WK, c_end - w0);
    if (valid <= 0) continue;
    if (fuse_rope && write_kv && pos >= w0 && pos < w0 + WK) {
      // this warp's tile holds the new token: its k (rotated) and v come from the fused qkv row,
      // go to the cache for later steps and replace the row that cp.async just fetched
      const __nv_bfloat16* krow = qkv + tok_row + (size_t)(Hq + kvh) * D;
      const __nv_bfloat16* vrow = qkv + tok_row + (size_t)(Hq + Hkv + kvh) * D;
      __nv_bfloat16* ks = tiles + stage * kStageElems + warp * WK * RS + (pos - w0) * RS;
      __nv_bfloat16* vs = ks + 4 * WK * RS;
      const int page = __ldg(table + pos / page_tokens);
      const bool held = page >= 0;
      if (!held) absent_page = true;
      const size_t grow = (((size_t)(held ? page : 0) * Hkv + kvh) * page_tokens + (pos % page_tokens)) * D;
      __nv_bfloat16* kdst = const_cast<__nv_bfloat16*>(k_pool) + grow;
      __nv_bfloat16* vdst = const_cast<__nv_bfloat16*>(v_pool) + grow;
      for (int i = lane; i < D / 2; i += 32) {
        const float a = __bfloat162float(ld_after_wait_bf16(krow + i)), c2 = __bfloat162float(ld_after_wait_bf16(krow + i + D / 2));
        const __nv_bfloat16 oa = __float2bfloat16_rn(a * cs_s[i] - c2 * cs_s[D / 2 + i]);
        const __nv_bfloat16 oc = __float2bfloat16_rn(c2 * cs_s[i] + a * cs_s[D / 2 + i]);
        ks[i] = oa; ks[i + D / 2] = oc;
        if (held) { kdst[i] = oa; kdst[i + D / 2] = oc; }
      }
      for (int d = lane; d < D; d += 32) {
        const __nv_bfloat16 v = ld_after_wait_bf16(vrow + d);
        vs[d] = v;
        if (held) vdst[d] = v;
      }
      __syncwarp();
    }
    const uint32_t kbase = smem_u32_generic(tiles + stage * kStageElems + warp * WK * RS);
    const uint32_t vbase = kbase + 4 * WK * RS * 2;
    // S = Q K^T : WK/8 key tiles of 8
    float s[WK / 8][4];
#pragma unroll
    for (int j = 0; j < WK / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int j = 0; j < WK / 8; ++j) {
#pragma unroll
      for (int kk = 0; kk < D / 16; kk += 2) {
        uint32_t bfr[4];
        // matrices: dims 16kk + 8m .. +7 (m = 0..3) of keys 8j .. 8j+7
        ldmatrix_x4(bfr, kbase + (uint32_t)(((8 * j + (lane & 7)) * RS + 16 * kk + 8 * (lane >> 3)) * 2));
        mma_bf16_16816(s[j], qa[kk], bfr[0], bfr[1]);
        mma_bf16_16816(s[j], qa[kk + 1], bfr[2], bfr[3]);
      }
    }
    // mask, running maxima, exponentials
    float mx[2] = {m_row[0], m_row[1]};
#pragma unroll
    for (int j = 0; j < WK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = 8 * j + 2 * q + (e & 1);
        const float v = key < valid ? s[j][e] * sl2 : -INFINITY;      // scores in the base-2 domain
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    mx[0] = quad_max(mx[0]);
    mx[1] = quad_max(mx[1]);
    float alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) alpha[h] = mx[h] == -INFINITY ? 1.f : fast_exp2(m_row[h] - mx[h]);
#pragma unroll
    for (int j = 0; j < WK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = s[j][e] == -INFINITY ? 0.f : fast_exp2(s[j][e] - mx[e >> 1]);
        s[j][e] = p;
        sum[e >> 1] += p;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_row[h] = l_row[h] * alpha[h] + quad_sum(sum[h]);
      m_row[h] = mx[h];
    }
    // the accumulators are rescaled only when some row's maximum moved (rare after the first tiles)
    if (it > 0 && __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
        o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
      }
    }
    // O += P V : WK/16 key steps of 16, D/8 dim tiles
#pragma unroll
    for (int t = 0; t < WK / 16; ++t) {
      uint32_t pa[4] = {pack_bf16(s[2 * t][0], s[2 * t][1]), pack_bf16(s[2 * t][2], s[2 * t][3]),
                        pack_bf16(s[2 * t + 1][0], s[2 * t + 1][1]), pack_bf16(s[2 * t + 1][2], s[2 * t + 1][3])};
#pragma unroll
      for (int j = 0; j < D / 8; j += 2) {
        uint32_t bfr[4];
        // matrices: (keys 16t + 8(m%2) .. +7, dims 8j + 8(m/2) .. +7), transposed on load
        const int mi = lane >> 3;
        ldmatrix_x4_trans(bfr, vbase + (uint32_t)(((16 * t + 8 * (mi & 1) + (lane & 7)) * RS + 8 * j + 8 * (mi >> 1)) * 2));
        mma_bf16_16816(o[j], pa, bfr[0], bfr[1]);
        mma_bf16_16816(o[j + 1], pa, bfr[2], bfr[3]);
      }
    }
  }
  cp_async_wait<0>();

  if (absent_page && status != nullptr && lane == 0) atomicOr(status, kStatusBadPage);
  if (past_grid && status != nullptr && threadIdx.x == 0) atomicOr(status, kStatusLengthPastGrid);
  // join the four warps: reuse the tile memory as float buffers
  SIAR_STAMP(3);
  __syncthreads();
  constexpr int MS = D + kJoinPad;                            // padded row: the eight rows a warp stores at once
                                                              // fall into different banks
  float* mo = reinterpret_cast<float*>(smem_raw);            // [4][16][MS]
  float* mm = mo + 4 * 16 * MS;                               // [4][16]
  float* ml = mm + 4 * 16;                                    // [4][16]
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const int d = 8 * j + 2 * q;
    if (g < G) *reinterpret_cast<float2*>(mo + (warp * 16 + g) * MS + d) = make_float2(o[j][0], o[j][1]);
    if (g + 8 < G) *reinterpret_cast<float2*>(mo + (warp * 16 + g + 8) * MS + d) = make_float2(o[j][2], o[j][3]);
  }
  if (q == 0) {
    mm[warp * 16 + g] = m_row[0]; ml[warp * 16 + g] = l_row[0];
    mm[warp * 16 + g + 8] = m_row[1]; ml[warp * 16 + g + 8] = l_row[1];
  }
  __syncthreads();
  __nv_bfloat16* orow = out + (size_t)q_start[b] * Hq * D + (size_t)kvh * G * D;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int h = idx / D, d = idx % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, mm[w * 16 + h]);
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mm[w * 16 + h];
      if (mw != -INFINITY) {
        const float f = fast_exp2(mw - mx);
        acc += mo[(w * 16 + h) * MS + d] * f;
        lsum += ml[w * 16 + h] * f;
      }
    }
    if (n_chunks == 1) {                       // the only chunk: finish here, no scratch
      orow[h * D + d] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    } else {
      const size_t pidx = ((size_t)b * Hq + kvh * G + h) * max_chunks + c;
      part_acc[pidx * D + d] = acc;
      if (d == 0) { part_ml[pidx * 2] = mx; part_ml[pidx * 2 + 1] = lsum; }
    }
  }
  SIAR_STAMP(4);
  if (n_chunks == 1) { SIAR_TRACE(20, 1); return; }

  // The block of this (sequence, kv head) that finishes last joins the chunks' partials
  // in chunk order (so the result does not depend on which block that was).
  // (Measured and not kept: the chunks of a (sequence, kv head) as one thread-block cluster along x,
  // partials left in shared memory, block 0 reading them through distributed shared memory between
  // two cluster barriers, so that neither scratch, fence nor counter is on the way.  A decode step at
  // batch 4 and 8 became 0.9 us a layer slower: a cluster's blocks are placed together, so fewer of
  // them are resident before the product in front has left, and every block stays until block 0 has
  // read, which holds back the blocks of the product behind.)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(counters + b * Hkv + kvh, 1);
    is_last = (old == n_chunks - 1);
    if (old == n_chunks - 1) counters[b * Hkv + kvh] = 0;
  }
  __syncthreads();
  SIAR_STAMP(5);
  if (!is_last) { SIAR_TRACE(20, 1); return; }
  __threadfence();
  // Each thread joins its output's partials itself, chunk after chunk with a running maximum (the
  // order of a sequential softmax, whatever block does it): the maxima, sums and values of eight
  // chunks are asked for together, so the join costs one trip to L2 per eight chunks and no barrier.
  const size_t pbase = ((size_t)b * Hq + kvh * G) * max_chunks;
  for (int item = threadIdx.x; item < G * (D / 4); item += blockDim.x) {     // four outputs of one head per thread
    const int h = item / (D / 4), d = (item % (D / 4)) * 4;
    const float2* pml = reinterpret_cast<const float2*>(part_ml) + pbase + (size_t)h * max_chunks;
    const float* pa = part_acc + (pbase + (size_t)h * max_chunks) * D + d;
    float run_m = -INFINITY, run_l = 0.f;
    float4 run_a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int cc = 0; cc < n_chunks; cc += 8) {
      float2 ml8[8];
      float4 a8[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool in = cc + u < n_chunks;
        ml8[u] = in ? __ldcg(pml + cc + u) : make_float2(-INFINITY, 0.f);
        a8[u] = in ? __ldcg(reinterpret_cast<const float4*>(pa + (size_t)(cc + u) * D)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float m_new = fmaxf(run_m, ml8[u].x);
        if (m_new != -INFINITY) {
          const float f_old = fast_exp2(run_m - m_new), f_new = fast_exp2(ml8[u].x - m_new);
          run_a.x = run_a.x * f_old + a8[u].x * f_new;
          run_a.y = run_a.y * f_old + a8[u].y * f_new;
          run_a.z = run_a.z * f_old + a8[u].z * f_new;
          run_a.w = run_a.w * f_old + a8[u].w * f_new;
          run_l = run_l * f_old + ml8[u].y * f_new;
          run_m = m_new;
        }
      }
    }
    const float inv = run_l > 0.f ? 1.f / run_l : 0.f;
    uint2 pk;
    pk.x = pack_bf16(run_a.x * inv, run_a.y * inv);
    pk.y = pack_bf16(run_a.z * inv, run_a.w * inv);
    *reinterpret_cast<uint2*>(orow + h * D + d) = pk;
  }
  SIAR_STAMP(6);
  SIAR_TRACE(20, 1);
}

// ------------------------------------------------------------------ prefill
// grid (row tiles, Hkv, B), 128 threads.  Shared memory (bf16):
//   q_s[64][D+8], k_s[2][64][D+8], v_s[2][64][D+8].
template <int D>
__global__ void __launch_bounds__(128)
attn_prefill_mma_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ block_table,
                        const int* __restrict__ slot_ids, const int* __restrict__ q_start,
                        const int* __restrict__ base_len, __nv_bfloat16* __restrict__ out, int Hq, int Hkv,
                        int page_tokens, int max_pages, float scale, int* __restrict__ status) {
  pdl_launch_dependents();
  SIAR_TRACE(21, 0);
  pdl_wait();
  SIAR_TRACE(21, 2);
  constexpr int RS = D + kPad;
  constexpr int CPR = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* k_s = q_s + kMmaPrefillRows * RS;
  __nv_bfloat16* v_s = k_s + 2 * kMmaKeyTile * RS;

  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = Hq / Hkv;
  const int t0 = q_start[b];
  const int q_len = q_start[b + 1] - t0;
  const int rows_total = q_len * G;
  const int row0 = blockIdx.x * kMmaPrefillRows;
  if (row0 >= rows_total) return;
  const int rows_here = min(kMmaPrefillRows, rows_total - row0);
  const int base = base_len[b];
  const int slot = slot_ids[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int qkv_stride = (Hq + 2 * Hkv) * D;
  const int block_kv_end = base + (row0 + rows_here - 1) / G + 1;
  const int n_tiles = (block_kv_end + kMmaKeyTile - 1) / kMmaKeyTile;

  // ---- stage the query rows
  for (int id = threadIdx.x; id < kMmaPrefillRows * CPR; id += blockDim.x) {
    const int r = id / CPR, ch = id % CPR;
    const int ok = r < rows_here ? 16 : 0;
    const int rr = ok ? row0 + r : row0;
    const __nv_bfloat16* src = qkv + (size_t)(t0 + rr / G) * qkv_stride + (size_t)(kvh * G + rr % G) * D + ch * 8;
    cp_async_16(smem_u32_generic(q_s + r * RS + ch * 8), src, ok);
  }
  const int* table = block_table + (size_t)slot * max_pages;
  // a cell below zero (a page the sequence does not hold) is read as page 0, an address that
  // exists, and reported through the status word
  bool absent_page = false;
  auto page_of = [&](int tile) {
    int page = tile < n_tiles ? __ldg(table + tile * kMmaKeyTile / page_tokens) : 0;
    if (page < 0) { absent_page = true; page = 0; }
    return page;
  };
  auto load_tile = [&](int tile, int stage, int page) {
    const int j0 = tile * kMmaKeyTile;
    const int valid = min(kMmaKeyTile, block_kv_end - j0);
    const size_t grow = ((size_t)page * Hkv + kvh) * page_tokens + (j0 % page_tokens);
    const __nv_bfloat16* kg = k_pool + grow * D;
    const __nv_bfloat16* vg = v_pool + grow * D;
    __nv_bfloat16* ks = k_s + stage * kMmaKeyTile * RS;
    __nv_bfloat16* vs = v_s + stage * kMmaKeyTile * RS;
    for (int id = threadIdx.x; id < kMmaKeyTile * CPR; id += blockDim.x) {
      const int r = id / CPR, ch = id % CPR;
      const int ok = r < valid ? 16 : 0;
      const size_t goff = (size_t)(ok ? r : 0) * D + ch * 8;
      cp_async_16(smem_u32_generic(ks + r * RS + ch * 8), kg + goff, ok);
      cp_async_16(smem_u32_generic(vs + r * RS + ch * 8), vg + goff, ok);
    }
  };
  int page_next = page_of(1);           // read one tile ahead of its use
  load_tile(0, 0, page_of(0));
  cp_async_commit();

  // rows of this thread: warp*16 + g and + 8
  int kv_end[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    kv_end[h] = r < rows_here ? base + (row0 + r) / G + 1 : 0;
  }
  // the furthest key any row of this warp sees (warp-uniform)
  const int warp_last_row = min(rows_here - 1, warp * 16 + 15);
  const int warp_kv_end = warp * 16 < rows_here ? base + (row0 + warp_last_row) / G + 1 : 0;
  // the nearest limit of any row of this warp (rows past rows_here count as 0: always masked)
  const int warp_kv_min = warp * 16 + 15 < rows_here ? base + (row0 + warp * 16) / G + 1 : 0;
  const float sl2 = scale * 1.4426950408889634f;

  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  uint32_t qa[D / 16][4];

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) load_tile(tile + 1, stage ^ 1, page_next);
    cp_async_commit();
    page_next = page_of(tile + 2);
    cp_async_wait<1>();
    __syncthreads();
    if (tile == 0) {
      const uint32_t qbase = smem_u32_generic(q_s + warp * 16 * RS);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qa[kk], qbase + (uint32_t)((((lane & 7) + 8 * ((lane >> 3) & 1)) * RS + 16 * kk + 8 * (lane >> 4)) * 2));
    }
    const int j0 = tile * kMmaKeyTile;
    if (j0 < warp_kv_end) {
      float s[kMmaKeyTile / 8][4];
#pragma unroll
      for (int j = 0; j < kMmaKeyTile / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      const uint32_t kbase = smem_u32_generic(k_s + stage * kMmaKeyTile * RS);
#pragma unroll
      for (int j = 0; j < kMmaKeyTile / 8; ++j) {
#pragma unroll
        for (int kk = 0; kk < D / 16; kk += 2) {
          uint32_t bfr[4];
          ldmatrix_x4(bfr, kbase + (uint32_t)(((8 * j + (lane & 7)) * RS + 16 * kk + 8 * (lane >> 3)) * 2));
          mma_bf16_16816(s[j], qa[kk], bfr[0], bfr[1]);
          mma_bf16_16816(s[j], qa[kk + 1], bfr[2], bfr[3]);
        }
      }
      // Softmax in the base-2 domain: with c = scale * log2(e), exp(s * scale - m) = 2^(s c - m c),
      // one FFMA and one EX2 per score; m_row holds the running maximum of s * c.  Keys past a
      // row's own position are masked only in the tiles that reach that far (warp-uniform test).
      if (j0 + kMmaKeyTile > warp_kv_min) {
#pragma unroll
        for (int j = 0; j < kMmaKeyTile / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (j0 + 8 * j + 2 * q + (e & 1) >= kv_end[e >> 1]) s[j][e] = -INFINITY;
      }
      float raw[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < kMmaKeyTile / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) raw[e >> 1] = fmaxf(raw[e >> 1], s[j][e]);
      float mx[2], alpha[2], neg_m[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(m_row[h], quad_max(raw[h]) * sl2);
        alpha[h] = mx[h] == -INFINITY ? 1.f : fast_exp2(m_row[h] - mx[h]);
        neg_m[h] = mx[h] == -INFINITY ? 0.f : -mx[h];
      }
#pragma unroll
      for (int j = 0; j < kMmaKeyTile / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = fast_exp2(fmaf(s[j][e], sl2, neg_m[e >> 1]));   // 2^(-inf) = 0 for masked keys
          s[j][e] = p;
          sum[e >> 1] += p;
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        l_row[h] = l_row[h] * alpha[h] + quad_sum(sum[h]);
        m_row[h] = mx[h];
      }
      // the output only needs rescaling when some row's maximum moved (rare after the first tiles)
      if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
          o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
        }
      }
      const uint32_t vbase = smem_u32_generic(v_s + stage * kMmaKeyTile * RS);
#pragma unroll
      for (int t = 0; t < kMmaKeyTile / 16; ++t) {
        uint32_t pa[4] = {pack_bf16(s[2 * t][0], s[2 * t][1]), pack_bf16(s[2 * t][2], s[2 * t][3]),
                          pack_bf16(s[2 * t + 1][0], s[2 * t + 1][1]), pack_bf16(s[2 * t + 1][2], s[2 * t + 1][3])};
#pragma unroll
        for (int j = 0; j < D / 8; j += 2) {
          uint32_t bfr[4];
          const int mi = lane >> 3;
          ldmatrix_x4_trans(bfr, vbase + (uint32_t)(((16 * t + 8 * (mi & 1) + (lane & 7)) * RS + 8 * j + 8 * (mi >> 1)) * 2));
          mma_bf16_16816(o[j], pa, bfr[0], bfr[1]);
          mma_bf16_16816(o[j + 1], pa, bfr[2], bfr[3]);
        }
      }
    }
    __syncthreads();   // everyone is done with this stage before it is refilled
  }

  if (absent_page && status != nullptr && threadIdx.x == 0) atomicOr(status, kStatusBadPage);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    if (r >= rows_here) continue;
    const int rr = row0 + r;
    const float inv = l_row[h] > 0.f ? 1.f / l_row[h] : 0.f;
    __nv_bfloat16* dst = out + (size_t)(t0 + rr / G) * Hq * D + (size_t)(kvh * G + rr % G) * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const int d = 8 * j + 2 * q;
      *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
    }
  }
}

// Keys per decode block for a batch of B sequences with kv heads Hkv and lengths up to
// max_kv_len: a multiple of 128 (t tiles of 128 keys).  kDecodeBlocksPerSM blocks fit on an SM; a block
// costs a fixed part (set-up, joining its warps, the partial, the counter) plus a part per
// tile, and blocks run in waves of kDecodeBlocksPerSM * sm_count.  The t with the smallest estimate wins, with
// at most 64 chunks per sequence.  (Measured on B200: about 6 us fixed and 2.8 us per tile
// with three blocks sharing an SM's bandwidth.  An estimate that let a block's fixed part hide behind
// its neighbour's streaming, and so cut batch 64 at 2,048 keys into two chunks per sequence instead of
// one, 1,024 blocks instead of 512, was 6% slower there: a block alone does not draw an SM's whole
// share of the bandwidth.)
static int decode_chunk_keys(int B, int Hkv, int max_kv_len, int sm_count) {
  const int tiles = (max_kv_len + kMmaDecodeChunk - 1) / kMmaDecodeChunk;
  const long long pairs = (long long)B * Hkv;
  const long long slots = (long long)kDecodeBlocksPerSM * sm_count;
  int best_t = tiles;
  double best = 1e30;
  for (int t = (tiles + 63) / 64; t <= tiles; ++t) {
    const long long chunks = (tiles + t - 1) / t;
    const long long waves = (pairs * chunks + slots - 1) / slots;
    const double fixed = chunks > 1 ? 6.0 : 4.0;
    const double cost = (double)waves * (fixed + 2.8 * t);
    if (cost < best - 1e-9) { best = cost; best_t = t; }
  }
  return best_t * kMmaDecodeChunk;
}

template <int D>
static int launch_decode(const void* qkv, const void* k_pool, const void* v_pool, const int* block_table,
                         const int* slot_ids, const int* q_start, const int* base_len, void* out, float* scratch,
                         int* counters, int B, int Hq, int Hkv, int page_tokens, int max_pages, int max_kv_len,
                         int sm_count, float scale, cudaStream_t s, const float* inv_freq = nullptr,
                         int fuse_rope = 0, int write_kv = 1, int* status = nullptr) {
  const int chunk_keys = decode_chunk_keys(B, Hkv, max_kv_len, sm_count);
  const int max_chunks = (max_kv_len + chunk_keys - 1) / chunk_keys;
  float* part_ml = scratch;
  float* part_acc = scratch + (size_t)B * Hq * max_chunks * 2;
  size_t smem = (size_t)kDecodeStages * 2 * 4 * decode_warp_keys(D) * (D + kPad) * 2;   // stages of K and V tiles
  const size_t merge = sizeof(float) * (4 * 16 * (D + kJoinPad) + 2 * 4 * 16);
  if (merge > smem) smem = merge;
  auto kern = attn_decode_mma_kernel<D>;
  // the shared-memory limit of a kernel is a property of the device's copy of it: set once per device
  static bool attr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  if (!attr[dev] && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr[dev] = true;
  }
  dim3 grid(max_chunks, Hkv, B);
  return (int)launch_kernel(kern, grid, dim3(128), smem, s, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)k_pool,
                            (const __nv_bfloat16*)v_pool, block_table, slot_ids, q_start, base_len, part_ml, part_acc,
                            counters, (__nv_bfloat16*)out, Hq, Hkv, page_tokens, max_pages, max_chunks, chunk_keys,
                            scale, inv_freq, fuse_rope, write_kv, status);
}

template <int D>
static int launch_prefill(const void* qkv, const void* k_pool, const void* v_pool, const int* block_table,
                          const int* slot_ids, const int* q_start, const int* base_len, void* out, int B, int Hq,
                          int Hkv, int page_tokens, int max_pages, int max_q_len, float scale, cudaStream_t s,
                          int* status) {
  const int G = Hq / Hkv;
  const size_t smem = (size_t)(kMmaPrefillRows + 4 * kMmaKeyTile) * (D + kPad) * 2;
  auto kern = attn_prefill_mma_kernel<D>;
  static bool attr = false;
  if (!attr && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  dim3 grid((max_q_len * G + kMmaPrefillRows - 1) / kMmaPrefillRows, Hkv, B);
  return (int)launch_kernel(kern, grid, dim3(128), smem, s, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)k_pool,
                            (const __nv_bfloat16*)v_pool, block_table, slot_ids, q_start, base_len,
                            (__nv_bfloat16*)out, Hq, Hkv, page_tokens, max_pages, scale, status);
}

}  // namespace siar

using namespace siar;

SIAR_DEFINE_PDL_SWITCH()

// Scratch floats siar_attn_mma_decode needs: the worst case is chunks of 128 keys.

#ifdef SIAR_TIMING
extern "C" void siar_attn_set_stamps(unsigned long long* p) { cudaMemcpyToSymbol(siar::g_attn_stamps, &p, sizeof(p)); }
#endif

// 1 when the tensor-core kernels take these sizes (bf16 only): head_dim 64 or 128, at most
// 16 query heads per kv head, pages that hold whole key tiles.
extern "C" int siar_attn_mma_supported(int Hq, int Hkv, int D, int page_tokens) {
  if (Hkv <= 0 || Hq % Hkv != 0) return 0;
  return (D == 64 || D == 128) && (Hq / Hkv) <= 16 && page_tokens % kMmaKeyTile == 0;
}

extern "C" long long siar_attn_mma_decode_scratch_floats(int B, int Hq, int Hkv, int D, int max_kv_len,
                                                         int sm_count) {
  const int chunk_keys = decode_chunk_keys(B, Hkv, max_kv_len, sm_count);
  const long long chunks = (max_kv_len + chunk_keys - 1) / chunk_keys;
  return (long long)B * Hq * chunks * (D + 2);
}

// counters: B * Hkv int32 zeros (left zero on return); scratch: siar_attn_mma_decode_scratch_floats floats.
extern "C" int siar_attn_mma_decode(const void* qkv, const void* k_pool, const void* v_pool, const int* block_table,
                                    const int* slot_ids, const int* q_start, const int* base_len, void* out,
                                    float* scratch, int* counters, int B, int Hq, int Hkv, int D, int page_tokens,
                                    int max_pages, int max_kv_len, int sm_count, float scale, void* stream,
                                    int* status) {
  if (B == 0) return 0;
  if (!siar_attn_mma_supported(Hq, Hkv, D, page_tokens) || Hkv > 65535 || B > 65535 || max_kv_len <= 0)
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 64)
    return launch_decode<64>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, scratch, counters,
                             B, Hq, Hkv, page_tokens, max_pages, max_kv_len, sm_count, scale, s, nullptr, 0, 1, status);
  return launch_decode<128>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, scratch, counters, B,
                            Hq, Hkv, page_tokens, max_pages, max_kv_len, sm_count, scale, s, nullptr, 0, 1, status);
}

// The same with the rotary encoding and the cache write of the new token fused in: qkv holds the
// product's output (q and k not rotated), inv_freq the rotary frequencies (nullptr: no rotation),
// write_kv == 0 leaves the cache alone (a layer that reads another layer's cache).  The kernel
// rotates the whole head in pairs (i, i + D/2); any other rotary layout (rotary_dim != D, interleaved
// pairs) is refused with cudaErrorInvalidValue, and the caller runs the separate rotary kernel.
extern "C" int siar_attn_mma_decode_rope(const void* qkv, void* k_pool, void* v_pool, const int* block_table,
                                         const int* slot_ids, const int* q_start, const int* base_len, void* out,
                                         float* scratch, int* counters, const float* inv_freq, int write_kv, int B,
                                         int Hq, int Hkv, int D, int page_tokens, int max_pages, int max_kv_len,
                                         int sm_count, float scale, void* stream, int* status, int rotary_dim,
                                         int interleaved) {
  if (B == 0) return 0;
  if (!siar_attn_mma_supported(Hq, Hkv, D, page_tokens) || Hkv > 65535 || B > 65535 || max_kv_len <= 0)
    return (int)cudaErrorInvalidValue;
  if (inv_freq != nullptr && (rotary_dim != D || interleaved)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 64)
    return launch_decode<64>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, scratch, counters,
                             B, Hq, Hkv, page_tokens, max_pages, max_kv_len, sm_count, scale, s, inv_freq, 1,
                             write_kv, status);
  return launch_decode<128>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, scratch, counters, B,
                            Hq, Hkv, page_tokens, max_pages, max_kv_len, sm_count, scale, s, inv_freq, 1, write_kv,
                            status);
}

extern "C" int siar_attn_mma_prefill(const void* qkv, const void* k_pool, const void* v_pool, const int* block_table,
                                     const int* slot_ids, const int* q_start, const int* base_len, void* out, int B,
                                     int Hq, int Hkv, int D, int page_tokens, int max_pages, int max_q_len,
                                     float scale, void* stream, int* status) {
  if (B == 0 || max_q_len == 0) return 0;
  if (!siar_attn_mma_supported(Hq, Hkv, D, page_tokens) || Hkv > 65535 || B > 65535)
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 64)
    return launch_prefill<64>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, B, Hq, Hkv,
                              page_tokens, max_pages, max_q_len, scale, s, status);
  return launch_prefill<128>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, B, Hq, Hkv,
                             page_tokens, max_pages, max_q_len, scale, s, status);
}

// ------------------------------------------------------------------ decode without allocation
// See no_alloc.h.  One array in the shared object serves as the scratch of
// siar_attn_mma_decode: the first SIAR_NOALLOC_MAX_PAIRS 32-bit words are the counters, the
// rest holds the float partials.  In host code `noalloc_scratch` is only a handle for the
// symbol, not a device address; the address comes from cudaGetSymbolAddress.
#include "no_alloc.h"

#include <stdio.h>

static __device__ __align__(256) float noalloc_scratch[SIAR_NOALLOC_SCRATCH_BYTES / sizeof(float)];

static float* noalloc_base[64];   // device address of the array, per device, looked up once

extern "C" long long siar_attn_mma_noalloc_max_floats(void) {
  return (long long)(SIAR_NOALLOC_SCRATCH_BYTES / sizeof(float)) - SIAR_NOALLOC_MAX_PAIRS;
}

extern "C" int siar_attn_mma_decode_noalloc(const void* qkv, const void* k_pool, const void* v_pool,
                                            const int* block_table, const int* slot_ids, const int* q_start,
                                            const int* base_len, void* out, int B, int Hq, int Hkv, int D,
                                            int page_tokens, int max_pages, int max_kv_len, int sm_count,
                                            float scale, void* stream, char* message, int message_len) {
  auto say = [&](const char* fmt, long long a, long long b) {
    if (message != nullptr && message_len > 0) snprintf(message, (size_t)message_len, fmt, a, b);
  };
  if (message != nullptr && message_len > 0) message[0] = 0;
  if (B <= 0) return 0;
  if (!siar_attn_mma_supported(Hq, Hkv, D, page_tokens) || B > 65535 || max_kv_len <= 0 || sm_count <= 0) {
    say("sizes not taken by the tensor-core decode attention (head_dim %lld, %lld query heads per kv head)",
        (long long)D, (long long)(Hkv > 0 ? Hq / Hkv : 0));
    return -2;
  }
  const long long need = siar_attn_mma_decode_scratch_floats(B, Hq, Hkv, D, max_kv_len, sm_count);
  if (need > siar_attn_mma_noalloc_max_floats()) {
    say("these sizes need %lld floats of scratch; the built-in array holds %lld", need,
        siar_attn_mma_noalloc_max_floats());
    return -3;
  }
  if ((long long)B * Hkv > SIAR_NOALLOC_MAX_PAIRS) {
    say("%lld (sequence, kv head) pairs; the built-in array has counters for %lld", (long long)B * Hkv,
        (long long)SIAR_NOALLOC_MAX_PAIRS);
    return -3;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    say("cudaGetDevice failed or device index out of range (error %lld, device %lld)", (long long)e, (long long)dev);
    return e != cudaSuccess ? (int)e : (int)cudaErrorInvalidDevice;
  }
  if (noalloc_base[dev] == nullptr) {
    // set-up, once per device: the device address of the array on the current device
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      say("cudaGetSymbolAddress failed (error %lld) on device %lld", (long long)e, (long long)dev);
      return e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol;
    }
    noalloc_base[dev] = ptr;
  }
  int* counters = reinterpret_cast<int*>(noalloc_base[dev]);
  float* partials = noalloc_base[dev] + SIAR_NOALLOC_MAX_PAIRS;
  cudaStream_t s = (cudaStream_t)stream;
  // the counters must start at zero; an earlier call that was cut short may have left some
  e = cudaMemsetAsync(counters, 0, sizeof(int) * (size_t)B * Hkv, s);
  if (e != cudaSuccess) {
    say("cudaMemsetAsync on the counters failed (error %lld) on device %lld", (long long)e, (long long)dev);
    return (int)e;
  }
  int rc;
  if (D == 64)
    rc = launch_decode<64>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, partials, counters, B,
                           Hq, Hkv, page_tokens, max_pages, max_kv_len, sm_count, scale, s);
  else
    rc = launch_decode<128>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, partials, counters,
                            B, Hq, Hkv, page_tokens, max_pages, max_kv_len, sm_count, scale, s);
  if (rc != 0) say("the kernel launch failed (error %lld) on device %lld", (long long)rc, (long long)dev);
  return rc;
}
