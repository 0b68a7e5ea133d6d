// Causal grouped-query attention over the paged cache, on the CUDA cores with
// 32-bit softmax state.  Two kernels:
//
//  * attn_prefill: any mix of new-token counts.  Row i of sequence b (absolute
//    position p = base_len[b] + i) sees keys [0, p] of its own slot: the
//    bottom-right aligned causal rule of the reference's flash kernel
//    (kernels/attention_kernel.py:184,206-209).  Scores are (q . k) * scale with
//    the scale applied after the dot (kernels/attention_kernel.py:204), the softmax
//    is the running-max form (kernels/attention_kernel.py:212-222), the output is
//    divided by the row sum at the end and a row without keys yields 0
//    (kernels/attention_kernel.py:225-226).  Query head hq reads kv head hq / G
//    (kernels/attention_kernel.py:169).
//  * attn_decode (+ combine): one new token per sequence.  The keys of a
//    sequence are cut into chunks of kDecodeChunk positions at absolute
//    boundaries; one block per (chunk, kv head, sequence) produces a partial
//    (max, sum, weighted values) for each of the G query heads into scratch
//    memory, and a second kernel joins the partials in chunk order.  The
//    reference's decode kernel walks all keys in one program
//    (kernels/flash_decode_kernel.py:89-114); splitting is what fills 148 SMs at
//    small batch.
//
// Keys are always consumed in tiles of 32 that start at multiples of 32, so the
// order of the floating-point reduction for a row depends only on its position.
#include "common.cuh"

#include <math.h>

namespace siar {

constexpr int kTile = 32;
constexpr int kPrefillRows = 16;   // rows (query x head-in-group) per block
constexpr int kPrefillWarps = 8;
constexpr int kDecodeChunk = 256;  // keys per decode block
constexpr int kDecodeWarps = 4;
constexpr int kDecodeRound = kDecodeWarps * kTile;  // keys staged in shared memory at a time

template <typename T>
__device__ __forceinline__ const T* key_row(const T* __restrict__ pool, const int* __restrict__ block_table,
                                            int slot, int max_pages, int page_tokens, int Hkv, int kvh, int D,
                                            int key, int* __restrict__ status) {
  // a cell below zero is a page the sequence does not hold: read page 0, an address that
  // exists, and say so through the status word, so that the host raises instead of using the result
  int page = block_table[(size_t)slot * max_pages + key / page_tokens];
  if (page < 0) {
    if (status != nullptr) atomicOr(status, kStatusBadPage);
    page = 0;
  }
  return pool + (((size_t)page * Hkv + kvh) * page_tokens + (key % page_tokens)) * D;
}

// ------------------------------------------------------------------ prefill
// grid (row tiles, Hkv, B), 256 threads.  Shared memory (floats):
//   q_s[kPrefillRows][D], k_s[kTile][D + 1], v_s[kTile][D].
template <typename T, int NDIM>
__global__ void __launch_bounds__(kPrefillWarps * 32)
attn_prefill_kernel(const T* __restrict__ qkv, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                    const int* __restrict__ block_table, const int* __restrict__ slot_ids,
                    const int* __restrict__ q_start, const int* __restrict__ base_len, T* __restrict__ out,
                    int Hq, int Hkv, int D, int page_tokens, int max_pages, float scale, int window,
                    int* __restrict__ status) {
  // window > 0: a query at position p sees keys p - window + 1 .. p only (0 = all keys up to p);
  // keys in front of a block's first window are never touched (their pages may be gone).
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = Hq / Hkv;
  const int t0 = q_start[b];
  const int q_len = q_start[b + 1] - t0;
  const int rows_total = q_len * G;
  const int row0 = blockIdx.x * kPrefillRows;
  if (row0 >= rows_total) return;
  const int base = base_len[b];
  const int slot = slot_ids[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qkv_stride = (Hq + 2 * Hkv) * D;

  float* q_s = smem;
  float* k_s = q_s + kPrefillRows * D;
  float* v_s = k_s + kTile * (D + 1);

  const int rows_here = min(kPrefillRows, rows_total - row0);
  for (int idx = threadIdx.x; idx < kPrefillRows * D; idx += blockDim.x) {
    const int r = idx / D, d = idx % D;
    float v = 0.f;
    if (r < rows_here) {
      const int ql = (row0 + r) / G, g = (row0 + r) % G;
      v = to_f32(qkv[(size_t)(t0 + ql) * qkv_stride + (size_t)(kvh * G + g) * D + d]);
    }
    q_s[idx] = v;
  }

  constexpr int RPW = kPrefillRows / kPrefillWarps;
  float m[RPW], l[RPW], acc[RPW][NDIM];
  int kv_end[RPW], kv_begin[RPW];
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
    const int r = warp * RPW + i;
    kv_end[i] = (r < rows_here) ? base + (row0 + r) / G + 1 : 0;
    kv_begin[i] = window > 0 ? max(0, kv_end[i] - window) : 0;
#pragma unroll
    for (int n = 0; n < NDIM; ++n) acc[i][n] = 0.f;
  }
  const int block_kv_end = base + (row0 + rows_here - 1) / G + 1;
  const int block_kv_begin = window > 0 ? max(0, base + row0 / G + 1 - window) : 0;

  for (int j0 = (block_kv_begin / kTile) * kTile; j0 < block_kv_end; j0 += kTile) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < kTile * D; idx += blockDim.x) {
      const int j = idx / D, d = idx % D;
      const int key = j0 + j;
      float kval = 0.f, vval = 0.f;
      if (key < block_kv_end && key >= block_kv_begin) {
        kval = to_f32(key_row(k_pool, block_table, slot, max_pages, page_tokens, Hkv, kvh, D, key, status)[d]);
        vval = to_f32(key_row(v_pool, block_table, slot, max_pages, page_tokens, Hkv, kvh, D, key, status)[d]);
      }
      k_s[j * (D + 1) + d] = kval;
      v_s[j * D + d] = vval;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      if (j0 >= kv_end[i] || j0 + kTile <= kv_begin[i]) continue;  // whole tile masked for this row (warp-uniform)
      const float* q = q_s + (warp * RPW + i) * D;
      const float* kr = k_s + lane * (D + 1);
      float s = 0.f;
      for (int d = 0; d < D; ++d) s = fmaf(q[d], kr[d], s);
      const bool valid = (j0 + lane) < kv_end[i] && (j0 + lane) >= kv_begin[i];
      s = valid ? s * scale : -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(s));
      const float alpha = expf(m[i] - m_new);
      const float p = valid ? expf(s - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(p);
      m[i] = m_new;
#pragma unroll
      for (int n = 0; n < NDIM; ++n) acc[i][n] *= alpha;
      for (int j = 0; j < kTile; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
        for (int n = 0; n < NDIM; ++n) {
          const int d = lane + 32 * n;
          if (d < D) acc[i][n] = fmaf(pj, v_s[j * D + d], acc[i][n]);
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int r = warp * RPW + i;
    if (r >= rows_here) continue;
    const int ql = (row0 + r) / G, g = (row0 + r) % G;
    const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
    T* o = out + (size_t)(t0 + ql) * Hq * D + (size_t)(kvh * G + g) * D;
#pragma unroll
    for (int n = 0; n < NDIM; ++n) {
      const int d = lane + 32 * n;
      if (d < D) o[d] = from_f32<T>(acc[i][n] * inv);
    }
  }
}

// ------------------------------------------------------------------ decode, partials
// grid (chunks, Hkv, B), 128 threads.  Shared memory:
//   T   k_s[kDecodeRound][D + KPAD], v_s[kDecodeRound][D]
//   f32 q_s[G][D], st_m[W][G], st_l[W][G], st_acc[W][G][D]
// Scratch layout: part_ml[(b*Hq + hq) * max_chunks + c][2], part_acc[... ][D].
template <typename T>
__global__ void __launch_bounds__(kDecodeWarps * 32)
attn_decode_partial_kernel(const T* __restrict__ qkv, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                           const int* __restrict__ block_table, const int* __restrict__ slot_ids,
                           const int* __restrict__ q_start, const int* __restrict__ base_len,
                           float* __restrict__ part_ml, float* __restrict__ part_acc, int Hq, int Hkv, int D,
                           int page_tokens, int max_pages, int max_chunks, float scale, int window,
                           int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  int kv_len = base_len[b] + 1;
  if (kv_len > max_chunks * kDecodeChunk) {
    // the sequence is longer than the launch was sized for (a captured step replayed past its
    // length bucket): the keys beyond the grid are not read, and the status word says so
    if (status != nullptr && threadIdx.x == 0) atomicOr(status, kStatusLengthPastGrid);
    kv_len = max_chunks * kDecodeChunk;
  }
  const int c0 = c * kDecodeChunk;
  if (c0 >= kv_len) return;
  const int c_end = min(kv_len, c0 + kDecodeChunk);
  const int slot = slot_ids[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_begin = window > 0 ? max(0, kv_len - window) : 0;   // first key the new token sees
  if (c_end <= kv_begin) {
    // a chunk in front of the window: an empty partial, so that the join needs no special case
    for (int g = warp; g < G; g += kDecodeWarps) {
      const size_t pidx = ((size_t)b * Hq + kvh * G + g) * max_chunks + c;
      if (lane == 0) {
        part_ml[pidx * 2] = -INFINITY;
        part_ml[pidx * 2 + 1] = 0.f;
      }
      for (int d = lane; d < D; d += 32) part_acc[pidx * D + d] = 0.f;
    }
    return;
  }
  constexpr int KPAD = (sizeof(T) == 2) ? 2 : 1;
  const int ks = D + KPAD;

  T* k_s = reinterpret_cast<T*>(smem_raw);
  T* v_s = k_s + kDecodeRound * ks;
  size_t off = (size_t)(kDecodeRound * ks + kDecodeRound * D) * sizeof(T);
  off = (off + 15) & ~(size_t)15;
  float* q_s = reinterpret_cast<float*>(smem_raw + off);
  float* st_m = q_s + G * D;
  float* st_l = st_m + kDecodeWarps * G;
  float* st_acc = st_l + kDecodeWarps * G;

  const T* qrow = qkv + (size_t)q_start[b] * (Hq + 2 * Hkv) * D + (size_t)kvh * G * D;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) q_s[idx] = to_f32(qrow[idx]);
  for (int idx = threadIdx.x; idx < kDecodeWarps * G; idx += blockDim.x) {
    st_m[idx] = -INFINITY;
    st_l[idx] = 0.f;
  }
  for (int idx = threadIdx.x; idx < kDecodeWarps * G * D; idx += blockDim.x) st_acc[idx] = 0.f;

  const int first_round = kv_begin > c0 ? c0 + ((kv_begin - c0) / kDecodeRound) * kDecodeRound : c0;
  for (int r0 = first_round; r0 < c_end; r0 += kDecodeRound) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < kDecodeRound * D; idx += blockDim.x) {
      const int j = idx / D, d = idx % D;
      const int key = r0 + j;
      T kval = from_f32<T>(0.f), vval = from_f32<T>(0.f);
      if (key < c_end && key >= kv_begin) {
        kval = key_row(k_pool, block_table, slot, max_pages, page_tokens, Hkv, kvh, D, key, status)[d];
        vval = key_row(v_pool, block_table, slot, max_pages, page_tokens, Hkv, kvh, D, key, status)[d];
      }
      k_s[j * ks + d] = kval;
      v_s[j * D + d] = vval;
    }
    __syncthreads();
    const int w0 = r0 + warp * kTile;
    if (w0 < c_end && w0 + kTile > kv_begin) {
      const bool valid = (w0 + lane) < c_end && (w0 + lane) >= kv_begin;
      const T* kr = k_s + (warp * kTile + lane) * ks;
      for (int g = 0; g < G; ++g) {
        const float* q = q_s + g * D;
        float s = 0.f;
        for (int d = 0; d < D; ++d) s = fmaf(q[d], to_f32(kr[d]), s);
        s = valid ? s * scale : -INFINITY;
        const float m_old = st_m[warp * G + g];
        const float m_new = fmaxf(m_old, warp_max(s));
        const float alpha = expf(m_old - m_new);
        const float p = valid ? expf(s - m_new) : 0.f;
        const float lsum = warp_sum(p);
        float* accp = st_acc + (size_t)(warp * G + g) * D;
        for (int d0 = 0; d0 < D; d0 += 32) {  // uniform trip count: every lane shuffles
          const int d = d0 + lane;
          const bool in = d < D;
          float a = in ? accp[d] * alpha : 0.f;
          for (int j = 0; j < kTile; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (in) a = fmaf(pj, to_f32(v_s[(warp * kTile + j) * D + d]), a);
          }
          if (in) accp[d] = a;
        }
        __syncwarp();
        if (lane == 0) {
          st_m[warp * G + g] = m_new;
          st_l[warp * G + g] = st_l[warp * G + g] * alpha + lsum;
        }
        __syncwarp();
      }
    }
  }
  __syncthreads();

  // Join the warps' states in warp order and write the chunk's partial.
  for (int g = warp; g < G; g += kDecodeWarps) {
    float mx = -INFINITY;
    for (int w = 0; w < kDecodeWarps; ++w) mx = fmaxf(mx, st_m[w * G + g]);
    float lsum = 0.f;
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float mw = st_m[w * G + g];
      lsum += (mw == -INFINITY) ? 0.f : st_l[w * G + g] * expf(mw - mx);
    }
    const size_t pidx = ((size_t)b * Hq + kvh * G + g) * max_chunks + c;
    if (lane == 0) {
      part_ml[pidx * 2] = mx;
      part_ml[pidx * 2 + 1] = lsum;
    }
    for (int d = lane; d < D; d += 32) {
      float a = 0.f;
      for (int w = 0; w < kDecodeWarps; ++w) {
        const float mw = st_m[w * G + g];
        if (mw != -INFINITY) a += st_acc[(size_t)(w * G + g) * D + d] * expf(mw - mx);
      }
      part_acc[pidx * D + d] = a;
    }
  }
}

// ------------------------------------------------------------------ decode, combine
// grid (Hq, B), 128 threads.
template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_ml, const float* __restrict__ part_acc,
                                           const int* __restrict__ q_start, const int* __restrict__ base_len,
                                           T* __restrict__ out, int Hq, int D, int max_chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int hq = blockIdx.x, b = blockIdx.y;
  const int kv_len = base_len[b] + 1;
  const int n_chunks = min((kv_len + kDecodeChunk - 1) / kDecodeChunk, max_chunks);   // the partial kernel reports a longer sequence
  const size_t p0 = ((size_t)b * Hq + hq) * max_chunks;
  float mx = -INFINITY;
  for (int c = 0; c < n_chunks; ++c) mx = fmaxf(mx, part_ml[(p0 + c) * 2]);
  float lsum = 0.f;
  for (int c = 0; c < n_chunks; ++c) lsum += part_ml[(p0 + c) * 2 + 1] * expf(part_ml[(p0 + c) * 2] - mx);
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  T* o = out + (size_t)q_start[b] * Hq * D + (size_t)hq * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int c = 0; c < n_chunks; ++c) a += part_acc[(p0 + c) * D + d] * expf(part_ml[(p0 + c) * 2] - mx);
    o[d] = from_f32<T>(a * inv);
  }
}

template <typename T>
static size_t decode_smem_bytes(int G, int D) {
  const int kpad = sizeof(T) == 2 ? 2 : 1;
  size_t off = (size_t)(kDecodeRound * (D + kpad) + kDecodeRound * D) * sizeof(T);
  off = (off + 15) & ~(size_t)15;
  return off + sizeof(float) * ((size_t)G * D + 2 * kDecodeWarps * G + (size_t)kDecodeWarps * G * D);
}

template <typename T, int NDIM>
static int launch_prefill(const void* qkv, const void* k_pool, const void* v_pool, const int* block_table,
                          const int* slot_ids, const int* q_start, const int* base_len, void* out, int B, int Hq,
                          int Hkv, int D, int page_tokens, int max_pages, int max_q_len, float scale, int window,
                          cudaStream_t s, int* status) {
  const int G = Hq / Hkv;
  const size_t smem = sizeof(float) * ((size_t)kPrefillRows * D + kTile * (D + 1) + kTile * D);
  auto kern = attn_prefill_kernel<T, NDIM>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((max_q_len * G + kPrefillRows - 1) / kPrefillRows, Hkv, B);
  launch_kernel(kern, grid, kPrefillWarps * 32, smem, s, (const T*)qkv, (const T*)k_pool, (const T*)v_pool, block_table,
                                              slot_ids, q_start, base_len, (T*)out, Hq, Hkv, D, page_tokens,
                                              max_pages, scale, window, status);
  return (int)cudaGetLastError();
}

}  // namespace siar

using namespace siar;

SIAR_DEFINE_PDL_SWITCH()

extern "C" int siar_attn_decode_chunk() { return kDecodeChunk; }

// Largest head_dim the kernels take; head_dim must be a multiple of 16.
extern "C" int siar_attn_max_head_dim() { return 256; }

extern "C" int siar_attn_prefill(int is_bf16, const void* qkv, const void* k_pool, const void* v_pool,
                                 const int* block_table, const int* slot_ids, const int* q_start,
                                 const int* base_len, void* out, int B, int Hq, int Hkv, int D, int page_tokens,
                                 int max_pages, int max_q_len, int window, float scale, void* stream, int* status) {
  if (B == 0 || max_q_len == 0) return 0;
  if (D % 16 != 0 || D > 256 || D <= 0 || Hq % Hkv != 0 || Hkv > 65535 || B > 65535 || window < 0)
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
#define SIAR_PREFILL(T, ND)                                                                                   \
  return launch_prefill<T, ND>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, B, Hq, Hkv, \
                               D, page_tokens, max_pages, max_q_len, scale, window, s, status)
  const int nd = (D + 31) / 32;
  if (is_bf16) {
    if (nd <= 1) SIAR_PREFILL(__nv_bfloat16, 1);
    if (nd <= 2) SIAR_PREFILL(__nv_bfloat16, 2);
    if (nd <= 4) SIAR_PREFILL(__nv_bfloat16, 4);
    SIAR_PREFILL(__nv_bfloat16, 8);
  } else {
    if (nd <= 1) SIAR_PREFILL(float, 1);
    if (nd <= 2) SIAR_PREFILL(float, 2);
    if (nd <= 4) SIAR_PREFILL(float, 4);
    SIAR_PREFILL(float, 8);
  }
#undef SIAR_PREFILL
}

// Bytes of scratch memory siar_attn_decode needs for these sizes.
extern "C" long long siar_attn_decode_scratch_bytes(int B, int Hq, int D, int max_kv_len) {
  const long long chunks = (max_kv_len + kDecodeChunk - 1) / kDecodeChunk;
  return (long long)B * Hq * chunks * (D + 2) * (long long)sizeof(float);
}

template <typename T>
static int launch_decode(const void* qkv, const void* k_pool, const void* v_pool, const int* block_table,
                         const int* slot_ids, const int* q_start, const int* base_len, void* out, float* scratch,
                         int B, int Hq, int Hkv, int D, int page_tokens, int max_pages, int max_kv_len,
                         float scale, int window, cudaStream_t s, int* status) {
  const int G = Hq / Hkv;
  const int max_chunks = (max_kv_len + kDecodeChunk - 1) / kDecodeChunk;
  float* part_ml = scratch;
  float* part_acc = scratch + (size_t)B * Hq * max_chunks * 2;
  const size_t smem = decode_smem_bytes<T>(G, D);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  auto kern = attn_decode_partial_kernel<T>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(max_chunks, Hkv, B);
  launch_kernel(kern, grid, kDecodeWarps * 32, smem, s, (const T*)qkv, (const T*)k_pool, (const T*)v_pool, block_table,
                                             slot_ids, q_start, base_len, part_ml, part_acc, Hq, Hkv, D,
                                             page_tokens, max_pages, max_chunks, scale, window, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  dim3 grid2(Hq, B);
  launch_kernel(attn_decode_combine_kernel<T>, grid2, 128, 0, s, part_ml, part_acc, q_start, base_len, (T*)out, Hq, D,
                                                      max_chunks);
  return (int)cudaGetLastError();
}

// One new token per sequence.  max_kv_len bounds base_len[b] + 1 over the batch
// and fixes the grid and the scratch layout (so a captured launch stays valid
// while lengths grow up to it).
extern "C" int siar_attn_decode(int is_bf16, const void* qkv, const void* k_pool, const void* v_pool,
                                const int* block_table, const int* slot_ids, const int* q_start,
                                const int* base_len, void* out, float* scratch, int B, int Hq, int Hkv, int D,
                                int page_tokens, int max_pages, int max_kv_len, int window, float scale,
                                void* stream, int* status) {
  if (B == 0) return 0;
  if (D % 16 != 0 || D > 256 || D <= 0 || Hq % Hkv != 0 || Hkv > 65535 || B > 65535 || max_kv_len <= 0 || window < 0)
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (is_bf16)
    return launch_decode<__nv_bfloat16>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out,
                                        scratch, B, Hq, Hkv, D, page_tokens, max_pages, max_kv_len, scale, window, s, status);
  return launch_decode<float>(qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, scratch, B, Hq,
                              Hkv, D, page_tokens, max_pages, max_kv_len, scale, window, s, status);
}
