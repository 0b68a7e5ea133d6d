// Memory-bound kernels of the decoder: embedding gather, fused residual-add +
// RMSNorm, rotary position encoding fused with the cache write, SwiGLU, row
// gather, and the per-step length bookkeeping.  All arithmetic is 32-bit; only
// loads and stores touch the storage dtype.
//
// Formulas (reference files are cited by their path inside the reference project):
//  * embedding           x[t] = W[ids[t]]                        ops/embedding.py:62-65
//  * add + RMSNorm       r = r + delta (fp32); y = r * rsqrt(mean(r^2) + eps) * w
//                                                                kernels/add_rmsnorm_kernel.py:86-103
//  * rotary (split-half) out_i = x_i cos - x_{i+D/2} sin; out_{i+D/2} = x_{i+D/2} cos + x_i sin
//                                                                kernels/rope_kernel.py:143-152
//    with angle = position * inv_freq[i] formed in fp32           ops/rope.py:108-118
//  * cache write         K[slot, pos] = rotated k, V[slot, pos] = v   model/kv_cache.py:178-179
//  * SwiGLU              f = gate * sigmoid(gate) * up             kernels/swiglu_kernel.py:139-140
#include "common.cuh"

namespace siar {

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                    float* __restrict__ out, int H, int V, int* __restrict__ status) {
  pdl_launch_dependents();
  SIAR_TRACE(1, 0);
  pdl_wait();
  SIAR_TRACE(1, 2);
  const int t = blockIdx.x;
  int id = tokens[t];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicOr(status, kStatusTokenOutOfRange);
    for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)t * H + j] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)t * H + j] = to_f32(row[j]);
}

// The same for a bfloat16 table whose rows are whole 16-byte pieces: eight values per thread and
// load, every load of a thread asked for before the first is used.
__global__ void embed_gather_bf16x8_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                                           float* __restrict__ out, int H, int V, int* __restrict__ status) {
  pdl_launch_dependents();
  SIAR_TRACE(1, 0);
  pdl_wait();
  SIAR_TRACE(1, 2);
  const int t = blockIdx.x;
  const int id = tokens[t];
  const bool bad = id < 0 || id >= V;
  if (bad && threadIdx.x == 0) atomicOr(status, kStatusTokenOutOfRange);
  const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)(bad ? 0 : id) * H);
  float4* dst = reinterpret_cast<float4*>(out + (size_t)t * H);
  const int pieces = H / 8;
  for (int j0 = threadIdx.x; j0 < pieces; j0 += 4 * blockDim.x) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * blockDim.x;
      v[u] = (j < pieces && !bad) ? __ldg(row + j) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * blockDim.x;
      if (j >= pieces) break;
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v[u].x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v[u].y));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v[u].z));
      const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v[u].w));
      dst[2 * j] = make_float4(a.x, a.y, b.x, b.y);
      dst[2 * j + 1] = make_float4(c.x, c.y, d.x, d.y);
    }
  }
}

// ------------------------------------------------------------------ row gather
__global__ void gather_rows_kernel(const float* __restrict__ src, const int* __restrict__ rows,
                                   float* __restrict__ dst, int H) {
  pdl_launch_dependents();
  SIAR_TRACE(5, 0);
  pdl_wait();
  SIAR_TRACE(5, 2);
  const int r = blockIdx.x;
  const float* s = src + (size_t)rows[r] * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) dst[(size_t)r * H + j] = s[j];
}

// ------------------------------------------------------------------ add + RMSNorm
// One block per row.  Pass 1 forms r = residual + delta in fp32, stores it and
// accumulates the sum of squares; pass 2 re-reads the stored row (same thread,
// same addresses) and writes the normed output.
template <typename TOut, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                   const TW* __restrict__ weight, TOut* __restrict__ out, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  if (delta != nullptr) {
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      float r = residual[base + j] + delta[base + j];
      residual[base + j] = r;
      ss += r * r;
    }
  } else {
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      float r = residual[base + j];
      ss += r * r;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float r = residual[base + j];
    out[base + j] = from_f32<TOut>(r * inv * to_f32(weight[j]));
  }
}

// Vector form for H % 4 == 0 and H <= 4 * 4 * blockDim: the row stays in registers
// (one read of residual and delta, one write of each output).  The sum of squares is
// formed per thread over its own elements in index order, then by block_sum.
template <typename TW> __device__ __forceinline__ float4 load_w4(const TW* w, int c);
template <> __device__ __forceinline__ float4 load_w4<float>(const float* w, int c) {
  return reinterpret_cast<const float4*>(w)[c];
}
template <> __device__ __forceinline__ float4 load_w4<__nv_bfloat16>(const __nv_bfloat16* w, int c) {
  const uint2 u = reinterpret_cast<const uint2*>(w)[c];
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* o, int c, float4 v) { reinterpret_cast<float4*>(o)[c] = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* o, int c, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  reinterpret_cast<uint2*>(o)[c] = u;
}

template <typename TOut, typename TW>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                       const TW* __restrict__ weight, TOut* __restrict__ out, int H, float eps) {
  pdl_launch_dependents();
  SIAR_TRACE(2, 0);
  __shared__ float scratch[32];
  constexpr int VPT = 4;
  const int chunks = H >> 2;
  const size_t base = (size_t)blockIdx.x * chunks;
  float4 w[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {           // weights are written by no kernel: load them before the wait
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) w[i] = load_w4<TW>(weight, c);
  }
  pdl_wait();
  SIAR_TRACE(2, 2);
  float4 r[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      float4 v = reinterpret_cast<const float4*>(residual)[base + c];
      if (delta != nullptr) {
        const float4 d = reinterpret_cast<const float4*>(delta)[base + c];
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        reinterpret_cast<float4*>(residual)[base + c] = v;
      }
      r[i] = v;
      ss += v.x * v.x;
      ss += v.y * v.y;
      ss += v.z * v.z;
      ss += v.w * v.w;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)H + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks)
      store4(out + (size_t)blockIdx.x * H, c,
             make_float4(r[i].x * inv * w[i].x, r[i].y * inv * w[i].y, r[i].z * inv * w[i].z, r[i].w * inv * w[i].w));
  }
  SIAR_TRACE(2, 1);
}

// ------------------------------------------------------------------ rotary + cache write
// One block per token.  The token's sin/cos (one pair per rotary frequency, shared by all
// heads) are formed once in shared memory; then q heads are rotated in place, k heads are
// rotated into the cache and v heads are copied into the cache.  inv_freq == nullptr means
// "no rotation".  This kernel takes every rotary layout: the first `rotary_dim` dims of a head are
// rotated (the rest pass through), in pairs (i, i + rotary_dim/2) or, `interleaved`, (2i, 2i+1);
// inv_freq holds rotary_dim/2 frequencies.  (The reference's kernel has the same two pairings,
// kernels/rope_kernel.py:139-152, and always rotates the whole head.)
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ inv_freq,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const int* __restrict__ block_table, const int* __restrict__ slot_ids,
                                     const int* __restrict__ q_start, const int* __restrict__ base_len,
                                     int B, int Hq, int Hkv, int D, int page_tokens, int max_pages,
                                     int n_pages, int write_kv, int* __restrict__ status, int rotary_dim,
                                     int interleaved) {
  pdl_launch_dependents();
  SIAR_TRACE(3, 0);
  extern __shared__ float cs[];   // cos[half], sin[half]
  const int half = rotary_dim >> 1;
  const int flat = threadIdx.y * blockDim.x + threadIdx.x, nthreads = blockDim.x * blockDim.y;
  for (int i = flat; i < half; i += nthreads) cs[i] = inv_freq != nullptr ? inv_freq[i] : 0.f;
  pdl_wait();
  SIAR_TRACE(3, 2);
  const int t = blockIdx.x;
  const int b = find_sequence(q_start, B, t);
  const int pos = base_len[b] + (t - q_start[b]);
  for (int i = flat; i < half; i += nthreads) {
    float sn = 0.f, c = 1.f;
    if (inv_freq != nullptr) sincosf((float)pos * cs[i], &sn, &c);
    cs[i] = c;
    cs[half + i] = sn;
  }
  T* row = qkv + (size_t)t * (Hq + 2 * Hkv) * D;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (write_kv) {
    const int slot = slot_ids[b];
    const int page = block_table[(size_t)slot * max_pages + pos / page_tokens];
    if (page < 0 || page >= n_pages) {
      if (flat == 0) atomicOr(status, kStatusBadPage);
    } else {
      const size_t off = ((size_t)page * Hkv * page_tokens + (pos % page_tokens)) * D;   // kv head 0
      kdst = k_pool + off;
      vdst = v_pool + off;
    }
  }
  __syncthreads();
  const size_t head_stride = (size_t)page_tokens * D;   // between kv heads inside a page
  const int n_rot = Hq + (kdst != nullptr ? Hkv : 0);
  // Heads are dealt to the blocks of a token (gridDim.y of them: more than one when few tokens
  // run) and, inside a block, to its threadIdx.y rows; threadIdx.x walks the pairs of a head.
  const int hstep = gridDim.y * blockDim.y;
  for (int head = blockIdx.y * blockDim.y + threadIdx.y; head < n_rot; head += hstep) {
    T* dst = head < Hq ? row + head * D : kdst + (size_t)(head - Hq) * head_stride;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
      const float a = to_f32(row[head * D + i0]), c = to_f32(row[head * D + i1]);
      const float cosv = cs[i], sinv = cs[half + i];
      dst[i0] = from_f32<T>(a * cosv - c * sinv);
      dst[i1] = from_f32<T>(c * cosv + a * sinv);
    }
    if (head >= Hq)      // the dims of a key past the rotary part go to the cache as they are
      for (int i = rotary_dim + threadIdx.x; i < D; i += blockDim.x) dst[i] = row[head * D + i];
  }
  if (vdst != nullptr) {
    const T* vrow = row + (size_t)(Hq + Hkv) * D;
    for (int head = blockIdx.y * blockDim.y + threadIdx.y; head < Hkv; head += hstep)
      for (int i = threadIdx.x; i < D; i += blockDim.x) vdst[(size_t)head * head_stride + i] = vrow[head * D + i];
  }
}

// The same for many bfloat16 tokens, 16 bytes at a time: one block of 128 threads per token,
// thread (head slot, piece) rotates 8 pairs of one head per pass; all loads of up to kRopePasses
// passes are asked for before the first value is used.  D % 16 == 0.
constexpr int kRopePasses = 4;

__global__ void __launch_bounds__(128)
rope_kv_write_bf16x8_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ inv_freq,
                            __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                            const int* __restrict__ block_table, const int* __restrict__ slot_ids,
                            const int* __restrict__ q_start, const int* __restrict__ base_len, int B, int Hq,
                            int Hkv, int D, int page_tokens, int max_pages, int n_pages, int write_kv,
                            int* __restrict__ status) {
  pdl_launch_dependents();
  SIAR_TRACE(3, 0);
  extern __shared__ float cs[];   // cos[half], sin[half]
  const int half = D >> 1;
  const int tid = threadIdx.x;
  float freq = 0.f;
  if (tid < half && inv_freq != nullptr) freq = inv_freq[tid];     // half <= 128
  pdl_wait();
  SIAR_TRACE(3, 2);
  const int t = blockIdx.x;
  const int b = find_sequence(q_start, B, t);
  const int pos = base_len[b] + (t - q_start[b]);
  __nv_bfloat16* row = qkv + (size_t)t * (Hq + 2 * Hkv) * D;
  // thread -> (head slot, piece of 8 pairs)
  const int pieces = half >> 3;
  const int slots = 128 / pieces;
  const int hs = tid / pieces, pc = tid % pieces;
  const bool active = hs < slots;
  const int n_heads_rot = Hq + Hkv;
  uint4 lo[kRopePasses], hi[kRopePasses];
#pragma unroll
  for (int p = 0; p < kRopePasses; ++p) {
    const int head = p * slots + hs;
    if (active && head < n_heads_rot) {
      lo[p] = *reinterpret_cast<const uint4*>(row + (size_t)head * D + pc * 8);
      hi[p] = *reinterpret_cast<const uint4*>(row + (size_t)head * D + half + pc * 8);
    }
  }
  if (tid < half) {
    float sn = 0.f, c = 1.f;
    if (inv_freq != nullptr) sincosf((float)pos * freq, &sn, &c);
    cs[tid] = c;
    cs[half + tid] = sn;
  }
  __nv_bfloat16* kdst = nullptr;
  __nv_bfloat16* vdst = nullptr;
  if (write_kv) {
    const int slot = slot_ids[b];
    const int page = block_table[(size_t)slot * max_pages + pos / page_tokens];
    if (page < 0 || page >= n_pages) {
      if (tid == 0) atomicOr(status, kStatusBadPage);
    } else {
      const size_t off = ((size_t)page * Hkv * page_tokens + (pos % page_tokens)) * D;   // kv head 0
      kdst = k_pool + off;
      vdst = v_pool + off;
    }
  }
  __syncthreads();
  const size_t head_stride = (size_t)page_tokens * D;   // between kv heads inside a page
  const int n_rot = Hq + (kdst != nullptr ? Hkv : 0);
  float cv[8], sv[8];
  if (active) {
#pragma unroll
    for (int e = 0; e < 8; ++e) { cv[e] = cs[pc * 8 + e]; sv[e] = cs[half + pc * 8 + e]; }
  }
  auto rotate_store = [&](int head, const uint4& a4, const uint4& c4) {
    __nv_bfloat16* dst = head < Hq ? row + (size_t)head * D : kdst + (size_t)(head - Hq) * head_stride;
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a4);
    const __nv_bfloat162* cp = reinterpret_cast<const __nv_bfloat162*>(&c4);
    uint4 o_lo, o_hi;
    uint32_t* ol = reinterpret_cast<uint32_t*>(&o_lo);
    uint32_t* oh = reinterpret_cast<uint32_t*>(&o_hi);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(ap[e]), c = __bfloat1622float2(cp[e]);
      __nv_bfloat162 l2 = __floats2bfloat162_rn(a.x * cv[2 * e] - c.x * sv[2 * e], a.y * cv[2 * e + 1] - c.y * sv[2 * e + 1]);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(c.x * cv[2 * e] + a.x * sv[2 * e], c.y * cv[2 * e + 1] + a.y * sv[2 * e + 1]);
      ol[e] = *reinterpret_cast<uint32_t*>(&l2);
      oh[e] = *reinterpret_cast<uint32_t*>(&h2);
    }
    *reinterpret_cast<uint4*>(dst + pc * 8) = o_lo;
    *reinterpret_cast<uint4*>(dst + half + pc * 8) = o_hi;
  };
  if (active) {
#pragma unroll
    for (int p = 0; p < kRopePasses; ++p) {
      const int head = p * slots + hs;
      if (head < n_rot) rotate_store(head, lo[p], hi[p]);
    }
    // more heads than kRopePasses passes cover: the rest one pass at a time
    for (int head = kRopePasses * slots + hs; head < n_rot; head += slots) {
      const uint4 a4 = *reinterpret_cast<const uint4*>(row + (size_t)head * D + pc * 8);
      const uint4 c4 = *reinterpret_cast<const uint4*>(row + (size_t)head * D + half + pc * 8);
      rotate_store(head, a4, c4);
    }
  }
  if (vdst != nullptr) {
    const __nv_bfloat16* vrow = row + (size_t)(Hq + Hkv) * D;
    const int per_head = D >> 3;
    for (int idx = tid; idx < Hkv * per_head; idx += 128) {
      const int head = idx / per_head, c = idx % per_head;
      *reinterpret_cast<uint4*>(vdst + (size_t)head * head_stride + c * 8) =
          *reinterpret_cast<const uint4*>(vrow + (size_t)head * D + c * 8);
    }
  }
}

// ------------------------------------------------------------------ SwiGLU
// interleaved == 0: rows are [gate (I) | up (I)]; interleaved == 1: rows are (gate_0, up_0, gate_1, ...).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int interleaved) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  if (j >= I) return;
  const float g = to_f32(gu[row * 2 * I + (interleaved ? 2 * j : j)]);
  const float u = to_f32(gu[row * 2 * I + (interleaved ? 2 * j + 1 : I + j)]);
  const float s = g / (1.f + expf(-g));
  out[row * I + j] = from_f32<T>(s * u);
}

// bf16, I % 8 == 0, 16-byte aligned rows: eight outputs per thread with 16-byte accesses.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I) {
  pdl_launch_dependents();
  SIAR_TRACE(4, 0);
  pdl_wait();
  SIAR_TRACE(4, 2);
  const size_t row = blockIdx.x;
  const int j = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (j >= I) return;
  const uint4 gv = *reinterpret_cast<const uint4*>(gu + row * 2 * I + j);
  const uint4 uv = *reinterpret_cast<const uint4*>(gu + row * 2 * I + I + j);
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
  uint4 ov;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 g = __bfloat1622float2(gp[e]), u = __bfloat1622float2(up[e]);
    op[e] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
  }
  *reinterpret_cast<uint4*>(out + row * I + j) = ov;
}

// ------------------------------------------------------------------ bookkeeping
// base_len[b] += q_start[b+1] - q_start[b]; used by the captured decode step so
// that a replay sees the lengths the previous replay left.
__global__ void advance_lengths_kernel(int* __restrict__ base_len, const int* __restrict__ q_start, int B) {
  pdl_launch_dependents();
  SIAR_TRACE(6, 0);
  pdl_wait();
  SIAR_TRACE(6, 2);
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) base_len[b] += q_start[b + 1] - q_start[b];
}

// table[row][col] = value for n (row, col, value) triples: the pages a step gave to or took from
// sequences, written into the block table of a group of layers.
__global__ void set_table_cells_kernel(int* __restrict__ table, const int* __restrict__ cells, int n, int rows,
                                       int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = cells[3 * i], c = cells[3 * i + 1];
  if (r >= 0 && r < rows && c >= 0 && c < cols) table[(size_t)r * cols + c] = cells[3 * i + 2];
}

}  // namespace siar

using namespace siar;

SIAR_DEFINE_PDL_SWITCH()

#define LAUNCH_END() return (int)cudaGetLastError()

extern "C" int siar_embed_gather(int is_bf16, const int* tokens, const void* table, float* out, int N, int H,
                                 int V, int* status, void* stream) {
  if (N == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (is_bf16 && H % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) % 16) == 0)
    launch_kernel(embed_gather_bf16x8_kernel, N, 128, 0, s, tokens, (const __nv_bfloat16*)table, out, H, V, status);
  else if (is_bf16)
    launch_kernel(embed_gather_kernel<__nv_bfloat16>, N, 256, 0, s, tokens, (const __nv_bfloat16*)table, out, H, V, status);
  else
    launch_kernel(embed_gather_kernel<float>, N, 256, 0, s, tokens, (const float*)table, out, H, V, status);
  LAUNCH_END();
}

extern "C" int siar_gather_rows(const float* src, const int* rows, float* dst, int R, int H, void* stream) {
  if (R == 0) return 0;
  launch_kernel(gather_rows_kernel, R, 256, 0, (cudaStream_t)stream, src, rows, dst, H);
  LAUNCH_END();
}

extern "C" int siar_add_rmsnorm(int out_bf16, int weight_bf16, float* residual, const float* delta,
                                const void* weight, void* out, int N, int H, float eps, void* stream) {
  if (N == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)out) % 16 == 0) &&
                       ((uintptr_t)weight % 16 == 0);
  if (H % 4 == 0 && H <= 16384 && aligned) {
    int threads = ((H / 4 + 3) / 4 + 31) / 32 * 32;
    if (threads < 64) threads = 64;
    if (out_bf16 && weight_bf16)
      launch_kernel(add_rmsnorm_vec_kernel<__nv_bfloat16, __nv_bfloat16>, N, threads, 0, s, residual, delta,
                    (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, H, eps);
    else if (out_bf16)
      launch_kernel(add_rmsnorm_vec_kernel<__nv_bfloat16, float>, N, threads, 0, s, residual, delta,
                    (const float*)weight, (__nv_bfloat16*)out, H, eps);
    else if (weight_bf16)
      launch_kernel(add_rmsnorm_vec_kernel<float, __nv_bfloat16>, N, threads, 0, s, residual, delta,
                    (const __nv_bfloat16*)weight, (float*)out, H, eps);
    else
      launch_kernel(add_rmsnorm_vec_kernel<float, float>, N, threads, 0, s, residual, delta, (const float*)weight,
                    (float*)out, H, eps);
    LAUNCH_END();
  }
  const int threads = H >= 2048 ? 512 : 256;
  if (out_bf16 && weight_bf16)
    launch_kernel(add_rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16>, N, threads, 0, s, residual, delta,
                  (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, H, eps);
  else if (out_bf16)
    launch_kernel(add_rmsnorm_kernel<__nv_bfloat16, float>, N, threads, 0, s, residual, delta, (const float*)weight,
                  (__nv_bfloat16*)out, H, eps);
  else if (weight_bf16)
    launch_kernel(add_rmsnorm_kernel<float, __nv_bfloat16>, N, threads, 0, s, residual, delta,
                  (const __nv_bfloat16*)weight, (float*)out, H, eps);
  else
    launch_kernel(add_rmsnorm_kernel<float, float>, N, threads, 0, s, residual, delta, (const float*)weight,
                  (float*)out, H, eps);
  LAUNCH_END();
}

extern "C" int siar_rope_kv_write(int is_bf16, void* qkv, const float* inv_freq, void* k_pool, void* v_pool,
                                  const int* block_table, const int* slot_ids, const int* q_start,
                                  const int* base_len, int N, int B, int Hq, int Hkv, int D, int page_tokens,
                                  int max_pages, int n_pages, int write_kv, int* status, void* stream,
                                  int rotary_dim, int interleaved) {
  if (N == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (D % 2 != 0 || rotary_dim < 0 || rotary_dim > D || rotary_dim % 2 != 0) return (int)cudaErrorInvalidValue;
  if (inv_freq == nullptr) rotary_dim = D;      // no rotation: every dim passes through the pair loop with angle 0
  const bool whole_split_half = rotary_dim == D && !interleaved;
  // many tokens: one block per token walks all heads; few tokens: several blocks share a token
  const int ysplit = N >= 256 ? 1 : (Hq + Hkv < 16 ? Hq + Hkv : 16);
  const int tx = D / 2 > 64 ? 128 : D / 2 > 32 ? 64 : 32;   // one pass over the D/2 pairs of a head
  const dim3 threads(tx, ysplit == 1 ? 256 / tx : 1);        // many tokens: several heads at a time per block
  const size_t smem = sizeof(float) * D;
  if (whole_split_half && is_bf16 && N >= 256 && D % 16 == 0 && D <= 256 && (((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) % 16) == 0) {
    launch_kernel(rope_kv_write_bf16x8_kernel, dim3(N), dim3(128), smem, s, (__nv_bfloat16*)qkv, inv_freq,
                  (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, block_table, slot_ids, q_start, base_len, B, Hq, Hkv,
                  D, page_tokens, max_pages, n_pages, write_kv, status);
    LAUNCH_END();
  }
  if (is_bf16)
    launch_kernel(rope_kv_write_kernel<__nv_bfloat16>, dim3(N, ysplit), dim3(threads), smem, s, (__nv_bfloat16*)qkv, inv_freq,
                  (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, block_table, slot_ids, q_start, base_len, B, Hq, Hkv,
                  D, page_tokens, max_pages, n_pages, write_kv, status, rotary_dim, interleaved);
  else
    launch_kernel(rope_kv_write_kernel<float>, dim3(N, ysplit), dim3(threads), smem, s, (float*)qkv, inv_freq, (float*)k_pool,
                  (float*)v_pool, block_table, slot_ids, q_start, base_len, B, Hq, Hkv, D, page_tokens, max_pages,
                  n_pages, write_kv, status, rotary_dim, interleaved);
  LAUNCH_END();
}

extern "C" int siar_swiglu(int is_bf16, const void* gu, void* out, int N, int I, int interleaved, void* stream) {
  if (N == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (!interleaved && is_bf16 && I % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) % 16) == 0) {
    dim3 grid8(N, (I / 8 + 255) / 256);
    launch_kernel(swiglu_bf16x8_kernel, grid8, dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I);
    LAUNCH_END();
  }
  dim3 grid(N, (I + 255) / 256);
  if (is_bf16)
    launch_kernel(swiglu_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, interleaved);
  else
    launch_kernel(swiglu_kernel<float>, grid, 256, 0, s, (const float*)gu, (float*)out, I, interleaved);
  LAUNCH_END();
}

extern "C" int siar_set_table_cells(int* table, const int* cells, int n, int rows, int cols, void* stream) {
  if (n == 0) return 0;
  launch_kernel(set_table_cells_kernel, (n + 127) / 128, 128, 0, (cudaStream_t)stream, table, cells, n, rows, cols);
  LAUNCH_END();
}

extern "C" int siar_advance_lengths(int* base_len, const int* q_start, int B, void* stream) {
  if (B == 0) return 0;
  launch_kernel(advance_lengths_kernel, (B + 127) / 128, 128, 0, (cudaStream_t)stream, base_len, q_start, B);
  LAUNCH_END();
}
