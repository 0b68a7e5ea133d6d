// Next-token choice from one row of 32-bit logits per sequence: greedy, or
// temperature -> top-k -> top-p -> one categorical draw, the order and meaning of
// the reference's sample() (sampling.py:151-236):
//   temperature == 0        argmax, the other options ignored   (sampling.py:170-171)
//   top_k <= 0 or >= V      no top-k                            (sampling.py:87-88,174)
//   top-k                   exactly k candidates                (sampling.py:203)
//   top_p >= 1              no nucleus                          (sampling.py:119-120)
//   nucleus                 in descending order keep a token iff the mass before
//                           it is <= top_p; the top token always stays
//                           (sampling.py:216-221, kernels/sampling_kernel.py:77-79)
//   draw                    inverse CDF over the kept tokens on a uniform u
//                           (kernels/sampling_kernel.py:89-92)
// The reference sorts the vocabulary (torch.topk / torch.sort).  Here nothing is
// sorted: thresholds on the order-preserving integer image of the logits are
// found by bisection with exact counts and fixed-order sums, so the kept set is
// the same one, ties at the k-th value go to the lower token ids, tokens of equal
// logit enter or leave the nucleus together, and the draw walks the kept tokens in
// token-id order.  The uniform comes from a counter-based generator keyed by a
// per-request seed and the index of the token being drawn, so a request draws the
// same tokens alone or in any batch (the reference uses the global torch
// generator, sampling.py:224,236).
//
// One block of 1024 threads per row.  All sums are formed in a fixed order.
#include "common.cuh"

#include <math.h>

namespace siar {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned int order_key(float x) {
  unsigned int b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float uniform_from_counter(unsigned long long seed, unsigned long long index) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (index + 1ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

struct Shared {
  float f[32];
  int i[32];
  unsigned int u[32];
  int found;
  float carry;
};

__device__ __forceinline__ int block_sum_int(int v, Shared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sh.i[warp] = v;
  __syncthreads();
  int total = 0;
  for (int w = 0; w < kSampleThreads / 32; ++w) total += sh.i[w];
  return total;
}

__device__ __forceinline__ float block_sum_float(float v, Shared& sh) { return block_sum(v, sh.f); }

// Inclusive scan over the block in thread order; returns this thread's prefix and
// the block total through `total`.
__device__ __forceinline__ float block_scan_float(float v, Shared& sh, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  __syncthreads();
  if (lane == 31) sh.f[warp] = v;
  __syncthreads();
  float before = 0.f, all = 0.f;
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    if (w == warp) before = all;
    all += sh.f[w];
  }
  *total = all;
  return before + v;
}

__device__ __forceinline__ int block_scan_int(int v, Shared& sh, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  __syncthreads();
  if (lane == 31) sh.i[warp] = v;
  __syncthreads();
  int before = 0, all = 0;
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    if (w == warp) before = all;
    all += sh.i[w];
  }
  *total = all;
  return before + v;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const long long* __restrict__ seeds, int* __restrict__ draw_index, int advance_index,
              int* __restrict__ out) {
  pdl_launch_dependents();
  SIAR_TRACE(30, 0);
  pdl_wait();
  SIAR_TRACE(30, 2);
  __shared__ Shared sh;
  const int r = blockIdx.x;
  const float* x = logits + (size_t)r * V;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;

  // ---- 1. maximum and its lowest index
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float v = x[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { sh.f[warp] = best; sh.i[warp] = best_i; }
  __syncthreads();
  best = sh.f[0];
  best_i = sh.i[0];
  for (int w = 1; w < kSampleThreads / 32; ++w) {
    const float ov = sh.f[w];
    const int oi = sh.i[w];
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  __syncthreads();
  if (best_i == 0x7fffffff) best_i = 0;  // a row of NaN or -inf only

  const float temp = temperature[r];
  if (!(temp > 0.f)) {
    if (tid == 0) out[r] = best_i;
    return;
  }
  const float inv_temp = 1.f / temp;
  const unsigned int key_max = order_key(best);

  // ---- 2. top-k: threshold key T and the index E up to which ties at T are kept
  int k = top_k[r];
  unsigned int T = 0u;
  int E = V;
  if (k > 0 && k < V) {
    unsigned int lo = 0u, hi = key_max;
    while (lo < hi) {
      const unsigned int mid = lo + ((hi - lo) >> 1) + ((hi - lo) & 1u);
      int c = 0;
      for (int i = tid; i < V; i += kSampleThreads) c += order_key(x[i]) >= mid;
      if (block_sum_int(c, sh) >= k) lo = mid; else hi = mid - 1u;
    }
    T = lo;
    int c = 0;
    for (int i = tid; i < V; i += kSampleThreads) c += order_key(x[i]) > T;
    const int need_eq = k - block_sum_int(c, sh);
    // index of the need_eq-th token whose key equals T
    int running = 0;
    if (tid == 0) sh.found = V;
    __syncthreads();
    for (int i0 = 0; i0 < V; i0 += kSampleThreads) {
      const int i = i0 + tid;
      const int eq = (i < V) && (order_key(x[i]) == T);
      int total;
      const int incl = block_scan_int(eq, sh, &total);
      if (eq && running + incl == need_eq) sh.found = i;
      running += total;
      __syncthreads();
      if (running >= need_eq) break;
    }
    E = sh.found;
    __syncthreads();
  }
#define KEPT_K(key, i) ((key) > T || ((key) == T && (i) <= E))

  // ---- 3. mass of the top-k set
  float z = 0.f;
  for (int i = tid; i < V; i += kSampleThreads) {
    const unsigned int key = order_key(x[i]);
    if (KEPT_K(key, i)) z += expf((x[i] - best) * inv_temp);
  }
  const float Z = block_sum_float(z, sh);

  // ---- 4. nucleus: smallest key T2 with mass(key > T2) <= top_p * Z
  unsigned int T2 = 0u;
  const float p = top_p[r];
  if (p < 1.f) {
    const float limit = p * Z;
    unsigned int lo = 0u, hi = key_max;
    while (lo < hi) {
      const unsigned int mid = lo + ((hi - lo) >> 1);
      float mgt = 0.f;
      for (int i = tid; i < V; i += kSampleThreads) {
        const unsigned int key = order_key(x[i]);
        if (key > mid && KEPT_K(key, i)) mgt += expf((x[i] - best) * inv_temp);
      }
      if (block_sum_float(mgt, sh) <= limit) hi = mid; else lo = mid + 1u;
    }
    T2 = lo;
  }
#define KEPT(key, i) (KEPT_K(key, i) && (key) >= T2)

  // ---- 5. mass of the final set and the draw
  float z2 = 0.f;
  for (int i = tid; i < V; i += kSampleThreads) {
    const unsigned int key = order_key(x[i]);
    if (KEPT(key, i)) z2 += expf((x[i] - best) * inv_temp);
  }
  const float Z2 = block_sum_float(z2, sh);
  const int index = draw_index[r];
  const float u = uniform_from_counter((unsigned long long)seeds[r], (unsigned long long)(unsigned int)index);
  const float target = u * Z2;

  if (tid == 0) { sh.found = 0x7fffffff; sh.carry = 0.f; }
  __syncthreads();
  float carry = 0.f;
  int last_kept = -1;
  for (int i0 = 0; i0 < V; i0 += kSampleThreads) {
    const int i = i0 + tid;
    float w = 0.f;
    bool kept = false;
    if (i < V) {
      const unsigned int key = order_key(x[i]);
      kept = KEPT(key, i);
      if (kept) { w = expf((x[i] - best) * inv_temp); last_kept = i; }
    }
    float total;
    const float incl = carry + block_scan_float(w, sh, &total);
    if (kept && incl >= target) atomicMin(&sh.found, i);
    carry += total;
    __syncthreads();
    if (sh.found != 0x7fffffff) break;
    __syncthreads();
  }
  int chosen = sh.found;
  if (chosen == 0x7fffffff) {  // rounding left the walk short of the target: last kept token
    __syncthreads();
    if (tid == 0) sh.found = -1;
    __syncthreads();
    if (last_kept >= 0) atomicMax(&sh.found, last_kept);
    __syncthreads();
    chosen = sh.found >= 0 ? sh.found : best_i;
  }
  if (tid == 0) {
    out[r] = chosen;
    if (advance_index) draw_index[r] = index + 1;
  }
#undef KEPT
#undef KEPT_K
}

}  // namespace siar

using namespace siar;

SIAR_DEFINE_PDL_SWITCH()

extern "C" int siar_sample(const float* logits, int R, int V, const float* temperature, const int* top_k,
                           const float* top_p, const long long* seeds, int* draw_index, int advance_index,
                           int* out, void* stream) {
  if (R == 0) return 0;
  launch_kernel(sample_kernel, R, kSampleThreads, 0, (cudaStream_t)stream, logits, V, temperature, top_k, top_p, seeds,
                                                               draw_index, advance_index, out);
  return (int)cudaGetLastError();
}
