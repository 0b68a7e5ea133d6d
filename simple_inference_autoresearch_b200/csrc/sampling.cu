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
//
// Two ways to the thresholds.  The short one (top-k up to 512, or a nucleus that lies within
// the few hundred largest logits) collects the candidates in shared memory: the k'-th largest of
// the threads' own maxima is a pivot with at least k' logits at or above it; those are gathered
// in one pass, sorted by (logit descending, token id ascending), and top-k, nucleus and the draw
// are prefix sums over at most 2,048 entries.  Masses on this way are 64-bit fixed-point numbers
// (weight * 2^40, truncated), so that they do not depend on the order in which the gathering pass
// happened to store the candidates.  The long one (any k, any nucleus) bisects over the whole
// row as described above; a row takes it when the short one does not apply, which depends on
// the row alone.  Without top-k and nucleus, and at the end of the long way, the draw is an
// ordered walk: every thread sums a run of consecutive tokens, the runs' sums are scanned in
// thread order, and the thread whose run holds the target walks it again.
#include "common.cuh"

#include <math.h>

namespace siar {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned int order_key(float x) {
  unsigned int b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// exp((x - max) / temperature) by the hardware's base-2 exponential (about 2^-21 relative): the
// same function wherever a weight is formed, so every way through the kernel sees the same weights.
__device__ __forceinline__ float token_weight(float x, float best, float inv_temp) { return __expf((x - best) * inv_temp); }

__device__ __forceinline__ float uniform_from_counter(unsigned long long seed, unsigned long long index) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (index + 1ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// f(value, index) for every logit of the row, a thread's calls in ascending index order.  Eight
// loads are on their way before the first value is used; with `vec` (rows that are whole,
// aligned 16-byte pieces) a load brings four consecutive logits.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ x, int V, bool vec, F f) {
  constexpr int U = 8;
  if (vec) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int n4 = V >> 2;
    int q = threadIdx.x;
    for (; q + (U - 1) * kSampleThreads < n4; q += U * kSampleThreads) {
      float4 v[U];
#pragma unroll
      for (int j = 0; j < U; ++j) v[j] = x4[q + j * kSampleThreads];
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int i = 4 * (q + j * kSampleThreads);
        f(v[j].x, i); f(v[j].y, i + 1); f(v[j].z, i + 2); f(v[j].w, i + 3);
      }
    }
    for (; q < n4; q += kSampleThreads) {
      const float4 v = x4[q];
      f(v.x, 4 * q); f(v.y, 4 * q + 1); f(v.z, 4 * q + 2); f(v.w, 4 * q + 3);
    }
    return;
  }
  int i = threadIdx.x;
  for (; i + (U - 1) * kSampleThreads < V; i += U * kSampleThreads) {
    float v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) v[j] = x[i + j * kSampleThreads];
#pragma unroll
    for (int j = 0; j < U; ++j) f(v[j], i + j * kSampleThreads);
  }
  for (; i < V; i += kSampleThreads) f(x[i], i);
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

__device__ __forceinline__ float key_value(unsigned int key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

constexpr int kCand = 2048;      // candidates the short way holds
constexpr int kFastK = 512;      // largest top-k it takes, and the nucleus size it aims at

struct Candidates {
  unsigned long long entry[kCand];   // sort entries
  unsigned long long mass[kCand];    // inclusive fixed-point masses, then single weights
  unsigned long long wsum[32];
  int count;
  int chosen;
};

__device__ __forceinline__ unsigned long long fixed_weight(float w) { return __float2ull_rz(w * 1099511627776.f); }

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* wsum) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) wsum[warp] = v;
  __syncthreads();
  unsigned long long total = 0ull;
  for (int w = 0; w < kSampleThreads / 32; ++w) total += wsum[w];
  return total;
}

// Inclusive scan over 2 * kSampleThreads values, thread t holding values 2t and 2t + 1.
__device__ __forceinline__ void block_scan2_u64(unsigned long long a0, unsigned long long a1, unsigned long long* i0,
                                                unsigned long long* i1, unsigned long long* wsum) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long s = a0 + a1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long n = __shfl_up_sync(0xffffffffu, s, o);
    if (lane >= o) s += n;
  }
  __syncthreads();
  if (lane == 31) wsum[warp] = s;
  __syncthreads();
  unsigned long long before = 0ull;
  for (int w = 0; w < warp; ++w) before += wsum[w];
  *i0 = before + s - a1;
  *i1 = before + s;
}

// Ascending bitonic sort of entry[0, n2), n2 a power of two of at most 2 * kSampleThreads.
__device__ __forceinline__ void sort_entries(unsigned long long* entry, int n2) {
  const int t = threadIdx.x;
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (t < (n2 >> 1)) {
        const int l = ((t / stride) * stride << 1) + (t % stride);
        const int r = l + stride;
        const bool up = (l & size) == 0;
        const unsigned long long a = entry[l], b = entry[r];
        if ((a > b) == up) { entry[l] = b; entry[r] = a; }
      }
      __syncthreads();
    }
  }
}

// The short way.  Returns the drawn token, or -1 when this row has to go the long way.
// thread_max_key: the largest key among the logits this thread read in the first pass.
__device__ int sample_from_candidates(const float* __restrict__ x, int V, float best, unsigned int key_max,
                                      float inv_temp, int k, float p, float u, unsigned int thread_max_key,
                                      bool vec, Candidates& cd) {
  const int tid = threadIdx.x;
  const bool topk = k > 0 && k < V;
  if (topk && k > kFastK) return -1;
  const int kp = topk ? k : min(kFastK, V);
  // pivot: the kp-th largest of the threads' maxima; at least kp logits are >= it
  unsigned int lo = 0u, hi = key_max;
  while (lo < hi) {
    const unsigned int mid = lo + ((hi - lo) >> 1) + ((hi - lo) & 1u);
    if (__syncthreads_count(thread_max_key >= mid) >= kp) lo = mid; else hi = mid - 1u;
  }
  const unsigned int pivot = lo;
  if (tid == 0) { cd.count = 0; cd.chosen = 0x7fffffff; }
  __syncthreads();
  unsigned long long zf = 0ull;       // without top-k: the mass of the whole row
  for_each_logit(x, V, vec, [&](float v, int i) {
    const unsigned int key = order_key(v);
    if (!topk) zf += fixed_weight(token_weight(v, best, inv_temp));
    if (key >= pivot) {
      const int slot = atomicAdd(&cd.count, 1);
      if (slot < kCand) cd.entry[slot] = ((unsigned long long)(~key) << 32) | (unsigned int)i;
    }
  });
  __syncthreads();
  const int n = cd.count;
  if (n > kCand) return -1;
  const unsigned long long z_row = topk ? 0ull : block_sum_u64(zf, cd.wsum);
  int n2 = 2;
  while (n2 < n) n2 <<= 1;
  for (int s = n + tid; s < n2; s += kSampleThreads) cd.entry[s] = ~0ull;
  __syncthreads();
  sort_entries(cd.entry, n2);            // logit descending, token id ascending

  // weights of the top-k set (the first k entries), inclusive masses
  const int nk = topk ? k : n;           // n >= k by the choice of the pivot
  const int q0 = 2 * tid, q1 = 2 * tid + 1;
  unsigned long long w0 = 0ull, w1 = 0ull;
  if (q0 < nk) w0 = fixed_weight(token_weight(key_value(~(unsigned int)(cd.entry[q0] >> 32)), best, inv_temp));
  if (q1 < nk) w1 = fixed_weight(token_weight(key_value(~(unsigned int)(cd.entry[q1] >> 32)), best, inv_temp));
  unsigned long long m0, m1;
  block_scan2_u64(w0, w1, &m0, &m1, cd.wsum);
  if (q0 < kCand) cd.mass[q0] = m0;
  if (q1 < kCand) cd.mass[q1] = m1;
  __syncthreads();
  int keep = nk;
  if (p < 1.f) {
    const unsigned long long z = topk ? cd.mass[nk - 1] : z_row;
    const unsigned long long limit = (unsigned long long)((double)(p > 0.f ? p : 0.f) * (double)z);
    if (!topk && cd.mass[n - 1] <= limit) return -1;      // the nucleus reaches past the candidates
    // an entry stays iff the mass of the strictly larger logits is <= limit: a prefix of whole tie groups
    bool ok0 = false, ok1 = false;
    if (q0 < nk) {
      int st = q0;
      const unsigned int kh = (unsigned int)(cd.entry[q0] >> 32);
      while (st > 0 && (unsigned int)(cd.entry[st - 1] >> 32) == kh) --st;
      ok0 = (st > 0 ? cd.mass[st - 1] : 0ull) <= limit;
    }
    if (q1 < nk) {
      int st = q1;
      const unsigned int kh = (unsigned int)(cd.entry[q1] >> 32);
      while (st > 0 && (unsigned int)(cd.entry[st - 1] >> 32) == kh) --st;
      ok1 = (st > 0 ? cd.mass[st - 1] : 0ull) <= limit;
    }
    keep = __syncthreads_count(ok0) + __syncthreads_count(ok1);
  }
  // the draw walks the kept entries in token-id order: sort them by id, scan their weights
  const unsigned long long z2 = cd.mass[keep - 1];
  const unsigned long long target = (unsigned long long)((double)u * (double)z2);
  __syncthreads();
  const unsigned long long e0 = q0 < n2 ? cd.entry[q0] : ~0ull, e1 = q1 < n2 ? cd.entry[q1] : ~0ull;
  __syncthreads();
  if (q0 < n2) { cd.mass[q0] = w0; cd.entry[q0] = q0 < keep ? ((e0 & 0xffffffffull) << 32) | (unsigned int)q0 : ~0ull; }
  if (q1 < n2) { cd.mass[q1] = w1; cd.entry[q1] = q1 < keep ? ((e1 & 0xffffffffull) << 32) | (unsigned int)q1 : ~0ull; }
  __syncthreads();
  int k2 = 2;
  while (k2 < keep) k2 <<= 1;
  sort_entries(cd.entry, k2);
  unsigned long long a0 = 0ull, a1 = 0ull;
  if (q0 < keep) a0 = cd.mass[(unsigned int)(cd.entry[q0] & 0xffffffffull)];
  if (q1 < keep) a1 = cd.mass[(unsigned int)(cd.entry[q1] & 0xffffffffull)];
  unsigned long long c0, c1;
  block_scan2_u64(a0, a1, &c0, &c1, cd.wsum);
  if (q0 < keep && c0 >= target) atomicMin(&cd.chosen, (int)(cd.entry[q0] >> 32));
  if (q1 < keep && c1 >= target) atomicMin(&cd.chosen, (int)(cd.entry[q1] >> 32));
  __syncthreads();
  return cd.chosen;        // the last kept entry has c == z2 >= target: always set
}

#define KEPT_K(key, i) ((key) > T || ((key) == T && (i) <= E))
#define KEPT(key, i) (KEPT_K(key, i) && (key) >= T2)

// The draw over the set given by the thresholds, in token-id order.  Warp w owns the tokens
// [w * W, (w + 1) * W), W a multiple of 128, as rows of 128: lane l of a row holds four consecutive
// tokens (one 16-byte load with `vec`).  The distribution function at the end of lane l of row r is
// before(w) + (carry(r) + scan(l)): the warps' totals added in warp order, the rows' totals added in
// row order, the lanes' sums by the warp's inclusive scan.  The first pass forms the totals; the
// warp whose total reaches the target forms the same numbers again and stops at the first row,
// lane and token that reach it, so it always finds one.
__device__ int ordered_draw(const float* __restrict__ x, int V, float best, float inv_temp, unsigned int T, int E,
                            unsigned int T2, float u, int fallback, bool vec, Shared& sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int W = (((V + 31) / 32) + 127) & ~127;
  const int w0 = min(V, warp * W), w1 = min(V, w0 + W);
  const int rows = (w1 - w0 + 127) >> 7;
  const bool all = T == 0u && T2 == 0u;       // no threshold: every token is kept
  auto weight = [&](float v, int i) {
    if (all) return i < V ? token_weight(v, best, inv_temp) : 0.f;
    const unsigned int key = order_key(v);
    return (i < V && KEPT(key, i)) ? token_weight(v, best, inv_temp) : 0.f;
  };
  auto load4 = [&](int i) {        // the four logits from token i on (zeros past the end of the row)
    if (vec) return i < V ? *reinterpret_cast<const float4*>(x + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    return make_float4(i < V ? x[i] : 0.f, i + 1 < V ? x[i + 1] : 0.f, i + 2 < V ? x[i + 2] : 0.f,
                       i + 3 < V ? x[i + 3] : 0.f);
  };
  auto lane_sum = [&](const float4& v, int i) {
    return ((weight(v.x, i) + weight(v.y, i + 1)) + weight(v.z, i + 2)) + weight(v.w, i + 3);
  };
  auto scan = [&](float q) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float nb = __shfl_up_sync(0xffffffffu, q, o);
      if (lane >= o) q += nb;
    }
    return q;
  };
  float carry = 0.f;
  for (int r0 = 0; r0 < rows; r0 += 8) {
    float4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = r0 + j < rows ? load4(w0 + ((r0 + j) << 7) + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (r0 + j >= rows) break;
      const float incl = scan(lane_sum(v[j], w0 + ((r0 + j) << 7) + 4 * lane));
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  if (lane == 0) sh.f[warp] = carry;
  if (tid == 0) sh.found = 0x7fffffff;
  __syncthreads();
  float before = 0.f, total = 0.f;
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    if (w == warp) before = total;
    total += sh.f[w];
  }
  const float target = u * total;
  if (lane == 0 && before + carry >= target) atomicMin(&sh.found, warp);
  __syncthreads();
  const int owner = sh.found;          // the last warp always qualifies (u < 1)
  __syncthreads();
  if (tid == 0) sh.found = fallback;   // stays if rounding leaves the chosen lane without a kept token
  __syncthreads();
  if (warp == owner) {
    float c = 0.f;
    for (int r = 0; r < rows; ++r) {
      const int i = w0 + (r << 7) + 4 * lane;
      const float4 v = load4(i);
      const float incl = scan(lane_sum(v, i));
      const float row_total = __shfl_sync(0xffffffffu, incl, 31);
      if (before + (c + row_total) >= target) {
        const unsigned int hit = __ballot_sync(0xffffffffu, before + (c + incl) >= target);
        const int first = __ffs(hit) - 1;              // lane 31 always qualifies
        float excl = __shfl_up_sync(0xffffffffu, incl, 1);
        if (lane == 0) excl = 0.f;
        if (lane == first) {
          const float wv[4] = {weight(v.x, i), weight(v.y, i + 1), weight(v.z, i + 2), weight(v.w, i + 3)};
          float part = 0.f;
          int last = -1;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (wv[j] > 0.f) {
              last = i + j;
              part += wv[j];
              if (before + (c + (excl + part)) >= target) break;
            }
          }
          if (last >= 0) sh.found = last;
        }
        break;
      }
      c += row_total;
    }
  }
  __syncthreads();
  return sh.found;
}

__global__ void __launch_bounds__(kSampleThreads, 1)
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
  // one choice for every row of the launch, so that a row's sums do not depend on its place in the batch
  const bool vec = (V % 4 == 0) && (reinterpret_cast<uintptr_t>(logits) % 16 == 0);
  for_each_logit(x, V, vec, [&](float v, int i) {
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  });
  const unsigned int thread_max_key = order_key(best);
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
  const int index = draw_index[r];
  const float u = uniform_from_counter((unsigned long long)seeds[r], (unsigned long long)(unsigned int)index);
  int k = top_k[r];
  const float p = top_p[r];
  unsigned int T = 0u, T2 = 0u;
  int E = V;
  int chosen = -1;
  if ((k > 0 && k < V) || p < 1.f) {
    __shared__ Candidates cd;
    if (best > -INFINITY && best < INFINITY)
      chosen = sample_from_candidates(x, V, best, key_max, inv_temp, k, p, u, thread_max_key, vec, cd);
  } else {
    chosen = ordered_draw(x, V, best, inv_temp, T, E, T2, u, best_i, vec, sh);
  }
  if (chosen >= 0) {
    if (tid == 0) {
      out[r] = chosen;
      if (advance_index) draw_index[r] = index + 1;
    }
    return;
  }

  // ---- 2. top-k: threshold key T and the index E up to which ties at T are kept
  if (k > 0 && k < V) {
    unsigned int lo = 0u, hi = key_max;
    while (lo < hi) {
      const unsigned int mid = lo + ((hi - lo) >> 1) + ((hi - lo) & 1u);
      int c = 0;
      for_each_logit(x, V, vec, [&](float v, int) { c += order_key(v) >= mid; });
      if (block_sum_int(c, sh) >= k) lo = mid; else hi = mid - 1u;
    }
    T = lo;
    int c = 0;
    for_each_logit(x, V, vec, [&](float v, int) { c += order_key(v) > T; });
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

  // ---- 3. mass of the top-k set
  float z = 0.f;
  for_each_logit(x, V, vec, [&](float v, int i) {
    const unsigned int key = order_key(v);
    if (KEPT_K(key, i)) z += token_weight(v, best, inv_temp);
  });
  const float Z = block_sum_float(z, sh);

  // ---- 4. nucleus: smallest key T2 with mass(key > T2) <= top_p * Z
  if (p < 1.f) {
    const float limit = p * Z;
    unsigned int lo = 0u, hi = key_max;
    while (lo < hi) {
      const unsigned int mid = lo + ((hi - lo) >> 1);
      float mgt = 0.f;
      for_each_logit(x, V, vec, [&](float v, int i) {
        const unsigned int key = order_key(v);
        if (key > mid && KEPT_K(key, i)) mgt += token_weight(v, best, inv_temp);
      });
      if (block_sum_float(mgt, sh) <= limit) hi = mid; else lo = mid + 1u;
    }
    T2 = lo;
  }
  // ---- 5. the draw
  chosen = ordered_draw(x, V, best, inv_temp, T, E, T2, u, best_i, vec, sh);
  if (tid == 0) {
    out[r] = chosen;
    if (advance_index) draw_index[r] = index + 1;
  }
}
#undef KEPT
#undef KEPT_K


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
