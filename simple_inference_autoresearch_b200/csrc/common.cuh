// Shared device helpers for the sm_100a kernels of this library.
//
// Conventions used by every unit in this folder:
//  * Entry points are `extern "C" int siar_<name>(..., void* stream)`; they launch
//    on the given stream and return the cudaError_t of the launch as an int.
//  * A batch of sequences is described by three int32 device arrays:
//      slot_ids[B]   cache slot of each sequence,
//      q_start[B+1]  first packed row of each sequence's new tokens,
//      base_len[B]   tokens the sequence already holds in the cache.
//    Row t of sequence b sits at absolute position base_len[b] + (t - q_start[b]).
//  * Keys and values live in pages of `page_tokens` positions:
//      pool[page][kv_head][page_tokens][head_dim],
//    and block_table[slot * max_pages + p] names the page of positions
//    [p * page_tokens, (p + 1) * page_tokens) of that slot.
//  * Reductions run in an order that depends only on the row itself (its width,
//    its absolute key positions), never on what else is in the batch.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace siar {

enum StatusBits : int {
  kStatusTokenOutOfRange = 1,
  kStatusWaitExpired = 2,
  kStatusBadPage = 4,
  kStatusLengthPastGrid = 8,
};

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// Largest b in [0, B) with q_start[b] <= t (q_start is non-decreasing, q_start[0] == 0).
__device__ __forceinline__ int find_sequence(const int* __restrict__ q_start, int B, int t) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (q_start[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum in a fixed order: lane tree inside each warp, then warp 0 adds
// the per-warp sums in warp order.  `scratch` holds at least 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel of the library is launched with the "programmatic stream serialization"
// attribute: its blocks may become resident while the kernel before it on the stream is
// still running, so that launch latency and the prologue (barrier set-up, tensor-memory
// allocation, loads of weights, which no earlier kernel writes) overlap the predecessor's
// tail.  A kernel calls pdl_launch_dependents() first (the next kernel may start its own
// prologue) and pdl_wait() before it reads or writes anything an earlier kernel touches;
// pdl_wait() returns once all earlier kernels have completed and their writes are visible.
// Both are no-ops for a kernel launched without the attribute.
// One rule for code in front of pdl_wait(): whatever is read there must have been written before
// the step's first kernel (weights, the batch description, the block table, cache positions of
// earlier steps).  And one for code behind it: data of the kernel in front must not be read through a
// const __restrict__ pointer when the address is known before the wait, because the compiler may
// move such ("invariant") loads above the wait; read it through a plain pointer or with the
// volatile loads of attention_mma.cu.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- timeline marks (profiling builds)
// With -DSIAR_TIMING thread 0 of every block appends (tag * 16 + phase + (blocks << 16), block, globaltimer)
// records to a buffer shared by all units: phase 0 = block started, 2 = its dependency wait
// returned, 1 = block done.  Without the flag the macro is empty.
#ifdef SIAR_TIMING
__device__ unsigned long long* g_trace_buf = nullptr;
__device__ unsigned int* g_trace_cursor = nullptr;
__device__ unsigned int g_trace_capacity = 0;
__device__ __forceinline__ void trace_mark(unsigned int tag, unsigned int phase) {
  if (g_trace_buf == nullptr || threadIdx.x != 0 || threadIdx.y != 0) return;
  const unsigned int rec = atomicAdd(g_trace_cursor, 1u);
  if (rec >= g_trace_capacity) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  g_trace_buf[rec * 3ull] = (unsigned long long)(tag * 16u + phase) |
                            ((unsigned long long)(gridDim.x * gridDim.y * gridDim.z) << 16);
  g_trace_buf[rec * 3ull + 1] = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  g_trace_buf[rec * 3ull + 2] = t;
}
#define SIAR_TRACE(tag, phase) siar::trace_mark(tag, phase)
#else
#define SIAR_TRACE(tag, phase)
#endif

inline bool& pdl_enabled() {
  static bool on = true;
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace siar

// One switch per shared object: siar_set_pdl(0) launches every kernel of the unit
// without the attribute (plain stream order).
#ifdef SIAR_TIMING
#define SIAR_DEFINE_PDL_SWITCH()                                                                      \
  extern "C" void siar_set_pdl(int on) { siar::pdl_enabled() = on != 0; }                             \
  extern "C" void siar_set_trace(unsigned long long* buf, unsigned int* cursor, unsigned int capacity) { \
    cudaMemcpyToSymbol(siar::g_trace_buf, &buf, sizeof(buf));                                         \
    cudaMemcpyToSymbol(siar::g_trace_cursor, &cursor, sizeof(cursor));                                \
    cudaMemcpyToSymbol(siar::g_trace_capacity, &capacity, sizeof(capacity));                          \
  }
#else
#define SIAR_DEFINE_PDL_SWITCH() \
  extern "C" void siar_set_pdl(int on) { siar::pdl_enabled() = on != 0; }
#endif
