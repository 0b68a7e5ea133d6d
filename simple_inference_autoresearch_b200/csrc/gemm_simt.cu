// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores, with 32-bit accumulation.
//
// Every linear layer of the reference is y = x W^T with W stored (out, in)
// row-major and no bias (ops/attention.py:107-177, ops/mlp.py:98-214,
// ops/embedding.py:123-141).  This unit is the true 32-bit path of those products
// (plain FFMA, no reduced-precision matrix mode) and the fallback of the bf16
// path for shapes the tensor-core unit refuses.
//
//  * gemm_nt_tiled: 64x64x16 tiles, 256 threads, 4x4 outputs per thread.  Each
//    output is one chain of fmaf over k = 0..K-1 in order, so a row's result does
//    not depend on M, on the row's place in the batch or on the tile it falls in.
//  * gemm_nt_skinny: for few rows (M <= 16) of bf16 data with K % 8 == 0.  One warp
//    per output column streams the weight row once with 16-byte loads; lanes own
//    k-chunks c = lane, lane+32, ...; a shuffle tree joins them.  Order depends on
//    K only.
#include "common.cuh"

namespace siar {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) gemm_nt_tiled_kernel(const TIn* __restrict__ A, const TIn* __restrict__ W,
                                                           TOut* __restrict__ C, int M, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int lrow = tid >> 2;        // 0..63
  const int lk = (tid & 3) * 4;     // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + e][lrow] = (am < M && k < K) ? to_f32(A[(size_t)am * K + k]) : 0.f;
      Ws[lk + e][lrow] = (wn < N && k < K) ? to_f32(W[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * N + n] = from_f32<TOut>(acc[i][j]);
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 p = __bfloat1622float2(h[i]);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}

template <typename TOut, int MB>
__global__ void __launch_bounds__(256) gemm_nt_skinny_kernel(const __nv_bfloat16* __restrict__ A,
                                                            const __nv_bfloat16* __restrict__ W,
                                                            TOut* __restrict__ C, int M, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const int m0 = blockIdx.y * MB;
  const int chunks = K >> 3;
  const uint4* wrow = reinterpret_cast<const uint4*>(W + (size_t)n * K);
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
  for (int c = lane; c < chunks; c += 32) {
    float w[8];
    unpack8(__ldg(wrow + c), w);
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (m0 + m < M) {
        float x[8];
        unpack8(*reinterpret_cast<const uint4*>(A + (size_t)(m0 + m) * K + (size_t)c * 8), x);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[m] = fmaf(x[e], w[e], acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < M) C[(size_t)(m0 + m) * N + n] = from_f32<TOut>(v);
  }
}

}  // namespace siar

using namespace siar;

SIAR_DEFINE_PDL_SWITCH()

// in_bf16: dtype of A and W; out_f32: dtype of C.  allow_skinny picks the
// streaming kernel where it applies (bf16, M <= 16, K % 8 == 0, 16-byte aligned).
extern "C" int siar_gemm_nt_simt(int in_bf16, int out_f32, const void* A, const void* W, void* C, int M, int N,
                                 int K, int allow_skinny, void* stream) {
  if (M == 0 || N == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (in_bf16 && allow_skinny && M <= 16 && (K % 8) == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0) {
    const __nv_bfloat16* a = (const __nv_bfloat16*)A;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
    if (M <= 4) {
      dim3 grid((N + 7) / 8, 1);
      if (out_f32) launch_kernel(gemm_nt_skinny_kernel<float, 4>, grid, 256, 0, s, a, w, (float*)C, M, N, K);
      else launch_kernel(gemm_nt_skinny_kernel<__nv_bfloat16, 4>, grid, 256, 0, s, a, w, (__nv_bfloat16*)C, M, N, K);
    } else {
      dim3 grid((N + 7) / 8, (M + 7) / 8);
      if (out_f32) launch_kernel(gemm_nt_skinny_kernel<float, 8>, grid, 256, 0, s, a, w, (float*)C, M, N, K);
      else launch_kernel(gemm_nt_skinny_kernel<__nv_bfloat16, 8>, grid, 256, 0, s, a, w, (__nv_bfloat16*)C, M, N, K);
    }
    return (int)cudaGetLastError();
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  if (in_bf16) {
    if (out_f32)
      launch_kernel(gemm_nt_tiled_kernel<__nv_bfloat16, float>, grid, 256, 0, s, (const __nv_bfloat16*)A,
                                                                     (const __nv_bfloat16*)W, (float*)C, M, N, K);
    else
      launch_kernel(gemm_nt_tiled_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, s, 
          (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K);
  } else {
    launch_kernel(gemm_nt_tiled_kernel<float, float>, grid, 256, 0, s, (const float*)A, (const float*)W, (float*)C, M, N, K);
  }
  return (int)cudaGetLastError();
}
