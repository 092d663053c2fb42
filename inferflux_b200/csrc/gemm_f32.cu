// True float32 matrix product for the 32-bit path: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
//
// The reference has no 32-bit model path (its traits cover half and bfloat16
// only, runtime/backends/cuda/native/common/dtype_traits.cuh:13-30) and calls
// cuBLAS with float32 accumulation for every projection
// (runtime/backends/cuda/native/cublas_gemm.cpp:84-102).  This kernel uses
// plain FFMA on CUDA cores, no tensor cores and no reduced-precision mode, and
// adds the K products of an output element in index order whatever M is, so a
// row's result does not depend on what else is in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K, long long lda, long long ldc) {
  pdl_enter();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;          // tx -> N direction, ty -> M direction
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  // each thread loads 4 elements of A and 4 of W per K-slab: row = tid / 4, k = (tid % 4) * 4 .. +3
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + u][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.0f;
      Ws[lk + u][lrow] = (wn < N && k < K) ? W[(size_t)wn * K + k] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.0f);
    }
  }
}
}  // namespace

IFX_API int ifx_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                         long long lda, long long ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return IFX_ERR_UNSUPPORTED;
  int ifx_rc = 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  ifx_rc = launch_pdl(gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, A, W, bias, C, M, N, K, lda, ldc);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}
