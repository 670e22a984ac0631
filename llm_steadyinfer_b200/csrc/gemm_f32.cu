// True 32-bit matrix product for the fp32 path: C[M, N] = A[M, K] * W[N, K]^T with plain
// FFMA and fp32 accumulation, no tensor cores and no reduced-precision mode. (The
// reference's "fp32" GEMM is cuBLAS TF32, src/source/op/kernels/cuda/matmul_kernel.cu:128-150;
// its exact fallback is the one-block-per-row kernel at :12-63.) The k loop runs in one
// fixed order for every output element, whatever M is, so a row's result does not depend
// on how many other rows share the step.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, long long lda, const float* __restrict__ W,
                long long ldw, float* __restrict__ C, long long ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 x 16 tile of A and of W: 1024 elements each, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;
      const int r = idx >> 4, c = idx & 15;
      const int k = k0 + c;
      As[c][r] = (m0 + r < M && k < K) ? A[(size_t)(m0 + r) * lda + k] : 0.f;
      Ws[c][r] = (n0 + r < N && k < K) ? W[(size_t)(n0 + r) * ldw + k] : 0.f;
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
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

SI_EXPORT int si_gemm_f32(const float* A, long long lda, const float* W, long long ldw, float* C,
                          long long ldc, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return -2;
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
  return si_last_error();
}
