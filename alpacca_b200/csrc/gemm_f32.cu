// C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]) in true 32-bit: plain FMA on the CUDA
// cores, no tensor-core mode of reduced precision anywhere.
//
// Every output element is one chain of fused multiply-adds over k = 0..K-1 in
// ascending order, so its value does not depend on M, on the tile it falls
// into, or on what other rows are in the batch: the same token gives the same
// bits alone and in any batch.  This is the matrix product of the 32-bit path
// (the reference's float32 path uses BLAS SGEMM, alpacca/tensor.py:91-97).
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

__global__ void __launch_bounds__(256)
gemm_f32_nt_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                   const float* __restrict__ bias, float* __restrict__ C, int ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // each thread stages 4 elements of A and 4 of W per k-tile: row = tid / 4, k = (tid % 4) * 4 ..+3
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + e][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + e][lrow] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
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
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

AB_API int ab_gemm_f32_nt(const float* A, int lda, const float* W, int ldw, const float* bias, float* C, int ldc,
                          int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return AB_OK;
  if (K < 0) return AB_BAD_ARG;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return AB_BAD_ARG;
  gemm_f32_nt_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, bias, C, ldc, M, N, K);
  return ab_launch_status();
}
