// True 32-bit matrix product on the CUDA cores: C[M,N] = A[M,K] * B[N,K]^T,
// the `x @ W.T` of gllm/model/layers/linear.py:20 with W stored [out, in].
//
// No tensor-core mode of any kind (no TF32): every product is an FFMA.  Each
// output element is accumulated by one thread over k = 0..K-1 in ascending
// order whatever M is, so a token's result does not depend on the batch it is
// in.  This is the reference path that shows faults bf16 hides; it is not
// meant to be fast.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N,
                int K, int64_t lda, int64_t ldb, int64_t ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread loads 4 elements of A and 4 of B per k-tile
  const int lrow = tid / 4;        // 0..63
  const int lk = (tid % 4) * 4;    // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lrow, bn = n0 + lrow;
      As[lk + e][lrow] = (am < M && k < K) ? A[(int64_t)am * lda + k] : 0.f;
      Bs[lk + e][lrow] = (bn < N && k < K) ? B[(int64_t)bn * ldb + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
      if (n < N) C[(int64_t)m * ldc + n] = acc[i][j];
    }
  }
}
}  // namespace

GLLM_API int gllm_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, int64_t lda,
                           int64_t ldb, int64_t ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
  return gllm_launch(gemm_f32_kernel, grid, dim3(256), 0, stream, A, B, C, M, N, K, lda, ldb, ldc);
}
