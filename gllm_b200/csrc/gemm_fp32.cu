// True 32-bit matrix product on the CUDA cores: C[M,N] = A[M,K] * B[N,K]^T,
// the `x @ W.T` of gllm/model/layers/linear.py:20 with W stored [out, in].
//
// No tensor-core mode of any kind (no TF32): every product is an FFMA.  Each
// output element is accumulated by one thread over k = 0..K-1 in ascending
// order whatever M is, so a token's result does not depend on the batch it is
// in.  This is the reference path that shows faults bf16 hides.  Two kernels:
// a 128 x 128 tile with 8 x 8 outputs per thread, 16-byte global loads and the
// next tile's loads in flight while this one is multiplied (rows 16-byte
// aligned, K a multiple of 4), and a plain 64 x 64 tile for everything else
// and for steps of few tokens, where the weight's trip from memory is the time.
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

// ---- 128 x 128 x 16 tile, 256 threads, 8 x 8 outputs per thread (as 2 x 2 blocks of 4 x 4, 64 apart, so
// that a warp's shared-memory reads are 16-byte vectors without bank conflicts)
constexpr int WM = 128, WN = 128, WK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_wide_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N,
                     int K, int64_t lda, int64_t ldb, int64_t ldc) {
  __shared__ __align__(16) float As[WK][WM];
  __shared__ __align__(16) float Bs[WK][WN];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * WM, n0 = blockIdx.x * WN;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  // a thread loads two 16-byte pieces of A and two of B per k-tile: rows lrow and lrow + 64, columns lk .. lk + 3
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  float4 ra[2], rb[2];
  auto load_tile = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int am = m0 + lrow + h * 64, bn = n0 + lrow + h * 64, k = k0 + lk;
      ra[h] = (am < M && k < K) ? *reinterpret_cast<const float4*>(A + (int64_t)am * lda + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      rb[h] = (bn < N && k < K) ? *reinterpret_cast<const float4*>(B + (int64_t)bn * ldb + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto store_tile = [&]() {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = lrow + h * 64;
      As[lk + 0][r] = ra[h].x; As[lk + 1][r] = ra[h].y; As[lk + 2][r] = ra[h].z; As[lk + 3][r] = ra[h].w;
      Bs[lk + 0][r] = rb[h].x; Bs[lk + 1][r] = rb[h].y; Bs[lk + 2][r] = rb[h].z; Bs[lk + 3][r] = rb[h].w;
    }
  };
  load_tile(0);
  for (int k0 = 0; k0 < K; k0 += WK) {
    store_tile();
    __syncthreads();
    if (k0 + WK < K) load_tile(k0 + WK);               // in flight while this tile is multiplied
#pragma unroll
    for (int kk = 0; kk < WK; ++kk) {
      float a[8], b[8];
      const float4 a0 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[kk][64 + tx * 4]);
      a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
      b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= M) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int n = n0 + jh * 64 + tx * 4;
      float* dst = C + (int64_t)m * ldc + n;
      if (n + 3 < N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
        *reinterpret_cast<float4*>(dst) = make_float4(acc[i][jh * 4], acc[i][jh * 4 + 1], acc[i][jh * 4 + 2], acc[i][jh * 4 + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < N) dst[j] = acc[i][jh * 4 + j];
      }
    }
  }
}
}  // namespace

GLLM_API int gllm_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, int64_t lda,
                           int64_t ldb, int64_t ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  const bool vectors = K % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(B) & 15) == 0;
  if (vectors && M > 64) {
    dim3 wide((N + WN - 1) / WN, (M + WM - 1) / WM);
    if (wide.y > 65535) return (int)cudaErrorInvalidValue;
    return gllm_launch(gemm_f32_wide_kernel, wide, dim3(256), 0, stream, A, B, C, M, N, K, lda, ldb, ldc);
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
  return gllm_launch(gemm_f32_kernel, grid, dim3(256), 0, stream, A, B, C, M, N, K, lda, ldb, ldc);
}
