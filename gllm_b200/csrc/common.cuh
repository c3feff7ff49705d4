// Shared helpers for the sm_100a kernels of this engine.
//
// Every exported entry point is `extern "C"`, takes raw device pointers, sizes
// and a CUDA stream, launches on that stream and returns the cudaError_t of the
// launch as an int (0 = success).  Nothing here allocates.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define GLLM_API extern "C" __attribute__((visibility("default")))

// Bits of the device status word that kernels set instead of trapping.
enum GllmStatus : int {
  GLLM_STATUS_OK = 0,
  GLLM_STATUS_TOKEN_RANGE = 1,    // a token id outside [0, vocab)
  GLLM_STATUS_PAGE_RANGE = 2,     // a page id outside the pool
  GLLM_STATUS_WAIT_TIMEOUT = 4,   // a bounded wait on an mbarrier ran out
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
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

// Sum over a whole block in one fixed order (lanes by butterfly, then warps in
// index order), so a row's statistic does not depend on what else is in the
// batch.  `scratch` holds at least 32 floats.  Every thread gets the result.
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

static inline int gllm_launch_result() { return (int)cudaGetLastError(); }
