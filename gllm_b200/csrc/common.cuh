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

// Sum of up to 16 unsummed splits of a product, in ascending order; all loads are issued
// before the first add so that they overlap.
__device__ __forceinline__ float sum_parts16(const float* __restrict__ p, int n_parts, int64_t stride) {
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = i < n_parts ? __ldcg(p + (int64_t)i * stride) : 0.f;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) s += v[i];
  return s;
}

// ---- programmatic dependent launch
// Every kernel of the engine is launched so that it may be scheduled while the kernel before it
// on the stream is still draining (its blocks become resident and run their set-up).  The rule
// that keeps this safe: a kernel calls pdl_wait() before its first access to global memory, which
// returns only when every earlier kernel has completed and its writes are visible; and it calls
// pdl_trigger() at once, which lets the kernel after it be scheduled early in turn.  Both are
// no-ops for a kernel that was launched the ordinary way.
// A block may touch another block's shared memory (or allocate tensor memory as a pair) only once that
// block runs.  The blocks of a cluster usually start together, but microseconds apart when the kernel
// is scheduled early and SMs come free one by one.  Every thread calls cluster_arrive_started() at the
// kernel's top and cluster_wait_started() before the first such access: the wait is over as soon as
// every block of the cluster has started, which by then it normally has.
__device__ __forceinline__ void cluster_arrive_started() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_started() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
// Streaming multiprocessors of the current device (asked once; grid sizes and split counts follow it).
static inline int gllm_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0, count = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && count > 0)
      n = count;
    else
      return 1;
  }
  return n;
}

static inline bool gllm_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("GLLM_B200_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on != 0;
}

// Launches `kernel` on `stream` with programmatic stream serialization allowed (see above);
// returns the cudaError_t as an int.
template <typename... KArgs, typename... Args>
static inline int gllm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gllm_pdl_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose blocks form clusters of `cluster_x` along x (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
static inline int gllm_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gllm_pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
