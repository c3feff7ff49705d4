// Embedding lookup, residual add + RMSNorm, SiLU·up, rotary positions + cache
// store.  Each replaces a chain of PyTorch calls in the reference
// (gllm/model/model.py:175-182, gllm/model/layers/norm.py:15-22,
// gllm/model/transformer.py:58-75, gllm/model/layers/mlp.py:44-47,
// gllm/model/layers/attention.py:76-119,156-161).
//
// T is the activation / weight-matrix type (float or bf16).  The residual
// stream, norm weights, norm statistics and rotation angles are always fp32.
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

// ------------------------------------------------- 8 elements at a time
// Vec8<T>: eight consecutive elements of an activation row as fp32, moved with 16-byte
// (bf16) or 2 x 16-byte (fp32) accesses.  The wide kernels below need rows whose length is a
// multiple of 8 and 16-byte aligned pointers; otherwise the plain kernels run.
template <typename T> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------- embedding
// resid[n, :] = table[tokens[n], :] (upcast to fp32).  A token outside the
// vocabulary sets a status bit and yields zeros: no fault, the host raises.
// A negative token id means "the token last sampled for this request": it is read from
// sampled[token_row[n]], which the previous step's argmax left on the device.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const int* __restrict__ sampled,
                                 const int* __restrict__ token_row, const T* __restrict__ table,
                                 float* __restrict__ resid, int n_tokens, int hidden, int vocab, float scale,
                                 int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  int tok = tokens[n];
  if (tok < 0 && sampled) tok = sampled[token_row[n]];
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && threadIdx.x == 0) atomicOr(status, GLLM_STATUS_TOKEN_RANGE);
  const T* row = table + (size_t)(ok ? tok : 0) * hidden;
  float* dst = resid + (size_t)n * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_float(row[i]) * scale : 0.f;
}

template <typename T>
__global__ void embedding_wide_kernel(const int* __restrict__ tokens, const int* __restrict__ sampled,
                                      const int* __restrict__ token_row, const T* __restrict__ table,
                                      float* __restrict__ resid, int n_tokens, int hidden, int vocab,
                                      float scale, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  int tok = tokens[n];
  if (tok < 0 && sampled) tok = sampled[token_row[n]];
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && threadIdx.x == 0) atomicOr(status, GLLM_STATUS_TOKEN_RANGE);
  const T* row = table + (size_t)(ok ? tok : 0) * hidden;
  float* dst = resid + (size_t)n * hidden;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
    float v[8];
    Vec8<T>::load(row + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = ok ? v[i] * scale : 0.f;
    Vec8<float>::store(dst + c, v);
  }
}

template <typename T>
static int embedding_launch(const int* tokens, const int* sampled, const int* token_row, const T* table,
                            float* resid, int n_tokens, int hidden, int vocab, float scale, int* status,
                            cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
  if (hidden % 8 == 0 && aligned16(table) && aligned16(resid))
    return gllm_launch(embedding_wide_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, tokens, sampled,
                       token_row, table, resid, n_tokens, hidden, vocab, scale, status);
  return gllm_launch(embedding_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, tokens, sampled, token_row,
                     table, resid, n_tokens, hidden, vocab, scale, status);
}

// `scale` multiplies every looked-up row (1 for an architecture without an embedding multiplier).
GLLM_API int gllm_embedding_f32(const int* tokens, const int* sampled, const int* token_row, const float* table,
                                float* resid, int n_tokens, int hidden, int vocab, float scale, int* status,
                                cudaStream_t stream) {
  return embedding_launch<float>(tokens, sampled, token_row, table, resid, n_tokens, hidden, vocab, scale, status,
                                 stream);
}
GLLM_API int gllm_embedding_bf16(const int* tokens, const int* sampled, const int* token_row,
                                 const __nv_bfloat16* table, float* resid, int n_tokens, int hidden, int vocab,
                                 float scale, int* status, cudaStream_t stream) {
  return embedding_launch<__nv_bfloat16>(tokens, sampled, token_row, table, resid, n_tokens, hidden, vocab, scale,
                                         status, stream);
}

// ------------------------------------------------------------ int32 scatter
// dst[idx[i]] = val[i] (block-table entries that changed since the last step; indices are distinct).
__global__ void scatter_i32_kernel(int* __restrict__ dst, int64_t dst_size, const int* __restrict__ idx,
                                   const int* __restrict__ val, int n, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int64_t at = idx[i];
    if (at < 0 || at >= dst_size) {
      atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      continue;
    }
    dst[at] = val[i];
  }
}
GLLM_API int gllm_scatter_i32(int* dst, int64_t dst_size, const int* idx, const int* val, int n, int* status,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  const int blocks = (n + 255) / 256;
  return gllm_launch(scatter_i32_kernel, dim3(blocks < 1024 ? blocks : 1024), dim3(256), 0, stream, dst, dst_size,
                     idx, val, n, status);
}

// ------------------------------------------------- logit scale and soft cap
// x = x * scale; then, with cap > 0, x = cap * tanh(x / cap).  fp32, in place, over n values.
__global__ void scale_softcap_kernel(float* __restrict__ x, int64_t n, float scale, float cap) {
  pdl_trigger();
  pdl_wait();
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float v = x[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v * inv_cap);
    x[i] = v;
  }
}
GLLM_API int gllm_scale_softcap_f32(float* x, int64_t n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const int64_t blocks = (n + threads - 1) / threads;
  return gllm_launch(scale_softcap_kernel, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(threads), 0, stream,
                     x, n, scale, cap);
}

// ------------------------------------------------------------ bias of a product
// x[r][c] += bias[c], in place, the sum rounded to T (a projection with a bias: the reference has none,
// gllm/model/layers/linear.py:20; other architectures do).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, int64_t stride, const float* __restrict__ bias, int rows, int n) {
  pdl_trigger();
  pdl_wait();
  for (int r = blockIdx.y; r < rows; r += gridDim.y) {
    T* row = x + (int64_t)r * stride;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < n; c += gridDim.x * blockDim.x)
      row[c] = from_float<T>(to_float(row[c]) + bias[c]);
  }
}
template <typename T>
static int add_bias_launch(T* x, int64_t stride, const float* bias, int rows, int n, cudaStream_t stream) {
  if (rows <= 0 || n <= 0) return 0;
  const int bx = (n + 255) / 256;
  return gllm_launch(add_bias_kernel<T>, dim3(bx < 64 ? bx : 64, rows < 4096 ? rows : 4096), dim3(256), 0, stream, x,
                     stride, bias, rows, n);
}
GLLM_API int gllm_add_bias_f32(float* x, int64_t stride, const float* bias, int rows, int n, cudaStream_t stream) {
  return add_bias_launch<float>(x, stride, bias, rows, n, stream);
}
GLLM_API int gllm_add_bias_bf16(__nv_bfloat16* x, int64_t stride, const float* bias, int rows, int n,
                                cudaStream_t stream) {
  return add_bias_launch<__nv_bfloat16>(x, stride, bias, rows, n, stream);
}

// ------------------------------------------------------- RMSNorm of every head
// Heads first_head .. first_head + n_heads - 1 of every row of x (a row is heads of d columns side by side): each
// head's d values are divided by sqrt(mean of their squares + eps) and multiplied by weight[0 .. d) (or 1 + weight),
// in place; statistics in fp32.  One warp per (row, head); d up to 256.  (A norm of the queries and the keys before
// the rotation: the reference has none; other architectures do.)
template <typename T>
__global__ void rmsnorm_heads_kernel(T* __restrict__ x, int64_t stride, const float* __restrict__ weight, int rows,
                                     int first_head, int n_heads, int d, float eps, int unit_offset) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  float w[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = lane + 32 * k;
    w[k] = c < d ? (unit_offset ? 1.0f + weight[c] : weight[c]) : 0.f;
  }
  pdl_wait();
  if (item >= (int64_t)rows * n_heads) return;
  const int r = (int)(item / n_heads), h = (int)(item - (int64_t)r * n_heads);
  T* v = x + (int64_t)r * stride + (int64_t)(first_head + h) * d;
  float a[8], ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = lane + 32 * k;
    a[k] = c < d ? to_float(v[c]) : 0.f;
    ss += a[k] * a[k];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = lane + 32 * k;
    if (c < d) v[c] = from_float<T>(a[k] * inv * w[k]);
  }
}
template <typename T>
static int rmsnorm_heads_launch(T* x, int64_t stride, const float* weight, int rows, int first_head, int n_heads, int d,
                                float eps, int unit_offset, cudaStream_t stream) {
  if (rows <= 0 || n_heads <= 0) return 0;
  if (d <= 0 || d > 256 || first_head < 0) return (int)cudaErrorInvalidValue;
  const int64_t items = (int64_t)rows * n_heads;
  const int64_t blocks = (items + 7) / 8;                 // eight warps a block
  if (blocks > 0x7fffffff) return (int)cudaErrorInvalidValue;
  return gllm_launch(rmsnorm_heads_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, x, stride, weight, rows,
                     first_head, n_heads, d, eps, unit_offset);
}
GLLM_API int gllm_rmsnorm_heads_f32(float* x, int64_t stride, const float* weight, int rows, int first_head, int n_heads,
                                    int d, float eps, int unit_offset, cudaStream_t stream) {
  return rmsnorm_heads_launch<float>(x, stride, weight, rows, first_head, n_heads, d, eps, unit_offset, stream);
}
GLLM_API int gllm_rmsnorm_heads_bf16(__nv_bfloat16* x, int64_t stride, const float* weight, int rows, int first_head,
                                     int n_heads, int d, float eps, int unit_offset, cudaStream_t stream) {
  return rmsnorm_heads_launch<__nv_bfloat16>(x, stride, weight, rows, first_head, n_heads, d, eps, unit_offset, stream);
}

// ------------------------------------------------------ add + RMSNorm (fused)
// For output row i (source row r = rows ? rows[i] : i):
//   x = resid[r] (+ branch[r])            fp32
//   if (!rows) resid[r] = x               the residual stream moves on
//   out[i] = x * rsqrt(mean(x^2) + eps) * (w or 1 + w)
// y = x / sqrt(mean + eps) * w as gllm/model/layers/norm.py:20-22, with the
// statistic in fp32 whatever T is.  One block per row; the row lives in
// shared memory between the two passes, so it is read from HBM once.
// The branch may come as `n_parts` fp32 partial sums (a product cut along K whose splits
// were left unsummed, laid out [part][row][hidden]): they are added in ascending order.
template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ branch, const float* __restrict__ parts, int n_parts,
                                   int64_t part_stride, float* __restrict__ resid,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int n_rows, int hidden, float eps,
                                   int unit_offset) {
  extern __shared__ float row_buf[];  // hidden floats + 32 scratch
  float* scratch = row_buf + hidden;
  pdl_trigger();
  // the norm's weight never depends on the kernel before this one: it is fetched before the wait
  constexpr int WPRE = 4;
  float wpre[WPRE];
#pragma unroll
  for (int k = 0; k < WPRE; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    wpre[k] = c < hidden ? weight[c] : 0.f;
  }
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= n_rows) return;
  const size_t r = rows ? (size_t)rows[i] : (size_t)i;
  float* res = resid + r * hidden;
  const T* br = branch ? branch + r * hidden : nullptr;
  const float* pr = parts ? parts + r * hidden : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x = res[c];
    if (pr) {
      const float b = sum_parts16(pr + c, n_parts, part_stride);
      x += to_float(from_float<T>(b));           // rounded as the product itself would have rounded it
    } else if (br) {
      x += to_float(br[c]);
    }
    row_buf[c] = x;
    if ((br || pr) && !rows) res[c] = x;
    ss += x * x;
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* o = out + (size_t)i * hidden;
#pragma unroll
  for (int k = 0; k < WPRE; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < hidden) o[c] = from_float<T>(row_buf[c] * inv * (unit_offset ? 1.0f + wpre[k] : wpre[k]));
  }
  for (int c = threadIdx.x + WPRE * blockDim.x; c < hidden; c += blockDim.x) {
    const float w = unit_offset ? 1.0f + weight[c] : weight[c];
    o[c] = from_float<T>(row_buf[c] * inv * w);
  }
}

// The same with 8 columns per access and the row kept in registers (up to MAXC chunks of 8 per thread;
// the launcher picks the smallest MAXC that holds a row, since registers decide how many rows an SM has
// in flight).  The norm's weight does not depend on
// the kernel before this one and is fetched before the dependency wait.
template <typename T, int MAXC, bool PARTS>
__global__ void add_rmsnorm_wide_kernel(const T* __restrict__ branch, const float* __restrict__ parts, int n_parts,
                                        int64_t part_stride, float* __restrict__ resid,
                                        const float* __restrict__ weight, T* __restrict__ out,
                                        const int* __restrict__ rows, int n_rows, int hidden, float eps,
                                        int unit_offset) {
  __shared__ float scratch[32];
  pdl_trigger();
  const int i = blockIdx.x;
  float x[MAXC][8], w[MAXC][8];
#pragma unroll
  for (int k = 0; k < MAXC; ++k) {
    const int c = (threadIdx.x + k * blockDim.x) * 8;
    if (c < hidden) Vec8<float>::load(weight + c, w[k]);
  }
  const size_t r = rows ? (size_t)rows[i] : (size_t)i;   // a step input
  pdl_wait();
  float* res = resid + r * hidden;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXC; ++k) {
    const int c = (threadIdx.x + k * blockDim.x) * 8;
    if (c >= hidden) break;
    Vec8<float>::load(res + c, x[k]);
    if (PARTS) {                                          // unsummed splits, 8 columns of a split per load
      float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      const float* src = parts + r * hidden + c;
#pragma unroll 4
      for (int p = 0; p < n_parts; ++p) {
        float t[8];
        Vec8<float>::load(src + (int64_t)p * part_stride, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) b[e] += t[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) x[k][e] += to_float(from_float<T>(b[e]));   // rounded as the product would be
      if (!rows) Vec8<float>::store(res + c, x[k]);
    } else if (branch) {
      float b[8];
      Vec8<T>::load(branch + r * hidden + c, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[k][e] += b[e];
      if (!rows) Vec8<float>::store(res + c, x[k]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += x[k][e] * x[k][e];
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* o = out + (size_t)i * hidden;
#pragma unroll
  for (int k = 0; k < MAXC; ++k) {
    const int c = (threadIdx.x + k * blockDim.x) * 8;
    if (c >= hidden) break;
    float y[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = x[k][e] * inv * (unit_offset ? 1.0f + w[k][e] : w[k][e]);
    Vec8<T>::store(o + c, y);
  }
}

// The same for rows whose branch arrives as unsummed splits (decoding, short portions): a cluster of blocks
// shares one row, each block sums, adds and squares its stretch of columns, the blocks exchange
// their sums of squares through distributed shared memory (added in rank order) and each
// normalises its own stretch.  A row of a handful of tokens is then read through many SMs' ports
// instead of one.  Up to 4 columns per thread.
template <typename T>
__global__ void add_rmsnorm_cluster_kernel(const float* __restrict__ parts, int n_parts, int64_t part_stride,
                                           float* __restrict__ resid, const float* __restrict__ weight,
                                           T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps,
                                           int unit_offset) {
  __shared__ float scratch[32];
  __shared__ float all_ss[16];
  pdl_trigger();
  cluster_arrive_started();
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank(), n_ranks = (int)cluster.num_blocks();
  const int cols_per = (hidden + n_ranks - 1) / n_ranks;
  const int c_begin = rank * cols_per, c_end = min(hidden, c_begin + cols_per);
  constexpr int PER = 4;
  float w[PER], x[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {                       // the weight does not depend on the kernel before
    const int c = c_begin + threadIdx.x + k * blockDim.x;
    w[k] = c < c_end ? weight[c] : 0.f;
  }
  const int i = blockIdx.y;
  const size_t r = rows ? (size_t)rows[i] : (size_t)i;
  pdl_wait();
  float* res = resid + r * hidden;
  const float* pr = parts + r * hidden;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = c_begin + threadIdx.x + k * blockDim.x;
    x[k] = 0.f;
    if (c < c_end) {
      const float b = sum_parts16(pr + c, n_parts, part_stride);
      x[k] = res[c] + to_float(from_float<T>(b));       // rounded as the product itself would have rounded it
      if (!rows) res[c] = x[k];
      ss += x[k] * x[k];
    }
  }
  // every block pushes its sum into all blocks' slots: after one cluster barrier each reads only its
  // own shared memory, so none has to stay for the others
  const float mine = block_sum(ss, scratch);
  cluster_wait_started();
  if (threadIdx.x < n_ranks) *cluster.map_shared_rank(&all_ss[rank], threadIdx.x) = mine;
  cluster.sync();
  float total = 0.f;
  for (int rk = 0; rk < n_ranks; ++rk) total += all_ss[rk];
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* o = out + (size_t)i * hidden;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = c_begin + threadIdx.x + k * blockDim.x;
    if (c < c_end) o[c] = from_float<T>(x[k] * inv * (unit_offset ? 1.0f + w[k] : w[k]));
  }
}

template <typename T>
static int add_rmsnorm_launch(const T* branch, const float* parts, int n_parts, int64_t part_stride, float* resid,
                              const float* weight, T* out, const int* rows, int n_rows, int hidden, float eps,
                              int unit_offset, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_parts > 16) return (int)cudaErrorInvalidValue;
  // few rows of unsummed splits: a cluster of blocks per row (below)
  const bool few_rows_of_parts = parts && !branch && n_rows <= 64 && hidden >= 1024 && hidden <= 8 * 4 * 256;
  if (!few_rows_of_parts && hidden % 8 == 0 && aligned16(resid) && aligned16(weight) && aligned16(out) &&
      (!branch || aligned16(branch)) && (!parts || (aligned16(parts) && part_stride % 4 == 0))) {
    const int chunks = hidden / 8;
    const int wide_threads = chunks >= 256 ? 256 : (chunks >= 128 ? 128 : (chunks >= 64 ? 64 : 32));
    // as few chunks per thread as the row needs: the kernel keeps them in registers, and the registers
    // decide how many rows an SM works on at a time
    if (chunks <= wide_threads)
      return parts ? gllm_launch(add_rmsnorm_wide_kernel<T, 1, true>, dim3(n_rows), dim3(wide_threads), 0, stream,
                                 branch, parts, n_parts, part_stride, resid, weight, out, rows, n_rows, hidden, eps,
                                 unit_offset)
                   : gllm_launch(add_rmsnorm_wide_kernel<T, 1, false>, dim3(n_rows), dim3(wide_threads), 0, stream,
                                 branch, parts, n_parts, part_stride, resid, weight, out, rows, n_rows, hidden, eps,
                                 unit_offset);
    if (chunks <= wide_threads * 2)
      return parts ? gllm_launch(add_rmsnorm_wide_kernel<T, 2, true>, dim3(n_rows), dim3(wide_threads), 0, stream,
                                 branch, parts, n_parts, part_stride, resid, weight, out, rows, n_rows, hidden, eps,
                                 unit_offset)
                   : gllm_launch(add_rmsnorm_wide_kernel<T, 2, false>, dim3(n_rows), dim3(wide_threads), 0, stream,
                                 branch, parts, n_parts, part_stride, resid, weight, out, rows, n_rows, hidden, eps,
                                 unit_offset);
    if (chunks <= wide_threads * 4)
      return parts ? gllm_launch(add_rmsnorm_wide_kernel<T, 4, true>, dim3(n_rows), dim3(wide_threads), 0, stream,
                                 branch, parts, n_parts, part_stride, resid, weight, out, rows, n_rows, hidden, eps,
                                 unit_offset)
                   : gllm_launch(add_rmsnorm_wide_kernel<T, 4, false>, dim3(n_rows), dim3(wide_threads), 0, stream,
                                 branch, parts, n_parts, part_stride, resid, weight, out, rows, n_rows, hidden, eps,
                                 unit_offset);
  }
  if (parts && !branch && n_rows <= 64 && hidden >= 1024 && hidden <= 8 * 4 * 256) {
    return gllm_launch_cluster(add_rmsnorm_cluster_kernel<T>, dim3(8, n_rows), dim3(256), 0, stream, 8u, parts,
                               n_parts, part_stride, resid, weight, out, rows, hidden, eps, unit_offset);
  }
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (parts) threads = hidden >= 1024 ? 1024 : threads;
  size_t smem = (size_t)(hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return gllm_launch(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, stream, branch, parts, n_parts,
                     part_stride, resid, weight, out, rows, n_rows, hidden, eps, unit_offset);
}

GLLM_API int gllm_add_rmsnorm_f32(const float* branch, const float* parts, int n_parts, int64_t part_stride,
                                  float* resid, const float* weight, float* out, const int* rows, int n_rows,
                                  int hidden, float eps, int unit_offset, cudaStream_t stream) {
  return add_rmsnorm_launch<float>(branch, parts, n_parts, part_stride, resid, weight, out, rows, n_rows, hidden,
                                   eps, unit_offset, stream);
}
GLLM_API int gllm_add_rmsnorm_bf16(const __nv_bfloat16* branch, const float* parts, int n_parts,
                                   int64_t part_stride, float* resid, const float* weight, __nv_bfloat16* out,
                                   const int* rows, int n_rows, int hidden, float eps, int unit_offset,
                                   cudaStream_t stream) {
  return add_rmsnorm_launch<__nv_bfloat16>(branch, parts, n_parts, part_stride, resid, weight, out, rows, n_rows,
                                           hidden, eps, unit_offset, stream);
}

// ------------------------------------------------- sum of unsummed splits
// out[i] = parts[0][i] + parts[1][i] + ... in ascending order, rounded to T.
template <typename T>
__global__ void sum_parts_kernel(const float* __restrict__ parts, int n_parts, int64_t part_stride,
                                 T* __restrict__ out, int64_t n) {
  pdl_trigger();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    out[i] = from_float<T>(sum_parts16(parts + i, n_parts, part_stride));
  }
}
template <typename T>
static int sum_parts_launch(const float* parts, int n_parts, int64_t part_stride, T* out, int64_t n,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > gllm_sm_count() * 8) blocks = gllm_sm_count() * 8;
  return gllm_launch(sum_parts_kernel<T>, dim3(blocks), dim3(256), 0, stream, parts, n_parts, part_stride, out, n);
}
GLLM_API int gllm_sum_parts_f32(const float* parts, int n_parts, int64_t part_stride, float* out, int64_t n,
                                cudaStream_t stream) {
  return sum_parts_launch<float>(parts, n_parts, part_stride, out, n, stream);
}
GLLM_API int gllm_sum_parts_bf16(const float* parts, int n_parts, int64_t part_stride, __nv_bfloat16* out,
                                 int64_t n, cudaStream_t stream) {
  return sum_parts_launch<__nv_bfloat16>(parts, n_parts, part_stride, out, n, stream);
}

// ------------------------------------------------------------------ SiLU · up
// gate_up is [n, 2*inter]: out = silu(gate) * up, silu(z) = z / (1 + exp(-z))
// (gllm/model/layers/mlp.py:44-47).  block == 0: the gate is the first `inter` columns, the up the
// rest.  block > 0: blocks of `block` gate columns alternate with the `block` up columns of the
// same features (the layout the gated product's weight uses).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int n_rows, int inter,
                                int block) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n_rows * inter;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / inter, c = idx - r * inter;
    const size_t gc = block ? (c / block) * 2 * block + c % block : c;
    const float g = to_float(gate_up[r * 2 * inter + gc]);
    const float u = to_float(gate_up[r * 2 * inter + gc + (block ? block : inter)]);
    const float s = g / (1.0f + expf(-g));
    out[idx] = from_float<T>(s * u);
  }
}

template <typename T>
__global__ void silu_mul_wide_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int n_rows, int inter,
                                     int block) {
  pdl_trigger();
  pdl_wait();
  const int per_row = inter / 8;
  const size_t total = (size_t)n_rows * per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / per_row;
    const int c = (int)(idx - r * per_row) * 8;
    float g[8], u[8], y[8];
    const int gc = block ? (c / block) * 2 * block + c % block : c;
    Vec8<T>::load(gate_up + r * 2 * inter + gc, g);
    Vec8<T>::load(gate_up + r * 2 * inter + gc + (block ? block : inter), u);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = g[e] / (1.0f + expf(-g[e])) * u[e];
    Vec8<T>::store(out + r * inter + c, y);
  }
}

template <typename T>
static int silu_mul_launch(const T* gate_up, T* out, int n_rows, int inter, int block, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (block < 0 || (block > 0 && inter % block)) return (int)cudaErrorInvalidValue;
  if (inter % 8 == 0 && block % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
    const size_t chunks = (size_t)n_rows * (inter / 8);
    int wide_blocks = (int)((chunks + 255) / 256);
    if (wide_blocks > gllm_sm_count() * 16) wide_blocks = gllm_sm_count() * 16;
    return gllm_launch(silu_mul_wide_kernel<T>, dim3(wide_blocks), dim3(256), 0, stream, gate_up, out, n_rows, inter,
                       block);
  }
  const size_t total = (size_t)n_rows * inter;
  int blocks = (int)((total + 255) / 256);
  if (blocks > gllm_sm_count() * 16) blocks = gllm_sm_count() * 16;
  return gllm_launch(silu_mul_kernel<T>, dim3(blocks), dim3(256), 0, stream, gate_up, out, n_rows, inter, block);
}
GLLM_API int gllm_silu_mul_f32(const float* gate_up, float* out, int n_rows, int inter, int block,
                               cudaStream_t stream) {
  return silu_mul_launch<float>(gate_up, out, n_rows, inter, block, stream);
}
GLLM_API int gllm_silu_mul_bf16(const __nv_bfloat16* gate_up, __nv_bfloat16* out, int n_rows, int inter, int block,
                                cudaStream_t stream) {
  return silu_mul_launch<__nv_bfloat16>(gate_up, out, n_rows, inter, block, stream);
}

// ------------------------------------------- rotary positions + cache store
// qkv is [n, (hq + 2*hkv) * d]: q heads, then k heads, then v heads.
// For every token: rotate q and k in place (first `rotary_dim` dims of each
// head; pairs are the two halves (i, i + rotary_dim/2) as
// gllm/model/layers/attention.py:91-118, or neighbours (2i, 2i+1) when
// `interleaved`), angle = position * inv_freq[i] in fp32, and store the
// rotated k and the v into the token's cache slot (post-rotation keys are
// cached, gllm/model/layers/attention.py:156-161).
// Cache layer layout: [page][k|v][kv_head][block_size][d].
// inv_freq == nullptr: no rotation.  slot_mapping == nullptr or slot < 0: no store.
// qkv may arrive as `n_parts` unsummed fp32 splits of the projection ([part][token][width]):
// the kernel first sums them in ascending order into qkv (rounded to T, as the product would have).
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const float* __restrict__ parts, int n_parts,
                                  int64_t part_stride, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping,
                                  T* __restrict__ cache, int n_tokens, int hq, int hkv, int d, int rotary_dim,
                                  int interleaved, int block_size, int num_pages, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  T* row = qkv + (size_t)n * (hq + 2 * hkv) * d;
  const int half = rotary_dim / 2;
  if (parts) {
    const int width = (hq + 2 * hkv) * d;
    const float* src = parts + (size_t)n * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
      row[c] = from_float<T>(sum_parts16(src + c, n_parts, part_stride));
    __syncthreads();
  }
  if (inv_freq) {
    const float pos = (float)positions[n];
    // one (head, pair) per thread-iteration over q and k heads
    const int pairs = (hq + hkv) * half;
    for (int idx = threadIdx.x; idx < pairs; idx += blockDim.x) {
      const int h = idx / half, i = idx - h * half;
      const float ang = pos * inv_freq[i];
      float s, c;
      sincosf(ang, &s, &c);
      T* head = row + (size_t)h * d;  // q heads then k heads are contiguous
      const int i0 = interleaved ? 2 * i : i;
      const int i1 = interleaved ? 2 * i + 1 : i + half;
      const float x0 = to_float(head[i0]), x1 = to_float(head[i1]);
      head[i0] = from_float<T>(x0 * c - x1 * s);
      head[i1] = from_float<T>(x0 * s + x1 * c);
    }
  }
  if (!slot_mapping) return;
  const int slot = slot_mapping[n];
  if (slot < 0) return;
  const int page = slot / block_size, off = slot - page * block_size;
  if (page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, GLLM_STATUS_PAGE_RANGE);
    return;
  }
  __syncthreads();  // rotated k is complete
  const T* k = row + (size_t)hq * d;
  const T* v = k + (size_t)hkv * d;
  const size_t page_base = (size_t)page * 2 * hkv * block_size * d;
  for (int idx = threadIdx.x; idx < hkv * d; idx += blockDim.x) {
    const int h = idx / d, j = idx - h * d;
    const size_t o = page_base + ((size_t)h * block_size + off) * d + j;
    cache[o] = k[idx];
    cache[o + (size_t)hkv * block_size * d] = v[idx];
  }
}

// The same for the common case (a summed projection; pairs are the two halves; rotary_dim and head size
// multiples of 16): one thread owns 8 consecutive pairs, takes sine and cosine once and reuses them for
// every head, moves 16 bytes at a time and writes the rotated k and the v straight to the cache.  The
// position, the cache slot and so sine and cosine are step inputs: they are ready before the
// dependency wait returns.  A thread's heads are all loaded before the first is stored.
template <typename T, bool PARTS>
__global__ void rope_store_wide_kernel(T* __restrict__ qkv, const float* __restrict__ parts, int n_parts,
                                       int64_t part_stride, const int* __restrict__ positions,
                                       const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping,
                                       T* __restrict__ cache, int n_tokens, int hq, int hkv, int d, int rotary_dim,
                                       int block_size, int num_pages, int* __restrict__ status) {
  pdl_trigger();
  const int n = blockIdx.x;
  const int width = (hq + 2 * hkv) * d;
  T* row = qkv + (size_t)n * width;
  const int half = rotary_dim / 2;
  // where this token's k and v go
  int64_t cache_base = -1;
  if (slot_mapping) {
    const int slot = slot_mapping[n];
    if (slot >= 0) {
      const int page = slot / block_size, off = slot - page * block_size;
      if (page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      } else {
        cache_base = ((int64_t)page * 2 * hkv * block_size + off) * d;
      }
    }
  }
  const int64_t head_stride = (int64_t)block_size * d, v_plane = (int64_t)hkv * block_size * d;
  const int chunks = inv_freq ? half / 8 : 0;
  const int my_chunk = chunks > 0 ? threadIdx.x % chunks : 0;
  float sn[8], cs[8];
  if (chunks > 0) {
    const float pos = (float)positions[n];
#pragma unroll
    for (int e = 0; e < 8; ++e) sincosf(pos * inv_freq[my_chunk * 8 + e], &sn[e], &cs[e]);
  }
  pdl_wait();
  // 8 columns of this token: from qkv, or the sum of the unsummed splits (8 columns of a split per load,
  // rounded to T as the product would have been)
  const float* prow = PARTS ? parts + (size_t)n * width : nullptr;
  auto load8 = [&](int col, float* v) {
    if (PARTS) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
#pragma unroll 4
      for (int p = 0; p < n_parts; ++p) {
        float t[8];
        Vec8<float>::load(prow + col + (int64_t)p * part_stride, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += t[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = to_float(from_float<T>(v[e]));
    } else {
      Vec8<T>::load(row + col, v);
    }
  };
  // rotated part of q and k heads: (head, chunk of 8 pairs), two heads per turn
  if (chunks > 0) {
    const int step = blockDim.x / chunks;
    for (int h = threadIdx.x / chunks; h < hq + hkv; h += 2 * step) {
      const int h2 = h + step;
      const bool two = h2 < hq + hkv;
      const int c0 = h * d + my_chunk * 8, c1 = c0 + half;
      const int e0 = h2 * d + my_chunk * 8, e1 = e0 + half;
      float a[8], b[8], a2[8], b2[8];
      load8(c0, a);
      load8(c1, b);
      if (two) {
        load8(e0, a2);
        load8(e1, b2);
      }
      auto finish = [&](int hh, int x0, int x1, float* u, float* v) {
        float ra[8], rb[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          ra[e] = u[e] * cs[e] - v[e] * sn[e];
          rb[e] = u[e] * sn[e] + v[e] * cs[e];
        }
        Vec8<T>::store(row + x0, ra);
        Vec8<T>::store(row + x1, rb);
        if (hh >= hq && cache_base >= 0) {
          T* kdst = cache + cache_base + (int64_t)(hh - hq) * head_stride;
          Vec8<T>::store(kdst + my_chunk * 8, ra);
          Vec8<T>::store(kdst + half + my_chunk * 8, rb);
        }
      };
      finish(h, c0, c1, a, b);
      if (two) finish(h2, e0, e1, a2, b2);
    }
  }
  // everything that is not rotated and has to move: the tail of k heads past rotary_dim, and v, to the
  // cache; with unsummed splits also the tails of the q heads, and all of it into qkv
  if (cache_base < 0 && !PARTS) return;
  const int rot = chunks > 0 ? rotary_dim : 0;
  const int tail_chunks = (d - rot) / 8;
  const int v_chunks = d / 8;
  const int first_head = PARTS ? 0 : hq;                // q tails only when they have to be summed
  const int tail_heads = hq + hkv - first_head;
  const int plain_items = tail_heads * tail_chunks + hkv * v_chunks;
  for (int item = threadIdx.x; item < plain_items; item += blockDim.x) {
    int h, col_in_head;
    if (item < tail_heads * tail_chunks) {
      h = first_head + item / tail_chunks;
      col_in_head = rot + (item % tail_chunks) * 8;
    } else {
      const int j = item - tail_heads * tail_chunks;
      h = hq + hkv + j / v_chunks;
      col_in_head = (j % v_chunks) * 8;
    }
    float v[8];
    load8(h * d + col_in_head, v);
    if (PARTS) Vec8<T>::store(row + h * d + col_in_head, v);
    if (h >= hq && cache_base >= 0) {
      const bool is_v = h >= hq + hkv;
      const int kvh = is_v ? h - hq - hkv : h - hq;
      Vec8<T>::store(cache + cache_base + (is_v ? v_plane : 0) + (int64_t)kvh * head_stride + col_in_head, v);
    }
  }
}

// The same for a projection that arrives as unsummed splits (decoding, short portions):
// one thread owns one pair of one head, sums the splits of its two elements, rotates them and
// writes them to qkv and, for k and v, to the cache: no value makes a second trip through global
// memory.  The position, the cache slot, the frequency and so the sine and cosine do not depend on
// the kernel before this one: they are ready when the dependency wait returns.
template <typename T>
__global__ void rope_store_parts_kernel(T* __restrict__ qkv, const float* __restrict__ parts, int n_parts,
                                        int64_t part_stride, const int* __restrict__ positions,
                                        const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping,
                                        T* __restrict__ cache, int n_tokens, int hq, int hkv, int d, int rotary_dim,
                                        int interleaved, int block_size, int num_pages, int* __restrict__ status) {
  pdl_trigger();
  const int n = blockIdx.y;
  const int half_d = d / 2;
  const int item = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = item < (hq + 2 * hkv) * half_d;
  const int h = live ? item / half_d : 0, i = live ? item - h * half_d : 0;
  const int half = inv_freq ? rotary_dim / 2 : 0;
  const bool rotated = h < hq + hkv && i < half;
  int i0, i1;
  if (rotated) {
    i0 = interleaved ? 2 * i : i;
    i1 = interleaved ? 2 * i + 1 : i + half;
  } else if (h < hq + hkv) {
    i0 = 2 * half + 2 * (i - half);                      // the head's tail past the rotated dims
    i1 = i0 + 1;
  } else {
    i0 = 2 * i;
    i1 = i0 + 1;
  }
  float sn = 0.f, cs = 1.f;
  if (live && rotated) sincosf((float)positions[n] * inv_freq[i], &sn, &cs);
  int64_t cache_base = -1;
  if (live && slot_mapping && h >= hq) {
    const int slot = slot_mapping[n];
    if (slot >= 0) {
      const int page = slot / block_size, off = slot - page * block_size;
      if (page >= num_pages) atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      else {
        const bool is_v = h >= hq + hkv;
        const int kvh = is_v ? h - hq - hkv : h - hq;
        cache_base = (((int64_t)page * 2 + (is_v ? 1 : 0)) * hkv + kvh) * block_size * d + (int64_t)off * d;
      }
    }
  }
  pdl_wait();
  if (!live) return;
  const int width = (hq + 2 * hkv) * d;
  const float* src = parts + (size_t)n * width + (size_t)h * d;
  const T x0 = from_float<T>(sum_parts16(src + i0, n_parts, part_stride));   // rounded as the product would be
  const T x1 = from_float<T>(sum_parts16(src + i1, n_parts, part_stride));
  const T y0 = from_float<T>(to_float(x0) * cs - to_float(x1) * sn);
  const T y1 = from_float<T>(to_float(x0) * sn + to_float(x1) * cs);
  T* row = qkv + (size_t)n * width + (size_t)h * d;
  row[i0] = rotated ? y0 : x0;
  row[i1] = rotated ? y1 : x1;
  if (cache_base >= 0) {
    cache[cache_base + i0] = rotated ? y0 : x0;
    cache[cache_base + i1] = rotated ? y1 : x1;
  }
}

template <typename T>
static int rope_store_launch(T* qkv, const float* parts, int n_parts, int64_t part_stride, const int* positions,
                             const float* inv_freq, const int* slot_mapping,
                             T* cache, int n_tokens, int hq, int hkv, int d, int rotary_dim, int interleaved,
                             int block_size, int num_pages, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || n_parts > 16) return (int)cudaErrorInvalidValue;
  const int eff_rot = inv_freq ? rotary_dim : 0;
  // a few tokens of unsummed splits take the pair-per-thread kernel below (more blocks, less latency)
  const bool few_tokens_of_parts = parts && n_tokens <= 64 && d % 2 == 0;
  if (!few_tokens_of_parts && !interleaved && d % 8 == 0 && eff_rot % 16 == 0 && aligned16(qkv) &&
      (!slot_mapping || aligned16(cache)) && (!parts || (aligned16(parts) && part_stride % 4 == 0)) &&
      (eff_rot == 0 || 128 % (eff_rot / 16) == 0)) {
    return parts ? gllm_launch(rope_store_wide_kernel<T, true>, dim3(n_tokens), dim3(128), 0, stream, qkv, parts,
                               n_parts, part_stride, positions, inv_freq, slot_mapping, cache, n_tokens, hq, hkv, d,
                               rotary_dim, block_size, num_pages, status)
                 : gllm_launch(rope_store_wide_kernel<T, false>, dim3(n_tokens), dim3(128), 0, stream, qkv, parts,
                               n_parts, part_stride, positions, inv_freq, slot_mapping, cache, n_tokens, hq, hkv, d,
                               rotary_dim, block_size, num_pages, status);
  }
  if (parts && n_tokens <= 65535 && d % 2 == 0) {   // few tokens, or sizes the wide kernel does not take
    const int items = (hq + 2 * hkv) * (d / 2);
    return gllm_launch(rope_store_parts_kernel<T>, dim3((items + 255) / 256, n_tokens), dim3(256), 0, stream, qkv,
                       parts, n_parts, part_stride, positions, inv_freq, slot_mapping, cache, n_tokens, hq, hkv, d,
                       rotary_dim, interleaved, block_size, num_pages, status);
  }
  int work = max((hq + hkv) * (rotary_dim / 2), hkv * d);
  int threads = work >= 512 ? 256 : (work >= 128 ? 128 : 64);
  if (parts && (hq + 2 * hkv) * d >= 1024) threads = 1024;   // unsummed splits: one column per thread and turn
  return gllm_launch(rope_store_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, qkv, parts, n_parts,
                     part_stride, positions, inv_freq, slot_mapping, cache, n_tokens, hq, hkv, d, rotary_dim,
                     interleaved, block_size, num_pages, status);
}
GLLM_API int gllm_rope_store_f32(float* qkv, const float* parts, int n_parts, int64_t part_stride,
                                 const int* positions, const float* inv_freq, const int* slot_mapping,
                                 float* cache, int n_tokens, int hq, int hkv, int d, int rotary_dim,
                                 int interleaved, int block_size, int num_pages, int* status,
                                 cudaStream_t stream) {
  return rope_store_launch<float>(qkv, parts, n_parts, part_stride, positions, inv_freq, slot_mapping, cache,
                                  n_tokens, hq, hkv, d, rotary_dim, interleaved, block_size, num_pages, status,
                                  stream);
}
GLLM_API int gllm_rope_store_bf16(__nv_bfloat16* qkv, const float* parts, int n_parts, int64_t part_stride,
                                  const int* positions, const float* inv_freq, const int* slot_mapping,
                                  __nv_bfloat16* cache, int n_tokens, int hq, int hkv, int d, int rotary_dim,
                                  int interleaved, int block_size, int num_pages, int* status,
                                  cudaStream_t stream) {
  return rope_store_launch<__nv_bfloat16>(qkv, parts, n_parts, part_stride, positions, inv_freq, slot_mapping,
                                          cache, n_tokens, hq, hkv, d, rotary_dim, interleaved, block_size,
                                          num_pages, status, stream);
}
