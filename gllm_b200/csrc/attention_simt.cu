// Causal attention over the paged cache on the CUDA cores, for any head size
// that is a multiple of 16 up to 256 and any number of heads and groups.
// It is the whole attention of the 32-bit path and the fallback of the bf16
// path for head sizes its tensor-core kernels do not take.
//
// It replaces the gather of the padded context plus the dense
// softmax(QK^T / sqrt(D) + bias) V of the reference
// (gllm/model/layers/attention.py:165-173,
// gllm/ops/attention/reference_attention.py:40-48): no bias tensor, no score
// tensor and no gathered copy exist here.  A token at position p of a request
// sees the keys at positions max(0, p - window + 1) .. p of that request
// (window <= 0: all of them), found through the request's row of the block
// table.  Scores, the running maximum, the running sum and the output
// accumulator are fp32; the order of accumulation depends only on absolute
// key positions (blocks of 32 keys aligned to multiples of 32), never on how
// the request was cut into steps or on the rest of the batch.
//
// One warp per (token, query head).
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t out_stride,
                      const T* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                      const int* __restrict__ positions, const int* __restrict__ token_row, int n_tokens, int hq,
                      int hkv, int d, int block_size, int num_pages, float scale, int window,
                      int* __restrict__ status) {
  __shared__ float q_s[WARPS][MAX_D];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * WARPS + warp;
  if (item >= (int64_t)n_tokens * hq) return;
  const int n = (int)(item / hq), h = (int)(item - (int64_t)n * hq);
  const int kvh = h / (hq / hkv);
  const int qpos = positions[n];
  const int* bt = block_table + (int64_t)token_row[n] * bt_stride;
  const T* qv = q + (int64_t)n * q_stride + (int64_t)h * d;
  for (int i = lane; i < d; i += 32) q_s[warp][i] = to_float(qv[i]);
  __syncwarp();

  const int kstart = window > 0 ? max(0, qpos - window + 1) : 0;
  const size_t head_elems = (size_t)block_size * d;
  const size_t page_elems = (size_t)2 * hkv * head_elems;
  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  for (int j0 = kstart & ~31; j0 <= qpos; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j >= kstart && j <= qpos;
    float s = -INFINITY;
    int64_t kbase = -1;
    if (valid) {
      const int page = bt[j / block_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, GLLM_STATUS_PAGE_RANGE);
      } else {
        kbase = (int64_t)((size_t)page * page_elems + (size_t)kvh * head_elems + (size_t)(j % block_size) * d);
        const T* kp = cache + kbase;
        float dot = 0.f;
        for (int i = 0; i < d; ++i) dot = fmaf(q_s[warp][i], to_float(kp[i]), dot);
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    // every block holds at least one key the token sees, so m_new is finite
    // (unless a page id was bad: then the whole block may be -inf; skip it)
    if (m_new == -INFINITY) continue;
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
    const int count = min(32, qpos - j0 + 1);
    const int64_t vhalf = (int64_t)hkv * head_elems;
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t kb = __shfl_sync(0xffffffffu, kbase, jj);
      if (kb < 0) continue;  // uniform across the warp
      const T* vp = cache + kb + vhalf;
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < d) acc[i] = fmaf(pj, to_float(vp[c]), acc[i]);
      }
    }
    m = m_new;
  }
  T* o = out + (int64_t)n * out_stride + (int64_t)h * d;
  const float inv_l = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < d) o[c] = from_float<T>(acc[i] * inv_l);
  }
}

template <typename T>
int attention_simt_launch(const T* q, int64_t q_stride, T* out, int64_t out_stride, const T* cache,
                          const int* block_table, int bt_stride, const int* positions, const int* token_row,
                          int n_tokens, int hq, int hkv, int d, int block_size, int num_pages, float scale,
                          int window, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || d > MAX_D || d % 16 || hq <= 0 || hkv <= 0 || hq % hkv) return (int)cudaErrorInvalidValue;
  const int64_t items = (int64_t)n_tokens * hq;
  const int64_t blocks = (items + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return gllm_launch(attention_simt_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, q, q_stride, out,
                     out_stride, cache, block_table, bt_stride, positions, token_row, n_tokens, hq, hkv, d,
                     block_size, num_pages, scale, window, status);
}
}  // namespace

GLLM_API int gllm_attention_simt_f32(const float* q, int64_t q_stride, float* out, int64_t out_stride,
                                     const float* cache, const int* block_table, int bt_stride,
                                     const int* positions, const int* token_row, int n_tokens, int hq, int hkv,
                                     int d, int block_size, int num_pages, float scale, int window, int* status,
                                     cudaStream_t stream) {
  return attention_simt_launch<float>(q, q_stride, out, out_stride, cache, block_table, bt_stride, positions,
                                      token_row, n_tokens, hq, hkv, d, block_size, num_pages, scale, window,
                                      status, stream);
}
GLLM_API int gllm_attention_simt_bf16(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                                      int64_t out_stride, const __nv_bfloat16* cache, const int* block_table,
                                      int bt_stride, const int* positions, const int* token_row, int n_tokens,
                                      int hq, int hkv, int d, int block_size, int num_pages, float scale,
                                      int window, int* status, cudaStream_t stream) {
  return attention_simt_launch<__nv_bfloat16>(q, q_stride, out, out_stride, cache, block_table, bt_stride,
                                              positions, token_row, n_tokens, hq, hkv, d, block_size, num_pages,
                                              scale, window, status, stream);
}
