// Attention kernels of the bf16 path over the paged cache.
//
// (1) Split-KV decode attention: one query token per request (the decoding
//     requests of a step).  It replaces the reference's per-step gather of the
//     whole padded context plus dense softmax(QK^T/sqrt(D) + bias)V
//     (gllm/model/layers/attention.py:165-173,
//     gllm/ops/attention/reference_attention.py:40-48).
//     The keys of a request are cut into chunks of CHUNK positions aligned to
//     multiples of CHUNK (so the cut depends on absolute positions only, never
//     on the batch or on how the prompt was fed); one CTA handles one
//     (chunk, kv head, request) for all query heads of that kv head, streams
//     the chunk's K and V pages once with 16-byte loads and keeps scores,
//     maximum, sum and the output accumulator in fp32.  A second kernel merges
//     the chunks in ascending order.  Decode is bandwidth-bound: the arithmetic
//     stays on the CUDA cores.
//
// Cache layer layout: [page][k|v][kv_head][block_size][head_dim].
#include "common.cuh"

namespace {

constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

// D: head size (16, 32, 64, 128).  GT: query heads of one kv head handled by a
// CTA (1, 2, 4, 8); a group larger than 8 takes several CTAs.
template <int D, int GT>
__global__ void __launch_bounds__(DEC_THREADS)
decode_split_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_stride,
                    const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                    const int* __restrict__ positions, const int* __restrict__ token_row,
                    const int* __restrict__ query_rows, float* __restrict__ part_o, float* __restrict__ part_ml,
                    int hq, int hkv, int block_size, int num_pages, int chunk, int num_chunks, float scale,
                    int window, int* __restrict__ status) {
  constexpr int DG = D / 8;        // lanes that share one cache row (8 dims each)
  constexpr int KG = 32 / DG;      // rows covered by one warp-wide 16-byte load
  __shared__ __align__(16) float q_s[GT][D];
  __shared__ float p_s[DEC_WARPS][GT][32];
  __shared__ float red_m[DEC_WARPS][GT], red_l[DEC_WARPS][GT];
  __shared__ __align__(16) float red_o[DEC_WARPS][GT][D];

  const int split = blockIdx.x;
  const int group = hq / hkv;
  const int tiles = (group + GT - 1) / GT;
  const int kvh = blockIdx.y / tiles, tile = blockIdx.y - kvh * tiles;
  const int r = blockIdx.z;
  const int n = query_rows ? query_rows[r] : r;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h0 = kvh * group + tile * GT;               // first query head of this CTA
  const int heads = min(GT, group - tile * GT);         // valid heads in the tile

  const int qpos = positions[n];
  const int kstart = window > 0 ? max(0, qpos - window + 1) : 0;
  const int c0 = max(split * chunk, kstart);
  const int c1 = min((split + 1) * chunk, qpos + 1);
  float* my_ml = part_ml + (((int64_t)r * hq + h0) * num_chunks + split) * 2;
  if (c0 >= c1) {                                       // nothing of this chunk is visible
    if (threadIdx.x < heads) {
      float* ml = my_ml + (int64_t)threadIdx.x * num_chunks * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    return;
  }
  const int* bt = block_table + (int64_t)token_row[n] * bt_stride;
  for (int i = threadIdx.x; i < GT * D; i += DEC_THREADS) {
    const int g = i / D, d = i - g * D;
    q_s[g][d] = g < heads ? __bfloat162float(q[(int64_t)n * q_stride + (int64_t)(h0 + g) * D + d]) * scale : 0.f;
  }
  __syncthreads();

  const int64_t head_elems = (int64_t)block_size * D;
  const int64_t page_elems = 2 * (int64_t)hkv * head_elems;
  const int64_t v_off = (int64_t)hkv * head_elems;

  float m[GT], l[GT], acc[GT][8];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }
  const int kg = lane / DG, dg = lane - kg * DG;
  // blocks of 32 keys aligned to absolute positions; warps take them round-robin
  const int first_block = (split * chunk) / 32;
  const int last_block = (c1 - 1) / 32;
  constexpr int V_LOADS = 32 / KG;               // 16-byte value loads per lane and block of 32 keys
  constexpr int V_BATCH = V_LOADS < 8 ? V_LOADS : 8;
  for (int blk = first_block + warp; blk <= last_block; blk += DEC_WARPS) {
    const int j0 = blk * 32;
    if (j0 + 31 < c0) continue;
    // ---- every lane looks its own key's page up once; all loads of the block are issued before any is used
    const int j = j0 + lane;
    const bool valid = j >= c0 && j < c1;
    int page = -1;
    if (valid) {
      page = bt[j / block_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, GLLM_STATUS_PAGE_RANGE);
        page = -1;
      }
    }
    uint4 kraw[DG];
    if (page >= 0) {
      const uint4* kp = reinterpret_cast<const uint4*>(
          cache + (int64_t)page * page_elems + (int64_t)kvh * head_elems + (int64_t)(j % block_size) * D);
#pragma unroll
      for (int c = 0; c < DG; ++c) kraw[c] = __ldg(kp + c);
    }
    uint4 vraw[V_BATCH];
    auto load_values = [&](int first) {
#pragma unroll
      for (int i = 0; i < V_BATCH; ++i) {
        const int jj = (first + i) * KG + kg;
        const int pg = __shfl_sync(0xffffffffu, page, jj);
        const int key = j0 + jj;
        vraw[i] = make_uint4(0u, 0u, 0u, 0u);
        if (pg >= 0)
          vraw[i] = __ldg(reinterpret_cast<const uint4*>(cache + (int64_t)pg * page_elems + v_off +
                                                         (int64_t)kvh * head_elems +
                                                         (int64_t)(key % block_size) * D) + dg);
      }
    };
    load_values(0);
    // ---- scores: lane <-> key j0 + lane
    float s[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) s[g] = 0.f;
    if (page >= 0) {
#pragma unroll
      for (int c = 0; c < DG; ++c) {
        float kf[8];
        unpack8(kraw[c], kf);
#pragma unroll
        for (int g = 0; g < GT; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][c * 8 + 4]);
          s[g] = fmaf(qa.x, kf[0], s[g]); s[g] = fmaf(qa.y, kf[1], s[g]);
          s[g] = fmaf(qa.z, kf[2], s[g]); s[g] = fmaf(qa.w, kf[3], s[g]);
          s[g] = fmaf(qb.x, kf[4], s[g]); s[g] = fmaf(qb.y, kf[5], s[g]);
          s[g] = fmaf(qb.z, kf[6], s[g]); s[g] = fmaf(qb.w, kf[7], s[g]);
        }
      }
    }
    const bool use = page >= 0;
    float corr[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float sg = use ? s[g] : -INFINITY;
      const float m_new = fmaxf(m[g], warp_max(sg));
      const float p = (m_new == -INFINITY || !use) ? 0.f : __expf(sg - m_new);
      corr[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - m_new);
      l[g] = l[g] * corr[g] + warp_sum(p);
      m[g] = m_new;
      p_s[warp][g][lane] = p;
    }
    __syncwarp();
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] *= corr[g];
    // ---- values: each 16-byte load covers KG rows; lane (kg, dg) owns 8 dims of its rows
#pragma unroll
    for (int first = 0; first < V_LOADS; first += V_BATCH) {
      if (first > 0) load_values(first);
#pragma unroll
      for (int i = 0; i < V_BATCH; ++i) {
        const int jj = (first + i) * KG + kg;
        float vf[8];
        unpack8(vraw[i], vf);
#pragma unroll
        for (int g = 0; g < GT; ++g) {
          const float p = p_s[warp][g][jj];      // 0 for keys outside the chunk
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(p, vf[e], acc[g][e]);
        }
      }
    }
    __syncwarp();
  }
  // ---- fold the key groups of a warp, then the warps of the CTA
#pragma unroll
  for (int g = 0; g < GT; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = acc[g][e];
#pragma unroll
      for (int o = DG; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[g][e] = v;
    }
  if (kg == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) red_o[warp][g][dg * 8 + e] = acc[g][e];
  }
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      red_m[warp][g] = m[g];
      red_l[warp][g] = l[g];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < heads * D; i += DEC_THREADS) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, red_m[w][g]);
    float o = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float f = red_m[w][g] == -INFINITY ? 0.f : __expf(red_m[w][g] - mm);
      o += red_o[w][g][d] * f;
      ll += red_l[w][g] * f;
    }
    part_o[(((int64_t)r * hq + h0 + g) * num_chunks + split) * D + d] = o;
    if (d == 0) {
      float* ml = my_ml + (int64_t)g * num_chunks * 2;
      ml[0] = mm;
      ml[1] = ll;
    }
  }
}

// Merges the chunks of one (request, query head) in ascending order.
template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ query_rows, __nv_bfloat16* __restrict__ out,
                                    int64_t out_stride, int hq, int num_chunks) {
  const int r = blockIdx.y, h = blockIdx.x, d = threadIdx.x;
  const int n = query_rows ? query_rows[r] : r;
  const float* ml = part_ml + ((int64_t)r * hq + h) * num_chunks * 2;
  const float* po = part_o + ((int64_t)r * hq + h) * num_chunks * D;
  float mm = -INFINITY;
  for (int s = 0; s < num_chunks; ++s) mm = fmaxf(mm, ml[2 * s]);
  float o = 0.f, l = 0.f;
  for (int s = 0; s < num_chunks; ++s) {
    const float ms = ml[2 * s];
    if (ms == -INFINITY) continue;
    const float f = __expf(ms - mm);
    o += po[(int64_t)s * D + d] * f;
    l += ml[2 * s + 1] * f;
  }
  out[(int64_t)n * out_stride + (int64_t)h * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
}

template <int D, int GT>
int decode_launch(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out, int64_t out_stride,
                  const __nv_bfloat16* cache, const int* block_table, int bt_stride, const int* positions,
                  const int* token_row, const int* query_rows, int num_queries, float* part_o, float* part_ml,
                  int hq, int hkv, int block_size, int num_pages, int chunk, int num_chunks, float scale,
                  int window, int* status, cudaStream_t stream) {
  const int group = hq / hkv;
  const int tiles = (group + GT - 1) / GT;
  dim3 grid(num_chunks, hkv * tiles, num_queries);
  decode_split_kernel<D, GT><<<grid, DEC_THREADS, 0, stream>>>(
      q, q_stride, cache, block_table, bt_stride, positions, token_row, query_rows, part_o, part_ml, hq, hkv,
      block_size, num_pages, chunk, num_chunks, scale, window, status);
  int e = gllm_launch_result();
  if (e) return e;
  decode_merge_kernel<D><<<dim3(hq, num_queries), D, 0, stream>>>(part_o, part_ml, query_rows, out, out_stride,
                                                                    hq, num_chunks);
  return gllm_launch_result();
}

template <int D>
int decode_dispatch_group(int group, const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                          int64_t out_stride, const __nv_bfloat16* cache, const int* block_table, int bt_stride,
                          const int* positions, const int* token_row, const int* query_rows, int num_queries,
                          float* part_o, float* part_ml, int hq, int hkv, int block_size, int num_pages,
                          int chunk, int num_chunks, float scale, int window, int* status, cudaStream_t stream) {
#define GLLM_DEC(GT)                                                                                           \
  return decode_launch<D, GT>(q, q_stride, out, out_stride, cache, block_table, bt_stride, positions,          \
                              token_row, query_rows, num_queries, part_o, part_ml, hq, hkv, block_size,        \
                              num_pages, chunk, num_chunks, scale, window, status, stream)
  if (group == 1) GLLM_DEC(1);
  if (group == 2) GLLM_DEC(2);
  if (group <= 4) GLLM_DEC(4);
  GLLM_DEC(8);
#undef GLLM_DEC
}
}  // namespace

// Scratch the caller provides: part_o  [num_queries * hq * num_chunks * d] floats,
//                              part_ml [num_queries * hq * num_chunks * 2] floats.
// `chunk` must be a multiple of 32; num_chunks = ceil(longest sequence / chunk).
GLLM_API int gllm_attention_decode_bf16(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                                        int64_t out_stride, const __nv_bfloat16* cache, const int* block_table,
                                        int bt_stride, const int* positions, const int* token_row,
                                        const int* query_rows, int num_queries, float* part_o, float* part_ml,
                                        int hq, int hkv, int d, int block_size, int num_pages, int chunk,
                                        int num_chunks, float scale, int window, int* status,
                                        cudaStream_t stream) {
  if (num_queries <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || hq % hkv || chunk <= 0 || chunk % 32 || num_chunks <= 0 || num_queries > 65535 ||
      (q_stride % 8) || ((block_size * d) % 8))
    return (int)cudaErrorInvalidValue;
  const int group = hq / hkv;
#define GLLM_DEC_D(DD)                                                                                          \
  return decode_dispatch_group<DD>(group, q, q_stride, out, out_stride, cache, block_table, bt_stride,          \
                                   positions, token_row, query_rows, num_queries, part_o, part_ml, hq, hkv,     \
                                   block_size, num_pages, chunk, num_chunks, scale, window, status, stream)
  switch (d) {
    case 16: GLLM_DEC_D(16);
    case 32: GLLM_DEC_D(32);
    case 64: GLLM_DEC_D(64);
    case 128: GLLM_DEC_D(128);
    default: return (int)cudaErrorInvalidValue;
  }
#undef GLLM_DEC_D
}

// Head sizes the decode kernel takes (others run the general kernel).
GLLM_API int gllm_attention_decode_supports(int d) { return d == 16 || d == 32 || d == 64 || d == 128; }
