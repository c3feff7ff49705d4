// Split-KV decode attention of the bf16 path: one query token per request (the
// decoding requests of a step) over the paged cache.  It replaces the
// reference's per-step gather of the whole padded context plus dense
// softmax(QK^T/sqrt(D) + bias)V (gllm/model/layers/attention.py:165-173,
// gllm/ops/attention/reference_attention.py:40-48).
//
// A request's keys are cut into chunks of W*32 positions aligned to multiples
// of the chunk (the cut depends on absolute positions only, never on the batch
// or on how the prompt was fed).  One CTA owns one (chunk, kv head, request):
// each of its W warps copies 32 keys and 32 values of the chunk into shared
// memory with cp.async (16-byte pieces, everything in flight at once; decode
// is bound by this traffic) and runs Q K^T and P V for all query heads of the
// kv head on the tensor cores (mma.sync m16n8k16, the heads are the 16 rows of
// the tile; bf16 in, fp32 accumulate).  Scores, maximum, sum and output are
// fp32.  The warps' partial results are folded in shared memory and written
// per chunk; a second kernel merges the chunks in ascending order.
//
// Cache layer layout: [page][k|v][kv_head][block_size][head_dim].
#include "mma_utils.cuh"

namespace {
constexpr int TILE = 32;     // keys per warp
constexpr int ROWS = 16;     // query heads per CTA (rows of the MMA tile)

template <int D>
struct DecodeShape {
  static constexpr int W = D <= 64 ? 8 : 4;   // warps per CTA
  static constexpr int CHUNK = W * TILE;
  static constexpr int TILE_BYTES = TILE * D * 2;
  // per warp K and V tiles, then the Q tile
  static constexpr int SMEM = W * 2 * TILE_BYTES + ROWS * D * 2;
};

template <int D>
__global__ void __launch_bounds__(DecodeShape<D>::W * 32)
decode_split_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_stride,
                    const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                    const int* __restrict__ positions, const int* __restrict__ token_row,
                    float* __restrict__ part_o, float* __restrict__ part_ml, int hq, int hkv, int block_size,
                    int num_pages, int num_chunks, float scale_log2, int window, int* __restrict__ status) {
  using S = DecodeShape<D>;
  constexpr int C = D / 8, W = S::W;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* k_sm = smem_raw + warp * 2 * S::TILE_BYTES;
  unsigned char* v_sm = k_sm + S::TILE_BYTES;
  unsigned char* q_sm = smem_raw + W * 2 * S::TILE_BYTES;
  __shared__ float red_m[W][ROWS], red_l[W][ROWS];

  pdl_trigger();
  // chunk-major: all (request, kv head) pairs of chunk 0 come first, and the chunks past every request's end (the
  // grid is sized for the longest sequence of the step's bucket) come last: 0.913 -> 0.900 ms per decode step at
  // batch 8, 0.780 -> 0.765 at batch 1, against the chunks of one request side by side
  const int split = blockIdx.y;
  const int group = hq / hkv;
  const int head_tiles = (group + ROWS - 1) / ROWS;
  const int n = (int)blockIdx.x / (hkv * head_tiles), by = (int)blockIdx.x - n * (hkv * head_tiles);
  const int kvh = by / head_tiles, tile_idx = by - kvh * head_tiles;
  const int h0 = kvh * group + tile_idx * ROWS;
  const int heads = min(ROWS, group - tile_idx * ROWS);

  const int qpos = positions[n];
  const int kstart = window > 0 ? max(0, qpos - window + 1) : 0;
  const int c0 = max(split * S::CHUNK, kstart);
  const int c1 = min((split + 1) * S::CHUNK, qpos + 1);
  float* my_ml = part_ml + (((int64_t)n * hq + h0) * num_chunks + split) * 2;
  if (c0 >= c1) {                                       // nothing of this chunk is visible
    pdl_wait();
    if (threadIdx.x < heads) {
      float* ml = my_ml + (int64_t)threadIdx.x * num_chunks * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    return;
  }
  const int* bt = block_table + (int64_t)token_row[n] * bt_stride;
  const int64_t head_elems = (int64_t)block_size * D;
  const int64_t page_elems = 2 * (int64_t)hkv * head_elems;
  const int64_t v_off = (int64_t)hkv * head_elems;

  // ---- this warp's keys and values: all copies are issued before anything waits.
  // The positions, the block table and every cached row but the newest (key == qpos, written by the
  // kernel just before this one) are older than the step's kernels: they are requested before the
  // dependency wait, so the cache streams in while the kernels before this one still run.
  const int k0 = split * S::CHUNK + warp * TILE;
  const bool warp_has_keys = k0 < c1 && k0 + TILE > c0;
  // Every lane first resolves its share of the tile's rows (page lookup, offset in the page) and leaves
  // the rows' element offsets in shared memory, so the copy loop below has no dependent loads.
  __shared__ int64_t row_base[W][TILE];
  if (warp_has_keys) {
#pragma unroll
    for (int half = 0; half < TILE / 32; ++half) {
      const int row = lane + 32 * half;
      const int key = k0 + row;
      int64_t base = -1;
      if (key >= c0 && key < c1) {
        const int blk = key / block_size;
        const int page = bt[blk];
        if (page < 0 || page >= num_pages) atomicOr(status, GLLM_STATUS_PAGE_RANGE);
        else base = (int64_t)page * page_elems + (int64_t)kvh * head_elems + (int64_t)(key - blk * block_size) * D;
      }
      row_base[warp][row] = base;
    }
    __syncwarp();
#pragma unroll
    for (int it = 0; it < TILE * C / 32; ++it) {
      const int idx = it * 32 + lane;
      const int row = idx / C, piece = idx - row * C;
      const int64_t base = row_base[warp][row];
      const bool ok = base >= 0;
      if (k0 + row == qpos) continue;                   // the newest row: after the wait
      const __nv_bfloat16* src = cache + (ok ? base : 0) + piece * 8;
      const int off = (row * C + swizzle<C>(row, piece)) * 16;
      cp_async16(smem_u32(k_sm + off), src, ok);
      cp_async16(smem_u32(v_sm + off), src + v_off, ok);
    }
  }
  pdl_wait();
  if (warp_has_keys && qpos >= k0 && qpos < k0 + TILE && lane < C) {
    const int row = qpos - k0, piece = lane;
    const int64_t base = row_base[warp][row];
    const bool ok = base >= 0;
    const __nv_bfloat16* src = cache + (ok ? base : 0) + piece * 8;
    const int off = (row * C + swizzle<C>(row, piece)) * 16;
    cp_async16(smem_u32(k_sm + off), src, ok);
    cp_async16(smem_u32(v_sm + off), src + v_off, ok);
  }
  // ---- the query heads of this kv head: row i <-> head h0 + i (rows past the group are zeros)
  for (int idx = threadIdx.x; idx < ROWS * C; idx += W * 32) {
    const int row = idx / C, piece = idx - row * C;
    const bool ok = row < heads;
    const __nv_bfloat16* src = q + (int64_t)n * q_stride + (int64_t)(h0 + (ok ? row : 0)) * D + piece * 8;
    cp_async16(smem_u32(q_sm + (row * C + swizzle<C>(row, piece)) * 16), src, ok);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int g8 = lane >> 2, t4 = lane & 3;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int nd = 0; nd < D / 8; ++nd)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nd][e] = 0.f;

  if (warp_has_keys) {
    // ---- S = Q K^T (16 heads x 64 keys)
    float s[TILE / 8][4];
#pragma unroll
    for (int nt = 0; nt < TILE / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int mat = lane >> 3, rl = lane & 7;
      uint32_t qf[4];
      {
        const int row = (mat & 1) * 8 + rl, piece = 2 * ks + (mat >> 1);
        ldmatrix_x4(qf, smem_u32(q_sm + (row * C + swizzle<C>(row, piece)) * 16));
      }
#pragma unroll
      for (int np = 0; np < TILE / 16; ++np) {
        const int row = np * 16 + (mat >> 1) * 8 + rl, piece = 2 * ks + (mat & 1);
        uint32_t b[4];
        ldmatrix_x4(b, smem_u32(k_sm + (row * C + swizzle<C>(row, piece)) * 16));
        mma_bf16(s[2 * np], qf, b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf, b[2], b[3]);
      }
    }
    // ---- mask, scale, softmax over this warp's keys (rows g8 and g8 + 8)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < TILE / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + nt * 8 + 2 * t4 + (e & 1);
        const float v = (key >= c0 && key < c1) ? s[nt][e] * scale_log2 : -INFINITY;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      m[i] = mx[i];                                   // finite: the warp has at least one visible key
    }
#pragma unroll
    for (int nt = 0; nt < TILE / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = fast_exp2(s[nt][e] - m[e >> 1]);
        s[nt][e] = p;
        l[e >> 1] += p;
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
      l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    // ---- O = P V
#pragma unroll
    for (int kk = 0; kk < TILE / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int nd2 = 0; nd2 < D / 16; ++nd2) {
        const int mat = lane >> 3, rl = lane & 7;
        const int row = kk * 16 + (mat & 1) * 8 + rl, piece = 2 * nd2 + (mat >> 1);
        uint32_t b[4];
        ldmatrix_x4_trans(b, smem_u32(v_sm + (row * C + swizzle<C>(row, piece)) * 16));
        mma_bf16(o[2 * nd2], a, b[0], b[1]);
        mma_bf16(o[2 * nd2 + 1], a, b[2], b[3]);
      }
    }
  }
  // ---- fold the warps: every warp leaves (m, l, O) in shared memory (its own K tile's space)
  __syncthreads();
  float* red_o = reinterpret_cast<float*>(smem_raw) + (size_t)warp * ROWS * D;   // W*16*D*4 <= W*2*TILE_BYTES
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = g8 + 8 * i;
    if (t4 == 0) {
      red_m[warp][row] = m[i];
      red_l[warp][row] = l[i];
    }
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd) {
      red_o[row * D + nd * 8 + 2 * t4] = o[nd][2 * i];
      red_o[row * D + nd * 8 + 2 * t4 + 1] = o[nd][2 * i + 1];
    }
  }
  __syncthreads();
  const float* all_o = reinterpret_cast<const float*>(smem_raw);
  for (int idx = threadIdx.x; idx < heads * D; idx += W * 32) {
    const int row = idx / D, d = idx - row * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < W; ++w) mm = fmaxf(mm, red_m[w][row]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float f = red_m[w][row] == -INFINITY ? 0.f : fast_exp2(red_m[w][row] - mm);
      acc += all_o[((size_t)w * ROWS + row) * D + d] * f;
      ll += red_l[w][row] * f;
    }
    part_o[(((int64_t)n * hq + h0 + row) * num_chunks + split) * D + d] = acc;
    if (d == 0) {
      float* ml = my_ml + (int64_t)row * num_chunks * 2;
      ml[0] = mm;                                       // in units of log2
      ml[1] = ll;
    }
  }
}

// Merges the partial results of one (request, query head) in ascending order, in one pass (running
// maximum, sum and output).  Only the chunks that can hold a visible key are read: those of the keys
// kstart .. qpos, `per_span` consecutive chunks for every `span_keys` keys.
template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                     __nv_bfloat16* __restrict__ out, int64_t out_stride, int hq, int num_chunks,
                     const int* __restrict__ positions, int window, int span_keys, int per_span) {
  pdl_trigger();
  const int n = blockIdx.y, h = blockIdx.x, d = threadIdx.x;
  const int qpos = positions[n];                          // a step input: older than the step's kernels
  const int kstart = window > 0 ? max(0, qpos - window + 1) : 0;
  const int first = (kstart / span_keys) * per_span;
  const int last = min(num_chunks, (qpos / span_keys + 1) * per_span);
  pdl_wait();
  const float* ml = part_ml + ((int64_t)n * hq + h) * num_chunks * 2;
  const float* po = part_o + ((int64_t)n * hq + h) * num_chunks * D;
  float mm = -INFINITY, o = 0.f, l = 0.f;
  constexpr int B = 16;                                   // chunks whose loads are in flight together
  for (int s0 = first; s0 < last; s0 += B) {
    float ms[B], ls[B], os[B];
#pragma unroll
    for (int i = 0; i < B; ++i) {
      const bool in = s0 + i < last;
      const float2 v = in ? __ldcg(reinterpret_cast<const float2*>(ml) + s0 + i) : make_float2(-INFINITY, 0.f);
      ms[i] = v.x;
      ls[i] = v.y;
      os[i] = in ? __ldcg(po + (int64_t)(s0 + i) * D + d) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < B; ++i) {
      if (ms[i] == -INFINITY) continue;
      const float m_new = fmaxf(mm, ms[i]);
      const float f_old = fast_exp2(mm - m_new), f_new = fast_exp2(ms[i] - m_new);   // f_old = 0 at the first chunk
      o = o * f_old + os[i] * f_new;
      l = l * f_old + ls[i] * f_new;
      mm = m_new;
    }
  }
  out[(int64_t)n * out_stride + (int64_t)h * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
}

template <int D>
int decode_launch(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out, int64_t out_stride,
                  const __nv_bfloat16* cache, const int* block_table, int bt_stride, const int* positions,
                  const int* token_row, int num_queries, float* part_o, float* part_ml, int hq, int hkv,
                  int block_size, int num_pages, int num_chunks, float scale, int window, int* status,
                  cudaStream_t stream) {
  using S = DecodeShape<D>;
  const int group = hq / hkv;
  const int head_tiles = (group + ROWS - 1) / ROWS;
  if (S::SMEM > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_split_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((unsigned)(hkv * head_tiles * num_queries), num_chunks);
  int e = gllm_launch(decode_split_kernel<D>, grid, dim3(S::W * 32), (size_t)S::SMEM, stream, q, q_stride, cache,
                      block_table, bt_stride, positions, token_row, part_o, part_ml, hq, hkv, block_size, num_pages,
                      num_chunks, scale * 1.4426950408889634f, window, status);
  if (e) return e;
  return gllm_launch(decode_merge_kernel<D>, dim3(hq, num_queries), dim3(D), 0, stream, part_o, part_ml, out,
                     out_stride, hq, num_chunks, positions, window, S::CHUNK, 1);
}
}  // namespace

// Keys per chunk for head size d (0: the head size is not taken).
GLLM_API int gllm_attention_decode_chunk(int d) {
  switch (d) {
    case 32: return DecodeShape<32>::CHUNK;
    case 64: return DecodeShape<64>::CHUNK;
    case 128: return DecodeShape<128>::CHUNK;
    default: return 0;
  }
}

// Query token i of the call is row i of q / out / positions / token_row.
// Scratch the caller provides: part_o  [num_queries * hq * num_chunks * d] floats,
//                              part_ml [num_queries * hq * num_chunks * 2] floats,
// num_chunks = ceil(longest sequence / gllm_attention_decode_chunk(d)) (or more).
GLLM_API int gllm_attention_decode_bf16(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                                        int64_t out_stride, const __nv_bfloat16* cache, const int* block_table,
                                        int bt_stride, const int* positions, const int* token_row,
                                        int num_queries, float* part_o, float* part_ml, int hq, int hkv, int d,
                                        int block_size, int num_pages, int num_chunks, float scale, int window,
                                        int* status, cudaStream_t stream) {
  if (num_queries <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || hq % hkv || num_chunks <= 0 || num_chunks > 65535 || num_queries > 65535 || (q_stride % 8) ||
      ((block_size * d) % 8))
    return (int)cudaErrorInvalidValue;
#define GLLM_DEC_D(DD)                                                                                         \
  return decode_launch<DD>(q, q_stride, out, out_stride, cache, block_table, bt_stride, positions, token_row,  \
                           num_queries, part_o, part_ml, hq, hkv, block_size, num_pages, num_chunks, scale,    \
                           window, status, stream)
  switch (d) {
    case 32: GLLM_DEC_D(32);
    case 64: GLLM_DEC_D(64);
    case 128: GLLM_DEC_D(128);
    default: return (int)cudaErrorInvalidValue;
  }
#undef GLLM_DEC_D
}

// ---------------------------------------------------------------------------
// The same attention for callers that cannot allocate (see attention_decode_noalloc.h).
#include "attention_decode_noalloc.h"

namespace {
// Scratch for the per-chunk partial results, part of the library's device image.
static __device__ __align__(256) float g_decode_noalloc_scratch[GLLM_DECODE_NOALLOC_MAX_FLOATS];
constexpr int NOALLOC_MAX_DEVICES = 64;
// Device address of the array on each device, looked up on the first call there.  In host
// code the array's name is only a handle for the runtime, not an address a kernel can use.
float* g_decode_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
}  // namespace

GLLM_API int gllm_attention_decode_bf16_noalloc(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                                                int64_t out_stride, const __nv_bfloat16* cache,
                                                const int* block_table, int bt_stride, const int* positions,
                                                const int* token_row, int num_queries, int hq, int hkv, int d,
                                                int block_size, int num_pages, int num_chunks, float scale,
                                                int window, int* status, cudaStream_t stream) {
  if (num_queries <= 0) return 0;
  // Bound every factor before multiplying, and test the limit by division: the product of
  // unchecked arguments could wrap around and pass.
  if ((d != 32 && d != 64 && d != 128) || hq <= 0 || hkv <= 0 || hq % hkv || num_chunks <= 0 ||
      num_queries > 65535)
    return (int)cudaErrorInvalidValue;
  const int64_t per_chunk = (int64_t)num_queries * hq * (d + 2);          // <= 65535 * 2^31 * 130 < 2^63
  if ((int64_t)num_chunks > (int64_t)GLLM_DECODE_NOALLOC_MAX_FLOATS / per_chunk) return (int)cudaErrorInvalidValue;
  const int64_t o_floats = (int64_t)num_queries * hq * num_chunks * d;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
  // The cache is written without a lock: two threads that race here both look the address up and
  // both store the same value.
  if (!g_decode_noalloc_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_decode_noalloc_ptr[dev] = p;
  }
  float* part_o = g_decode_noalloc_ptr[dev];
  float* part_ml = part_o + o_floats;
  return gllm_attention_decode_bf16(q, q_stride, out, out_stride, cache, block_table, bt_stride, positions,
                                    token_row, num_queries, part_o, part_ml, hq, hkv, d, block_size, num_pages,
                                    num_chunks, scale, window, status, stream);
}
