// Causal prefill attention of the bf16 path over the paged cache: portions of
// prompts (any length, cut anywhere) attend over everything their request has
// cached so far, this step's own tokens included, through the block table.
//
// It replaces the reference's gather of the padded context plus dense
// softmax(QK^T/sqrt(D) + bias)V (gllm/model/layers/attention.py:165-173,
// gllm/ops/attention/reference_attention.py:40-48) and its unused Triton
// kernel (gllm/ops/attention/flash_attention.py:7-152): no bias tensor, no
// score tensor, tiles above the diagonal are never visited.
//
// One CTA (4 warps) owns 64 rows = (64 / G') query tokens x G' query heads that
// share one kv head (G' = heads per kv head when that divides 64, else 1), so
// a K/V tile brought into shared memory serves the whole group.  K/V tiles of
// 64 keys are fetched page by page with cp.async (16-byte pieces, two stages),
// Q K^T and P V run on the tensor cores (mma.sync m16n8k16, bf16 in, fp32
// accumulate), the running maximum, sum and output stay in fp32 registers.
// Keys are visited in ascending tiles aligned to multiples of 64 positions.
#include "mma_utils.cuh"

namespace {
constexpr int BM = 64, BN = 64, PF_THREADS = 128;  // 4 warps, 16 rows each

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
prefill_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_stride, __nv_bfloat16* __restrict__ out,
               int64_t out_stride, const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table,
               int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
               const int* __restrict__ slots, int hq, int hkv, int gp, int block_size, int num_pages,
               float scale_log2, int window, int* __restrict__ status) {
  constexpr int C = D / 8;                 // 16-byte pieces per row
  constexpr int TILE_BYTES = BN * D * 2;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* q_sm = smem_raw;                       // [BM][D]
  unsigned char* kv_sm = smem_raw + BM * D * 2;         // [2 stages][K | V][BN][D]

  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.z;
  const int group = hq / hkv;
  const int tiles_per_kv = group / gp;                  // CTAs that share a kv head
  const int kvh = blockIdx.y / tiles_per_kv;
  const int h0 = kvh * group + (blockIdx.y - kvh * tiles_per_kv) * gp;  // first query head of the CTA
  const int qt = BM / gp;                               // query tokens per CTA
  const int tok_begin = cu_q[r], q_len = cu_q[r + 1] - tok_begin;
  const int n_qtiles = (q_len + qt - 1) / qt;
  if ((int)blockIdx.x >= n_qtiles) return;
  const int qtile = n_qtiles - 1 - blockIdx.x;          // longest rows first
  const int t0 = qtile * qt;
  const int t_count = min(qt, q_len - t0);
  const int ctx = ctx_lens[r];
  const int* bt = block_table + (int64_t)slots[r] * bt_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;

  const int pos_first = ctx + t0, pos_last = ctx + t0 + t_count - 1;
  const int kv_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int tile_first = kv_lo / BN, tile_last = pos_last / BN;

  const int64_t head_elems = (int64_t)block_size * D;
  const int64_t page_elems = 2 * (int64_t)hkv * head_elems;
  const int64_t v_off = (int64_t)hkv * head_elems;

  // ---- Q tile -> shared memory (row rr <-> token t0 + rr / gp, head h0 + rr % gp)
  for (int idx = threadIdx.x; idx < BM * C; idx += PF_THREADS) {
    const int rr = idx / C, piece = idx - rr * C;
    const int tl = rr / gp, g = rr - tl * gp;
    const bool ok = tl < t_count;
    const __nv_bfloat16* src = q + (int64_t)(tok_begin + t0 + (ok ? tl : 0)) * q_stride + (int64_t)(h0 + g) * D + piece * 8;
    cp_async16(smem_u32(q_sm + (rr * C + swizzle<C>(rr, piece)) * 16), src, ok);
  }
  auto load_kv = [&](int tile, int stage) {
    unsigned char* k_dst = kv_sm + stage * 2 * TILE_BYTES;
    unsigned char* v_dst = k_dst + TILE_BYTES;
    for (int idx = threadIdx.x; idx < BN * C; idx += PF_THREADS) {
      const int row = idx / C, piece = idx - row * C;
      const int key = tile * BN + row;
      bool ok = key >= kv_lo && key <= pos_last;
      int page = 0;
      if (ok) {
        page = bt[key / block_size];
        if (page < 0 || page >= num_pages) {
          atomicOr(status, GLLM_STATUS_PAGE_RANGE);
          ok = false;
          page = 0;
        }
      }
      const __nv_bfloat16* src = cache + (int64_t)page * page_elems + (int64_t)kvh * head_elems +
                                 (int64_t)(key % block_size) * D + piece * 8;
      const int off = (row * C + swizzle<C>(row, piece)) * 16;
      cp_async16(smem_u32(k_dst + off), ok ? src : cache, ok);
      cp_async16(smem_u32(v_dst + off), ok ? src + v_off : cache, ok);
    }
  };
  load_kv(tile_first, 0);
  cp_async_commit();

  // per-thread rows: rr0 = warp*16 + g8 and rr0 + 8
  int qpos[2];
  bool row_ok[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = warp * 16 + g8 + 8 * i;
    const int tl = rr / gp;
    row_ok[i] = tl < t_count;
    qpos[i] = pos_first + tl;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int nd = 0; nd < D / 8; ++nd)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nd][e] = 0.f;
  uint32_t qf[D / 16][4];

  for (int tile = tile_first; tile <= tile_last; ++tile) {
    const int stage = (tile - tile_first) & 1;
    if (tile < tile_last) {
      load_kv(tile + 1, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (tile == tile_first) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int mat = lane >> 3, rl = lane & 7;
        const int row = warp * 16 + (mat & 1) * 8 + rl;
        const int piece = 2 * ks + (mat >> 1);
        ldmatrix_x4(qf[ks], smem_u32(q_sm + (row * C + swizzle<C>(row, piece)) * 16));
      }
    }
    const unsigned char* k_sm = kv_sm + stage * 2 * TILE_BYTES;
    const unsigned char* v_sm = k_sm + TILE_BYTES;
    const int kv0 = tile * BN;

    // ---- S = Q K^T for 64 keys
    float s[BN / 8][4];
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        const int mat = lane >> 3, rl = lane & 7;
        const int row = np * 16 + (mat >> 1) * 8 + rl;
        const int piece = 2 * ks + (mat & 1);
        uint32_t b[4];
        ldmatrix_x4(b, smem_u32(k_sm + (row * C + swizzle<C>(row, piece)) * 16));
        mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
      }
    }
    // ---- mask, online softmax (rows g8 and g8 + 8 of the warp's 16).  The maximum is kept in raw
    // score units; the scale enters through the exponent's FMA: p = 2^(s*c - m*c), c = scale*log2(e)
    const bool need_mask = (kv0 + BN - 1 > pos_first) || (window > 0) || (t_count < qt);
    float mx[2] = {-INFINITY, -INFINITY};
    if (need_mask) {
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const int key = kv0 + nt * 8 + 2 * t4 + (e & 1);
          const bool hidden = !row_ok[i] || key > qpos[i] || (window > 0 && key <= qpos[i] - window);
          if (hidden) s[nt][e] = -INFINITY;
        }
    }
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
    float corr[2], neg_mc[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float m_new = fmaxf(m[i], mx[i]);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      corr[i] = m[i] == -INFINITY ? 0.f : fast_exp2((m[i] - m_use) * scale_log2);
      neg_mc[i] = -m_use * scale_log2;
      m[i] = m_new;
    }
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const float p = fast_exp2(fmaf(s[nt][e], scale_log2, neg_mc[i]));
        s[nt][e] = p;
        l[i] = (e & 1) || nt ? l[i] + p : fmaf(l[i], corr[i], p);
      }
    // the output only needs rescaling when some row's maximum moved (rare after the first tiles)
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
      for (int nd = 0; nd < D / 8; ++nd) {
        o[nd][0] *= corr[0]; o[nd][1] *= corr[0];
        o[nd][2] *= corr[1]; o[nd][3] *= corr[1];
      }
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int nd2 = 0; nd2 < D / 16; ++nd2) {
        const int mat = lane >> 3, rl = lane & 7;
        const int row = kk * 16 + (mat & 1) * 8 + rl;
        const int piece = 2 * nd2 + (mat >> 1);
        uint32_t b[4];
        ldmatrix_x4_trans(b, smem_u32(v_sm + (row * C + swizzle<C>(row, piece)) * 16));
        mma_bf16(o[2 * nd2], a, b[0], b[1]);
        mma_bf16(o[2 * nd2 + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();   // everyone is done with this stage before it is filled again
  }
  // ---- normalise and store
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!row_ok[i]) continue;
    const int rr = warp * 16 + g8 + 8 * i;
    const int tl = rr / gp, g = rr - tl * gp;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
    __nv_bfloat16* dst = out + (int64_t)(tok_begin + t0 + tl) * out_stride + (int64_t)(h0 + g) * D;
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(o[nd][2 * i] * inv, o[nd][2 * i + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(dst + nd * 8 + 2 * t4) = v;
    }
  }
}

template <int D>
int prefill_launch(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out, int64_t out_stride,
                   const __nv_bfloat16* cache, const int* block_table, int bt_stride, const int* cu_q,
                   const int* ctx_lens, const int* slots, int num_requests, int max_q_len, int hq, int hkv,
                   int block_size, int num_pages, float scale, int window, int* status, cudaStream_t stream) {
  const int group = hq / hkv;
  const int gp = (group <= BM && BM % group == 0) ? group : 1;
  const int qt = BM / gp;
  const size_t smem = (size_t)BM * D * 2 + 4 * (size_t)BN * D * 2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((max_q_len + qt - 1) / qt, hkv * (group / gp), num_requests);
  const float scale_log2 = scale * 1.4426950408889634f;
  return gllm_launch(prefill_kernel<D>, grid, dim3(PF_THREADS), smem, stream, q, q_stride, out, out_stride, cache,
                     block_table, bt_stride, cu_q, ctx_lens, slots, hq, hkv, gp, block_size, num_pages, scale_log2,
                     window, status);
}
}  // namespace

// Requests 0 .. num_requests-1 of the flat batch: tokens cu_q[r] .. cu_q[r+1]-1 at
// positions ctx_lens[r] .., block-table row slots[r].  Their keys and values are
// already in the cache.  max_q_len >= every request's token count.
GLLM_API int gllm_attention_prefill_bf16(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                                         int64_t out_stride, const __nv_bfloat16* cache, const int* block_table,
                                         int bt_stride, const int* cu_q, const int* ctx_lens, const int* slots,
                                         int num_requests, int max_q_len, int hq, int hkv, int d, int block_size,
                                         int num_pages, float scale, int window, int* status,
                                         cudaStream_t stream) {
  if (num_requests <= 0 || max_q_len <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || hq % hkv || num_requests > 65535 || (q_stride % 8) || (out_stride % 2) ||
      ((block_size * d) % 8))
    return (int)cudaErrorInvalidValue;
#define GLLM_PF(DD)                                                                                              \
  return prefill_launch<DD>(q, q_stride, out, out_stride, cache, block_table, bt_stride, cu_q, ctx_lens, slots,  \
                            num_requests, max_q_len, hq, hkv, block_size, num_pages, scale, window, status, stream)
  switch (d) {
    case 32: GLLM_PF(32);
    case 64: GLLM_PF(64);
    case 128: GLLM_PF(128);
    default: return (int)cudaErrorInvalidValue;
  }
#undef GLLM_PF
}

GLLM_API int gllm_attention_prefill_supports(int d) { return d == 32 || d == 64 || d == 128; }
