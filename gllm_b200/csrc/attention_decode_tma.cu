// Split-KV decode attention of the bf16 path as one persistent stream: one query token per request
// over the paged cache (it replaces the reference's per-step gather of the whole padded context plus
// dense softmax(QK^T/sqrt(D) + bias)V, gllm/model/layers/attention.py:165-173,
// gllm/ops/attention/reference_attention.py:40-48), for head sizes of 64 and 128, up to 8 kv heads
// with up to 16 query heads each, and pages of 16 or 32 tokens.  Made for steps with many keys to
// read (large batches): attention_bf16.cu has more, smaller work items for the small ones.
//
// Decoding is bound by the trip of the keys and values from HBM, so the kernel keeps that stream
// going without a gap.  A page of the cache holds the keys of all kv heads side by side, then their
// values: 16 KB each at 8 heads x 16 tokens x 64 dims, one TMA box each.  One CTA per SM walks over
// work items (a span of 128 keys of one request, all heads):
//   warp 0 looks the span's pages up (one lane per page) and requests them page by page into a ring
//          of stages (128-byte swizzle), the query heads of the request with the span's first stage;
//   warps 1-8 own one kv head each (with fewer kv heads: one head of one of several pages of a
//          stage).  A warp takes the stages as they fill and runs Q K^T and P V for its head on the
//          tensor cores (mma.sync m16n8k16, the head's query heads are the rows; bf16 in, fp32
//          accumulate), with the running maximum, sum and output in registers (fp32); nothing is
//          shared between warps, so none waits for another.  At the end of the span it writes its
//          partial result; a second kernel merges the partial results in ascending order.
//
// Everything a request cached before this step is older than the step's kernels: the first stages
// are requested before the dependency wait, all but the pages that hold a newest key (and the
// queries).  Value rows that hold no visible key are zeroed in shared memory before they are
// multiplied, so stale pool contents never reach the output.  Every mbarrier wait is bounded.
// No TMA load uses cluster multicast.
//
// Cache layer layout: [page][k|v][kv_head][block_size][head_dim].
#include "umma_utils.cuh"
#include "mma_utils.cuh"

namespace {
constexpr int ROWS = 16;        // query heads per kv head at most (rows of the MMA tile)
constexpr int CWARPS = 8;       // consumer warps
constexpr int THREADS = (1 + CWARPS) * 32;
constexpr int SPAN = 128;       // keys per work item
// keys a warp takes from a stage: 32 (two pages of 16, or one of 32); 16 where 32 would not leave
// room for two stages (head size 128 with pages of 16)
__host__ __device__ constexpr int keys_per_warp(int d, int block_size) { return (d <= 64 || block_size == 32) ? 32 : 16; }
constexpr int MAXQ = 512;       // requests whose position and block-table row are kept in shared memory
constexpr int SMEM_BUDGET = 214 * 1024;

static __device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Sizes of a launch, the same on host and device.
struct StreamPlan {
  int pps;            // warp tiles (of keys_per_warp keys) per stage and kv head (hkv * pps <= 8 warps)
  int pages;          // pages per stage: pps * keys_per_warp / block_size
  int page_bytes;     // K (or V) of one page, all kv heads, one 64-dim block
  int kv_bytes;       // K (or V) of one stage
  int q_bytes;        // the query area of a stage: (hq + 16) rows of D
  int stage_bytes;
  int stages;
};
__host__ __device__ inline StreamPlan make_plan(int d, int hq, int hkv, int block_size) {
  StreamPlan p;
  const int kpw = keys_per_warp(d, block_size);
  p.pps = CWARPS / hkv;
  if (p.pps > SPAN / kpw) p.pps = SPAN / kpw;
  p.pages = p.pps * (kpw / block_size);
  p.page_bytes = hkv * block_size * 128;
  p.kv_bytes = (d / 64) * p.pages * p.page_bytes;
  p.q_bytes = (((hq + ROWS) * d * 2 + 1023) / 1024) * 1024;
  p.stage_bytes = 2 * p.kv_bytes + p.q_bytes;
  p.stages = SMEM_BUDGET / p.stage_bytes;
  if (p.stages > 8) p.stages = 8;
  return p;
}

struct WorkItem {
  int n, span, qpos, c0, c1;
  bool empty;
};

template <int D, int BS>
__global__ void __launch_bounds__(THREADS, 1)
decode_stream_kernel(const __grid_constant__ CUtensorMap map_kv, const __nv_bfloat16* __restrict__ q,
                     int64_t q_stride, const int* __restrict__ block_table, int bt_stride,
                     const int* __restrict__ positions, const int* __restrict__ token_row,
                     float* __restrict__ part_o, float* __restrict__ part_ml, int num_queries, int hq, int hkv,
                     int num_pages, int num_spans, float scale_log2, int window, int* __restrict__ status) {
  constexpr int DB = D / 64;
  constexpr int KPW = keys_per_warp(D, BS);
  constexpr int PAGES_PER_SPAN = SPAN / BS;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8];
  __shared__ int abort_flag;
  __shared__ int s_qpos[MAXQ], s_row[MAXQ];
  pdl_trigger();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const StreamPlan plan = make_plan(D, hq, hkv, BS);
  const int STAGES = plan.stages;
  // positions and block-table rows are step inputs (older than the step's kernels): read at once
  for (int i = threadIdx.x; i < min(num_queries, MAXQ); i += THREADS) {
    s_qpos[i] = positions[i];
    s_row[i] = token_row[i];
  }
  const uint32_t base = (smem_addr(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - smem_addr(smem_dyn));
  const int group = hq / hkv;
  const int num_items = num_queries * num_spans;
  const int chunks_total = num_spans * plan.pps;          // partial results per (request, query head)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 1);
      mbar_init(smem_addr(&empty_bar[s]), CWARPS);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the rows after the last query head of a stage's query area stay zero for the whole kernel
  for (int i = threadIdx.x; i < STAGES * (ROWS * D * 2 / 16); i += THREADS) {
    const int s = i / (ROWS * D * 2 / 16), o = i - s * (ROWS * D * 2 / 16);
    reinterpret_cast<uint4*>(base_ptr + s * plan.stage_bytes + 2 * plan.kv_bytes + hq * D * 2)[o] =
        make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  // Item w: the span index is the slowest digit, so the spans every request has come first and the
  // ones that hold the newest keys last.
  auto item_of = [&](int w) -> WorkItem {
    WorkItem it;
    it.span = w / num_queries;
    it.n = w - it.span * num_queries;
    it.qpos = it.n < MAXQ ? s_qpos[it.n] : positions[it.n];
    const int kstart = window > 0 ? max(0, it.qpos - window + 1) : 0;
    it.c0 = max(it.span * SPAN, kstart);
    it.c1 = min((it.span + 1) * SPAN, it.qpos + 1);
    it.empty = it.c0 >= it.c1;
    return it;
  };
  // the stages of an item: groups of plan.pages pages from the first page with a visible key to the last
  auto first_group = [&](const WorkItem& it) { return (it.c0 - it.span * SPAN) / (BS * plan.pages); };
  auto last_group = [&](const WorkItem& it) { return (it.c1 - 1 - it.span * SPAN) / (BS * plan.pages); };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    bool ok = true;
    auto next_item = [&](int w) -> int {                 // the first item at or after w that has keys
      while (w < num_items && item_of(w).empty) w += gridDim.x;
      return w;
    };
    // this lane's page of the item's span, unchecked (-1: none); the load is not waited for here
    auto lookup = [&](const WorkItem& item) -> int {
      const int key = item.span * SPAN + lane * BS;
      if (lane < PAGES_PER_SPAN && key < item.c1 && key + BS > item.c0) {
        const int row = item.n < MAXQ ? s_row[item.n] : token_row[item.n];
        return block_table[(int64_t)row * bt_stride + key / BS];
      }
      return -1;
    };
    // pass 0: the first STAGES stages, all pages but those with a newest key; then the wait;
    // pass 1: what was held back of those stages (queries, newest pages), then every later stage.
    // The pages of the item after the current one are looked up while the current one is requested.
    for (int pass = 0; pass < 2 && ok; ++pass) {
      if (pass == 1) pdl_wait();
      uint32_t it = 0;                                    // stages requested so far
      int w = next_item(blockIdx.x);
      WorkItem item = item_of(min(w, num_items - 1));
      int my_page = w < num_items ? lookup(item) : -1;
      bool more = true;
      while (w < num_items && ok && more) {
        const int w_next = next_item(w + gridDim.x);
        const WorkItem item_next = item_of(min(w_next, num_items - 1));
        const int page_next = w_next < num_items ? lookup(item_next) : -1;
        if (my_page >= num_pages) {
          atomicOr(status, GLLM_STATUS_PAGE_RANGE);
          my_page = -1;
        }
        const int g0 = first_group(item), g1 = last_group(item);
        for (int g = g0; g <= g1; ++g, ++it) {
          const uint32_t s = it % STAGES, round = it / STAGES;
          if (pass == 0 && round > 0) { more = false; break; }
          // lanes 0 .. pages-1 take the pages of this stage
          const int page = __shfl_sync(0xffffffffu, my_page, min(g * plan.pages + lane, 31));
          const int key = item.span * SPAN + (g * plan.pages + lane) * BS;
          const bool mine = lane < plan.pages && page >= 0;
          const bool newest = key <= item.qpos && item.qpos < key + BS;
          const int n_present = __popc(__ballot_sync(0xffffffffu, mine));
          const bool with_q = g == g0;
          const uint32_t bar = smem_addr(&full_bar[s]);
          const uint32_t stage = base + s * plan.stage_bytes;
          if (pass == 1 && round > 0) {
            // (every lane waits: one waiting lane under a branch makes the wait several hundred cycles longer)
            ok = __all_sync(0xffffffffu, mbar_wait(smem_addr(&empty_bar[s]), (round & 1u) ^ 1u, status, &abort_flag)) != 0;
            if (!ok) break;
          }
          if (lane == 0 && (pass == 0 || round > 0))
            mbar_expect_tx(bar, (uint32_t)(n_present * 2 * DB * plan.page_bytes) + (with_q ? (uint32_t)(hq * D * 2) : 0u));
          __syncwarp();                                   // the expectation is posted before any copy can land
          const bool first_round = round == 0;
          if (mine && (!first_round || (pass == 0 ? !newest : newest))) {
            const int row_k = (page * 2 + 0) * hkv * BS, row_v = (page * 2 + 1) * hkv * BS;
            const uint32_t dst = stage + (uint32_t)(lane * plan.page_bytes);
#pragma unroll
            for (int db = 0; db < DB; ++db) {
              tma_load_2d(dst + db * plan.pages * plan.page_bytes, &map_kv, db * 64, row_k, bar);
              tma_load_2d(dst + plan.kv_bytes + db * plan.pages * plan.page_bytes, &map_kv, db * 64, row_v, bar);
            }
          }
          if (lane == 0 && with_q && pass == 1)
            bulk_load(stage + 2 * plan.kv_bytes, q + (int64_t)item.n * q_stride, (uint32_t)(hq * D * 2), bar);
        }
        w = w_next;
        item = item_next;
        my_page = page_next;
      }
      if (pass == 1 && abort_flag && lane == 0) {
        // let the copies already requested land before the CTA leaves (bounded)
        const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0u;
        for (uint32_t i = first; i < it; ++i) {
          const unsigned long long t0 = global_timer();
          while (!mbar_try_wait(smem_addr(&full_bar[i % STAGES]), (i / STAGES) & 1u)) {
            if (global_timer() - t0 > UMMA_WAIT_LIMIT_NS) break;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    pdl_wait();                                           // they write: nothing before the previous kernel is done
    const int cw = warp - 1;                              // 0 .. 7
    const int slot = cw / hkv, kvh = cw - slot * hkv;     // this warp's page of a stage and its kv head
    const bool working = slot < plan.pps;                 // warps past pps * hkv only hand the stages back
    const int heads = min(ROWS, group);
    const int h0 = kvh * group;
    const int g8 = lane >> 2, t4 = lane & 3;
    const int mat = lane >> 3, rl = lane & 7;
    uint32_t it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
      const WorkItem item = item_of(w);
      if (item.empty) {                                   // nothing of this span is visible
        if (working && lane < heads) {
          float* ml = part_ml + (((int64_t)item.n * hq + h0 + lane) * chunks_total + item.span * plan.pps + slot) * 2;
          ml[0] = -INFINITY;
          ml[1] = 0.f;
        }
        continue;
      }
      float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
      float o[D / 8][4];
#pragma unroll
      for (int nd = 0; nd < D / 8; ++nd)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nd][e] = 0.f;
      uint32_t qf[D / 16][4];
      const int g0 = first_group(item), g1 = last_group(item);
      for (int g = g0; g <= g1; ++g, ++it) {
        const uint32_t s = it % STAGES;
        if (!mbar_wait(smem_addr(&full_bar[s]), (it / STAGES) & 1u, status, &abort_flag)) { ok = false; break; }
        unsigned char* k_sm = base_ptr + s * plan.stage_bytes;
        unsigned char* v_sm = k_sm + plan.kv_bytes;
        if (working) {
          if (g == g0) {
            // the head's query rows, kept in registers for the whole span
            const unsigned char* q_sm = v_sm + plan.kv_bytes;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const int row = h0 + (mat & 1) * 8 + rl, piece = 2 * ks + (mat >> 1);
              ldmatrix_x4(qf[ks], smem_u32(q_sm + row * (D * 2) + piece * 16));
            }
          }
          // this warp's tile of the stage: KPW keys of head kvh, i.e. the pages slot * PPW .. of the
          // stage; a page's rows of one head are BS rows of 128 bytes per 64-dim block
          constexpr int PPW = KPW / BS;
          const int k0 = item.span * SPAN + (g * plan.pps + slot) * KPW;
          if (k0 < item.c1 && k0 + KPW > item.c0) {
            const uint32_t blk = (uint32_t)(plan.pages * plan.page_bytes);
            // byte offset of key kk (0 .. KPW-1) of the tile inside a 64-dim block
            auto key_row = [&](int kk) -> uint32_t {
              return (uint32_t)((slot * PPW + kk / BS) * plan.page_bytes + kvh * BS * 128 + (kk % BS) * 128);
            };
            // value rows without a visible key (the unwritten tail of a page, a page that was not read,
            // keys before the window)
            if (k0 < item.c0 || k0 + KPW > item.c1) {
              for (int idx = lane; idx < KPW * DB * 8; idx += 32) {
                const int r = idx / (DB * 8), rest = idx - r * (DB * 8);
                if (k0 + r < item.c0 || k0 + r >= item.c1)
                  *reinterpret_cast<uint4*>(v_sm + key_row(r) + (rest >> 3) * blk + ((rest & 7) << 4)) =
                      make_uint4(0u, 0u, 0u, 0u);
              }
              __syncwarp();
            }
            // ---- S = Q K^T (16 heads x KPW keys)
            float sc[KPW / 8][4];
#pragma unroll
            for (int nt = 0; nt < KPW / 8; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e) sc[nt][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
              for (int np = 0; np < KPW / 16; ++np) {
                const int row = np * 16 + (mat >> 1) * 8 + rl, piece = 2 * ks + (mat & 1);
                uint32_t b[4];
                ldmatrix_x4(b, smem_u32(k_sm + key_row(row) + (piece >> 3) * blk + (((piece & 7) ^ (row & 7)) << 4)));
                mma_bf16(sc[2 * np], qf[ks], b[0], b[1]);
                mma_bf16(sc[2 * np + 1], qf[ks], b[2], b[3]);
              }
            }
            // ---- mask, scale, running softmax (rows g8 and g8 + 8)
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < KPW / 8; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int key = k0 + nt * 8 + 2 * t4 + (e & 1);
                const float v = (key >= item.c0 && key < item.c1) ? sc[nt][e] * scale_log2 : -INFINITY;
                sc[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
              }
            float corr[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
              mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
              const float m_new = fmaxf(m[i], mx[i]);     // finite: the tile has at least one visible key
              corr[i] = fast_exp2(m[i] - m_new);          // 0 for the first tile (m = -inf)
              m[i] = m_new;
              l[i] *= corr[i];
            }
            float ls[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < KPW / 8; ++nt)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float p = fast_exp2(sc[nt][e] - m[e >> 1]);
                sc[nt][e] = p;
                ls[e >> 1] += p;
              }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              ls[i] += __shfl_xor_sync(0xffffffffu, ls[i], 1);
              ls[i] += __shfl_xor_sync(0xffffffffu, ls[i], 2);
              l[i] += ls[i];
            }
#pragma unroll
            for (int nd = 0; nd < D / 8; ++nd) {
              o[nd][0] *= corr[0];
              o[nd][1] *= corr[0];
              o[nd][2] *= corr[1];
              o[nd][3] *= corr[1];
            }
            // ---- O += P V
#pragma unroll
            for (int kk = 0; kk < KPW / 16; ++kk) {
              uint32_t a[4];
              a[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
              a[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
              a[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
              a[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
              for (int nd2 = 0; nd2 < D / 16; ++nd2) {
                const int row = kk * 16 + (mat & 1) * 8 + rl, piece = 2 * nd2 + (mat >> 1);
                uint32_t b[4];
                ldmatrix_x4_trans(b, smem_u32(v_sm + key_row(row) + (piece >> 3) * blk + (((piece & 7) ^ (row & 7)) << 4)));
                mma_bf16(o[2 * nd2], a, b[0], b[1]);
                mma_bf16(o[2 * nd2 + 1], a, b[2], b[3]);
              }
            }
          }
        }
        // the stage goes back to the producer: this warp's reads and writes of it are done
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&empty_bar[s]));
      }
      if (!ok) break;
      // ---- this warp's partial result of the span: one chunk per (span, page slot)
      if (working) {
        const int chunk = item.span * plan.pps + slot;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int row = g8 + 8 * i;
          if (row < heads) {
            const int64_t rec = ((int64_t)item.n * hq + h0 + row) * chunks_total + chunk;
            if (t4 == 0) {
              part_ml[rec * 2] = m[i];                    // in units of log2; -inf when the slot saw no key
              part_ml[rec * 2 + 1] = l[i];
            }
            float* po = part_o + rec * D;
#pragma unroll
            for (int nd = 0; nd < D / 8; ++nd)
              *reinterpret_cast<float2*>(po + nd * 8 + 2 * t4) = make_float2(o[nd][2 * i], o[nd][2 * i + 1]);
          }
        }
      }
    }
  }
}

// Merges the partial results of one (request, query head) in ascending order, in one pass (running
// maximum, sum and output).  Only the chunks that can hold a visible key are read: those of the keys
// kstart .. qpos, `per_span` consecutive chunks for every `span_keys` keys.
template <int D>
__global__ void decode_stream_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

bool plan_ok(int d, int hq, int hkv, int block_size) {
  if ((d != 64 && d != 128) || (block_size != 16 && block_size != 32)) return false;
  if (hq <= 0 || hkv <= 0 || hq % hkv || hkv > CWARPS || hq / hkv > ROWS) return false;
  if (hkv * block_size > 256) return false;              // one TMA box holds a page's keys of all heads
  const StreamPlan p = make_plan(d, hq, hkv, block_size);
  return p.stages >= 2;
}

template <int D, int BS>
int stream_launch(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out, int64_t out_stride,
                  const __nv_bfloat16* cache, const int* block_table, int bt_stride, const int* positions,
                  const int* token_row, int num_queries, float* part_o, float* part_ml, int hq, int hkv,
                  int num_pages, int num_spans, float scale, int window, int sms, int* status, cudaStream_t stream) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return (int)cudaErrorNotSupported;
  const StreamPlan plan = make_plan(D, hq, hkv, BS);
  CUtensorMap map_kv;
  {
    // the cache layer as rows of D: [pages * 2 * kv_heads * block_size][D]; one box = the keys (or the
    // values) of one page, all heads, 64 dims wide
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * 2 * hkv * BS};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)(hkv * BS)};
    cuuint32_t elem[2] = {1, 1};
    if (fn(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(cache), dims, strides, box,
           elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  const int smem = plan.stages * plan.stage_bytes + 1024;
  static int attr_smem = 0;
  if (smem > attr_smem) {
    cudaError_t e = cudaFuncSetAttribute(decode_stream_kernel<D, BS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_smem = smem;
  }
  const int64_t items = (int64_t)num_queries * num_spans;
  const int grid = (int)(items < sms ? items : sms);
  int e = gllm_launch(decode_stream_kernel<D, BS>, dim3(grid), dim3(THREADS), (size_t)smem, stream, map_kv, q, q_stride,
                      block_table, bt_stride, positions, token_row, part_o, part_ml, num_queries, hq, hkv, num_pages,
                      num_spans, scale * 1.4426950408889634f, window, status);
  if (e) return e;
  return gllm_launch(decode_stream_merge_kernel<D>, dim3(hq, num_queries), dim3(D), 0, stream, part_o, part_ml, out,
                     out_stride, hq, num_spans * plan.pps, positions, window, SPAN, plan.pps);
}

int sm_count() {
  static int sms[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    sms[dev] = n;
  }
  return sms[dev];
}
}  // namespace

// Partial results per 128 keys of a request for these sizes (0: this kernel does not take them).
GLLM_API int gllm_attention_decode_stream_parts(int d, int hq, int hkv, int block_size) {
  if (!plan_ok(d, hq, hkv, block_size)) return 0;
  return make_plan(d, hq, hkv, block_size).pps;
}

// Query token i of the call is row i of q / out / positions / token_row.  num_spans =
// ceil(longest sequence / 128) (or more); with parts = gllm_attention_decode_stream_parts(...) the
// caller provides scratch: part_o  [num_queries * hq * num_spans * parts * d] floats,
//                          part_ml [num_queries * hq * num_spans * parts * 2] floats.
// q and the cache layer must be 16-byte aligned, q_stride a multiple of 8.
GLLM_API int gllm_attention_decode_stream(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                                          int64_t out_stride, const __nv_bfloat16* cache, const int* block_table,
                                          int bt_stride, const int* positions, const int* token_row,
                                          int num_queries, float* part_o, float* part_ml, int hq, int hkv, int d,
                                          int block_size, int num_pages, int num_spans, float scale, int window,
                                          int* status, cudaStream_t stream) {
  if (num_queries <= 0) return 0;
  if (!plan_ok(d, hq, hkv, block_size) || num_spans <= 0 || (q_stride % 8) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(cache) & 15) || num_pages < 1 ||
      (int64_t)num_queries * hq * num_spans * 8 > (int64_t)1 << 30)
    return (int)cudaErrorInvalidValue;
  const int sms = sm_count();
  if (sms <= 0) return (int)cudaErrorInvalidDevice;
#define GLLM_STREAM(DD, BB)                                                                                     \
  return stream_launch<DD, BB>(q, q_stride, out, out_stride, cache, block_table, bt_stride, positions,          \
                               token_row, num_queries, part_o, part_ml, hq, hkv, num_pages, num_spans, scale,   \
                               window, sms, status, stream)
  if (d == 64 && block_size == 16) GLLM_STREAM(64, 16);
  if (d == 64 && block_size == 32) GLLM_STREAM(64, 32);
  if (d == 128 && block_size == 16) GLLM_STREAM(128, 16);
  if (d == 128 && block_size == 32) GLLM_STREAM(128, 32);
#undef GLLM_STREAM
  return (int)cudaErrorInvalidValue;
}
