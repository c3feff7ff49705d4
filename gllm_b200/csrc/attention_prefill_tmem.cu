// Causal prefill attention over the paged cache on the 5th-generation tensor cores.
//
// The same job as attention_prefill_bf16.cu (portions of prompts attend over everything their
// request has cached, through the block table; replaces the reference's gather + dense
// softmax(QK^T/sqrt(D) + bias)V, gllm/model/layers/attention.py:165-173,
// gllm/ops/attention/reference_attention.py:40-48), but both products run as tcgen05.mma with
// their accumulators in tensor memory, so they take no issue slots from the softmax:
//
//   one CTA = 128 rows (128/G' query tokens x the G' query heads of one kv head), key tiles of 128;
//   warp 0: TMA loads. Q once (a 3-D box: 64 dims x G' heads x tokens); per key tile the K and V
//           pages straight out of the cache pool, one box per page, each lane issuing its own page's
//           boxes, 128-byte swizzle;
//   warp 1 (one thread): S = Q K^T into tensor memory (128 x 128 fp32), later O += P V (128 x D).
//           Head size 128: two score buffers, the scores of the next tile are computed while this one
//           is exponentiated.  Head size 64: one buffer, and two CTAs per SM that fill one another's gaps;
//   warps 2-9 (two threads per row, each with half of a tile's keys): read S from tensor memory, mask,
//           running maximum and sum in fp32, rescale O in tensor memory when the maximum moved, write
//           P (bf16) back into tensor memory, from where the second product takes it as its A
//           operand; at the end O / sum -> global.
//
// A grid so small that twice as many CTAs still fit the GPU at once is launched as pairs of CTAs (clusters of
// two) with the same rows: rows with ten key tiles or more have their tiles dealt out to the two CTAs in
// turn, and the first merges the two (reference maximum, sum, output) through distributed shared memory
// at the end; the chain of tiles, which bounds a small grid, is half as long.
//
// V is used as it lies in the cache ([key][dim], i.e. the "MN-major" operand of the second
// product); nothing is transposed or gathered.  Keys outside a row's view get probability 0 and the
// value rows that hold no key of the request are zeroed in shared memory before they are
// multiplied, so stale pool contents never reach the output.  Every mbarrier wait is bounded.
// No TMA load uses cluster multicast.
#include "umma_utils.cuh"
#include <type_traits>

#ifndef GLLM_PREFILL_SPECULATE
#define GLLM_PREFILL_SPECULATE (NB == 1)
#endif

namespace {
constexpr int BM = 128, BN = 128, THREADS = 320;       // TMA warp, MMA warp, eight softmax warps

// 2^x in one instruction (ex2.approx: about 2 ulp; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two fp32 operations in one instruction (sm_100: fma.rn.f32x2, add.rn.f32x2 on register pairs) and
// the maximum of three: the softmax below is bound by the number of instructions it issues per score.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  unsigned long long ra, rb, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// One chunk of 32 scores of a row.  MASKED: key i of the chunk is seen iff (unsigned)(key_rel + i) <= span.
// WITH_MAX: the maximum of the seen scores joins mx.  WITH_EXP: probabilities 2^(v * scale_log2 + neg_mc) of
// the seen scores (0 for the others) are summed into lsum (two running sums) and packed as bf16 pairs.
template <bool MASKED, bool WITH_MAX, bool WITH_EXP>
__device__ __forceinline__ void softmax_chunk(const float (&v)[32], int key_rel, unsigned span, float scale_log2,
                                              float neg_mc, float& mx, float2& lsum, uint32_t (&packed)[16]) {
  if (MASKED) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const bool s0 = (unsigned)(key_rel + i) <= span, s1 = (unsigned)(key_rel + i + 1) <= span;
      if (WITH_MAX) mx = fmax3(mx, s0 ? v[i] : -INFINITY, s1 ? v[i + 1] : -INFINITY);
      if (WITH_EXP) {
        const float p0 = s0 ? fast_exp2(fmaf(v[i], scale_log2, neg_mc)) : 0.f;
        const float p1 = s1 ? fast_exp2(fmaf(v[i + 1], scale_log2, neg_mc)) : 0.f;
        lsum.x += p0;
        lsum.y += p1;
        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
  } else {
    const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(neg_mc, neg_mc);
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      if (WITH_MAX) mx = fmax3(mx, v[i], v[i + 1]);
      if (WITH_EXP) {
        const float2 t = ffma2(make_float2(v[i], v[i + 1]), sc2, nm2);
        const float2 pr = make_float2(fast_exp2(t.x), fast_exp2(t.y));
        lsum = fadd2(lsum, pr);
        __nv_bfloat162 h = __floats2bfloat162_rn(pr.x, pr.y);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
  }
}

template <int D>
struct TShape {
  static constexpr int DB = D / 64;                     // 64-wide blocks of the head dimension
  static constexpr int TILE = 128 * 128;                // bytes of a [128 x 64] bf16 tile
  static constexpr int Q_BYTES = DB * TILE;
  // Head size 64: two CTAs share an SM (one score buffer each in tensor memory), and overlap one
  // another's softmax and products.  Head size 128: one CTA with two score buffers.
  static constexpr int NBUF = D <= 64 ? 1 : 2;
  static constexpr int CTAS_PER_SM = D <= 64 ? 2 : 1;
  static constexpr int KV_STAGE = DB * TILE;            // K (or V) of one key tile
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;         // 2 stages
  static constexpr int KV_STAGES = 2;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_STAGE;
  static constexpr int SMEM = OFF_V + KV_STAGES * KV_STAGE + 1024;
  // S: 128 columns per buffer (fp32), O: D columns (fp32), P: 64 columns (128 bf16 per row)
  static constexpr int TMEM_COLS = NBUF == 1 ? 256 : 512;
  static constexpr int COL_S = 0, COL_O = NBUF * 128, COL_P = COL_O + D;
  static_assert(COL_P + 64 <= TMEM_COLS, "tensor memory columns");
};

template <int D>
__global__ void __launch_bounds__(THREADS, TShape<D>::CTAS_PER_SM)
prefill_tmem_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                    __nv_bfloat16* __restrict__ out, int64_t out_stride, const int* __restrict__ block_table,
                    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                    const int* __restrict__ slots, int hq, int hkv, int gp, int block_size, int num_pages,
                    float scale_log2, int window, int* __restrict__ status, int pair, int split_min) {
  using S = TShape<D>;
  constexpr int NB = S::NBUF;                            // score buffers in tensor memory
  constexpr int KS = S::KV_STAGES;                       // K (and V) stages in shared memory
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full, o_ready;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float row_max[2][BM];                      // the two halves of a row exchange their maxima here
  pdl_trigger();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (smem_addr(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - smem_addr(smem_dyn));

  // ---- which rows and keys this CTA owns (host-side sizes only; device data is read after pdl_wait)
  const int r = blockIdx.z;
  const int group = hq / hkv;
  const int tiles_per_kv = group / gp;
  // pair == 2: the kernel runs as clusters of two CTAs that have the same rows.  Where the rows have `split_min` key
  // tiles or more, the CTA of rank k takes the tiles first + k, first + k + 2, .. and the first CTA merges the two
  // results at the end (a small grid is bound by its longest chain of tiles); where they have fewer, the first
  // CTA takes them all and the second leaves at once.
  uint32_t rank = 0;
  if (pair > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int head_tile = (int)blockIdx.x / pair;
  const int kvh = head_tile / tiles_per_kv;
  const int h0 = kvh * group + (head_tile - kvh * tiles_per_kv) * gp;
  const int qt = BM / gp;                               // query tokens per CTA

  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_addr(&k_full[s]), 1);
      mbar_init(smem_addr(&v_full[s]), 1);
      mbar_init(smem_addr(&k_empty[s]), 1);
      mbar_init(smem_addr(&v_empty[s]), 1);
      mbar_init(smem_addr(&s_full[s]), 1);
    }
    mbar_init(smem_addr(&p_full), 8);                   // one arrival per softmax warp
    mbar_init(smem_addr(&o_ready), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)),
                 "r"((uint32_t)S::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();

  const int tok_begin = cu_q[r], q_len = cu_q[r + 1] - tok_begin;
  const int n_qtiles = (q_len + qt - 1) / qt;
  const bool has_rows = (int)blockIdx.y < n_qtiles;     // uniform over the CTA (and over the pair)
  const int qtile = n_qtiles - 1 - (int)blockIdx.y;     // longest rows first (y is the slower grid axis)
  const int t0 = qtile * qt;
  const int t_count = has_rows ? min(qt, q_len - t0) : 0;
  const int ctx = ctx_lens[r];
  const int pos_first = ctx + t0, pos_last = ctx + t0 + t_count - 1;
  const int kv_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int tile_first = kv_lo / BN, tile_last = pos_last / BN;
  const int n_all = has_rows ? tile_last - tile_first + 1 : 0;        // key tiles of these rows
  const int nsplit = (pair > 1 && n_all >= split_min) ? 2 : 1;        // the same in both CTAs of a pair
  const bool active = has_rows && (nsplit == 2 || rank == 0);
  const int n_tiles = active ? (n_all - (int)rank + nsplit - 1) / nsplit : 0;   // this CTA's: tile_of(0), tile_of(1), ..
  auto tile_of = [&](int j) { return tile_first + (int)rank + nsplit * j; };

  if (active && warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp takes part: lane p looks page p of the tile up and issues the boxes of that page
    // (one box = the rows of one page of one kv head, 64 dims wide), so the block-table reads and the
    // copies of a tile are in flight together.  Pages the rows cannot see are not read at all.
    const int* bt = block_table + (int64_t)slots[r] * bt_stride;
    const int pages_per_tile = BN / block_size;
    const uint32_t page_bytes = (uint32_t)(S::DB * block_size * 128);
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(smem_addr(&q_full), (uint32_t)S::Q_BYTES);
      for (int db = 0; db < S::DB; ++db)
        tma_load_3d(base + S::OFF_Q + db * S::TILE, &map_q, db * 64, h0, tok_begin + t0, smem_addr(&q_full));
    }
    // this lane's page of tile j (-1: nothing to read) and how many lanes have one
    auto lookup = [&](int j) -> int {
      int page = -1;
      const int key = tile_of(j) * BN + lane * block_size;
      if (j < n_tiles && lane < pages_per_tile && key <= pos_last && key + block_size > kv_lo) {
        page = bt[key / block_size];
        if (page >= num_pages) {
          atomicOr(status, GLLM_STATUS_PAGE_RANGE);
          page = -1;
        }
      }
      return page;
    };
    // K (plane 0) or V (plane 1) of tile j into its stage, once the product that read the stage's
    // previous tile is done
    auto load = [&](int j, int page, int plane) -> bool {
      const int s = j % KS;
      const uint32_t full = smem_addr(plane ? &v_full[s] : &k_full[s]);
      const int n_present = __popc(__ballot_sync(0xffffffffu, page >= 0));
      // (every lane waits: one waiting lane under a branch makes the wait several hundred cycles longer)
      const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_addr(plane ? &v_empty[s] : &k_empty[s]),
                                                        ((uint32_t)(j / KS) & 1u) ^ 1u, status, &abort_flag)) != 0;
      if (!ok) return false;
      if (lane == 0) mbar_expect_tx(full, (uint32_t)n_present * page_bytes);
      __syncwarp();                                     // the expectation is posted before any lane's copies
      if (page >= 0) {
        const int row0 = ((page * 2 + plane) * hkv + kvh) * block_size;
        const uint32_t dst = base + (plane ? S::OFF_V : S::OFF_K) + (uint32_t)(s * S::KV_STAGE + lane * block_size * 128);
#pragma unroll
        for (int db = 0; db < S::DB; ++db) tma_load_2d(dst + db * S::TILE, &map_kv, db * 64, row0, full);
      }
      return true;
    };
    // order: K0, then (two buffers) K(j+1) before V(j): the next scores are issued before this tile's
    // values are used
    int page = lookup(0);
    bool ok = n_tiles > 0 && load(0, page, 0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int page_next = lookup(j + 1);
      if (j + 1 < n_tiles) ok = load(j + 1, page_next, 0);
      if (ok) ok = load(j, page, 1);
      page = page_next;
    }
  } else if (active && warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop with warp-uniform values and waits on the barriers; one elected thread
    // issues the products and their commits (in a branch that only lane 0 takes, every tcgen05.mma cost
    // about 110 cycles to issue, whatever its size; here about 40).
    {
      const bool leader = elect_one();
      const int n_tiles_u = __shfl_sync(0xffffffffu, n_tiles, 0);
      auto wait_u = [&](uint64_t* bar, uint32_t parity) -> bool {
        // every lane waits: a single waiting lane under a branch made each wait several hundred cycles longer
        const bool good = mbar_wait(smem_addr(bar), parity, status, &abort_flag);
        return __all_sync(0xffffffffu, good) != 0;
      };
      constexpr uint32_t idesc_o = umma_idesc_b_mn(BM, 64);
      constexpr uint32_t idesc_s = umma_idesc(BM, BN);
      const uint32_t tmem_s = tmem_base + S::COL_S, tmem_o = tmem_base + S::COL_O, tmem_p = tmem_base + S::COL_P;
      // descriptors once: a tile's address sits in the low 14 bits (in units of 16 bytes), so the other
      // tiles' descriptors are this one plus a constant
      const uint64_t desc_q = umma_desc(base + S::OFF_Q), desc_k = umma_desc(base + S::OFF_K),
                     desc_v = umma_desc(base + S::OFF_V);
      auto wait_k = [&](int j) -> bool { return wait_u(&k_full[j % KS], (uint32_t)(j / KS) & 1u); };
      auto issue_s = [&](int j) -> bool {                // after wait_k(j)
        const int s = j % KS, sb = j % NB;
        const uint64_t dk = desc_k + (uint64_t)((s * S::KV_STAGE) >> 4);
        if (leader) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int db = 0; db < S::DB; ++db)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16(tmem_s + sb * BN, desc_q + (uint64_t)((db * S::TILE + k * 32) >> 4),
                        dk + (uint64_t)((db * S::TILE + k * 32) >> 4), idesc_s, (db > 0 || k > 0) ? 1u : 0u);
          umma_commit(smem_addr(&k_empty[s]));            // K of this stage is consumed
          umma_commit(smem_addr(&s_full[sb]));
        }
        __syncwarp();
        return true;
      };
      // Scores run ahead of the softmax.  Two score buffers: S(j+1) is computed while tile j is
      // exponentiated.  One buffer: S(j+1) is issued as soon as the softmax has read S(j), BEFORE P(j) V(j),
      // so that the softmax of tile j+1 starts while that product still runs (it waits for it before it
      // overwrites P).
      bool ok = n_tiles_u > 0 && wait_u(&q_full, 0u);     // (the second CTA of a pair may have no tile)
      if (ok) ok = wait_k(0) && issue_s(0);
      if (NB > 1 && ok && n_tiles_u > 1) ok = wait_k(1) && issue_s(1);
      for (int j = 0; j < n_tiles_u && ok; ++j) {
        const int s = j % KS;
        // (the keys of the next tile arrive long before the softmax is done: wait for them first)
        if (NB == 1 && j + 1 < n_tiles_u) ok = wait_k(j + 1);
        if (ok) ok = wait_u(&p_full, (uint32_t)j & 1u);  // P(j) written, S(j) read
        if (NB == 1 && ok && j + 1 < n_tiles_u) ok = issue_s(j + 1);
        if (ok) ok = wait_u(&v_full[s], (uint32_t)(j / KS) & 1u);
        if (!ok) break;
        const uint64_t dv = desc_v + (uint64_t)((s * S::KV_STAGE) >> 4);
        if (leader) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int db = 0; db < S::DB; ++db)
#pragma unroll
            for (int k = 0; k < 8; ++k)    // 16 keys per MMA: 8 columns of P (two bf16 each); V rows 16 k ..
              umma_bf16_ts(tmem_o + db * 64, tmem_p + k * 8, dv + (uint64_t)((db * S::TILE + k * 16 * 128) >> 4),
                           idesc_o, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(smem_addr(&v_empty[s]));            // V of this stage is consumed
          umma_commit(smem_addr(&o_ready));               // O holds tiles 0 .. j, P may be overwritten
        }
        __syncwarp();
        if (NB > 1 && j + NB < n_tiles_u) ok = wait_k(j + NB) && issue_s(j + NB);
      }
    }
  } else if (active && warp >= 2) {
    // ------------------------------------------------- softmax, correction, epilogue
    // Two threads per row: warps 2-5 take the keys 0 .. 63 of a tile (and the lower half of the output
    // columns), warps 6-9 the keys 64 .. 127 (and the upper half).  A warp reads the tensor-memory
    // lanes 32 * (warp % 4) ..: warps w and w + 4 work on the same rows and exchange their rows' maxima
    // through shared memory.
    const int quarter = warp & 3;
    const int hsel = (warp - 2) >> 2;                     // which half of the keys and of the output columns
    const int row = quarter * 32 + lane;                 // row of the tile = TMEM lane
    const int tl = row / gp, g = row - tl * gp;
    const bool row_ok = tl < t_count;
    const int qpos = pos_first + tl;
    constexpr int HK = BN / 2, HD = D / 2;               // keys and output columns per thread
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_s0 = tmem_base + S::COL_S + lane_addr + (uint32_t)(hsel * HK);
    const uint32_t tmem_o = tmem_base + S::COL_O + lane_addr + (uint32_t)(hsel * HD);
    const uint32_t tmem_p = tmem_base + S::COL_P + lane_addr + (uint32_t)(hsel * HK / 2);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // Head size 64: one pass per tile.  The probabilities are taken against the reference maximum the row
    // already has while the tile's maximum is found on the side; only when some row's maximum has outgrown
    // its reference (or the row had none) does the warp take the tile again against the new one.
    constexpr bool SPECULATE = GLLM_PREFILL_SPECULATE;
    enum { CHUNK_SKIP = 0, CHUNK_FAST = 1, CHUNK_MASK = 2 };
    for (int j = 0; j < n_tiles; ++j) {
      const int kv0 = tile_of(j) * BN + hsel * HK;        // this thread's first key of the tile
      const uint32_t tmem_s = tmem_s0 + (uint32_t)((j % NB) * BN);
      mbar_wait(smem_addr(&s_full[j % NB]), (uint32_t)(j / NB) & 1u, status, &abort_flag);
      asm volatile("bar.sync 1, 256;" ::: "memory");     // the eight warps go on together
      if (abort_flag) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // keys this row sees in the tile: lo <= key <= hi (hi < lo: none)
      const int hi = row_ok ? qpos : -1;
      const int lo = window > 0 ? max(0, qpos - window + 1) : 0;
      const unsigned span = hi >= lo ? (unsigned)(hi - lo) : 0u;
      const int lo_eff = hi >= lo ? lo : 0x7fffff00;     // no key passes when the row sees nothing
      // Each chunk of 32 keys is, for all rows of the CTA alike: seen by no row (nothing is computed, its
      // probabilities are 0), seen whole by every row (no mask; rows past the portion's end compute values
      // that are never stored), or in between (masked key by key).
      int cls[HK / 32];
#pragma unroll
      for (int ci = 0; ci < HK / 32; ++ci) {
        const int k0 = kv0 + ci * 32;
        const bool none = k0 > pos_last || k0 + 31 < kv_lo;
        const bool all = k0 + 31 <= pos_first && (window <= 0 || k0 >= pos_last - window + 1);
        cls[ci] = none ? CHUNK_SKIP : all ? CHUNK_FAST : CHUNK_MASK;
      }
      // the tile's scores -> (maximum) and/or (probabilities in tensor memory, their sums)
      auto pass = [&](auto with_max, auto with_exp, bool wait_o, float neg_mc, float& mx, float2& lsum) {
        constexpr bool WM = decltype(with_max)::value, WE = decltype(with_exp)::value;
        float v[HK / 32][32];
#pragma unroll
        for (int ci = 0; ci < HK / 32; ++ci) tmem_ld32_nowait(tmem_s + (uint32_t)(ci * 32), v[ci]);
        tmem_wait_ld();
#pragma unroll
        for (int ci = 0; ci < HK / 32; ++ci) {
          tmem_ld_fence16(&v[ci][0]);
          tmem_ld_fence16(&v[ci][16]);
        }
#pragma unroll
        for (int ci = 0; ci < HK / 32; ++ci) {
          uint32_t packed[16];
          if (cls[ci] == CHUNK_FAST) {
            softmax_chunk<false, WM, WE>(v[ci], 0, 0u, scale_log2, neg_mc, mx, lsum, packed);
          } else if (cls[ci] == CHUNK_MASK) {
            softmax_chunk<true, WM, WE>(v[ci], kv0 + ci * 32 - lo_eff, span, scale_log2, neg_mc, mx, lsum, packed);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) packed[i] = 0u;
          }
          if (WE) {
            if (ci == 0 && wait_o) {
              // the previous tile's P V must be done before its P is overwritten
              mbar_wait(smem_addr(&o_ready), (uint32_t)(j - 1) & 1u, status, &abort_flag);
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            tmem_st16_b32(tmem_p + (uint32_t)(ci * 16), packed);   // 32 keys = 16 columns of two bf16
          }
        }
      };
      using Yes = std::true_type;
      using No = std::false_type;
      const bool speculate = SPECULATE && j > 0;
      float mx = -INFINITY;
      float2 lsum = make_float2(0.f, 0.f);
      if (speculate) {
        pass(Yes{}, Yes{}, true, -(m == -INFINITY ? 0.f : m) * scale_log2, mx, lsum);
      } else {
        pass(Yes{}, No{}, false, 0.f, mx, lsum);
      }
      // the two warps of a row exchange their maxima: each arrives on its own barrier when its maximum is
      // written and waits on the other's (two barriers of 64 threads per pair of warps); the stores of the
      // probabilities complete meanwhile
      row_max[hsel][row] = mx;
      asm volatile("bar.arrive %0, 64;" ::"r"(2 + 2 * quarter + hsel) : "memory");
      if (speculate) tmem_wait_st();
      asm volatile("bar.sync %0, 64;" ::"r"(2 + 2 * quarter + (hsel ^ 1)) : "memory");
      mx = fmaxf(mx, row_max[hsel ^ 1][row]);
      // The reference maximum moves only when the row's maximum has grown by more than 2^8 in the
      // exponent: until then the exponentials are taken against the old one (they stay below 256, exact
      // enough in fp32 and bf16, and the final division by the row's sum takes the common factor out),
      // and the output so far needs no rescaling, which is the usual case after a row's first tiles.
      const bool moves = mx > -INFINITY && (m == -INFINITY || (mx - m) * scale_log2 > 8.0f);
      const float m_new = moves ? fmaxf(m, mx) : m;
      if (!speculate || __any_sync(0xffffffffu, moves)) {
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float corr = m == -INFINITY ? 0.f : fast_exp2((m - m_use) * scale_log2);
        // the output so far is rescaled when some row of the warp saw its maximum move
        if (j > 0) {
          if (!speculate) {
            mbar_wait(smem_addr(&o_ready), (uint32_t)(j - 1) & 1u, status, &abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          }
          if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
              float v[32];
              tmem_ld32(tmem_o + (uint32_t)c, v);
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= corr;
              tmem_st32(tmem_o + (uint32_t)c, v);
            }
          }
        }
        l *= corr;
        lsum = make_float2(0.f, 0.f);
        float unused = 0.f;
        pass(No{}, Yes{}, false, -m_use * scale_log2, unused, lsum);
        tmem_wait_st();
      }
      m = m_new;
      l += lsum.x + lsum.y;
      // value rows of keys the request does not hold (a page's unwritten tail, a page that was not
      // read): zero them, so that probability 0 times a stale value never reaches the output
      const int tile0 = tile_of(j) * BN;
      if (tile0 + BN - 1 > pos_last || tile0 < kv_lo) {
        mbar_wait(smem_addr(&v_full[j % KS]), (uint32_t)(j / KS) & 1u, status, &abort_flag);
        const int key = tile0 + row;                     // thread <-> key row of the V tile (lower-half warps)
        if (hsel == 0 && (key > pos_last || key < kv_lo)) {
          for (int db = 0; db < S::DB; ++db) {
            uint4* vrow =
                reinterpret_cast<uint4*>(base_ptr + S::OFF_V + (j % KS) * S::KV_STAGE + db * S::TILE + row * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) vrow[i] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // these writes -> visible to the tensor core
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&p_full));
    }
    // ---- O / l -> global: the row's sum is the two halves' sums
    if (n_tiles > 0) mbar_wait(smem_addr(&o_ready), (uint32_t)(n_tiles - 1) & 1u, status, &abort_flag);
    row_max[hsel][row] = l;                              // (the exchange buffer is free: every maximum was read)
    asm volatile("bar.sync 1, 256;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const float l_row = l + row_max[hsel ^ 1][row];
    __nv_bfloat16* dst = out + (int64_t)(tok_begin + t0 + tl) * out_stride + (int64_t)(h0 + g) * D + hsel * HD;
    auto store32 = [&](int c, const float (&v)[32], float inv) {
      if (row_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 pk;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[q4 * 8 + 2 * i] * inv, v[q4 * 8 + 2 * i + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c + q4 * 8) = pk;
        }
      }
    };
    if (nsplit == 1) {
      if (ok && n_tiles > 0 && !abort_flag) {
        const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          float v[32];
          tmem_ld32(tmem_o + (uint32_t)c, v);            // every lane takes part in the load
          store32(c, v, inv);
        }
      }
    } else {
      // The second CTA leaves its rows' reference maximum, sum and unnormalised output in its own shared memory
      // (the K stages, free now: column-major, so that a warp's rows lie side by side); after the cluster's
      // barrier the first CTA reads them there, brings both results to one reference and stores the rows; a
      // second barrier keeps the second CTA's memory alive until it has.
      float* xo = reinterpret_cast<float*>(base_ptr + S::OFF_K);
      asm volatile("bar.sync 1, 256;" ::: "memory");     // every l was read: row_max carries m and l now
      if (rank == 1) {
        if (hsel == 0) {
          row_max[0][row] = m;
          row_max[1][row] = l_row;
        }
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          float v[32];
          if (n_tiles > 0) {
            tmem_ld32(tmem_o + (uint32_t)c, v);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) xo[(hsel * HD + c + i) * BM + row] = v[i];
        }
      }
      asm volatile("barrier.cluster.arrive.release;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
      if (rank == 0) {
        uint32_t r_m, r_l, r_o;
        asm volatile("mapa.shared::cluster.u32 %0, %1, 1;" : "=r"(r_m) : "r"(smem_addr(&row_max[0][row])));
        asm volatile("mapa.shared::cluster.u32 %0, %1, 1;" : "=r"(r_l) : "r"(smem_addr(&row_max[1][row])));
        asm volatile("mapa.shared::cluster.u32 %0, %1, 1;" : "=r"(r_o) : "r"(base + S::OFF_K + (uint32_t)row * 4u));
        float m1, l1;
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(m1) : "r"(r_m) : "memory");
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(l1) : "r"(r_l) : "memory");
        // (this CTA has a tile whenever the rows have one; a row that saw nothing keeps m = -inf, l = 0)
        const float mm = fmaxf(m, m1);
        const float a0 = m == -INFINITY ? 0.f : fast_exp2((m - mm) * scale_log2);
        const float a1 = m1 == -INFINITY ? 0.f : fast_exp2((m1 - mm) * scale_log2);
        const float l_all = a0 * l_row + a1 * l1;
        const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
        const bool good = ok && !abort_flag;
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          float v[32];
          tmem_ld32(tmem_o + (uint32_t)c, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float o1;
            asm volatile("ld.shared::cluster.f32 %0, [%1];"
                         : "=f"(o1) : "r"(r_o + (uint32_t)((hsel * HD + c + i) * BM * 4)) : "memory");
            v[i] = a0 * v[i] + a1 * o1;
          }
          if (good) store32(c, v, inv);
        }
      }
      asm volatile("barrier.cluster.arrive.release;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  if (active && nsplit > 1 && warp < 2) {
    // the loading and the issuing warp take part in the cluster's two barriers
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------------------------ host side
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

template <int D>
int prefill_tmem_launch(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out, int64_t out_stride,
                        const __nv_bfloat16* cache, const int* block_table, int bt_stride, const int* cu_q,
                        const int* ctx_lens, const int* slots, int num_requests, int max_q_len, int n_tokens,
                        int hq, int hkv, int block_size, int num_pages, float scale, int window, int* status,
                        cudaStream_t stream) {
  using S = TShape<D>;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return (int)cudaErrorNotSupported;
  const int group = hq / hkv;
  const int gp = (group <= BM && BM % group == 0) ? group : 1;
  const int qt = BM / gp;
  CUtensorMap map_q, map_kv;
  {
    // q as [tokens][heads][D]: boxes of 64 dims x gp heads x qt tokens
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)hq, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)gp, (cuuint32_t)qt};
    cuuint32_t elem[3] = {1, 1, 1};
    if (fn(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16*>(q), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  {
    // the cache layer as rows of D: [pages * 2 * kv_heads * block_size][D]; one box = one page of one head
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * 2 * hkv * block_size};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)block_size};
    cuuint32_t elem[2] = {1, 1};
    if (fn(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(cache), dims, strides, box,
           elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(prefill_tmem_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(hkv * (group / gp), (max_q_len + qt - 1) / qt, num_requests);
  // A small grid is bound by its longest CTA's chain of key tiles, not by the SMs' throughput.  Where twice the grid
  // still fits the GPU at once (two CTAs per SM at head size 64), the kernel runs as pairs of CTAs; a pair whose rows
  // have `split_min` key tiles or more shares them (the kernel decides from the lengths it reads on the device, so
  // the launch depends on the step's sizes only).  Measured at head size 64: 512 tokens over 1,536 cached 35.8 -> 29.7 us,
  // 256 over 3,840 58.4 -> 37.9 us; pairs that do not fit at once cost more than they give (1,024 tokens: 25.6 -> 35.8 us).
  static int pair_on = -1, split_min = -1;
  if (pair_on < 0) {
    const char* e = getenv("GLLM_B200_PREFILL_PAIR");
    pair_on = e ? atoi(e) : 1;
    const char* m = getenv("GLLM_B200_PREFILL_SPLIT_MIN_TILES");
    split_min = m ? atoi(m) : 10;
  }
  const int64_t places = (int64_t)gllm_sm_count() * S::CTAS_PER_SM;
  if (pair_on && 2 * (int64_t)grid.x * grid.y * grid.z <= places) {
    grid.x *= 2;
    return gllm_launch_cluster(prefill_tmem_kernel<D>, grid, dim3(THREADS), (size_t)S::SMEM, stream, 2u, map_q, map_kv, out,
                               out_stride, block_table, bt_stride, cu_q, ctx_lens, slots, hq, hkv, gp, block_size,
                               num_pages, scale * 1.4426950408889634f, window, status, 2, split_min);
  }
  return gllm_launch(prefill_tmem_kernel<D>, grid, dim3(THREADS), (size_t)S::SMEM, stream, map_q, map_kv, out,
                     out_stride, block_table, bt_stride, cu_q, ctx_lens, slots, hq, hkv, gp, block_size, num_pages,
                     scale * 1.4426950408889634f, window, status, 1, split_min);
}
}  // namespace

// 1 when the kernel takes this head size and page size.
GLLM_API int gllm_attention_prefill_tmem_supports(int d, int block_size) {
  return (d == 64 || d == 128) && block_size >= 8 && block_size <= 128 && (block_size & (block_size - 1)) == 0;
}

// As gllm_attention_prefill_bf16, plus n_tokens (rows of q).  q and the cache layer must be 16-byte
// aligned, q_stride a multiple of 8.
GLLM_API int gllm_attention_prefill_tmem(const __nv_bfloat16* q, int64_t q_stride, __nv_bfloat16* out,
                                         int64_t out_stride, const __nv_bfloat16* cache, const int* block_table,
                                         int bt_stride, const int* cu_q, const int* ctx_lens, const int* slots,
                                         int num_requests, int max_q_len, int n_tokens, int hq, int hkv, int d,
                                         int block_size, int num_pages, float scale, int window, int* status,
                                         cudaStream_t stream) {
  if (num_requests <= 0 || max_q_len <= 0) return 0;
  if (!gllm_attention_prefill_tmem_supports(d, block_size) || hq <= 0 || hkv <= 0 || hq % hkv ||
      num_requests > 65535 || (q_stride % 8) || (out_stride % 8) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(cache) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || num_pages < 1)
    return (int)cudaErrorInvalidValue;
  if (d == 64)
    return prefill_tmem_launch<64>(q, q_stride, out, out_stride, cache, block_table, bt_stride, cu_q, ctx_lens, slots,
                                   num_requests, max_q_len, n_tokens, hq, hkv, block_size, num_pages, scale, window,
                                   status, stream);
  return prefill_tmem_launch<128>(q, q_stride, out, out_stride, cache, block_table, bt_stride, cu_q, ctx_lens, slots,
                                  num_requests, max_q_len, n_tokens, hq, hkv, block_size, num_pages, scale, window,
                                  status, stream);
}
