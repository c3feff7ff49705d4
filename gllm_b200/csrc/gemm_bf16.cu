// bf16 matrix product out[M, N] = X[M, K] * W[N, K]^T on the 5th-generation
// tensor cores: tcgen05.mma with the accumulator in tensor memory, operands
// brought into shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle),
// fp32 accumulation.  It stands where the reference calls the library
// (gllm/model/layers/linear.py:20, gllm/model/model.py:239).
//
// The kernel is persistent: one CTA per SM walks over work items, each a
// 128 x BN accumulator tile D = A[128, K] * B[BN, K]^T (times a range of K):
//   normal  (many tokens):  A = X (128 tokens),        B = W (BN = 256 weight rows)
//   swapped (few tokens):   A = W (128 weight rows),   B = X (BN = tokens padded to 16/32/64)
// so a decode step streams the weight through the 128-row operand and wastes
// no tensor-core rows on padding.  Six warps: warp 0 issues the TMA loads,
// warp 1 allocates tensor memory and issues the MMAs (one thread), warps 2-5
// read the accumulator back with tcgen05.ld and store.  A ring of shared-memory
// stages is handed back and forth with mbarriers; tcgen05.commit releases a
// stage when the MMAs that read it are done.  Tensor memory holds two
// accumulators, so the loads and MMAs of the next item run while the epilogue
// warps drain the previous one.
//
// With few tokens a weight is cut along K into S splits (S from (N, K) and the
// bucket M falls in: <= 16, <= 32, <= 64); each item writes its fp32 tile to
// scratch and takes a ticket, and the one that draws the last ticket of a tile
// sums the splits in ascending order, so no CTA waits for another and, within a
// bucket, a token's result does not depend on its batch.
//
// Every wait on an mbarrier is bounded: when it runs out, the kernel sets a
// status bit, stops issuing work, lets its copies in flight land (bounded
// again), frees its tensor memory and returns.
//
// accumulate (the few-token orientation only): the epilogue adds its (partial) tile into an fp32
// matrix with red.global.add, so a product that ends a branch adds itself to the residual stream: no
// partial sums are written, and the norm after it reads the residual alone.  The order of these
// additions is not fixed, so results may differ in the last fp32 bit between runs.
//
// No TMA load here uses cluster multicast; every CTA fetches its own tiles.
#include "umma_utils.cuh"

namespace {
constexpr int BM = 128;          // rows of the accumulator tile (MMA M)
constexpr int BK = 64;           // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;
// Most stages of a ring (reached by the small stages of the few-token orientation).
#ifndef GLLM_GEMM_MAX_STAGES
#define GLLM_GEMM_MAX_STAGES 8
#endif

template <typename OutT> __device__ __forceinline__ OutT cast_out(float v);
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <int BN>
struct Shape {
  static constexpr int STAGE_A = BM * BK * 2;
  static constexpr int STAGE_B = BN * BK * 2;
  static constexpr int STAGE = STAGE_A + ((STAGE_B + 1023) / 1024) * 1024;   // keeps every tile 1024-aligned
  static constexpr int STAGES = (SMEM_BUDGET / STAGE) > GLLM_GEMM_MAX_STAGES ? GLLM_GEMM_MAX_STAGES : (SMEM_BUDGET / STAGE);
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;                // two accumulators; a power of two >= 32
  static constexpr int SMEM = STAGES * STAGE + 1024;                         // + slack to align the base
};

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct Item {
  int a_row0, b_row0, split, tile_id;
};
// Work item w of a launch.  Normal: neighbouring CTAs share a weight tile.  Swapped:
// neighbouring CTAs take the K ranges of the same weight rows.
template <int BN, bool SWAPPED>
__device__ __forceinline__ Item item_of(int w, int tiles_a, int splits) {
  Item it;
  const int t = w / splits;
  it.split = w - t * splits;
  const int tb = t / tiles_a, ta = t - tb * tiles_a;
  it.a_row0 = ta * BM;
  it.b_row0 = tb * BN;
  it.tile_id = t;
  return it;
}

// SWAPPED = false: A = X (tile rows are tokens), B = W (tile columns are weight rows).
// SWAPPED = true : A = W (tile rows are weight rows), B = X (tile columns are tokens).
// GATED: the weight rows come in blocks of 64 gate rows followed by the 64 up rows of the same
// features; the epilogue writes silu(gate) * up, [M, N/2] (gllm/model/layers/mlp.py:44-47), instead
// of the [M, N] product.  Only with splits == 1.
template <int BN, bool SWAPPED, typename OutT, bool GATED>
__global__ void __launch_bounds__(THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 OutT* __restrict__ out, int M, int N, int K, int64_t ldo, int splits, int kb_per_split,
                 int tiles_a, int num_items, float* __restrict__ partial, int* __restrict__ tickets,
                 int reduce_in_kernel, int* __restrict__ status, int accumulate) {
  using S = Shape<BN>;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[S::STAGES], empty_bar[S::STAGES], tmem_full_bar[2], tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag, is_last;

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tile_base = (smem_addr(smem_dyn) + 1023u) & ~1023u;
  const int num_kb_total = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 1);
      mbar_init(smem_addr(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&tmem_full_bar[b]), 1);
      mbar_init(smem_addr(&tmem_empty_bar[b]), 4);      // one arrival per epilogue warp
    }
    abort_flag = 0;
    is_last = 0;
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
  // set-up is done (barriers, tensor memory).  The weight never depends on the kernel before this
  // one, so its first tiles are requested before the dependency wait: the weight stream starts while
  // the previous kernel is still running.  Activations are read, and anything is written, after it.

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const CUtensorMap* map_w = SWAPPED ? &map_a : &map_b;
      const CUtensorMap* map_x = SWAPPED ? &map_b : &map_a;
      const uint32_t off_w = SWAPPED ? 0u : (uint32_t)S::STAGE_A, off_x = SWAPPED ? (uint32_t)S::STAGE_A : 0u;
      uint32_t it = 0;                                   // k-blocks issued so far, over all items
      bool ok = true;
      // pass 0: the weight tiles of the first STAGES k-blocks; pass 1: their activation tiles, then
      // both operands of every later block as stages come free
      for (int pass = 0; pass < 2 && ok; ++pass) {
        if (pass == 1) pdl_wait();
        it = 0;
        bool more = true;
        for (int w = blockIdx.x; w < num_items && ok && more; w += gridDim.x) {
          const Item item = item_of<BN, SWAPPED>(w, tiles_a, splits);
          const int kb_begin = item.split * kb_per_split;
          const int kb_end = min(num_kb_total, kb_begin + kb_per_split);
          const int row_w = SWAPPED ? item.a_row0 : item.b_row0, row_x = SWAPPED ? item.b_row0 : item.a_row0;
          for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
            const uint32_t s = it % S::STAGES, round = it / S::STAGES;
            const uint32_t bar = smem_addr(&full_bar[s]);
            const uint32_t dst = tile_base + s * S::STAGE;
            if (pass == 0) {
              if (round > 0) { more = false; break; }
              mbar_expect_tx(bar, (uint32_t)(S::STAGE_A + S::STAGE_B));
              tma_load_2d(dst + off_w, map_w, kb * BK, row_w, bar);
            } else if (round == 0) {
              tma_load_2d(dst + off_x, map_x, kb * BK, row_x, bar);
            } else {
              ok = mbar_wait(smem_addr(&empty_bar[s]), (round & 1u) ^ 1u, status, &abort_flag);
              if (!ok) break;
              mbar_expect_tx(bar, (uint32_t)(S::STAGE_A + S::STAGE_B));
              tma_load_2d(dst + off_w, map_w, kb * BK, row_w, bar);
              tma_load_2d(dst + off_x, map_x, kb * BK, row_x, bar);
            }
          }
        }
      }
      if (abort_flag) {
        // let the copies already issued land before the CTA leaves (bounded)
        const uint32_t first = it > (uint32_t)S::STAGES ? it - S::STAGES : 0u;
        for (uint32_t i = first; i < it; ++i) {
          const unsigned long long t0 = global_timer();
          while (!mbar_try_wait(smem_addr(&full_bar[i % S::STAGES]), (i / S::STAGES) & 1u)) {
            if (global_timer() - t0 > UMMA_WAIT_LIMIT_NS) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop with warp-uniform values and waits on the barriers; one elected thread
    // issues the products and their commits (in a branch that only lane 0 takes, a tcgen05.mma costs about
    // 110 cycles to issue, whatever its size; this way about 40).
    {
      const bool leader = elect_one();
      auto wait_u = [&](uint64_t* bar, uint32_t parity) -> bool {
        const bool good = mbar_wait(smem_addr(bar), parity, status, &abort_flag);
        return __all_sync(0xffffffffu, good) != 0;
      };
      constexpr uint32_t idesc = umma_idesc(BM, BN);
      uint32_t it = 0, n_used = 0;                       // k-blocks consumed; accumulators handed over
      bool ok = true;
      for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
        const Item item = item_of<BN, SWAPPED>(w, tiles_a, splits);
        const int kb_begin = item.split * kb_per_split;
        const int kb_end = min(num_kb_total, kb_begin + kb_per_split);
        if (kb_end <= kb_begin) continue;                // an empty K range: the epilogue writes zeros
        const uint32_t acc = n_used & 1u;
        // the epilogue must have drained this accumulator (two uses ago)
        ok = wait_u(&tmem_empty_bar[acc], ((n_used >> 1) & 1u) ^ 1u);
        if (!ok) break;
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % S::STAGES;
          ok = wait_u(&full_bar[s], (it / S::STAGES) & 1u);
          if (!ok) break;
          const uint64_t a_desc = umma_desc(tile_base + s * S::STAGE);
          const uint64_t b_desc = umma_desc(tile_base + s * S::STAGE + S::STAGE_A);
          if (leader) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // (a tile's address sits in the descriptor's low bits in units of 16 bytes)
              umma_bf16(tmem_d, a_desc + (uint64_t)((k * UMMA_K * 2) >> 4), b_desc + (uint64_t)((k * UMMA_K * 2) >> 4), idesc,
                        (kb > kb_begin || k > 0) ? 1u : 0u);
            }
            umma_commit(smem_addr(&empty_bar[s]));       // the stage is free once these MMAs have read it
          }
          __syncwarp();
        }
        if (ok && leader) umma_commit(smem_addr(&tmem_full_bar[acc]));   // the accumulator is complete
        __syncwarp();
        ++n_used;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    pdl_wait();                                          // nothing is written before the previous kernel is done
    const int quarter = warp & 3;                        // the TMEM lanes this warp may read: 32*quarter ..
    const int row = quarter * 32 + lane;                 // row of the accumulator tile
    const int ep_thread = (warp - 2) * 32 + lane;        // 0 .. 127
    uint32_t n_used = 0;
    for (int w = blockIdx.x; w < num_items; w += gridDim.x) {
      const Item item = item_of<BN, SWAPPED>(w, tiles_a, splits);
      const int kb_begin = item.split * kb_per_split;
      const int kb_end = min(num_kb_total, kb_begin + kb_per_split);
      const bool has_k = kb_end > kb_begin;
      const uint32_t acc = n_used & 1u;
      if (has_k) {
        mbar_wait(smem_addr(&tmem_full_bar[acc]), (n_used >> 1) & 1u, status, &abort_flag);
        // the four warps leave together: one that gave up has set abort_flag before this barrier
        epilogue_sync();
        if (abort_flag) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      float* mine = partial + (int64_t)item.split * M * N;
      if (GATED) {
        const int n_out = N / 2;
        if (!SWAPPED) {
          // this thread's token row holds, per 128 columns, 64 gates then their 64 ups
          const int m = item.a_row0 + row;
#pragma unroll 1
          for (int c2 = 0; c2 < BN / 2; c2 += 16) {
            const int gate_col = (c2 / 64) * 128 + (c2 % 64);
            float g[16], u[16];
            tmem_ld16(taddr + (uint32_t)gate_col, g);
            tmem_ld16(taddr + (uint32_t)(gate_col + 64), u);
            const int f0 = item.b_row0 / 2 + c2;
            if (m < M && f0 < n_out) {
              float y[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) y[i] = g[i] / (1.0f + __expf(-g[i])) * u[i];
              OutT* dst = out + (int64_t)m * ldo + f0;
              if (f0 + 16 <= n_out && sizeof(OutT) == 2 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
                uint4 p0, p1;
                __nv_bfloat162* h0 = reinterpret_cast<__nv_bfloat162*>(&p0);
                __nv_bfloat162* h1 = reinterpret_cast<__nv_bfloat162*>(&p1);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  h0[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
                  h1[i] = __floats2bfloat162_rn(y[8 + 2 * i], y[8 + 2 * i + 1]);
                }
                reinterpret_cast<uint4*>(dst)[0] = p0;
                reinterpret_cast<uint4*>(dst)[1] = p1;
              } else {
                for (int i = 0; i < 16 && f0 + i < n_out; ++i) dst[i] = cast_out<OutT>(y[i]);
              }
            }
          }
        } else {
          // rows 0..63 of the tile are gates, rows 64..127 the ups of the same 64 features.  The two
          // halves trade values through shared memory so that both work: of every 32 token columns the
          // gate rows finish the first 16 (with the ups handed over) and the up rows the second 16 (with
          // the gates handed over); with 16 columns in all only the gate rows have work.
          __shared__ float exch[64][(BN <= 64 ? BN : 1) + 1];
          constexpr int CH = BN >= 32 ? 32 : 16;
          const int f = item.a_row0 / 2 + (row & 63);
#pragma unroll 1
          for (int c = 0; c < BN; c += CH) {
            float v[CH];
            tmem_ld_cols(taddr + (uint32_t)c, v);
            if (row >= 64) {
#pragma unroll
              for (int i = 0; i < 16; ++i) exch[row - 64][c + i] = v[i];
            } else if (CH == 32) {
#pragma unroll
              for (int i = 0; i < 16; ++i) exch[row][c + 16 + i] = v[CH - 16 + i];
            }
            epilogue_sync();
            if (f < n_out && (row < 64 || CH == 32)) {
              const int off = row < 64 ? 0 : 16;               // which 16 columns this thread finishes
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int m = item.b_row0 + c + off + i;
                if (m < M) {
                  const float mine_v = row < 64 ? v[i] : v[CH - 16 + i], other = exch[row & 63][c + off + i];
                  const float g = row < 64 ? mine_v : other, u = row < 64 ? other : mine_v;
                  out[(int64_t)m * ldo + f] = cast_out<OutT>(g / (1.0f + __expf(-g)) * u);
                }
              }
            }
          }
        }
      } else if (SWAPPED) {
        // the accumulator's rows are weight rows, its columns tokens: 32 columns a load where there are that many
        constexpr int CH = BN >= 32 ? 32 : 16;
        const int n = item.a_row0 + row;                 // weight row
#pragma unroll 1
        for (int c = 0; c < BN; c += CH) {
          float v[CH];
          if (has_k) {
            tmem_ld_cols(taddr + (uint32_t)c, v);
          } else {
#pragma unroll
            for (int i = 0; i < CH; ++i) v[i] = 0.f;
          }
          if (n < N) {
#pragma unroll
            for (int i = 0; i < CH; ++i) {
              const int m = item.b_row0 + c + i;         // token
              if (m < M) {
                const float val = v[i];
                if (accumulate) {
                  // every split adds its part into the fp32 matrix itself (a warp's 32 rows are contiguous)
                  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(reinterpret_cast<float*>(out) + (int64_t)m * ldo + n),
                               "f"(val)
                               : "memory");
                } else if (splits > 1) {
                  mine[(int64_t)m * N + n] = val;
                } else {
                  out[(int64_t)m * ldo + n] = cast_out<OutT>(val);
                }
              }
            }
          }
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float v[16];
        if (has_k) {
          tmem_ld16(taddr + (uint32_t)c, v);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
        const int m = item.a_row0 + row, n0 = item.b_row0 + c;
        if (m < M && n0 < N) {
          if (splits > 1) {
            float* dst = mine + (int64_t)m * N + n0;
            if (n0 + 16 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
              for (int i = 0; i < 16 && n0 + i < N; ++i) dst[i] = v[i];
            }
          } else {
            OutT* dst = out + (int64_t)m * ldo + n0;
            if (n0 + 16 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
              if (sizeof(OutT) == 2) {
                uint4 p0, p1;
                __nv_bfloat162* h0 = reinterpret_cast<__nv_bfloat162*>(&p0);
                __nv_bfloat162* h1 = reinterpret_cast<__nv_bfloat162*>(&p1);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  h0[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                  h1[i] = __floats2bfloat162_rn(v[8 + 2 * i], v[8 + 2 * i + 1]);
                }
                reinterpret_cast<uint4*>(dst)[0] = p0;
                reinterpret_cast<uint4*>(dst)[1] = p1;
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
              }
            } else {
              for (int i = 0; i < 16 && n0 + i < N; ++i) dst[i] = cast_out<OutT>(v[i]);
            }
          }
        }
      }
      if (has_k) {
        // this warp is done reading the accumulator: hand it back to the MMA warp
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&tmem_empty_bar[acc]));
        ++n_used;
      }
      if (splits > 1 && reduce_in_kernel && !accumulate) {
        // the CTA that draws the last ticket of this tile sums the splits in ascending order
        __threadfence();
        epilogue_sync();
        if (ep_thread == 0) is_last = (atomicAdd(&tickets[item.tile_id], 1) == splits - 1);
        epilogue_sync();
        if (is_last) {
          __threadfence();
          const int m0 = SWAPPED ? item.b_row0 : item.a_row0, n0 = SWAPPED ? item.a_row0 : item.b_row0;
          const int rows = min(SWAPPED ? BN : BM, M - m0), cols = min(SWAPPED ? BM : BN, N - n0);
          for (int idx = ep_thread; idx < rows * cols; idx += 128) {
            const int m = m0 + idx / cols, n = n0 + idx % cols;
            out[(int64_t)m * ldo + n] = cast_out<OutT>(sum_parts16(partial + (int64_t)m * N + n, splits, (int64_t)M * N));
          }
          if (ep_thread == 0) tickets[item.tile_id] = 0;
        }
        epilogue_sync();                                 // is_last is rewritten for the next item
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
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

// A [rows, cols] bf16 matrix with `ld` elements between rows; boxes of 64 columns x box_rows rows.
bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() { return gllm_sm_count(); }

template <int BN, bool SWAPPED, typename OutT, bool GATED>
int umma_launch(const __nv_bfloat16* X, const __nv_bfloat16* W, OutT* out, int M, int N, int K, int64_t ldx,
                int64_t ldw, int64_t ldo, int splits, float* partial, int* tickets, int reduce_in_kernel, int* status,
                cudaStream_t stream, int accumulate = 0) {
  using S = Shape<BN>;
  CUtensorMap map_a, map_b;
  const bool ok = SWAPPED ? (make_map(&map_a, W, N, K, ldw, BM) && make_map(&map_b, X, M, K, ldx, BN))
                          : (make_map(&map_a, X, M, K, ldx, BM) && make_map(&map_b, W, N, K, ldw, BN));
  if (!ok) return (int)cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(umma_gemm_kernel<BN, SWAPPED, OutT, GATED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int a_rows = SWAPPED ? N : M, b_rows = SWAPPED ? M : N;
  const int num_kb = (K + BK - 1) / BK;
  const int kb_per_split = (num_kb + splits - 1) / splits;
  const int tiles_a = (a_rows + BM - 1) / BM, tiles_b = (b_rows + BN - 1) / BN;
  const int num_items = tiles_a * tiles_b * splits;
  const int grid = num_items < sm_count() ? num_items : sm_count();
  return gllm_launch(umma_gemm_kernel<BN, SWAPPED, OutT, GATED>, dim3(grid), dim3(THREADS), (size_t)S::SMEM, stream, map_a,
                     map_b, out, M, N, K, ldo, splits, kb_per_split, tiles_a, num_items, partial, tickets,
                     reduce_in_kernel, status, accumulate);
}

// Width of the weight tile for more than 64 tokens: 256 rows; 64 for a single tile of tokens (65 .. 128) times a
// narrow weight, where 256 would leave most SMs without a tile (more tiles, and less to write and read back where
// the product is cut along K as well); 128 for 129 .. 512 tokens, and for up to 256 tokens of the gated product:
// twice the work items of half the size, each with a longer range of K (measured alone, 256 -> 128 wide: q/k/v at
// 256 tokens 23.6 -> 17.4 us, o 19.5 -> 15.4, down 25.6 -> 23.6, gate/up at 128 tokens 35.8 -> 27.7; from 768 tokens on
// the wide tile wins again: gate/up 58 against 65 us).
static int normal_tile_rows(int M, int N, bool gated) {
  if (gated) return M <= 256 ? 128 : 256;
  if (M <= BM) return (N + 255) / 256 < 64 ? 64 : 256;
  return M <= 512 ? 128 : 256;
}

template <typename OutT, bool GATED>
int umma_dispatch(const __nv_bfloat16* X, const __nv_bfloat16* W, OutT* out, int M, int N, int K, int64_t ldx,
                  int64_t ldw, int64_t ldo, int splits, float* partial, int* tickets, int reduce_in_kernel, int* status,
                  cudaStream_t stream) {
#define GLLM_UMMA(BN, SW) \
  return umma_launch<BN, SW, OutT, GATED>(X, W, out, M, N, K, ldx, ldw, ldo, splits, partial, tickets, reduce_in_kernel, \
                                   status, stream)
  if (M <= 16) GLLM_UMMA(16, true);
  if (M <= 32) GLLM_UMMA(32, true);
  if (M <= 64) GLLM_UMMA(64, true);
  if (normal_tile_rows(M, N, GATED) == 64) GLLM_UMMA(64, false);
  if (normal_tile_rows(M, N, GATED) == 128) GLLM_UMMA(128, false);
  GLLM_UMMA(256, false);
#undef GLLM_UMMA
}
}  // namespace

// Splits along K for M tokens and an [N, K] weight.  It depends on (N, K) and on the bucket M falls
// in (<= 16, <= 32, <= 64, then multiples of 128), never on M itself: enough items to keep every SM
// busy, as long as the fp32 partial tiles stay a small part of the weight's bytes.
GLLM_API int gllm_gemm_bf16_splits(int M, int N, int K) {
  const int num_kb = (K + BK - 1) / BK;
  int tiles, limit;
  if (M <= 64) {
    const int bucket = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    tiles = (N + BM - 1) / BM;                   // swapped orientation: 128 weight rows per tile
    limit = K / (4 * bucket);
  } else {
    const int bn = normal_tile_rows(M, N, false);
    tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);   // 128 tokens x 256 (or 64) weight rows per tile
    limit = K / 512;
  }
  if (tiles >= 96) return 1;                    // wide enough to keep most SMs busy without a cut
  // as many splits as give every SM at most one item (one pipeline ramp per SM), each at least two
  // k-blocks long, none empty
  int best = 1;
  for (int s = 2; s <= 16; ++s) {
    if (tiles * s > gllm_sm_count() || s > limit || num_kb / s < 2) break;
    const int per = (num_kb + s - 1) / s;
    if (per * (s - 1) < num_kb) best = s;        // the last split is not empty
  }
  return best;
}

// Output tiles of the launch (the ticket array needs this many zeroed ints when splits > 1).
GLLM_API int gllm_gemm_bf16_tiles(int M, int N) {
  if (M <= 64) return (N + BM - 1) / BM;
  const int bn = normal_tile_rows(M, N, false);
  return ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
}

// out_is_f32: 0 = bf16 output, 1 = fp32 output.  Needs K % 8 == 0 and 16-byte aligned rows of X and W.
// partial: splits * M * N floats of scratch when splits > 1, laid out [split][M][N].
// reduce_in_kernel != 0: the kernel sums the splits itself into `out` (tickets: zeroed ints, left at
// zero).  reduce_in_kernel == 0 with splits > 1: `out` is not written; the caller's next kernel sums
// partial[0..splits) in ascending order.
GLLM_API int gllm_gemm_bf16(const __nv_bfloat16* X, const __nv_bfloat16* W, void* out, int out_is_f32, int M,
                            int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int splits, float* partial,
                            int* tickets, int reduce_in_kernel, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || splits < 1 || splits > 16 ||
      (reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return (int)cudaErrorInvalidValue;
  if (out_is_f32)
    return umma_dispatch<float, false>(X, W, (float*)out, M, N, K, ldx, ldw, ldo, splits, partial, tickets, reduce_in_kernel,
                                status, stream);
  return umma_dispatch<__nv_bfloat16, false>(X, W, (__nv_bfloat16*)out, M, N, K, ldx, ldw, ldo, splits, partial,
                                             tickets, reduce_in_kernel, status, stream);
}

// The gated feed-forward's first product with SiLU(gate) * up in the epilogue: W is [2*I, K] with
// rows in blocks of 64 gate rows followed by the 64 up rows of the same features (I % 64 == 0);
// out is [M, I] bf16.  Never cut along K.
GLLM_API int gllm_gemm_bf16_gated(const __nv_bfloat16* X, const __nv_bfloat16* W, __nv_bfloat16* out, int M,
                                  int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int* status,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || N % 128 || (reinterpret_cast<uintptr_t>(X) & 15) ||
      (reinterpret_cast<uintptr_t>(W) & 15))
    return (int)cudaErrorInvalidValue;
  return umma_dispatch<__nv_bfloat16, true>(X, W, out, M, N, K, ldx, ldw, ldo, 1, nullptr, nullptr, 0, status,
                                            stream);
}

// The product of few tokens (M <= 64) added into an fp32 matrix: acc[M, N] += X[M, K] * W[N, K]^T, each
// of the `splits` K ranges adding its part with red.global.add (no scratch, nothing to sum afterwards).
// For a product that ends a branch of a layer: `acc` is the residual stream.
GLLM_API int gllm_gemm_bf16_accumulate(const __nv_bfloat16* X, const __nv_bfloat16* W, float* acc, int M, int N,
                                       int K, int64_t ldx, int64_t ldw, int64_t ldo, int splits, int* status,
                                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || splits < 1 || splits > 16 ||
      (reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return (int)cudaErrorInvalidValue;
#define GLLM_ACC(BN) \
  return umma_launch<BN, true, float, false>(X, W, acc, M, N, K, ldx, ldw, ldo, splits, nullptr, nullptr, 0, status, \
                                             stream, 1)
  if (M <= 16) GLLM_ACC(16);
  if (M <= 32) GLLM_ACC(32);
  GLLM_ACC(64);
#undef GLLM_ACC
}
