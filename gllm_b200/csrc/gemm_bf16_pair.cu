// out[M, N] = X[M, K] @ W[N, K]^T in bf16 with fp32 accumulation, for many tokens, with pairs of CTAs
// (the reference's torch linear, gllm/model/layers/linear.py:20, and with GATED the gate/up product of
// gllm/model/layers/mlp.py:44-47 with SiLU(gate) * up in the epilogue).
//
// Two CTAs of a cluster, on two SMs, work on one tile of 256 tokens x 256 weight rows
// (tcgen05.mma.cta_group::2): each CTA loads 128 of the tile's token rows and 128 of its weight rows,
// the pair's tensor cores read both halves of the weight operand, and each CTA ends up with its 128
// token rows x 256 columns of the result in its own tensor memory.  Against the one-CTA kernel of
// gemm_bf16.cu (128 x 256 tiles) a CTA moves two thirds of the shared-memory bytes per FLOP and
// holds 6 stages instead of 4.
//
//   warp 0 (one thread, both CTAs): TMA producer into a ring of 6 stages; every copy reports to the
//           barrier of the pair's first CTA;
//   warp 1 (one thread, first CTA only): waits for a stage of both CTAs, issues the MMAs of the pair,
//           commits to both CTAs' barriers;
//   warps 2-5 (both CTAs): epilogue from their CTA's tensor memory (two accumulators of 256 columns),
//           then hand the accumulator back to the first CTA's MMA thread.
// Every mbarrier wait is bounded; a CTA that gives up leaves its partner to its own time limit.
// No TMA load uses cluster multicast.
#include "umma_utils.cuh"

namespace {
constexpr int BM = 128;          // token rows per CTA (256 per pair)
constexpr int BNH = 128;         // weight rows a CTA loads (256 per pair)
constexpr int BN = 256;          // columns of the accumulator
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int STAGE_A = BM * BK * 2, STAGE_B = BNH * BK * 2, STAGE = STAGE_A + STAGE_B;
constexpr int STAGES = 6;
constexpr int SMEM = STAGES * STAGE + 1024;
constexpr int TMEM_COLS = 512;

template <typename OutT> __device__ __forceinline__ OutT cast_out(float v);
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address of the same shared-memory variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives (once the MMAs issued so far are done) on the barrier at this address in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}

template <typename OutT, bool GATED>
__global__ void __launch_bounds__(THREADS, 1)
umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                      OutT* __restrict__ out, int M, int N, int K, int64_t ldo, int tiles_m, int num_items,
                      int* __restrict__ status) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], tmem_full_bar[2], tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                   // 0: the pair's first CTA (issues the MMAs)
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t tile_base = (smem_addr(smem_dyn) + 1023u) & ~1023u;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 2);              // one arrival (with its bytes) per CTA of the pair
      mbar_init(smem_addr(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&tmem_full_bar[b]), 1);
      mbar_init(smem_addr(&tmem_empty_bar[b]), 8);        // one arrival per epilogue warp of both CTAs
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The paired allocation is an operation of both CTAs: it must not start before the partner runs (the
  // two CTAs of a cluster may start microseconds apart when the kernel is scheduled early, while the
  // kernel before it still holds most of the GPU), so the cluster meets once before it and once after.
  __syncthreads();
  cluster_sync_all();                                     // both CTAs run, and their barriers exist
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                     // both CTAs hold their tensor memory before an MMA writes it
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  // The weight never depends on the kernel before this one: its first tiles are requested before the
  // dependency wait.  Tokens are read, and anything is written, after it.

  auto tile_of = [&](int w, int& row_x, int& row_w) {
    const int tn = w / tiles_m, tm = w - tn * tiles_m;    // neighbouring pairs share a weight tile
    row_x = tm * 2 * BM + (int)rank * BM;
    row_w = tn * BN + (int)rank * BNH;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      bool ok = true;
      // pass 0: the weight tiles of the first STAGES k-blocks; pass 1: their token tiles, then both
      // operands of every later block as stages come free
      for (int pass = 0; pass < 2 && ok; ++pass) {
        if (pass == 1) pdl_wait();
        uint32_t it = 0;
        bool more = true;
        for (int w = pair; w < num_items && ok && more; w += num_pairs) {
          int row_x, row_w;
          tile_of(w, row_x, row_w);
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const uint32_t s = it % STAGES, round = it / STAGES;
            const uint32_t bar = mapa(smem_addr(&full_bar[s]), 0);     // the first CTA's barrier
            const uint32_t dst = tile_base + s * STAGE;
            if (pass == 0) {
              if (round > 0) { more = false; break; }
              mbar_expect_tx_cluster(bar, (uint32_t)STAGE);
              tma_load_2d_pair(dst + STAGE_A, &map_w, kb * BK, row_w, bar);
            } else if (round == 0) {
              tma_load_2d_pair(dst, &map_x, kb * BK, row_x, bar);
            } else {
              ok = mbar_wait(smem_addr(&empty_bar[s]), (round & 1u) ^ 1u, status, &abort_flag);
              if (!ok) break;
              mbar_expect_tx_cluster(bar, (uint32_t)STAGE);
              tma_load_2d_pair(dst, &map_x, kb * BK, row_x, bar);
              tma_load_2d_pair(dst + STAGE_A, &map_w, kb * BK, row_w, bar);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (first CTA only)
    // The whole warp runs the loop with warp-uniform values and waits on the barriers; one elected thread
    // issues the products and their commits.
    if (rank == 0) {
      const bool leader = elect_one();
      auto wait_u = [&](uint64_t* bar, uint32_t parity) -> bool {
        const bool good = mbar_wait(smem_addr(bar), parity, status, &abort_flag);
        return __all_sync(0xffffffffu, good) != 0;
      };
      constexpr uint32_t idesc = umma_idesc(2 * BM, BN);
      uint32_t it = 0, n_used = 0;
      bool ok = true;
      for (int w = pair; w < num_items && ok; w += num_pairs) {
        const uint32_t acc = n_used & 1u;
        ok = wait_u(&tmem_empty_bar[acc], ((n_used >> 1) & 1u) ^ 1u);
        if (!ok) break;
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          ok = wait_u(&full_bar[s], (it / STAGES) & 1u);
          if (!ok) break;
          const uint64_t a_desc = umma_desc(tile_base + s * STAGE);
          const uint64_t b_desc = umma_desc(tile_base + s * STAGE + STAGE_A);
          if (leader) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_bf16_pair(tmem_d, a_desc + (uint64_t)((k * UMMA_K * 2) >> 4), b_desc + (uint64_t)((k * UMMA_K * 2) >> 4),
                             idesc, (kb > 0 || k > 0) ? 1u : 0u);
            umma_commit_pair(smem_addr(&empty_bar[s]));    // both CTAs' stages are free once these MMAs have read them
          }
          __syncwarp();
        }
        if (ok && leader) umma_commit_pair(smem_addr(&tmem_full_bar[acc]));
        __syncwarp();
        ++n_used;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    pdl_wait();                                           // nothing is written before the previous kernel is done
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    uint32_t n_used = 0;
    for (int w = pair; w < num_items; w += num_pairs) {
      int row_x, row_w;
      tile_of(w, row_x, row_w);
      const int col0 = row_w - (int)rank * BNH;            // the tile's first column
      const uint32_t acc = n_used & 1u;
      mbar_wait(smem_addr(&tmem_full_bar[acc]), (n_used >> 1) & 1u, status, &abort_flag);
      epilogue_sync();                                    // a warp that gave up has set abort_flag before this
      if (abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      const int m = row_x + row;
      if (GATED) {
        // this thread's token row holds, per 128 columns, 64 gates then their 64 ups
        const int n_out = N / 2;
#pragma unroll 1
        for (int c2 = 0; c2 < BN / 2; c2 += 16) {
          const int gate_col = (c2 / 64) * 128 + (c2 % 64);
          float g[16], u[16];
          tmem_ld16(taddr + (uint32_t)gate_col, g);
          tmem_ld16(taddr + (uint32_t)(gate_col + 64), u);
          const int f0 = col0 / 2 + c2;
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
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          tmem_ld16(taddr + (uint32_t)c, v);
          const int n0 = col0 + c;
          if (m < M && n0 < N) {
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
      // this warp is done reading the accumulator: hand it back to the first CTA's MMA thread
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(smem_addr(&tmem_empty_bar[acc]), 0));
      ++n_used;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  cluster_sync_all();                                     // neither CTA leaves, or frees tensor memory, while the other may still use it
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
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

template <typename OutT, bool GATED>
int pair_launch(const __nv_bfloat16* X, const __nv_bfloat16* W, OutT* out, int M, int N, int K, int64_t ldx,
                int64_t ldw, int64_t ldo, int* status, cudaStream_t stream) {
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, X, M, K, ldx, BM) || !make_map(&map_w, W, N, K, ldw, BNH)) return (int)cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(umma_gemm_pair_kernel<OutT, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
  const int num_items = tiles_m * tiles_n;
  const int pairs = num_items < sm_count() / 2 ? num_items : sm_count() / 2;
  return gllm_launch_cluster(umma_gemm_pair_kernel<OutT, GATED>, dim3(2 * pairs), dim3(THREADS), (size_t)SMEM, stream,
                             2u, map_x, map_w, out, M, N, K, ldo, tiles_m, num_items, status);
}
}  // namespace

// out_is_f32: 0 = bf16 output, 1 = fp32 output; gated != 0: W is [2*I, K] in blocks of 64 gate rows and
// the 64 up rows of the same features (N = 2*I, I % 64 == 0), out is [M, I] bf16.  Needs K % 8 == 0
// and 16-byte aligned rows of X and W.
GLLM_API int gllm_gemm_bf16_pair(const __nv_bfloat16* X, const __nv_bfloat16* W, void* out, int out_is_f32, int gated,
                                 int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int* status,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || (reinterpret_cast<uintptr_t>(X) & 15) ||
      (reinterpret_cast<uintptr_t>(W) & 15) || (gated && (out_is_f32 || N % 128)))
    return (int)cudaErrorInvalidValue;
  if (gated)
    return pair_launch<__nv_bfloat16, true>(X, W, (__nv_bfloat16*)out, M, N, K, ldx, ldw, ldo, status, stream);
  if (out_is_f32) return pair_launch<float, false>(X, W, (float*)out, M, N, K, ldx, ldw, ldo, status, stream);
  return pair_launch<__nv_bfloat16, false>(X, W, (__nv_bfloat16*)out, M, N, K, ldx, ldw, ldo, status, stream);
}
