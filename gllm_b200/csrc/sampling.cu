// Sampling from fp32 logits: greedy, temperature, top-k, top-p, log-probabilities.
//
// The semantics are the reference sampler's (gllm/sample/sampler.py:67-107):
//   z = logits / temperature; keep the top_k highest z (0 = whole vocabulary);
//   over those, in descending order, keep the entries whose cumulative softmax
//   probability is <= top_p and always the first (the entry that crosses top_p
//   is dropped); draw from the softmax of what is left; log-probabilities are
//   log_softmax of the RAW logits at the highest candidates, at most
//   min(max_num_logprobs, number of candidates) of them, in descending order.
// Added here: temperature == 0 or top_k == 1 is an exact argmax (the reference
// divides by zero at temperature 0); the draw uses a counter-based generator
// keyed by (seed, counter) of the row, so a request's tokens do not depend on
// what else is in the batch; the sampled token's own log-probability is
// returned as well.
//
// No sort: the k-th largest value and the top-p cut are found by a 3-pass
// radix selection over order-preserving 32-bit keys (11+11+10 bits) with
// shared-memory histograms of counts or of probability mass.  Entries equal
// to the k-th largest value are all kept; entries equal to the value at which
// the cumulative probability crosses top_p are all dropped.
//
// One block of 1024 threads per row.
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

namespace {
constexpr int THREADS = 1024;
constexpr int BINS = 2048;
constexpr int MAX_LOGPROBS = 32;
constexpr int LIST_MAX = 128;

__device__ __forceinline__ uint32_t to_key(float v) {
  uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Smem {
  uint32_t hist_count[BINS];
  float hist_mass[BINS];
  float scratch[32];
  int scratch_i[32];
  uint32_t bcast[4];
  float bcast_f[2];
  float list_val[LIST_MAX];
  int list_idx[LIST_MAX];
  int list_n;
};

__device__ float block_max_arg(float v, int idx, int* out_idx, Smem& s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if (lane == 0) { s.scratch[warp] = v; s.scratch_i[warp] = idx; }
  __syncthreads();
  float bv = s.scratch[0];
  int bi = s.scratch_i[0];
  for (int w = 1; w < THREADS / 32; ++w) {
    const float ov = s.scratch[w];
    const int oi = s.scratch_i[w];
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  *out_idx = bi;
  return bv;
}

// Philox4x32-10, one block of four words for (seed, counter).
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t counter) {
  uint32_t c0 = counter, c1 = 0u, c2 = 0x5eedu, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return (float)(c0 >> 8) * (1.0f / 16777216.0f);  // [0, 1)
}

// Scans the bins from the top with warp 0.  COUNT mode: finds the bin where the
// count from the top reaches `need`.  MASS mode: finds the bin whose inclusion
// first makes the mass from the top exceed `limit`.  Results in s.bcast:
// [0] = bin, [1] = found, and the amount above that bin in bcast[2] (count) or
// bcast_f[0] (mass).
template <bool MASS>
__device__ void scan_bins(Smem& s, int nbins, uint32_t need, float limit) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    uint32_t run_c = 0;
    float run_m = 0.f;
    bool found = false;
    for (int c = 0; c < nbins / 32 && !found; ++c) {
      const int bin = nbins - 1 - (c * 32 + lane);
      uint32_t vc = MASS ? 0u : s.hist_count[bin];
      float vm = MASS ? s.hist_mass[bin] : 0.f;
      uint32_t ic = vc;
      float im = vm;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t tc = __shfl_up_sync(0xffffffffu, ic, o);
        const float tm = __shfl_up_sync(0xffffffffu, im, o);
        if (lane >= o) { ic += tc; im += tm; }
      }
      const bool hit = MASS ? (run_m + im > limit && vm > 0.f) : (run_c + ic >= need);
      const uint32_t ballot = __ballot_sync(0xffffffffu, hit);
      if (ballot) {
        const int first = __ffs(ballot) - 1;
        if (lane == first) {
          s.bcast[0] = (uint32_t)bin;
          s.bcast[1] = 1u;
          s.bcast[2] = run_c + ic - vc;
          s.bcast_f[0] = run_m + im - vm;
        }
        found = true;
      } else {
        run_c += __shfl_sync(0xffffffffu, ic, 31);
        run_m += __shfl_sync(0xffffffffu, im, 31);
      }
    }
    if (!found && lane == 0) s.bcast[1] = 0u;
  }
  __syncthreads();
}

// Key of the k-th largest element (k >= 1, k <= V).
__device__ uint32_t select_kth(const float* x, int V, uint32_t k, Smem& s) {
  uint32_t prefix = 0, mask = 0, need = k;
  const int shifts[3] = {21, 10, 0}, bits[3] = {11, 11, 10};
  for (int p = 0; p < 3; ++p) {
    const int nb = 1 << bits[p];
    for (int i = threadIdx.x; i < nb; i += THREADS) s.hist_count[i] = 0;
    __syncthreads();
    for (int j = threadIdx.x; j < V; j += THREADS) {
      const uint32_t key = to_key(x[j]);
      if ((key & mask) == prefix) atomicAdd(&s.hist_count[(key >> shifts[p]) & (nb - 1)], 1u);
    }
    __syncthreads();
    scan_bins<false>(s, nb, need, 0.f);
    const uint32_t bin = s.bcast[0];
    need -= s.bcast[2];
    prefix |= bin << shifts[p];
    mask |= (uint32_t)(nb - 1) << shifts[p];
    __syncthreads();
  }
  return prefix;
}

// Largest key T such that the mass of {key >= key_floor and key >= T} exceeds
// `limit` (so {key > T} is the set whose cumulative mass stays <= limit).
// Returns false when even the whole set stays within the limit.
__device__ bool select_mass_cut(const float* x, int V, float xmax, float inv_t, uint32_t key_floor, float limit,
                                uint32_t* cut, Smem& s) {
  uint32_t prefix = 0, mask = 0;
  const int shifts[3] = {21, 10, 0}, bits[3] = {11, 11, 10};
  for (int p = 0; p < 3; ++p) {
    const int nb = 1 << bits[p];
    for (int i = threadIdx.x; i < nb; i += THREADS) s.hist_mass[i] = 0.f;
    __syncthreads();
    for (int j = threadIdx.x; j < V; j += THREADS) {
      const float v = x[j];
      const uint32_t key = to_key(v);
      if (key >= key_floor && (key & mask) == prefix)
        atomicAdd(&s.hist_mass[(key >> shifts[p]) & (nb - 1)], expf((v - xmax) * inv_t));
    }
    __syncthreads();
    scan_bins<true>(s, nb, 0u, limit);
    const bool found = s.bcast[1] != 0u;
    const uint32_t bin = s.bcast[0];
    const float above = s.bcast_f[0];
    __syncthreads();
    if (!found) {
      if (p == 0) return false;
      // rounding: the finer histogram sums to a hair less than the coarse bin did;
      // the crossing element is then the smallest key of this prefix
      *cut = prefix;
      return true;
    }
    limit -= above;
    prefix |= bin << shifts[p];
    mask |= (uint32_t)(nb - 1) << shifts[p];
  }
  *cut = prefix;
  return true;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int64_t row_stride, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const int64_t* __restrict__ seed,
              const int* __restrict__ counter, const int* __restrict__ n_logprobs, int lp_stride,
              int* __restrict__ out_token, float* __restrict__ out_logprob, int* __restrict__ out_ncand,
              float* __restrict__ out_top_lp, int* __restrict__ out_top_id, float* __restrict__ probs_out) {
  __shared__ Smem s;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const float* x = logits + (int64_t)row * row_stride;
  const int tid = threadIdx.x;

  // pass 1: maximum and its (lowest) index
  float vmax = -INFINITY;
  int imax = 0x7fffffff;
  for (int j = tid; j < V; j += THREADS) {
    const float v = x[j];
    if (v > vmax) { vmax = v; imax = j; }
  }
  int arg;
  const float xmax = block_max_arg(vmax, imax, &arg, s);
  // pass 2: log-sum-exp of the raw logits
  float se = 0.f;
  for (int j = tid; j < V; j += THREADS) se += expf(x[j] - xmax);
  const float log_z = xmax + logf(block_sum(se, s.scratch));

  const float temp = temperature ? temperature[row] : 0.f;
  const int k_in = top_k ? top_k[row] : 0;
  const float p_in = top_p ? top_p[row] : 1.f;
  const bool greedy = !(temp > 0.f) || k_in == 1;
  const uint32_t key_max = to_key(xmax);
  int token = arg;
  int ncand = 1;
  uint32_t key_cut = key_max;
  float inv_t = 1.f, z_kept = 1.f;

  if (!greedy) {
    inv_t = 1.0f / temp;
    const uint32_t k = (k_in <= 0 || k_in >= V) ? (uint32_t)V : (uint32_t)k_in;
    const uint32_t key_k = k < (uint32_t)V ? select_kth(x, V, k, s) : 0u;
    key_cut = key_k;
    if (p_in < 1.f) {
      float zk = 0.f;
      for (int j = tid; j < V; j += THREADS) {
        const float v = x[j];
        if (to_key(v) >= key_k) zk += expf((v - xmax) * inv_t);
      }
      zk = block_sum(zk, s.scratch);
      uint32_t cross;
      if (select_mass_cut(x, V, xmax, inv_t, key_k, p_in * zk, &cross, s)) {
        // everything above the crossing value is kept; the maximum always is
        key_cut = cross >= key_max ? key_max : max(key_k, cross + 1u);
      }
    }
    // mass and count of what is kept; per-thread contiguous chunks give an index-ordered prefix
    const int chunk = (V + THREADS - 1) / THREADS;
    const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
    float mine = 0.f;
    int cnt = 0;
    for (int j = lo; j < hi; ++j) {
      const float v = x[j];
      if (to_key(v) >= key_cut) { mine += expf((v - xmax) * inv_t); ++cnt; }
    }
    // inclusive scan over threads (warp scan, then warps in order)
    const int lane = tid & 31, warp = tid >> 5;
    float inc = mine;
    int inc_c = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, inc, o);
      const int tc = __shfl_up_sync(0xffffffffu, inc_c, o);
      if (lane >= o) { inc += t; inc_c += tc; }
    }
    __syncthreads();
    if (lane == 31) { s.scratch[warp] = inc; s.scratch_i[warp] = inc_c; }
    __syncthreads();
    float before = 0.f, total = 0.f;
    int total_c = 0;
    for (int w = 0; w < THREADS / 32; ++w) {
      if (w < warp) before += s.scratch[w];
      total += s.scratch[w];
      total_c += s.scratch_i[w];
    }
    z_kept = total;
    ncand = total_c;
    const float u = philox_uniform((uint64_t)(seed ? seed[row] : 0), (uint32_t)(counter ? counter[row] : 0));
    const float target = u * total;
    const float start = before + inc - mine;
    if (tid == 0) s.bcast[3] = 0xffffffffu;
    __syncthreads();
    if (cnt > 0 && target >= start && target < start + mine) {
      float run = start;
      int pick = -1;
      for (int j = lo; j < hi; ++j) {
        const float v = x[j];
        if (to_key(v) >= key_cut) {
          pick = j;
          run += expf((v - xmax) * inv_t);
          if (target < run) break;
        }
      }
      atomicMin(&s.bcast[3], (uint32_t)pick);
    }
    __syncthreads();
    // rounding can leave the target past the last chunk: take the maximum then
    token = s.bcast[3] == 0xffffffffu ? arg : (int)s.bcast[3];
  }

  if (probs_out) {
    float* po = probs_out + (int64_t)row * V;
    for (int j = tid; j < V; j += THREADS) {
      const float v = x[j];
      float p = 0.f;
      if (greedy) p = (j == arg) ? 1.f : 0.f;
      else if (to_key(v) >= key_cut) p = expf((v - xmax) * inv_t) / z_kept;
      po[j] = p;
    }
  }
  if (tid == 0) {
    out_token[row] = token;
    out_logprob[row] = x[token] - log_z;
    out_ncand[row] = ncand;
  }

  // log-probabilities of the highest candidates
  int n_lp = n_logprobs ? n_logprobs[row] : 0;
  n_lp = min(min(n_lp, ncand), min(MAX_LOGPROBS, lp_stride));
  if (n_lp > 0) {
    __syncthreads();
    const uint32_t key_n = select_kth(x, V, (uint32_t)n_lp, s);
    if (tid == 0) s.list_n = 0;
    __syncthreads();
    for (int j = tid; j < V; j += THREADS) {
      const float v = x[j];
      if (to_key(v) >= key_n) {
        const int slot = atomicAdd(&s.list_n, 1);
        if (slot < LIST_MAX) { s.list_val[slot] = v; s.list_idx[slot] = j; }
      }
    }
    __syncthreads();
    const int n_list = min(s.list_n, LIST_MAX);
    if (tid < n_list) {
      const float v = s.list_val[tid];
      const int id = s.list_idx[tid];
      int rank = 0;
      for (int o = 0; o < n_list; ++o) {
        const float ov = s.list_val[o];
        const int oi = s.list_idx[o];
        if (ov > v || (ov == v && oi < id)) ++rank;
      }
      if (rank < n_lp) {
        out_top_lp[(int64_t)row * lp_stride + rank] = v - log_z;
        out_top_id[(int64_t)row * lp_stride + rank] = id;
      }
    }
  }
}

// A cluster of ARGMAX_CLUSTER blocks shares one row (a row of a large vocabulary read through one
// SM's port takes longer than the rest of a decode step's tail): each block takes a stretch of the
// row, pushes its (maximum, index) into every block's shared memory, and after one cluster barrier
// rank 0 picks the winner (the lowest index among equal maxima, as a single block would).
constexpr int ARGMAX_CLUSTER = 8;
__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int64_t row_stride, int V, int* __restrict__ out_token,
              const int* __restrict__ out_index) {
  __shared__ Smem s;
  __shared__ float peer_v[ARGMAX_CLUSTER];
  __shared__ int peer_i[ARGMAX_CLUSTER];
  pdl_trigger();
  cluster_arrive_started();
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank(), n_ranks = (int)cluster.num_blocks();
  const int row = blockIdx.y;
  const int per = (V + n_ranks - 1) / n_ranks;
  const int j0 = rank * per, j1 = min(V, j0 + per);
  pdl_wait();
  const float* x = logits + (int64_t)row * row_stride;
  float vmax = -INFINITY;
  int imax = 0x7fffffff;
  for (int j = j0 + threadIdx.x; j < j1; j += THREADS) {
    const float v = x[j];
    if (v > vmax) { vmax = v; imax = j; }
  }
  int arg;
  const float best = block_max_arg(vmax, imax, &arg, s);
  cluster_wait_started();
  if (threadIdx.x == 0) {
    *cluster.map_shared_rank(&peer_v[rank], 0) = best;
    *cluster.map_shared_rank(&peer_i[rank], 0) = arg;
  }
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    float bv = peer_v[0];
    int bi = peer_i[0];
    for (int r = 1; r < n_ranks; ++r)
      if (peer_v[r] > bv || (peer_v[r] == bv && peer_i[r] < bi)) { bv = peer_v[r]; bi = peer_i[r]; }
    out_token[out_index ? out_index[row] : row] = bi;
  }
}
}  // namespace

GLLM_API int gllm_sample(const float* logits, int64_t row_stride, int rows, int V, const float* temperature,
                         const int* top_k, const float* top_p, const int64_t* seed, const int* counter,
                         const int* n_logprobs, int lp_stride, int* out_token, float* out_logprob,
                         int* out_ncand, float* out_top_lp, int* out_top_id, float* probs_out,
                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return (int)cudaErrorInvalidValue;
  return gllm_launch(sample_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, row_stride, V, temperature, top_k,
                     top_p, seed, counter, n_logprobs, lp_stride, out_token, out_logprob, out_ncand, out_top_lp,
                     out_top_id, probs_out);
}

// out_index (optional): row r's result goes to out_token[out_index[r]] instead of out_token[r].
GLLM_API int gllm_argmax(const float* logits, int64_t row_stride, int rows, int V, int* out_token,
                         const int* out_index, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return (int)cudaErrorInvalidValue;
  return gllm_launch_cluster(argmax_kernel, dim3(ARGMAX_CLUSTER, rows), dim3(THREADS), 0, stream,
                             (unsigned)ARGMAX_CLUSTER, logits, row_stride, V, out_token, out_index);
}
