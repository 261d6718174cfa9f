// Device side of the replay engine's boundary reselection: the registry score
// of every configuration that reselects at this step, and the exact
// distributed top-k over it, without a host round trip.
//
//   replay_score      fp32 score of one configuration on its pre-commit state
//                     (computed in fp64 in the operation order of the PyTorch
//                     score registry, stored as fp32, so selections are the
//                     bits the per-configuration replay would choose)
//   find_bin          after the shards' histograms have been summed: the
//                     crossing bin of the high 16 key bits (stage 0), then the
//                     exact k-th key, the number of ties to take and whether
//                     all ties are taken (stage 1)
//   hist_low16_dev    the low-digit histogram with the crossing bin read from
//                     device memory
//   mask / tie_scan / tie_fill
//                     support mask = keys above the threshold; ties at the
//                     threshold are filled in global index order: shards are
//                     contiguous and ordered by rank, so a shard takes
//                     need - (ties on lower ranks) of its own, lowest index first
//
// Only the two histograms and one tie count per configuration cross ranks
// (the host enqueues one collective for all configurations of a boundary);
// every decision between the passes is taken here.
//
// Replaces sga/replay_kernels.py:114-160 (_k_update, _k_coi), :218-267 (_k_hist,
// _k_cand_count, _k_cand_fill, _k_gt_eq) and the host-driven shard_select of
// sga/replay_fused.py:290-402. Compiled without fast-math and FMA contraction.
#include "common.cuh"

namespace sga {

struct RSCfg {  // same layout as ReplayCfg in replay.cu
  int boundary, fold, dual, adams, horizon;
  float fold_div, coef, lr, lr_inactive, bc1, bc2;
};

// per configuration, int64 words
enum { RS_BIN = 0, RS_ABOVE, RS_T, RS_NEED, RS_EQ, RS_ALL, RS_TIES, RS_K, RS_WORDS };

constexpr int RS_THREADS = 256;
constexpr int RS_ITEMS = 16;
constexpr int RS_TILE = RS_THREADS * RS_ITEMS;  // elements per tie-count block

template <typename GT>
__device__ __forceinline__ float rs_load(const GT* g, long long i);
template <>
__device__ __forceinline__ float rs_load<float>(const float* g, long long i) { return g[i]; }
template <>
__device__ __forceinline__ float rs_load<__nv_bfloat16>(const __nv_bfloat16* g, long long i) {
  return __bfloat162float(g[i]);
}

__device__ __forceinline__ uint32_t rs_key(float x) { return __float_as_uint(x) & 0x7FFFFFFFu; }

// code: 0 update, 1 abs_g, 2 abs_m, 3 coi (EMIT_CODES of the score registry), 4 |step gradient| (replay only)
template <typename GT>
__global__ void __launch_bounds__(RS_THREADS) replay_score_kernel(
    const GT* __restrict__ gl, float coef_dense, const float* __restrict__ W, const float* __restrict__ M,
    const float* __restrict__ V, const float* __restrict__ RES, const uint8_t* __restrict__ SEL,
    const float* __restrict__ wd, const RSCfg* __restrict__ cfg, int code, double beta1, double beta2, double eps,
    double bc1, double bc2, long long n, float* __restrict__ out) {
  const RSCfg c = *cfg;
  const double omb1 = 1.0 - beta1, omb2 = 1.0 - beta2;
  const long long stride = (long long)gridDim.x * RS_THREADS;
  for (long long i = (long long)blockIdx.x * RS_THREADS + threadIdx.x; i < n; i += stride) {
    const float g = rs_load<GT>(gl, i) / coef_dense;
    float qp;
    if (c.boundary) {
      const float res = RES[i];
      qp = g + (c.fold ? res / c.fold_div : res);
    } else {
      qp = SEL[i] ? g : 0.0f;
    }
    const float q32 = qp * c.coef;
    float sc;
    if (code == 4) {
      sc = fabsf(g);
    } else if (code == 1) {
      sc = fabsf(q32);
    } else if (code == 2) {
      sc = fabsf(M[i]);
    } else {
      const double q = (double)q32, m = (double)M[i], v = (double)V[i];
      const double m1 = m * beta1 + q * omb1;
      const double g2 = (q * omb2) * q;
      double mh, vh;
      if (c.adams) {
        mh = m1;
        vh = (m * m) * beta2 + g2;
      } else {
        mh = bc1 == 1.0 ? m1 : m1 / bc1;
        const double v1 = v * beta2 + g2;
        vh = bc2 == 1.0 ? v1 : v1 / bc2;
      }
      const double u = mh / (sqrt(vh) + eps);
      if (code == 0) {
        sc = (float)((double)wd[i] * (double)W[i] + u);
      } else {
        double u0;
        if (c.adams) {
          u0 = (m * beta1) / (sqrt((m * m) * beta2) + eps);
        } else {
          const double a = m * beta1, b = v * beta2;
          u0 = (bc1 == 1.0 ? a : a / bc1) / (sqrt(bc2 == 1.0 ? b : b / bc2) + eps);
        }
        sc = (float)fabs(u - u0);
      }
    }
    out[i] = sc;
  }
}

// One CTA per configuration. Thread t owns a contiguous run of bins, highest first; a block scan of
// the runs' sums finds the run in which the suffix count reaches `want`, and its owner walks it.
__global__ void __launch_bounds__(RS_THREADS) replay_find_bin_kernel(const long long* __restrict__ hist, int nb,
                                                                     long long* __restrict__ state, int stage) {
  __shared__ long long sh[RS_THREADS];
  __shared__ long long res[2];
  const long long* h = hist + (long long)blockIdx.x * nb;
  long long* st = state + (long long)blockIdx.x * RS_WORDS;
  const long long want = stage == 0 ? st[RS_K] : st[RS_K] - st[RS_ABOVE];
  const int per = (nb + RS_THREADS - 1) / RS_THREADS;
  const int hi = nb - (int)threadIdx.x * per;
  const int lo = max(0, hi - per);
  long long mysum = 0;
  for (int i = hi - 1; i >= lo; --i) mysum += h[i];
  sh[threadIdx.x] = mysum;
  if (threadIdx.x == 0) { res[0] = -1; res[1] = 0; }
  __syncthreads();
  long long before = 0;
  for (int t = 0; t < (int)threadIdx.x; ++t) before += sh[t];
  if (hi > 0 && before < want && before + mysum >= want) {
    long long run = before;
    for (int i = hi - 1; i >= lo; --i) {
      if (run + h[i] >= want) { res[0] = i; res[1] = run; break; }
      run += h[i];
    }
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  // fewer scored elements than k cannot happen (k <= n); guard anyway: select everything
  const long long bin = res[0] < 0 ? 0 : res[0];
  if (stage == 0) {
    st[RS_BIN] = bin;
    st[RS_ABOVE] = res[1];
  } else {
    const long long n_gt = st[RS_ABOVE] + res[1];
    const long long need = st[RS_K] - n_gt;
    const long long eq = h[bin];
    st[RS_T] = (st[RS_BIN] << 16) | bin;
    st[RS_ABOVE] = n_gt;
    st[RS_NEED] = need;
    st[RS_EQ] = eq;
    st[RS_ALL] = need >= eq ? 1 : 0;
    st[RS_TIES] = 0;
  }
}

__global__ void __launch_bounds__(512) replay_hist_low16_dev_kernel(const float* __restrict__ x, long long n,
                                                                    const long long* __restrict__ state,
                                                                    long long* __restrict__ hist) {
  extern __shared__ uint32_t shh[];  // one half (32768 counters) per blockIdx.y
  const uint32_t half = blockIdx.y;
  const int bin = (int)state[RS_BIN];
  for (int i = threadIdx.x; i < 32768; i += blockDim.x) shh[i] = 0;
  __syncthreads();
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x; s < n; s += gstride) {
    const uint32_t b = rs_key(x[s]);
    if ((int)(b >> 16) == bin && ((b >> 15) & 1u) == half) atomicAdd(&shh[b & 0x7FFFu], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 32768; i += blockDim.x) {
    const uint32_t c = shh[i];
    if (c) atomicAdd(reinterpret_cast<unsigned long long*>(hist + half * 32768 + i), (unsigned long long)c);
  }
}

// sel = key > T, or key >= T when every tie is taken; otherwise also the number of ties per 4096-element block.
__global__ void __launch_bounds__(RS_THREADS) replay_mask_kernel(const float* __restrict__ x, long long n,
                                                                 const long long* __restrict__ state,
                                                                 uint8_t* __restrict__ sel, int* __restrict__ blockcnt) {
  __shared__ int red[RS_THREADS];
  const uint32_t T = (uint32_t)state[RS_T];
  const bool all = state[RS_ALL] != 0;
  const long long nblk = (n + RS_TILE - 1) / RS_TILE;
  for (long long b = blockIdx.x; b < nblk; b += gridDim.x) {
    const long long base = b * RS_TILE + (long long)threadIdx.x * RS_ITEMS;
    int ties = 0;
#pragma unroll
    for (int j = 0; j < RS_ITEMS; ++j) {
      const long long i = base + j;
      if (i < n) {
        const uint32_t k = rs_key(x[i]);
        sel[i] = (k > T || (all && k == T)) ? 1 : 0;
        ties += k == T;
      }
    }
    if (!all) {
      red[threadIdx.x] = ties;
      __syncthreads();
      for (int s = RS_THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
      }
      if (threadIdx.x == 0) blockcnt[b] = red[0];
      __syncthreads();
    }
  }
}

// Exclusive scan of the per-block tie counts in place (one CTA); the shard's tie total goes to the state.
__global__ void __launch_bounds__(RS_THREADS) replay_tie_scan_kernel(int* __restrict__ blockcnt, long long nblk,
                                                                     long long* __restrict__ state) {
  __shared__ long long sh[RS_THREADS];
  if (state[RS_ALL] != 0) {
    if (threadIdx.x == 0) state[RS_TIES] = 0;
    return;
  }
  const long long per = (nblk + RS_THREADS - 1) / RS_THREADS;
  const long long lo = min(nblk, (long long)threadIdx.x * per), hi = min(nblk, lo + per);
  long long mysum = 0;
  for (long long i = lo; i < hi; ++i) mysum += blockcnt[i];
  sh[threadIdx.x] = mysum;
  __syncthreads();
  long long run = 0;
  for (int t = 0; t < (int)threadIdx.x; ++t) run += sh[t];
  for (long long i = lo; i < hi; ++i) {
    const int c = blockcnt[i];
    blockcnt[i] = (int)run;
    run += c;
  }
  if (threadIdx.x == RS_THREADS - 1) state[RS_TIES] = run;
}

// totals: [W][Rb] tie totals of every shard (all-gathered); this shard takes the first
// need - (ties of lower ranks) of its own ties, in index order.
__global__ void __launch_bounds__(RS_THREADS) replay_tie_fill_kernel(const float* __restrict__ x, long long n,
                                                                     const long long* __restrict__ state,
                                                                     const int* __restrict__ blockoff,
                                                                     const long long* __restrict__ totals, int rank,
                                                                     int Rb, int r, uint8_t* __restrict__ sel) {
  __shared__ int sh[RS_THREADS];
  if (state[RS_ALL] != 0) return;
  const uint32_t T = (uint32_t)state[RS_T];
  long long before = 0;
  for (int s = 0; s < rank; ++s) before += totals[(long long)s * Rb + r];
  const long long take = max(0LL, min(state[RS_TIES], state[RS_NEED] - before));
  if (take <= 0) return;
  const long long nblk = (n + RS_TILE - 1) / RS_TILE;
  for (long long b = blockIdx.x; b < nblk; b += gridDim.x) {
    const long long off = blockoff[b];
    if (off >= take) break;  // later blocks only hold later ties
    const long long base = b * RS_TILE + (long long)threadIdx.x * RS_ITEMS;
    int mine = 0;
    uint32_t bits = 0;
#pragma unroll
    for (int j = 0; j < RS_ITEMS; ++j) {
      const long long i = base + j;
      if (i < n && rs_key(x[i]) == T) { bits |= 1u << j; ++mine; }
    }
    sh[threadIdx.x] = mine;
    __syncthreads();
    long long rankv = off;
    for (int t = 0; t < (int)threadIdx.x; ++t) rankv += sh[t];
    __syncthreads();
    for (int j = 0; j < RS_ITEMS; ++j)
      if (bits & (1u << j)) {
        if (rankv < take) sel[base + j] = 1;
        ++rankv;
      }
  }
}

static inline int rs_grid(long long n, int per_block) {
  long long g = (n + per_block - 1) / per_block;
  if (g > 148 * 8) g = 148 * 8;
  return g < 1 ? 1 : (int)g;
}

}  // namespace sga

using namespace sga;

SGA_API int sga_replay_score(const void* g, int g_is_bf16, float coef_dense, const float* W, const float* M,
                             const float* V, const float* RES, const uint8_t* SEL, const float* wd, const void* cfg,
                             int code, double beta1, double beta2, double eps, double bc1, double bc2, long long n,
                             float* out, void* stream) {
  if (n <= 0) return 0;
  if (code < 0 || code > 4) return -6;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = rs_grid(n, RS_THREADS * 4);
  if (g_is_bf16)
    replay_score_kernel<__nv_bfloat16><<<grid, RS_THREADS, 0, st>>>((const __nv_bfloat16*)g, coef_dense, W, M, V, RES,
                                                                    SEL, wd, (const RSCfg*)cfg, code, beta1, beta2, eps,
                                                                    bc1, bc2, n, out);
  else
    replay_score_kernel<float><<<grid, RS_THREADS, 0, st>>>((const float*)g, coef_dense, W, M, V, RES, SEL, wd,
                                                            (const RSCfg*)cfg, code, beta1, beta2, eps, bc1, bc2, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// hist: [Rb][nb] int64 (already summed over the shards); state: [Rb][8] int64 with the budget k at word 7.
SGA_API int sga_replay_find_bin(const long long* hist, int nb, long long* state, int stage, int Rb, void* stream) {
  if (Rb < 1) return 0;
  replay_find_bin_kernel<<<Rb, RS_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(hist, nb, state, stage);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

SGA_API int sga_replay_hist_low16(const float* x, long long n, const long long* state, long long* hist, void* stream) {
  if (n <= 0) return 0;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(replay_hist_low16_dev_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4) !=
        cudaSuccess)
      return -3;
    attr = true;
  }
  dim3 grid(rs_grid(n, 512 * 16) > 148 ? 148 : rs_grid(n, 512 * 16), 2);
  replay_hist_low16_dev_kernel<<<grid, 512, 32768 * 4, reinterpret_cast<cudaStream_t>(stream)>>>(x, n, state, hist);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// blockcnt: ceil(n / 4096) ints of scratch per configuration.
SGA_API int sga_replay_mask(const float* x, long long n, const long long* state, uint8_t* sel, int* blockcnt,
                            void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  replay_mask_kernel<<<rs_grid(n, RS_TILE), RS_THREADS, 0, st>>>(x, n, state, sel, blockcnt);
  replay_tie_scan_kernel<<<1, RS_THREADS, 0, st>>>(blockcnt, (n + RS_TILE - 1) / RS_TILE, const_cast<long long*>(state));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

SGA_API int sga_replay_tie_fill(const float* x, long long n, const long long* state, const int* blockoff,
                                const long long* totals, int rank, int Rb, int r, uint8_t* sel, void* stream) {
  if (n <= 0) return 0;
  replay_tie_fill_kernel<<<rs_grid(n, RS_TILE), RS_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      x, n, state, blockoff, totals, rank, Rb, r, sel);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
