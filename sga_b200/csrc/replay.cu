// Fused multi-configuration replay step: one read of the logged gradient
// advances R replay configurations that share it.
//
//   replay_pass1   per configuration, the squared norm of the gradient it is
//                  about to commit (g + residual on a boundary, g * support
//                  otherwise), accumulated in fp64 with a fixed reduction
//                  order -> the clip coefficients
//   replay_pass3   per configuration: clip, residual update, Adam commit in
//                  the form w * (1 - lr * wd) - lr * u (AdamW or AdamS,
//                  optional boundary dual lr), and at horizon steps the fp64
//                  sum of (w - w_dense)^2
//
// State is laid out [R, n] per array. Compiled with -fmad=false and without
// fast-math: each fp32 operation rounds on its own, in the order of the
// PyTorch replay in sga_b200/replay/core.py, so one shard reproduces the
// per-configuration replay bit for bit.
//
// Replaces the per-config, per-chunk Triton launches of
// sga/replay_kernels.py:108-216 (_k_abs/_k_update/_k_coi/_k_adam) and the three
// Python passes of sga/replay_fused.py:1592-1963.
#include "common.cuh"

namespace sga {

struct ReplayCfg {
  int boundary, fold, dual, adams, horizon;
  float fold_div, coef, lr, lr_inactive, bc1, bc2;
};

constexpr int RP_THREADS = 256;
constexpr int RP_MAXR = 32;

template <typename GT>
__device__ __forceinline__ float load_g(const GT* g, long long i);
template <>
__device__ __forceinline__ float load_g<float>(const float* g, long long i) { return g[i]; }
template <>
__device__ __forceinline__ float load_g<__nv_bfloat16>(const __nv_bfloat16* g, long long i) {
  return __bfloat162float(g[i]);
}

__device__ __forceinline__ float q_pre_of(const ReplayCfg& c, float g, float res, uint8_t sel) {
  if (c.boundary) {
    const float r = c.fold ? res / c.fold_div : res;
    return g + r;
  }
  return sel ? g : 0.0f;
}

template <typename GT>
__global__ void __launch_bounds__(RP_THREADS) replay_pass1_kernel(const GT* __restrict__ gl, float coef_dense,
                                                                  const float* __restrict__ RES,
                                                                  const uint8_t* __restrict__ SEL,
                                                                  const ReplayCfg* __restrict__ cfgs, int R,
                                                                  long long n, double* __restrict__ partials) {
  __shared__ double red[RP_THREADS];
  __shared__ ReplayCfg sc[RP_MAXR];
  for (int r = threadIdx.x; r < R; r += RP_THREADS) sc[r] = cfgs[r];
  __syncthreads();
  double acc[RP_MAXR];
#pragma unroll
  for (int r = 0; r < RP_MAXR; ++r) acc[r] = 0.0;
  const long long stride = (long long)gridDim.x * RP_THREADS;
  for (long long i = (long long)blockIdx.x * RP_THREADS + threadIdx.x; i < n; i += stride) {
    const float g = load_g<GT>(gl, i) / coef_dense;
#pragma unroll
    for (int r = 0; r < RP_MAXR; ++r) {
      if (r < R) {
        const float q = q_pre_of(sc[r], g, RES[(long long)r * n + i], SEL[(long long)r * n + i]);
        acc[r] += (double)q * (double)q;
      }
    }
  }
  for (int r = 0; r < R; ++r) {
    red[threadIdx.x] = acc[r];
    __syncthreads();
    for (int s = RP_THREADS / 2; s > 0; s >>= 1) {
      if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
      __syncthreads();
    }
    if (threadIdx.x == 0) partials[(long long)r * gridDim.x + blockIdx.x] = red[0];
    __syncthreads();
  }
}

// out[r] = sum over blocks, in block order
__global__ void replay_reduce_kernel(const double* __restrict__ partials, int nblocks, int R, double* __restrict__ out) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  double t = 0.0;
  for (int b = 0; b < nblocks; ++b) t += partials[(long long)r * nblocks + b];
  out[r] = t;
}

template <typename GT>
__global__ void __launch_bounds__(RP_THREADS) replay_pass3_kernel(
    const GT* __restrict__ gl, float coef_dense, float* __restrict__ W, float* __restrict__ M, float* __restrict__ V,
    float* __restrict__ RES, const uint8_t* __restrict__ SEL, const float* __restrict__ wd,
    const float* __restrict__ w_dense, const ReplayCfg* __restrict__ cfgs, int R, long long n, float beta1,
    float omb1, float beta2, float omb2, float eps, double* __restrict__ partials) {
  __shared__ double red[RP_THREADS];
  __shared__ ReplayCfg sc[RP_MAXR];
  for (int r = threadIdx.x; r < R; r += RP_THREADS) sc[r] = cfgs[r];
  __syncthreads();
  double acc[RP_MAXR];
#pragma unroll
  for (int r = 0; r < RP_MAXR; ++r) acc[r] = 0.0;
  const long long stride = (long long)gridDim.x * RP_THREADS;
  for (long long i = (long long)blockIdx.x * RP_THREADS + threadIdx.x; i < n; i += stride) {
    const float g = load_g<GT>(gl, i) / coef_dense;
    const float wdi = wd[i];
    const float wden = w_dense ? w_dense[i] : 0.0f;
#pragma unroll
    for (int r = 0; r < RP_MAXR; ++r) {
      if (r < R) {
        const ReplayCfg c = sc[r];
        const long long o = (long long)r * n + i;
        const float res = RES[o];
        const uint8_t sel = SEL[o];
        const float q = q_pre_of(c, g, res, sel) * c.coef;
        RES[o] = c.boundary ? 0.0f : res + (sel ? 0.0f : g);
        const float m0 = M[o], v0 = V[o], w0 = W[o];
        const float m1 = m0 * beta1 + q * omb1;
        const float g2 = (q * omb2) * q;
        float v1, mh, vh;
        if (c.adams) {
          v1 = (m0 * m0) * beta2 + g2;
          mh = m1;
          vh = v1;
        } else {
          v1 = v0 * beta2 + g2;
          mh = m1 / c.bc1;
          vh = v1 / c.bc2;
        }
        const float u = mh / (sqrtf(vh) + eps);
        const float lr = (c.dual && c.boundary && !sel) ? c.lr_inactive : c.lr;
        const float decay = 1.0f - lr * wdi;
        const float w1 = w0 * decay - lr * u;
        W[o] = w1;
        M[o] = m1;
        V[o] = v1;
        if (c.horizon) {
          const double d = (double)w1 - (double)wden;
          acc[r] += d * d;
        }
      }
    }
  }
  if (!partials) return;
  for (int r = 0; r < R; ++r) {
    red[threadIdx.x] = acc[r];
    __syncthreads();
    for (int s = RP_THREADS / 2; s > 0; s >>= 1) {
      if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
      __syncthreads();
    }
    if (threadIdx.x == 0) partials[(long long)r * gridDim.x + blockIdx.x] = red[0];
    __syncthreads();
  }
}

}  // namespace sga

using namespace sga;

SGA_API int sga_replay_blocks() { return 148 * 4; }

// partials: [R * sga_replay_blocks()] doubles; out: [R] doubles.
SGA_API int sga_replay_pass1(const void* g, int g_is_bf16, float coef_dense, const float* RES, const uint8_t* SEL,
                             const void* cfgs, int R, long long n, double* partials, double* out, void* stream) {
  if (R < 1 || R > RP_MAXR) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nb = sga_replay_blocks();
  if (g_is_bf16)
    replay_pass1_kernel<__nv_bfloat16><<<nb, RP_THREADS, 0, st>>>((const __nv_bfloat16*)g, coef_dense, RES, SEL,
                                                                  (const ReplayCfg*)cfgs, R, n, partials);
  else
    replay_pass1_kernel<float><<<nb, RP_THREADS, 0, st>>>((const float*)g, coef_dense, RES, SEL,
                                                          (const ReplayCfg*)cfgs, R, n, partials);
  replay_reduce_kernel<<<1, 32, 0, st>>>(partials, nb, R, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

SGA_API int sga_replay_pass3(const void* g, int g_is_bf16, float coef_dense, float* W, float* M, float* V, float* RES,
                             const uint8_t* SEL, const float* wd, const float* w_dense, const void* cfgs, int R,
                             long long n, float beta1, float omb1, float beta2, float omb2, float eps,
                             double* partials, double* out, void* stream) {
  if (R < 1 || R > RP_MAXR) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nb = sga_replay_blocks();
  if (g_is_bf16)
    replay_pass3_kernel<__nv_bfloat16><<<nb, RP_THREADS, 0, st>>>((const __nv_bfloat16*)g, coef_dense, W, M, V, RES,
                                                                  SEL, wd, w_dense, (const ReplayCfg*)cfgs, R, n,
                                                                  beta1, omb1, beta2, omb2, eps, partials);
  else
    replay_pass3_kernel<float><<<nb, RP_THREADS, 0, st>>>((const float*)g, coef_dense, W, M, V, RES, SEL, wd, w_dense,
                                                          (const ReplayCfg*)cfgs, R, n, beta1, omb1, beta2, omb2, eps,
                                                          partials);
  if (partials && out) replay_reduce_kernel<<<1, 32, 0, st>>>(partials, nb, R, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
