// Fused multi-configuration replay step: one read of the logged gradient
// advances R replay configurations that share it.
//
//   replay_pass1   per configuration, the squared norm of the gradient it is
//                  about to commit (g + residual on a boundary, g * support
//                  otherwise), accumulated in fp64 with a fixed reduction
//                  order -> the clip coefficients
//   replay_pass3   per configuration: clip, residual update, Adam commit in
//                  the form w * (1 - lr * wd) - lr * u (AdamW or AdamS; on a
//                  dual-lr boundary w - (w * wd + u) * step with the lane's
//                  step size, the form of sga/replay.py:674-684), and at
//                  horizon steps the fp64 sum of (w - w_dense)^2
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
        float w1;
        if (c.dual && c.boundary) {
          // boundary dual lr: the whole displacement (decay term included) scales with the lane's step size
          const float step = sel ? c.lr : c.lr_inactive;
          const float full = w0 * wdi + u;
          w1 = w0 - full * step;
        } else {
          const float decay = 1.0f - c.lr * wdi;
          w1 = w0 * decay - c.lr * u;
        }
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


// ---- vector forms: four consecutive elements per thread (n % 4 == 0, 16-byte aligned rows) ----
// Every element sees the same fp32 operations in the same order as in the scalar kernels above;
// only the element -> thread mapping (and with it the order of the fp64 sums) differs. The state of
// configuration r + 1 is loaded before configuration r is stored, so a thread keeps two
// configurations' 68 bytes in flight; per-configuration fp64 sums sit in shared memory
// ([R][RP_THREADS] doubles), which keeps the register count independent of R.
struct RV4 {
  float4 res, m, v, w;
  uchar4 sel;
};

__device__ __forceinline__ RV4 rv4_load(const float* __restrict__ W, const float* __restrict__ M,
                                         const float* __restrict__ V, const float* __restrict__ RES,
                                         const uint8_t* __restrict__ SEL, long long o) {
  RV4 x;
  x.res = __ldcs(reinterpret_cast<const float4*>(RES + o));
  x.m = __ldcs(reinterpret_cast<const float4*>(M + o));
  x.v = __ldcs(reinterpret_cast<const float4*>(V + o));
  x.w = __ldcs(reinterpret_cast<const float4*>(W + o));
  x.sel = __ldcs(reinterpret_cast<const uchar4*>(SEL + o));
  return x;
}

template <typename GT>
__device__ __forceinline__ float4 load_g4(const GT* g, long long i);
template <>
__device__ __forceinline__ float4 load_g4<float>(const float* g, long long i) {
  return __ldcs(reinterpret_cast<const float4*>(g + i));
}
template <>
__device__ __forceinline__ float4 load_g4<__nv_bfloat16>(const __nv_bfloat16* g, long long i) {
  const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(g + i));
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y));
}

// block tree-reduction of sacc[r][*] into partials[r][block], r = 0..R-1
__device__ __forceinline__ void rv_block_reduce(double* sacc, double* red, int R, double* __restrict__ partials) {
  for (int r = 0; r < R; ++r) {
    red[threadIdx.x] = sacc[r * RP_THREADS + threadIdx.x];
    __syncthreads();
    for (int s = RP_THREADS / 2; s > 0; s >>= 1) {
      if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
      __syncthreads();
    }
    if (threadIdx.x == 0) partials[(long long)r * gridDim.x + blockIdx.x] = red[0];
    __syncthreads();
  }
}

template <typename GT>
__global__ void __launch_bounds__(RP_THREADS) replay_pass1_vec_kernel(const GT* __restrict__ gl, float coef_dense,
                                                                      const float* __restrict__ RES,
                                                                      const uint8_t* __restrict__ SEL,
                                                                      const ReplayCfg* __restrict__ cfgs, int R,
                                                                      long long n, double* __restrict__ partials) {
  extern __shared__ double sacc[];  // [R][RP_THREADS]
  __shared__ double red[RP_THREADS];
  __shared__ ReplayCfg sc[RP_MAXR];
  for (int r = threadIdx.x; r < R; r += RP_THREADS) sc[r] = cfgs[r];
  for (int r = 0; r < R; ++r) sacc[r * RP_THREADS + threadIdx.x] = 0.0;
  __syncthreads();
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * RP_THREADS;
  for (long long i4 = (long long)blockIdx.x * RP_THREADS + threadIdx.x; i4 < n4; i4 += stride) {
    const long long i = i4 << 2;
    float4 g = load_g4<GT>(gl, i);
    g.x = g.x / coef_dense, g.y = g.y / coef_dense, g.z = g.z / coef_dense, g.w = g.w / coef_dense;
    float4 res = __ldcs(reinterpret_cast<const float4*>(RES + i));
    uchar4 sel = __ldcs(reinterpret_cast<const uchar4*>(SEL + i));
    for (int r = 0; r < R; ++r) {
      float4 res_n = res;
      uchar4 sel_n = sel;
      if (r + 1 < R) {
        const long long o = (long long)(r + 1) * n + i;
        res_n = __ldcs(reinterpret_cast<const float4*>(RES + o));
        sel_n = __ldcs(reinterpret_cast<const uchar4*>(SEL + o));
      }
      const ReplayCfg& c = sc[r];
      const float q0 = q_pre_of(c, g.x, res.x, sel.x), q1 = q_pre_of(c, g.y, res.y, sel.y);
      const float q2 = q_pre_of(c, g.z, res.z, sel.z), q3 = q_pre_of(c, g.w, res.w, sel.w);
      double a = sacc[r * RP_THREADS + threadIdx.x];
      a += (double)q0 * (double)q0;
      a += (double)q1 * (double)q1;
      a += (double)q2 * (double)q2;
      a += (double)q3 * (double)q3;
      sacc[r * RP_THREADS + threadIdx.x] = a;
      res = res_n;
      sel = sel_n;
    }
  }
  rv_block_reduce(sacc, red, R, partials);
}

__device__ __forceinline__ void rv_lane(const ReplayCfg& c, float g, float wdi, float beta1, float omb1, float beta2,
                                        float omb2, float eps, float& res, float& m, float& v, float& w,
                                        uint8_t sel) {
  const float q = q_pre_of(c, g, res, sel) * c.coef;
  res = c.boundary ? 0.0f : res + (sel ? 0.0f : g);
  const float m0 = m, v0 = v, w0 = w;
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
  if (c.dual && c.boundary) {
    const float step = sel ? c.lr : c.lr_inactive;
    const float full = w0 * wdi + u;
    w = w0 - full * step;
  } else {
    const float decay = 1.0f - c.lr * wdi;
    w = w0 * decay - c.lr * u;
  }
  m = m1;
  v = v1;
}

template <typename GT, bool HORIZON>
__global__ void __launch_bounds__(RP_THREADS, 3) replay_pass3_vec_kernel(
    const GT* __restrict__ gl, float coef_dense, float* __restrict__ W, float* __restrict__ M, float* __restrict__ V,
    float* __restrict__ RES, const uint8_t* __restrict__ SEL, const float* __restrict__ wd,
    const float* __restrict__ w_dense, const ReplayCfg* __restrict__ cfgs, int R, long long n, float beta1,
    float omb1, float beta2, float omb2, float eps, double* __restrict__ partials) {
  extern __shared__ double sacc[];  // HORIZON: [R][RP_THREADS]
  __shared__ double red[RP_THREADS];
  __shared__ ReplayCfg sc[RP_MAXR];
  for (int r = threadIdx.x; r < R; r += RP_THREADS) sc[r] = cfgs[r];
  if (HORIZON)
    for (int r = 0; r < R; ++r) sacc[r * RP_THREADS + threadIdx.x] = 0.0;
  __syncthreads();
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * RP_THREADS;
  for (long long i4 = (long long)blockIdx.x * RP_THREADS + threadIdx.x; i4 < n4; i4 += stride) {
    const long long i = i4 << 2;
    float4 g = load_g4<GT>(gl, i);
    g.x = g.x / coef_dense, g.y = g.y / coef_dense, g.z = g.z / coef_dense, g.w = g.w / coef_dense;
    const float4 wd4 = __ldg(reinterpret_cast<const float4*>(wd + i));
    float4 wden = make_float4(0.f, 0.f, 0.f, 0.f);
    if (HORIZON) wden = __ldg(reinterpret_cast<const float4*>(w_dense + i));
    RV4 cur = rv4_load(W, M, V, RES, SEL, i);
    for (int r = 0; r < R; ++r) {
      RV4 nxt = cur;
      if (r + 1 < R) nxt = rv4_load(W, M, V, RES, SEL, (long long)(r + 1) * n + i);
      const ReplayCfg& c = sc[r];
      rv_lane(c, g.x, wd4.x, beta1, omb1, beta2, omb2, eps, cur.res.x, cur.m.x, cur.v.x, cur.w.x, cur.sel.x);
      rv_lane(c, g.y, wd4.y, beta1, omb1, beta2, omb2, eps, cur.res.y, cur.m.y, cur.v.y, cur.w.y, cur.sel.y);
      rv_lane(c, g.z, wd4.z, beta1, omb1, beta2, omb2, eps, cur.res.z, cur.m.z, cur.v.z, cur.w.z, cur.sel.z);
      rv_lane(c, g.w, wd4.w, beta1, omb1, beta2, omb2, eps, cur.res.w, cur.m.w, cur.v.w, cur.w.w, cur.sel.w);
      const long long o = (long long)r * n + i;
      __stcs(reinterpret_cast<float4*>(RES + o), cur.res);
      __stcs(reinterpret_cast<float4*>(W + o), cur.w);
      __stcs(reinterpret_cast<float4*>(M + o), cur.m);
      __stcs(reinterpret_cast<float4*>(V + o), cur.v);
      if (HORIZON && c.horizon) {
        double a = sacc[r * RP_THREADS + threadIdx.x];
        double d = (double)cur.w.x - (double)wden.x;
        a += d * d;
        d = (double)cur.w.y - (double)wden.y;
        a += d * d;
        d = (double)cur.w.z - (double)wden.z;
        a += d * d;
        d = (double)cur.w.w - (double)wden.w;
        a += d * d;
        sacc[r * RP_THREADS + threadIdx.x] = a;
      }
      cur = nxt;
    }
  }
  if (HORIZON) rv_block_reduce(sacc, red, R, partials);
}

__host__ inline bool rv_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace sga

using namespace sga;

// three resident blocks per SM (the vector commit kernel's register budget): one full wave
SGA_API int sga_replay_blocks() { return 148 * 3; }

// partials: [R * sga_replay_blocks()] doubles; out: [R] doubles.
SGA_API int sga_replay_pass1(const void* g, int g_is_bf16, float coef_dense, const float* RES, const uint8_t* SEL,
                             const void* cfgs, int R, long long n, double* partials, double* out, void* stream) {
  if (R < 1 || R > RP_MAXR) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nb = sga_replay_blocks();
  if (n % 4 == 0 && n > 0 && rv_aligned(g, 16) && rv_aligned(RES, 16) && rv_aligned(SEL, 4)) {
    const size_t sm = (size_t)R * RP_THREADS * sizeof(double);
    if (g_is_bf16) {
      cudaFuncSetAttribute(replay_pass1_vec_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
      replay_pass1_vec_kernel<__nv_bfloat16><<<nb, RP_THREADS, sm, st>>>((const __nv_bfloat16*)g, coef_dense, RES, SEL,
                                                                         (const ReplayCfg*)cfgs, R, n, partials);
    } else {
      cudaFuncSetAttribute(replay_pass1_vec_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
      replay_pass1_vec_kernel<float><<<nb, RP_THREADS, sm, st>>>((const float*)g, coef_dense, RES, SEL,
                                                                 (const ReplayCfg*)cfgs, R, n, partials);
    }
  } else if (g_is_bf16)
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
  const bool hz = partials != nullptr && w_dense != nullptr;
  if (n % 4 == 0 && n > 0 && (partials == nullptr || hz) && rv_aligned(g, 16) && rv_aligned(W, 16) &&
      rv_aligned(M, 16) && rv_aligned(V, 16) && rv_aligned(RES, 16) && rv_aligned(SEL, 4) && rv_aligned(wd, 16) &&
      rv_aligned(w_dense, 16)) {
    const size_t sm = hz ? (size_t)R * RP_THREADS * sizeof(double) : 0;
#define SGA_RP3(GT, HZ)                                                                                              \
  do {                                                                                                               \
    cudaFuncSetAttribute(replay_pass3_vec_kernel<GT, HZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);     \
    replay_pass3_vec_kernel<GT, HZ><<<nb, RP_THREADS, sm, st>>>((const GT*)g, coef_dense, W, M, V, RES, SEL, wd,     \
                                                                w_dense, (const ReplayCfg*)cfgs, R, n, beta1, omb1,  \
                                                                beta2, omb2, eps, partials);                         \
  } while (0)
    if (g_is_bf16) {
      if (hz) SGA_RP3(__nv_bfloat16, true); else SGA_RP3(__nv_bfloat16, false);
    } else {
      if (hz) SGA_RP3(float, true); else SGA_RP3(float, false);
    }
#undef SGA_RP3
  } else if (g_is_bf16)
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
