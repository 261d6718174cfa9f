// Residual-aware Adam step over a flat fp32 arena: one launch covers every
// parameter ("multi-tensor"), each parameter being a segment of the arena with
// a hyper-parameter group id. All variants of the reference's per-parameter
// Triton kernel are run-time switches of this one kernel:
//
//   mask        uint8 support mask; on a sparse step masked-out lanes see g = 0
//   emit        full step: which score is written into the grad buffer
//               (-1 none, 0 update, 1 abs_g, 2 abs_m, 3 coi)
//   coeff       clip coefficient read from device memory, multiplied into g at
//               active lanes (no host round trip)
//   clear       active lanes of the grad buffer <- 0 after use
//   fold        grad buffer /= interval after the clear (residual mean)
//   lr_split    full-step dual lr: lanes outside the mask use lr * scale
//   adams       v = beta2 * m_old^2 + (1 - beta2) g^2, no bias correction
//   model       bf16 copy of the updated parameter written in the same pass
//
// The file is compiled without fast-math and with -fmad=false: every fp32
// operation is individually rounded in the order of the PyTorch reference
// (sga_b200/plugins/optimizer/reference.py), so results match it bit for bit.
//
// Replaces sga/plugins/optimizer/adamw.py:87-213 (_grad_correct_kernel),
// adams.py:86-202 and the separate fp32 -> bf16 parameter copy.
#include "common.cuh"

namespace sga {

struct AdamGroup {
  float lr;
  float wd;
};

struct AdamArgs {
  float* w;
  float* g;
  float* m;
  float* v;
  __nv_bfloat16* model;        // nullable
  const uint8_t* mask;         // nullable
  const float* coeff;          // nullable (device scalar)
  const long long* seg_start;  // [nseg + 1], ascending, seg_start[nseg] = n
  const int* seg_group;        // [nseg]
  int nseg;
  long long n;
  AdamGroup groups[8];
  float beta1, omb1, beta2, omb2, bc1, bc2, eps;
  float interval, lr_scale;
  int emit, clear, fold, lr_split, adams, use_coeff;
};

constexpr int ADAM_THREADS = 256;
constexpr int ADAM_VEC = 4;
constexpr int ADAM_CHUNK = ADAM_THREADS * ADAM_VEC * 4;  // 4096 elements per CTA iteration

__global__ void __launch_bounds__(ADAM_THREADS) sga_adam_kernel(const AdamArgs a) {
  __shared__ int s_seg;
  const float coeff = (a.use_coeff && a.coeff) ? *a.coeff : 1.0f;
  const bool do_coeff = a.use_coeff && coeff != 1.0f;
  for (long long base = (long long)blockIdx.x * ADAM_CHUNK; base < a.n; base += (long long)gridDim.x * ADAM_CHUNK) {
    if (threadIdx.x == 0) {
      int lo = 0, hi = a.nseg - 1;  // last segment whose start <= base
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (a.seg_start[mid] <= base) lo = mid; else hi = mid - 1;
      }
      s_seg = lo;
    }
    __syncthreads();
    int seg = s_seg;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const long long i = base + ((long long)it * ADAM_THREADS + threadIdx.x) * ADAM_VEC;
      if (i >= a.n) break;
      while (seg + 1 < a.nseg && a.seg_start[seg + 1] <= i) ++seg;
      const AdamGroup grp = a.groups[a.seg_group[seg]];
      float wv[4], gv[4], mv[4], vv[4];
      uint8_t mk[4] = {1, 1, 1, 1};
      const bool vec = (i + ADAM_VEC <= a.n);
      if (vec) {
        *reinterpret_cast<float4*>(wv) = *reinterpret_cast<const float4*>(a.w + i);
        *reinterpret_cast<float4*>(gv) = *reinterpret_cast<const float4*>(a.g + i);
        *reinterpret_cast<float4*>(mv) = *reinterpret_cast<const float4*>(a.m + i);
        *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(a.v + i);
        if (a.mask) *reinterpret_cast<uchar4*>(mk) = *reinterpret_cast<const uchar4*>(a.mask + i);
      } else {
        for (int j = 0; j < 4; ++j) {
          const bool ok = i + j < a.n;
          wv[j] = ok ? a.w[i + j] : 0.f;
          gv[j] = ok ? a.g[i + j] : 0.f;
          mv[j] = ok ? a.m[i + j] : 0.f;
          vv[j] = ok ? a.v[i + j] : 0.f;
          if (a.mask) mk[j] = ok ? a.mask[i + j] : 0;
        }
      }
      float gout[4];
      __nv_bfloat16 bout[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool active = mk[j] != 0;
        float g = gv[j];
        float lr = grp.lr;
        if (a.lr_split) {
          if (!active) lr = grp.lr * a.lr_scale;
        } else if (a.mask && !active) {
          g = 0.f;
        }
        if (do_coeff && (active || a.lr_split)) g = g * coeff;  // the dual-lr boundary commits every lane
        const float m0 = mv[j], v0 = vv[j], w0 = wv[j];
        const float m1 = m0 * a.beta1 + g * a.omb1;
        const float g2 = (g * a.omb2) * g;
        float v1, mh, vh;
        if (a.adams) {
          v1 = (m0 * m0) * a.beta2 + g2;
          mh = m1;
          vh = v1;
        } else {
          v1 = v0 * a.beta2 + g2;
          mh = m1 / a.bc1;
          vh = v1 / a.bc2;
        }
        const float u = mh / (sqrtf(vh) + a.eps);
        const float update = grp.wd * w0 + u;
        const float w1 = w0 - lr * update;
        float go = gv[j];
        if (a.emit >= 0) {
          if (a.emit == 0) go = update;
          else if (a.emit == 1) go = fabsf(g);
          else if (a.emit == 2) go = fabsf(m0);
          else {
            float u0;
            if (a.adams) u0 = (m0 * a.beta1) / (sqrtf((m0 * m0) * a.beta2) + a.eps);
            else u0 = ((m0 * a.beta1) / a.bc1) / (sqrtf((v0 * a.beta2) / a.bc2) + a.eps);
            go = fabsf(u - u0);
          }
        } else {
          if (a.clear && active) go = 0.f;
          if (a.fold) go = go / a.interval;
        }
        mv[j] = m1;
        vv[j] = v1;
        wv[j] = w1;
        gout[j] = go;
        bout[j] = __float2bfloat16_rn(w1);
      }
      const bool write_g = (a.emit >= 0) || a.clear || a.fold;
      if (vec) {
        *reinterpret_cast<float4*>(a.w + i) = *reinterpret_cast<float4*>(wv);
        *reinterpret_cast<float4*>(a.m + i) = *reinterpret_cast<float4*>(mv);
        *reinterpret_cast<float4*>(a.v + i) = *reinterpret_cast<float4*>(vv);
        if (write_g) *reinterpret_cast<float4*>(a.g + i) = *reinterpret_cast<float4*>(gout);
        if (a.model) *reinterpret_cast<uint2*>(a.model + i) = *reinterpret_cast<uint2*>(bout);
      } else {
        for (int j = 0; j < 4 && i + j < a.n; ++j) {
          a.w[i + j] = wv[j];
          a.m[i + j] = mv[j];
          a.v[i + j] = vv[j];
          if (write_g) a.g[i + j] = gout[j];
          if (a.model) a.model[i + j] = bout[j];
        }
      }
    }
    __syncthreads();
  }
}

// Deterministic sum of squares: fixed grid, fixed per-thread order, block tree,
// partials[gridDim.x] written to global; a second tiny kernel sums partials in
// index order. With a mask only active lanes count.
constexpr int NORM_THREADS = 256;

__global__ void __launch_bounds__(NORM_THREADS) sga_sumsq_stage1(const float* __restrict__ x,
                                                                 const uint8_t* __restrict__ mask, long long n,
                                                                 float* __restrict__ partials) {
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * NORM_THREADS * 4;
  for (long long i = ((long long)blockIdx.x * NORM_THREADS + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      const float4 xv = *reinterpret_cast<const float4*>(x + i);
      float a0 = xv.x, a1 = xv.y, a2 = xv.z, a3 = xv.w;
      if (mask) {
        const uchar4 mk = *reinterpret_cast<const uchar4*>(mask + i);
        if (!mk.x) a0 = 0.f;
        if (!mk.y) a1 = 0.f;
        if (!mk.z) a2 = 0.f;
        if (!mk.w) a3 = 0.f;
      }
      acc = acc + a0 * a0;
      acc = acc + a1 * a1;
      acc = acc + a2 * a2;
      acc = acc + a3 * a3;
    } else {
      for (long long j = i; j < n; ++j) {
        float a0 = x[j];
        if (mask && !mask[j]) a0 = 0.f;
        acc = acc + a0 * a0;
      }
    }
  }
  __shared__ float red[NORM_THREADS];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = NORM_THREADS / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] = red[threadIdx.x] + red[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) partials[blockIdx.x] = red[0];
}

// out[0] (+)= sum(partials[0..np)) in index order (single thread block).
__global__ void sga_sumsq_stage2(const float* __restrict__ partials, int np, float* out, int accumulate) {
  __shared__ float red[256];
  float acc = 0.f;
  for (int i = threadIdx.x; i < np; i += 256) acc = acc + partials[i];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] = red[threadIdx.x] + red[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + red[0] : red[0];
}

// coeff[0] = min(1, clip / (sqrt(sumsq * inv_world) + 1e-6)); norm_out[0] = the norm.
__global__ void sga_clip_coeff_kernel(const float* sumsq, float inv_world, float clip, float* coeff, float* norm_out) {
  const float norm = sqrtf(sumsq[0] * inv_world);
  norm_out[0] = norm;
  float c = 1.0f;
  if (clip > 0.f) {
    const float r = clip / (norm + 1e-6f);
    if (r < 1.0f) c = r;
  }
  coeff[0] = c;
}

__global__ void sga_scale_kernel(float* x, long long n, const float* coeff_ptr, float factor) {
  const float c = (coeff_ptr ? *coeff_ptr : 1.0f) * factor;
  if (c == 1.0f) return;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 v = *reinterpret_cast<float4*>(x + i);
      v.x = v.x * c; v.y = v.y * c; v.z = v.z * c; v.w = v.w * c;
      *reinterpret_cast<float4*>(x + i) = v;
    } else {
      for (long long j = i; j < n; ++j) x[j] = x[j] * c;
    }
  }
}

// fp32 -> bf16 cast of a flat range (initial model-parameter materialisation).
__global__ void sga_cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = __float2bfloat16_rn(src[i]);
}

}  // namespace sga

SGA_API int sga_adam_step(float* w, float* g, float* m, float* v, void* model_bf16, const uint8_t* mask,
                          const float* coeff, const long long* seg_start, const int* seg_group, int nseg,
                          long long n, const float* group_lr, const float* group_wd, int ngroups, float beta1,
                          float omb1, float beta2, float omb2, float bc1, float bc2, float eps, float interval,
                          float lr_scale, int emit, int clear, int fold, int lr_split, int adams, int use_coeff,
                          int max_ctas, void* stream) {
  using namespace sga;
  if (n <= 0) return 0;
  if (ngroups > 8 || nseg < 1) return -1;
  AdamArgs a;
  a.w = w; a.g = g; a.m = m; a.v = v;
  a.model = reinterpret_cast<__nv_bfloat16*>(model_bf16);
  a.mask = mask; a.coeff = coeff; a.seg_start = seg_start; a.seg_group = seg_group; a.nseg = nseg; a.n = n;
  for (int i = 0; i < ngroups; ++i) { a.groups[i].lr = group_lr[i]; a.groups[i].wd = group_wd[i]; }
  a.beta1 = beta1; a.omb1 = omb1; a.beta2 = beta2; a.omb2 = omb2; a.bc1 = bc1; a.bc2 = bc2; a.eps = eps;
  a.interval = interval; a.lr_scale = lr_scale;
  a.emit = emit; a.clear = clear; a.fold = fold; a.lr_split = lr_split; a.adams = adams; a.use_coeff = use_coeff;
  long long blocks = (n + ADAM_CHUNK - 1) / ADAM_CHUNK;
  const long long cap = max_ctas > 0 ? max_ctas : 148 * 8;
  if (blocks > cap) blocks = cap;
  sga_adam_kernel<<<(int)blocks, ADAM_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// out[0] (+)= sum of squares of x (masked if mask != null). `partials` must hold >= 1184 floats.
SGA_API int sga_sumsq(const float* x, const uint8_t* mask, long long n, float* partials, float* out, int accumulate,
                      void* stream) {
  using namespace sga;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  long long blocks = (n + NORM_THREADS * 4 - 1) / (NORM_THREADS * 4);
  if (blocks > 1184) blocks = 1184;
  if (blocks < 1) blocks = 1;
  sga_sumsq_stage1<<<(int)blocks, NORM_THREADS, 0, st>>>(x, mask, n, partials);
  sga_sumsq_stage2<<<1, 256, 0, st>>>(partials, (int)blocks, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

SGA_API int sga_clip_coeff(const float* sumsq, float inv_world, float clip, float* coeff, float* norm_out,
                           void* stream) {
  sga::sga_clip_coeff_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sumsq, inv_world, clip, coeff,
                                                                                   norm_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

SGA_API int sga_scale(float* x, long long n, const float* coeff_ptr, float factor, void* stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 1023) / 1024;
  if (blocks > 148 * 8) blocks = 148 * 8;
  sga::sga_scale_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, n, coeff_ptr, factor);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

SGA_API int sga_cast_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  sga::sga_cast_bf16_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
