// Bandwidth-bound model ops in bf16 with fp32 math: RMSNorm (also per-head
// QK-norm) forward / backward, rotary embedding, SwiGLU, fused softmax
// cross-entropy (loss and logit gradient in one kernel), embedding gather and
// its scatter-add backward into the fp32 main-grad buffer.
//
// These stand where the reference's external stack calls TransformerEngine /
// Apex fused ops (examples/llama3/train_1b_adamw.yaml:89-107); none of that
// source is part of the reference tree.
#include "common.cuh"

namespace sga {

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// ---------------------------------------------------------------- RMSNorm
// One warp per row of H elements (H % 8 == 0). y = x * rstd * w.
// Rows may be strided (row_stride elements) so the kernel also serves the
// per-head QK-norm on a slice of the fused QKV activation.
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                          long long rows, int H, long long x_stride,
                                                          long long y_stride, int rows_per_group,
                                                          long long group_stride_x, long long group_stride_y,
                                                          float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  // row -> (group, r): address = group * group_stride + r * stride
  const long long grp = row / rows_per_group, r = row % rows_per_group;
  const __nv_bfloat16* xr = x + grp * group_stride_x + r * x_stride;
  __nv_bfloat16* yr = y + grp * group_stride_y + r * y_stride;
  const int nch = H >> 3;
  float ss = 0.f;
  for (int c = lane; c < nch; c += 32) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / (float)H + eps);
  if (lane == 0 && rstd) rstd[row] = rs;
  for (int c = lane; c < nch; c += 32) {
    float f[8], g[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c * 8), f);
    unpack8(*reinterpret_cast<const uint4*>(w + c * 8), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * rs * g[i];
    *reinterpret_cast<uint4*>(yr + c * 8) = pack8(f);
  }
}

// The same row kept in registers: CPL 16-byte chunks per lane (H <= CPL * 256), all loads of the row issued
// before the first use, the second pass served from registers. Same summation order as the kernel above, so the
// results are bit-identical.
template <int CPL>
__global__ void __launch_bounds__(256) rmsnorm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x,
                                                              const __nv_bfloat16* __restrict__ w,
                                                              __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                              long long rows, int H, long long x_stride,
                                                              long long y_stride, int rows_per_group,
                                                              long long group_stride_x, long long group_stride_y,
                                                              float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const long long grp = row / rows_per_group, r = row % rows_per_group;
  const __nv_bfloat16* xr = x + grp * group_stride_x + r * x_stride;
  __nv_bfloat16* yr = y + grp * group_stride_y + r * y_stride;
  const int nch = H >> 3;
  uint4 raw[CPL];
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    const int c = lane + 32 * j;
    raw[j] = c < nch ? *reinterpret_cast<const uint4*>(xr + c * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    if (lane + 32 * j < nch) {
      float f[8];
      unpack8(raw[j], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / (float)H + eps);
  if (lane == 0 && rstd) rstd[row] = rs;
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    const int c = lane + 32 * j;
    if (c < nch) {
      float f[8], g[8];
      unpack8(raw[j], f);
      unpack8(*reinterpret_cast<const uint4*>(w + c * 8), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rs * g[i];
      *reinterpret_cast<uint4*>(yr + c * 8) = pack8(f);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)); dw partial per CTA.
// Each warp walks rows (strided by total warps); lanes own column chunks.
template <int NCH>  // chunks of 8 columns per lane: H <= NCH * 256
__global__ void __launch_bounds__(256, NCH <= 8 ? 2 : 1) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                             const __nv_bfloat16* __restrict__ w,
                                                             const __nv_bfloat16* __restrict__ dy,
                                                             const float* __restrict__ rstd,
                                                             __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part,
                                                             long long rows, int H, long long x_stride,
                                                             long long dy_stride, long long dx_stride,
                                                             int rows_per_group, long long gsx, long long gsdy,
                                                             long long gsdx, int accumulate_dx) {
  // shared: one fp32 row of H per warp; every lane owns fixed columns of its warp's row, so no atomics
  extern __shared__ float sdw[];
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int nwarp = blockDim.x >> 5;
  const int nch = H >> 3;
  float* myrow = sdw + (size_t)wid * H;
  for (int i = lane; i < H; i += 32) myrow[i] = 0.f;
  __syncwarp();
  const long long warps = (long long)gridDim.x * nwarp;
  for (long long row = (long long)blockIdx.x * nwarp + wid; row < rows; row += warps) {
    const long long grp = row / rows_per_group, r = row % rows_per_group;
    const __nv_bfloat16* xr = x + grp * gsx + r * x_stride;
    const __nv_bfloat16* dyr = dy + grp * gsdy + r * dy_stride;
    __nv_bfloat16* dxr = dx + grp * gsdx + r * dx_stride;
    const float rs = rstd[row];
    float dot = 0.f;
    // rows up to 2048 wide stay in registers between the two passes; wider rows are re-read (L1/L2 hits)
    constexpr bool kCache = NCH <= 8;
    constexpr int kRegs = kCache ? NCH : 1;
    uint4 px[kRegs], pd[kRegs];
    if constexpr (kCache) {
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int c = lane + 32 * j;
        if (c < nch) {
          px[j] = *reinterpret_cast<const uint4*>(xr + c * 8);
          pd[j] = *reinterpret_cast<const uint4*>(dyr + c * 8);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = lane + 32 * j;
      if (c < nch) {
        float fx[8], fw[8], fd[8];
        unpack8(kCache ? px[j] : *reinterpret_cast<const uint4*>(xr + c * 8), fx);
        unpack8(kCache ? pd[j] : *reinterpret_cast<const uint4*>(dyr + c * 8), fd);
        unpack8(*reinterpret_cast<const uint4*>(w + c * 8), fw);
        float4* acc = reinterpret_cast<float4*>(myrow + c * 8);
        float4 a0 = acc[0], a1 = acc[1];
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = fx[i] * rs;
          dot += fd[i] * fw[i] * xh;
          t[i] = fd[i] * xh;
        }
        a0.x += t[0]; a0.y += t[1]; a0.z += t[2]; a0.w += t[3];
        a1.x += t[4]; a1.y += t[5]; a1.z += t[6]; a1.w += t[7];
        acc[0] = a0;
        acc[1] = a1;
      }
    }
    dot = warp_sum(dot) / (float)H;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = lane + 32 * j;
      if (c < nch) {
        float fx[8], fw[8], fd[8], o[8];
        unpack8(kCache ? px[j] : *reinterpret_cast<const uint4*>(xr + c * 8), fx);
        unpack8(kCache ? pd[j] : *reinterpret_cast<const uint4*>(dyr + c * 8), fd);
        unpack8(*reinterpret_cast<const uint4*>(w + c * 8), fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rs * (fd[i] * fw[i] - (fx[i] * rs) * dot);
        if (accumulate_dx) {
          float prev[8];
          unpack8(*reinterpret_cast<const uint4*>(dxr + c * 8), prev);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += prev[i];
        }
        *reinterpret_cast<uint4*>(dxr + c * 8) = pack8(o);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float t = 0.f;
    for (int wv = 0; wv < nwarp; ++wv) t += sdw[(size_t)wv * H + i];
    dw_part[(long long)blockIdx.x * H + i] = t;
  }
}

// out[i] (+)= sum_b part[b][i]. A CTA owns 32 columns; its 8 warps each add every eighth row of the
// partials and the 8 partial sums are added in warp order: the order of summation is fixed.
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ part, int nb, int H,
                                                      float* __restrict__ out, int accumulate) {
  __shared__ float sh[8][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (i < H)
    for (int b = w; b < nb; b += 8) s += part[(long long)b * H + i];
  sh[w][lane] = s;
  __syncthreads();
  if (w == 0 && i < H) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sh[k][lane];
    out[i] = accumulate ? out[i] + t : t;
  }
}

// ------------------------------------------------------------------- RoPE
// In place on rows of [T, nheads, hd] embedded in a wider activation
// (row pitch `pitch` elements, heads start at column `col0`). Pairs are
// (i, i + hd/2). cos/sin: [S, hd/2] fp32. sign = +1 forward, -1 backward.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            long long T, int S, int nheads, int hd, long long pitch, int col0, float sign) {
  // one thread rotates 8 pairs: columns [8c, 8c+8) of the first half with the same columns of the second half
  const int half = hd >> 1;
  const int hc = half >> 3;
  const long long total = T * nheads * hc;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gstride) {
    const int c = (int)(e % hc);
    const long long th = e / hc;
    const int h = (int)(th % nheads);
    const long long t = th / nheads;
    const int pos = (int)(t % S);
    __nv_bfloat16* p = x + t * pitch + col0 + (long long)h * hd + c * 8;
    float a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(p), a);
    unpack8(*reinterpret_cast<const uint4*>(p + half), b);
    const float4 c0 = *reinterpret_cast<const float4*>(cs + pos * half + c * 8);
    const float4 c1 = *reinterpret_cast<const float4*>(cs + pos * half + c * 8 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sn + pos * half + c * 8);
    const float4 s1 = *reinterpret_cast<const float4*>(sn + pos * half + c * 8 + 4);
    const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float oa[8], ob[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = ss[i] * sign;
      oa[i] = a[i] * cc[i] - b[i] * sg;
      ob[i] = b[i] * cc[i] + a[i] * sg;
    }
    *reinterpret_cast<uint4*>(p) = pack8(oa);
    *reinterpret_cast<uint4*>(p + half) = pack8(ob);
  }
}

// ----------------------------------------------------------------- SwiGLU
// in: [T, 2F] = gate | up ; out: [T, F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long T,
                                  int F) {
  const long long total = T * (F >> 3);
  const long long gstride = (long long)gridDim.x * blockDim.x;
  const int fc = F >> 3;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gstride) {
    const long long t = e / fc;
    const int c = (int)(e % fc);
    float g[8], u[8];
    unpack8(*reinterpret_cast<const uint4*>(in + t * 2 * F + c * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(in + t * 2 * F + F + c * 8), u);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    *reinterpret_cast<uint4*>(out + t * F + c * 8) = pack8(g);
  }
}
// din: [T, 2F] from dout [T, F] and the saved input.
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ din, long long T, int F) {
  const long long total = T * (F >> 3);
  const long long gstride = (long long)gridDim.x * blockDim.x;
  const int fc = F >> 3;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gstride) {
    const long long t = e / fc;
    const int c = (int)(e % fc);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(in + t * 2 * F + c * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(in + t * 2 * F + F + c * 8), u);
    unpack8(*reinterpret_cast<const uint4*>(dout + t * F + c * 8), d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = 1.f / (1.f + __expf(-g[i]));
      const float silu = g[i] * sg;
      du[i] = d[i] * silu;
      dg[i] = d[i] * u[i] * (sg * (1.f + g[i] * (1.f - sg)));
    }
    *reinterpret_cast<uint4*>(din + t * 2 * F + c * 8) = pack8(dg);
    *reinterpret_cast<uint4*>(din + t * 2 * F + F + c * 8) = pack8(du);
  }
}

// ---------------------------------------------------------- cross-entropy
// One CTA per row. loss[t] = logsumexp(z) - z[target]; logits are replaced in
// place by (softmax - onehot) * grad_scale (the gradient of mean loss).
__global__ void __launch_bounds__(1024) ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits,
                                                          const long long* __restrict__ targets,
                                                          float* __restrict__ loss, int V, long long pitch,
                                                          float grad_scale, int write_grad) {
  __shared__ float red[32];
  __shared__ float bc[2];
  const long long t = blockIdx.x;
  __nv_bfloat16* z = logits + t * pitch;
  const int nch = V >> 3;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < nch; c += blockDim.x) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(z + c * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, f[i]);
  }
  mx = warp_max(mx);
  if (lane == 0) red[wid] = mx;
  __syncthreads();
  if (wid == 0) {
    float v = lane < (int)(blockDim.x >> 5) ? red[lane] : -INFINITY;
    v = warp_max(v);
    if (lane == 0) bc[0] = v;
  }
  __syncthreads();
  mx = bc[0];
  float se = 0.f;
  for (int c = threadIdx.x; c < nch; c += blockDim.x) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(z + c * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) se += __expf(f[i] - mx);
  }
  se = warp_sum(se);
  __syncthreads();
  if (lane == 0) red[wid] = se;
  __syncthreads();
  if (wid == 0) {
    float v = lane < (int)(blockDim.x >> 5) ? red[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) bc[1] = v;
  }
  __syncthreads();
  se = bc[1];
  const long long tgt = targets[t];
  const float lse = mx + __logf(se);
  if (threadIdx.x == 0) {
    const bool valid = tgt >= 0 && tgt < V;
    loss[t] = valid ? lse - __bfloat162float(z[tgt]) : 0.f;
  }
  if (!write_grad) return;
  __syncthreads();  // z[tgt] read above before it is overwritten
  const float inv = 1.f / se;
  const bool valid = tgt >= 0 && tgt < V;
  const float gs = valid ? grad_scale : 0.f;
  for (int c = threadIdx.x; c < nch; c += blockDim.x) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(z + c * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float p = __expf(f[i] - mx) * inv;
      if ((long long)(c * 8 + i) == tgt) p -= 1.f;
      f[i] = p * gs;
    }
    *reinterpret_cast<uint4*>(z + c * 8) = pack8(f);
  }
}

// -------------------------------------------------------------- embedding
__global__ void embed_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ W,
                                 __nv_bfloat16* __restrict__ out, long long T, int H) {
  const int hc = H >> 3;
  const long long total = T * hc;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gstride) {
    const long long t = e / hc;
    const int c = (int)(e % hc);
    *reinterpret_cast<uint4*>(out + t * H + c * 8) = *reinterpret_cast<const uint4*>(W + ids[t] * H + c * 8);
  }
}
// Scatter-add of the token gradients into the embedding rows without atomics: the tokens arrive
// sorted by id (stable, so equal ids keep their position order); the CTA that sits on the first
// token of a run adds the run's rows in that order and owns the embedding row, the others leave.
// The sum is the same bits on every run and every rank.
__global__ void embed_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ perm,
                                 const __nv_bfloat16* __restrict__ dout, float* __restrict__ main_grad, long long T,
                                 int H) {
  const long long p0 = blockIdx.x;
  const long long id = sorted_ids[p0];
  if (p0 > 0 && sorted_ids[p0 - 1] == id) return;
  const int hc = H >> 3;
  for (int c = threadIdx.x; c < hc; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (long long q = p0; q < T && sorted_ids[q] == id; ++q) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(dout + perm[q] * H + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    float4* g = reinterpret_cast<float4*>(main_grad + id * H + c * 8);
    float4 g0 = g[0], g1 = g[1];
    g0.x += acc[0]; g0.y += acc[1]; g0.z += acc[2]; g0.w += acc[3];
    g1.x += acc[4]; g1.y += acc[5]; g1.z += acc[6]; g1.w += acc[7];
    g[0] = g0;
    g[1] = g1;
  }
}

// bf16 elementwise add: out = a + b (residual joins not covered by a GEMM epilogue)
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, long long n8) {
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n8; e += gstride) {
    float fa[8], fb[8];
    unpack8(*reinterpret_cast<const uint4*>(a + e * 8), fa);
    unpack8(*reinterpret_cast<const uint4*>(b + e * 8), fb);
#pragma unroll
    for (int i = 0; i < 8; ++i) fa[i] += fb[i];
    *reinterpret_cast<uint4*>(out + e * 8) = pack8(fa);
  }
}

static inline int grid1d(long long n, int threads, int cap = 148 * 16) {
  long long b = (n + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return (int)b;
}

}  // namespace sga

using namespace sga;
#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -4)

SGA_API int sga_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int H,
                            long long x_stride, long long y_stride, int rows_per_group, long long gsx,
                            long long gsy, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (H & 7) return -5;
  const int wpb = 8;
  const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
  const int cpl = (H / 8 + 31) / 32;  // 16-byte chunks per lane
#define RF(N)                                                                                                  \
  rmsnorm_fwd_reg_kernel<N><<<grid, wpb * 32, 0, ST(stream)>>>(                                                 \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, rows, H, x_stride, y_stride,   \
      rows_per_group, gsx, gsy, eps)
  if (cpl <= 1) RF(1);
  else if (cpl <= 2) RF(2);
  else if (cpl <= 4) RF(4);
  else if (cpl <= 8) RF(8);
  else if (cpl <= 16) RF(16);
  else
    rmsnorm_fwd_kernel<<<grid, wpb * 32, 0, ST(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                         (__nv_bfloat16*)y, rstd, rows, H, x_stride, y_stride,
                                                         rows_per_group, gsx, gsy, eps);
#undef RF
  return LAUNCH_OK();
}

// dw_part: scratch [nblocks * H] floats with nblocks = sga_rmsnorm_bwd_blocks().
SGA_API int sga_rmsnorm_bwd_blocks() { return 148 * 2; }

SGA_API int sga_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                            float* dw_part, float* dw_out, int accumulate_dw, long long rows, int H,
                            long long x_stride, long long dy_stride, long long dx_stride, int rows_per_group,
                            long long gsx, long long gsdy, long long gsdx, int accumulate_dx, void* stream) {
  if (rows <= 0) return 0;
  if (H & 7 || H > 6144) return -5;
  const int nb = sga_rmsnorm_bwd_blocks();
  const int nch = (H / 8 + 31) / 32;
  const size_t smem = (size_t)H * 4 * 8;  // one fp32 row per warp
  if (smem > 48 * 1024) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      attr_set[dev & 63] = true;
    }
  }
#define RB(N)                                                                                                     \
  rmsnorm_bwd_kernel<N><<<nb, 256, smem, ST(stream)>>>(                                                            \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, rstd, (__nv_bfloat16*)dx, dw_part, \
      rows, H, x_stride, dy_stride, dx_stride, rows_per_group, gsx, gsdy, gsdx, accumulate_dx)
  if (nch <= 1) RB(1);
  else if (nch <= 2) RB(2);
  else if (nch <= 4) RB(4);
  else if (nch <= 8) RB(8);
  else if (nch <= 16) RB(16);
  else RB(32);
#undef RB
  colsum_kernel<<<(H + 31) / 32, 256, 0, ST(stream)>>>(dw_part, nb, H, dw_out, accumulate_dw);
  return LAUNCH_OK();
}

SGA_API int sga_rope(void* x, const float* cs, const float* sn, long long T, int S, int nheads, int hd,
                     long long pitch, int col0, float sign, void* stream) {
  if (hd & 15) return -5;  // 8-wide chunks in each half
  const long long total = T * nheads * (hd / 16);
  if (total <= 0) return 0;
  rope_kernel<<<grid1d(total, 256), 256, 0, ST(stream)>>>((__nv_bfloat16*)x, cs, sn, T, S, nheads, hd, pitch, col0,
                                                           sign);
  return LAUNCH_OK();
}

SGA_API int sga_swiglu_fwd(const void* in, void* out, long long T, int F, void* stream) {
  if (T <= 0) return 0;
  if (F & 7) return -5;
  swiglu_fwd_kernel<<<grid1d(T * (F / 8), 256), 256, 0, ST(stream)>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out,
                                                                      T, F);
  return LAUNCH_OK();
}
SGA_API int sga_swiglu_bwd(const void* in, const void* dout, void* din, long long T, int F, void* stream) {
  if (T <= 0) return 0;
  if (F & 7) return -5;
  swiglu_bwd_kernel<<<grid1d(T * (F / 8), 256), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)in, (const __nv_bfloat16*)dout, (__nv_bfloat16*)din, T, F);
  return LAUNCH_OK();
}

SGA_API int sga_cross_entropy(void* logits, const long long* targets, float* loss, long long T, int V,
                              long long pitch, float grad_scale, int write_grad, void* stream) {
  if (T <= 0) return 0;
  if (V & 7 || pitch & 7) return -5;
  ce_fwd_bwd_kernel<<<(unsigned)T, 1024, 0, ST(stream)>>>((__nv_bfloat16*)logits, targets, loss, V, pitch, grad_scale,
                                                          write_grad);
  return LAUNCH_OK();
}

SGA_API int sga_embed_fwd(const long long* ids, const void* W, void* out, long long T, int H, void* stream) {
  if (T <= 0) return 0;
  if (H & 7) return -5;
  embed_fwd_kernel<<<grid1d(T * (H / 8), 256), 256, 0, ST(stream)>>>(ids, (const __nv_bfloat16*)W,
                                                                     (__nv_bfloat16*)out, T, H);
  return LAUNCH_OK();
}
// sorted_ids / perm: the token ids in ascending order (stable) and the position each came from.
SGA_API int sga_embed_bwd(const long long* sorted_ids, const long long* perm, const void* dout, float* main_grad,
                          long long T, int H, void* stream) {
  if (T <= 0) return 0;
  if (H & 7) return -5;
  const int threads = H / 8 >= 256 ? 256 : (H / 8 >= 128 ? 128 : 64);
  embed_bwd_kernel<<<(unsigned)T, threads, 0, ST(stream)>>>(sorted_ids, perm, (const __nv_bfloat16*)dout, main_grad,
                                                            T, H);
  return LAUNCH_OK();
}
SGA_API int sga_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n & 7) return -5;
  add_bf16_kernel<<<grid1d(n / 8, 256), 256, 0, ST(stream)>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                              (__nv_bfloat16*)out, n / 8);
  return LAUNCH_OK();
}
