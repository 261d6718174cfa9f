// Dense (SGA-off) step, second half: residual-free AdamW on the slice of every
// bucket that this rank owns after the reduce-scatter, with the bf16 parameter
// all-gather fused into the same kernel as peer stores. The first half is
// sga_p2p_allreduce with rs_only = 1 (one launch per bucket, overlapped with
// the backward pass); the global-norm clip coefficient is read from device
// memory, so the step has no host round trip.
//
// Ownership: a bucket of n elements is cut at float4 granularity into W equal
// slices, slice r belongs to rank r (the same cut as the reduce-scatter).
// Only the owner's fp32 master weights and moments for that slice are live;
// a checkpoint gathers them into the replicated torch-Adam layout.
//
// Compiled with -fmad=false and without fast-math (see adam_math.cuh).
// Replaces the reference's dense path: stock DDP all-reduce
// (sga/engine.py:442-446), the full-step optimizer kernel and the separate
// fp32 -> bf16 parameter copy (sga/engine.py:585-586).
#include "common.cuh"
#include "peer.cuh"
#include "adam_math.cuh"

namespace sga {

struct DenseAdamArgs {
  PeerCtx c;
  float* w;
  const float* g;
  float* m;
  float* v;
  __nv_bfloat16* model[MAXW];  // every rank's bf16 parameter arena (same layout)
  const long long* bucket_start;  // [nb]
  const long long* bucket_len;    // [nb]
  int nb;
  const long long* seg_start;  // [nseg (+1)] ascending over the arena
  const int* seg_group;
  int nseg;
  float group_lr[8], group_wd[8];
  const float* coeff;  // nullable
  AdamScalars s;
  int adams;
};

__global__ void __launch_bounds__(256) dense_adamw_ag_kernel(const DenseAdamArgs a) {
  const PeerCtx& c = a.c;
  int gen = 0;
  const float coeff = a.coeff ? *a.coeff : 1.0f;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  for (int b = 0; b < a.nb; ++b) {
    const long long start = a.bucket_start[b];
    const long long n = a.bucket_len[b];
    const long long n4 = (n + 3) / 4;
    const long long per = (n4 + c.W - 1) / c.W;
    const long long s4 = per * c.rank;
    const long long e4 = min(n4, s4 + per);
    int seg = 0;
    bool seg_init = false;
    for (long long q = s4 + tid; q < e4; q += nth) {
      const long long i = start + q * 4;
      if (!seg_init) {
        int lo = 0, hi = a.nseg - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (a.seg_start[mid] <= i) lo = mid; else hi = mid - 1;
        }
        seg = lo;
        seg_init = true;
      }
      while (seg + 1 < a.nseg && a.seg_start[seg + 1] <= i) ++seg;
      const int grp = a.seg_group[seg];
      const float lr = a.group_lr[grp], wd = a.group_wd[grp];
      const int lim = (int)min((long long)4, start + n - i);
      float wv[4], mv[4], vv[4], gv[4];
      if (lim == 4) {  // bucket starts and the slice cut are 16-byte aligned: one 128-bit access per array
        *reinterpret_cast<float4*>(wv) = *reinterpret_cast<const float4*>(a.w + i);
        *reinterpret_cast<float4*>(gv) = *reinterpret_cast<const float4*>(a.g + i);
        *reinterpret_cast<float4*>(mv) = *reinterpret_cast<const float4*>(a.m + i);
        *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(a.v + i);
      } else {
        for (int j = 0; j < lim; ++j) {
          wv[j] = a.w[i + j];
          gv[j] = a.g[i + j];
          mv[j] = a.m[i + j];
          vv[j] = a.v[i + j];
        }
      }
      __nv_bfloat16 bo[4];
      for (int j = 0; j < lim; ++j) {
        float g = gv[j];
        if (coeff != 1.0f) g = g * coeff;
        const float upd = adam_update(wv[j], g, mv[j], vv[j], wd, a.adams, a.s);
        wv[j] = wv[j] - lr * upd;
        bo[j] = __float2bfloat16_rn(wv[j]);
      }
      if (lim == 4) {
        *reinterpret_cast<float4*>(a.w + i) = *reinterpret_cast<float4*>(wv);
        *reinterpret_cast<float4*>(a.m + i) = *reinterpret_cast<float4*>(mv);
        *reinterpret_cast<float4*>(a.v + i) = *reinterpret_cast<float4*>(vv);
      } else {
        for (int j = 0; j < lim; ++j) {
          a.w[i + j] = wv[j];
          a.m[i + j] = mv[j];
          a.v[i + j] = vv[j];
        }
      }
      if (lim == 4) {
#pragma unroll
        for (int r = 0; r < MAXW; ++r)
          if (r < c.W) *reinterpret_cast<uint2*>(a.model[r] + i) = *reinterpret_cast<uint2*>(bo);
      } else {
        for (int r = 0; r < c.W; ++r)
          for (int j = 0; j < lim; ++j) a.model[r][i + j] = bo[j];
      }
    }
  }
  __threadfence_system();
  grid_barrier(c.grid_counter, gen, c.err);
  peer_signal(c, 1);
  peer_wait(c, 1, c.seq);
}

}  // namespace sga

using namespace sga;

SGA_API int sga_dense_adamw_ag(const SgaPeerDesc* d, float* w, const float* g, float* m, float* v,
                               void* const* model_arenas, const long long* bucket_start,
                               const long long* bucket_len, int nb, const long long* seg_start,
                               const int* seg_group, int nseg, const float* group_lr, const float* group_wd,
                               int ngroups, const float* coeff, float beta1, float omb1, float beta2, float omb2,
                               float bc1, float bc2, float eps, int adams, int max_ctas, void* stream) {
  if (d->W > MAXW || ngroups > 8) return -1;
  DenseAdamArgs a;
  a.c = make_ctx(d);
  a.w = w; a.g = g; a.m = m; a.v = v;
  for (int i = 0; i < MAXW; ++i) a.model[i] = i < d->W ? reinterpret_cast<__nv_bfloat16*>(model_arenas[i]) : nullptr;
  a.bucket_start = bucket_start; a.bucket_len = bucket_len; a.nb = nb;
  a.seg_start = seg_start; a.seg_group = seg_group; a.nseg = nseg;
  for (int i = 0; i < ngroups; ++i) { a.group_lr[i] = group_lr[i]; a.group_wd[i] = group_wd[i]; }
  a.coeff = coeff;
  a.s.beta1 = beta1; a.s.omb1 = omb1; a.s.beta2 = beta2; a.s.omb2 = omb2; a.s.bc1 = bc1; a.s.bc2 = bc2; a.s.eps = eps;
  a.adams = adams;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaMemsetAsync(a.c.grid_counter, 0, sizeof(int), st);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms * 4;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  void* params[] = {&a};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dense_adamw_ag_kernel), dim3(grid), dim3(256),
                                              params, 0, st);
  return e == cudaSuccess ? 0 : -4;
}
