// Dense all-reduce of a symmetric fp32 buffer through the NVSwitch's in-switch
// reduction (NVLS): an optional, gated alternative to the peer-load kernel of
// p2p_sync.cu for buffers that are bound to an NVLink multicast object.
//
// Every rank owns a contiguous slice of the buffer. For each 16-byte group of
// its slice a thread issues one multimem.ld_reduce on the multicast address:
// the switch reads the group from every GPU's copy and returns the sum, so a
// GPU receives one group per element of its slice instead of W - 1. The
// result goes back out with one multimem.st (the switch writes it to every
// copy), or stays local in the reduce-scatter form. Flags, bounded waits, the
// grid barrier and the rank-ordered norm exchange are those of the peer
// kernels; only the data path differs. The order in which the switch adds the
// ranks' values is the hardware's, so the sum can differ from the peer
// kernel's rank-ordered one in the last bit; every rank still ends with the
// same bits, because each element is reduced once, by its owner.
//
// The multicast mapping itself (creation of the multicast object, binding of
// every rank's allocation, exchange of the handles) is done by the framework
// layer (torch.distributed's symmetric memory); this file only needs the
// multicast address and the local one.
//
// Counterpart in the reference: none of its own; NCCL's NVLS algorithm serves
// its dense all-reduce calls (sga/backends/torch_pipelined_index.py:393-520).
#include "common.cuh"
#include "peer.cuh"

namespace sga {

__device__ __forceinline__ float4 multimem_ld_reduce_add(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(float* mc, const float4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

struct NvlsArgs {
  PeerCtx c;
  float* local;   // this rank's copy
  float* mc;      // the same buffer through the multicast mapping
  long long n;    // a multiple of 4 (the host pads the bucket view)
  float scale;
  int rs_only;
  float* norm_slots[MAXW];
  float* cta_partials;
  float* sumsq_out;
  int accumulate;
};

__global__ void __launch_bounds__(512) nvls_allreduce_kernel(const NvlsArgs a) {
  __shared__ float red[512];
  const PeerCtx& c = a.c;
  int gen = 0;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  // every rank's input is in place (and visible at system scope) before anyone reduces
  __threadfence_system();
  grid_barrier(c.grid_counter, gen, c.err);
  peer_signal(c, 0);
  peer_wait(c, 0, c.seq);

  const long long n4 = a.n >> 2;
  const long long per = (n4 + c.W - 1) / c.W;
  const long long s4 = per * c.rank;
  const long long e4 = min(n4, s4 + per);
  float sq = 0.f;
  for (long long q = s4 + tid; q < e4; q += nth) {
    float4 acc = multimem_ld_reduce_add(a.mc + q * 4);
    acc.x *= a.scale; acc.y *= a.scale; acc.z *= a.scale; acc.w *= a.scale;
    sq += acc.x * acc.x; sq += acc.y * acc.y; sq += acc.z * acc.z; sq += acc.w * acc.w;
    if (a.rs_only) *reinterpret_cast<float4*>(a.local + q * 4) = acc;
    else multimem_st(a.mc + q * 4, acc);
  }
  const float bs = block_sum(sq, red);
  if (threadIdx.x == 0) a.cta_partials[blockIdx.x] = bs;
  __threadfence_system();
  grid_barrier(c.grid_counter, gen, c.err);
  publish_norm(c, a.cta_partials, a.norm_slots);
  peer_signal(c, 1);
  peer_wait(c, 1, c.seq);
  collect_norm(c, a.norm_slots, a.sumsq_out, a.accumulate);
}

}  // namespace sga

using namespace sga;

// local / mc: this rank's address and the multicast address of the same n fp32 values (n % 4 == 0, both
// 16-byte aligned). Returns 0, or a negative code before anything was launched.
SGA_API int sga_nvls_allreduce(const SgaPeerDesc* d, float* local, float* mc, long long n, float scale, int rs_only,
                               void* const* norm_slots, float* cta_partials, float* sumsq_out, int accumulate,
                               int max_ctas, void* stream) {
  if (d->W > MAXW) return -1;
  if (!local || !mc || n <= 0 || (n & 3)) return -6;
  if ((reinterpret_cast<uintptr_t>(local) & 15) || (reinterpret_cast<uintptr_t>(mc) & 15)) return -9;
  NvlsArgs a;
  a.c = make_ctx(d);
  a.local = local;
  a.mc = mc;
  a.n = n;
  a.scale = scale;
  a.rs_only = rs_only;
  for (int i = 0; i < MAXW; ++i) a.norm_slots[i] = i < d->W ? reinterpret_cast<float*>(norm_slots[i]) : nullptr;
  a.cta_partials = cta_partials;
  a.sumsq_out = sumsq_out;
  a.accumulate = accumulate;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaMemsetAsync(a.c.grid_counter, 0, sizeof(int), st);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms;  // one co-resident wave: the kernel contains grid barriers
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  long long need = (n + 2047) / 2048;
  if (need < grid) grid = (int)need;
  void* params[] = {&a};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(nvls_allreduce_kernel), dim3(grid), dim3(512),
                                              params, 0, st);
  return e == cudaSuccess ? 0 : -4;
}
