// Cross-rank signalling shared by the peer-memory kernels: sequence-numbered
// ready / done flags in symmetric memory, bounded waits, and the deterministic
// per-rank norm exchange.
#pragma once
#include "common.cuh"

namespace sga {

constexpr int MAXW = 8;

struct PeerCtx {
  int W, rank;
  int* flags[MAXW];  // flags[p]: peer p's int[16]: [0,8) ready by source rank, [8,16) done by source rank
  int seq;           // this launch's sequence number on the channel (monotonic, > 0)
  int prev_seq;      // sequence number of the previous launch on the channel (0 = none)
  int* grid_counter; // local, zero on entry
  int* err;
  long long wait_cycles;
};

__device__ __forceinline__ void peer_signal(const PeerCtx& c, int slot) {
  if (blockIdx.x == 0 && threadIdx.x < c.W) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + slot * 8 + c.rank, c.seq);
  }
}
__device__ __forceinline__ void peer_wait(const PeerCtx& c, int slot, int target) {
  if (threadIdx.x < c.W) wait_flag_sys(c.flags[c.rank] + slot * 8 + threadIdx.x, target, c.wait_cycles, c.err);
  __syncthreads();
}

// Deterministic block sum (power-of-two blockDim <= 1024); result valid in thread 0.
__device__ __forceinline__ float block_sum(float v, float* red) {
  red[threadIdx.x] = v;
  __syncthreads();
  for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
    __syncthreads();
  }
  return red[0];
}

// After a grid barrier: block 0 adds the per-CTA partials in index order,
// publishes this rank's partial into slot [rank] of every peer's norm array.
__device__ __forceinline__ void publish_norm(const PeerCtx& c, const float* cta_partials, float* const* norm_slots) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)gridDim.x; ++i) t += cta_partials[i];
    for (int p = 0; p < c.W; ++p) norm_slots[p][c.rank] = t;
    __threadfence_system();
  }
  __syncthreads();
}
__device__ __forceinline__ void collect_norm(const PeerCtx& c, float* const* norm_slots, float* sumsq_out,
                                             int accumulate) {
  if (blockIdx.x == 0 && threadIdx.x == 0 && sumsq_out) {
    float t = 0.f;
    for (int r = 0; r < c.W; ++r) t += reinterpret_cast<volatile float*>(norm_slots[c.rank])[r];
    sumsq_out[0] = accumulate ? sumsq_out[0] + t : t;
  }
}

}  // namespace sga

struct SgaPeerDesc {  // host-side mirror passed from Python (ctypes.Structure)
  int W, rank;
  void* flags[sga::MAXW];
  int seq, prev_seq;
  void* grid_counter;
  void* err;
  long long wait_cycles;
};

static inline sga::PeerCtx make_ctx(const SgaPeerDesc* d) {
  sga::PeerCtx c;
  c.W = d->W;
  c.rank = d->rank;
  for (int i = 0; i < sga::MAXW; ++i) c.flags[i] = reinterpret_cast<int*>(d->flags[i]);
  c.seq = d->seq;
  c.prev_seq = d->prev_seq;
  c.grid_counter = reinterpret_cast<int*>(d->grid_counter);
  c.err = reinterpret_cast<int*>(d->err);
  c.wait_cycles = d->wait_cycles > 0 ? d->wait_cycles : SGA_WAIT_CYCLES;
  return c;
}

