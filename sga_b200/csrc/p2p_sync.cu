// Fused compute + collective kernels over NVLink peer memory (plain P2P loads
// and stores issued from the kernel; no TMA from peer memory, no multicast).
//
//   sga_p2p_allreduce        [pack ->] two-shot all-reduce of a symmetric fp32
//                            buffer (owner reduces its slice in rank order and
//                            writes the result to every peer) [-> scatter],
//                            with the squared norm of the reduced payload
//   sga_p2p_mask_union       OR of the ranks' bit masks + reduction of the
//                            masked entries of the gradient bucket, in place
//
// (The rank-local top-k + (index, value) exchange lives in index_sync.cu.)
//
// Cross-rank ordering uses sequence-numbered flags in symmetric memory
// (st.release.sys / ld.acquire.sys); every wait is bounded and reports through
// the status word. Reductions run in a fixed rank order, so every rank ends
// with the same bits. Kernels are launched cooperatively (all CTAs resident)
// because they contain software grid barriers.
//
// Replaces the NCCL all-reduce call sites of
// sga/backends/torch_pipelined_index.py:393-520, torch_pipelined_mask.py:100-132
// and the external nccl-sar collective (nccl_pipelined_index.py:425-460).
#include "common.cuh"
#include "peer.cuh"
#include <string.h>

namespace sga {


// ------------------------------------------------------------ all-reduce
struct AllreduceArgs {
  PeerCtx c;
  float* buf[MAXW];
  long long n;
  float scale;
  float* grad;
  const int* idx;
  float factor;
  int do_pack, zero_after_pack, do_scatter;
  int block_x;  // 0: idx holds element positions. > 0: idx holds packed `head | tail_len` descriptors of
                // block_x-element runs (a power of two >= 4, heads block_x-aligned) and the payload is
                // n / block_x whole blocks, moved 16 bytes at a time
  int rs_only;  // reduce-scatter only: the owner keeps the reduced slice, nothing is written to peers
  float* norm_slots[MAXW];
  float* cta_partials;
  float* sumsq_out;
  int accumulate;
};

__global__ void __launch_bounds__(512) p2p_allreduce_kernel(const AllreduceArgs a) {
  __shared__ float red[512];
  const PeerCtx& c = a.c;
  int gen = 0;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  float* mine = a.buf[c.rank];
  if (a.do_pack && a.block_x > 0) {
    // descriptor wire form: runs of 16 to 256 bytes, gathered with 128-bit loads and stores
    const int x = a.block_x;
    for (long long q = tid; q * 4 < a.n; q += nth) {
      const long long i = q * 4;
      const int d = a.idx[i / x];
      const int off = (int)(i % x);
      const int head = d & ~(x - 1), tail = d & (x - 1);
      const int run = tail ? tail : x;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      float* src = a.grad + head + off;
      if (off + 4 <= run) {
        v = *reinterpret_cast<const float4*>(src);
        if (a.zero_after_pack) *reinterpret_cast<float4*>(src) = make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
        float t[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < 4 && off + j < run; ++j) {
          t[j] = src[j];
          if (a.zero_after_pack) src[j] = 0.f;
        }
        v = make_float4(t[0], t[1], t[2], t[3]);
      }
      v.x *= a.factor; v.y *= a.factor; v.z *= a.factor; v.w *= a.factor;
      *reinterpret_cast<float4*>(mine + i) = v;
    }
    __threadfence_system();
  } else if (a.do_pack) {
    for (long long i = tid; i < a.n; i += nth) {
      const int p = a.idx[i];
      const float v = a.grad[p];
      mine[i] = v * a.factor;
      if (a.zero_after_pack) a.grad[p] = 0.f;
    }
    __threadfence_system();
  }
  grid_barrier(c.grid_counter, gen, c.err);
  peer_signal(c, 0);
  peer_wait(c, 0, c.seq);

  // owner slice, float4 granularity
  const long long n4 = (a.n + 3) / 4;
  const long long per = (n4 + c.W - 1) / c.W;
  const long long s4 = per * c.rank;
  const long long e4 = min(n4, s4 + per);
  float sq = 0.f;
  for (long long q = s4 + tid; q < e4; q += nth) {
    const long long i = q * 4;
    if (i + 4 <= a.n) {
      float4 v[MAXW];
#pragma unroll
      for (int r = 0; r < MAXW; ++r)
        if (r < c.W) v[r] = *reinterpret_cast<const float4*>(a.buf[r] + i);
      float4 acc = v[0];
#pragma unroll
      for (int r = 1; r < MAXW; ++r)
        if (r < c.W) {
          acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
        }
      acc.x *= a.scale; acc.y *= a.scale; acc.z *= a.scale; acc.w *= a.scale;
      sq += acc.x * acc.x; sq += acc.y * acc.y; sq += acc.z * acc.z; sq += acc.w * acc.w;
#pragma unroll
      for (int r = 0; r < MAXW; ++r)
        if (r < c.W && (!a.rs_only || r == c.rank)) *reinterpret_cast<float4*>(a.buf[r] + i) = acc;
    } else {
      for (long long j = i; j < a.n; ++j) {
        float acc = 0.f;
        for (int r = 0; r < c.W; ++r) acc += a.buf[r][j];
        acc *= a.scale;
        sq += acc * acc;
        for (int r = 0; r < c.W; ++r)
          if (!a.rs_only || r == c.rank) a.buf[r][j] = acc;
      }
    }
  }
  const float bs = block_sum(sq, red);
  if (threadIdx.x == 0) a.cta_partials[blockIdx.x] = bs;
  __threadfence_system();
  grid_barrier(c.grid_counter, gen, c.err);
  publish_norm(c, a.cta_partials, a.norm_slots);
  peer_signal(c, 1);
  peer_wait(c, 1, c.seq);
  if (a.do_scatter && a.block_x > 0) {
    const int x = a.block_x;
    for (long long q = tid; q * 4 < a.n; q += nth) {
      const long long i = q * 4;
      const int d = a.idx[i / x];
      const int off = (int)(i % x);
      const int head = d & ~(x - 1), tail = d & (x - 1);
      const int run = tail ? tail : x;
      float* dst = a.grad + head + off;
      if (off + 4 <= run) {
        *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(mine + i);
      } else {
        for (int j = 0; j < 4 && off + j < run; ++j) dst[j] = mine[i + j];
      }
    }
  } else if (a.do_scatter) {
    for (long long i = tid; i < a.n; i += nth) a.grad[a.idx[i]] = mine[i];
  }
  collect_norm(c, a.norm_slots, a.sumsq_out, a.accumulate);
}

// ------------------------------------------------------- mask union reduce
struct MaskUnionArgs {
  PeerCtx c;
  float* grad[MAXW];
  const uint32_t* bits[MAXW];
  uint32_t* ubits[MAXW];
  long long n;
  float scale;
  uint8_t* mask_u8;  // nullable: local expansion of the union
  float* norm_slots[MAXW];
  float* cta_partials;
  float* sumsq_out;
  int accumulate;
  long long* count_out;  // nullable: number of union coordinates in the owned slice is added here
};

__global__ void __launch_bounds__(512) p2p_mask_union_kernel(const MaskUnionArgs a) {
  __shared__ float red[512];
  const PeerCtx& c = a.c;
  int gen = 0;
  grid_barrier(c.grid_counter, gen, c.err);
  peer_signal(c, 0);
  peer_wait(c, 0, c.seq);

  const long long nwords = (a.n + 31) / 32;
  const long long per = (nwords + c.W - 1) / c.W;
  const long long w0 = per * c.rank;
  const long long w1 = min(nwords, w0 + per);
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  float sq = 0.f;
  long long cnt = 0;
  // A warp takes 32 mask words (1024 coordinates) per trip: each lane loads one word, ORs it over the ranks,
  // coalesced, and stores the union back. The set positions of the trip are then compacted into a list in
  // shared memory (a warp scan of the words' bit counts gives every lane its slot), so that every lane holds
  // a coordinate of the union whatever its density: two coordinates per lane and every rank's value of both
  // are in flight before either is reduced, in rank order, and written back to every rank.
  __shared__ uint16_t s_list[16][1024];
  uint16_t* list = s_list[threadIdx.x >> 5];
  for (long long wb = w0 + warp * 32; wb < w1; wb += nwarps * 32) {
    const long long myw = wb + lane;
    uint32_t u = 0;
    if (myw < w1) {
#pragma unroll
      for (int r = 0; r < MAXW; ++r)
        if (r < c.W) u |= a.bits[r][myw];
#pragma unroll
      for (int r = 0; r < MAXW; ++r)
        if (r < c.W) a.ubits[r][myw] = u;
      const long long left = a.n - myw * 32;   // coordinates of this word that exist
      if (left < 32) u &= left > 0 ? ((1u << left) - 1u) : 0u;
    }
    if (__ballot_sync(0xffffffffu, u != 0u) == 0u) continue;
    const int mine = __popc(u);
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    {
      int pos = incl - mine;
      uint32_t bits = u;
      while (bits) {
        const int b = __ffs(bits) - 1;
        bits &= bits - 1;
        list[pos++] = (uint16_t)(lane * 32 + b);
      }
    }
    __syncwarp();
    for (int e0 = 0; e0 < total; e0 += 64) {
      long long idx[2];
      bool on[2];
      float v[2][MAXW];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int e = e0 + t * 32 + lane;
        on[t] = e < total;
        idx[t] = wb * 32 + (on[t] ? (int)list[e] : 0);
        if (on[t]) {
#pragma unroll
          for (int r = 0; r < MAXW; ++r)
            if (r < c.W) v[t][r] = a.grad[r][idx[t]];
        }
      }
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (on[t]) {
          float acc = v[t][0];
#pragma unroll
          for (int r = 1; r < MAXW; ++r)
            if (r < c.W) acc += v[t][r];
          acc *= a.scale;
          sq += acc * acc;
          ++cnt;
#pragma unroll
          for (int r = 0; r < MAXW; ++r)
            if (r < c.W) a.grad[r][idx[t]] = acc;
        }
    }
    __syncwarp();  // the list is rewritten by the next trip
  }
  if (a.count_out) {
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0 && cnt) atomicAdd(reinterpret_cast<unsigned long long*>(a.count_out), (unsigned long long)cnt);
  }
  const float bs = block_sum(sq, red);
  if (threadIdx.x == 0) a.cta_partials[blockIdx.x] = bs;
  __threadfence_system();
  grid_barrier(c.grid_counter, gen, c.err);
  publish_norm(c, a.cta_partials, a.norm_slots);
  peer_signal(c, 1);
  peer_wait(c, 1, c.seq);
  if (a.mask_u8) {
    const uint32_t* ub = a.ubits[c.rank];
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nth = (long long)gridDim.x * blockDim.x;
    for (long long q = tid; q * 4 < a.n; q += nth) {
      const long long i = q * 4;
      const uint32_t word = ub[i >> 5];
      const uint32_t nib = (word >> (i & 31)) & 0xFu;
      if (i + 4 <= a.n) {
        uchar4 m;
        m.x = nib & 1u; m.y = (nib >> 1) & 1u; m.z = (nib >> 2) & 1u; m.w = (nib >> 3) & 1u;
        *reinterpret_cast<uchar4*>(a.mask_u8 + i) = m;
      } else {
        for (long long j = i; j < a.n; ++j) a.mask_u8[j] = (nib >> (j - i)) & 1u;
      }
    }
  }
  collect_norm(c, a.norm_slots, a.sumsq_out, a.accumulate);
}

static int g_sms = 0;
static int num_sms() {
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sms;
}

template <typename K, typename A>
static int coop_launch(K kern, const A& args, int grid, int threads, size_t smem, cudaStream_t st) {
  void* params[] = {const_cast<A*>(&args)};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), dim3(grid), dim3(threads), params, smem, st);
  return e == cudaSuccess ? 0 : -4;
}

}  // namespace sga

using namespace sga;

SGA_API int sga_p2p_allreduce(const SgaPeerDesc* d, void* const* bufs, long long n, float scale, float* grad,
                              const int* idx, float factor, int do_pack, int zero_after_pack, int do_scatter,
                              int block_x, int rs_only, void* const* norm_slots, float* cta_partials, float* sumsq_out, int accumulate,
                              int max_ctas, void* stream) {
  if (d->W > MAXW) return -1;
  AllreduceArgs a;
  a.c = make_ctx(d);
  for (int i = 0; i < MAXW; ++i) {
    a.buf[i] = i < d->W ? reinterpret_cast<float*>(bufs[i]) : nullptr;
    a.norm_slots[i] = i < d->W ? reinterpret_cast<float*>(norm_slots[i]) : nullptr;
  }
  a.n = n; a.scale = scale; a.grad = grad; a.idx = idx; a.factor = factor;
  if (block_x != 0) {
    if (block_x < 4 || (block_x & (block_x - 1)) || n % block_x || (reinterpret_cast<uintptr_t>(grad) & 15)) return -6;
  }
  a.do_pack = do_pack; a.zero_after_pack = zero_after_pack; a.do_scatter = do_scatter; a.rs_only = rs_only;
  a.block_x = block_x;
  a.cta_partials = cta_partials; a.sumsq_out = sumsq_out; a.accumulate = accumulate;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaMemsetAsync(a.c.grid_counter, 0, sizeof(int), st);
  int grid = num_sms();  // one CTA per SM: the grid must be co-resident, beside the backward pass's GEMM CTAs
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  long long need = (n + 2047) / 2048;
  if (need < 1) need = 1;
  if (need < grid) grid = (int)need;
  return coop_launch(p2p_allreduce_kernel, a, grid, 512, 0, st);
}

SGA_API int sga_p2p_mask_union(const SgaPeerDesc* d, void* const* grads, void* const* bits, void* const* ubits,
                               long long n, float scale, uint8_t* mask_u8, void* const* norm_slots,
                               float* cta_partials, float* sumsq_out, int accumulate, long long* count_out,
                               int max_ctas, void* stream) {
  if (d->W > MAXW) return -1;
  MaskUnionArgs a;
  a.c = make_ctx(d);
  for (int i = 0; i < MAXW; ++i) {
    a.grad[i] = i < d->W ? reinterpret_cast<float*>(grads[i]) : nullptr;
    a.bits[i] = i < d->W ? reinterpret_cast<const uint32_t*>(bits[i]) : nullptr;
    a.ubits[i] = i < d->W ? reinterpret_cast<uint32_t*>(ubits[i]) : nullptr;
    a.norm_slots[i] = i < d->W ? reinterpret_cast<float*>(norm_slots[i]) : nullptr;
  }
  a.n = n; a.scale = scale; a.mask_u8 = mask_u8;
  a.cta_partials = cta_partials; a.sumsq_out = sumsq_out; a.accumulate = accumulate; a.count_out = count_out;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaMemsetAsync(a.c.grid_counter, 0, sizeof(int), st);
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  long long need = (n + 16383) / 16384;
  if (need < 1) need = 1;
  if (need < grid) grid = (int)need;
  return coop_launch(p2p_mask_union_kernel, a, grid, 512, 0, st);
}

// ---------------------------------------------------------- symmetric memory
SGA_API int sga_symm_alloc(long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();  // a failed allocation must not poison the next runtime call
    return -(int)e;
  }
  e = cudaMemset(*out, 0, (size_t)bytes);
  if (e != cudaSuccess) return -(int)e;
  // The fill runs on the default stream, which non-blocking streams do not wait for: finish it here,
  // so that no kernel on another stream can write the new buffer before it has been zeroed.
  e = cudaDeviceSynchronize();
  return e == cudaSuccess ? 0 : -(int)e;
}
SGA_API int sga_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
SGA_API int sga_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -1;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
SGA_API int sga_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -(int)e;
}
SGA_API int sga_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }
