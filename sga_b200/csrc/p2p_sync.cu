// Fused compute + collective kernels over NVLink peer memory (plain P2P loads
// and stores issued from the kernel; no TMA from peer memory, no multicast).
//
//   sga_p2p_allreduce        [pack ->] two-shot all-reduce of a symmetric fp32
//                            buffer (owner reduces its slice in rank order and
//                            writes the result to every peer) [-> scatter],
//                            with the squared norm of the reduced payload
//   sga_p2p_mask_union       OR of the ranks' bit masks + reduction of the
//                            masked entries of the gradient bucket, in place
//   sga_bucket_index_sync    per-bucket exact top-k of |grad + residual| by a
//                            two-digit radix select, (index, value) pairs
//                            pushed into every peer's receive slot, selected
//                            coordinates zeroed (what stays is the residual),
//                            then a rank-ordered scatter-add of all received
//                            lists into the dense staging buffer with its norm
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
  if (a.do_pack) {
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
  if (a.do_scatter) {
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
  for (long long w = w0 + warp; w < w1; w += nwarps) {
    uint32_t u = 0;
#pragma unroll
    for (int r = 0; r < MAXW; ++r)
      if (r < c.W) u |= a.bits[r][w];
    const long long i = w * 32 + lane;
    if (((u >> lane) & 1u) && i < a.n) {
      float v[MAXW];
#pragma unroll
      for (int r = 0; r < MAXW; ++r)
        if (r < c.W) v[r] = a.grad[r][i];
      float acc = v[0];
#pragma unroll
      for (int r = 1; r < MAXW; ++r)
        if (r < c.W) acc += v[r];
      acc *= a.scale;
      sq += acc * acc;
      ++cnt;
#pragma unroll
      for (int r = 0; r < MAXW; ++r)
        if (r < c.W) a.grad[r][i] = acc;
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < MAXW; ++r)
        if (r < c.W) a.ubits[r][w] = u;
    }
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

// ------------------------------------------------------ bucket index sync
constexpr int IS_THREADS = 1024;
constexpr int IS_TILE = IS_THREADS * 4;
constexpr int IS_LIST = 8192;  // per-CTA list of the low key halves met inside the crossing bin
constexpr int IS_SMEM = 32772 * 4 + IS_LIST * 2;

struct IndexSyncArgs {
  PeerCtx c;
  float* acc;         // local bucket: gradient + residual
  long long n;
  int k;              // exact number selected per rank
  unsigned* hist1;    // [32769] zero on entry, zero on exit
  unsigned* hist2;    // [65536] zero on entry, zero on exit
  int* cta_gt;        // [grid]
  int* cta_eq;        // [grid]
  int2* slots[MAXW];  // slots[p]: peer p's receive area [W][kcap]
  int kcap;
  float* comm;        // local dense staging (zero on entry)
  uint32_t* touched;  // local bit mask [ceil(n/32)] (written here)
  float scale;
  float* cta_partials;
  float* sumsq_out;
  int accumulate;
  int mode;           // 0 = full exchange; 1 = select only: write the bit mask of the selection to `touched`
  int zero_selected;  // mode 0: zero selected coordinates of acc (residual write-back)
  unsigned* result;   // [4]: threshold key, need_ties, n_above, k actually produced
};

__device__ __forceinline__ uint32_t key_of(float x) { return __float_as_uint(x) & 0x7FFFFFFFu; }

// Four consecutive values from element i (a multiple of 4); returns how many lie inside [0, limit)
// (0 when i is past it). Entries past the end are left at zero and must be ignored by the caller.
__device__ __forceinline__ int load4(const float* __restrict__ acc, long long i, long long limit, float (&v)[4]) {
  if (i + 4 <= limit) {
    *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(acc + i);
    return 4;
  }
  int lim = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = 0.f;
    if (i + j < limit) {
      v[j] = acc[i + j];
      lim = j + 1;
    }
  }
  return lim;
}

// Block-wide exclusive scan of one int per thread (1024 threads); returns the
// exclusive prefix, total in `total` (same for all threads).
__device__ __forceinline__ int block_excl_scan(int v, int* warp_tot, int& total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();  // protect warp_tot reuse
  if (lane == 31) warp_tot[wid] = x;
  __syncthreads();
  if (wid == 0) {
    int t = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += y;
    }
    warp_tot[lane] = t;
  }
  __syncthreads();
  total = warp_tot[31];
  const int wp = wid ? warp_tot[wid - 1] : 0;
  return wp + x - v;
}

// Find, over a histogram of `nb` bins read from global memory, the largest bin
// b with suffix_count(b) >= want; returns b and above = count in bins > b.
// All threads of the block participate; result broadcast through shared memory.
__device__ __forceinline__ void find_bin(const unsigned* hist, int nb, long long want, int* sh_i, int& b_out,
                                         long long& above_out, int* warp_tot) {
  // each thread owns a contiguous chunk of bins, scanned from the top
  const int per = (nb + IS_THREADS - 1) / IS_THREADS;
  const int t = threadIdx.x;
  // thread t owns bins [nb - (t+1)*per, nb - t*per) (descending ownership)
  const int hi = nb - t * per;
  const int lo = max(0, hi - per);
  int mysum = 0;
  for (int i = hi - 1; i >= lo; --i) mysum += (int)hist[i];
  int total;
  const int before = block_excl_scan(mysum, warp_tot, total);  // count in bins above my chunk
  if (t == 0) { sh_i[0] = -1; sh_i[1] = 0; }
  __syncthreads();
  if ((long long)before < want && (long long)before + mysum >= want && hi > 0) {
    int run = before;
    for (int i = hi - 1; i >= lo; --i) {
      const int h = (int)hist[i];
      if ((long long)run + h >= want) { sh_i[0] = i; sh_i[1] = run; break; }
      run += h;
    }
  }
  __syncthreads();
  b_out = sh_i[0];
  above_out = sh_i[1];
  __syncthreads();
}

__global__ void __launch_bounds__(IS_THREADS, 1) bucket_index_sync_kernel(const IndexSyncArgs a) {
  extern __shared__ unsigned sh_hist[];  // 32769 counters, then the crossing-bin list
  unsigned short* sh_list = reinterpret_cast<unsigned short*>(sh_hist + 32772);
  __shared__ int sh_nlist;
  __shared__ int warp_tot[32];
  __shared__ int tile_cnt[64];
  __shared__ int sh_i[4];
  __shared__ float red[IS_THREADS];
  const PeerCtx& c = a.c;
  int gen = 0;
  const int G = gridDim.x;
  // contiguous element range of this CTA, multiple of IS_TILE
  const long long tiles = (a.n + IS_TILE - 1) / IS_TILE;
  const long long tpc = (tiles + G - 1) / G;
  const long long r0 = min(a.n, (long long)blockIdx.x * tpc * IS_TILE);
  const long long r1 = min(a.n, r0 + tpc * IS_TILE);

  // ---- phase 1: histogram of the top 16 key bits
  for (int i = threadIdx.x; i < 32769; i += IS_THREADS) sh_hist[i] = 0;
  if (a.mode == 0) {
    for (long long w = (r0 >> 5) + threadIdx.x; w < ((r1 + 31) >> 5); w += IS_THREADS) a.touched[w] = 0;
  }
  __syncthreads();
  const long long lim_all = min(a.n, r1);
  for (long long i = r0 + (long long)threadIdx.x * 4; i < r1; i += 2 * IS_TILE) {
    // two tiles per trip: both loads are in flight before either is used
    float v0[4], v1[4];
    const int l0 = load4(a.acc, i, lim_all, v0);
    const int l1 = load4(a.acc, i + IS_TILE, lim_all, v1);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (j < l0) atomicAdd(&sh_hist[key_of(v0[j]) >> 16], 1u);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (j < l1) atomicAdd(&sh_hist[key_of(v1[j]) >> 16], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 32769; i += IS_THREADS) {
    const unsigned h = sh_hist[i];
    if (h) atomicAdd(&a.hist1[i], h);
  }
  __threadfence();
  grid_barrier(c.grid_counter, gen, c.err);

  // ---- phase 2: crossing bin, then histogram of the low 16 bits inside it
  int bin;
  long long above;
  find_bin(a.hist1, 32769, a.k, sh_i, bin, above, warp_tot);
  // The crossing bin holds a sliver of the bucket. Its low key halves are also kept in a per-CTA
  // list, so that once the threshold is known this CTA can count its keys above / equal to it from the
  // phase-1 histogram and the list instead of reading its range a third time.
  if (threadIdx.x == 0) sh_nlist = 0;
  __syncthreads();
  for (long long i = r0 + (long long)threadIdx.x * 4; i < r1; i += 2 * IS_TILE) {
    float v0[4], v1[4];
    const int l0 = load4(a.acc, i, lim_all, v0);
    const int l1 = load4(a.acc, i + IS_TILE, lim_all, v1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t k0 = key_of(v0[j]), k1 = key_of(v1[j]);
      if (j < l0 && (int)(k0 >> 16) == bin) {
        atomicAdd(&a.hist2[k0 & 0xFFFFu], 1u);
        const int at = atomicAdd(&sh_nlist, 1);
        if (at < IS_LIST) sh_list[at] = (unsigned short)(k0 & 0xFFFFu);
      }
      if (j < l1 && (int)(k1 >> 16) == bin) {
        atomicAdd(&a.hist2[k1 & 0xFFFFu], 1u);
        const int at = atomicAdd(&sh_nlist, 1);
        if (at < IS_LIST) sh_list[at] = (unsigned short)(k1 & 0xFFFFu);
      }
    }
  }
  __threadfence();
  grid_barrier(c.grid_counter, gen, c.err);

  // ---- phase 3: exact threshold key T and the number of ties to take
  int lowbin;
  long long above2;
  find_bin(a.hist2, 65536, (long long)a.k - above, sh_i, lowbin, above2, warp_tot);
  const uint32_t T = ((uint32_t)bin << 16) | (uint32_t)(lowbin & 0xFFFF);
  const long long n_gt = above + above2;           // keys strictly greater than T
  const int need = (int)((long long)a.k - n_gt);   // ties (key == T) to take, in index order
  int my_gt = 0, my_eq = 0;
  const int nlist = sh_nlist;  // written before the grid barrier
  if (nlist <= IS_LIST) {
    // keys in higher bins (this CTA's own phase-1 histogram) + listed keys of the crossing bin
    for (int bb = bin + 1 + threadIdx.x; bb < 32769; bb += IS_THREADS) my_gt += (int)sh_hist[bb];
    for (int q = threadIdx.x; q < nlist; q += IS_THREADS) {
      const int lowk = sh_list[q];
      my_gt += lowk > (lowbin & 0xFFFF);
      my_eq += lowk == (lowbin & 0xFFFF);
    }
  } else {
    // the list overflowed (a bucket crowded into one bin): count by reading the range again
    for (long long i = r0 + (long long)threadIdx.x * 4; i < r1; i += 2 * IS_TILE) {
      float v0[4], v1[4];
      const int l0 = load4(a.acc, i, lim_all, v0);
      const int l1 = load4(a.acc, i + IS_TILE, lim_all, v1);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t k0 = key_of(v0[j]), k1 = key_of(v1[j]);
        my_gt += (j < l0 && k0 > T) + (j < l1 && k1 > T);
        my_eq += (j < l0 && k0 == T) + (j < l1 && k1 == T);
      }
    }
  }
  {
    int tot;
    block_excl_scan(my_gt, warp_tot, tot);
    if (threadIdx.x == 0) a.cta_gt[blockIdx.x] = tot;
    block_excl_scan(my_eq, warp_tot, tot);
    if (threadIdx.x == 0) a.cta_eq[blockIdx.x] = tot;
  }
  __threadfence();
  grid_barrier(c.grid_counter, gen, c.err);
  // hist1 is dead now: restore its zero-on-exit invariant
  for (int i = blockIdx.x * IS_THREADS + threadIdx.x; i < 32769; i += G * IS_THREADS) a.hist1[i] = 0;

  // ---- phase 4: ordered compaction, push to every peer, residual write-back
  long long gt_before = 0, eq_before = 0;
  {
    int g = 0, e = 0;
    for (int i = threadIdx.x; i < (int)blockIdx.x; i += IS_THREADS) { g += a.cta_gt[i]; e += a.cta_eq[i]; }
    int tot;
    block_excl_scan(g, warp_tot, tot);
    gt_before = tot;
    block_excl_scan(e, warp_tot, tot);
    eq_before = tot;
  }
  long long out_base = gt_before + min((long long)need, eq_before);
  long long tie_base = eq_before;
  if (a.mode == 0 && c.prev_seq > 0) peer_wait(c, 1, c.prev_seq);  // peers finished reading my previous payload
  float nv[4];
  int nlim = load4(a.acc, r0 + (long long)threadIdx.x * 4, lim_all, nv);
  for (long long t0 = r0; t0 < r1; t0 += IS_TILE) {
    const long long i = t0 + (long long)threadIdx.x * 4;
    float v[4];
    uint32_t key[4];
    const int lim = nlim;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = nv[j];
      key[j] = key_of(v[j]);
    }
    // the next tile's values are on their way while this one is scanned
    nlim = load4(a.acc, i + IS_TILE, lim_all, nv);
    // Ordered positions with one barrier per tile: a packed (greater | ties << 16) count is scanned
    // inside each warp, the warp totals go through shared memory (double-buffered by tile parity), and
    // every warp derives from the 32 totals where its own ties and its own selections start.
    int gtc = 0, eqc = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      gtc += j < lim && key[j] > T;
      eqc += j < lim && key[j] == T;
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int packed = gtc | (eqc << 16);
    int incl = packed;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    int* wcnt = tile_cnt + (((t0 - r0) / IS_TILE) & 1) * 32;
    if (lane == 31) wcnt[wid] = incl;
    __syncthreads();
    const int wp = wcnt[lane];                 // lane l looks at warp l's totals
    const int g_l = wp & 0xFFFF, e_l = wp >> 16;
    int e_incl = e_l;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, e_incl, o);
      if (lane >= o) e_incl += y;
    }
    const long long ties_before_l = tie_base + (e_incl - e_l);
    const int take_l = (int)max(0LL, min((long long)e_l, (long long)need - ties_before_l));
    const int s_l = g_l + take_l;              // selections of warp l in this tile
    int s_incl = s_l;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, s_incl, o);
      if (lane >= o) s_incl += y;
    }
    const int eq_tot = __shfl_sync(0xffffffffu, e_incl, 31);
    const int sel_tot = __shfl_sync(0xffffffffu, s_incl, 31);
    const int warp_tie0 = __shfl_sync(0xffffffffu, e_incl - e_l, wid);   // ties of the tile before my warp
    const int warp_sel0 = __shfl_sync(0xffffffffu, s_incl - s_l, wid);   // selections of the tile before my warp
    const int eq_pre = warp_tie0 + ((incl - packed) >> 16);               // ties of the tile before my elements
    int selc = 0;
    uint32_t selbits = 0;
    {
      long long tr = tie_base + eq_pre;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j < lim) {
          bool s = key[j] > T;
          if (key[j] == T) { s = tr < need; ++tr; }
          if (s) { selbits |= 1u << j; ++selc; }
        }
      }
    }
    int sc_incl = selc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, sc_incl, o);
      if (lane >= o) sc_incl += y;
    }
    const int sel_pre = warp_sel0 + sc_incl - selc;
    if (a.mode == 1) {
      // compose the 32-bit mask word from 8 consecutive lanes' nibbles
      uint32_t word = selbits << ((threadIdx.x & 7) * 4);
      word |= __shfl_xor_sync(0xffffffffu, word, 1);
      word |= __shfl_xor_sync(0xffffffffu, word, 2);
      word |= __shfl_xor_sync(0xffffffffu, word, 4);
      if ((threadIdx.x & 7) == 0 && i < ((a.n + 31) & ~31LL)) a.touched[i >> 5] = word;
    } else if (selc) {
      long long pos = out_base + sel_pre;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (selbits & (1u << j)) {
          if (pos < a.kcap) {
            int2 pr;
            pr.x = (int)(i + j);
            pr.y = __float_as_int(v[j]);
#pragma unroll
            for (int r = 0; r < MAXW; ++r)
              if (r < c.W) a.slots[r][(long long)c.rank * a.kcap + pos] = pr;
          } else {
            atomicOr(c.err, SGA_ERR_CAPACITY);
          }
          ++pos;
          if (a.zero_selected) a.acc[i + j] = 0.f;
        }
      }
    }
    out_base += sel_tot;
    tie_base += eq_tot;
  }
  if (blockIdx.x == G - 1 && threadIdx.x == 0 && a.result) {
    a.result[0] = T;
    a.result[1] = (unsigned)need;
    a.result[2] = (unsigned)n_gt;
    a.result[3] = (unsigned)out_base;
  }
  __threadfence_system();
  grid_barrier(c.grid_counter, gen, c.err);
  for (int i = blockIdx.x * IS_THREADS + threadIdx.x; i < 65536; i += G * IS_THREADS) a.hist2[i] = 0;
  if (a.mode == 1) return;
  peer_signal(c, 0);
  peer_wait(c, 0, c.seq);

  // ---- phase 5: rank-ordered scatter-add of every list into my element range
  const int2* my_slots = a.slots[c.rank];
  for (int r = 0; r < c.W; ++r) {
    const int2* list = my_slots + (long long)r * a.kcap;
    if (threadIdx.x < 2) {
      const long long target = threadIdx.x == 0 ? r0 : r1;
      int lo = 0, hi = a.k;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if ((long long)list[mid].x < target) lo = mid + 1; else hi = mid;
      }
      sh_i[threadIdx.x] = lo;
    }
    __syncthreads();
    const int lo = sh_i[0], hi = sh_i[1];
    for (int j = lo + threadIdx.x; j < hi; j += IS_THREADS) {
      const int2 pr = list[j];
      const long long p = pr.x;
      if (p >= r0 && p < r1) {
        a.comm[p] += __int_as_float(pr.y) * a.scale;
        atomicOr(&a.touched[p >> 5], 1u << (p & 31));
      } else {
        atomicOr(c.err, SGA_ERR_BOUNDS);
      }
    }
    __syncthreads();
  }
  // norm^2 of the reduced sparse gradient over the touched coordinates
  float sq = 0.f;
  for (long long w = (r0 >> 5) + threadIdx.x; w < ((r1 + 31) >> 5); w += IS_THREADS) {
    uint32_t bits = a.touched[w];
    while (bits) {
      const int b = __ffs(bits) - 1;
      bits &= bits - 1;
      const float x = a.comm[w * 32 + b];
      sq += x * x;
    }
  }
  const float bs = block_sum(sq, red);
  if (threadIdx.x == 0) a.cta_partials[blockIdx.x] = bs;
  __threadfence();
  grid_barrier(c.grid_counter, gen, c.err);
  peer_signal(c, 1);  // done reading my receive slots
  if (blockIdx.x == 0 && threadIdx.x == 0 && a.sumsq_out) {
    float t = 0.f;
    for (int i = 0; i < G; ++i) t += a.cta_partials[i];
    a.sumsq_out[0] = a.accumulate ? a.sumsq_out[0] + t : t;
  }
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
                              int rs_only, void* const* norm_slots, float* cta_partials, float* sumsq_out, int accumulate,
                              int max_ctas, void* stream) {
  if (d->W > MAXW) return -1;
  AllreduceArgs a;
  a.c = make_ctx(d);
  for (int i = 0; i < MAXW; ++i) {
    a.buf[i] = i < d->W ? reinterpret_cast<float*>(bufs[i]) : nullptr;
    a.norm_slots[i] = i < d->W ? reinterpret_cast<float*>(norm_slots[i]) : nullptr;
  }
  a.n = n; a.scale = scale; a.grad = grad; a.idx = idx; a.factor = factor;
  a.do_pack = do_pack; a.zero_after_pack = zero_after_pack; a.do_scatter = do_scatter; a.rs_only = rs_only;
  a.cta_partials = cta_partials; a.sumsq_out = sumsq_out; a.accumulate = accumulate;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaMemsetAsync(a.c.grid_counter, 0, sizeof(int), st);
  int grid = num_sms();
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

SGA_API int sga_bucket_index_sync(const SgaPeerDesc* d, float* acc, long long n, int k, unsigned* hist1,
                                  unsigned* hist2, int* cta_gt, int* cta_eq, void* const* slots, int kcap,
                                  float* comm, unsigned* touched, float scale, float* cta_partials,
                                  float* sumsq_out, int accumulate, int mode, int zero_selected, unsigned* result,
                                  int max_ctas, void* stream) {
  if (d->W > MAXW) return -1;
  if (n <= 0 || n >= (1LL << 31) || k < 1 || k > n) return -6;
  if (mode == 0 && k > kcap) return -7;
  IndexSyncArgs a;
  a.c = make_ctx(d);
  a.acc = acc; a.n = n; a.k = k; a.hist1 = hist1; a.hist2 = hist2; a.cta_gt = cta_gt; a.cta_eq = cta_eq;
  for (int i = 0; i < MAXW; ++i) a.slots[i] = (i < d->W && slots) ? reinterpret_cast<int2*>(slots[i]) : nullptr;
  a.kcap = kcap; a.comm = comm; a.touched = touched; a.scale = scale;
  a.cta_partials = cta_partials; a.sumsq_out = sumsq_out; a.accumulate = accumulate;
  a.mode = mode; a.zero_selected = zero_selected; a.result = result;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(bucket_index_sync_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, IS_SMEM) !=
        cudaSuccess)
      return -3;
    attr = true;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaMemsetAsync(a.c.grid_counter, 0, sizeof(int), st);
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  long long need = (n + IS_TILE - 1) / IS_TILE;
  if (need < grid) grid = (int)need;
  return coop_launch(bucket_index_sync_kernel, a, grid, IS_THREADS, IS_SMEM, st);
}

// ---------------------------------------------------------- symmetric memory
SGA_API int sga_symm_alloc(long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();  // a failed allocation must not poison the next runtime call
    return -(int)e;
  }
  e = cudaMemset(*out, 0, (size_t)bytes);
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
