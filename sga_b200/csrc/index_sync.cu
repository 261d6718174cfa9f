// Rank-local sparse gradient synchronisation of one bucket: exact top-k of a
// score over the bucket, (index, value) pairs pushed into every peer's receive
// area over NVLink peer memory, rank-ordered scatter-add on the receive side.
//
// The bucket is read from HBM once. A 1/64 sample (one hashed 16-byte group in
// every 1 KiB) gives a lower bound of the k-th largest key with a six-sigma
// margin; one streaming pass keeps every element at or above the bound as a
// candidate (1.1 to 1.6 k of them) and counts the candidates' first radix
// digit (12 bits) on the way. Everything else that makes the selection exact
// -- the remaining 19 key bits in one pass (11-bit digit + a 512 K-bin fine
// histogram), the index-order tie cut, the per-segment counts and their scan
// -- touches the candidates only. If the sample bound turns out too high
// (fewer than k candidates) a second pass takes every non-zero element, so the
// result is exact for any input.
//
// Chain per bucket: sample, filter, filter (level 1, normally returns at once),
// digit, count, emit, reduce; each is launched as a programmatic dependent of
// its predecessor, so its launch latency hides behind the predecessor's tail.
//
// Every kernel here is an ordinary launch with at most 20 KB of shared memory
// and 256 threads per CTA, so its CTAs fit beside the persistent GEMM CTAs of
// the backward pass they overlap with. Nothing waits on another CTA of the same
// grid: serial steps (histogram scans, prefix sums, flag signalling) are done by
// whichever CTA takes the last ticket. The only waits are on peers' flags, bounded.
//
// Semantics: the selected set is the k coordinates with the largest keys
// (key = bits of |score| without the sign), ties at the k-th key taken in index
// order; coordinates whose key is zero are never selected, so a bucket with
// fewer than k non-zero scores selects exactly those. Scores follow
// sga/plugins/scores.py:147-269 of the reference (update, abs_g, abs_m, coi),
// with the gradient being gradient + residual of this rank.
//
// Candidates of segment s (8192 elements) live at [s * 8192, s * 8192 + count)
// of the candidate arrays, so no allocation cursor and no overflow exists; the
// payload a rank pushes is grouped by segment (offset table pushed with it),
// and the receiver's CTA for a range of segments adds the ranks' pairs in rank
// order, which makes the reduced gradient bit-identical on every rank.
//
// Replaces sga/kernels.py:63-81 (pack), sga/plugins/selection/_histogram.py and
// the all-reduce of sga/backends/torch_pipelined_index.py:503-520.
//
// Compiled without fast-math and without FMA contraction: the score formulas
// round operation by operation like their PyTorch reference.
#include "common.cuh"
#include "peer.cuh"
#include <stdlib.h>

namespace sga {

constexpr int IS_SEG = 8192;          // elements per segment (one warp streams a segment)
constexpr int IS_SEG_PER_RANGE = 4;   // receive-side CTA range: 4 segments = 32768 elements
constexpr int IS_THREADS = 256;
constexpr int IS_ABINS = 4096;        // first digit, also the sample's histogram: key >> 19
constexpr int IS_BBINS = 2048;        // second digit: bits 18..8
constexpr int IS_FBINS = 1 << 19;     // fine histogram of the low 19 bits inside the crossing first-digit bin
constexpr int IS_REP = 8;             // replicas of the two coarse global histograms
constexpr int IS_CU = 4;             // candidate trips (of 32, or of 256 in the reduce) whose loads are issued together
constexpr int IS_WBINS = 1024;        // the filter's shared-memory window of first-digit bins (4 KB: its CTAs fit beside a GEMM CTA)

// Word offsets inside the state block (unsigned[64], zeroed by the host before each bucket).
enum {
  ST_TLO = 0, ST_LEVEL, ST_C, ST_SKIP, ST_BA, ST_ABOVE, ST_T, ST_NEED, ST_EQ, ST_ICUT, ST_NSEL, ST_SAMPLES,
  ST_TOP, ST_INVLOW,  // first-digit bins in use: highest bin + 1, IS_ABINS - lowest bin (0 = none)
  ST_TICKET0 = 16  // tickets: one word per kernel of the chain
};

struct ISyncArgs {
  PeerCtx c;
  float* acc;            // gradient + residual of this rank
  const float* w;        // fp32 master weights / moments: only for scores other than abs_g
  const float* m;
  const float* v;
  long long n;
  int k;
  int nseg;
  int score;             // 0 update, 1 abs_g, 2 abs_m, 3 coi
  int adams;
  float beta1, omb1, beta2, omb2, bc1, bc2, eps;
  const int* span_start; // [nspan + 1] parameter spans of the bucket (score update: weight decay per span)
  const float* span_wd;  // [nspan]
  int nspan;
  int gshift;            // the sample takes one 16-byte group in every 2^gshift
  unsigned* state;
  unsigned* histA;       // [8][4096] first-digit replicas: zero on entry, zero on exit
  unsigned* histB;       // [8][2048] second-digit replicas (zero on exit), then [2^19] fine bins (zeroed by the sample)
  int* cand_idx;         // [nseg * IS_SEG]
  unsigned* cand_key;
  float* cand_val;
  int* segcnt;           // [nseg] candidates per segment
  int* segsel;           // [nseg] selected per segment
  int* segeq;            // [nseg] ties at the threshold per segment
  int* roff;             // [nseg + 1] exclusive scan of segsel
  float* partials;       // [number of receive ranges]
  int2* slots[MAXW];     // slots[p]: peer p's pair area [W][kcap]
  int* hdr[MAXW];        // hdr[p]: peer p's offset tables [W][hstride]
  int kcap, hstride;
  float* comm;           // dense staging of the reduced sparse gradient
  float scale;
  float* sumsq_out;
  int accumulate;
  int zero_selected;
  unsigned* bits;        // select-only mode: bit mask of the selection (zeroed by the host)
  unsigned* result;      // [4]: threshold key, ties taken, keys above the threshold, pairs produced
  unsigned long long* wait_ns;  // nullable: nanoseconds CTA 0 spent waiting on peers' flags are added here
  unsigned* reduce_ticket;  // the reduce kernel's own ticket word (zero between launches): the reduce may run
                            // long after its bucket's chain, when the shared state block belongs to another bucket
};

// Programmatic dependent launch: every kernel of the chain first lets the next one be scheduled
// (its CTAs then sit in their own wait until this grid has finished and its writes are visible),
// then waits for its predecessor. Both are no-ops for a launch without the attribute.
__device__ __forceinline__ void chain_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// peer_wait with the time CTA 0 spent in it added to *wait_ns: how long this rank stood still for
// slower peers, as opposed to working (the step's synchronisation time is reported with and without it).
__device__ __forceinline__ void timed_peer_wait(const PeerCtx& c, int slot, int target, unsigned long long* wait_ns) {
  const bool timing = wait_ns != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
  const unsigned long long t0 = timing ? global_ns() : 0ULL;
  peer_wait(c, slot, target);
  if (timing) atomicAdd(wait_ns, global_ns() - t0);
}

__device__ __forceinline__ unsigned key_bits(float x) { return __float_as_uint(x) & 0x7FFFFFFFu; }
__device__ __forceinline__ unsigned ldv(const unsigned* p) { return *reinterpret_cast<const volatile unsigned*>(p); }

// The CTA that takes the last ticket of a grid sees every other CTA's writes. The block barrier
// orders the CTA's writes before thread 0's fence, and the fence is cumulative, so one thread per
// CTA fences (at system scope when the writes went to peers' memory) instead of all 256.
template <bool SYSTEM = false>
__device__ __forceinline__ bool last_cta(unsigned* ticket) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (SYSTEM) __threadfence_system(); else __threadfence();
    const unsigned t = atomicAdd(ticket, 1u);
    s_last = (t == gridDim.x - 1);
    if (s_last) {
      *ticket = 0;
      __threadfence();
    }
  }
  __syncthreads();
  if (s_last) __threadfence();
  return s_last != 0;
}

// Block-wide exclusive scan of one value per thread (256 threads).
__device__ __forceinline__ unsigned block_excl_scan256(unsigned v, unsigned* sh, unsigned& total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  unsigned x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();
  if (lane == 31) sh[wid] = x;
  __syncthreads();
  if (wid == 0) {
    unsigned t = lane < IS_THREADS / 32 ? sh[lane] : 0;
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      const unsigned y = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += y;
    }
    if (lane < IS_THREADS / 32) sh[lane] = t;
  }
  __syncthreads();
  total = sh[IS_THREADS / 32 - 1];
  const unsigned wp = wid ? sh[wid - 1] : 0;
  const unsigned r = wp + x - v;
  __syncthreads();
  return r;
}

// Over the sum of `rep` replicas hist[r * nb + i] (global): the largest bin b <= top whose suffix
// count (bins b..top) reaches `want`, and the count in the bins above it. Scans downwards from
// `top`, 256 bins per round (one per thread, every replica's load in flight at once), and stops at
// the crossing, so a crossing near the top costs one round. Returns false when bins low..top hold
// fewer than `want`. One CTA; result uniform over its threads.
__device__ __forceinline__ bool find_suffix_bin(const unsigned* hist, int nb, int rep, unsigned want, int top, int low,
                                                unsigned* sh, unsigned& bin, unsigned& above) {
  __shared__ unsigned s_res[2];
  if (threadIdx.x == 0) { s_res[0] = 0xFFFFFFFFu; s_res[1] = 0; }
  unsigned run = 0;
  for (int hi = top; hi >= low; hi -= IS_THREADS) {
    const int i = hi - (int)threadIdx.x;
    unsigned h = 0;
    if (i >= low)
      for (int r = 0; r < rep; ++r) h += __ldcg(hist + r * nb + i);
    unsigned total;
    const unsigned before = run + block_excl_scan256(h, sh, total);
    if (before < want && before + h >= want) { s_res[0] = (unsigned)i; s_res[1] = before; }
    __syncthreads();
    if (s_res[0] != 0xFFFFFFFFu) break;
    run += total;
  }
  __syncthreads();
  bin = s_res[0];
  above = s_res[1];
  __syncthreads();
  return bin != 0xFFFFFFFFu;
}

// The same over all `NB` bins in one round: thread t owns bins NB-1 - t*PER .. NB - (t+1)*PER
// (descending), with every replica's load in flight at once, then one block scan and a walk over
// the owner's own bins. One CTA of 256 threads; result uniform over its threads.
template <int NB>
__device__ __forceinline__ bool find_suffix_bin_all(const unsigned* hist, int rep, unsigned want, unsigned* sh,
                                                    unsigned& bin, unsigned& above) {
  constexpr int PER = NB / IS_THREADS;
  static_assert(NB % IS_THREADS == 0, "bins must divide over the CTA");
  __shared__ unsigned s_res[2];
  if (threadIdx.x == 0) { s_res[0] = 0xFFFFFFFFu; s_res[1] = 0; }
  unsigned h[PER];
  const int hi = NB - 1 - (int)threadIdx.x * PER;
#pragma unroll
  for (int j = 0; j < PER; ++j) h[j] = 0;
  for (int r = 0; r < rep; ++r)
#pragma unroll
    for (int j = 0; j < PER; ++j) h[j] += __ldcg(hist + r * NB + hi - j);
  unsigned mine = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) mine += h[j];
  unsigned total;
  const unsigned before = block_excl_scan256(mine, sh, total);  // barriers inside order the reset of s_res
  if (before < want && before + mine >= want) {
    unsigned run = before;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (run < want && run + h[j] >= want) { s_res[0] = (unsigned)(hi - j); s_res[1] = run; }
      run += h[j];
    }
  }
  __syncthreads();
  bin = s_res[0];
  above = s_res[1];
  __syncthreads();
  return bin != 0xFFFFFFFFu;
}

// Flush a CTA's shared first-digit histogram into its global replica and widen the global window
// of bins in use.
// sh_hist[i] counts absolute bin min(first + i, IS_ABINS - 1).
__device__ __forceinline__ void flush_first_digit(const unsigned* sh_hist, int nbins, int first, unsigned* replica,
                                                  unsigned* state) {
  __shared__ unsigned s_win[2];
  if (threadIdx.x == 0) { s_win[0] = 0; s_win[1] = 0; }
  __syncthreads();
  unsigned top = 0, invlow = 0;
  for (int j = threadIdx.x; j < nbins; j += IS_THREADS) {
    const unsigned c = sh_hist[j];
    if (c) {
      const int i = min(first + j, IS_ABINS - 1);
      atomicAdd(&replica[i], c);
      top = max(top, (unsigned)i + 1u);
      invlow = max(invlow, (unsigned)(IS_ABINS - i));
    }
  }
  if (top) { atomicMax(&s_win[0], top); atomicMax(&s_win[1], invlow); }
  __syncthreads();
  if (threadIdx.x == 0 && s_win[0]) { atomicMax(state + ST_TOP, s_win[0]); atomicMax(state + ST_INVLOW, s_win[1]); }
}

// Zero bins low..top of every replica (the last CTA, after its scan).
__device__ __forceinline__ void zero_window(unsigned* hist, int nb, int rep, int top, int low) {
  const int w = top - low + 1;
  for (int i = threadIdx.x; i < w * rep; i += IS_THREADS) hist[(i / w) * nb + low + (i % w)] = 0;
}

__device__ __forceinline__ int load4z(const float* __restrict__ p, long long i, long long limit, float (&v)[4]) {
  if (i + 4 <= limit) {
    *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(p + i);
    return 4;
  }
  int lim = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = 0.f;
    if (i + j < limit) { v[j] = p[i + j]; lim = j + 1; }
  }
  return lim;
}

// Weight decay of element i (score update): spans are few, a binary search per 16-byte group.
__device__ __forceinline__ float wd_of(const ISyncArgs& a, long long i) {
  int lo = 0, hi = a.nspan - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((long long)a.span_start[mid] <= i) lo = mid; else hi = mid - 1;
  }
  return a.span_wd[lo];
}

template <int SCORE>
__device__ __forceinline__ unsigned score_key(const ISyncArgs& a, float g, float w, float m0, float v0, float wd) {
  if (SCORE == 1) return key_bits(g);
  if (SCORE == 2) return key_bits(m0);
  const float m1 = m0 * a.beta1 + g * a.omb1;
  const float g2 = (g * a.omb2) * g;
  float mh, vh;
  if (a.adams) {
    mh = m1;
    vh = (m0 * m0) * a.beta2 + g2;
  } else {
    mh = m1 / a.bc1;
    vh = (v0 * a.beta2 + g2) / a.bc2;
  }
  const float u = mh / (sqrtf(vh) + a.eps);
  if (SCORE == 0) return key_bits(wd * w + u);
  float u0;
  if (a.adams) u0 = (m0 * a.beta1) / (sqrtf((m0 * m0) * a.beta2) + a.eps);
  else u0 = ((m0 * a.beta1) / a.bc1) / (sqrtf((v0 * a.beta2) / a.bc2) + a.eps);
  return key_bits(u - u0);
}

// Keys of the four elements from i (lanes past `limit` get key 0, which is never a candidate).
template <int SCORE>
__device__ __forceinline__ void keys4(const ISyncArgs& a, long long i, long long limit, float (&g)[4],
                                      unsigned (&key)[4]) {
  const int lim = load4z(a.acc, i, limit, g);
  float w[4] = {0.f, 0.f, 0.f, 0.f}, m[4] = {0.f, 0.f, 0.f, 0.f}, v[4] = {0.f, 0.f, 0.f, 0.f};
  if (SCORE == 0) load4z(a.w, i, limit, w);
  if (SCORE != 1) load4z(a.m, i, limit, m);
  if (SCORE == 0 || SCORE == 3) load4z(a.v, i, limit, v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float wd = 0.f;
    if (SCORE == 0 && j < lim) wd = wd_of(a, i + j);
    key[j] = j < lim ? score_key<SCORE>(a, g[j], w[j], m[j], v[j], wd) : 0u;
  }
}

// Value and key of the single element i (the filter re-reads its few hits).
template <int SCORE>
__device__ __forceinline__ void key1(const ISyncArgs& a, long long i, float& g, unsigned& key) {
  g = a.acc[i];
  const float w = SCORE == 0 ? a.w[i] : 0.f;
  const float m = SCORE != 1 ? a.m[i] : 0.f;
  const float v = (SCORE == 0 || SCORE == 3) ? a.v[i] : 0.f;
  key = score_key<SCORE>(a, g, w, m, v, SCORE == 0 ? wd_of(a, i) : 0.f);
}

// ------------------------------------------------------------------ sample
// Histogram (4096 bins of key >> 19) of one hashed 16-byte group in every 2^gshift; the CTA that
// finishes last turns it into the candidate bound: the lower edge of the bin at which the sample's
// suffix count reaches the expected share of k plus six standard deviations. With gshift == 0 the
// histogram covers the whole bucket and the bound is exact. The grid also zeroes the fine
// histogram of the digit pass that follows.
template <int SCORE>
__global__ void __launch_bounds__(IS_THREADS) isync_sample_kernel(const ISyncArgs a) {
  chain_enter();
  __shared__ unsigned sh_hist[IS_ABINS];
  __shared__ unsigned sh_scan[8];
  for (int i = threadIdx.x; i < IS_ABINS; i += IS_THREADS) sh_hist[i] = 0;
  {
    uint4* fine = reinterpret_cast<uint4*>(a.histB + IS_REP * IS_BBINS);
    for (int i = blockIdx.x * IS_THREADS + threadIdx.x; i < IS_FBINS / 4; i += gridDim.x * IS_THREADS)
      fine[i] = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  const long long n4 = (a.n + 3) >> 2;
  const long long ngroups = (n4 + (1LL << a.gshift) - 1) >> a.gshift;
  const long long stride = (long long)gridDim.x * IS_THREADS;
  for (long long g0 = (long long)blockIdx.x * IS_THREADS + threadIdx.x; g0 < ngroups; g0 += 4 * stride) {
    float gv[4][4];
    unsigned key[4][4];
    int lim[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {  // four independent groups in flight per thread
      const long long g = g0 + u * stride;
      const unsigned h = a.gshift ? (((unsigned)g * 2654435761u) >> (32 - a.gshift)) : 0u;
      const long long q = (g << a.gshift) + h;
      lim[u] = (g < ngroups && q < n4) ? (int)min(4LL, a.n - q * 4) : 0;
      if (lim[u] > 0) keys4<SCORE>(a, q * 4, a.n, gv[u], key[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (j < lim[u]) atomicAdd(&sh_hist[key[u][j] >> 19], 1u);
  }
  __syncthreads();
  flush_first_digit(sh_hist, IS_ABINS, 0, a.histA + (blockIdx.x % IS_REP) * IS_ABINS, a.state);
  {
    unsigned mine = 0;  // elements this CTA sampled
    for (int i = threadIdx.x; i < IS_ABINS; i += IS_THREADS) mine += sh_hist[i];
    unsigned tot;
    block_excl_scan256(mine, sh_scan, tot);
    if (threadIdx.x == 0 && tot) atomicAdd(a.state + ST_SAMPLES, tot);
  }
  if (!last_cta(a.state + ST_TICKET0 + 0)) return;
  const unsigned samples = ldv(a.state + ST_SAMPLES);
  unsigned want = (unsigned)a.k;
  if (a.gshift) {
    const float ks = (float)a.k * ((float)samples / (float)a.n);
    want = (unsigned)ceilf(ks + 6.0f * sqrtf(ks) + 16.0f);
  }
  const int top = (int)ldv(a.state + ST_TOP) - 1, low = IS_ABINS - (int)ldv(a.state + ST_INVLOW);
  unsigned bin = 0, above = 0;
  bool found = false;
  if (top >= 0) {
    found = find_suffix_bin(a.histA, IS_ABINS, IS_REP, want, top, low, sh_scan, bin, above);
    zero_window(a.histA, IS_ABINS, IS_REP, top, low);
  }
  if (threadIdx.x == 0) {
    a.state[ST_TLO] = found ? (bin << 19) : 0u;
    a.state[ST_TOP] = 0u;
    a.state[ST_INVLOW] = 0u;
  }
}

// ------------------------------------------------------------------ filter
// The one pass over the bucket. A warp streams a segment (8192 elements, 512 per trip with four
// 16-byte loads per lane in flight) and appends the elements whose key reaches the bound to the
// segment's own slice of the candidate arrays; positions come from warp ballots, so there is no
// atomic, no barrier and no overflow. The candidates' first radix digit (key >> 19) is counted in
// a shared-memory histogram on the way and flushed into one of eight global replicas (a handful
// of bins is hot; replicas keep the same-address atomics short). The last CTA either publishes the
// crossing bin of that digit or, when fewer than k candidates were found under the sample bound,
// arms level 1 (every non-zero key), which is the next launch and normally returns at once.
template <int SCORE, int LEVEL>
__global__ void __launch_bounds__(IS_THREADS) isync_filter_kernel(const ISyncArgs a) {
  chain_enter();
  constexpr int HBINS = LEVEL == 0 ? IS_WBINS : IS_ABINS;
  __shared__ unsigned sh_hist[HBINS];
  __shared__ unsigned sh_cnt[IS_THREADS / 32];
  if (LEVEL == 1 && ldv(a.state + ST_LEVEL) != 1u) return;
  unsigned tlo = LEVEL == 0 ? ldv(a.state + ST_TLO) : 1u;
  if (tlo < 1u) tlo = 1u;
  // Level 0 counts the first digit in a shared window of 1024 bins from the bound's bin (64 binades:
  // what lies above lands in the window's last bin, and a crossing found there sends the bucket to
  // level 1), which keeps its shared memory at 4 KB. Level 1, the rare exact fallback, takes the
  // whole range of 4096 bins.
  const unsigned b_lo = LEVEL == 0 ? (tlo >> 19) : 0u;
  unsigned* replica = a.histA + (blockIdx.x % IS_REP) * IS_ABINS;
  for (int i = threadIdx.x; i < HBINS; i += IS_THREADS) sh_hist[i] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  constexpr int U = SCORE == 1 ? 8 : 4;  // 16-byte loads in flight per lane and array
  unsigned warp_total = 0;
  for (long long seg = (long long)blockIdx.x * (IS_THREADS / 32) + wib; seg < a.nseg;
       seg += (long long)gridDim.x * (IS_THREADS / 32)) {
    const long long s0 = seg * IS_SEG;
    const long long s1 = min(a.n, s0 + IS_SEG);
    int* ci = a.cand_idx + s0;
    unsigned* ck = a.cand_key + s0;
    float* cv = a.cand_val + s0;
    unsigned cnt = 0;
    for (long long base = s0; base < s1; base += U * 128) {
      // One trip: U rows of 128 elements. Every lane first collects a bit mask of its qualifying
      // elements over the whole trip (bit u * 4 + j), with no warp-wide step per row; the trip's
      // few hits (about 1.5 % of its elements) are then placed by one warp scan and written by a
      // loop that runs once per hit of the busiest lane, re-reading the value through L1.
      const bool whole = base + U * 128 <= s1;  // every lane's loads lie inside the segment
      unsigned M = 0;
      if (SCORE == 1) {
        float g[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = base + u * 128 + lane * 4;
          if (whole) *reinterpret_cast<float4*>(g[u]) = *reinterpret_cast<const float4*>(a.acc + i);
          else load4z(a.acc, i, s1, g[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int j = 0; j < 4; ++j) M |= (key_bits(g[u][j]) >= tlo ? 1u : 0u) << (u * 4 + j);
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float g[4];
          unsigned key[4];
          keys4<SCORE>(a, base + u * 128 + lane * 4, s1, g, key);
#pragma unroll
          for (int j = 0; j < 4; ++j) M |= (key[j] >= tlo ? 1u : 0u) << (u * 4 + j);
        }
      }
      if (__ballot_sync(0xffffffffu, M != 0u) == 0u) continue;
      const int c = __popc(M);
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
      }
      unsigned pos = cnt + (unsigned)(incl - c);
      cnt += (unsigned)__shfl_sync(0xffffffffu, incl, 31);
      while (M) {
        const int bit = __ffs(M) - 1;
        M &= M - 1;
        const long long i = base + (bit >> 2) * 128 + lane * 4 + (bit & 3);
        float val;
        unsigned kk;
        if (SCORE == 1) {
          val = a.acc[i];
          kk = key_bits(val);
        } else {
          key1<SCORE>(a, i, val, kk);
        }
        ci[pos] = (int)i;
        ck[pos] = kk;
        cv[pos] = val;
        atomicAdd(&sh_hist[min((kk >> 19) - b_lo, (unsigned)(HBINS - 1))], 1u);
        ++pos;
      }
    }
    if (lane == 0) a.segcnt[seg] = (int)cnt;
    warp_total += cnt;
  }
  if (lane == 0) sh_cnt[wib] = warp_total;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned t = 0;
    for (int i = 0; i < IS_THREADS / 32; ++i) t += sh_cnt[i];
    if (t) atomicAdd(a.state + ST_C, t);
  }
  flush_first_digit(sh_hist, HBINS, (int)b_lo, replica, a.state);
  if (!last_cta(a.state + ST_TICKET0 + 1 + LEVEL)) return;
  const unsigned C = ldv(a.state + ST_C), k = (unsigned)a.k;
  bool retry = LEVEL == 0 && C < k && tlo > 1u;
  const int top = (int)ldv(a.state + ST_TOP) - 1, low = IS_ABINS - (int)ldv(a.state + ST_INVLOW);
  unsigned bin = 0, above = 0;
  bool found = false;
  if (top >= 0) {
    if (!retry && C > k) found = find_suffix_bin(a.histA, IS_ABINS, IS_REP, k, top, low, sh_cnt, bin, above);
    // a crossing in the window's last bin is a crossing somewhere above the window
    if (LEVEL == 0 && found && bin == b_lo + IS_WBINS - 1 && bin < IS_ABINS - 1) retry = true;
    zero_window(a.histA, IS_ABINS, IS_REP, top, low);
  }
  if (threadIdx.x == 0) { a.state[ST_TOP] = 0u; a.state[ST_INVLOW] = 0u; }
  if (threadIdx.x != 0) return;
  if (retry) {
    a.state[ST_LEVEL] = 1u;  // the sample bound was too high: take every non-zero element
    a.state[ST_C] = 0u;
  } else if (C <= k) {
    // no more non-zero keys than k: every candidate is selected
    a.state[ST_SKIP] = 1u; a.state[ST_T] = 0u; a.state[ST_NEED] = 0u; a.state[ST_EQ] = 0u;
    a.state[ST_ICUT] = 0x7FFFFFFFu; a.state[ST_ABOVE] = C;
  } else {
    if (!found) atomicOr(a.c.err, SGA_ERR_BOUNDS);
    a.state[ST_BA] = bin;
    a.state[ST_ABOVE] = above;
  }
}

// ------------------------------------------------------------- radix digits
// The remaining 19 key bits in one pass over the candidates of the crossing bin: an 11-bit digit
// in replicated global histograms and the full 19 bits in a 512 K-bin histogram (the values are
// spread over it, so its atomics rarely meet; a warp's equal keys are merged first). The last CTA
// finds the 11-bit bin, then reads the 256 fine bins under it: the exact k-th key T, the number
// of keys above it and the number of ties at T to take.
__global__ void __launch_bounds__(IS_THREADS) isync_digit_kernel(const ISyncArgs a) {
  chain_enter();
  __shared__ unsigned sh_scan[8];
  if (ldv(a.state + ST_SKIP) || ldv(a.state + ST_C) < (unsigned)a.k) return;
  const unsigned bA = ldv(a.state + ST_BA);
  unsigned* coarse = a.histB + (blockIdx.x % IS_REP) * IS_BBINS;
  unsigned* fine = a.histB + IS_REP * IS_BBINS;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  for (long long seg = (long long)blockIdx.x * (IS_THREADS / 32) + wib; seg < a.nseg;
       seg += (long long)gridDim.x * (IS_THREADS / 32)) {
    const long long s0 = seg * IS_SEG;
    const int cnt = a.segcnt[seg];
    // IS_CU trips of 32 candidates are loaded before the first is used: a segment holds about 120
    // candidates, so its keys arrive in one round trip instead of four dependent ones
    for (int j0 = 0; j0 < cnt; j0 += 32 * IS_CU) {
      unsigned key[IS_CU];
#pragma unroll
      for (int t = 0; t < IS_CU; ++t) {
        const int j = j0 + t * 32 + lane;
        key[t] = j < cnt ? a.cand_key[s0 + j] : 0u;
      }
#pragma unroll
      for (int t = 0; t < IS_CU; ++t) {
        const bool valid = j0 + t * 32 + lane < cnt && (key[t] >> 19) == bA;
        const unsigned act = __ballot_sync(0xffffffffu, valid);
        if (valid) {
          const unsigned low = key[t] & 0x7FFFFu;
          const unsigned peers = __match_any_sync(act, low);
          if (lane == __ffs(peers) - 1) {
            const unsigned c = (unsigned)__popc(peers);
            atomicAdd(&fine[low], c);
            atomicAdd(&coarse[low >> 8], c);
          }
        }
      }
    }
  }
  if (!last_cta(a.state + ST_TICKET0 + 3)) return;
  const unsigned k = (unsigned)a.k, aboveA = ldv(a.state + ST_ABOVE);
  unsigned bB, aboveB;
  if (!find_suffix_bin_all<IS_BBINS>(a.histB, IS_REP, k - aboveA, sh_scan, bB, aboveB)) {
    if (threadIdx.x == 0) atomicOr(a.c.err, SGA_ERR_BOUNDS);
    bB = 0; aboveB = 0;
  }
  for (int i = threadIdx.x; i < IS_REP * IS_BBINS / 4; i += IS_THREADS)
    reinterpret_cast<uint4*>(a.histB)[i] = make_uint4(0, 0, 0, 0);
  // thread t looks at fine bin 255 - t of the crossing 11-bit bin: a descending scan
  const unsigned mine = __ldcg(fine + (bB << 8) + (255u - threadIdx.x));
  unsigned total;
  const unsigned before = block_excl_scan256(mine, sh_scan, total);
  const unsigned want = k - aboveA - aboveB;
  if (before < want && before + mine >= want) {
    const unsigned n_gt = aboveA + aboveB + before, need = k - n_gt;
    a.state[ST_T] = (bA << 19) | (bB << 8) | (255u - threadIdx.x);
    a.state[ST_ABOVE] = n_gt;
    a.state[ST_NEED] = need;
    a.state[ST_EQ] = mine;
    a.state[ST_ICUT] = 0x7FFFFFFFu;
  }
  if (threadIdx.x == 0 && total < want) atomicOr(a.c.err, SGA_ERR_BOUNDS);
}

__device__ __forceinline__ bool is_selected(unsigned key, int idx, unsigned T, unsigned icut) {
  return key > T || (key == T && idx <= (int)icut);  // icut: index of the last tie taken (INT_MAX: all)
}

// ------------------------------------------------------------------- count
// Selected per segment, then (last CTA) the payload's offset table. When every tie at T is taken
// (nearly always) a segment's count is final at once. Otherwise the ties are taken in index order:
// segments are in index order, and inside the one segment that is cut a bitmap of its ties gives
// the index of the last tie taken.
__global__ void __launch_bounds__(IS_THREADS) isync_count_kernel(const ISyncArgs a) {
  chain_enter();
  __shared__ unsigned sh_scan[8];
  __shared__ unsigned sh_bm[IS_SEG / 32];
  __shared__ unsigned sh_cut[3];
  const unsigned T = ldv(a.state + ST_T), need = ldv(a.state + ST_NEED), eq_total = ldv(a.state + ST_EQ);
  const bool all_ties = need >= eq_total;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  for (long long seg = (long long)blockIdx.x * (IS_THREADS / 32) + wib; seg < a.nseg;
       seg += (long long)gridDim.x * (IS_THREADS / 32)) {
    const long long s0 = seg * IS_SEG;
    const int cnt = a.segcnt[seg];
    int g = 0, e = 0;
    for (int j0 = 0; j0 < cnt; j0 += 32 * IS_CU) {
      unsigned key[IS_CU];
#pragma unroll
      for (int t = 0; t < IS_CU; ++t) {
        const int j = j0 + t * 32 + lane;
        key[t] = j < cnt ? a.cand_key[s0 + j] : 0u;
      }
#pragma unroll
      for (int t = 0; t < IS_CU; ++t) {
        const bool have = j0 + t * 32 + lane < cnt;
        g += have && key[t] > T;
        e += have && key[t] == T;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      g += __shfl_xor_sync(0xffffffffu, g, o);
      e += __shfl_xor_sync(0xffffffffu, e, o);
    }
    if (lane == 0) {
      a.segsel[seg] = all_ties ? g + e : g;
      if (!all_ties) a.segeq[seg] = e;
    }
  }
  if (!last_cta(a.state + ST_TICKET0 + 4)) return;
  unsigned icut = 0x7FFFFFFFu;
  if (!all_ties) {
    // the segment where the running count of ties passes `need`, and how many of its ties are taken
    const int per = (a.nseg + IS_THREADS - 1) / IS_THREADS;
    const int lo = min(a.nseg, (int)threadIdx.x * per), hi = min(a.nseg, lo + per);
    unsigned myeq = 0;
    for (int i = lo; i < hi; ++i) myeq += (unsigned)__ldcg(a.segeq + i);
    unsigned tot;
    const unsigned eq_before = block_excl_scan256(myeq, sh_scan, tot);
    if (threadIdx.x == 0) { sh_cut[0] = (unsigned)a.nseg; sh_cut[1] = 0; sh_cut[2] = 0x7FFFFFFFu; }
    __syncthreads();
    if (eq_before <= need && eq_before + myeq > need) {
      unsigned run = eq_before;
      for (int i = lo; i < hi; ++i) {
        const unsigned e = (unsigned)__ldcg(a.segeq + i);
        if (run + e > need) { sh_cut[0] = (unsigned)i; sh_cut[1] = need - run; break; }
        run += e;
      }
    }
    __syncthreads();
    const unsigned cut_seg = sh_cut[0], cut_take = sh_cut[1];
    if (cut_seg < (unsigned)a.nseg) {
      for (int i = threadIdx.x; i < IS_SEG / 32; i += IS_THREADS) sh_bm[i] = 0;
      __syncthreads();
      const long long s0 = (long long)cut_seg * IS_SEG;
      const int cnt = __ldcg(a.segcnt + cut_seg);
      for (int j = threadIdx.x; j < cnt; j += IS_THREADS)
        if (__ldcg(a.cand_key + s0 + j) == T) {
          const int rel = __ldcg(a.cand_idx + s0 + j) - (int)s0;
          atomicOr(&sh_bm[rel >> 5], 1u << (rel & 31));
        }
      __syncthreads();
      const unsigned w = sh_bm[threadIdx.x];  // IS_SEG / 32 == IS_THREADS words
      const unsigned pc = (unsigned)__popc(w);
      const unsigned pre = block_excl_scan256(pc, sh_scan, tot);
      if (cut_take == 0) {
        if (threadIdx.x == 0) sh_cut[2] = (unsigned)(s0 - 1);  // nothing of this segment (need >= 1, so s0 > 0)
      } else if (pre < cut_take && pre + pc >= cut_take) {
        unsigned bits = w;
        for (unsigned r = pre + 1; r < cut_take; ++r) bits &= bits - 1;
        sh_cut[2] = (unsigned)s0 + threadIdx.x * 32 + (__ffs(bits) - 1);
      }
      __syncthreads();
    }
    icut = sh_cut[2];
    for (int i = lo; i < hi; ++i) {
      const unsigned e = (unsigned)__ldcg(a.segeq + i);
      const unsigned take = (unsigned)i < cut_seg ? e : ((unsigned)i == cut_seg ? cut_take : 0u);
      a.segsel[i] = __ldcg(a.segsel + i) + (int)take;
    }
    __syncthreads();
  }
  // exclusive scan of the per-segment counts, 4096 segments per round, 16 per thread
  unsigned carry = 0;
  for (int t0 = 0; t0 < a.nseg; t0 += IS_THREADS * 16) {
    const int i0 = t0 + (int)threadIdx.x * 16;
    int v[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = i0 + q * 4;
      if (i + 4 <= a.nseg) {
        *reinterpret_cast<int4*>(v + q * 4) = __ldcg(reinterpret_cast<const int4*>(a.segsel + i));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[q * 4 + j] = i + j < a.nseg ? __ldcg(a.segsel + i + j) : 0;
      }
    }
    unsigned mysum = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) mysum += (unsigned)v[j];
    unsigned tot;
    unsigned run = carry + block_excl_scan256(mysum, sh_scan, tot);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (i0 + j < a.nseg) a.roff[i0 + j] = (int)run;
      run += (unsigned)v[j];
    }
    carry += tot;
  }
  if (threadIdx.x == 0) {
    a.roff[a.nseg] = (int)carry;
    a.state[ST_NSEL] = carry;
    a.state[ST_ICUT] = icut;
    if (a.result) {
      a.result[0] = T;
      a.result[1] = need;
      a.result[2] = ldv(a.state + ST_ABOVE);
      a.result[3] = carry;
    }
    if (carry > (unsigned)a.kcap && a.kcap > 0) atomicOr(a.c.err, SGA_ERR_CAPACITY);
  }
}

// -------------------------------------------------------------------- emit
// Push the selected (index, value) pairs, grouped by segment, and the offset table into every
// rank's receive area (this rank's own included); zero the selected coordinates of the bucket
// (what stays is the residual). The last CTA raises this rank's "ready" flag on every peer.
__global__ void __launch_bounds__(IS_THREADS) isync_emit_kernel(const ISyncArgs a) {
  chain_enter();
  const PeerCtx& c = a.c;
  if (c.prev_seq > 0) timed_peer_wait(c, 1, c.prev_seq, a.wait_ns);  // peers are done reading my previous payload
  const unsigned T = ldv(a.state + ST_T), icut = ldv(a.state + ST_ICUT);
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const unsigned lt = (1u << lane) - 1u;
  for (long long seg = (long long)blockIdx.x * (IS_THREADS / 32) + wib; seg < a.nseg;
       seg += (long long)gridDim.x * (IS_THREADS / 32)) {
    const long long s0 = seg * IS_SEG;
    const int cnt = a.segcnt[seg];
    int pos0 = a.roff[seg];
    for (int j0 = 0; j0 < cnt; j0 += 32 * IS_CU) {
      int2 pr[IS_CU];
      unsigned key[IS_CU];
#pragma unroll
      for (int t = 0; t < IS_CU; ++t) {
        const int j = j0 + t * 32 + lane;
        pr[t] = make_int2(0, 0);
        key[t] = 0u;
        if (j < cnt) {
          pr[t].x = a.cand_idx[s0 + j];
          pr[t].y = __float_as_int(a.cand_val[s0 + j]);
          key[t] = a.cand_key[s0 + j];
        }
      }
#pragma unroll
      for (int t = 0; t < IS_CU; ++t) {
        const bool sel = j0 + t * 32 + lane < cnt && is_selected(key[t], pr[t].x, T, icut);
        const unsigned bal = __ballot_sync(0xffffffffu, sel);
        if (sel) {
          const int pos = pos0 + __popc(bal & lt);
          if (pos < a.kcap) {
#pragma unroll
            for (int r = 0; r < MAXW; ++r)
              if (r < c.W) a.slots[r][(long long)c.rank * a.kcap + pos] = pr[t];
          }
          if (a.zero_selected) a.acc[pr[t].x] = 0.f;
        }
        pos0 += __popc(bal);
      }
    }
  }
  for (long long i = (long long)blockIdx.x * IS_THREADS + threadIdx.x; i <= a.nseg;
       i += (long long)gridDim.x * IS_THREADS) {
    const int off = a.roff[i];
#pragma unroll
    for (int r = 0; r < MAXW; ++r)
      if (r < c.W) a.hdr[r][(long long)c.rank * a.hstride + i] = off;
  }
  if (!last_cta<true>(a.state + ST_TICKET0 + 5)) return;
  if (threadIdx.x < c.W) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + 0 * 8 + c.rank, c.seq);
  }
}

// Select-only form: the selection as a bit mask (zeroed by the host), nothing is exchanged.
__global__ void __launch_bounds__(IS_THREADS) isync_mask_kernel(const ISyncArgs a) {
  chain_enter();
  const unsigned T = ldv(a.state + ST_T), icut = ldv(a.state + ST_ICUT);
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  for (long long seg = (long long)blockIdx.x * (IS_THREADS / 32) + wib; seg < a.nseg;
       seg += (long long)gridDim.x * (IS_THREADS / 32)) {
    const long long s0 = seg * IS_SEG;
    const int cnt = a.segcnt[seg];
    for (int j0 = 0; j0 < cnt; j0 += 32 * IS_CU) {
      int idx[IS_CU];
      unsigned key[IS_CU];
#pragma unroll
      for (int t = 0; t < IS_CU; ++t) {
        const int j = j0 + t * 32 + lane;
        idx[t] = j < cnt ? a.cand_idx[s0 + j] : 0;
        key[t] = j < cnt ? a.cand_key[s0 + j] : 0u;
      }
#pragma unroll
      for (int t = 0; t < IS_CU; ++t)
        if (j0 + t * 32 + lane < cnt && is_selected(key[t], idx[t], T, icut))
          atomicOr(&a.bits[idx[t] >> 5], 1u << (idx[t] & 31));
    }
  }
}

// ------------------------------------------------------------------ reduce
// One CTA per range of four segments: once every rank's payload has landed, add the ranks' pairs
// of the range into the dense staging buffer in rank order (each rank lists a coordinate at most
// once, so a rank's pairs need no atomics), then the squared norm over the coordinates touched.
// The last CTA adds the per-range partials in index order and raises "done" on every peer.
__global__ void __launch_bounds__(IS_THREADS) isync_reduce_kernel(const ISyncArgs a) {
  chain_enter();
  __shared__ unsigned sh_bm[IS_SEG_PER_RANGE * IS_SEG / 32];
  __shared__ float red[IS_THREADS];
  const PeerCtx& c = a.c;
  timed_peer_wait(c, 0, c.seq, a.wait_ns);
  const int nranges = (a.nseg + IS_SEG_PER_RANGE - 1) / IS_SEG_PER_RANGE;
  const int2* my_slots = a.slots[c.rank];
  const int* my_hdr = a.hdr[c.rank];
  for (int range = blockIdx.x; range < nranges; range += gridDim.x) {
    const int seg0 = range * IS_SEG_PER_RANGE, seg1 = min(a.nseg, seg0 + IS_SEG_PER_RANGE);
    const long long r0 = (long long)seg0 * IS_SEG, r1 = min(a.n, (long long)seg1 * IS_SEG);
    for (int i = threadIdx.x; i < IS_SEG_PER_RANGE * IS_SEG / 32; i += IS_THREADS) sh_bm[i] = 0;
    __syncthreads();
    for (int r = 0; r < c.W; ++r) {
      const int lo = __ldcg(my_hdr + (long long)r * a.hstride + seg0);
      const int hi = __ldcg(my_hdr + (long long)r * a.hstride + seg1);
      if (lo < 0 || hi < lo || hi > a.kcap) {
        if (threadIdx.x == 0) atomicOr(c.err, SGA_ERR_BOUNDS);
      } else {
        const int2* list = my_slots + (long long)r * a.kcap;
        // a rank lists a coordinate at most once, so the IS_CU pairs a thread holds touch different
        // entries: their loads of the staging buffer are issued together, then the stores
        for (int j = lo + threadIdx.x; j < hi; j += IS_THREADS * IS_CU) {
          int2 pr[IS_CU];
          float cur[IS_CU];
          bool in[IS_CU];
#pragma unroll
          for (int u = 0; u < IS_CU; ++u) {
            const int jj = j + u * IS_THREADS;
            pr[u] = jj < hi ? __ldcg(list + jj) : make_int2(-1, 0);
          }
#pragma unroll
          for (int u = 0; u < IS_CU; ++u) {
            const long long p = pr[u].x;
            in[u] = j + u * IS_THREADS < hi && p >= r0 && p < r1;
            cur[u] = in[u] ? a.comm[p] : 0.f;
          }
#pragma unroll
          for (int u = 0; u < IS_CU; ++u) {
            if (in[u]) {
              const long long p = pr[u].x;
              a.comm[p] = cur[u] + __int_as_float(pr[u].y) * a.scale;
              atomicOr(&sh_bm[(p - r0) >> 5], 1u << ((p - r0) & 31));
            } else if (j + u * IS_THREADS < hi) {
              atomicOr(c.err, SGA_ERR_BOUNDS);
            }
          }
        }
      }
      __syncthreads();
    }
    float sq = 0.f;
    for (int w = threadIdx.x; w < IS_SEG_PER_RANGE * IS_SEG / 32; w += IS_THREADS) {
      unsigned bits = sh_bm[w];
      while (bits) {
        const int b = __ffs(bits) - 1;
        bits &= bits - 1;
        const float x = a.comm[r0 + w * 32 + b];
        sq = sq + x * x;
      }
    }
    const float bs = block_sum(sq, red);
    if (threadIdx.x == 0) a.partials[range] = bs;
    __syncthreads();
  }
  if (!last_cta<true>(a.reduce_ticket)) return;
  float t = 0.f;
  for (int i = threadIdx.x; i < nranges; i += IS_THREADS) t = t + __ldcg(a.partials + i);
  const float tot = block_sum(t, red);
  if (threadIdx.x == 0 && a.sumsq_out) a.sumsq_out[0] = a.accumulate ? a.sumsq_out[0] + tot : tot;
  if (threadIdx.x < c.W) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + 1 * 8 + c.rank, c.seq);
  }
}

}  // namespace sga

using namespace sga;

// Host-side description of one bucket synchronisation (mirrored by a ctypes.Structure).
struct SgaISyncDesc {
  void* acc; const void* w; const void* m; const void* v;
  long long n;
  int k, score, adams, nspan;
  float beta1, omb1, beta2, omb2, bc1, bc2, eps, scale;
  const void* span_start; const void* span_wd;
  void* state; void* histA; void* histB; void* cand_idx; void* cand_key; void* cand_val;
  void* segcnt; void* segsel; void* segeq; void* roff; void* partials;
  void* slots[sga::MAXW]; void* hdr[sga::MAXW];
  int kcap, hstride;
  void* comm; void* sumsq_out; void* bits; void* result;
  long long cand_capacity;   // elements the candidate arrays hold
  int seg_capacity;          // entries of segcnt / segsel (roff holds one more)
  int partials_capacity;
  int accumulate, zero_selected, mode, max_ctas;
  int phase;                 // 0: whole chain. 1: up to the push (no reduce). 2: the reduce alone
  void* reduce_ticket;       // one zeroed word per channel
  void* wait_ns;             // nullable uint64 counter: time spent waiting for peers
};

// Launch one kernel of the chain; `dependent` lets it be scheduled while its predecessor (the
// previous kernel on the stream) is still running.
static void launch_chain(void (*kern)(const ISyncArgs), int grid, cudaStream_t st, const ISyncArgs& a, bool dependent) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(IS_THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kern, a);
}

template <int SCORE>
static void launch_select(const ISyncArgs& base, int grid_seg, int grid_sample, cudaStream_t st, bool pdl) {
  ISyncArgs a = base;
  launch_chain(isync_sample_kernel<SCORE>, grid_sample, st, a, false);  // follows a memset, not a kernel
  launch_chain(isync_filter_kernel<SCORE, 0>, grid_seg, st, a, pdl);
  launch_chain(isync_filter_kernel<SCORE, 1>, grid_seg, st, a, pdl);
}

// mode 0: select + exchange + reduce into comm. mode 1: select only, bit mask of the selection
// into `bits` (ceil(n / 32) words). Returns 0, or a negative code before anything was launched.
SGA_API int sga_index_sync(const SgaPeerDesc* d, const SgaISyncDesc* s, void* stream) {
  if (d->W > MAXW) return -1;
  if (s->n <= 0 || s->n >= (1LL << 31) || s->k < 1 || s->k > s->n) return -6;
  if (s->score < 0 || s->score > 3) return -6;
  if ((reinterpret_cast<uintptr_t>(s->acc) & 15) != 0) return -9;
  const int nseg = (int)((s->n + IS_SEG - 1) / IS_SEG);
  if ((long long)nseg * IS_SEG > s->cand_capacity || nseg > s->seg_capacity) return -7;
  const int nranges = (nseg + IS_SEG_PER_RANGE - 1) / IS_SEG_PER_RANGE;
  if (s->phase < 0 || s->phase > 2 || (s->phase != 0 && s->mode != 0)) return -6;
  if (s->mode == 0) {
    if (s->k > s->kcap || nseg + 1 > s->hstride || nranges > s->partials_capacity || !s->comm) return -7;
    if (!s->reduce_ticket) return -6;
  } else if (!s->bits) {
    return -6;
  }
  if (s->score != 1 && (!s->m || (s->score != 2 && !s->v) || (s->score == 0 && (!s->w || s->nspan < 1)))) return -6;
  ISyncArgs a;
  a.c = make_ctx(d);
  a.acc = reinterpret_cast<float*>(s->acc);
  a.w = reinterpret_cast<const float*>(s->w);
  a.m = reinterpret_cast<const float*>(s->m);
  a.v = reinterpret_cast<const float*>(s->v);
  a.n = s->n; a.k = s->k; a.nseg = nseg; a.score = s->score; a.adams = s->adams;
  a.beta1 = s->beta1; a.omb1 = s->omb1; a.beta2 = s->beta2; a.omb2 = s->omb2;
  a.bc1 = s->bc1; a.bc2 = s->bc2; a.eps = s->eps;
  a.span_start = reinterpret_cast<const int*>(s->span_start);
  a.span_wd = reinterpret_cast<const float*>(s->span_wd);
  a.nspan = s->nspan;
  a.gshift = s->n > (1LL << 20) ? 6 : 0;
  a.state = reinterpret_cast<unsigned*>(s->state);
  a.histA = reinterpret_cast<unsigned*>(s->histA);
  a.histB = reinterpret_cast<unsigned*>(s->histB);
  a.cand_idx = reinterpret_cast<int*>(s->cand_idx);
  a.cand_key = reinterpret_cast<unsigned*>(s->cand_key);
  a.cand_val = reinterpret_cast<float*>(s->cand_val);
  a.segcnt = reinterpret_cast<int*>(s->segcnt);
  a.segsel = reinterpret_cast<int*>(s->segsel);
  a.segeq = reinterpret_cast<int*>(s->segeq);
  a.roff = reinterpret_cast<int*>(s->roff);
  a.partials = reinterpret_cast<float*>(s->partials);
  for (int i = 0; i < MAXW; ++i) {
    a.slots[i] = i < d->W ? reinterpret_cast<int2*>(s->slots[i]) : nullptr;
    a.hdr[i] = i < d->W ? reinterpret_cast<int*>(s->hdr[i]) : nullptr;
  }
  a.kcap = s->mode == 0 ? s->kcap : 0;
  a.hstride = s->hstride;
  a.comm = reinterpret_cast<float*>(s->comm);
  a.scale = s->scale;
  a.sumsq_out = reinterpret_cast<float*>(s->sumsq_out);
  a.accumulate = s->accumulate; a.zero_selected = s->zero_selected;
  a.bits = reinterpret_cast<unsigned*>(s->bits);
  a.result = reinterpret_cast<unsigned*>(s->result);
  a.reduce_ticket = reinterpret_cast<unsigned*>(s->reduce_ticket);
  a.wait_ns = reinterpret_cast<unsigned long long*>(s->wait_ns);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int cap = s->max_ctas > 0 ? s->max_ctas : 148 * 8;
  const int wpc = IS_THREADS / 32;
  int grid_seg = (nseg + wpc - 1) / wpc;
  if (grid_seg > cap) grid_seg = cap;
  const long long ngroups = (((s->n + 3) >> 2) + (1LL << a.gshift) - 1) >> a.gshift;
  int grid_sample = (int)((ngroups + IS_THREADS * 4 - 1) / (IS_THREADS * 4));
  if (grid_sample > 148) grid_sample = 148;
  if (grid_sample < 1) grid_sample = 1;
  int grid_range = nranges < cap ? nranges : cap;
  static const bool pdl = [] { const char* e = getenv("SGA_ISYNC_PDL"); return !(e && e[0] == '0'); }();
  if (s->phase == 2) {  // the deferred reduce of a bucket whose pairs were pushed by an earlier call
    launch_chain(isync_reduce_kernel, grid_range, st, a, false);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  cudaMemsetAsync(a.state, 0, 64 * sizeof(unsigned), st);
  if (s->mode == 1) cudaMemsetAsync(a.bits, 0, (size_t)((s->n + 31) / 32) * 4, st);
  switch (s->score) {
    case 0: launch_select<0>(a, grid_seg, grid_sample, st, pdl); break;
    case 1: launch_select<1>(a, grid_seg, grid_sample, st, pdl); break;
    case 2: launch_select<2>(a, grid_seg, grid_sample, st, pdl); break;
    default: launch_select<3>(a, grid_seg, grid_sample, st, pdl); break;
  }
  launch_chain(isync_digit_kernel, grid_seg, st, a, pdl);
  launch_chain(isync_count_kernel, grid_seg, st, a, pdl);
  if (s->mode == 1) {
    launch_chain(isync_mask_kernel, grid_seg, st, a, pdl);
  } else {
    launch_chain(isync_emit_kernel, grid_seg, st, a, pdl);
    if (s->phase == 0) launch_chain(isync_reduce_kernel, grid_range, st, a, pdl);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
