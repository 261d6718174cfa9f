// Support selection and support-form kernels (single GPU):
//
//   sga_hist_top        histogram of the top bits of |x|'s bit pattern, with
//                       stride subsampling (the exact / balanced / fast tiers)
//   sga_hist_low16      second radix digit: low-16-bit histogram of the
//                       elements whose top-16 key equals one bin (gives the
//                       exact k-th value without gathering candidates)
//   sga_mask_ge         uint8 mask of (key >= bin) or (|x| >= thr), plus count
//   sga_mask_stats      count + the two position checksums of a mask
//   sga_compact_mask    mask -> ascending int32 index list (block counts,
//                       scan, ordered scatter); also emits the 1024-stride
//                       directory table of lower bounds
//   sga_pack / sga_scatter / block variants / descriptors
//   sga_block_reduce    per-block mean|max of |x|
//   sga_expand_blocks   block mask -> element mask
//
// Replaces sga/plugins/selection/_histogram.py (bincount/cumsum/kthvalue
// loops), sga/support.py:57-206 (chunked nonzero, block heads, descriptors),
// sga/kernels.py:49-139 (pack / scatter / block gather / block scatter) and the
// chunked checksum loop of sga/engine.py:1341-1359.
#include "common.cuh"

namespace sga {

__device__ __forceinline__ uint32_t abs_bits(float x) { return __float_as_uint(x) & 0x7FFFFFFFu; }

// ------------------------------------------------------------- histograms
// Global int64 histogram; each CTA privatises into 32-bit shared counters when
// nbins fits (<= 32769 bins -> 128 KB + 4 B of dynamic shared memory).
__global__ void __launch_bounds__(512) hist_top_kernel(const float* __restrict__ x, long long n, int shift,
                                                       int stride, int nbins, long long* __restrict__ hist,
                                                       long long* __restrict__ nonfinite) {
  extern __shared__ uint32_t sh[];
  for (int i = threadIdx.x; i < nbins; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const long long ns = (n + stride - 1) / stride;  // sampled count
  const long long gstride = (long long)gridDim.x * blockDim.x;
  int bad = 0;
  for (long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x; s < ns; s += gstride) {
    const uint32_t b = abs_bits(x[s * stride]);
    if (b >= 0x7F800000u) ++bad;
    atomicAdd(&sh[b >> shift], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nbins; i += blockDim.x) {
    const uint32_t c = sh[i];
    if (c) atomicAdd(reinterpret_cast<unsigned long long*>(hist + i), (unsigned long long)c);
  }
  if (nonfinite && bad) atomicAdd(reinterpret_cast<unsigned long long*>(nonfinite), (unsigned long long)bad);
}

__global__ void __launch_bounds__(512) hist_low16_kernel(const float* __restrict__ x, long long n, int bin,
                                                         long long* __restrict__ hist) {
  extern __shared__ uint32_t sh[];  // 65536 counters = 256 KB is too large: use 2 passes of 32768
  // The low 16 bits are split by their top bit into two half-histograms of
  // 32768 counters; blockIdx.y selects the half so shared memory stays 128 KB.
  const uint32_t half = blockIdx.y;
  for (int i = threadIdx.x; i < 32768; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x; s < n; s += gstride) {
    const uint32_t b = abs_bits(x[s]);
    if ((int)(b >> 16) == bin && ((b >> 15) & 1u) == half) atomicAdd(&sh[b & 0x7FFFu], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 32768; i += blockDim.x) {
    const uint32_t c = sh[i];
    if (c) atomicAdd(reinterpret_cast<unsigned long long*>(hist + half * 32768 + i), (unsigned long long)c);
  }
}

// ------------------------------------------------------------------ masks
// mode 0: mask = (abs_bits(x) >> shift) >= bin ; mode 1: mask = |x| >= thr.
__global__ void __launch_bounds__(256) mask_ge_kernel(const float* __restrict__ x, long long n, int mode, int shift,
                                                      int bin, float thr, uint8_t* __restrict__ mask,
                                                      long long* __restrict__ count) {
  long long local = 0;
  const long long gstride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += gstride) {
    uint8_t mk[4];
    const int lim = (int)min((long long)4, n - i);
    for (int j = 0; j < lim; ++j) {
      const float v = x[i + j];
      const bool on = mode == 0 ? (int)(abs_bits(v) >> shift) >= bin : fabsf(v) >= thr;
      mk[j] = on ? 1 : 0;
      local += on;
    }
    if (lim == 4) *reinterpret_cast<uchar4*>(mask + i) = *reinterpret_cast<uchar4*>(mk);
    else for (int j = 0; j < lim; ++j) mask[i + j] = mk[j];
  }
  // warp + block reduce then one atomic per block
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  __shared__ long long red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0 && count) {
    long long t = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    if (t) atomicAdd(reinterpret_cast<unsigned long long*>(count), (unsigned long long)t);
  }
}

// out[0] += count, out[1] += sum(pos), out[2] += sum((pos % 9973) * (pos % 1009)) over mask-on positions.
// Sixteen mask bytes per load (the unaligned head and the tail go byte by byte); all-zero words, the common
// case of a sparse support, cost one test. Integer sums: the result does not depend on the order.
__global__ void __launch_bounds__(256) mask_stats_kernel(const uint8_t* __restrict__ mask, long long n,
                                                         long long* __restrict__ out) {
  long long c = 0, s1 = 0, s2 = 0;
  const bool small = n < (1LL << 32);  // 32-bit remainders by constants are a multiply and a shift
  auto hit = [&](long long pos) {
    ++c;
    s1 += pos;
    if (small) {
      const uint32_t p = (uint32_t)pos;
      s2 += (long long)((p % 9973u) * (p % 1009u));
    } else {
      s2 += (pos % 9973) * (pos % 1009);
    }
  };
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  long long head = (16 - (long long)(reinterpret_cast<uintptr_t>(mask) & 15)) & 15;
  if (head > n) head = n;
  const long long nvec = (n - head) >> 4;
  const uint4* v = reinterpret_cast<const uint4*>(mask + head);
  for (long long j = gtid; j < nvec; j += gstride) {
    const uint4 q = __ldg(v + j);
    if ((q.x | q.y | q.z | q.w) == 0u) continue;
    const uint32_t wds[4] = {q.x, q.y, q.z, q.w};
    const long long base = head + (j << 4);
    // one bit per non-zero byte: bit 0 of every byte of the SIMD compare, gathered into the top nibble by a
    // multiply whose partial products do not overlap; then only the set bits are visited
    uint32_t bits = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w)
      bits |= (((__vcmpne4(wds[w], 0u) & 0x01010101u) * 0x01020408u) >> 24 & 0xFu) << (4 * w);
    while (bits) {
      hit(base + (__ffs(bits) - 1));
      bits &= bits - 1;
    }
  }
  // byte-wise edges: [0, head) and [head + 16 * nvec, n), at most 30 positions
  const long long tail0 = head + (nvec << 4);
  const long long edges = head + (n - tail0);
  if (gtid < edges) {
    const long long pos = gtid < head ? gtid : tail0 + (gtid - head);
    if (mask[pos]) hit(pos);
  }
  for (int o = 16; o > 0; o >>= 1) {
    c += __shfl_xor_sync(0xffffffffu, c, o);
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if ((threadIdx.x & 31) == 0 && c) {
    atomicAdd(reinterpret_cast<unsigned long long*>(out + 0), (unsigned long long)c);
    atomicAdd(reinterpret_cast<unsigned long long*>(out + 1), (unsigned long long)s1);
    atomicAdd(reinterpret_cast<unsigned long long*>(out + 2), (unsigned long long)s2);
  }
}

// ------------------------------------------------------------- compaction
constexpr int CP_THREADS = 256;
constexpr int CP_ITEMS = 16;                       // consecutive mask bytes per thread
constexpr int CP_TILE = CP_THREADS * CP_ITEMS;     // 4096 elements per CTA

__global__ void __launch_bounds__(CP_THREADS) compact_count_kernel(const uint8_t* __restrict__ mask, long long n,
                                                                   int* __restrict__ block_counts) {
  const long long base = (long long)blockIdx.x * CP_TILE + (long long)threadIdx.x * CP_ITEMS;
  int c = 0;
  if (base + CP_ITEMS <= n) {
    const uint4 v = *reinterpret_cast<const uint4*>(mask + base);
    const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      for (int b = 0; b < 4; ++b) c += ((wds[j] >> (8 * b)) & 0xFFu) != 0;
  } else {
    for (long long i = base; i < n && i < base + CP_ITEMS; ++i) c += mask[i] != 0;
  }
  __shared__ int red[CP_THREADS / 32];
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < CP_THREADS / 32; ++w) t += red[w];
    block_counts[blockIdx.x] = t;
  }
}

// Exclusive scan of block counts in place (single CTA, any length); total -> *total_out.
__global__ void __launch_bounds__(1024) scan_counts_kernel(int* __restrict__ counts, int nblocks,
                                                           long long* __restrict__ total_out) {
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < nblocks; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < nblocks ? counts[i] : 0;
    int x = v;
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if ((threadIdx.x & 31) >= o) x += y;
    }
    if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = x;
    __syncthreads();
    if (threadIdx.x < 32) {
      int t = warp_tot[threadIdx.x];
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, t, o);
        if (threadIdx.x >= o) t += y;
      }
      warp_tot[threadIdx.x] = t;
    }
    __syncthreads();
    const int warp_prefix = (threadIdx.x >> 5) ? warp_tot[(threadIdx.x >> 5) - 1] : 0;
    const int carry = carry_s;
    if (i < nblocks) counts[i] = carry + warp_prefix + x - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + warp_prefix + x;
    __syncthreads();
  }
  if (threadIdx.x == 0 && total_out) *total_out = carry_s;
}

__global__ void __launch_bounds__(CP_THREADS) compact_scatter_kernel(const uint8_t* __restrict__ mask, long long n,
                                                                     const int* __restrict__ block_offsets,
                                                                     int* __restrict__ idx_out, long long cap,
                                                                     int* __restrict__ err) {
  const long long base = (long long)blockIdx.x * CP_TILE + (long long)threadIdx.x * CP_ITEMS;
  uint8_t mk[CP_ITEMS];
  int c = 0;
#pragma unroll
  for (int j = 0; j < CP_ITEMS; ++j) {
    mk[j] = (base + j < n) ? mask[base + j] : 0;
    c += mk[j] != 0;
  }
  // block exclusive scan of c
  __shared__ int warp_tot[CP_THREADS / 32];
  int x = c;
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, o);
    if ((threadIdx.x & 31) >= o) x += y;
  }
  if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = x;
  __syncthreads();
  int prefix = 0;
  for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) prefix += warp_tot[w];
  long long pos = (long long)block_offsets[blockIdx.x] + prefix + x - c;
#pragma unroll
  for (int j = 0; j < CP_ITEMS; ++j) {
    if (mk[j]) {
      if (pos < cap) idx_out[pos] = (int)(base + j);
      else if (err) atomicOr(err, SGA_ERR_CAPACITY);
      ++pos;
    }
  }
}

// table[j] = lower_bound(idx[0..k), j * 1024) for j in [0, ntable).
__global__ void dir_table_kernel(const int* __restrict__ idx, long long k, int* __restrict__ table, int ntable) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= ntable) return;
  const long long target = (long long)j * 1024;
  long long lo = 0, hi = k;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if ((long long)idx[mid] < target) lo = mid + 1; else hi = mid;
  }
  table[j] = (int)lo;
}

// ----------------------------------------------------------- pack/scatter
// Debug build (-DSGA_BOUNDS, libsga_b200_bounds.so): the index-following kernels below check every
// index against a window the host registers with sga_bounds_set_limit(); an index outside it is
// counted and its access skipped. The production build compiles the checks away.
#ifdef SGA_BOUNDS
static __device__ long long g_bounds_limit = 0x7fffffffffffffffLL;
static __device__ unsigned long long g_bounds_hits = 0ULL;
__device__ __forceinline__ bool sga_index_ok(long long p) {
  if (p >= 0 && p < g_bounds_limit) return true;
  atomicAdd(&g_bounds_hits, 1ULL);
  return false;
}
#else
__device__ __forceinline__ bool sga_index_ok(long long) { return true; }
#endif

// vals[i] = grad[idx[i]] * factor; optionally grad[idx[i]] = 0.
__global__ void pack_kernel(float* __restrict__ grad, const int* __restrict__ idx, long long k,
                            float* __restrict__ vals, float factor, int scale, int zero) {
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < k; i += gstride) {
    const int p = idx[i];
    if (!sga_index_ok(p)) {
      vals[i] = 0.f;
      continue;
    }
    const float v = grad[p];
    vals[i] = scale ? v * factor : v;
    if (zero) grad[p] = 0.f;
  }
}
__global__ void scatter_kernel(float* __restrict__ dst, const int* __restrict__ idx, const float* __restrict__ vals,
                               long long k, int add) {
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < k; i += gstride) {
    if (!sga_index_ok(idx[i])) continue;
    if (add) dst[idx[i]] += vals[i]; else dst[idx[i]] = vals[i];
  }
}
// Block forms: heads[b] is the first element of an X-element run clamped by
// mask (lanes whose mask byte is 0 carry 0 on gather and are skipped on scatter).
__global__ void gather_blocks_kernel(float* __restrict__ grad, const uint8_t* __restrict__ mask,
                                     const int* __restrict__ heads, long long kb, int X, long long n,
                                     float* __restrict__ vals, float factor, int scale, int zero) {
  const long long total = kb * X;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gstride) {
    const long long p = (long long)heads[t / X] + (t % X);
    float v = 0.f;
    if (p < n && sga_index_ok(p) && mask[p]) {
      v = grad[p];
      if (scale) v = v * factor;
      if (zero) grad[p] = 0.f;
    }
    vals[t] = v;
  }
}
__global__ void scatter_blocks_kernel(float* __restrict__ grad, const uint8_t* __restrict__ mask,
                                      const int* __restrict__ heads, long long kb, int X, long long n,
                                      const float* __restrict__ vals) {
  const long long total = kb * X;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gstride) {
    const long long p = (long long)heads[t / X] + (t % X);
    if (p < n && sga_index_ok(p) && mask[p]) grad[p] = vals[t];
  }
}

// Per-block reduce of |x| over blocks of X elements inside one span [0, n):
// out[b] = mean or max over the block's real length.
__global__ void block_reduce_kernel(const float* __restrict__ x, long long n, int X, int use_max,
                                    float* __restrict__ out, long long nblocks) {
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += gstride) {
    const long long s = b * X;
    const long long e = min(n, s + X);
    float acc = 0.f;
    for (long long i = s; i < e; ++i) {
      const float a = fabsf(x[i]);
      acc = use_max ? fmaxf(acc, a) : acc + a;
    }
    out[b] = use_max ? acc : acc / (float)(e - s);
  }
}
__global__ void expand_blocks_kernel(const uint8_t* __restrict__ bmask, long long nblocks, int X, long long n,
                                     uint8_t* __restrict__ mask) {
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gstride) mask[i] = bmask[i / X];
}

// ------------------------------------------------------------ block forms
// Blocks of X elements tile every parameter span from its start and never cross a span boundary.
// Block b belongs to the span s with span_boff[s] <= b < span_boff[s + 1]; its head is
// span_start[s] + (b - span_boff[s]) * X and it is span_end[s] - head long when that is below X.
// block_flags_kernel writes, per block, 1 when any of its elements is selected, and counts the
// blocks that are selected only in part (the descriptor wire form moves whole runs and refuses
// those). The flags then go through the mask compaction above; block_heads_kernel turns the
// surviving block numbers into heads or packed `head | tail_len` descriptors.
// Replaces the per-span loops of sga/support.py:102-206.
__device__ __forceinline__ int span_of_block(const long long* __restrict__ span_boff, int nspan, long long b) {
  int lo = 0, hi = nspan - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (span_boff[mid] <= b) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void block_flags_kernel(const uint8_t* __restrict__ mask, const long long* __restrict__ span_start,
                                   const long long* __restrict__ span_end, const long long* __restrict__ span_boff,
                                   int nspan, int X, long long nblocks, uint8_t* __restrict__ flags,
                                   unsigned long long* __restrict__ partial) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += stride) {
    const int s = span_of_block(span_boff, nspan, b);
    const long long head = span_start[s] + (b - span_boff[s]) * X;
    const int len = (int)min((long long)X, span_end[s] - head);
    int on = 0;
    if (len == X && X % 4 == 0 && (head & 3) == 0) {
      for (int i = 0; i < X; i += 4) {
        const uchar4 m = *reinterpret_cast<const uchar4*>(mask + head + i);
        on += (m.x != 0) + (m.y != 0) + (m.z != 0) + (m.w != 0);
      }
    } else {
      for (int i = 0; i < len; ++i) on += mask[head + i] != 0;
    }
    flags[b] = on ? 1 : 0;
    if (on && on < len && partial) atomicAdd(partial, 1ULL);
  }
}

__global__ void block_heads_kernel(const int* __restrict__ block_ids, long long kb,
                                   const long long* __restrict__ span_start, const long long* __restrict__ span_end,
                                   const long long* __restrict__ span_boff, int nspan, int X, int as_desc,
                                   int* __restrict__ out) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < kb; j += stride) {
    const long long b = block_ids[j];
    const int s = span_of_block(span_boff, nspan, b);
    const long long head = span_start[s] + (b - span_boff[s]) * X;
    long long v = head;
    if (as_desc) {
      const long long len = min((long long)X, span_end[s] - head);
      v = head | (len < X ? len : 0);
    }
    out[j] = (int)v;
  }
}

static inline int grid_for(long long n, int per_block, int cap = 148 * 8) {
  long long b = (n + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return (int)b;
}

}  // namespace sga

using namespace sga;
#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -4)

SGA_API int sga_hist_top(const float* x, long long n, int shift, int stride, int nbins, long long* hist,
                         long long* nonfinite, void* stream) {
  if (n <= 0) return 0;
  if (nbins > 32769) return -1;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(hist_top_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32769 * 4) != cudaSuccess)
      return -3;
    attr = true;
  }
  const long long ns = (n + stride - 1) / stride;
  hist_top_kernel<<<grid_for(ns, 512 * 16, 148), 512, nbins * 4, ST(stream)>>>(x, n, shift, stride, nbins, hist,
                                                                                nonfinite);
  return LAUNCH_OK();
}

SGA_API int sga_hist_low16(const float* x, long long n, int bin, long long* hist, void* stream) {
  if (n <= 0) return 0;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(hist_low16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4) !=
        cudaSuccess)
      return -3;
    attr = true;
  }
  dim3 grid(grid_for(n, 512 * 16, 74), 2);
  hist_low16_kernel<<<grid, 512, 32768 * 4, ST(stream)>>>(x, n, bin, hist);
  return LAUNCH_OK();
}

SGA_API int sga_mask_ge(const float* x, long long n, int mode, int shift, int bin, float thr, uint8_t* mask,
                        long long* count, void* stream) {
  if (n <= 0) return 0;
  mask_ge_kernel<<<grid_for(n, 1024), 256, 0, ST(stream)>>>(x, n, mode, shift, bin, thr, mask, count);
  return LAUNCH_OK();
}

SGA_API int sga_mask_stats(const uint8_t* mask, long long n, long long* out3, void* stream) {
  if (n <= 0) return 0;
  // one 16-byte word per thread and iteration; at most eight CTAs per SM, grid-stride beyond that
  long long blocks = ((n >> 4) + 255) / 256 + 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  mask_stats_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(mask, n, out3);
  return LAUNCH_OK();
}

// idx_out receives the ascending positions of non-zero mask bytes; *total_out
// the count. `block_counts` is scratch of ceil(n / 4096) ints. Positions
// beyond `cap` are dropped and SGA_ERR_CAPACITY is set in *err.
SGA_API int sga_compact_mask(const uint8_t* mask, long long n, int* block_counts, int* idx_out, long long cap,
                             long long* total_out, int* err, void* stream) {
  if (n <= 0) return 0;
  if (n >= (1LL << 31)) return -6;
  if ((reinterpret_cast<uintptr_t>(mask) & 15) != 0) return -10;  // the kernels read the mask 16 bytes at a time
  const int nb = (int)((n + CP_TILE - 1) / CP_TILE);
  compact_count_kernel<<<nb, CP_THREADS, 0, ST(stream)>>>(mask, n, block_counts);
  scan_counts_kernel<<<1, 1024, 0, ST(stream)>>>(block_counts, nb, total_out);
  compact_scatter_kernel<<<nb, CP_THREADS, 0, ST(stream)>>>(mask, n, block_counts, idx_out, cap, err);
  return LAUNCH_OK();
}

// Per-block "any element selected" flags over the spans' block tiling; *partial (nullable, zeroed by
// the caller) counts blocks that are selected only in part.
SGA_API int sga_block_flags(const uint8_t* mask, const long long* span_start, const long long* span_end,
                            const long long* span_boff, int nspan, int X, long long nblocks, uint8_t* flags,
                            unsigned long long* partial, void* stream) {
  if (nblocks <= 0) return 0;
  if (nspan < 1 || X < 1) return -6;
  block_flags_kernel<<<grid_for(nblocks, 256), 256, 0, ST(stream)>>>(mask, span_start, span_end, span_boff, nspan, X,
                                                                    nblocks, flags, partial);
  return LAUNCH_OK();
}

// Ascending block numbers -> block heads (as_desc = 0) or packed head | tail_len descriptors (1).
SGA_API int sga_block_heads(const int* block_ids, long long kb, const long long* span_start,
                            const long long* span_end, const long long* span_boff, int nspan, int X, int as_desc,
                            int* out, void* stream) {
  if (kb <= 0) return 0;
  block_heads_kernel<<<grid_for(kb, 256), 256, 0, ST(stream)>>>(block_ids, kb, span_start, span_end, span_boff, nspan,
                                                              X, as_desc, out);
  return LAUNCH_OK();
}

SGA_API int sga_dir_table(const int* idx, long long k, int* table, int ntable, void* stream) {
  if (ntable <= 0) return 0;
  dir_table_kernel<<<(ntable + 255) / 256, 256, 0, ST(stream)>>>(idx, k, table, ntable);
  return LAUNCH_OK();
}

// Bounds build only: register the window [0, limit) / read and clear the count of indices seen
// outside it. The production build answers -1 to both.
SGA_API long long sga_bounds_set_limit(long long limit) {
#ifdef SGA_BOUNDS
  return cudaMemcpyToSymbol(g_bounds_limit, &limit, sizeof(limit)) == cudaSuccess ? 0 : -2;
#else
  (void)limit;
  return -1;
#endif
}
SGA_API long long sga_bounds_hits() {
#ifdef SGA_BOUNDS
  unsigned long long h = 0, z = 0;
  if (cudaMemcpyFromSymbol(&h, g_bounds_hits, sizeof(h)) != cudaSuccess) return -2;
  cudaMemcpyToSymbol(g_bounds_hits, &z, sizeof(z));
  return (long long)h;
#else
  return -1;
#endif
}

SGA_API int sga_pack(float* grad, const int* idx, long long k, float* vals, float factor, int scale, int zero,
                     void* stream) {
  if (k <= 0) return 0;
  pack_kernel<<<grid_for(k, 256), 256, 0, ST(stream)>>>(grad, idx, k, vals, factor, scale, zero);
  return LAUNCH_OK();
}

SGA_API int sga_scatter(float* dst, const int* idx, const float* vals, long long k, int add, void* stream) {
  if (k <= 0) return 0;
  scatter_kernel<<<grid_for(k, 256), 256, 0, ST(stream)>>>(dst, idx, vals, k, add);
  return LAUNCH_OK();
}

SGA_API int sga_gather_blocks(float* grad, const uint8_t* mask, const int* heads, long long kb, int X, long long n,
                              float* vals, float factor, int scale, int zero, void* stream) {
  if (kb <= 0) return 0;
  gather_blocks_kernel<<<grid_for(kb * X, 256), 256, 0, ST(stream)>>>(grad, mask, heads, kb, X, n, vals, factor,
                                                                      scale, zero);
  return LAUNCH_OK();
}

SGA_API int sga_scatter_blocks(float* grad, const uint8_t* mask, const int* heads, long long kb, int X, long long n,
                               const float* vals, void* stream) {
  if (kb <= 0) return 0;
  scatter_blocks_kernel<<<grid_for(kb * X, 256), 256, 0, ST(stream)>>>(grad, mask, heads, kb, X, n, vals);
  return LAUNCH_OK();
}

SGA_API int sga_block_reduce(const float* x, long long n, int X, int use_max, float* out, void* stream) {
  if (n <= 0) return 0;
  const long long nb = (n + X - 1) / X;
  block_reduce_kernel<<<grid_for(nb, 256), 256, 0, ST(stream)>>>(x, n, X, use_max, out, nb);
  return LAUNCH_OK();
}

SGA_API int sga_expand_blocks(const uint8_t* bmask, long long nblocks, int X, long long n, uint8_t* mask,
                              void* stream) {
  if (n <= 0) return 0;
  expand_blocks_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(bmask, nblocks, X, n, mask);
  return LAUNCH_OK();
}

// ---------------------------------------------------------------------------
// Compaction without a caller-supplied work array (see compact_noalloc.h).
//
// For hosts that cannot allocate device memory themselves -- all of it belongs
// to their own arena, or they may not pay the synchronisation an allocation
// implies, or they only ever receive input and output buffers -- the per-block
// counters of the compaction live in this file-scope device array instead.
// 65536 ints = 256 KiB per GPU for the life of the process; masks of up to
// 65536 * 4096 bytes are accepted, longer ones are refused.
//
// Host code must not hand `g_compact_noalloc_counts` to a kernel: on the host
// that name is only a stand-in for the symbol, not a device address. The
// address is looked up once per device with cudaGetSymbolAddress while that
// device is current (the first call on a device does it; do that call at
// start-up, before any stream capture), then passed to the same three kernels
// sga_compact_mask() uses. The array is shared by every call and keeps its
// old contents; compact_count_kernel rewrites each entry before it is read,
// so nothing has to be cleared, but calls that overlap on the GPU race.
// ---------------------------------------------------------------------------
#include "compact_noalloc.h"
#include <mutex>
#include <stdio.h>

static __device__ __align__(256) int g_compact_noalloc_counts[SGA_COMPACT_NOALLOC_MAX_BLOCKS];

namespace {
constexpr int kNoallocMaxDevices = 64;
int* g_noalloc_ptr[kNoallocMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;

// Device address of the work array on the current device, resolved on first use.
int* noalloc_scratch_for_current_device(int* rc) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices) {
    *rc = SGA_COMPACT_NOALLOC_E_SETUP;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    int* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_compact_noalloc_counts);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "sga_compact_mask_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      *rc = SGA_COMPACT_NOALLOC_E_SETUP;
      return nullptr;
    }
    g_noalloc_ptr[dev] = p;
  }
  *rc = 0;
  return g_noalloc_ptr[dev];
}
}  // namespace

SGA_API int sga_compact_mask_noalloc(const uint8_t* mask, long long n, int* idx_out, long long cap,
                                     long long* total_out, int* err, void* stream) {
  if (n <= 0) return 0;
  if (n > SGA_COMPACT_NOALLOC_MAX_ELEMS) {
    fprintf(stderr,
            "sga_compact_mask_noalloc: mask of %lld bytes exceeds the built-in work array (at most %lld bytes); "
            "use sga_compact_mask with your own work array\n",
            n, (long long)SGA_COMPACT_NOALLOC_MAX_ELEMS);
    return SGA_COMPACT_NOALLOC_E_TOO_LARGE;
  }
  if ((reinterpret_cast<uintptr_t>(mask) & 15) != 0) {
    fprintf(stderr, "sga_compact_mask_noalloc: the mask must start on a 16-byte boundary (got %p)\n",
            static_cast<const void*>(mask));
    return SGA_COMPACT_NOALLOC_E_ALIGN;
  }
  int rc = 0;
  int* counts = noalloc_scratch_for_current_device(&rc);
  if (counts == nullptr) return rc;
  const int nb = (int)((n + CP_TILE - 1) / CP_TILE);
  compact_count_kernel<<<nb, CP_THREADS, 0, ST(stream)>>>(mask, n, counts);
  scan_counts_kernel<<<1, 1024, 0, ST(stream)>>>(counts, nb, total_out);
  compact_scatter_kernel<<<nb, CP_THREADS, 0, ST(stream)>>>(mask, n, counts, idx_out, cap, err);
  return cudaGetLastError() == cudaSuccess ? 0 : SGA_COMPACT_NOALLOC_E_LAUNCH;
}
