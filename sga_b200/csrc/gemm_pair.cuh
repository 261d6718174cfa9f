// The CTA-pair tcgen05 GEMM kernel, shared by the plain launcher (gemm_pair.cu)
// and the tensor-parallel launchers that fuse a collective into it (gemm_tp.cu).
//
// tcgen05.mma.cta_group::2 computes a 256 x 256 tile over two SMs. Each CTA
// stages its own 128 rows of A and its own 128 of the tile's 256 B rows, holds
// the accumulator of its 128 rows in its own TMEM, and writes those rows out.
// One elected thread of the leader CTA (cluster rank 0) issues every MMA.
//
// Barriers: "stage full" lives in the leader; both CTAs' TMA loads credit their
// bytes to it through its shared::cluster address (plain per-CTA tile loads).
// "stage empty" and "accumulator full" live in both CTAs and are signalled
// together by tcgen05.commit with a CTA mask. "accumulator empty" lives in the
// leader; the peer's epilogue warps arrive on it remotely. Every wait is
// bounded; on expiry the status word is set and the kernel still runs to its
// end, joins the cluster and frees TMEM.
//
// Template parameter TP selects the fused collective:
//   TP_NONE  plain C = A B^T.
//   TP_AG    all-gather -> GEMM. A is this rank's gathered buffer [M, K]; row
//            chunk r of it is produced by rank r in rank r's copy of the buffer.
//            A seventh warp in every CTA pulls the peers' chunks over NVLink
//            with bulk copies (peer global -> shared -> local global) and counts
//            each finished 16 KB unit on its 256-row block; the TMA producer
//            runs the own chunk's tiles first and, for a remote block, waits
//            for the block's count before its loads (local memory only).
//   TP_RS    GEMM -> reduce-scatter. Tiles of the peers' row chunks run first;
//            their epilogue stores the bf16 partial straight into the owner's
//            receive slot and raises a per-warp tile flag there. The own
//            chunk's tiles run last; their epilogue waits for the same warp's
//            flag from every peer, adds the received partials in rank order and
//            writes the [M/W, N] result (optionally plus a residual).
#pragma once
#include "gemm_common.cuh"
#include "peer.cuh"

namespace sga {

constexpr int P_BM = 128;   // rows of A per CTA (pair tile: 256)
constexpr int P_BN = 256;   // tile columns (each CTA stages 128 of them)
constexpr int P_BNH = 128;
constexpr int P_BK = 64;
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = P_BM * P_BK * 2;    // 16 KB
constexpr int P_B_BYTES = P_BNH * P_BK * 2;   // 16 KB
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_THREADS = 192;
constexpr int P_THREADS_AG = 224;             // + the copy warp
constexpr int P_TMEM_COLS = 512;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256;
constexpr int P_COPY_UNIT = 16384;
constexpr int P_COPY_STAGES = 2;
constexpr int P_SMEM_BYTES_AG = P_SMEM_BYTES + P_COPY_STAGES * P_COPY_UNIT;  // also the reduce-scatter staging

enum TpMode { TP_NONE = 0, TP_AG = 1, TP_RS = 2 };

struct TpParams {
  PeerCtx ctx;
  int tmc;             // pair tiles along M per row chunk: (M / W) / 256
  int rows_pc;         // rows per chunk: M / W
  // TP_AG
  const uint8_t* src[MAXW];  // rank r's copy of the gathered buffer (bytes)
  uint8_t* gathered;         // this rank's copy
  long long chunk_bytes;     // rows_pc * K * 2
  int* ready;                // [W * tmc] finished-unit counts per 256-row block, zero on entry
  int upb;                   // units per block: 256 * K * 2 / P_COPY_UNIT
  // TP_RS
  __nv_bfloat16* recv[MAXW]; // rank r's receive buffer [W][rows_pc][N]
  int* tflag[MAXW];          // rank r's tile flags [W][tmc * tiles_n][8]
};

template <int TP>
__device__ __forceinline__ void tp_tile_coords(int tile, const GemmParams& p, const TpParams& tp, int& tm, int& tn,
                                               int& chunk, int& ltile) {
  if (TP == TP_NONE) {
    tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
    chunk = 0;
    ltile = 0;
    return;
  }
  const int per_chunk = tp.tmc * p.tiles_n;
  const int slot = tile / per_chunk;
  // all-gather: own chunk first, then the peers in ring order; reduce-scatter: peers first, own chunk last
  chunk = (tp.ctx.rank + slot + (TP == TP_RS ? 1 : 0)) % tp.ctx.W;
  int ltm;
  tile_coords(tile - slot * per_chunk, tp.tmc, p.tiles_n, ltm, tn);
  tm = chunk * tp.tmc + ltm;
  ltile = ltm * p.tiles_n + tn;
}

__device__ __forceinline__ bool wait_count_gpu(const int* counter, int target, long long limit, int* err) {
  long long t0 = clock64();
  while (ld_acquire_gpu(counter) < target) {
    if (sga_aborted(err)) return false;
    if (clock64() - t0 > limit) {
      if (err) atomicOr(err, SGA_ERR_PEER_TIMEOUT);
      return false;
    }
    __nanosleep(128);
  }
  return true;
}

// The copy warp of the all-gather form (one elected lane): pulls this CTA's
// share of the peers' chunks, 16 KB units dealt round-robin over the grid in
// arrival order, two units in flight.
__device__ __forceinline__ void tp_ag_pull(const TpParams& tp, uint8_t* cbuf, uint64_t* cbar) {
  const PeerCtx& c = tp.ctx;
  const int G = (int)gridDim.x;
  const long long total = (long long)(c.W - 1) * tp.tmc * tp.upb;
  uint32_t phase[P_COPY_STAGES] = {0, 0};
  unsigned ready_seen = 0;
  bool ok = true;
  for (long long g0 = blockIdx.x; g0 < total && ok; g0 += (long long)G * P_COPY_STAGES) {
    uint8_t* dst[P_COPY_STAGES];
    int blk[P_COPY_STAGES];
    int nissued = 0;
    for (int j = 0; j < P_COPY_STAGES; ++j) {
      const long long g = g0 + (long long)j * G;
      if (g >= total) break;
      const int u = (int)(g % tp.upb);
      const long long sb = g / tp.upb;
      const int b = (int)(sb % tp.tmc);
      const int s = (int)(sb / tp.tmc) + 1;
      const int r = (c.rank + s) % c.W;
      if (!((ready_seen >> r) & 1)) {
        if (!wait_flag_sys(c.flags[c.rank] + r, c.seq, c.wait_cycles, c.err)) {
          ok = false;
          break;
        }
        fence_proxy_async_all();  // the peer's rows are read through the async proxy
        ready_seen |= 1u << r;
      }
      const long long off = (long long)r * tp.chunk_bytes + ((long long)b * tp.upb + u) * P_COPY_UNIT;
      dst[j] = tp.gathered + off;
      blk[j] = r * tp.tmc + b;
      mbar_expect_tx(&cbar[j], P_COPY_UNIT);
      bulk_load(cbuf + j * P_COPY_UNIT, tp.src[r] + off, P_COPY_UNIT, &cbar[j]);
      ++nissued;
    }
    for (int j = 0; j < nissued; ++j) {
      if (!mbar_wait(&cbar[j], phase[j], c.err)) ok = false;
      phase[j] ^= 1;
    }
    if (!ok) break;  // every issued load was waited for (or its wait ran out)
    for (int j = 0; j < nissued; ++j) bulk_store(dst[j], cbuf + j * P_COPY_UNIT, P_COPY_UNIT);
    tma_store_commit();
    tma_store_wait<0>();
    fence_proxy_async_all();
    __threadfence();
    for (int j = 0; j < nissued; ++j) red_release_gpu_add(tp.ready + blk[j], 1);
  }
  if (!ok) __nanosleep(200000);  // let a load that is still in flight land before the CTA can exit
}

template <int A_MN, int B_MN, int TP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TP == TP_AG ? P_THREADS_AG : P_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const GemmParams p, const TpParams tp) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + P_STAGES;
  uint64_t* tfull_bar = empty_bar + P_STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* copy_bar = tempty_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(copy_bar + P_COPY_STAGES);
  uint8_t* copy_buf = smem + P_STAGES * P_STAGE_BYTES + 1024;  // all-gather pull ring / reduce-scatter staging

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + P_BK - 1) / P_BK;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);  // 4 epilogue warps in each CTA of the pair
    }
    for (int s = 0; s < P_COPY_STAGES; ++s) mbar_init(&copy_bar[s], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, P_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = pair_id; tile < num_tiles; tile += num_pairs) {
        int tm, tn, chunk, ltile;
        tp_tile_coords<TP>(tile, p, tp, tm, tn, chunk, ltile);
        if (TP == TP_AG && chunk != tp.ctx.rank) {
          // the block's rows were written by bulk copies of other SMs: order them before this SM's TMA reads
          if (!wait_count_gpu(tp.ready + tm, tp.upb, tp.ctx.wait_cycles, p.err)) goto producer_done;
          fence_proxy_async_all();
        }
        const int m0 = tm * (2 * P_BM) + (int)rank * P_BM;
        const int n0 = tn * P_BN + (int)rank * P_BNH;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait_cluster(&empty_bar[stage], phase ^ 1, p.err)) goto producer_done;
          uint8_t* sa = smem + stage * P_STAGE_BYTES;
          uint8_t* sb = sa + P_A_BYTES;
          const uint32_t full_leader = mapa_shared(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * P_STAGE_BYTES);
          const int k0 = kb * P_BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < P_BM / 64; ++j)
              tma_load_2d_pair(sa + j * (64 * P_BK * 2), &tmA, full_leader, m0 + 64 * j, k0);
          } else {
            tma_load_2d_pair(sa, &tmA, full_leader, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < P_BNH / 64; ++j)
              tma_load_2d_pair(sb + j * (64 * P_BK * 2), &tmB, full_leader, n0 + 64 * j, k0);
          } else {
            tma_load_2d_pair(sb, &tmB, full_leader, k0, n0);
          }
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    producer_done:
      // after a failed wait: give the loads already issued time to land before the CTA can exit
      if (sga_aborted(p.err)) __nanosleep(200000);
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * P_BM, P_BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int t = 0;
      for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++t) {
        const int acc = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        if (!mbar_wait_cluster(&tempty_bar[acc], acc_phase ^ 1, p.err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * P_BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait_cluster(&full_bar[stage], phase, p.err)) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * P_STAGE_BYTES);
          const uint32_t sb = sa + P_A_BYTES;
#pragma unroll
          for (int k = 0; k < P_BK / 16; ++k) {
            const uint64_t da = A_MN ? umma_smem_desc_sw128(sa + k * 2048, 64 * P_BK * 2, 1024)
                                     : umma_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(sb + k * 2048, 64 * P_BK * 2, 1024)
                                     : umma_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit_pair(&empty_bar[stage], 3);
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        umma_commit_pair(&tfull_bar[acc], 3);
      }
    }
  } else if (warp < 6) {
    const int lg = warp & 3;
    int t = 0;
    unsigned done_seen = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++t) {
      int tm, tn, chunk, ltile;
      tp_tile_coords<TP>(tile, p, tp, tm, tn, chunk, ltile);
      const int acc = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait_cluster(&tfull_bar[acc], acc_phase, p.err))) break;
      tc_fence_after();
      const int row = tm * (2 * P_BM) + (int)rank * P_BM + lg * 32 + lane;
      const int n0 = tn * P_BN;
      if (TP != TP_RS) {
#pragma unroll 1
        for (int c = 0; c < P_BN; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(lg * 32) << 16) + acc * P_BN + c, r);
          tmem_ld_wait();
          store_row32(p, r, row, n0 + c);
        }
      } else {
        const PeerCtx& cx = tp.ctx;
        const int lrow = row - chunk * tp.rows_pc;
        const int tiles_local = tp.tmc * p.tiles_n;
        const int wslot = (int)rank * 4 + lg;
        if (chunk != cx.rank) {
          // the owner must have consumed what the previous launch on this channel left in its receive slot
          bool ok = true;
          if (!((done_seen >> chunk) & 1)) {
            if (lane == 0) ok = wait_flag_sys(cx.flags[cx.rank] + 8 + chunk, cx.prev_seq, cx.wait_cycles, cx.err);
            done_seen |= 1u << chunk;
          }
          if (!__all_sync(0xffffffffu, ok)) break;
          // Stage 32 rows x 128 columns of bf16 in this warp's shared buffer (16-byte chunks XOR-swizzled
          // by row), then write them out two rows per instruction: 256 contiguous bytes per row cross
          // NVLink as full packets instead of one 16-byte piece per lane.
          uint8_t* stg = copy_buf + (warp - 2) * (32 * 256);
          const int row0 = row - lane - chunk * tp.rows_pc;  // first local row of this warp
          __nv_bfloat16* dst0 = tp.recv[chunk] + ((size_t)cx.rank * tp.rows_pc + row0) * p.N + n0;
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
              uint32_t r[32];
              tmem_ld32(tmem_base + ((uint32_t)(lg * 32) << 16) + acc * P_BN + half * 128 + c, r);
              tmem_ld_wait();
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 o;
                __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  ob[i] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * i]) * p.alpha,
                                                __uint_as_float(r[v * 8 + 2 * i + 1]) * p.alpha);
                const int k16 = (c >> 3) + v;  // 16-byte chunk index within the 256-byte row
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((k16 ^ (lane & 15)) << 4)) = o;
              }
            }
            __syncwarp();
            const int k16 = lane & 15;
            const int col = n0 + half * 128 + k16 * 8;
            if (col < p.N) {
#pragma unroll 4
              for (int rr = 0; rr < 16; ++rr) {
                const int rw = rr * 2 + (lane >> 4);
                const uint4 o = *reinterpret_cast<const uint4*>(stg + rw * 256 + ((k16 ^ (rw & 15)) << 4));
                *reinterpret_cast<uint4*>(dst0 + (size_t)rw * p.N + half * 128 + k16 * 8) = o;
              }
            }
            __syncwarp();
          }
          __threadfence_system();
          __syncwarp();
          if (lane == 0) st_release_sys(tp.tflag[chunk] + ((size_t)cx.rank * tiles_local + ltile) * 8 + wslot, cx.seq);
        } else {
          bool ok = true;
          if (lane == 0) {
            for (int s = 0; s < cx.W && ok; ++s)
              if (s != cx.rank)
                ok = wait_flag_sys(tp.tflag[cx.rank] + ((size_t)s * tiles_local + ltile) * 8 + wslot, cx.seq,
                                   cx.wait_cycles, cx.err);
          }
          if (!__all_sync(0xffffffffu, ok)) break;
          GemmParams q = p;
          q.alpha = 1.f;
          q.M = tp.rows_pc;
#pragma unroll 1
          for (int c = 0; c < P_BN; c += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(lg * 32) << 16) + acc * P_BN + c, r);
            tmem_ld_wait();
            if (n0 + c < p.N) {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * p.alpha);
              for (int s = 0; s < cx.W; ++s) {
                if (s == cx.rank) continue;
                const __nv_bfloat16* src = tp.recv[cx.rank] + ((size_t)s * tp.rows_pc + lrow) * p.N + n0 + c;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  const uint4 rv = __ldcg(reinterpret_cast<const uint4*>(src + v * 8));
                  const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float2 x = __bfloat1622float2(rb[i]);
                    r[v * 8 + 2 * i] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * i]) + x.x);
                    r[v * 8 + 2 * i + 1] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * i + 1]) + x.y);
                  }
                }
              }
              store_row32(q, r, lrow, n0 + c);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
    }
  } else if (TP == TP_AG) {
    // warp 6: NVLink pull of the peers' chunks
    if (lane == 0) {
      if (blockIdx.x == 0) {
        __threadfence_system();
        for (int r = 0; r < tp.ctx.W; ++r) st_release_sys(tp.ctx.flags[r] + tp.ctx.rank, tp.ctx.seq);
      }
      tp_ag_pull(tp, copy_buf, copy_bar);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (TP != TP_NONE && threadIdx.x == 0) {
    // the last CTA to get here tells the peers that this rank is finished with their memory
    // (all-gather: pulled their chunks; reduce-scatter: consumed its receive slot)
    const PeerCtx& cx = tp.ctx;
    __threadfence();
    const int old = atomicAdd(cx.grid_counter, 1);
    if (old == (int)gridDim.x - 1) {
      *cx.grid_counter = 0;
      __threadfence_system();
      for (int r = 0; r < cx.W; ++r) st_release_sys(cx.flags[r] + 8 + cx.rank, cx.seq);
      if (TP == TP_AG) {
        // this rank's chunk may be rewritten once the kernel ends: hold until every peer has pulled it
        for (int r = 0; r < cx.W; ++r)
          if (r != cx.rank) wait_flag_sys(cx.flags[cx.rank] + 8 + r, cx.seq, cx.wait_cycles, cx.err);
      }
    }
  }
  cluster_sync_all();  // nobody signals into, or reads from, a CTA that has left
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, P_TMEM_COLS);
  }
}

// Host side shared by the launchers.
struct PairLaunch {
  TmaEncoder enc;
  int sms = 0;
  int num_sms() {
    if (sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return sms;
  }
  // tensor maps of A [M,K] / B [N,K] (or their MN-major forms) for the pair kernel's boxes
  int maps(CUtensorMap* ta, CUtensorMap* tb, const void* A, const void* B, int M, int N, int K, int a_mn, int b_mn,
           int lda, int ldb) {
    if (enc.ensure()) return -1;
    if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
      return -5;
    int rc = a_mn ? enc.make(ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, P_BK)
                  : enc.make(ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, P_BK, P_BM);
    if (rc) return rc;
    return b_mn ? enc.make(tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, P_BK)
                : enc.make(tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, P_BK, P_BNH);
  }
};

template <int A_MN, int B_MN, int TP>
static int launch_pair_kernel(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, const TpParams& tp,
                              int grid, cudaStream_t st) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, TP>;
  constexpr int smem = TP != TP_NONE ? P_SMEM_BYTES_AG : P_SMEM_BYTES;
  constexpr int threads = TP == TP_AG ? P_THREADS_AG : P_THREADS;
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
    attr[dev & 63] = true;
  }
  kern<<<grid, threads, smem, st>>>(ta, tb, p, tp);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace sga
