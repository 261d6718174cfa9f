// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 computes a 256 x 256 tile
// over two SMs. Each CTA stages its own 128 rows of A and its own 128 of the
// tile's 256 B rows (half the B traffic per SM of the single-CTA kernel, so
// more pipeline stages fit and the shared-memory fill rate per SM drops from
// 96 to 64 bytes per clock), holds the accumulator of its 128 rows in its own
// TMEM, and writes those rows out. One elected thread of the leader CTA
// (cluster rank 0) issues every MMA for the pair.
//
// Barriers: the "stage full" barrier lives in the leader; both CTAs' TMA loads
// credit their bytes to it through its shared::cluster address (plain per-CTA
// tile loads, nothing is multicast). "stage empty" and "accumulator full" live
// in both CTAs and are signalled together by tcgen05.commit with a CTA mask.
// "accumulator empty" lives in the leader; the peer's epilogue warps arrive on
// it remotely. Waits are bounded; on expiry the status word is set and the
// kernel still runs to its end, joins the cluster and frees TMEM.
//
// Same contract as sga_gemm_bf16 (gemm_tcgen05.cu), which remains the path
// for M < 256.
#include "gemm_common.cuh"

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
constexpr int P_TMEM_COLS = 512;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256;

template <int A_MN, int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + P_STAGES;
  uint64_t* tfull_bar = empty_bar + P_STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

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
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
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
  } else {
    const int lg = warp & 3;
    int t = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++t) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait_cluster(&tfull_bar[acc], acc_phase, p.err))) break;
      tc_fence_after();
      const int row = tm * (2 * P_BM) + (int)rank * P_BM + lg * 32 + lane;
      const int n0 = tn * P_BN;
#pragma unroll 1
      for (int c = 0; c < P_BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(lg * 32) << 16) + acc * P_BN + c, r);
        tmem_ld_wait();
        store_row32(p, r, row, n0 + c);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody signals into, or reads from, a CTA that has left
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, P_TMEM_COLS);
  }
}

}  // namespace sga

namespace sga {
static TmaEncoder g_pair_enc;
static int g_pair_sms = 0;
static bool g_pair_attr[4] = {false, false, false, false};

template <int A_MN, int B_MN>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN>;
  const int idx = A_MN * 2 + B_MN;
  if (!g_pair_attr[idx]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess)
      return -3;
    g_pair_attr[idx] = true;
  }
  kern<<<grid, P_THREADS, P_SMEM_BYTES, st>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
}  // namespace sga

// Same arguments and meaning as sga_gemm_bf16; tiles are 256 x 256 over CTA pairs.
SGA_API int sga_gemm_bf16_pair(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int a_mn,
                               int b_mn, int lda, int ldb, int ldc, int epi, float alpha, int* err, int max_ctas,
                               void* stream) {
  using namespace sga;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (g_pair_enc.ensure()) return -1;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -5;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc & 7)) return -5;
  if (g_pair_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_pair_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int rc = a_mn ? g_pair_enc.make(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, P_BK)
                : g_pair_enc.make(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, P_BK, P_BM);
  if (rc) return rc;
  rc = b_mn ? g_pair_enc.make(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, P_BK)
            : g_pair_enc.make(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, P_BK, P_BNH);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.epi = epi;
  p.tiles_m = (M + 2 * P_BM - 1) / (2 * P_BM);
  p.tiles_n = (N + P_BN - 1) / P_BN;
  p.alpha = alpha; p.C = C; p.R = R ? R : C; p.err = err;
  int pairs = p.tiles_m * p.tiles_n;
  int cap = g_pair_sms / 2;
  if (max_ctas > 0 && max_ctas / 2 < cap) cap = max_ctas / 2;
  if (cap < 1) cap = 1;
  if (pairs > cap) pairs = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn && b_mn) return launch_pair<1, 1>(ta, tb, p, 2 * pairs, st);
  if (a_mn) return launch_pair<1, 0>(ta, tb, p, 2 * pairs, st);
  if (b_mn) return launch_pair<0, 1>(ta, tb, p, 2 * pairs, st);
  return launch_pair<0, 0>(ta, tb, p, 2 * pairs, st);
}
