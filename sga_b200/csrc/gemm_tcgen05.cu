// bf16 GEMM on the sm_100a tensor cores: tcgen05.mma with the accumulator in
// TMEM, operands staged into 128-byte-swizzled shared memory by TMA (plain
// per-CTA loads, no multicast), a persistent warp-specialised CTA per SM:
//
//   warp 0      TMA producer   (one lane)
//   warp 1      MMA issuer     (one lane; also owns TMEM alloc / dealloc)
//   warps 2..5  epilogue       (tcgen05.ld -> registers -> global)
//
// Two TMEM accumulators (2 x 256 columns) let the epilogue of tile i overlap
// the main loop of tile i+1. Every wait is bounded (common.cuh); on expiry the
// status word is set and the kernel still runs to its end and frees TMEM.
//
// C[M,N] = A[M,K] * B[N,K]^T with each operand either K-major (stored
// [rows, K], K contiguous) or MN-major (stored [K, rows], rows contiguous), so
// the forward (x W^T), dgrad (dy W) and wgrad (dy^T x) products of a linear
// layer all run without a transpose pass. The epilogue stores bf16, stores
// fp32, or accumulates into an fp32 C (main-grad accumulation for wgrad).
//
// Replaces the cuBLAS / TransformerEngine GEMMs that the reference reaches
// through its external Megatron stack (examples/llama3/train_1b_adamw.yaml:89,107).
#include "gemm_common.cuh"

namespace sga {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GEMM_SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1, p.err);
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (64 * BK * 2), &tmA, &full_bar[stage], m0 + 64 * j, k0);
          } else {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (64 * BK * 2), &tmB, &full_bar[stage], n0 + 64 * j, k0);
          } else {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int t = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
        const int acc = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.err);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(&full_bar[stage], phase, p.err);
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 16 bf16 = 32 bytes further inside the 128-byte swizzle row;
            //          8-row groups are 1024 bytes apart (stride byte offset).
            // MN-major: 16 K-rows of 128 bytes = 2048 bytes further; 64-wide MN
            //          groups are one 64x64 chunk (8192 bytes) apart (leading byte offset).
            const uint64_t da = A_MN ? umma_smem_desc_sw128(sa + k * 2048, 64 * BK * 2, 1024)
                                     : umma_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(sb + k * 2048, 64 * BK * 2, 1024)
                                     : umma_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        umma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    const int lg = warp & 3;  // TMEM lane group this warp may access
    int t = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1;
      mbar_wait(&tfull_bar[acc], acc_phase, p.err);
      tc_fence_after();
      const int row = tm * BM + lg * 32 + lane;
      const int n0 = tn * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(lg * 32) << 16) + acc * BN + c, r);
        tmem_ld_wait();
        store_row32(p, r, row, n0 + c);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host
static TmaEncoder g_enc;

static int g_num_sms = 0;
static bool g_attr_set[4] = {false, false, false, false};

template <int A_MN, int B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN>;
  const int idx = A_MN * 2 + B_MN;
  if (!g_attr_set[idx]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess)
      return -3;
    g_attr_set[idx] = true;
  }
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace sga

// C[M,N] (epi) = alpha * A * B^T. a_mn / b_mn: 0 = operand stored [rows, K]
// (K contiguous), 1 = stored [K, rows] (rows contiguous). lda / ldb / ldc are
// row pitches in elements of the stored matrices. Returns 0 or a negative code.
SGA_API int sga_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int a_mn,
                          int b_mn, int lda, int ldb, int ldc, int epi, float alpha, int* err, int max_ctas,
                          void* stream) {
  using namespace sga;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (g_enc.ensure()) return -1;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -5;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc & 7)) return -5;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int rc;
  if (a_mn)
    rc = g_enc.make(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK);
  else
    rc = g_enc.make(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (rc) return rc;
  if (b_mn)
    rc = g_enc.make(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK);
  else
    rc = g_enc.make(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN);
  if (rc) return rc;
  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.epi = epi;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.alpha = alpha;
  p.C = C;
  p.R = R ? R : C;
  p.err = err;
  int grid = p.tiles_m * p.tiles_n;
  int cap = g_num_sms;
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn && b_mn) return launch<1, 1>(ta, tb, p, grid, st);
  if (a_mn) return launch<1, 0>(ta, tb, p, grid, st);
  if (b_mn) return launch<0, 1>(ta, tb, p, grid, st);
  return launch<0, 0>(ta, tb, p, grid, st);
}
