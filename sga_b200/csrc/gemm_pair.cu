// bf16 GEMM on CTA pairs (tcgen05.mma.cta_group::2, 256 x 256 tiles over two
// SMs): the plain launcher. The kernel itself is in gemm_pair.cuh, where its
// pipeline and barriers are described; the tensor-parallel launchers that fuse
// an all-gather or a reduce-scatter into it are in gemm_tp.cu.
//
// Same contract as sga_gemm_bf16 (gemm_tcgen05.cu), which remains the path
// for M < 256.
#include "gemm_pair.cuh"

namespace sga {
static PairLaunch g_pair;
}

// Same arguments and meaning as sga_gemm_bf16; tiles are 256 x 256 over CTA pairs.
SGA_API int sga_gemm_bf16_pair(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int a_mn,
                               int b_mn, int lda, int ldb, int ldc, int epi, float alpha, int* err, int max_ctas,
                               void* stream) {
  using namespace sga;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc & 7)) return -5;
  CUtensorMap ta, tb;
  int rc = g_pair.maps(&ta, &tb, A, B, M, N, K, a_mn, b_mn, lda, ldb);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.epi = epi;
  p.tiles_m = (M + 2 * P_BM - 1) / (2 * P_BM);
  p.tiles_n = (N + P_BN - 1) / P_BN;
  p.alpha = alpha; p.C = C; p.R = R ? R : C; p.err = err;
  int pairs = p.tiles_m * p.tiles_n;
  int cap = g_pair.num_sms() / 2;
  if (max_ctas > 0 && max_ctas / 2 < cap) cap = max_ctas / 2;
  if (cap < 1) cap = 1;
  if (pairs > cap) pairs = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TpParams tp = {};
  if (a_mn && b_mn) return launch_pair_kernel<1, 1, TP_NONE>(ta, tb, p, tp, 2 * pairs, st);
  if (a_mn) return launch_pair_kernel<1, 0, TP_NONE>(ta, tb, p, tp, 2 * pairs, st);
  if (b_mn) return launch_pair_kernel<0, 1, TP_NONE>(ta, tb, p, tp, 2 * pairs, st);
  return launch_pair_kernel<0, 0, TP_NONE>(ta, tb, p, tp, 2 * pairs, st);
}
