// Tensor-parallel linear layers with the collective inside the GEMM kernel
// (sequence-parallel form: activations outside the linears are sharded by
// rows over the tensor-parallel ranks).
//
//   sga_tp_ag_gemm   C[M, N] = gather_rows(A)[M, K] @ B^T      (column-parallel
//                    forward; row-parallel input gradient with b_mn)
//   sga_tp_gemm_rs   C[M/W, N] = reduce_scatter_rows(A[M, K] @ B^T) (+ R)
//                    (row-parallel forward; column-parallel input gradient)
//
// Both run the CTA-pair tcgen05 kernel of gemm_pair.cuh; how the transfer is
// interleaved with the tiles is described there. Peer memory is touched only
// by bulk copies without multicast (the pull) and by plain stores / loads
// (the partial tiles and flags); every TMA tile load reads this GPU's memory.
//
// The reference leaves tensor parallelism to its external training stack and
// refuses it for sparse steps (sga/runtime.py:50-52); here the data-parallel
// gradient machinery runs unchanged on each tensor-parallel shard.
#include "gemm_pair.cuh"

namespace sga {
static PairLaunch g_tp;

static int tp_grid(const GemmParams& p, int max_ctas) {
  int pairs = p.tiles_m * p.tiles_n;
  int cap = g_tp.num_sms() / 2;
  if (max_ctas > 0 && max_ctas / 2 < cap) cap = max_ctas / 2;
  if (cap < 1) cap = 1;
  return 2 * (pairs > cap ? cap : pairs);
}
}  // namespace sga

// gathered: void*[8], rank r's copy of the [M, K] bf16 gathered buffer (contiguous rows, pitch K);
// this rank's row chunk [rank * M/W, (rank+1) * M/W) must be final in its own copy before the launch.
// ready: int[M / 256] zeroed by the caller on the launching stream before every launch.
// Requires M % (256 * W) == 0, K % 32 == 0.
SGA_API int sga_tp_ag_gemm(const SgaPeerDesc* d, void* const* gathered, const void* B, void* C, int M, int N, int K,
                           int b_mn, int ldb, int ldc, int epi, float alpha, int* ready, int max_ctas, void* stream) {
  using namespace sga;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int W = d->W;
  if (W < 1 || W > MAXW || M % (2 * P_BM * W) || (K & 31)) return -5;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc & 7)) return -5;
  CUtensorMap ta, tb;
  int rc = g_tp.maps(&ta, &tb, gathered[d->rank], B, M, N, K, 0, b_mn, K, ldb);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.epi = epi;
  p.tiles_m = M / (2 * P_BM);
  p.tiles_n = (N + P_BN - 1) / P_BN;
  p.alpha = alpha; p.C = C; p.R = C; p.err = reinterpret_cast<int*>(d->err);
  TpParams tp = {};
  tp.ctx = make_ctx(d);
  tp.rows_pc = M / W;
  tp.tmc = tp.rows_pc / (2 * P_BM);
  for (int r = 0; r < W; ++r) tp.src[r] = reinterpret_cast<const uint8_t*>(gathered[r]);
  tp.gathered = reinterpret_cast<uint8_t*>(gathered[d->rank]);
  tp.chunk_bytes = (long long)tp.rows_pc * K * 2;
  tp.ready = ready;
  tp.upb = (2 * P_BM * K * 2) / P_COPY_UNIT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = tp_grid(p, max_ctas);
  if (b_mn) return launch_pair_kernel<0, 1, TP_AG>(ta, tb, p, tp, grid, st);
  return launch_pair_kernel<0, 0, TP_AG>(ta, tb, p, tp, grid, st);
}

// A: [M, K] (or MN-major with a_mn), B: [N, K] (or MN-major). recv: void*[8], rank r's receive
// buffer of W * (M/W) * N bf16; tflag: void*[8], rank r's int[W * tiles * 8] tile flags (never reset:
// they carry the channel's sequence number). C / R: [M/W, N] bf16, pitch ldc; epi is EPI_BF16 or
// EPI_BF16_ADD. Requires M % (256 * W) == 0, N % 32 == 0.
SGA_API int sga_tp_gemm_rs(const SgaPeerDesc* d, const void* A, const void* B, void* C, const void* R,
                           void* const* recv, void* const* tflag, int M, int N, int K, int a_mn, int b_mn, int lda,
                           int ldb, int ldc, int epi, float alpha, int max_ctas, void* stream) {
  using namespace sga;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int W = d->W;
  if (W < 1 || W > MAXW || M % (2 * P_BM * W) || (N & 31)) return -5;
  if (epi != EPI_BF16 && epi != EPI_BF16_ADD) return -5;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc & 7)) return -5;
  CUtensorMap ta, tb;
  int rc = g_tp.maps(&ta, &tb, A, B, M, N, K, a_mn, b_mn, lda, ldb);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.epi = epi;
  p.tiles_m = M / (2 * P_BM);
  p.tiles_n = (N + P_BN - 1) / P_BN;
  p.alpha = alpha; p.C = C; p.R = R ? R : C; p.err = reinterpret_cast<int*>(d->err);
  TpParams tp = {};
  tp.ctx = make_ctx(d);
  tp.rows_pc = M / W;
  tp.tmc = tp.rows_pc / (2 * P_BM);
  for (int r = 0; r < W; ++r) {
    tp.recv[r] = reinterpret_cast<__nv_bfloat16*>(recv[r]);
    tp.tflag[r] = reinterpret_cast<int*>(tflag[r]);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = tp_grid(p, max_ctas);
  if (a_mn && b_mn) return launch_pair_kernel<1, 1, TP_RS>(ta, tb, p, tp, grid, st);
  if (a_mn) return launch_pair_kernel<1, 0, TP_RS>(ta, tb, p, tp, grid, st);
  if (b_mn) return launch_pair_kernel<0, 1, TP_RS>(ta, tb, p, tp, grid, st);
  return launch_pair_kernel<0, 0, TP_RS>(ta, tb, p, tp, grid, st);
}
