// Building blocks of the tcgen05 attention kernels (attention.cu).
//
// Every operand tile in shared memory has one physical form: for each 64-column
// slab of the head dimension, `rows` rows of 128 bytes, written by TMA with the
// 128-byte swizzle (or by threads with the same XOR pattern). The same bytes
// serve as a K-major operand (contraction over the head dimension) and as an
// MN-major operand (contraction over the rows), only the descriptor differs.
#pragma once
#include "gemm_common.cuh"

namespace sga {
namespace attn {

// [rows x hd] tile of the fused QKV (or dO) matrix -> shared memory, 64 x 64 boxes.
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int col0, int row0,
                                          int rows, int hd) {
  for (int c = 0; c < hd / 64; ++c)
    for (int p = 0; p < rows / 64; ++p)
      tma_load_2d(dst + c * rows * 128 + p * 8192, tm, bar, col0 + 64 * c, row0 + 64 * p);
}

// K-major view: slab c of the head dimension, 16-element step kk within it.
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int rows, int c, int kk) {
  return umma_smem_desc_sw128(base + c * rows * 128 + kk * 32, 16, 1024);
}
// MN-major view: 16-row step kk16 of the contraction over rows; the slabs of the
// head dimension (the N extent) lie rows * 128 bytes apart.
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int rows, int kk16) {
  return umma_smem_desc_sw128(base + kk16 * 2048, rows * 128, 1024);
}

// D[128 x N] (+)= A[128 x hd] B[N x hd]^T, both K-major tiles.
__device__ __forceinline__ void mma_over_hd(uint32_t d_tmem, uint32_t a_base, int a_rows, uint32_t b_base,
                                            int b_rows, int hd, uint32_t idesc) {
  for (int c = 0; c < hd / 64; ++c)
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      umma_f16(d_tmem, desc_k(a_base, a_rows, c, kk), desc_k(b_base, b_rows, c, kk), idesc, (c | kk) != 0);
}

// D[128 x hd] (+)= A[128 x kdim] B[kdim x hd]: A K-major ([128 rows][kdim] in 64-column slabs),
// B MN-major (the [kdim rows x hd] tile as loaded).
__device__ __forceinline__ void mma_over_rows(uint32_t d_tmem, uint32_t a_base, uint32_t b_base, int kdim,
                                              uint32_t idesc, bool accumulate) {
  for (int k16 = 0; k16 < kdim / 16; ++k16)
    umma_f16(d_tmem, desc_k(a_base, 128, k16 >> 2, k16 & 3), desc_mn(b_base, kdim, k16), idesc,
             accumulate || k16 != 0);
}

// One thread's 32 consecutive values of row `r`, columns [col, col + 32), as bf16 into a
// K-major [128 rows][ncols] operand tile (the layout TMA would have produced).
__device__ __forceinline__ void store_p32(uint8_t* tile, int r, int col, const float (&p)[32]) {
  uint8_t* slab = tile + (col >> 6) * (128 * 128) + r * 128;
  const int k0 = (col & 63) >> 3;
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) ob[i] = __floats2bfloat162_rn(p[v * 8 + 2 * i], p[v * 8 + 2 * i + 1]);
    *reinterpret_cast<uint4*>(slab + (((k0 + v) ^ (r & 7)) << 4)) = o;
  }
}

}  // namespace attn
}  // namespace sga
