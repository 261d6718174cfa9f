// Building blocks of the tcgen05 attention kernels (attention.cu).
//
// Every operand tile in shared memory has one physical form: for each 64-column
// slab of the head dimension, `rows` rows of 128 bytes, written by TMA with the
// 128-byte swizzle (or by threads with the same XOR pattern). The same bytes
// serve as a K-major operand (contraction over the head dimension) and as an
// MN-major operand (contraction over the rows), only the descriptor differs.
#pragma once
#include "gemm_common.cuh"
#include <stdlib.h>

namespace sga {
namespace attn {

// How the softmax threads tell the MMA thread that an operand tile is in shared memory. Default: every
// thread fences its own stores, the warp synchronises, one lane arrives (4 to 16 arrivals on the barrier
// per tile instead of 128 to 512 serialised ones). SGA_ATTN_ARRIVE=thread restores one arrival per thread.
static inline int attn_warp_arrive() {
  static const int v = [] {
    const char* e = getenv("SGA_ATTN_ARRIVE");
    return (e && e[0] == 't') ? 0 : 1;
  }();
  return v;
}

// [rows x hd] tile of the fused QKV (or dO) matrix -> shared memory, 64 x 64 boxes.
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int col0, int row0,
                                          int rows, int hd) {
  for (int c = 0; c < hd / 64; ++c)
    for (int p = 0; p < rows / 64; ++p)
      tma_load_2d(dst + c * rows * 128 + p * 8192, tm, bar, col0 + 64 * c, row0 + 64 * p);
}

// Descriptors. The start-address field of a shared-memory descriptor counts 16-byte units in its low
// bits, so the descriptor of "base + x bytes" is the base descriptor plus (x >> 4): one thread issues
// every MMA of a CTA, and with the offsets folded to constants an MMA costs it two integer adds.
// K-major view of a tile (contraction over the head dimension).
__device__ __forceinline__ uint64_t desc_k(uint32_t base) { return umma_smem_desc_sw128(base, 16, 1024); }
// MN-major view (contraction over the tile's rows); the 64-column slabs of the head dimension, which
// form the N extent, lie rows * 128 bytes apart.
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int rows) {
  return umma_smem_desc_sw128(base, rows * 128, 1024);
}

// D[128 x N] = A[128 x HD] B[N x HD]^T, both K-major tiles of A_ROWS / B_ROWS rows.
template <int HD, int A_ROWS, int B_ROWS>
__device__ __forceinline__ void mma_over_hd(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
#pragma unroll
  for (int c = 0; c < HD / 64; ++c)
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      umma_f16(d_tmem, a_desc + (uint64_t)((c * A_ROWS * 128 + kk * 32) >> 4),
               b_desc + (uint64_t)((c * B_ROWS * 128 + kk * 32) >> 4), idesc, (c | kk) != 0);
}

// D[128 x hd] (+)= A[128 x KDIM] B[KDIM x hd]: A K-major ([128 rows][KDIM] in 64-column slabs),
// B MN-major (the [KDIM rows x hd] tile as loaded).
template <int KDIM>
__device__ __forceinline__ void mma_over_rows(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              bool accumulate) {
#pragma unroll
  for (int k16 = 0; k16 < KDIM / 16; ++k16)
    umma_f16(d_tmem, a_desc + (uint64_t)(((k16 >> 2) * 128 * 128 + (k16 & 3) * 32) >> 4),
             b_desc + (uint64_t)((k16 * 2048) >> 4), idesc, accumulate || k16 != 0);
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

// The same from 16 already packed bf16 pairs (pair i = columns col + 2i, col + 2i + 1).
__device__ __forceinline__ void store_pk32(uint8_t* tile, int r, int col, const uint32_t (&pk)[16]) {
  uint8_t* slab = tile + (col >> 6) * (128 * 128) + r * 128;
  const int k0 = (col & 63) >> 3;
#pragma unroll
  for (int v = 0; v < 4; ++v)
    *reinterpret_cast<uint4*>(slab + (((k0 + v) ^ (r & 7)) << 4)) =
        make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
}

// The same for 16 values, columns [col, col + 16).
__device__ __forceinline__ void store_p16(uint8_t* tile, int r, int col, const float (&p)[16]) {
  uint8_t* slab = tile + (col >> 6) * (128 * 128) + r * 128;
  const int k0 = (col & 63) >> 3;
#pragma unroll
  for (int v = 0; v < 2; ++v) {
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) ob[i] = __floats2bfloat162_rn(p[v * 8 + 2 * i], p[v * 8 + 2 * i + 1]);
    *reinterpret_cast<uint4*>(slab + (((k0 + v) ^ (r & 7)) << 4)) = o;
  }
}

}  // namespace attn
}  // namespace sga
