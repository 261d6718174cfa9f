// Pieces shared by the single-CTA and the CTA-pair tcgen05 GEMM kernels:
// parameters, epilogue modes, the accumulator-row store and the host-side
// tensor-map encoder.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>

namespace sga {

enum EpiMode { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2, EPI_BF16_ADD = 3 };

struct GemmParams {
  int M, N, K;
  int ldc;
  int epi;
  int tiles_m, tiles_n;
  float alpha;
  void* C;
  const void* R;  // optional bf16 residual added in EPI_BF16_ADD (same pitch as C)
  int* err;
};

// Grouped raster: GROUP row-tiles share each column sweep so that the B tile
// (weights) and a band of A stay hot in L2 for the CTAs running together.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP = 16;
  const int per_group = GROUP * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsize = min(tiles_m - first_m, GROUP);
  const int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

// One thread's 32 consecutive fp32 accumulator columns of one row -> C.
__device__ __forceinline__ void store_row32(const GemmParams& p, const uint32_t (&r)[32], int row, int col) {
  if (row >= p.M || col >= p.N) return;
  const bool full = (col + 32 <= p.N);
  const size_t off = (size_t)row * p.ldc + col;
  if (p.epi == EPI_BF16 || p.epi == EPI_BF16_ADD) {
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
    const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(p.R) + off;
    if (full) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]) * p.alpha;
        if (p.epi == EPI_BF16_ADD) {
          const uint4 rv = *reinterpret_cast<const uint4*>(res + v * 8);
          const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 x = __bfloat1622float2(rb[i]);
            f[2 * i] += x.x;
            f[2 * i + 1] += x.y;
          }
        }
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) ob[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(out + v * 8) = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col + i < p.N) {
          float f = __uint_as_float(r[i]) * p.alpha;
          if (p.epi == EPI_BF16_ADD) f += __bfloat162float(res[i]);
          out[i] = __float2bfloat16_rn(f);
        }
      }
    }
  } else {
    float* out = reinterpret_cast<float*>(p.C) + off;
    if (full) {
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        float4 o;
        o.x = __uint_as_float(r[v * 4 + 0]) * p.alpha;
        o.y = __uint_as_float(r[v * 4 + 1]) * p.alpha;
        o.z = __uint_as_float(r[v * 4 + 2]) * p.alpha;
        o.w = __uint_as_float(r[v * 4 + 3]) * p.alpha;
        if (p.epi == EPI_F32_ACC) {
          const float4 old = *reinterpret_cast<const float4*>(out + v * 4);
          o.x += old.x;
          o.y += old.y;
          o.z += old.z;
          o.w += old.w;
        }
        *reinterpret_cast<float4*>(out + v * 4) = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col + i < p.N) {
          float f = __uint_as_float(r[i]) * p.alpha;
          if (p.epi == EPI_F32_ACC) f += out[i];
          out[i] = f;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ host
struct TmaEncoder {
  PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  int ensure() {
    if (fn) return 0;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) return -1;
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    return 0;
  }
  // 2-D bf16 map: `inner` contiguous elements per row, `outer` rows, pitch `ld`
  // elements, box (box_inner x box_outer), 128-byte swizzle.
  int make(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
           uint32_t box_outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -2;
  }
};

}  // namespace sga
