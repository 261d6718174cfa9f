// Backward of the causal grouped-query attention (tcgen05 + TMEM), in three
// launches and without atomics, so gradients are reproducible bit for bit:
//
//   sga_attn_bwd step 1  delta[b, h, s] = sum_d dO * O                         (one warp per row and head)
//   step 2 (dQ kernel)   one CTA per (256 query rows, head, batch), two warpgroups as in the
//                        forward: S = Q K^T and dP = dO V^T into TMEM, threads form
//                        dS = P (dP - delta) with P = exp2(S - lse), the tensor core accumulates
//                        dQ += dS K in TMEM over the key blocks.
//   step 3 (dK/dV)       one CTA per (128 keys, KV head, batch); it walks the query heads of the
//                        group and their 64-row query blocks from the diagonal down:
//                        S^T = K Q^T and dP^T = V dO^T into TMEM (double-buffered), threads form
//                        P^T and dS^T (a key row and 16 queries each; lse and delta of the 64 queries are
//                        broadcast from shared memory), and dV += P^T dO, dK += dS^T Q accumulate
//                        in TMEM over the whole walk: the sum over the group's query heads
//                        happens in the accumulator.
//
// The score matrix is recomputed in both kernels (seven products instead of five) in exchange
// for the fixed order of summation. Tiles and descriptors are those of attention.cuh.
#include "attention.cuh"

namespace sga {
namespace attn {

struct BwdParams {
  int B, S, nq, nkv, hd;
  int ld_dqkv;            // row pitch of dqkv in elements
  float scale, scale_log2;
  const float* lse;       // [B, nq, S]
  const float* delta;     // [B, nq, S]
  __nv_bfloat16* dqkv;    // [T, (nq + 2 nkv) * hd]
  int* err;
  int warp_arrive;        // see attn_warp_arrive()
};

// ------------------------------------------------------------------ delta
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dctx, const __nv_bfloat16* __restrict__ ctx,
                                  float* __restrict__ delta, int B, int S, int nq, int hd, long long ld_d,
                                  long long ld_c) {
  // hd / 8 consecutive lanes share one (token, head): each loads 16 bytes of dO and of O
  const int per = hd >> 3;                      // 8 (hd 64) or 16 (hd 128) lanes per row
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gt / per;               // (token, head) index
  const int part = (int)(gt % per);
  const long long total = (long long)B * S * nq;
  float acc = 0.f;
  int h = 0;
  long long t = 0;
  if (row < total) {
    h = (int)(row % nq);
    t = row / nq;
    const uint4 a = *reinterpret_cast<const uint4*>(dctx + t * ld_d + (long long)h * hd + part * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(ctx + t * ld_c + (long long)h * hd + part * 8);
    const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* cb = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ab[i]), y = __bfloat1622float2(cb[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  for (int o = per >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (row < total && part == 0) {
    const int b = (int)(t / S), s = (int)(t % S);
    delta[((long long)b * nq + h) * S + s] = acc;
  }
}

// --------------------------------------------------------------- dQ kernel
constexpr int DQ_THREADS = 576;  // 16 softmax warps (two threads per query row) + TMA warp + MMA warp
constexpr int DQ_BN = 64;

template <int HD>
struct DqCfg {
  static constexpr int STAGES = HD == 64 ? 3 : 2;
  static constexpr int QDO_BYTES = 4 * 128 * HD * 2;       // Q and dO of both sub-blocks
  static constexpr int STAGE_BYTES = 2 * DQ_BN * HD * 2;   // K block + V block
  static constexpr int DS_BYTES = 128 * DQ_BN * 2;         // one warpgroup's dS tile
  static constexpr int SMEM = QDO_BYTES + STAGES * STAGE_BYTES + 2 * DS_BYTES + 1024 + 256;
};

template <int HD>
__global__ void __launch_bounds__(DQ_THREADS, 1) attn_dq_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                                                const __grid_constant__ CUtensorMap tmDO,
                                                                const BwdParams p) {
  using C = DqCfg<HD>;
  constexpr int BN = DQ_BN;
  constexpr int TILE = 128 * HD * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                    // [2] Q tiles, then [2] dO tiles
  uint8_t* sDO = sQ + 2 * TILE;
  uint8_t* sKV = sQ + C::QDO_BYTES;
  uint8_t* sDS = sKV + C::STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * C::DS_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + C::STAGES;
  uint64_t* sd_full = kv_empty + C::STAGES;   // S and dP of warpgroup w are in TMEM
  uint64_t* ds_full = sd_full + 2;            // dS tile of warpgroup w is in shared memory
  uint64_t* dq_done = ds_full + 2;            // the dQ product that read the dS tile has finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_done + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.nq / p.nkv);
  const int q0 = qblk * 256;
  const int nblk_seq = (p.S + BN - 1) / BN;
  int nw[2];
  for (int w = 0; w < 2; ++w) {
    const int last_row = min(q0 + 128 * w + 127, p.S - 1);
    nw[w] = q0 + 128 * w < p.S ? min(nblk_seq, last_row / BN + 1) : 0;
  }
  const int n_all = max(nw[0], nw[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&sd_full[w], 1);
      mbar_init(&ds_full[w], p.warp_arrive ? 8 : 256);
      mbar_init(&dq_done[w], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 17) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // per warpgroup: S [0,64), dP [64,128), dQ [128, 128 + HD)
  const uint32_t tW[2] = {tmem_base, tmem_base + 256};
  const int row_base = b * p.S;

  if (warp == 16) {
    if (lane == 0 && n_all > 0) {
      mbar_expect_tx(q_full, C::QDO_BYTES);
      for (int w = 0; w < 2; ++w) {
        load_tile(sQ + w * TILE, &tmQKV, q_full, h * HD, row_base + q0 + 128 * w, 128, HD);
        load_tile(sDO + w * TILE, &tmDO, q_full, h * HD, row_base + q0 + 128 * w, 128, HD);
      }
      for (int j = 0; j < n_all; ++j) {
        const int st = j % C::STAGES;
        if (!mbar_wait(&kv_empty[st], ((j / C::STAGES) & 1) ^ 1, p.err)) break;
        uint8_t* sk = sKV + st * C::STAGE_BYTES;
        mbar_expect_tx(&kv_full[st], C::STAGE_BYTES);
        load_tile(sk, &tmQKV, &kv_full[st], (p.nq + g) * HD, row_base + j * BN, BN, HD);
        load_tile(sk + BN * HD * 2, &tmQKV, &kv_full[st], (p.nq + p.nkv + g) * HD, row_base + j * BN, BN, HD);
      }
      if (sga_aborted(p.err)) __nanosleep(200000);
    }
  } else if (warp == 17) {
    if (lane == 0 && n_all > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BN, 0, 0);
      constexpr uint32_t idesc_q = umma_idesc_bf16(128, HD, 0, 1);
      const uint64_t dQ0 = desc_k(smem_u32(sQ)), dDO0 = desc_k(smem_u32(sDO)), dDS0 = desc_k(smem_u32(sDS));
      const uint64_t dK0 = desc_k(smem_u32(sKV)), dV0 = desc_k(smem_u32(sKV + BN * HD * 2));
      const uint64_t dKmn0 = desc_mn(smem_u32(sKV), BN);
      constexpr uint64_t T_STEP = TILE >> 4, DS_STEP = C::DS_BYTES >> 4, KV_STEP = C::STAGE_BYTES >> 4;
      auto scores = [&](int w, int st) {
        mma_over_hd<HD, 128, BN>(tW[w], dQ0 + w * T_STEP, dK0 + st * KV_STEP, idesc_s);
        mma_over_hd<HD, 128, BN>(tW[w] + 64, dDO0 + w * T_STEP, dV0 + st * KV_STEP, idesc_s);
        umma_commit(&sd_full[w]);
      };
      bool ok = mbar_wait(q_full, 0, p.err) && mbar_wait(&kv_full[0], 0, p.err);
      if (ok) {
        tc_fence_after();
        for (int w = 0; w < 2; ++w)
          if (nw[w] > 0) scores(w, 0);
      }
      for (int j = 0; j < n_all && ok; ++j) {
        const int st = j % C::STAGES;
        bool next_ready = false;
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= nw[w]) continue;
          ok = mbar_wait(&ds_full[w], j & 1, p.err);
          if (!ok) break;
          tc_fence_after();
          mma_over_rows<BN>(tW[w] + 128, dDS0 + w * DS_STEP, dKmn0 + st * KV_STEP, idesc_q, j > 0);
          umma_commit(&dq_done[w]);
          if (j + 1 < nw[w]) {
            const int sn = (j + 1) % C::STAGES;
            if (!next_ready) {
              ok = mbar_wait(&kv_full[sn], ((j + 1) / C::STAGES) & 1, p.err);
              if (!ok) break;
              tc_fence_after();
              next_ready = true;
            }
            scores(w, sn);
          }
        }
        if (ok) umma_commit(&kv_empty[st]);
      }
    }
  } else {
    const int w = warp >> 3;                   // query sub-block
    const int half = (warp >> 2) & 1;          // which 32 of the block's 64 keys this thread covers
    const int r = (warp & 3) * 32 + lane;
    const int qrow = q0 + 128 * w + r;
    const bool live = qrow < p.S;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint8_t* myDS = sDS + w * C::DS_BYTES;
    const size_t stat = ((size_t)b * p.nq + h) * p.S + (live ? qrow : 0);
    const float lse2 = live ? p.lse[stat] * 1.4426950408889634f : 0.f;
    const float dlt = live ? p.delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < nw[w] && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(&sd_full[w], j & 1, p.err));
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * BN;
      // some key of the block lies past some row of the sub-block, or the sub-block has rows past the sequence
      const bool diag = kv0 + BN - 1 > q0 + 128 * w || q0 + 128 * w + 127 >= p.S;
      {
        const int c = half * 32;
        uint32_t vs[32], vd[32];
        tmem_ld32(tW[w] + lane_off + c, vs);
        tmem_ld32(tW[w] + 64 + lane_off + c, vd);
        tmem_ld_wait();
        float ds[32];
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool keep = live && kv0 + c + i <= qrow;
            const float pr = keep ? exp2f(fmaf(__uint_as_float(vs[i]), p.scale_log2, -lse2)) : 0.f;
            ds[i] = keep ? pr * (__uint_as_float(vd[i]) - dlt) : 0.f;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            ds[i] = exp2f(fmaf(__uint_as_float(vs[i]), p.scale_log2, -lse2)) * (__uint_as_float(vd[i]) - dlt);
        }
        // the dS tile is free once the previous block's dQ product has read it
        if (j > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(&dq_done[w], (j - 1) & 1, p.err));
          if (!ok) break;
        }
        store_p32(myDS, r, c, ds);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      if (p.warp_arrive) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_full[w]);
      } else {
        mbar_arrive(&ds_full[w]);
      }
    }
    if (ok && nw[w] > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&dq_done[w], (nw[w] - 1) & 1, p.err));
      if (ok) {
        tc_fence_after();
        __nv_bfloat16* dst = p.dqkv + (size_t)(row_base + qrow) * p.ld_dqkv + h * HD;
#pragma unroll 1
        for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
          uint32_t v[32];
          tmem_ld32(tW[w] + 128 + lane_off + c, v);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              __nv_bfloat162* ub = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                ub[i] = __floats2bfloat162_rn(__uint_as_float(v[q4 * 8 + 2 * i]) * p.scale,
                                              __uint_as_float(v[q4 * 8 + 2 * i + 1]) * p.scale);
              *reinterpret_cast<uint4*>(dst + c + q4 * 8) = u;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 17) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------ dK/dV kernel
constexpr int DKV_THREADS = 576;  // 16 softmax warps (four threads per key row: 16 queries each) + TMA warp + MMA warp
constexpr int DKV_BQ = 64;

template <int HD>
struct DkvCfg {
  static constexpr int STAGES = HD == 64 ? 4 : 3;
  static constexpr int KV_BYTES = 2 * 128 * HD * 2;         // K and V of the block
  static constexpr int STAGE_BYTES = 2 * DKV_BQ * HD * 2;   // Q block + dO block
  static constexpr int PT_BYTES = 128 * DKV_BQ * 2;         // P^T (or dS^T) tile
  static constexpr int SMEM = KV_BYTES + STAGES * STAGE_BYTES + 4 * PT_BYTES + 2048 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(DKV_THREADS, 1) attn_dkv_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                                                  const __grid_constant__ CUtensorMap tmDO,
                                                                  const BwdParams p) {
  using C = DkvCfg<HD>;
  constexpr int BQ = DKV_BQ;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + 128 * HD * 2;
  uint8_t* sQD = sK + C::KV_BYTES;                       // [stage]{Q [HD/64][64][128 B], dO the same}
  uint8_t* sPT = sQD + C::STAGES * C::STAGE_BYTES;       // [2] P^T tiles, then [2] dS^T tiles
  uint8_t* sDS = sPT + 2 * C::PT_BYTES;
  float* sStat = reinterpret_cast<float*>(sDS + 2 * C::PT_BYTES);  // [set][2]{lse2[64], delta[64]}
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 512);
  uint64_t* kv_full = bars;
  uint64_t* qd_full = bars + 1;
  uint64_t* qd_empty = qd_full + C::STAGES;
  uint64_t* st_full = qd_empty + C::STAGES;   // S^T and dP^T of buffer u are in TMEM
  uint64_t* pt_full = st_full + 2;            // P^T and dS^T tiles of buffer u are in shared memory
  uint64_t* acc_done = pt_full + 2;           // the dV / dK products that read buffer u have finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kvblk = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int rep = p.nq / p.nkv;
  const int kv0 = kvblk * 128;
  const int i0 = kv0 / BQ;                               // first query block that can see these keys
  const int nqb = (p.S + BQ - 1) / BQ - i0;              // query blocks per head
  const int nt = rep * nqb;                              // steps: heads of the group x query blocks
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&qd_full[s], 1);
      mbar_init(&qd_empty[s], 1);
    }
    for (int u = 0; u < 2; ++u) {
      mbar_init(&st_full[u], 1);
      mbar_init(&pt_full[u], p.warp_arrive ? 16 : 512);
      mbar_init(&acc_done[u], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 17) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // S^T buffers [0,64) [64,128); dP^T buffers [128,192) [192,256); dV [256, 256+HD); dK [384, 384+HD)
  const uint32_t tST[2] = {tmem_base, tmem_base + 64};
  const uint32_t tDP[2] = {tmem_base + 128, tmem_base + 192};
  const uint32_t tDV = tmem_base + 256, tDK = tmem_base + 384;

  if (warp == 16) {
    if (lane == 0 && nt > 0) {
      mbar_expect_tx(kv_full, C::KV_BYTES);
      load_tile(sK, &tmQKV, kv_full, (p.nq + g) * HD, row_base + kv0, 128, HD);
      load_tile(sV, &tmQKV, kv_full, (p.nq + p.nkv + g) * HD, row_base + kv0, 128, HD);
      for (int t = 0; t < nt; ++t) {
        const int st = t % C::STAGES;
        if (!mbar_wait(&qd_empty[st], ((t / C::STAGES) & 1) ^ 1, p.err)) break;
        const int h = g * rep + t / nqb, i = i0 + t % nqb;
        uint8_t* sq = sQD + st * C::STAGE_BYTES;
        mbar_expect_tx(&qd_full[st], C::STAGE_BYTES);
        load_tile(sq, &tmQKV, &qd_full[st], h * HD, row_base + i * BQ, BQ, HD);
        load_tile(sq + BQ * HD * 2, &tmDO, &qd_full[st], h * HD, row_base + i * BQ, BQ, HD);
      }
      if (sga_aborted(p.err)) __nanosleep(200000);
    }
  } else if (warp == 17) {
    if (lane == 0 && nt > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BQ, 0, 0);
      constexpr uint32_t idesc_a = umma_idesc_bf16(128, HD, 0, 1);
      const uint64_t dKk = desc_k(smem_u32(sK)), dVk = desc_k(smem_u32(sV));
      const uint64_t dQk0 = desc_k(smem_u32(sQD)), dDOk0 = desc_k(smem_u32(sQD + BQ * HD * 2));
      const uint64_t dQmn0 = desc_mn(smem_u32(sQD), BQ), dDOmn0 = desc_mn(smem_u32(sQD + BQ * HD * 2), BQ);
      const uint64_t dPT0 = desc_k(smem_u32(sPT)), dDS0 = desc_k(smem_u32(sDS));
      constexpr uint64_t ST_STEP = C::STAGE_BYTES >> 4, PT_STEP = C::PT_BYTES >> 4;
      auto scores = [&](int t) -> bool {
        const int st = t % C::STAGES, u = t & 1;
        if (!mbar_wait(&qd_full[st], (t / C::STAGES) & 1, p.err)) return false;
        tc_fence_after();
        mma_over_hd<HD, 128, BQ>(tST[u], dKk, dQk0 + st * ST_STEP, idesc_s);
        mma_over_hd<HD, 128, BQ>(tDP[u], dVk, dDOk0 + st * ST_STEP, idesc_s);
        umma_commit(&st_full[u]);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, p.err);
      if (ok) {
        tc_fence_after();
        ok = scores(0);
        if (ok && nt > 1) ok = scores(1);
      }
      for (int t = 0; t < nt && ok; ++t) {
        const int st = t % C::STAGES, u = t & 1;
        ok = mbar_wait(&pt_full[u], (t >> 1) & 1, p.err);
        if (!ok) break;
        tc_fence_after();
        mma_over_rows<BQ>(tDV, dPT0 + u * PT_STEP, dDOmn0 + st * ST_STEP, idesc_a, t > 0);
        mma_over_rows<BQ>(tDK, dDS0 + u * PT_STEP, dQmn0 + st * ST_STEP, idesc_a, t > 0);
        umma_commit(&acc_done[u]);
        umma_commit(&qd_empty[st]);
        if (t + 2 < nt) ok = scores(t + 2);
      }
    }
  } else {
    // Sixteen warps share a step: a key row belongs to four threads, 16 queries each.
    const int r = (warp & 3) * 32 + lane;      // key row within the block
    const int quarter = warp >> 2;
    const int kpos = kv0 + r;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    // lse (in log2 units) and delta of a step's 64 queries go through shared memory (threads 0..127 load
    // them one step ahead, so the global latency is off the step's critical path)
    auto load_stat = [&](int t) -> float {
      const int h = g * rep + t / nqb, i = i0 + t % nqb;
      const int qi = i * BQ + (threadIdx.x & 63);
      if (t >= nt || qi >= p.S) return 0.f;
      const size_t at = ((size_t)b * p.nq + h) * p.S + qi;
      return threadIdx.x < 64 ? p.lse[at] * 1.4426950408889634f : p.delta[at];
    };
    if (threadIdx.x < 128) sStat[threadIdx.x] = load_stat(0);
    // After a failed wait a warp keeps walking the steps (doing nothing) so that every warp meets the
    // same number of named barriers.
    for (int t = 0; t < nt; ++t) {
      const int u = t & 1;
      const int i = i0 + t % nqb;
      asm volatile("bar.sync 1, 512;" ::: "memory");
      // everyone has left step t - 1, whose statistics lived in the other buffer: refill it for step t + 1
      float nxt = 0.f;
      if (threadIdx.x < 128) nxt = load_stat(t + 1);
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&st_full[u], (t >> 1) & 1, p.err));
      if (ok) {
        tc_fence_after();
        const int qb0 = i * BQ;
        const int c = quarter * 16;
        const float4* l4 = reinterpret_cast<const float4*>(sStat + u * 128 + c);
        const float4* d4 = reinterpret_cast<const float4*>(sStat + u * 128 + 64 + c);
        // the block's first query lies before the block's last key, or its last query past the sequence
        const bool diag = qb0 < kv0 + 128 || qb0 + BQ > p.S;
        uint32_t vs[16], vd[16];
        tmem_ld16(tST[u] + lane_off + c, vs);
        tmem_ld16(tDP[u] + lane_off + c, vd);
        float l2[16], dl[16];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 a = l4[k], d = d4[k];
          l2[4 * k] = a.x; l2[4 * k + 1] = a.y; l2[4 * k + 2] = a.z; l2[4 * k + 3] = a.w;
          dl[4 * k] = d.x; dl[4 * k + 1] = d.y; dl[4 * k + 2] = d.z; dl[4 * k + 3] = d.w;
        }
        tmem_ld_wait();
        float pt[16], ds[16];
        if (diag) {
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const int qpos = qb0 + c + k;
            const bool keep = qpos >= kpos && qpos < p.S;
            const float pr = keep ? exp2f(fmaf(__uint_as_float(vs[k]), p.scale_log2, -l2[k])) : 0.f;
            pt[k] = pr;
            ds[k] = keep ? pr * (__uint_as_float(vd[k]) - dl[k]) : 0.f;
          }
        } else {
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const float pr = exp2f(fmaf(__uint_as_float(vs[k]), p.scale_log2, -l2[k]));
            pt[k] = pr;
            ds[k] = pr * (__uint_as_float(vd[k]) - dl[k]);
          }
        }
        // the tiles of buffer u are free once the products of step t - 2 have read them
        if (t >= 2) ok = __all_sync(0xffffffffu, mbar_wait(&acc_done[u], ((t - 2) >> 1) & 1, p.err));
        if (ok) {
          store_p16(sPT + u * C::PT_BYTES, r, c, pt);
          store_p16(sDS + u * C::PT_BYTES, r, c, ds);
          tc_fence_before();
          fence_proxy_async_smem();
          if (p.warp_arrive) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&pt_full[u]);
          } else {
            mbar_arrive(&pt_full[u]);
          }
        }
      }
      if (threadIdx.x < 128) sStat[(u ^ 1) * 128 + threadIdx.x] = nxt;
    }
    if (ok && nt > 0) {
      // the last commit covers every earlier product
      const int tl = nt - 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_done[tl & 1], (tl >> 1) & 1, p.err));
      if (ok) {
        tc_fence_after();
        const bool live = kpos < p.S;
        __nv_bfloat16* dk = p.dqkv + (size_t)(row_base + kpos) * p.ld_dqkv + (p.nq + g) * HD;
        __nv_bfloat16* dv = p.dqkv + (size_t)(row_base + kpos) * p.ld_dqkv + (p.nq + p.nkv + g) * HD;
#pragma unroll 1
        for (int c = quarter * (HD / 4); c < (quarter + 1) * (HD / 4); c += 16) {
          uint32_t a[16], bq[16];
          tmem_ld16(tDV + lane_off + c, a);
          tmem_ld16(tDK + lane_off + c, bq);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {
              uint4 u1, u2;
              __nv_bfloat162* b1 = reinterpret_cast<__nv_bfloat162*>(&u1);
              __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&u2);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int e = q4 * 8 + 2 * k;
                b1[k] = __floats2bfloat162_rn(__uint_as_float(a[e]), __uint_as_float(a[e + 1]));
                b2[k] = __floats2bfloat162_rn(__uint_as_float(bq[e]) * p.scale, __uint_as_float(bq[e + 1]) * p.scale);
              }
              *reinterpret_cast<uint4*>(dv + c + q4 * 8) = u1;
              *reinterpret_cast<uint4*>(dk + c + q4 * 8) = u2;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 17) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static TmaEncoder g_benc;

template <typename Kern>
static int set_smem(Kern kern, int bytes, bool* attr) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -3;
    attr[dev & 63] = true;
  }
  return 0;
}

template <int HD>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& td, const BwdParams& p, cudaStream_t st) {
  static bool a1[64] = {}, a2[64] = {};
  if (set_smem(attn_dq_kernel<HD>, DqCfg<HD>::SMEM, a1) || set_smem(attn_dkv_kernel<HD>, DkvCfg<HD>::SMEM, a2))
    return -3;
  dim3 g1((p.S + 255) / 256, p.nq, p.B);
  attn_dq_kernel<HD><<<g1, DQ_THREADS, DqCfg<HD>::SMEM, st>>>(tq, td, p);
  if (cudaGetLastError() != cudaSuccess) return -4;
  dim3 g2((p.S + 127) / 128, p.nkv, p.B);
  attn_dkv_kernel<HD><<<g2, DKV_THREADS, DkvCfg<HD>::SMEM, st>>>(tq, td, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace attn
}  // namespace sga

// dctx, ctx: [B*S, ld_ctx] bf16; qkv, dqkv: [B*S, ld_qkv] bf16; lse, delta: [B, nq, S] fp32 (delta is scratch).
SGA_API int sga_attn_bwd(const void* dctx, const void* qkv, const void* ctx, const float* lse, float* delta,
                         void* dqkv, int B, int S, int nq, int nkv, int hd, long long ld_qkv, long long ld_ctx,
                         float scale, int* err, void* stream) {
  using namespace sga;
  using namespace sga::attn;
  if (B <= 0 || S <= 0) return 0;
  if ((hd != 64 && hd != 128) || nq % nkv || (ld_qkv & 7) || (ld_ctx & 7)) return -5;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(dctx) & 15) ||
      (reinterpret_cast<uintptr_t>(dqkv) & 15))
    return -5;
  if (g_benc.ensure()) return -1;
  CUtensorMap tq, td;
  int rc = g_benc.make(&tq, qkv, (uint64_t)(nq + 2 * nkv) * hd, (uint64_t)B * S, (uint64_t)ld_qkv, 64, 64);
  if (rc) return rc;
  rc = g_benc.make(&td, dctx, (uint64_t)nq * hd, (uint64_t)B * S, (uint64_t)ld_ctx, 64, 64);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * S * nq;
  attn_delta_kernel<<<(unsigned)((rows * (hd / 8) + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(dctx), reinterpret_cast<const __nv_bfloat16*>(ctx), delta, B, S, nq, hd,
      ld_ctx, ld_ctx);
  if (cudaGetLastError() != cudaSuccess) return -4;
  BwdParams p;
  p.B = B; p.S = S; p.nq = nq; p.nkv = nkv; p.hd = hd;
  p.ld_dqkv = (int)ld_qkv;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse;
  p.delta = delta;
  p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  p.err = err;
  p.warp_arrive = attn_warp_arrive();
  return hd == 64 ? launch_bwd<64>(tq, td, p, st) : launch_bwd<128>(tq, td, p, st);
}
