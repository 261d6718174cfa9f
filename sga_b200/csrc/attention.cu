// Causal grouped-query attention on the fused QKV activation, tcgen05 + TMEM.
//
// qkv is [T, (nq + 2 nkv) * hd] bf16 with T = B * S tokens: the heads of Q, K
// and V are column ranges of one matrix, so a single 2-D tensor map (64 x 64
// boxes, 128-byte swizzle) feeds every tile and nothing is transposed or
// copied on the way in. hd is 64 or 128.
//
// Forward (sga_attn_fwd): one CTA per (256 query rows, head, batch). Two
// softmax warpgroups own 128 query rows each; one warp issues TMA loads, one
// warp issues every MMA:
//   S_w = Q_w K_j^T        (128 x BN, fp32 in TMEM)
//   P_w = exp2(S_w - m)    (threads: one row each, TMEM -> registers -> bf16 in shared memory)
//   O_w = P_w V_j          (128 x hd, fp32 in TMEM, read out and folded into registers)
// While warpgroup 0 works on its scores the tensor core runs warpgroup 1's
// products and the other way round. K/V blocks go through a three-stage ring.
// The kernel writes the normalised context and the row log-sum-exp.
//
// Stands where the reference's external stack calls flash-attn
// (examples/llama3/train_1b_adamw.yaml:107).
#include "attention.cuh"
#include <stdlib.h>

namespace sga {
namespace attn {

constexpr int F_THREADS = 320;   // 2 softmax warpgroups + TMA warp + MMA warp
constexpr int FS_THREADS = 576;  // split rows: 16 softmax warps + TMA warp + MMA warp
constexpr int F_STAGES = 3;
constexpr int F_STAGE_BYTES = 32768;  // K block + V block
constexpr int F_TMEM_COLS = 512;

struct FwdParams {
  int B, S, nq, nkv, hd;
  int ldo;            // row pitch of ctx in elements
  float scale_log2;   // softmax scale * log2(e)
  __nv_bfloat16* ctx; // [T, nq * hd]
  float* lse;         // [B, nq, S], natural log
  int* err;
  int warp_arrive;    // 1: one lane per warp signals "tile written" after a warp barrier; 0: every thread does
};

template <int HD>
struct FwdCfg {
  static constexpr int BN = HD == 64 ? 128 : 64;          // keys per block
  static constexpr int Q_BYTES = 2 * 128 * HD * 2;        // both query sub-blocks
  static constexpr int P_BYTES = 128 * BN * 2;            // one warpgroup's probabilities
  static constexpr int SMEM = Q_BYTES + F_STAGES * F_STAGE_BYTES + 2 * P_BYTES + 1024 + 256;
  static constexpr int SMEM_SPLIT = SMEM + 6144;  // + the halves' row maxima (4 KB) and row sums (2 KB)
};

template <int HD>
__global__ void __launch_bounds__(F_THREADS, 1) attn_fwd_kernel(const __grid_constant__ CUtensorMap tm,
                                                                const FwdParams p) {
  using C = FwdCfg<HD>;
  constexpr int BN = C::BN;
  constexpr int CH = HD == 64 ? 2 : 1;  // 32-column TMEM loads per wait (register budget)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                  // [2][HD/64][128][128 B]
  uint8_t* sKV = sQ + C::Q_BYTES;                      // [stage]{K [HD/64][BN][128 B], V the same}
  uint8_t* sP = sKV + F_STAGES * F_STAGE_BYTES;        // [2][BN/64][128][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * C::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + F_STAGES;
  uint64_t* s_full = kv_empty + F_STAGES;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavier (later) query blocks first
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
    for (int s = 0; s < F_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&s_full[w], 1);
      mbar_init(&p_full[w], 128);
      mbar_init(&o_full[w], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, F_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO[2] = {tmem_base + 256, tmem_base + 384};
  const int row_base = b * p.S;

  if (warp == 8) {
    if (lane == 0 && n_all > 0) {
      mbar_expect_tx(q_full, C::Q_BYTES);
      for (int w = 0; w < 2; ++w)
        load_tile(sQ + w * (128 * HD * 2), &tm, q_full, h * HD, row_base + q0 + 128 * w, 128, HD);
      for (int j = 0; j < n_all; ++j) {
        const int st = j % F_STAGES;
        if (!mbar_wait(&kv_empty[st], ((j / F_STAGES) & 1) ^ 1, p.err)) break;
        uint8_t* sk = sKV + st * F_STAGE_BYTES;
        mbar_expect_tx(&kv_full[st], F_STAGE_BYTES);
        load_tile(sk, &tm, &kv_full[st], (p.nq + g) * HD, row_base + j * BN, BN, HD);
        load_tile(sk + BN * HD * 2, &tm, &kv_full[st], (p.nq + p.nkv + g) * HD, row_base + j * BN, BN, HD);
      }
      if (sga_aborted(p.err)) __nanosleep(200000);
    }
  } else if (warp == 9) {
    if (lane == 0 && n_all > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BN, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
      const uint64_t dQ0 = desc_k(smem_u32(sQ)), dP0 = desc_k(smem_u32(sP));
      const uint64_t dK0 = desc_k(smem_u32(sKV)), dV0 = desc_mn(smem_u32(sKV + BN * HD * 2), BN);
      constexpr uint64_t Q_STEP = (128 * HD * 2) >> 4, P_STEP = C::P_BYTES >> 4, KV_STEP = F_STAGE_BYTES >> 4;
      bool ok = mbar_wait(q_full, 0, p.err) && mbar_wait(&kv_full[0], 0, p.err);
      if (ok) {
        tc_fence_after();
        for (int w = 0; w < 2; ++w)
          if (nw[w] > 0) {
            mma_over_hd<HD, 128, BN>(tS[w], dQ0 + w * Q_STEP, dK0, idesc_s);
            umma_commit(&s_full[w]);
          }
      }
      int st = 0;
      for (int j = 0; j < n_all && ok; ++j) {
        const int sn = st + 1 == F_STAGES ? 0 : st + 1;
        bool next_ready = false;
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= nw[w]) continue;
          ok = mbar_wait(&p_full[w], j & 1, p.err);
          if (!ok) break;
          tc_fence_after();
          mma_over_rows<BN>(tO[w], dP0 + w * P_STEP, dV0 + st * KV_STEP, idesc_o, false);
          umma_commit(&o_full[w]);
          if (j + 1 < nw[w]) {
            if (!next_ready) {
              ok = mbar_wait(&kv_full[sn], ((j + 1) / F_STAGES) & 1, p.err);
              if (!ok) break;
              tc_fence_after();
              next_ready = true;
            }
            mma_over_hd<HD, 128, BN>(tS[w], dQ0 + w * Q_STEP, dK0 + sn * KV_STEP, idesc_s);
            umma_commit(&s_full[w]);
          }
        }
        if (ok) umma_commit(&kv_empty[st]);
        st = sn;
      }
    }
  } else {
    const int w = warp >> 2;
    const int r = (warp & 3) * 32 + lane;       // row within the warpgroup's 128
    const int qrow = q0 + 128 * w + r;          // position in the sequence
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint8_t* myP = sP + w * C::P_BYTES;
    float m = -INFINITY, l = 0.f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < nw[w] && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[w], j & 1, p.err));
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * BN;
      const bool diag = kv0 + BN - 1 > q0 + 128 * w;  // some key of the block lies past some row of the sub-block
      // pass 1: row maximum of the raw scores (four independent chains)
      float mx4[4] = {m, m, m, m};
#pragma unroll 1
      for (int c = 0; c < BN; c += 32 * CH) {
        uint32_t v[32 * CH];
#pragma unroll
        for (int u = 0; u < CH; ++u) tmem_ld32(tS[w] + lane_off + c + 32 * u, *reinterpret_cast<uint32_t(*)[32]>(&v[32 * u]));
        tmem_ld_wait();
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32 * CH; ++i)
            if (kv0 + c + i <= qrow) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32 * CH; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float alpha = exp2f((m - mx) * p.scale_log2);  // m = -inf on the first block: 0
      // fold the previous block's P V into the running output, then move it to the new maximum
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&o_full[w], (j - 1) & 1, p.err));
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD; c += 32 * CH) {
          uint32_t v[32 * CH];
#pragma unroll
          for (int u = 0; u < CH; ++u) tmem_ld32(tO[w] + lane_off + c + 32 * u, *reinterpret_cast<uint32_t(*)[32]>(&v[32 * u]));
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32 * CH; ++i) o[c + i] = (o[c + i] + __uint_as_float(v[i])) * alpha;
        }
      }
      l *= alpha;
      m = mx;
      // pass 2: probabilities -> bf16 operand tile, row sum
      const float neg = -mx * p.scale_log2;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld32(tS[w] + lane_off + c, v);
        tmem_ld_wait();
        float pr[32];
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float e = kv0 + c + i <= qrow ? exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, neg)) : 0.f;
            pr[i] = e;
            l4[i & 3] += e;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float e = exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, neg));
            pr[i] = e;
            l4[i & 3] += e;
          }
        }
        store_p32(myP, r, c, pr);
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&p_full[w]);
    }
    if (ok && nw[w] > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[w], (nw[w] - 1) & 1, p.err));
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / l;
        const bool live = qrow < p.S;
        __nv_bfloat16* dst = p.ctx + (size_t)(row_base + qrow) * p.ldo + h * HD;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld32(tO[w] + lane_off + c, v);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              __nv_bfloat162* ub = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int e = q4 * 8 + 2 * i;
                ub[i] = __floats2bfloat162_rn((o[c + e] + __uint_as_float(v[e])) * inv,
                                              (o[c + e + 1] + __uint_as_float(v[e + 1])) * inv);
              }
              *reinterpret_cast<uint4*>(dst + c + q4 * 8) = u;
            }
          }
        }
        if (live) p.lse[((size_t)b * p.nq + h) * p.S + qrow] = (m * p.scale_log2 + log2f(l)) * 0.6931471805599453f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, F_TMEM_COLS);
  }
}

// The forward with the output accumulated in TMEM: P V of every block adds into the same accumulator, the
// softmax threads read a block's scores once (row maximum, probabilities and row sum from registers) and
// rescale the accumulator in TMEM only when the row maximum has moved by more than 2^8 since the last
// rescale, so the probabilities stay within bf16's range while the common block does no correction work.
template <int HD>
__global__ void __launch_bounds__(F_THREADS, 1) attn_fwd_acc_kernel(const __grid_constant__ CUtensorMap tm,
                                                                const FwdParams p) {
  using C = FwdCfg<HD>;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                  // [2][HD/64][128][128 B]
  uint8_t* sKV = sQ + C::Q_BYTES;                      // [stage]{K [HD/64][BN][128 B], V the same}
  uint8_t* sP = sKV + F_STAGES * F_STAGE_BYTES;        // [2][BN/64][128][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * C::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + F_STAGES;
  uint64_t* s_full = kv_empty + F_STAGES;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavier (later) query blocks first
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
    for (int s = 0; s < F_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&s_full[w], 1);
      mbar_init(&p_full[w], p.warp_arrive ? 4 : 128);
      mbar_init(&o_full[w], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, F_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO[2] = {tmem_base + 256, tmem_base + 384};
  const int row_base = b * p.S;

  if (warp == 8) {
    if (lane == 0 && n_all > 0) {
      mbar_expect_tx(q_full, C::Q_BYTES);
      for (int w = 0; w < 2; ++w)
        load_tile(sQ + w * (128 * HD * 2), &tm, q_full, h * HD, row_base + q0 + 128 * w, 128, HD);
      for (int j = 0; j < n_all; ++j) {
        const int st = j % F_STAGES;
        if (!mbar_wait(&kv_empty[st], ((j / F_STAGES) & 1) ^ 1, p.err)) break;
        uint8_t* sk = sKV + st * F_STAGE_BYTES;
        mbar_expect_tx(&kv_full[st], F_STAGE_BYTES);
        load_tile(sk, &tm, &kv_full[st], (p.nq + g) * HD, row_base + j * BN, BN, HD);
        load_tile(sk + BN * HD * 2, &tm, &kv_full[st], (p.nq + p.nkv + g) * HD, row_base + j * BN, BN, HD);
      }
      if (sga_aborted(p.err)) __nanosleep(200000);
    }
  } else if (warp == 9) {
    if (lane == 0 && n_all > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BN, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
      const uint64_t dQ0 = desc_k(smem_u32(sQ)), dP0 = desc_k(smem_u32(sP));
      const uint64_t dK0 = desc_k(smem_u32(sKV)), dV0 = desc_mn(smem_u32(sKV + BN * HD * 2), BN);
      constexpr uint64_t Q_STEP = (128 * HD * 2) >> 4, P_STEP = C::P_BYTES >> 4, KV_STEP = F_STAGE_BYTES >> 4;
      bool ok = mbar_wait(q_full, 0, p.err) && mbar_wait(&kv_full[0], 0, p.err);
      if (ok) {
        tc_fence_after();
        for (int w = 0; w < 2; ++w)
          if (nw[w] > 0) {
            mma_over_hd<HD, 128, BN>(tS[w], dQ0 + w * Q_STEP, dK0, idesc_s);
            umma_commit(&s_full[w]);
          }
      }
      int st = 0;
      for (int j = 0; j < n_all && ok; ++j) {
        const int sn = st + 1 == F_STAGES ? 0 : st + 1;
        bool next_ready = false;
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= nw[w]) continue;
          ok = mbar_wait(&p_full[w], j & 1, p.err);
          if (!ok) break;
          tc_fence_after();
          mma_over_rows<BN>(tO[w], dP0 + w * P_STEP, dV0 + st * KV_STEP, idesc_o, j > 0);
          umma_commit(&o_full[w]);
          if (j + 1 < nw[w]) {
            if (!next_ready) {
              ok = mbar_wait(&kv_full[sn], ((j + 1) / F_STAGES) & 1, p.err);
              if (!ok) break;
              tc_fence_after();
              next_ready = true;
            }
            mma_over_hd<HD, 128, BN>(tS[w], dQ0 + w * Q_STEP, dK0 + sn * KV_STEP, idesc_s);
            umma_commit(&s_full[w]);
          }
        }
        if (ok) umma_commit(&kv_empty[st]);
        st = sn;
      }
    }
  } else {
    const int w = warp >> 2;
    const int r = (warp & 3) * 32 + lane;       // row within the warpgroup's 128
    const int qrow = q0 + 128 * w + r;          // position in the sequence
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint8_t* myP = sP + w * C::P_BYTES;
    // m: the maximum the probabilities and the accumulator are currently expressed against. It follows the
    // running row maximum lazily: only when a block's maximum exceeds it by more than 2^8 in the exponent
    // is the accumulator in TMEM rescaled, so in the steady state a block costs one read of its scores.
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nw[w] && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[w], j & 1, p.err));
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * BN;
      const bool diag = kv0 + BN - 1 > q0 + 128 * w;  // some key of the block lies past some row of the sub-block
      uint32_t sv[BN];
#pragma unroll
      for (int c = 0; c < BN; c += 32) tmem_ld32(tS[w] + lane_off + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
      tmem_ld_wait();
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (diag) {
#pragma unroll
        for (int i = 0; i < BN; ++i)
          if (kv0 + i <= qrow) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
      } else {
#pragma unroll
        for (int i = 0; i < BN; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // first block: m = -inf, the difference is +inf. A row without a visible key in this block: mx = -inf, false.
      const bool move = (mx - m) * p.scale_log2 > 8.f;
      float alpha = 1.f;
      if (move) {
        alpha = exp2f((m - mx) * p.scale_log2);  // 0 on the first block
        m = mx;
        l *= alpha;
      }
      const bool rescale = j > 0 && __any_sync(0xffffffffu, move);
      const float neg = -m * p.scale_log2;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[BN / 2];
      if (diag) {
#pragma unroll
        for (int i = 0; i < BN; i += 2) {
          const float e0 = kv0 + i <= qrow ? exp2f(fmaf(__uint_as_float(sv[i]), p.scale_log2, neg)) : 0.f;
          const float e1 = kv0 + i + 1 <= qrow ? exp2f(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, neg)) : 0.f;
          l4[i & 3] += e0;
          l4[(i + 1) & 3] += e1;
          const __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
          pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&b);
        }
      } else {
#pragma unroll
        for (int i = 0; i < BN; i += 2) {
          const float e0 = exp2f(fmaf(__uint_as_float(sv[i]), p.scale_log2, neg));
          const float e1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, neg));
          l4[i & 3] += e0;
          l4[(i + 1) & 3] += e1;
          const __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
          pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&b);
        }
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      // The previous block's P V has to be finished before its P tile is overwritten (and before the
      // accumulator is touched). The tensor core ran it ahead of this block's scores, so this wait is short.
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&o_full[w], (j - 1) & 1, p.err));
        if (!ok) break;
        tc_fence_after();
        if (rescale) {
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            uint32_t v[32];
            tmem_ld32(tO[w] + lane_off + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st32(tO[w] + lane_off + c, v);
          }
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int c = 0; c < BN; c += 32) store_pk32(myP, r, c, *reinterpret_cast<const uint32_t(*)[16]>(&pk[c >> 1]));
      tc_fence_before();
      fence_proxy_async_smem();
      if (p.warp_arrive) {
        // every writer has fenced its own stores; the warp barrier orders them before the one arrival
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[w]);
      } else {
        mbar_arrive(&p_full[w]);
      }
    }
    if (ok && nw[w] > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[w], (nw[w] - 1) & 1, p.err));
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / l;
        const bool live = qrow < p.S;
        __nv_bfloat16* dst = p.ctx + (size_t)(row_base + qrow) * p.ldo + h * HD;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t v[32];
          tmem_ld32(tO[w] + lane_off + c, v);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              __nv_bfloat162* ub = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int e = q4 * 8 + 2 * i;
                ub[i] = __floats2bfloat162_rn(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
              }
              *reinterpret_cast<uint4*>(dst + c + q4 * 8) = u;
            }
          }
        }
        if (live) p.lse[((size_t)b * p.nq + h) * p.S + qrow] = (m * p.scale_log2 + log2f(l)) * 0.6931471805599453f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, F_TMEM_COLS);
  }
}

// The same forward with a query row split over two threads (sixteen softmax warps, four per scheduler): each
// thread walks half of a block's scores and half of the output columns, so the chain per block is half as long
// and twice as many warps are there to hide it.
template <int HD>
__global__ void __launch_bounds__(FS_THREADS, 1) attn_fwd_split_kernel(const __grid_constant__ CUtensorMap tm,
                                                                const FwdParams p) {
  using C = FwdCfg<HD>;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                  // [2][HD/64][128][128 B]
  uint8_t* sKV = sQ + C::Q_BYTES;                      // [stage]{K [HD/64][BN][128 B], V the same}
  uint8_t* sP = sKV + F_STAGES * F_STAGE_BYTES;        // [2][BN/64][128][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * C::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + F_STAGES;
  uint64_t* s_full = kv_empty + F_STAGES;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
  float* xch = reinterpret_cast<float*>(bars) + 64;   // [parity][warpgroup][half][128] row maxima, then [warpgroup][half][128] row sums

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavier (later) query blocks first
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
    for (int s = 0; s < F_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&s_full[w], 1);
      mbar_init(&p_full[w], p.warp_arrive ? 8 : 256);
      mbar_init(&o_full[w], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm);
  }
  if (warp == 17) {
    tmem_alloc(tmem_slot, F_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO[2] = {tmem_base + 256, tmem_base + 384};
  const int row_base = b * p.S;

  if (warp == 16) {
    if (lane == 0 && n_all > 0) {
      mbar_expect_tx(q_full, C::Q_BYTES);
      for (int w = 0; w < 2; ++w)
        load_tile(sQ + w * (128 * HD * 2), &tm, q_full, h * HD, row_base + q0 + 128 * w, 128, HD);
      for (int j = 0; j < n_all; ++j) {
        const int st = j % F_STAGES;
        if (!mbar_wait(&kv_empty[st], ((j / F_STAGES) & 1) ^ 1, p.err)) break;
        uint8_t* sk = sKV + st * F_STAGE_BYTES;
        mbar_expect_tx(&kv_full[st], F_STAGE_BYTES);
        load_tile(sk, &tm, &kv_full[st], (p.nq + g) * HD, row_base + j * BN, BN, HD);
        load_tile(sk + BN * HD * 2, &tm, &kv_full[st], (p.nq + p.nkv + g) * HD, row_base + j * BN, BN, HD);
      }
      if (sga_aborted(p.err)) __nanosleep(200000);
    }
  } else if (warp == 17) {
    if (lane == 0 && n_all > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BN, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
      const uint64_t dQ0 = desc_k(smem_u32(sQ)), dP0 = desc_k(smem_u32(sP));
      const uint64_t dK0 = desc_k(smem_u32(sKV)), dV0 = desc_mn(smem_u32(sKV + BN * HD * 2), BN);
      constexpr uint64_t Q_STEP = (128 * HD * 2) >> 4, P_STEP = C::P_BYTES >> 4, KV_STEP = F_STAGE_BYTES >> 4;
      bool ok = mbar_wait(q_full, 0, p.err) && mbar_wait(&kv_full[0], 0, p.err);
      if (ok) {
        tc_fence_after();
        for (int w = 0; w < 2; ++w)
          if (nw[w] > 0) {
            mma_over_hd<HD, 128, BN>(tS[w], dQ0 + w * Q_STEP, dK0, idesc_s);
            umma_commit(&s_full[w]);
          }
      }
      int st = 0;
      for (int j = 0; j < n_all && ok; ++j) {
        const int sn = st + 1 == F_STAGES ? 0 : st + 1;
        bool next_ready = false;
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= nw[w]) continue;
          ok = mbar_wait(&p_full[w], j & 1, p.err);
          if (!ok) break;
          tc_fence_after();
          mma_over_rows<BN>(tO[w], dP0 + w * P_STEP, dV0 + st * KV_STEP, idesc_o, j > 0);
          umma_commit(&o_full[w]);
          if (j + 1 < nw[w]) {
            if (!next_ready) {
              ok = mbar_wait(&kv_full[sn], ((j + 1) / F_STAGES) & 1, p.err);
              if (!ok) break;
              tc_fence_after();
              next_ready = true;
            }
            mma_over_hd<HD, 128, BN>(tS[w], dQ0 + w * Q_STEP, dK0 + sn * KV_STEP, idesc_s);
            umma_commit(&s_full[w]);
          }
        }
        if (ok) umma_commit(&kv_empty[st]);
        st = sn;
      }
    }
  } else {
    // Sixteen softmax warps: a query row belongs to two threads, each covering half of a block's keys
    // (warps 0-3 and 4-7 of a warpgroup see the same TMEM lanes). They exchange the halves' maxima through
    // shared memory once per block and the halves' row sums once at the end. Every warp meets the same
    // number of named barriers whatever its waits returned.
    constexpr int NC = BN / 2;                  // score columns per thread
    constexpr int OC = HD / 2;                  // output columns per thread
    const int w = warp >> 3;
    const int half = (warp >> 2) & 1;
    const int r = (warp & 3) * 32 + lane;       // row within the warpgroup's 128
    const int qrow = q0 + 128 * w + r;          // position in the sequence
    const int c0 = half * NC;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint8_t* myP = sP + w * C::P_BYTES;
    float* xmax = xch;                          // [2][2][2][128]
    float* xsum = xch + 1024;                   // [2][2][128]
    float m = -INFINITY, l = 0.f;               // l: this thread's half of the row sum
    bool ok = true;
    for (int j = 0; j < nw[w]; ++j) {
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&s_full[w], j & 1, p.err));
      const int kv0 = j * BN + c0;              // first key of this thread's half
      const bool diag = j * BN + BN - 1 > q0 + 128 * w;
      // Scores are walked 32 columns at a time; a thread with 64 of them (head dim 64) reads them from TMEM a
      // second time for the probabilities instead of holding all of them across the exchange of the maxima.
      constexpr bool REREAD = NC > 32;
      uint32_t sv[32];
      float mx = -INFINITY;
      if (ok) {
        tc_fence_after();
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < NC; c += 32) {
          tmem_ld32(tS[w] + lane_off + c0 + c, sv);
          tmem_ld_wait();
          if (diag) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kv0 + c + i <= qrow) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
          }
        }
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      float* slot = xmax + (((j & 1) * 2 + w) * 2) * 128;
      slot[half * 128 + r] = mx;
      asm volatile("bar.sync %0, 256;" ::"r"(1 + w) : "memory");
      mx = fmaxf(mx, slot[(half ^ 1) * 128 + r]);
      if (!ok) continue;
      // both threads of a row now hold the same block maximum and the same m: they take the same decision
      const bool move = (mx - m) * p.scale_log2 > 8.f;
      float alpha = 1.f;
      if (move) {
        alpha = exp2f((m - mx) * p.scale_log2);  // 0 on the first block
        m = mx;
        l *= alpha;
      }
      const bool rescale = j > 0 && __any_sync(0xffffffffu, move);
      const float neg = -m * p.scale_log2;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[NC / 2];
#pragma unroll
      for (int c = 0; c < NC; c += 32) {
        if (REREAD) {   // with one chunk its values are still in sv
          tmem_ld32(tS[w] + lane_off + c0 + c, sv);
          tmem_ld_wait();
        }
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = kv0 + c + i <= qrow ? exp2f(fmaf(__uint_as_float(sv[i]), p.scale_log2, neg)) : 0.f;
            const float e1 = kv0 + c + i + 1 <= qrow ? exp2f(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, neg)) : 0.f;
            l4[i & 3] += e0;
            l4[(i + 1) & 3] += e1;
            const __nv_bfloat162 bb = __floats2bfloat162_rn(e0, e1);
            pk[(c + i) >> 1] = *reinterpret_cast<const uint32_t*>(&bb);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = exp2f(fmaf(__uint_as_float(sv[i]), p.scale_log2, neg));
            const float e1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, neg));
            l4[i & 3] += e0;
            l4[(i + 1) & 3] += e1;
            const __nv_bfloat162 bb = __floats2bfloat162_rn(e0, e1);
            pk[(c + i) >> 1] = *reinterpret_cast<const uint32_t*>(&bb);
          }
        }
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&o_full[w], (j - 1) & 1, p.err));
        if (!ok) continue;
        tc_fence_after();
        if (rescale) {
#pragma unroll 1
          for (int c = 0; c < OC; c += 32) {
            uint32_t v[32];
            tmem_ld32(tO[w] + lane_off + half * OC + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st32(tO[w] + lane_off + half * OC + c, v);
          }
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int c = 0; c < NC; c += 32)
        store_pk32(myP, r, c0 + c, *reinterpret_cast<const uint32_t(*)[16]>(&pk[c >> 1]));
      tc_fence_before();
      fence_proxy_async_smem();
      if (p.warp_arrive) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[w]);
      } else {
        mbar_arrive(&p_full[w]);
      }
    }
    // the row sum: both threads add the halves in the same order
    xsum[(w * 2 + half) * 128 + r] = l;
    asm volatile("bar.sync %0, 256;" ::"r"(1 + w) : "memory");
    const float lt = xsum[(w * 2) * 128 + r] + xsum[(w * 2 + 1) * 128 + r];
    if (ok && nw[w] > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[w], (nw[w] - 1) & 1, p.err));
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / lt;
        const bool live = qrow < p.S;
        __nv_bfloat16* dst = p.ctx + (size_t)(row_base + qrow) * p.ldo + h * HD + half * OC;
#pragma unroll
        for (int c = 0; c < OC; c += 32) {
          uint32_t v[32];
          tmem_ld32(tO[w] + lane_off + half * OC + c, v);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              __nv_bfloat162* ub = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int e = q4 * 8 + 2 * i;
                ub[i] = __floats2bfloat162_rn(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
              }
              *reinterpret_cast<uint4*>(dst + c + q4 * 8) = u;
            }
          }
        }
        if (live && half == 0)
          p.lse[((size_t)b * p.nq + h) * p.S + qrow] = (m * p.scale_log2 + log2f(lt)) * 0.6931471805599453f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 17) {
    tc_fence_after();
    tmem_dealloc(tmem_base, F_TMEM_COLS);
  }
}

static TmaEncoder g_enc;

// The forward kernel. By default the measured faster form per head dimension: at 64 the row split over two
// threads (key blocks of 128: the per-thread walk is the limiter), at 128 the one-thread-per-row kernel with
// the TMEM accumulator (key blocks of 64). SGA_ATTN_FWD = accumulate | split | fold forces one form
// ("fold": output folded into registers after every block).
static int fwd_mode(int hd) {
  static const int forced = [] {
    const char* e = getenv("SGA_ATTN_FWD");
    if (e && e[0] == 'f') return 0;
    if (e && e[0] == 'a') return 1;
    if (e && e[0] == 's') return 2;
    return -1;
  }();
  if (forced >= 0) return forced;
  return hd == 64 ? 2 : 1;
}

template <int HD>
static int launch_fwd(const CUtensorMap& tm, const FwdParams& p, cudaStream_t st) {
  const int mode = fwd_mode(HD);
  auto kern = mode == 2 ? attn_fwd_split_kernel<HD> : (mode == 1 ? attn_fwd_acc_kernel<HD> : attn_fwd_kernel<HD>);
  const int smem = mode == 2 ? FwdCfg<HD>::SMEM_SPLIT : FwdCfg<HD>::SMEM;
  static bool attr[3][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr[mode][dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
    attr[mode][dev & 63] = true;
  }
  dim3 grid((p.S + 255) / 256, p.nq, p.B);
  kern<<<grid, mode == 2 ? FS_THREADS : F_THREADS, smem, st>>>(tm, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace attn
}  // namespace sga

// qkv: [B*S, ld_qkv] bf16 (ld_qkv >= (nq + 2 nkv) * hd); ctx: [B*S, ld_ctx] bf16; lse: [B, nq, S] fp32.
SGA_API int sga_attn_fwd(const void* qkv, void* ctx, float* lse, int B, int S, int nq, int nkv, int hd,
                         long long ld_qkv, long long ld_ctx, float scale, int* err, void* stream) {
  using namespace sga;
  using namespace sga::attn;
  if (B <= 0 || S <= 0) return 0;
  if ((hd != 64 && hd != 128) || nq % nkv || (ld_qkv & 7) || (ld_ctx & 7)) return -5;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(ctx) & 15)) return -5;
  if (g_enc.ensure()) return -1;
  CUtensorMap tm;
  int rc = g_enc.make(&tm, qkv, (uint64_t)(nq + 2 * nkv) * hd, (uint64_t)B * S, (uint64_t)ld_qkv, 64, 64);
  if (rc) return rc;
  FwdParams p;
  p.B = B; p.S = S; p.nq = nq; p.nkv = nkv; p.hd = hd;
  p.ldo = (int)ld_ctx;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.ctx = reinterpret_cast<__nv_bfloat16*>(ctx);
  p.lse = lse;
  p.err = err;
  p.warp_arrive = attn_warp_arrive();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return hd == 64 ? launch_fwd<64>(tm, p, st) : launch_fwd<128>(tm, p, st);
}
