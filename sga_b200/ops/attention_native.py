"""Host side of the tcgen05 attention kernels (``csrc/attention.cu``,
``csrc/attention_bwd.cu``): head dimension 64 or 128, causal, grouped-query,
reading Q, K and V in place from the fused QKV activation.

The backward runs three launches (row dot products, the dQ kernel, the dK/dV
kernel) with a fixed order of summation: the same inputs give the same
gradient bits on every run and every rank.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..csrc import lib
from ..kernels import _chk, _st


def attn_fwd(qkv, B, S, nq, nkv, hd, scale):
    T = B * S
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[0] == T
    ctx = torch.empty(T, nq * hd, dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty(B, nq, S, dtype=torch.float32, device=qkv.device)
    _chk(lib().sga_attn_fwd(qkv.data_ptr(), ctx.data_ptr(), lse.data_ptr(), B, S, nq, nkv, hd, qkv.stride(0),
                            ctx.stride(0), float(scale), K.gemm_err_word(qkv.device).data_ptr(), _st()),
         "sga_attn_fwd")
    return ctx, ("native", ctx, lse, scale)


def attn_bwd(dctx, qkv, saved, B, S, nq, nkv, hd, dqkv):
    _, ctx, lse, scale = saved
    assert dctx.dtype == torch.bfloat16 and dctx.stride(1) == 1 and dctx.stride(0) == ctx.stride(0)
    assert dqkv.stride(0) == qkv.stride(0)
    delta = torch.empty_like(lse)
    _chk(lib().sga_attn_bwd(dctx.data_ptr(), qkv.data_ptr(), ctx.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                            dqkv.data_ptr(), B, S, nq, nkv, hd, qkv.stride(0), ctx.stride(0), float(scale),
                            K.gemm_err_word(qkv.device).data_ptr(), _st()), "sga_attn_bwd")
    K._LAUNCHES[0] += 2  # delta, dQ and dK/dV kernels behind one launcher call
    return dqkv
