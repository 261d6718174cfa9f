"""Causal grouped-query attention, forward and backward, on the fused QKV
activation.

``qkv`` is the ``[T, (nq + 2 nkv) * hd]`` output of the QKV projection with
``T = B * S`` tokens; queries, keys and values are column ranges of it, so
nothing is copied or transposed on the way in. ``attn_fwd`` returns the
``[T, nq * hd]`` context and what the backward needs; ``attn_bwd`` writes
``d(qkv)`` into one ``[T, (nq + 2 nkv) * hd]`` buffer.

Two implementations sit behind the same two functions:

* ``native``: the hand-written sm_100a kernels of ``csrc/attention.cu``
  (tcgen05 QK^T and PV with TMEM accumulators);
* ``library``: PyTorch's fused SDPA kernels, kept as the numerical oracle and
  as the CPU path.

The reference gets attention from flash-attn through its external Megatron
stack (``examples/llama3/train_1b_adamw.yaml:107`` ``use_flash_attn``).
"""
from __future__ import annotations

import math
import os

import torch

_IMPL = os.environ.get("SGA_ATTENTION", "auto")  # auto | native | library


def _split(qkv, B, S, nq, nkv, hd):
    x = qkv.view(B, S, nq + 2 * nkv, hd)
    q = x[:, :, :nq].transpose(1, 2)
    k = x[:, :, nq:nq + nkv].transpose(1, 2)
    v = x[:, :, nq + nkv:].transpose(1, 2)
    return q, k, v


def native_available(qkv, hd: int = 64) -> bool:
    if not qkv.is_cuda or _IMPL == "library" or hd not in (64, 128) or qkv.dtype != torch.bfloat16:
        return False
    try:
        from ..csrc import lib

        return hasattr(lib(), "sga_attn_fwd")
    except Exception:
        return False


def _whole_sequences_only(cp_group) -> None:
    """``cp_group`` is the extension point for context parallelism (sequence shards exchanging key /
    value blocks around a ring): the entry points take it so that callers can already thread a group
    through, but every sequence must live whole on one rank for now."""
    if cp_group is None:
        return
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(cp_group) > 1:
        raise NotImplementedError("context-parallel attention (cp_group with more than one rank) is not built: "
                                  "the attention kernels take whole sequences")


def attn_fwd(qkv, B, S, nq, nkv, hd, cp_group=None):
    """Returns ``(ctx [T, nq*hd] bf16, saved)``."""
    _whole_sequences_only(cp_group)
    scale = 1.0 / math.sqrt(hd)
    if native_available(qkv, hd):
        from . import attention_native as AN

        return AN.attn_fwd(qkv, B, S, nq, nkv, hd, scale)
    if _IMPL == "native":
        raise RuntimeError("SGA_ATTENTION=native but the native attention kernel is not built")
    q, k, v = _split(qkv, B, S, nq, nkv, hd)
    if qkv.is_cuda:
        res = torch.ops.aten._scaled_dot_product_flash_attention(q, k, v, 0.0, True, False, scale=scale)
        out, lse, cq, ck, mq, mk, seed, offs = res[:8]
        ctx = out.transpose(1, 2).reshape(B * S, nq * hd)
        return ctx, ("lib", out, lse, cq, ck, mq, mk, seed, offs, scale)
    rep = nq // nkv
    kk = k.repeat_interleave(rep, 1).float()
    vv = v.repeat_interleave(rep, 1).float()
    qf = q.float()
    att = (qf @ kk.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool).tril()
    att = att.masked_fill(~mask, float("-inf"))
    p = torch.softmax(att, -1)
    out = (p @ vv)
    ctx = out.transpose(1, 2).reshape(B * S, nq * hd).to(qkv.dtype)
    return ctx, ("cpu", p, scale)


def attn_bwd(dctx, qkv, saved, B, S, nq, nkv, hd, dqkv=None, cp_group=None):
    """``dctx``: ``[T, nq*hd]``. Returns ``dqkv`` ``[T, (nq+2nkv)*hd]`` bf16."""
    _whole_sequences_only(cp_group)
    if dqkv is None:
        dqkv = torch.empty_like(qkv)
    kind = saved[0]
    if kind == "native":
        from . import attention_native as AN

        return AN.attn_bwd(dctx, qkv, saved, B, S, nq, nkv, hd, dqkv)
    q, k, v = _split(qkv, B, S, nq, nkv, hd)
    do = dctx.view(B, S, nq, hd).transpose(1, 2)
    dq_v, dk_v, dv_v = _split(dqkv, B, S, nq, nkv, hd)
    if kind == "lib":
        _, out, lse, cq, ck, mq, mk, seed, offs, scale = saved
        dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
            do, q, k, v, out, lse, cq, ck, mq, mk, 0.0, True, seed, offs, scale=scale)
        dq_v.copy_(dq)
        dk_v.copy_(dk)
        dv_v.copy_(dv)
        return dqkv
    _, p, scale = saved
    rep = nq // nkv
    kk = k.repeat_interleave(rep, 1).float()
    vv = v.repeat_interleave(rep, 1).float()
    dof = do.float()
    dv_full = p.transpose(-1, -2) @ dof
    dp = dof @ vv.transpose(-1, -2)
    ds = p * (dp - (dp * p).sum(-1, keepdim=True))
    dq = (ds @ kk) * scale
    dk_full = (ds.transpose(-1, -2) @ q.float()) * scale
    dq_v.copy_(dq.to(dqkv.dtype))
    dk_v.copy_(dk_full.view(B, nkv, rep, S, hd).sum(2).to(dqkv.dtype))
    dv_v.copy_(dv_full.view(B, nkv, rep, S, hd).sum(2).to(dqkv.dtype))
    return dqkv
