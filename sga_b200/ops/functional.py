"""Tensor-level entry points of the bf16 model ops (``csrc/ops.cu``).

CUDA tensors run the native kernels; CPU tensors run a PyTorch fp32
restatement of the same math so that the model also steps on a CPU-only
machine (gloo tests). There is no silent fallback on a GPU: a missing native
library raises.
"""
from __future__ import annotations

import torch

from ..kernels import _chk, _p, _st
from ..csrc import lib

_scratch = {}


def _dw_scratch(device, H):
    nb = lib().sga_rmsnorm_bwd_blocks()
    key = (torch.device(device).index or 0, "dw")
    need = nb * H
    if key not in _scratch or _scratch[key].numel() < need:
        _scratch[key] = torch.empty(need, dtype=torch.float32, device=device)
    return _scratch[key]


# ---------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x, w, eps, out=None, want_rstd=True):
    """``y = x * rsqrt(mean(x^2) + eps) * w`` over the last dim of a 2-D bf16 tensor."""
    T, H = x.shape
    if not x.is_cuda:
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        y = (xf * rstd[:, None] * w.float()).to(x.dtype)
        if out is not None:
            out.copy_(y)
            y = out
        return y, rstd
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    y = out if out is not None else torch.empty_like(x)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device) if want_rstd else None
    _chk(lib().sga_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), _p(rstd), T, H, x.stride(0), y.stride(0),
                               max(T, 1), 0, 0, float(eps), _st()), "sga_rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(x, w, dy, rstd, dw_out, accumulate_dw=True, dx_out=None, accumulate_dx=False):
    """Returns dx (bf16). ``dw_out`` (fp32 ``[H]``) receives or accumulates the weight gradient."""
    T, H = x.shape
    if not x.is_cuda:
        xh = x.float() * rstd[:, None]
        g = dy.float() * w.float()
        dot = (g * xh).mean(-1, keepdim=True)
        dx = (rstd[:, None] * (g - xh * dot))
        dwv = (dy.float() * xh).sum(0)
        if accumulate_dw:
            dw_out += dwv
        else:
            dw_out.copy_(dwv)
        if dx_out is not None:
            if accumulate_dx:
                dx_out.copy_((dx_out.float() + dx).to(dx_out.dtype))
            else:
                dx_out.copy_(dx.to(dx_out.dtype))
            return dx_out
        return dx.to(x.dtype)
    dx = dx_out if dx_out is not None else torch.empty_like(x)
    _chk(lib().sga_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                               _dw_scratch(x.device, H).data_ptr(), dw_out.data_ptr(), int(accumulate_dw), T, H,
                               x.stride(0), dy.stride(0), dx.stride(0), max(T, 1), 0, 0, 0, int(accumulate_dx),
                               _st()), "sga_rmsnorm_bwd")
    return dx


def headnorm_fwd_(buf, w, eps, T, nheads, hd, col0):
    """In-place per-head RMSNorm on columns ``[col0, col0 + nheads*hd)`` of a
    ``[T, pitch]`` activation (QK-norm). Returns rstd ``[T * nheads]``."""
    pitch = buf.stride(0)
    view = buf[:, col0:col0 + nheads * hd]
    if not buf.is_cuda:
        xf = view.float().reshape(T, nheads, hd)
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        view.copy_((xf * rstd[..., None] * w.float()).reshape(T, nheads * hd).to(buf.dtype))
        return rstd.reshape(-1)
    rstd = torch.empty(T * nheads, dtype=torch.float32, device=buf.device)
    _chk(lib().sga_rmsnorm_fwd(view.data_ptr(), w.data_ptr(), view.data_ptr(), rstd.data_ptr(), T * nheads, hd, hd,
                               hd, nheads, pitch, pitch, float(eps), _st()), "sga_rmsnorm_fwd(head)")
    return rstd


def headnorm_bwd_(x_pre, dbuf, w, rstd, dw_out, T, nheads, hd, col0_x, col0_d):
    """Backward of the per-head norm: ``dbuf`` columns are overwritten by dx.
    ``x_pre`` holds the pre-norm activations (columns at ``col0_x``)."""
    xv = x_pre[:, col0_x:col0_x + nheads * hd]
    dv = dbuf[:, col0_d:col0_d + nheads * hd]
    if not dbuf.is_cuda:
        xh = xv.float().reshape(T, nheads, hd) * rstd.reshape(T, nheads, 1)
        dy = dv.float().reshape(T, nheads, hd)
        g = dy * w.float()
        dot = (g * xh).mean(-1, keepdim=True)
        dx = rstd.reshape(T, nheads, 1) * (g - xh * dot)
        dw_out += (dy * xh).sum((0, 1))
        dv.copy_(dx.reshape(T, nheads * hd).to(dbuf.dtype))
        return
    _chk(lib().sga_rmsnorm_bwd(xv.data_ptr(), w.data_ptr(), dv.data_ptr(), rstd.data_ptr(), dv.data_ptr(),
                               _dw_scratch(dbuf.device, hd).data_ptr(), dw_out.data_ptr(), 1, T * nheads, hd, hd, hd,
                               hd, nheads, x_pre.stride(0), dbuf.stride(0), dbuf.stride(0), 0, _st()),
         "sga_rmsnorm_bwd(head)")


# ------------------------------------------------------------------- RoPE
def rope_tables(S, hd, theta, device):
    half = hd // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / hd))
    ang = torch.arange(S, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def rope_(buf, cs, sn, S, nheads, hd, col0, sign):
    """Rotate pairs ``(i, i + hd/2)`` of every head in place (``sign=-1`` inverts)."""
    T = buf.shape[0]
    if not buf.is_cuda:
        v = buf[:, col0:col0 + nheads * hd]
        xf = v.float().reshape(T, nheads, hd)
        pos = torch.arange(T) % S
        c, s = cs[pos][:, None, :], sn[pos][:, None, :] * sign
        a, b = xf[..., :hd // 2], xf[..., hd // 2:]
        v.copy_(torch.cat([a * c - b * s, b * c + a * s], -1).reshape(T, nheads * hd).to(buf.dtype))
        return buf
    _chk(lib().sga_rope(buf.data_ptr(), cs.data_ptr(), sn.data_ptr(), T, S, nheads, hd, buf.stride(0), col0,
                        float(sign), _st()), "sga_rope")
    return buf


# ----------------------------------------------------------------- SwiGLU
def swiglu_fwd(gu, out=None):
    T, F2 = gu.shape
    F = F2 // 2
    if not gu.is_cuda:
        y = (torch.nn.functional.silu(gu[:, :F].float()) * gu[:, F:].float()).to(gu.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    out = out if out is not None else torch.empty(T, F, dtype=gu.dtype, device=gu.device)
    _chk(lib().sga_swiglu_fwd(gu.data_ptr(), out.data_ptr(), T, F, _st()), "sga_swiglu_fwd")
    return out


def swiglu_bwd(gu, dout, out=None):
    T, F2 = gu.shape
    F = F2 // 2
    if not gu.is_cuda:
        g, u, d = gu[:, :F].float(), gu[:, F:].float(), dout.float()
        sg = torch.sigmoid(g)
        res = torch.cat([d * u * (sg * (1 + g * (1 - sg))), d * g * sg], 1).to(gu.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    out = out if out is not None else torch.empty_like(gu)
    _chk(lib().sga_swiglu_bwd(gu.data_ptr(), dout.data_ptr(), out.data_ptr(), T, F, _st()), "sga_swiglu_bwd")
    return out


# ---------------------------------------------------------- cross entropy
def cross_entropy_(logits, targets, grad_scale, write_grad=True):
    """Per-token loss (fp32); ``logits`` is overwritten by ``(softmax - onehot) * grad_scale``."""
    T, V = logits.shape
    if not logits.is_cuda:
        z = logits.float()
        lse = torch.logsumexp(z, -1)
        loss = lse - z.gather(1, targets[:, None]).squeeze(1)
        if write_grad:
            p = torch.softmax(z, -1)
            p[torch.arange(T), targets] -= 1.0
            logits.copy_((p * grad_scale).to(logits.dtype))
        return loss
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    _chk(lib().sga_cross_entropy(logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), T, V, logits.stride(0),
                                 float(grad_scale), int(write_grad), _st()), "sga_cross_entropy")
    return loss


# -------------------------------------------------------------- embedding
def embed_fwd(ids, W):
    if not W.is_cuda:
        return W[ids]
    T, H = ids.numel(), W.shape[1]
    out = torch.empty(T, H, dtype=W.dtype, device=W.device)
    _chk(lib().sga_embed_fwd(ids.data_ptr(), W.data_ptr(), out.data_ptr(), T, H, _st()), "sga_embed_fwd")
    return out


def embed_bwd(ids, dout, main_grad):
    if not dout.is_cuda:
        main_grad.index_add_(0, ids, dout.float())
        return
    T, H = dout.shape
    # stable sort: rows of a repeated token are summed in position order, so the result is reproducible
    sorted_ids, perm = torch.sort(ids.reshape(-1), stable=True)
    _chk(lib().sga_embed_bwd(sorted_ids.data_ptr(), perm.data_ptr(), dout.data_ptr(), main_grad.data_ptr(), T, H,
                             _st()), "sga_embed_bwd")
