"""PyTorch (CPU or any device) counterparts of the native support kernels.

Same names and semantics as the CUDA wrappers in ``kernels.py``; used on CPU
(gloo runs, unit tests) and as the oracles of the GPU tests. Counterpart of
``sga/kernels_torch.py`` in the reference.
"""
from __future__ import annotations

import torch


def abs_bit_key(x: torch.Tensor, shift: int = 0) -> torch.Tensor:
    """``(bits(|x|) & 0x7FFFFFFF) >> shift`` as int32 (monotone in ``|x|``)."""
    return (x.contiguous().view(torch.int32) & 0x7FFFFFFF) >> shift


def hist_top(x, shift, stride, nbins, hist=None, nonfinite=None):
    if hist is None:
        hist = torch.zeros(nbins, dtype=torch.int64, device=x.device)
    key = abs_bit_key(x[::stride] if stride > 1 else x, shift)
    hist += torch.bincount(key.long(), minlength=nbins)[:nbins]
    return hist


def hist_low16(x, bin_, hist=None):
    if hist is None:
        hist = torch.zeros(65536, dtype=torch.int64, device=x.device)
    key = abs_bit_key(x)
    sel = key[(key >> 16) == bin_] & 0xFFFF
    hist += torch.bincount(sel.long(), minlength=65536)
    return hist


def mask_ge(x, mask, *, bin_=None, shift=16, thr=None, count=None):
    on = (abs_bit_key(x, shift) >= bin_) if bin_ is not None else (x.abs() >= thr)
    mask.copy_(on.to(torch.uint8))
    if count is not None:
        count += on.sum()
    return mask


def mask_stats(mask, out3=None):
    if out3 is None:
        out3 = torch.zeros(3, dtype=torch.int64, device=mask.device)
    pos = torch.nonzero(mask, as_tuple=False).view(-1)
    out3[0] += pos.numel()
    out3[1] += pos.sum()
    out3[2] += ((pos % 9973) * (pos % 1009)).sum()
    return out3


def compact_mask_idx(mask: torch.Tensor) -> torch.Tensor:
    return torch.nonzero(mask, as_tuple=False).view(-1).to(torch.int32)


def dir_table(idx, k, n):
    nt = (n + 1023) // 1024 + 1
    targets = torch.arange(nt, dtype=torch.int64, device=idx.device) * 1024
    return torch.searchsorted(idx[:k].long(), targets).to(torch.int32)


def pack_selected(grad, idx, vals, factor=1.0, zero=True):
    li = idx.long()
    v = grad[li]
    vals.copy_(v * factor if factor != 1.0 else v)
    if zero:
        grad[li] = 0.0
    return vals


def scatter_selected(dst, idx, vals, add=False):
    li = idx.long()
    if add:
        dst.index_add_(0, li, vals)
    else:
        dst[li] = vals
    return dst


def _block_lanes(heads, x, n):
    pos = heads.long().unsqueeze(1) + torch.arange(x, device=heads.device).unsqueeze(0)
    return pos.view(-1)


def gather_selected_blocks(grad, mask, heads, x, vals, factor=1.0, zero=True):
    n = grad.numel()
    pos = _block_lanes(heads, x, n)
    ok = pos < n
    safe = pos.clamp(max=n - 1)
    ok = ok & (mask[safe] > 0)
    v = torch.where(ok, grad[safe], torch.zeros((), dtype=grad.dtype, device=grad.device))
    vals.copy_(v * factor if factor != 1.0 else v)
    if zero:
        grad[safe[ok]] = 0.0
    return vals


def scatter_selected_blocks(grad, mask, heads, x, vals):
    n = grad.numel()
    pos = _block_lanes(heads, x, n)
    ok = pos < n
    safe = pos.clamp(max=n - 1)
    ok = ok & (mask[safe] > 0)
    grad[safe[ok]] = vals[ok]
    return grad


def block_reduce(x, bs, use_max):
    n = x.numel()
    nb = (n + bs - 1) // bs
    a = x.abs()
    pad = nb * bs - n
    if pad:
        a = torch.cat([a, torch.zeros(pad, dtype=a.dtype, device=a.device)])
    a = a.view(nb, bs)
    if use_max:
        return a.amax(dim=1)
    lens = torch.full((nb,), bs, dtype=a.dtype, device=a.device)
    if pad:
        lens[-1] = bs - pad
    return a.sum(dim=1) / lens


def expand_blocks(bmask, bs, n):
    return bmask.repeat_interleave(bs)[:n].contiguous()


def sumsq(x, out, mask=None, accumulate=False):
    v = x if mask is None else torch.where(mask > 0, x, torch.zeros_like(x))
    s = (v.double() ** 2).sum().to(out.dtype)
    if accumulate:
        out[0] += s
    else:
        out[0] = s
    return out


def topk_exact_flat(score_abs: torch.Tensor, k: int) -> torch.Tensor:
    """Exactly ``k`` positions: everything strictly above the k-th value, then
    the first ties in index order. Returns a uint8 mask."""
    n = score_abs.numel()
    k = max(0, min(int(k), n))
    mask = torch.zeros(n, dtype=torch.uint8, device=score_abs.device)
    if k == 0:
        return mask
    key = abs_bit_key(score_abs)
    thr = torch.kthvalue(key, n - k + 1).values
    gt = key > thr
    mask[gt] = 1
    need = k - int(gt.sum())
    if need > 0:
        ties = torch.nonzero(key == thr, as_tuple=False).view(-1)[:need]
        mask[ties] = 1
    return mask


def topk_rank_local(score_abs: torch.Tensor, k: int) -> torch.Tensor:
    """Selection rule of the fused rank-local kernel (``csrc/index_sync.cu``): the exact top-``k``
    of :func:`topk_exact_flat`, minus the coordinates whose score is exactly zero (a zero carries
    nothing to send, so a bucket with fewer than ``k`` non-zero scores selects only those)."""
    mask = topk_exact_flat(score_abs, k)
    mask[abs_bit_key(score_abs) == 0] = 0
    return mask

