"""Thin tensor-level wrappers over the native launchers in ``csrc``.

Every function takes CUDA tensors, launches on the current stream and returns
immediately (no host synchronisation). Shape / dtype / alignment contracts are
asserted here so that a bad call fails in Python, not on the device. The CPU
counterparts used by the unit tests and by gloo runs live in
``kernels_torch.py`` with the same names and semantics.

Counterpart of the reference's Triton wrappers (``sga/kernels.py:142-365``).
"""
from __future__ import annotations

import ctypes

import torch

from .csrc import _D, _F, _I, _L, _P, lib, register_sigs

register_sigs({
    "sga_adam_step": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _L, _P, _P, _I, _F, _F, _F, _F, _F, _F, _F, _F, _F,
                      _I, _I, _I, _I, _I, _I, _I, _P],
    "sga_sumsq": [_P, _P, _L, _P, _P, _I, _P],
    "sga_clip_coeff": [_P, _F, _F, _P, _P, _P],
    "sga_scale": [_P, _L, _P, _F, _P],
    "sga_cast_bf16": [_P, _P, _L, _P],
    "sga_hist_top": [_P, _L, _I, _I, _I, _P, _P, _P],
    "sga_hist_low16": [_P, _L, _I, _P, _P],
    "sga_mask_ge": [_P, _L, _I, _I, _I, _F, _P, _P, _P],
    "sga_mask_stats": [_P, _L, _P, _P],
    "sga_compact_mask": [_P, _L, _P, _P, _L, _P, _P, _P],
    "sga_dir_table": [_P, _L, _P, _I, _P],
    "sga_block_flags": [_P, _P, _P, _P, _I, _I, _L, _P, _P, _P],
    "sga_block_heads": [_P, _L, _P, _P, _P, _I, _I, _I, _P, _P],
    "sga_pack": [_P, _P, _L, _P, _F, _I, _I, _P],
    "sga_scatter": [_P, _P, _P, _L, _I, _P],
    "sga_gather_blocks": [_P, _P, _P, _L, _I, _L, _P, _F, _I, _I, _P],
    "sga_scatter_blocks": [_P, _P, _P, _L, _I, _L, _P, _P],
    "sga_block_reduce": [_P, _L, _I, _I, _P, _P],
    "sga_expand_blocks": [_P, _L, _I, _L, _P, _P],
    "sga_rmsnorm_fwd": [_P, _P, _P, _P, _L, _I, _L, _L, _I, _L, _L, _F, _P],
    "sga_rmsnorm_bwd_blocks": [],
    "sga_rmsnorm_bwd": [_P, _P, _P, _P, _P, _P, _P, _I, _L, _I, _L, _L, _L, _I, _L, _L, _L, _I, _P],
    "sga_rope": [_P, _P, _P, _L, _I, _I, _I, _L, _I, _F, _P],
    "sga_swiglu_fwd": [_P, _P, _L, _I, _P],
    "sga_swiglu_bwd": [_P, _P, _P, _L, _I, _P],
    "sga_cross_entropy": [_P, _P, _P, _L, _I, _L, _F, _I, _P],
    "sga_embed_fwd": [_P, _P, _P, _L, _I, _P],
    "sga_embed_bwd": [_P, _P, _P, _P, _L, _I, _P],
    "sga_add_bf16": [_P, _P, _P, _L, _P],
    "sga_symm_alloc": [_L, _P],
    "sga_symm_free": [_P],
    "sga_ipc_get_handle": [_P, _P],
    "sga_ipc_open": [_P, _P],
    "sga_ipc_close": [_P],
    "sga_p2p_allreduce": [_P, _P, _L, _F, _P, _P, _F, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _P],
    "sga_p2p_mask_union": [_P, _P, _P, _P, _L, _F, _P, _P, _P, _P, _I, _P, _I, _P],
    "sga_nvls_allreduce": [_P, _P, _P, _L, _F, _I, _P, _P, _P, _I, _I, _P],
    "sga_index_sync": [_P, _P, _P],
    "sga_dense_adamw_ag": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _P, _P, _I, _P, _F, _F, _F, _F, _F, _F, _F,
                           _I, _I, _P],
    "sga_tp_ag_gemm": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _I, _P],
    "sga_tp_gemm_rs": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "sga_replay_blocks": [],
    "sga_replay_pass1": [_P, _I, _F, _P, _P, _P, _I, _L, _P, _P, _P],
    "sga_replay_pass3": [_P, _I, _F, _P, _P, _P, _P, _P, _P, _P, _P, _I, _L, _F, _F, _F, _F, _F, _P, _P, _P],
    "sga_replay_score": [_P, _I, _F, _P, _P, _P, _P, _P, _P, _P, _I, _D, _D, _D, _D, _D, _L, _P, _P],
    "sga_replay_find_bin": [_P, _I, _P, _I, _I, _P],
    "sga_replay_hist_low16": [_P, _L, _P, _P, _P],
    "sga_replay_mask": [_P, _L, _P, _P, _P, _P],
    "sga_replay_tie_fill": [_P, _L, _P, _P, _P, _I, _I, _I, _P, _P],
    "sga_attn_fwd": [_P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _F, _P, _P],
    "sga_attn_bwd": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _F, _P, _P],
})


class NativeError(RuntimeError):
    pass


_LAUNCHES = [0]


def _chk(rc: int, what: str) -> None:
    _LAUNCHES[0] += 1
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")


def launch_count() -> int:
    """Number of native launcher calls so far (each launches at least one kernel)."""
    return _LAUNCHES[0]


def _st() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------ GEMM
EPI_BF16, EPI_F32, EPI_F32_ACC, EPI_BF16_ADD = 0, 1, 2, 3
_gemm_err = {}


def gemm_err_word(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _gemm_err:
        _gemm_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _gemm_err[key]


import os as _os

GEMM_PAIR = _os.environ.get("SGA_GEMM_PAIR", "1") != "0"  # CTA-pair (256 x 256) tiles when M >= 256


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
              epi: int = EPI_BF16, residual: torch.Tensor | None = None, alpha: float = 1.0,
              max_ctas: int = 0, pair: bool | None = None) -> torch.Tensor:
    """``out (epi)= alpha * A @ B^T`` on the tcgen05 tensor cores.

    ``a`` holds the logical ``[M, K]`` operand either K-major (stored
    ``[M, K]``) or, with ``a_mn``, MN-major (stored ``[K, M]``); likewise ``b``
    for the logical ``[N, K]`` operand. Row pitches come from ``stride(0)``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
    K, M = (a.shape[0], a.shape[1]) if a_mn else (a.shape[1], a.shape[0])
    Kb, N = (b.shape[0], b.shape[1]) if b_mn else (b.shape[1], b.shape[0])
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    assert out.shape[0] == M and out.shape[1] == N, (out.shape, M, N)
    if epi in (EPI_BF16, EPI_BF16_ADD):
        assert out.dtype == torch.bfloat16
    else:
        assert out.dtype == torch.float32
    if epi == EPI_BF16_ADD:
        assert residual is not None and residual.dtype == torch.bfloat16 and residual.stride(0) == out.stride(0)
    use_pair = GEMM_PAIR if pair is None else pair
    fn = lib().sga_gemm_bf16_pair if (use_pair and M >= 256) else lib().sga_gemm_bf16
    rc = fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), _p(residual), M, N, K, int(a_mn),
                             int(b_mn), a.stride(0), b.stride(0), out.stride(0), epi, float(alpha),
                             gemm_err_word(a.device).data_ptr(), max_ctas, _st())
    _chk(rc, "sga_gemm_bf16")
    return out


# ------------------------------------------------------------- optimizer
class SegmentTable:
    """Device copy of the arena's parameter segments and their group ids."""

    def __init__(self, starts, groups, n, device):
        assert len(starts) == len(groups) and len(starts) >= 1 and starts[0] == 0
        self.nseg = len(starts)
        self.n = int(n)
        self.seg_start = torch.tensor(list(starts) + [n], dtype=torch.int64, device=device)
        self.seg_group = torch.tensor(list(groups), dtype=torch.int32, device=device)


def adam_step(w, g, m, v, table: SegmentTable, group_lr, group_wd, *, beta1, beta2, eps, step, model=None, mask=None,
              coeff=None, emit=-1, clear=False, fold=False, interval=1.0, lr_scale=1.0, adams=False, max_ctas=0):
    n = w.numel()
    assert g.numel() == n and m.numel() == n and v.numel() == n and table.n == n
    for t in (w, g, m, v):
        assert t.dtype == torch.float32 and t.is_contiguous()
    if mask is not None:
        assert mask.dtype == torch.uint8 and mask.numel() == n
    ng = len(group_lr)
    lr_arr = (ctypes.c_float * ng)(*[float(x) for x in group_lr])
    wd_arr = (ctypes.c_float * ng)(*[float(x) for x in group_wd])
    bc1 = 1.0 if adams else 1.0 - beta1 ** step
    bc2 = 1.0 if adams else 1.0 - beta2 ** step
    rc = lib().sga_adam_step(w.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _p(model), _p(mask), _p(coeff),
                             table.seg_start.data_ptr(), table.seg_group.data_ptr(), table.nseg, n,
                             ctypes.cast(lr_arr, ctypes.c_void_p), ctypes.cast(wd_arr, ctypes.c_void_p), ng,
                             float(beta1), float(1.0 - beta1), float(beta2), float(1.0 - beta2), float(bc1),
                             float(bc2), float(eps), float(interval), float(lr_scale), int(emit), int(clear),
                             int(fold), int(lr_scale != 1.0), int(adams), int(coeff is not None), max_ctas, _st())
    _chk(rc, "sga_adam_step")


_partials = {}


def _partials_for(device):
    key = torch.device(device).index or 0
    if key not in _partials:
        _partials[key] = torch.empty(2048, dtype=torch.float32, device=device)
    return _partials[key]


def sumsq(x, out, mask=None, accumulate=False):
    """``out[0] (+)= sum(x^2)`` over mask-active lanes, deterministic order."""
    assert x.dtype == torch.float32 and x.is_contiguous() and out.dtype == torch.float32
    _chk(lib().sga_sumsq(x.data_ptr(), _p(mask), x.numel(), _partials_for(x.device).data_ptr(), out.data_ptr(),
                         int(accumulate), _st()), "sga_sumsq")
    return out


def clip_coeff(sumsq_t, inv_world, clip, coeff_out, norm_out):
    _chk(lib().sga_clip_coeff(sumsq_t.data_ptr(), float(inv_world), float(clip), coeff_out.data_ptr(),
                              norm_out.data_ptr(), _st()), "sga_clip_coeff")


def scale_(x, coeff=None, factor=1.0):
    _chk(lib().sga_scale(x.data_ptr(), x.numel(), _p(coeff), float(factor), _st()), "sga_scale")
    return x


def cast_bf16(src, dst):
    assert src.dtype == torch.float32 and dst.dtype == torch.bfloat16 and src.numel() == dst.numel()
    _chk(lib().sga_cast_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), _st()), "sga_cast_bf16")
    return dst


# -------------------------------------------------------------- selection
def hist_top(x, shift, stride, nbins, hist=None, nonfinite=None):
    assert x.dtype == torch.float32 and x.is_contiguous()
    if hist is None:
        hist = torch.zeros(nbins, dtype=torch.int64, device=x.device)
    _chk(lib().sga_hist_top(x.data_ptr(), x.numel(), shift, stride, nbins, hist.data_ptr(), _p(nonfinite), _st()),
         "sga_hist_top")
    return hist


def hist_low16(x, bin_, hist=None):
    if hist is None:
        hist = torch.zeros(65536, dtype=torch.int64, device=x.device)
    _chk(lib().sga_hist_low16(x.data_ptr(), x.numel(), int(bin_), hist.data_ptr(), _st()), "sga_hist_low16")
    return hist


def mask_ge(x, mask, *, bin_=None, shift=16, thr=None, count=None):
    mode = 0 if bin_ is not None else 1
    _chk(lib().sga_mask_ge(x.data_ptr(), x.numel(), mode, shift, int(bin_ or 0), float(thr or 0.0), mask.data_ptr(),
                           _p(count), _st()), "sga_mask_ge")
    return mask


def mask_stats(mask, out3=None):
    if out3 is None:
        out3 = torch.zeros(3, dtype=torch.int64, device=mask.device)
    _chk(lib().sga_mask_stats(mask.data_ptr(), mask.numel(), out3.data_ptr(), _st()), "sga_mask_stats")
    return out3


def compact_mask(mask, idx_out, total_out, err=None):
    n = mask.numel()
    if mask.data_ptr() % 16:
        mask = mask.clone()  # the kernels read 16 bytes at a time; a view at an odd offset is copied
    scratch = torch.empty((n + 4095) // 4096, dtype=torch.int32, device=mask.device)
    _chk(lib().sga_compact_mask(mask.data_ptr(), n, scratch.data_ptr(), idx_out.data_ptr(), idx_out.numel(),
                                total_out.data_ptr(), _p(err), _st()), "sga_compact_mask")


class SpanTable:
    """Device copy of a bucket's parameter spans with the running block count of an X-element tiling."""

    def __init__(self, spans, x: int, device):
        starts = [int(s) for s, _e in spans]
        ends = [int(e) for _s, e in spans]
        boff, run = [], 0
        for s, e in zip(starts, ends):
            boff.append(run)
            run += (e - s + x - 1) // x
        self.nblocks, self.nspan, self.x = run, len(starts), int(x)
        t = lambda v: torch.tensor(v, dtype=torch.int64, device=device)  # noqa: E731
        self.start, self.end, self.boff = t(starts), t(ends), t(boff + [run])


def block_forms(mask, spans, x: int, as_desc: bool, require_whole: bool = False):
    """Block heads (or packed ``head | tail_len`` descriptors) of the blocks with any selected
    element, ascending: flags per block, the mask compaction over the flags, heads from the
    surviving block numbers. ``require_whole`` also returns the number of partly selected blocks."""
    tab = SpanTable(spans, x, mask.device)
    if tab.nblocks == 0 or tab.nspan == 0:
        return torch.empty(0, dtype=torch.int32, device=mask.device), 0
    flags = torch.empty(tab.nblocks, dtype=torch.uint8, device=mask.device)
    partial = torch.zeros(1, dtype=torch.int64, device=mask.device)
    _chk(lib().sga_block_flags(mask.data_ptr(), tab.start.data_ptr(), tab.end.data_ptr(), tab.boff.data_ptr(),
                               tab.nspan, tab.x, tab.nblocks, flags.data_ptr(), partial.data_ptr(), _st()),
         "sga_block_flags")
    ids = torch.empty(tab.nblocks, dtype=torch.int32, device=mask.device)
    total = torch.zeros(1, dtype=torch.int64, device=mask.device)
    compact_mask(flags, ids, total)
    kb = int(total.item())
    out = torch.empty(kb, dtype=torch.int32, device=mask.device)
    _chk(lib().sga_block_heads(ids.data_ptr(), kb, tab.start.data_ptr(), tab.end.data_ptr(), tab.boff.data_ptr(),
                               tab.nspan, tab.x, int(as_desc), out.data_ptr(), _st()), "sga_block_heads")
    return out, (int(partial.item()) if require_whole else 0)


def dir_table(idx, k, n):
    nt = (n + 1023) // 1024 + 1
    table = torch.empty(nt, dtype=torch.int32, device=idx.device)
    _chk(lib().sga_dir_table(idx.data_ptr(), int(k), table.data_ptr(), nt, _st()), "sga_dir_table")
    return table


def pack_selected(grad, idx, vals, factor=1.0, zero=True):
    k = idx.numel()
    _chk(lib().sga_pack(grad.data_ptr(), idx.data_ptr(), k, vals.data_ptr(), float(factor), int(factor != 1.0),
                        int(zero), _st()), "sga_pack")
    return vals


def scatter_selected(dst, idx, vals, add=False):
    _chk(lib().sga_scatter(dst.data_ptr(), idx.data_ptr(), vals.data_ptr(), idx.numel(), int(add), _st()),
         "sga_scatter")
    return dst


def gather_selected_blocks(grad, mask, heads, x, vals, factor=1.0, zero=True):
    _chk(lib().sga_gather_blocks(grad.data_ptr(), mask.data_ptr(), heads.data_ptr(), heads.numel(), x, grad.numel(),
                                 vals.data_ptr(), float(factor), int(factor != 1.0), int(zero), _st()),
         "sga_gather_blocks")
    return vals


def scatter_selected_blocks(grad, mask, heads, x, vals):
    _chk(lib().sga_scatter_blocks(grad.data_ptr(), mask.data_ptr(), heads.data_ptr(), heads.numel(), x, grad.numel(),
                                  vals.data_ptr(), _st()), "sga_scatter_blocks")
    return grad


def block_reduce(x, bs, use_max):
    nb = (x.numel() + bs - 1) // bs
    out = torch.empty(nb, dtype=torch.float32, device=x.device)
    _chk(lib().sga_block_reduce(x.data_ptr(), x.numel(), bs, int(use_max), out.data_ptr(), _st()), "sga_block_reduce")
    return out


def expand_blocks(bmask, bs, n):
    mask = torch.empty(n, dtype=torch.uint8, device=bmask.device)
    _chk(lib().sga_expand_blocks(bmask.data_ptr(), bmask.numel(), bs, n, mask.data_ptr(), _st()), "sga_expand_blocks")
    return mask
