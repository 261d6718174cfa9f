"""Bit-pattern histogram selection.

The key of a score ``x`` is ``(bits(|x|) & 0x7FFFFFFF) >> shift``: monotone in
``|x|``, so a histogram of keys locates the k-th largest magnitude without a
sort. Three tiers (``sga/plugins/selection/_histogram.py:48-216``):

  exact     shift 16, 32769 bins, every element. The crossing bin is refined
            to the exact k-th value; the mask is ``|x| >= thr`` (ties are all
            selected, so the count can exceed k).
  balanced  shift 16, 32769 bins, every 8th element of each view. The whole
            crossing bin is taken; the reported threshold is its lower edge.
  fast      shift 19, 4097 bins, every 8th element.

On CUDA the passes are native kernels (``csrc/select.cu``): one histogram
launch per view, a second-digit histogram for the exact refinement (no
candidate gather, no kthvalue), and one fused mask+count launch per view.
With ``block_size > 1`` the same machinery runs on per-block mean|max scores
and the block masks are expanded back to elements.
"""
from __future__ import annotations

import torch

from ... import kernels_torch as KT

HIST_SHIFT = 16
HIST_BINS = 32769
HIST_SHIFT_COARSE = 19
HIST_BINS_COARSE = 4097
HIST_SAMPLE_STRIDE = 8

HIST_MODES = {
    "exact": (HIST_SHIFT, HIST_BINS, 1),
    "balanced": (HIST_SHIFT, HIST_BINS, HIST_SAMPLE_STRIDE),
    "fast": (HIST_SHIFT_COARSE, HIST_BINS_COARSE, HIST_SAMPLE_STRIDE),
}


def _ops(t: torch.Tensor):
    if t.is_cuda:
        from ... import kernels as K

        return K
    return KT


def bin_edge_float(b: int, shift: int) -> float:
    """Lower edge of bin ``b`` as a float."""
    bits = (int(b) << shift) & 0x7FFFFFFF
    return torch.tensor([bits], dtype=torch.int32).view(torch.float32).item()


def sampled_count(n: int, stride: int) -> int:
    return (n + stride - 1) // stride


def build_histogram(grads, shift: int, nbins: int, stride: int) -> torch.Tensor:
    """Sum over views of the histogram of each view's own stride subsample."""
    device = grads[0].device
    hist = torch.zeros(nbins, dtype=torch.int64, device=device)
    for g in grads:
        if g.numel():
            _ops(g).hist_top(g.contiguous().view(-1), shift, stride, nbins, hist)
    return hist


def balanced_crossing_bin(hist, n_total, n_sampled, k, *, replicas=1) -> int:
    r = max(1, round(n_sampled * (n_total - k + 1) / n_total)) * replicas
    return int(torch.searchsorted(torch.cumsum(hist, 0), r).item())


def exact_threshold(hist, k, world, grads, shift=HIST_SHIFT) -> float:
    """The exact k-th largest ``|x|``: crossing bin from the top-16-bit
    histogram, then the crossing low-16-bit key inside that bin."""
    assert shift == 16, "the two-digit refinement splits the key 16 + 16"
    cum = torch.cumsum(hist, 0)
    total = int(cum[-1].item())
    r = total - k * world + 1
    b = int(torch.searchsorted(cum, r).item())
    n_above = (total - int(cum[b].item())) // world
    low = torch.zeros(65536, dtype=torch.int64, device=hist.device)
    for g in grads:
        if g.numel():
            _ops(g).hist_low16(g.contiguous().view(-1), b, low)
    want = k - n_above  # rank from the top inside bin b (local units: grads are this rank's own)
    in_bin = int(low.sum().item())
    assert 1 <= want <= in_bin, f"histogram select out of range: want={want}, in_bin={in_bin}, k={k}, above={n_above}"
    suffix = torch.cumsum(low.flip(0), 0)
    lb = 65535 - int(torch.searchsorted(suffix, want).item())
    bits = (b << 16) | lb
    return torch.tensor([bits], dtype=torch.int32).view(torch.float32).item()


def select_masks_histogram(grads, k, comm_group, mode="exact", global_allreduce=True, masks_out=None):
    """Returns ``(threshold, [uint8 mask per view])``."""
    try:
        shift, nbins, stride = HIST_MODES[mode]
    except KeyError:
        raise ValueError(f"unknown histogram_mode: {mode!r}") from None
    hist = build_histogram(grads, shift, nbins, stride)
    if global_allreduce and comm_group is not None and torch.distributed.is_initialized():
        torch.distributed.all_reduce(hist, op=torch.distributed.ReduceOp.SUM, group=comm_group)
        world = torch.distributed.get_world_size(comm_group)
    else:
        world = 1

    def _mask_for(i, g):
        if masks_out is not None:
            return masks_out[i]
        return torch.empty(g.numel(), dtype=torch.uint8, device=g.device)

    masks = []
    if mode == "exact":
        thr = exact_threshold(hist, k, world, grads, shift)
        for i, g in enumerate(grads):
            m = _mask_for(i, g)
            if g.numel():
                _ops(g).mask_ge(g.contiguous().view(-1), m, thr=thr)
            masks.append(m)
        return thr, masks
    n_total = sum(g.numel() for g in grads)
    n_sampled = sum(sampled_count(g.numel(), stride) for g in grads)
    b = balanced_crossing_bin(hist, n_total, n_sampled, k, replicas=world)
    for i, g in enumerate(grads):
        m = _mask_for(i, g)
        if g.numel():
            _ops(g).mask_ge(g.contiguous().view(-1), m, bin_=b, shift=shift)
        masks.append(m)
    return bin_edge_float(b, shift), masks


def block_reduce_views(grads, x, reduce):
    return [(_ops(g).block_reduce(g.contiguous().view(-1), x, reduce == "max") if g.numel()
             else torch.empty(0, device=g.device)) for g in grads]


class HistogramSelect:
    """``select(grads, k, comm_group, warmup_target) -> (threshold, masks)``."""

    def __init__(self, mode: str = "exact", block_size: int = 1, block_reduce: str = "mean",
                 global_allreduce: bool = True):
        if mode not in HIST_MODES:
            raise ValueError(f"unknown histogram_mode: {mode!r} (expected one of {sorted(HIST_MODES)})")
        if (not isinstance(block_size, int) or isinstance(block_size, bool) or block_size < 1 or block_size > 1024
                or block_size & (block_size - 1)):
            raise ValueError(f"block_size must be a power of two in [1, 1024], got {block_size!r}")
        if block_reduce not in ("mean", "max"):
            raise ValueError(f"block_reduce must be 'mean' or 'max', got {block_reduce!r}")
        if not isinstance(global_allreduce, bool):
            raise ValueError(f"global_allreduce must be a bool, got {global_allreduce!r}")
        self.mode = mode
        self.block_size = block_size
        self.block_reduce = block_reduce
        self.global_allreduce = global_allreduce

    def select(self, grads, k, comm_group, warmup_target=None):
        if self.block_size == 1:
            return select_masks_histogram(grads, k, comm_group, mode=self.mode,
                                          global_allreduce=self.global_allreduce)
        x = self.block_size
        k_blocks = max(1, int(round(k / x)))
        bviews = block_reduce_views(grads, x, self.block_reduce)
        thr, bmasks = select_masks_histogram(bviews, k_blocks, comm_group, mode=self.mode,
                                             global_allreduce=self.global_allreduce)
        masks = [_ops(g).expand_blocks(bm, x, g.numel()) if g.numel()
                 else torch.empty(0, dtype=torch.uint8, device=g.device) for bm, g in zip(bmasks, grads)]
        return thr, masks
