"""Support representation: what "selected" means for one gradient bucket.

The uint8 element mask is canonical; every other form is derived from it,
lazily and cached for the cycle in which the support is active:

  idx          ascending int32 positions of the selected elements
  block_idx    first element of every x-element block that has any selected
               element; blocks tile each parameter span from its start and
               never cross a span boundary
  block_desc   ``head | tail_len`` packed words (tail length in the low
               log2(x) bits, 0 = complete block)
  split        position in ``idx`` of the bucket midpoint (slice pipelining)
  dir_table    ``lower_bound(idx, j * 1024)`` directory for merge-joins

On CUDA the derivations run as native compaction kernels
(``csrc/select.cu``); on CPU as PyTorch ops. Same surface as the reference
(``sga/support.py:32-370``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import kernels_torch as KT

POOL_ROUND = 4 * 1024 * 1024  # index pools grow in 4 Mi-element steps and never shrink


class IndexPool:
    """Grow-only int32 buffer owned by one bucket (no allocator churn per cycle)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.buf: Optional[torch.Tensor] = None

    def get(self, k: int) -> torch.Tensor:
        if self.buf is None or self.buf.numel() < k:
            cap = max(POOL_ROUND, (k + POOL_ROUND - 1) // POOL_ROUND * POOL_ROUND)
            self.buf = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self.buf


def compact_mask_u8(mask_u8: torch.Tensor, pool: Optional[IndexPool] = None,
                    n_selected: Optional[int] = None) -> torch.Tensor:
    """mask -> ascending int32 index list. The mask must hold only 0 / 1 bytes."""
    n = mask_u8.numel()
    assert n < 2 ** 31, f"int32 indices assume < 2^31 elements per bucket, got {n}"
    if not mask_u8.is_cuda:
        return KT.compact_mask_idx(mask_u8)
    from . import kernels as K

    if n_selected is None:
        n_selected = int(K.mask_stats(mask_u8)[0].item())
    buf = pool.get(n_selected) if pool is not None else torch.empty(max(n_selected, 1), dtype=torch.int32,
                                                                    device=mask_u8.device)
    total = torch.zeros(1, dtype=torch.int64, device=mask_u8.device)
    K.compact_mask(mask_u8, buf, total)
    got = int(total.item())
    assert got == n_selected, f"compaction count {got} != mask count {n_selected} (mask holds bytes other than 0/1?)"
    return buf[:n_selected]


def _span_blocks(mask_u8, spans, x):
    """Per span: (any-selected per block, all-selected per block, block valid length)."""
    prev_end = 0
    for start, end in spans:
        assert start >= prev_end, f"spans must be ascending and non-overlapping ({start} after {prev_end})"
        prev_end = end
        n = end - start
        nb = (n + x - 1) // x
        if nb == 0:
            continue
        seg = mask_u8[start:end]
        pad = nb * x - n
        if pad:
            seg_any = torch.cat([seg, seg.new_zeros(pad)]).view(nb, x)
            seg_all = torch.cat([seg, seg.new_ones(pad)]).view(nb, x)
        else:
            seg_any = seg_all = seg.view(nb, x)
        yield start, end, nb, seg_any.any(dim=1), seg_all.all(dim=1)


def _check_spans(spans):
    prev_end = 0
    for start, end in spans:
        assert start >= prev_end, f"spans must be ascending and non-overlapping ({start} after {prev_end})"
        prev_end = end


def block_idx_from_mask(mask_u8: torch.Tensor, spans, x: int) -> torch.Tensor:
    """Block heads derived from the mask with the ANY rule, per parameter span."""
    assert mask_u8.numel() < 2 ** 31
    if mask_u8.is_cuda:
        from . import kernels as K

        _check_spans(spans)
        return K.block_forms(mask_u8, [(s, e) for s, e in spans if e > s], x, as_desc=False)[0]
    outs = []
    for start, _end, _nb, any_sel, _all in _span_blocks(mask_u8, spans, x):
        heads = torch.nonzero(any_sel, as_tuple=False).view(-1)
        if heads.numel():
            outs.append(heads * x + start)
    if not outs:
        return torch.empty(0, dtype=torch.int32, device=mask_u8.device)
    return torch.cat(outs).to(torch.int32)


def block_desc_from_mask(mask_u8: torch.Tensor, spans, x: int) -> torch.Tensor:
    """Packed ``head | tail_len`` descriptors; requires x a power of two >= 4,
    x-aligned span starts, and whole-run selection of every listed block."""
    assert x >= 4 and x & (x - 1) == 0, f"block_desc: block_size must be a power of two >= 4, got {x}"
    if mask_u8.is_cuda:
        from . import kernels as K

        _check_spans(spans)
        for start, _end in spans:
            assert start % x == 0, f"block_desc: span start {start} is not {x}-aligned"
        desc, partial = K.block_forms(mask_u8, [(s, e) for s, e in spans if e > s], x, as_desc=True,
                                      require_whole=True)
        assert partial == 0, (f"block_desc: {partial} partially selected {x}-block(s); descriptors transfer "
                              "whole runs")
        return desc
    outs = []
    for start, end, nb, any_sel, all_sel in _span_blocks(mask_u8, spans, x):
        assert start % x == 0, f"block_desc: span start {start} is not {x}-aligned"
        assert not bool((any_sel & ~all_sel).any()), (
            f"block_desc: partially selected {x}-block inside span [{start}, {end}); descriptors transfer whole runs")
        heads = torch.nonzero(any_sel, as_tuple=False).view(-1) * x + start
        if heads.numel():
            valid = torch.clamp(end - heads, max=x)
            tail = torch.where(valid < x, valid, torch.zeros_like(valid))
            outs.append(heads | tail)
    if not outs:
        return torch.empty(0, dtype=torch.int32, device=mask_u8.device)
    return torch.cat(outs).to(torch.int32)


@dataclass
class BucketSupport:
    mask_u8: torch.Tensor
    idx_pool: Optional[IndexPool] = field(default=None, repr=False)
    n_selected: Optional[int] = field(default=None, repr=False)
    block_size: int = 1
    block_spans: Optional[list] = field(default=None, repr=False)
    _idx: Optional[torch.Tensor] = field(default=None, repr=False)
    _block_idx: Optional[torch.Tensor] = field(default=None, repr=False)
    _block_desc: Optional[torch.Tensor] = field(default=None, repr=False)
    _split: Optional[int] = field(default=None, repr=False)
    _block_split: Optional[int] = field(default=None, repr=False)
    _dir_table: Optional[torch.Tensor] = field(default=None, repr=False)

    @property
    def count(self) -> int:
        return int(self.mask_u8.numel())

    def num_selected(self) -> int:
        if self.n_selected is None:
            if self.mask_u8.is_cuda:
                from . import kernels as K

                self.n_selected = int(K.mask_stats(self.mask_u8)[0].item())
            else:
                self.n_selected = int(torch.count_nonzero(self.mask_u8).item())
        return self.n_selected

    @property
    def idx(self) -> torch.Tensor:
        if self._idx is None:
            self._idx = compact_mask_u8(self.mask_u8, self.idx_pool, self.num_selected())
        return self._idx

    def _need_spans(self, what):
        if self.block_spans is None:
            raise ValueError(f"{what} needs block_spans (the bucket's parameter element spans)")

    @property
    def block_idx(self) -> torch.Tensor:
        if self.block_size == 1:
            return self.idx
        if self._block_idx is None:
            self._need_spans("block_idx")
            self._block_idx = block_idx_from_mask(self.mask_u8, self.block_spans, self.block_size)
        return self._block_idx

    @property
    def block_desc(self) -> torch.Tensor:
        if self.block_size == 1:
            raise ValueError("block_desc needs block_size > 1 (layout bb)")
        if self._block_desc is None:
            self._need_spans("block_desc")
            self._block_desc = block_desc_from_mask(self.mask_u8, self.block_spans, self.block_size)
        return self._block_desc

    @property
    def split(self) -> int:
        if self._split is None:
            mid = self.mask_u8.numel() // 2
            self._split = int(torch.searchsorted(self.idx, mid).item())
        return self._split

    @property
    def block_split(self) -> int:
        if self._block_split is None:
            mid = self.mask_u8.numel() // 2
            self._block_split = int(torch.searchsorted(self.block_idx, mid).item())
        return self._block_split

    @property
    def dir_table(self) -> torch.Tensor:
        if self._dir_table is None:
            if self.idx.is_cuda:
                from . import kernels as K

                self._dir_table = K.dir_table(self.idx, self.idx.numel(), self.count)
            else:
                self._dir_table = KT.dir_table(self.idx, self.idx.numel(), self.count)
        return self._dir_table


@dataclass
class Support:
    """Per-bucket supports, aligned with the engine's bucket order; active for one cycle."""

    buckets: list
    _total_selected: Optional[int] = field(default=None, repr=False)

    @property
    def total_selected(self) -> int:
        if self._total_selected is None:
            self._total_selected = sum(b.num_selected() for b in self.buckets)
        return self._total_selected

    @property
    def total_elements(self) -> int:
        return sum(b.count for b in self.buckets)
