"""``method=adaptive``: a persistent magnitude threshold tau steered toward
the target ratio.

Warm-up selects come from a histogram tier and are gated on the measured
ratio landing inside a +-0.01 dead band; a miss resets the consecutive count
(warm-up is extended, never escalated). Afterwards each reselection applies
``|x| >= tau`` and moves tau by ``(measured / target) ** 0.5`` clamped to
[0.9, 1.15] when outside the band. A zero measured ratio or a non-positive
tau re-bootstraps from the histogram, clamped to the smallest positive bin
edge. State is identical on every rank because the scores are.
``sga/plugins/selection/_adaptive.py:22-174``.
"""
from __future__ import annotations

import torch

from . import _histogram as H

ADAPT_BAND = 0.01
ADAPT_LOG_GAIN = 0.5
ADAPT_MAX_UP = 1.15
ADAPT_MAX_DOWN = 0.9


def adapt_threshold(thresh, measured_ratio, target_ratio, gain=ADAPT_LOG_GAIN, max_up=ADAPT_MAX_UP,
                    max_down=ADAPT_MAX_DOWN, band=ADAPT_BAND):
    if abs(measured_ratio - target_ratio) <= band:
        return thresh
    factor = (measured_ratio / target_ratio) ** gain
    return thresh * min(max(factor, max_down), max_up)


def count_on(mask: torch.Tensor) -> int:
    if mask.is_cuda:
        from ... import kernels as K

        return int(K.mask_stats(mask)[0].item())
    return int(torch.count_nonzero(mask).item())


def threshold_masks(grads, tau):
    masks = []
    for g in grads:
        m = torch.empty(g.numel(), dtype=torch.uint8, device=g.device)
        if g.numel():
            H._ops(g).mask_ge(g.contiguous().view(-1), m, thr=tau)
        masks.append(m)
    return masks


def tau_floor(warmup_mode) -> float:
    shift, _bins, _stride = H.HIST_MODES[warmup_mode]
    return H.bin_edge_float(1, shift)


class AdaptiveTau:
    def __init__(self, ratio_percent: float, warmup_syncs, warmup_mode: str, global_allreduce: bool = True):
        if warmup_mode not in H.HIST_MODES:
            raise ValueError(f"unknown adaptive_warmup_mode: {warmup_mode!r} (expected one of {sorted(H.HIST_MODES)})")
        if not isinstance(global_allreduce, bool):
            raise ValueError(f"global_allreduce must be a bool, got {global_allreduce!r}")
        self.target_ratio = ratio_percent / 100.0
        self.warmup_syncs = warmup_syncs
        self.warmup_mode = warmup_mode
        self.global_allreduce = global_allreduce
        self.tau = None
        self.warmup_passed = 0

    def warmup_sync_target(self, start_iter: int, period: int):
        """Gated selects left inside the warm-up window (``warmup_syncs * period``
        iterations from the run start) for a selection that starts at
        ``start_iter``; a boundary exactly at the window edge is post-warm-up."""
        if self.warmup_syncs is None:
            return None
        return max(0, (self.warmup_syncs * period - 1 - start_iter) // period)

    def _clamp(self, thresh: float) -> float:
        return thresh if thresh > 0.0 else tau_floor(self.warmup_mode)

    def _measure(self, masks, grads):
        return sum(count_on(m) for m in masks) / sum(g.numel() for g in grads)

    def select(self, grads, k, comm_group, warmup_target):
        required = max(warmup_target if warmup_target is not None
                       else (self.warmup_syncs if self.warmup_syncs is not None else 1), 1)
        if self.tau is None or self.warmup_passed < required:
            thr, masks = H.select_masks_histogram(grads, k, comm_group, mode=self.warmup_mode,
                                                  global_allreduce=self.global_allreduce)
            self.tau = self._clamp(thr)
            if abs(self._measure(masks, grads) - self.target_ratio) <= ADAPT_BAND:
                self.warmup_passed += 1
            else:
                self.warmup_passed = 0
            return self.tau, masks
        masks = threshold_masks(grads, self.tau)
        measured = self._measure(masks, grads)
        if measured == 0.0 or self.tau <= 0.0:
            thr, masks = H.select_masks_histogram(grads, k, comm_group, mode=self.warmup_mode,
                                                  global_allreduce=self.global_allreduce)
            self.tau = self._clamp(thr)
            return self.tau, masks
        used = self.tau
        self.tau = adapt_threshold(used, measured, self.target_ratio)
        return used, masks
