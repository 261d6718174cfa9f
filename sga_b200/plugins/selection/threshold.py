"""``method=adaptive``: selection by a persistent magnitude threshold that is
steered toward the target ratio instead of being recomputed every cycle.

Two parts. :class:`TauController` is a scalar state machine with no tensors in
it: it knows the threshold ``tau``, the streak of bootstrap selections that
landed inside the dead band, and how a measured ratio moves ``tau``.
:class:`AdaptiveThresholdSelect` is the tensor side the ``topk`` plugin calls:
while the controller asks for a bootstrap it selects with a histogram tier and
reports threshold and measured ratio back; afterwards one ``|x| >= tau`` pass
per tensor is the whole selection.

Rules (``sga/plugins/selection/_adaptive.py:22-174`` of the reference): the
dead band is +-0.01 around the target ratio; a bootstrap that misses it resets
the streak (warm-up gets longer, the tier is never changed); outside the band
``tau`` moves by ``(measured / target) ** 0.5`` limited to one step of
[0.9, 1.15]; a pass that selects nothing, or a non-positive ``tau``, goes
back to a bootstrap; ``tau`` never drops below the smallest positive bin edge
of the bootstrap tier. Scores are rank-identical at a boundary, hence so is
the controller's state.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _histogram as H

DEAD_BAND = 0.01
STEP_EXPONENT = 0.5
STEP_LIMITS = (0.9, 1.15)


def step_threshold(tau: float, measured: float, target: float) -> float:
    """The next threshold after a pass that selected ``measured`` of the coordinates."""
    if abs(measured - target) <= DEAD_BAND:
        return tau
    lo, hi = STEP_LIMITS
    return tau * min(hi, max(lo, (measured / target) ** STEP_EXPONENT))


def smallest_threshold(tier: str) -> float:
    """Lower edge of the first non-zero bin of a histogram tier: the floor of ``tau``."""
    shift = H.HIST_MODES[tier][0]
    return H.bin_edge_float(1, shift)


@dataclass
class TauController:
    target: float
    floor: float
    tau: float | None = None
    streak: int = 0

    def wants_bootstrap(self, required: int) -> bool:
        return self.tau is None or self.streak < max(required, 1)

    def bootstrapped(self, threshold: float, measured: float | None) -> float:
        """Adopt a histogram threshold; ``measured`` (``None`` after a collapse) feeds the streak."""
        self.tau = threshold if threshold > 0.0 else self.floor
        if measured is not None:
            self.streak = self.streak + 1 if abs(measured - self.target) <= DEAD_BAND else 0
        return self.tau

    def collapsed(self, measured: float) -> bool:
        return measured == 0.0 or self.tau is None or self.tau <= 0.0

    def steer(self, measured: float) -> float:
        """After a threshold pass: returns the threshold that pass used and moves ``tau``."""
        used = self.tau
        self.tau = step_threshold(used, measured, self.target)
        return used


def _selected_fraction(masks, grads) -> float:
    on = 0
    for m in masks:
        if m.is_cuda:
            from ... import kernels as K

            on += int(K.mask_stats(m)[0].item())
        else:
            on += int(torch.count_nonzero(m).item())
    return on / sum(g.numel() for g in grads)


class AdaptiveThresholdSelect:
    """Method object of the ``topk`` plugin for ``sga_selection_method adaptive``."""

    def __init__(self, ratio_percent: float, warmup_syncs, warmup_mode: str, global_allreduce: bool = True):
        if warmup_mode not in H.HIST_MODES:
            raise ValueError(f"unknown adaptive_warmup_mode: {warmup_mode!r} (expected one of {sorted(H.HIST_MODES)})")
        if not isinstance(global_allreduce, bool):
            raise ValueError(f"global_allreduce must be a bool, got {global_allreduce!r}")
        self.tier = warmup_mode
        self.warmup_syncs = warmup_syncs
        self.global_allreduce = global_allreduce
        self.ctl = TauController(target=ratio_percent / 100.0, floor=smallest_threshold(warmup_mode))

    # the controller's state under the names checkpoints and logs use
    @property
    def tau(self):
        return self.ctl.tau

    @tau.setter
    def tau(self, value):
        self.ctl.tau = value

    @property
    def warmup_passed(self) -> int:
        return self.ctl.streak

    @warmup_passed.setter
    def warmup_passed(self, value) -> None:
        self.ctl.streak = int(value)

    def state_dict(self) -> dict:
        return {"tau": self.ctl.tau, "warmup_passed": self.ctl.streak}

    def load_state_dict(self, state: dict) -> None:
        self.ctl.tau = state.get("tau", self.ctl.tau)
        self.ctl.streak = int(state.get("warmup_passed", self.ctl.streak))

    def warmup_sync_target(self, start_iter: int, period: int):
        """How many in-band bootstraps a selection that starts at ``start_iter`` still owes: the
        warm-up window is the first ``warmup_syncs * period`` iterations of the run, and a boundary
        that falls exactly on its end already counts as past it."""
        if self.warmup_syncs is None:
            return None
        window_end = self.warmup_syncs * period
        return max(0, (window_end - 1 - start_iter) // period)

    def _bootstrap(self, grads, k, comm_group):
        return H.select_masks_histogram(grads, k, comm_group, mode=self.tier, global_allreduce=self.global_allreduce)

    def _threshold_pass(self, grads):
        masks = []
        for g in grads:
            m = torch.empty(g.numel(), dtype=torch.uint8, device=g.device)
            if g.numel():
                H._ops(g).mask_ge(g.contiguous().view(-1), m, thr=self.ctl.tau)
            masks.append(m)
        return masks

    def select(self, grads, k, comm_group, warmup_target):
        if warmup_target is not None:
            required = warmup_target
        else:
            required = self.warmup_syncs if self.warmup_syncs is not None else 1
        if self.ctl.wants_bootstrap(required):
            thr, masks = self._bootstrap(grads, k, comm_group)
            return self.ctl.bootstrapped(thr, _selected_fraction(masks, grads)), masks
        masks = self._threshold_pass(grads)
        measured = _selected_fraction(masks, grads)
        if self.ctl.collapsed(measured):
            thr, masks = self._bootstrap(grads, k, comm_group)
            return self.ctl.bootstrapped(thr, None), masks
        return self.ctl.steer(measured), masks
