"""The ``topk`` selection plugin.

One budget for the whole model: ``k = max(1, round(n * ratio% / 100))`` over
the eligible coordinates the engine hands over, split among tensors by
whichever method the configuration names. Methods are looked up in a small
table of factories (histogram tiers, exact k-th value, adaptive threshold);
the plugin itself only owns the budget, the last threshold (for the log line)
and a once-per-run check that every rank agrees on whether histograms are
all-reduced, so that a split configuration fails with one clear message on
every rank instead of hanging in the collective.

Zero-argument construction from the args singleton, ``select(ctx) -> [mask]``,
``block_size``, ``k_for``, ``warmup_sync_target`` and ``last_threshold`` are
the plugin protocol of ``sga/plugins/selection/topk.py:57-167``.
"""
from __future__ import annotations

from ...config import get_args
from ...utils.agree import require_uniform
from ._exact import ExactKthvalue
from ._histogram import HistogramSelect
from .threshold import AdaptiveThresholdSelect


def _adaptive(args, ratio_percent, allreduce_hist):
    syncs = args.sga_selection_adaptive_warmup_syncs
    return AdaptiveThresholdSelect(ratio_percent, None if syncs is None else int(syncs),
                                   args.sga_selection_adaptive_warmup_mode, global_allreduce=allreduce_hist)


def _histogram(args, ratio_percent, allreduce_hist):
    return HistogramSelect(args.sga_selection_histogram_mode, block_size=int(args.sga_selection_block_size),
                           block_reduce=args.sga_selection_block_reduce, global_allreduce=allreduce_hist)


def _exact(args, ratio_percent, allreduce_hist):
    return ExactKthvalue()


METHODS = {"adaptive": _adaptive, "histogram": _histogram, "exact": _exact}


class TopkSelection:
    def __init__(self):
        args = get_args()
        self.method = args.sga_selection_method
        self.ratio_percent = float(args.sga_selection_ratio_percent)
        if not 0.0 < self.ratio_percent < 100.0:
            raise AssertionError(f"ratio_percent must be in (0, 100), got {self.ratio_percent}")
        if self.method not in METHODS:
            raise ValueError(f"sga_selection_method must be {'|'.join(sorted(METHODS))} (got {self.method!r})")
        self.worker = METHODS[self.method](args, self.ratio_percent,
                                           bool(args.sga_selection_topk_histogram_add_global_allreduce))
        self.last_threshold = None
        self._flag_agreed = False

    # ---- what the engine and the log line read
    @property
    def block_size(self) -> int:
        return getattr(self.worker, "block_size", 1)

    @property
    def tau(self):
        return getattr(self.worker, "tau", None)

    @property
    def warmup_passed(self):
        return getattr(self.worker, "warmup_passed", None)

    def k_for(self, n_total: int) -> int:
        return max(1, int(round(n_total * self.ratio_percent / 100.0)))

    def warmup_sync_target(self, start_iter: int, period: int):
        hook = getattr(self.worker, "warmup_sync_target", None)
        return hook(start_iter, period) if callable(hook) else None

    # ---- running state, for a bit-continuous resume
    def state_dict(self) -> dict:
        inner = getattr(self.worker, "state_dict", None)
        return {"last_threshold": self.last_threshold, "method": inner() if callable(inner) else None}

    def load_state_dict(self, state: dict) -> None:
        self.last_threshold = state.get("last_threshold", self.last_threshold)
        inner = getattr(self.worker, "load_state_dict", None)
        if callable(inner) and state.get("method") is not None:
            inner(state["method"])

    # ---- selection
    def _agree_on_histogram_allreduce(self, ctx) -> None:
        flag = getattr(self.worker, "global_allreduce", None)
        if flag is None:
            return
        device = ctx.grad_views[0].device if ctx.grad_views else "cpu"
        require_uniform(
            int(flag), ctx.comm_group, device,
            lambda local, lo, hi: ("sga_selection_topk_histogram_add_global_allreduce differs across the selection "
                                   f"group (local={local}, group=[{lo}, {hi}]): ranks would disagree on entering "
                                   "the histogram all-reduce; align the flag on every rank"))

    def select(self, ctx):
        if not self._flag_agreed:
            self._agree_on_histogram_allreduce(ctx)
            self._flag_agreed = True
        budget = self.k_for(sum(g.numel() for g in ctx.grad_views))
        self.last_threshold, masks = self.worker.select(ctx.grad_views, budget, ctx.comm_group,
                                                        getattr(ctx, "warmup_target", None))
        return masks
