"""The ``topk`` selection plugin: global ``k = max(1, round(n * ratio%))`` over
the eligible coordinates, dispatched to the configured method.

Built with no arguments; knobs come from the args singleton. A one-time
packed MIN/MAX probe makes a rank-split of the histogram all-reduce gate a
loud, symmetric error instead of a hang. ``sga/plugins/selection/topk.py:57-167``.
"""
from __future__ import annotations

import torch

from ...config import get_args
from ._adaptive import AdaptiveTau
from ._exact import ExactKthvalue
from ._histogram import HistogramSelect


class TopkSelection:
    def __init__(self):
        args = get_args()
        self.method = args.sga_selection_method
        self.ratio_percent = float(args.sga_selection_ratio_percent)
        assert 0.0 < self.ratio_percent < 100.0, f"ratio_percent must be in (0, 100), got {self.ratio_percent}"
        gate = bool(args.sga_selection_topk_histogram_add_global_allreduce)
        if self.method == "adaptive":
            ws = args.sga_selection_adaptive_warmup_syncs
            self._impl = AdaptiveTau(self.ratio_percent, int(ws) if ws is not None else None,
                                     args.sga_selection_adaptive_warmup_mode, global_allreduce=gate)
        elif self.method == "histogram":
            self._impl = HistogramSelect(args.sga_selection_histogram_mode,
                                         block_size=int(args.sga_selection_block_size),
                                         block_reduce=args.sga_selection_block_reduce, global_allreduce=gate)
        elif self.method == "exact":
            self._impl = ExactKthvalue()
        else:
            raise ValueError(f"sga_selection_method must be adaptive|exact|histogram (got {self.method!r})")
        self.last_threshold = None
        self._rank_gate_checked = False

    @property
    def block_size(self):
        return getattr(self._impl, "block_size", 1)

    @property
    def tau(self):
        return getattr(self._impl, "tau", None)

    @property
    def warmup_passed(self):
        return getattr(self._impl, "warmup_passed", None)

    def k_for(self, n_total: int) -> int:
        return max(1, int(round(n_total * self.ratio_percent / 100.0)))

    def warmup_sync_target(self, start_iter: int, period: int):
        hook = getattr(self._impl, "warmup_sync_target", None)
        return hook(start_iter, period) if callable(hook) else None

    def _check_rank_gate(self, ctx):
        gate = getattr(self._impl, "global_allreduce", None)
        if gate is None or ctx.comm_group is None or not torch.distributed.is_initialized():
            return True
        device = ctx.grad_views[0].device if ctx.grad_views else "cpu"
        packed = torch.tensor([int(gate), -int(gate)], dtype=torch.int64, device=device)
        torch.distributed.all_reduce(packed, op=torch.distributed.ReduceOp.MAX, group=ctx.comm_group)
        hi, lo = int(packed[0].item()), -int(packed[1].item())
        if lo != hi:
            raise ValueError("sga_selection_topk_histogram_add_global_allreduce differs across the selection "
                             f"group (local={int(gate)}, group=[{lo}, {hi}]): ranks would disagree on entering "
                             "the histogram all-reduce; align the flag on every rank")
        return True

    def select(self, ctx):
        if not self._rank_gate_checked:
            self._rank_gate_checked = self._check_rank_gate(ctx)
        k = self.k_for(sum(g.numel() for g in ctx.grad_views))
        thr, masks = self._impl.select(ctx.grad_views, k, ctx.comm_group, getattr(ctx, "warmup_target", None))
        self.last_threshold = thr
        return masks
