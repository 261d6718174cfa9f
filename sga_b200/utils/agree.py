"""Cross-rank agreement on small host-side integers before a collective that
would hang or corrupt if the ranks disagreed.

One packed MAX all-reduce of ``[v, -v]`` yields the group's maximum and
minimum of every value at once; a spread is reported on every rank with the
same message, so the job fails loudly and symmetrically. Used for the
histogram all-reduce switch of the selection plugin (the reference probes it
the same way, ``sga/plugins/selection/topk.py:121-151``) and for the
per-bucket support sizes (``sga/engine.py:1299-1330``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def group_min_max(values, group, device="cpu"):
    """``(mins, maxs)`` of each integer in ``values`` over ``group`` (one all-reduce)."""
    t = torch.tensor([int(v) for v in values], dtype=torch.int64, device=device)
    packed = torch.cat([t, -t])
    dist.all_reduce(packed, op=dist.ReduceOp.MAX, group=group)
    n = t.numel()
    return [-int(x) for x in packed[n:].tolist()], [int(x) for x in packed[:n].tolist()]


def require_uniform(value: int, group, device, describe) -> None:
    """Raise ``ValueError(describe(local, lo, hi))`` on every rank unless all ranks pass the same
    ``value``. A missing group or an uninitialised process group means one rank: nothing to check."""
    if group is None or not (dist.is_available() and dist.is_initialized()):
        return
    (lo,), (hi,) = group_min_max([value], group, device)
    if lo != hi:
        raise ValueError(describe(int(value), lo, hi))
