"""``method=exact``: one global k-th value over the concatenated scores, then
an OR-merge of the masks across ranks (MAX of 0/1 bytes is OR and cannot wrap
at any world size). Costs O(model) temporaries and a full-model uint8
all-reduce; kept as the plain oracle form. ``sga/plugins/selection/_exact.py:12-48``.
"""
from __future__ import annotations

import torch


def select_masks_exact_kthvalue(grads, k, comm_group):
    flat = torch.cat([g.reshape(-1) for g in grads]).abs_()
    thr = torch.kthvalue(flat, flat.numel() - k + 1).values.item()
    mask = (flat >= thr).to(torch.uint8)
    del flat
    if comm_group is not None and torch.distributed.is_initialized():
        torch.distributed.all_reduce(mask, op=torch.distributed.ReduceOp.MAX, group=comm_group)
    out, off = [], 0
    for g in grads:
        out.append(mask[off:off + g.numel()])
        off += g.numel()
    return thr, out


class ExactKthvalue:
    def select(self, grads, k, comm_group, warmup_target=None):
        return select_masks_exact_kthvalue(grads, k, comm_group)
