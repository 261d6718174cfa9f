"""In-place sparse all-reduce on the dense bucket, index or block-descriptor
form (writeback-inherent).

The reference's backend of this name drives an external NCCL fork through
ctypes (``ncclSparseAllReduceIndex`` / ``ncclSparseAllReduceBlockIndex`` on a
private communicator and stream,
``sga/backends/nccl_pipelined_index.py:133-669``). Here the same contract --
"given the dense fp32 bucket and the sorted support, leave the reduced values
at the support positions" -- is one fused peer-memory kernel
(``sga_p2p_allreduce``), so there is no library fork to load.

Block form (``layout bb``): the support travels as packed ``head | tail_len``
descriptors, built on the device (``csrc/select.cu``), and the kernel itself
follows them: every descriptor is a run of 16 to 256 bytes that is gathered
into the payload, reduced across the ranks and scattered back with 128-bit
loads and stores; nothing is expanded to element indices. On the library
transports (``nccl`` / ``gloo``, and CPU) the descriptors are expanded once per
cycle and the element path of the parent backend carries them.

Kept, like the reference's, as a separately named backend with its own
runtime probe; refuses resume unless ``SGA_ALLOW_RESUME_PIPELINED=1``.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..config import get_args
from . import ENV_ALLOW_RESUME_PIPELINED
from .torch_pipelined_index import TorchPipelinedIndexBackend


def expand_descriptors(desc: torch.Tensor, x: int) -> torch.Tensor:
    """Packed descriptors -> ascending element indices."""
    if desc.numel() == 0:
        return desc.to(torch.int32)
    d = desc.to(torch.int64)
    head = d & ~(x - 1)
    tail = d & (x - 1)
    run = torch.where(tail == 0, torch.full_like(tail, x), tail)
    lanes = torch.arange(x, device=desc.device).unsqueeze(0)
    pos = head.unsqueeze(1) + lanes
    keep = lanes < run.unsqueeze(1)
    return pos[keep].to(torch.int32)


class NcclPipelinedIndexBackend(TorchPipelinedIndexBackend):
    consumes = "idx"
    inherent_emission = "writeback"
    block_form = "block_desc"
    name = "nccl_pipelined_index"

    def __init__(self):
        args = get_args()
        if args.sga_backend_emission == "compact":
            raise ValueError("sga_backend (nccl_pipelined_index): emission 'compact' is only supported by "
                             "torch_pipelined_index; this backend is writeback-inherent")
        super().__init__()
        self.emission = "writeback"
        self._desc_idx = {}

    def validate_runtime(self, args) -> None:
        if getattr(args, "tensor_model_parallel_size", 1) not in (None, 1):
            raise ValueError("nccl_pipelined_index requires tensor_model_parallel_size == 1")
        if getattr(args, "pipeline_model_parallel_size", 1) not in (None, 1):
            raise ValueError("nccl_pipelined_index requires pipeline_model_parallel_size == 1")
        if getattr(args, "load", None) and os.environ.get(ENV_ALLOW_RESUME_PIPELINED) != "1":
            raise ValueError("nccl_pipelined_index refuses to resume from a checkpoint "
                             f"(set {ENV_ALLOW_RESUME_PIPELINED}=1 to override)")

    def _runs(self, sup):
        """Payload elements of a block-form bucket: whole blocks, the last one of a span zero-padded."""
        return sup.block_desc.numel() * sup.block_size

    def on_support_activated(self, support, bucket_states) -> None:
        self._desc_idx = {}
        p2p = self.transport == "p2p"
        offs, total = {}, 0
        for bs, sup in zip(bucket_states, support.buckets):
            blocks = sup.block_size > 1 and self._layout_for(sup) == "bb"
            if blocks and not p2p:
                self._desc_idx[id(sup)] = expand_descriptors(sup.block_desc, sup.block_size)
            k = self._runs(sup) if blocks else sup.num_selected()
            offs[id(bs)] = total
            total += (k + 63) // 64 * 64
        if not p2p:
            return
        self._payload_off = offs
        need = 4 * max(total, 64)
        if self._payload is None or self._payload.nbytes < need:
            self._payload = self.ddp.pool.alloc(need + need // 4)

    def _impl(self, grad_data, support, comm_group, factor_in, reduce_op, key, bucket_state):
        if self._layout_for(support) != "bb":
            return super()._impl(grad_data, support, comm_group, factor_in, reduce_op, key, bucket_state)
        if self.transport == "p2p":
            from ..parallel import p2p

            desc = support.block_desc
            if desc.numel() == 0:
                return None
            ddp = self.ddp
            avg = reduce_op == dist.ReduceOp.AVG
            factor = float(factor_in) if (reduce_op == dist.ReduceOp.SUM and factor_in != 1.0) else 1.0
            ch = ddp.channels[key % len(ddp.channels)] if isinstance(key, int) else ddp.channels[0]
            p2p.allreduce_(ch, self._payload, 4 * self._payload_off[id(bucket_state)], self._runs(support),
                           scale=(1.0 / ddp.world) if avg else 1.0, grad=grad_data, idx=desc, factor=factor,
                           pack=True, zero_after_pack=False, scatter=True, block_x=int(support.block_size),
                           sumsq_out=self.sumsq, accumulate=True, max_ctas=ddp.ddp_config.comm_max_ctas)
            return None
        idx = self._desc_idx.get(id(support))
        if idx is None:
            idx = expand_descriptors(support.block_desc, support.block_size)
        view = _ElementView(idx, grad_data.numel())
        saved_layout, self.layout = self.layout, "er"
        try:
            return super()._impl(grad_data, view, comm_group, factor_in, reduce_op, key, bucket_state)
        finally:
            self.layout = saved_layout


class _ElementView:
    """What the element path of the parent backend reads from a support, over expanded descriptors."""

    block_size = 1

    def __init__(self, idx: torch.Tensor, n: int):
        self.idx = idx
        self.n_selected = idx.numel()
        self.split = int(torch.searchsorted(idx, n // 2).item()) if idx.numel() else 0
