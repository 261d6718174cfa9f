"""Mask-form sparse all-reduce backend (writeback-inherent).

* ``p2p`` transport: the support's bit mask sits in symmetric memory and one
  fused kernel ORs the ranks' masks and reduces the masked entries of the
  gradient bucket in place, each rank owning a slice (``sga_p2p_mask_union``).
  With a shared support the union equals every rank's mask; with rank-local
  selection (``sync_rank_local``) the per-rank masks differ and the union
  becomes the step's support, expanded to the uint8 mask the optimizer reads.
* library transport: per slice, boolean-index gather -> payload-only scale ->
  async all-reduce -> masked scatter, pipelined over ``mask_slices`` slices.

``sga/backends/torch_pipelined_mask.py:27-138``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import kernels_torch as KT
from ..config import get_args
from ..plugins import resolve_emission
from ..utils import backend_timer


def pack_bits(mask_u8: torch.Tensor, out_words: torch.Tensor) -> torch.Tensor:
    """uint8 0/1 mask -> little-endian bit words (int32), ``out_words[ceil(n/32)]``."""
    n = mask_u8.numel()
    nw = (n + 31) // 32
    pad = nw * 32 - n
    m = mask_u8 if pad == 0 else torch.cat([mask_u8, mask_u8.new_zeros(pad)])
    w = torch.tensor([1 << i for i in range(31)] + [-(1 << 31)], dtype=torch.int64, device=m.device)
    words = (m.view(nw, 32).to(torch.int64) * w).sum(1)
    out_words[:nw].copy_(words.to(torch.int32))
    return out_words


class TorchPipelinedMaskBackend:
    consumes = "mask"
    inherent_emission = "writeback"
    block_form = "block_idx"
    name = "torch_pipelined_mask"

    def __init__(self):
        args = get_args()
        emission = args.sga_backend_emission
        if emission == "compact":
            raise ValueError("sga_backend (torch_pipelined_mask): emission 'compact' is only supported by "
                             "torch_pipelined_index; this backend is writeback-inherent")
        if emission not in (None, "auto", "writeback"):
            raise ValueError(f"sga_backend_emission must be auto|compact|writeback (got {emission!r})")
        self.emission = resolve_emission(emission, self.inherent_emission)
        self.layout = "mask"
        s = args.sga_backend_mask_slices
        if not isinstance(s, int) or isinstance(s, bool) or s < 1:
            raise ValueError(f"mask_slices must be an int >= 1, got {s!r}")
        self._mask_slices = s
        self.ddp = None
        self.sumsq = None
        self._bits = None      # symmetric: per-rank bit masks, arena-wide
        self._ubits = None     # symmetric: union bit masks, arena-wide
        self._bits_valid_for = None
        self._scratch = None
        self.union_count = None

    def bind(self, ddp) -> None:
        self.ddp = ddp
        if ddp.device.type == "cuda":
            self.sumsq = torch.zeros(1, dtype=torch.float32, device=ddp.device)
            self.union_count = torch.zeros(1, dtype=torch.int64, device=ddp.device)

    @property
    def transport(self):
        return self.ddp.transport if self.ddp is not None else "gloo"

    def validate_runtime(self, args) -> None:
        return None

    def _ensure_bits(self):
        if self._bits is None:
            nwords = (self.ddp.arena.numel + 31) // 32 + 2 * len(self.ddp.arena.buckets) + 8
            self._bits = self.ddp.pool.alloc(4 * nwords)
            self._ubits = self.ddp.pool.alloc(4 * nwords)

    def _word_off(self, bucket_state):
        # buckets start on 64-element boundaries, so every bucket owns whole words
        return bucket_state.arena_start // 32

    def on_support_activated(self, support, bucket_states) -> None:
        if self.transport != "p2p":
            return
        self._ensure_bits()
        for bs, sup in zip(bucket_states, support.buckets):
            nw = (sup.count + 31) // 32
            pack_bits(sup.mask_u8, self._bits.view(torch.int32, 4 * self._word_off(bs), nw))

    # ------------------------------------------------------ shared support
    def allreduce_sparse(self, grad_data, support, comm_group, gradient_scaling_factor, reduce_op, key=None,
                         bucket_state=None) -> None:
        with backend_timer.region("sparse", backend=self.name, layout="mask", block_size=None, bucket=key,
                                  k=getattr(support, "n_selected", None)):
            return self._impl(grad_data, support, comm_group, gradient_scaling_factor, reduce_op, key, bucket_state)

    def _impl(self, grad_data, support, comm_group, factor_in, reduce_op, key, bs):
        scale_payload = reduce_op == dist.ReduceOp.SUM and factor_in != 1.0
        if self.transport == "p2p":
            from ..parallel import p2p

            ddp = self.ddp
            scale = (1.0 / ddp.world) if reduce_op == dist.ReduceOp.AVG else (float(factor_in) if scale_payload else 1.0)
            woff = 4 * self._word_off(bs)
            p2p.mask_union_reduce_(ddp.channels[bs.bucket_id % len(ddp.channels)], ddp.arena.symm_grad,
                                   4 * bs.arena_start, self._bits, woff, self._ubits, woff, grad_data.numel(),
                                   scale=scale, mask_u8=None, sumsq_out=self.sumsq, accumulate=True,
                                   max_ctas=ddp.ddp_config.comm_max_ctas)
            return None
        element_mask = support.mask_u8 > 0
        numel = grad_data.numel()
        distributed = dist.is_available() and dist.is_initialized()
        ns = self._mask_slices
        if ns <= 1 or numel == 0:
            bounds = [(0, numel)]
        else:
            base = numel // ns
            bounds = [(i * base, (i + 1) * base if i < ns - 1 else numel) for i in range(ns)]
        prev = None
        for lo, hi in bounds:
            msl = element_mask[lo:hi]
            sel = grad_data[lo:hi][msl]
            if scale_payload:
                sel *= factor_in
            if prev is not None:
                if prev[0] is not None:
                    prev[0].wait()
                grad_data[prev[1]:prev[2]][prev[3]] = prev[4]
            work = (dist.all_reduce(sel, op=reduce_op, group=comm_group, async_op=True)
                    if (distributed and sel.numel() > 0) else None)
            prev = (work, lo, hi, msl, sel)
        if prev is not None:
            if prev[0] is not None:
                prev[0].wait()
            grad_data[prev[1]:prev[2]][prev[3]] = prev[4]
        return None

    # ---------------------------------------------------------- rank local
    def configure_rank_local(self, max_bucket_elems: int, max_k: int) -> None:
        self._max_bucket = int(max_bucket_elems)

    def sync_rank_local(self, bs, k: int, mask_view, comm_group, world: int) -> None:
        """Per-rank exact top-``k`` mask, OR across ranks, reduction (mean) of the
        union's entries in place in the bucket; ``mask_view`` receives the
        union as uint8."""
        with backend_timer.region("sparse", backend=self.name, layout="mask", block_size=None, bucket=bs.bucket_id,
                                  k=k):
            grad = bs.grad_data
            if self.transport == "p2p" or (grad.is_cuda and self.ddp is not None and self.ddp.channels):
                from ..parallel import p2p

                ddp = self.ddp
                self._ensure_bits()
                if self._scratch is None:
                    self._scratch = p2p.IndexSyncScratch(ddp.device, self._max_bucket)
                ch = ddp.channels[bs.bucket_id % len(ddp.channels)]
                woff = 4 * self._word_off(bs)
                nw = (grad.numel() + 31) // 32
                p2p.bucket_index_sync_(ch, self._scratch, grad, k, bits=self._bits.view(torch.int32, woff, nw),
                                       select_only=True, max_ctas=ddp.ddp_config.comm_max_ctas)
                p2p.mask_union_reduce_(ch, ddp.arena.symm_grad, 4 * bs.arena_start, self._bits, woff, self._ubits,
                                       woff, grad.numel(), scale=1.0 / ddp.world, mask_u8=mask_view,
                                       sumsq_out=self.sumsq, accumulate=True, count_out=self.union_count,
                                       max_ctas=ddp.ddp_config.comm_max_ctas)
                return
            mask = KT.topk_rank_local(grad.abs(), k)
            if world > 1 and dist.is_initialized():
                dist.all_reduce(mask, op=dist.ReduceOp.MAX, group=comm_group)
            on = mask > 0
            sel = grad[on]
            if world > 1 and dist.is_initialized():
                dist.all_reduce(sel, op=dist.ReduceOp.SUM, group=comm_group)
            grad[on] = sel * (1.0 / world)
            mask_view.copy_(mask)

