"""Index-form sparse all-reduce backend.

Shared-support mode (every rank holds the same sorted index list for the
cycle): only values cross the wire.

* ``p2p`` transport: one fused kernel per bucket packs ``grad[idx] * factor``
  into this rank's symmetric payload region, reduces its owned slice of the
  payload from every peer in rank order, writes the result to every peer,
  scatters the reduced values back into the dense bucket and accumulates the
  squared norm of the payload (``csrc/p2p_sync.cu``).
* ``nccl`` / ``gloo`` transport: pack -> async all-reduce -> scatter,
  pipelined over ``index_slices`` slices (the library baseline; also the CPU
  path), with an optional twin high-priority NCCL group.

``emission`` only decides what the call returns: ``compact`` hands back the
view of the reduced values (the engine computes the deterministic compact
norm from it and the trace collector reads it), ``writeback`` returns
``None``. In both cases the reduced values are also present in the dense
bucket at the support positions, which is where the optimizer kernel reads
them. ``layout bb`` moves whole blocks (mask-guarded lanes).

Rank-local mode (``sga_selection_locality rank_local``): ``sync_rank_local``
runs the fused select + (index, value) exchange + scatter-add kernel.

Contract and knobs follow ``sga/backends/torch_pipelined_index.py:103-520``.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import kernels_torch as KT
from ..config import get_args
from ..plugins import resolve_emission
from ..utils import backend_timer


def _ops(t):
    if t.is_cuda:
        from .. import kernels as K

        return K
    return KT


_DEBUG_SYNC = os.environ.get("SGA_ISYNC_DEBUG", "0") == "1"


def _score_abs(grad, score):
    """|score| of every bucket coordinate with the registry formulas (library / CPU path)."""
    if score is None or score.name == "abs_g":
        return grad.abs()
    from ..plugins.scores import compute_score

    out = torch.empty_like(grad)
    starts = score.span_start.tolist() if score.span_start is not None else [0, grad.numel()]
    wds = score.span_wd.tolist() if score.span_wd is not None else [0.0]
    for (s, e), wd in zip(zip(starts[:-1], starts[1:]), wds):
        out[s:e] = compute_score(score.name, score.w[s:e], score.m[s:e], score.v[s:e], grad[s:e],
                                 beta1=score.beta1, beta2=score.beta2, eps=score.eps, weight_decay=wd,
                                 bc1=score.bc1, bc2=score.bc2,
                                 optimizer="adams" if score.adams else "adamw").abs()
    return out


class TorchPipelinedIndexBackend:
    consumes = "idx"
    inherent_emission = "compact"
    block_form = "block_idx"
    name = "torch_pipelined_index"

    def __init__(self):
        args = get_args()
        emission = args.sga_backend_emission
        if emission not in (None, "auto", "compact", "writeback"):
            raise ValueError(f"sga_backend_emission must be auto|compact|writeback (got {emission!r})")
        self.emission = resolve_emission(emission, self.inherent_emission)
        self.layout = args.sga_backend_layout
        self._hiprio = bool(args.sga_backend_high_priority_group)
        s = args.sga_backend_index_slices
        if not isinstance(s, int) or isinstance(s, bool) or s < 1:
            raise ValueError(f"index_slices must be an int >= 1, got {s!r}")
        self._slices = s
        self._gather_bufs: dict = {}
        self._twins: dict = {}
        self.ddp = None            # bound by the engine at attach (transport, pool, channels)
        self._payload = None       # symmetric payload arena (p2p)
        self._payload_off: dict = {}
        self._slots = {}           # rank-local receive slots per channel
        self._scratch = None
        self._deferred = []        # tokens of buckets whose receive side is still to run this step
        self._touched = None
        self.sumsq = None          # device scalar: norm^2 of the payloads reduced this step

    # --------------------------------------------------------- set-up
    def bind(self, ddp) -> None:
        self.ddp = ddp
        if ddp.device.type == "cuda":
            self.sumsq = torch.zeros(1, dtype=torch.float32, device=ddp.device)

    @property
    def transport(self) -> str:
        return self.ddp.transport if self.ddp is not None else "gloo"

    def prepare(self, comm_group, device=None) -> None:
        """Twin high-priority NCCL group (library transport only), created and
        warmed eagerly so that no communicator set-up lands inside a step."""
        if not self._hiprio or comm_group is None or comm_group in self._twins or self.transport == "p2p":
            return
        if dist.is_available() and dist.is_initialized() and dist.get_backend(comm_group) == "nccl":
            from torch.distributed import ProcessGroupNCCL

            dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
            opts = ProcessGroupNCCL.Options()
            opts.is_high_priority_stream = True
            twin = dist.new_group(ranks=dist.get_process_group_ranks(comm_group), backend="nccl", pg_options=opts)
            warm = torch.zeros(8 << 20, dtype=torch.float32, device=dev)
            dist.all_reduce(warm, group=twin)
            dist.all_reduce(warm[:1], group=twin)
            torch.cuda.synchronize(dev)
            self._twins[comm_group] = twin

    def validate_runtime(self, args) -> None:
        return None

    def on_support_activated(self, support, bucket_states) -> None:
        """Size the symmetric payload arena for the new cycle (collective: every
        rank holds the same support, hence the same sizes)."""
        if self.transport != "p2p":
            return
        offs, total = {}, 0
        for bs, sup in zip(bucket_states, support.buckets):
            k = sup.num_selected() if self._layout_for(sup) != "bb" else sup.block_idx.numel() * sup.block_size
            offs[id(bs)] = total
            total += (k + 63) // 64 * 64
        self._payload_off = offs
        need = 4 * max(total, 64)
        if self._payload is None or self._payload.nbytes < need:
            self._payload = self.ddp.pool.alloc(need + need // 4)

    def _layout_for(self, support):
        layout = self.layout
        if layout in (None, "auto"):
            layout = "er" if support.block_size == 1 else "bb"
        return layout

    def _group_for(self, comm_group):
        if comm_group is None:
            return None
        return self._twins.get(comm_group, comm_group)

    def _gather_buf(self, key, k, dtype, device):
        buf = self._gather_bufs.get(key)
        cap = -(-k // (4 << 20)) * (4 << 20)
        if buf is None or buf.dtype != dtype or buf.device != device or buf.numel() < cap:
            buf = torch.empty(max(cap, buf.numel() if buf is not None else 0), dtype=dtype, device=device)
            self._gather_bufs[key] = buf
        return buf

    def _bounds(self, support, k):
        if not self._hiprio and self._slices == 2:
            n0 = support.split
            return [(0, n0), (n0, k)]
        s = self._slices
        return [(i * k // s, (i + 1) * k // s) for i in range(s)]

    # ------------------------------------------------------ shared support
    def allreduce_sparse(self, grad_data, support, comm_group, gradient_scaling_factor, reduce_op, key,
                         bucket_state=None):
        with backend_timer.region("sparse", backend=self.name, emission=self.emission, layout=self.layout,
                                  block_size=getattr(support, "block_size", None), bucket=key,
                                  k=getattr(support, "n_selected", None)):
            return self._impl(grad_data, support, comm_group, gradient_scaling_factor, reduce_op, key, bucket_state)

    def _impl(self, grad_data, support, comm_group, factor_in, reduce_op, key, bucket_state):
        if grad_data.numel() >= 2 ** 31:
            raise ValueError(f"int32 support indices assume < 2^31 bucket elements, got {grad_data.numel()}")
        avg = reduce_op == dist.ReduceOp.AVG
        factor = float(factor_in) if (reduce_op == dist.ReduceOp.SUM and factor_in != 1.0) else 1.0
        layout = self._layout_for(support)
        if layout == "bb":
            if self.emission != "writeback":
                raise ValueError("torch_pipelined_index: layout bb runs writeback emission only")
            if support.block_size == 1:
                raise ValueError("torch_pipelined_index: the block path needs block_size > 1")
            return self._block(grad_data, support, comm_group, factor, reduce_op, key, bucket_state)
        idx = support.idx
        k = idx.numel()
        if k == 0:
            return None if self.emission == "writeback" else torch.empty(0, dtype=grad_data.dtype,
                                                                         device=grad_data.device)
        if self.transport == "p2p":
            from ..parallel import p2p

            ddp = self.ddp
            off = 4 * self._payload_off[id(bucket_state)]
            world = ddp.world
            scale = (1.0 / world) if avg else 1.0
            p2p.allreduce_(ddp.channels[key % len(ddp.channels)] if isinstance(key, int) else ddp.channels[0],
                           self._payload, off, k, scale=scale, grad=grad_data, idx=idx, factor=factor, pack=True,
                           zero_after_pack=False, scatter=True, sumsq_out=self.sumsq, accumulate=True,
                           max_ctas=ddp.ddp_config.comm_max_ctas)
            vals = self._payload.view(torch.float32, off, k)
            return vals if self.emission == "compact" else None
        ops = _ops(grad_data)
        group = self._group_for(comm_group)
        buf = self._gather_buf(key, k, grad_data.dtype, grad_data.device)
        distributed = dist.is_available() and dist.is_initialized()
        prev = None
        for lo, hi in self._bounds(support, k):
            if hi <= lo:
                continue
            sl_idx, sel = idx[lo:hi], buf[lo:hi]
            ops.pack_selected(grad_data, sl_idx, sel, factor, zero=False)
            if prev is not None:
                if prev[0] is not None:
                    prev[0].wait()
                ops.scatter_selected(grad_data, prev[1], prev[2])
            work = dist.all_reduce(sel, op=reduce_op, group=group, async_op=True) if distributed else None
            prev = (work, sl_idx, sel)
        if prev is not None:
            if prev[0] is not None:
                prev[0].wait()
            ops.scatter_selected(grad_data, prev[1], prev[2])
        return buf[:k] if self.emission == "compact" else None

    def _block(self, grad_data, support, comm_group, factor, reduce_op, key, bucket_state):
        x = int(support.block_size)
        blk = support.block_idx
        kb = blk.numel()
        if kb == 0:
            return None
        ops = _ops(grad_data)
        if self.transport == "p2p":
            from ..parallel import p2p

            ddp = self.ddp
            off = 4 * self._payload_off[id(bucket_state)]
            vals = self._payload.view(torch.float32, off, kb * x)
            ops.gather_selected_blocks(grad_data, support.mask_u8, blk, x, vals, factor, zero=False)
            scale = (1.0 / ddp.world) if reduce_op == dist.ReduceOp.AVG else 1.0
            p2p.allreduce_(ddp.channels[key % len(ddp.channels)] if isinstance(key, int) else ddp.channels[0],
                           self._payload, off, kb * x, scale=scale, sumsq_out=self.sumsq, accumulate=True,
                           max_ctas=ddp.ddp_config.comm_max_ctas)
            ops.scatter_selected_blocks(grad_data, support.mask_u8, blk, x, vals)
            return None
        group = self._group_for(comm_group)
        buf = self._gather_buf(key, kb * x, grad_data.dtype, grad_data.device)
        if not self._hiprio and self._slices == 2:
            n0 = support.block_split
            bounds = [(0, n0), (n0, kb)]
        else:
            s = self._slices
            bounds = [(i * kb // s, (i + 1) * kb // s) for i in range(s)]
        distributed = dist.is_available() and dist.is_initialized()
        prev = None
        for lo, hi in bounds:
            if hi <= lo:
                continue
            bidx, sel = blk[lo:hi], buf[lo * x:hi * x]
            ops.gather_selected_blocks(grad_data, support.mask_u8, bidx, x, sel, factor, zero=False)
            if prev is not None:
                if prev[0] is not None:
                    prev[0].wait()
                ops.scatter_selected_blocks(grad_data, support.mask_u8, prev[1], x, prev[2])
            work = dist.all_reduce(sel, op=reduce_op, group=group, async_op=True) if distributed else None
            prev = (work, bidx, sel)
        if prev is not None:
            if prev[0] is not None:
                prev[0].wait()
            ops.scatter_selected_blocks(grad_data, support.mask_u8, prev[1], x, prev[2])
        return None

    # ---------------------------------------------------------- rank local
    def sync_rank_local(self, bucket_state, k: int, comm_view, comm_group, world: int, score=None,
                        defer_reduce: bool = False) -> None:
        """Exact per-bucket top-``k`` of the score (``None``: ``|grad + residual|``; otherwise a
        ``ScoreInputs`` with the bucket's weights, moments and Adam scalars) on this rank, exchange of
        (int32 index, fp32 value) pairs, rank-ordered sum / world into ``comm_view``; the selected
        coordinates of the bucket are zeroed. Coordinates with a zero score are never selected.
        ``defer_reduce`` (peer-memory transport): only select and push now; the receive side of every
        deferred bucket runs in ``flush_rank_local``, which the caller invokes once all buckets have
        been launched -- by then no rank has to wait for a slower peer's pairs."""
        with backend_timer.region("sparse", backend=self.name, emission="rank_local", layout="er", block_size=1,
                                  bucket=bucket_state.bucket_id, k=k):
            self._rank_local_impl(bucket_state, k, comm_view, comm_group, world, score, defer_reduce)

    def _rank_local_impl(self, bs, k, comm_view, comm_group, world, score=None, defer_reduce=False):
        grad = bs.grad_data
        n = grad.numel()
        if self.transport == "p2p" or (grad.is_cuda and world == 1 and self.ddp is not None and self.ddp.channels):
            from ..parallel import p2p

            ddp = self.ddp
            ci = bs.bucket_id % len(ddp.channels)
            ch = ddp.channels[ci]
            if ci not in self._slots:
                self._slots[ci] = p2p.IndexSyncSlots(ddp.pool, self._kcap, self._max_bucket)
            if self._scratch is None:
                self._scratch = p2p.IndexSyncScratch(ddp.device, self._max_bucket)
            token = p2p.bucket_index_sync_(ch, self._scratch, grad, k, slots=self._slots[ci], comm=comm_view,
                                           scale=1.0 / ddp.world, sumsq_out=self.sumsq, accumulate=True,
                                           score=score, max_ctas=ddp.ddp_config.comm_max_ctas,
                                           defer_reduce=defer_reduce and not _DEBUG_SYNC)
            if token is not None:
                self._deferred.append(token)
            if _DEBUG_SYNC:
                # debugging aid (SGA_ISYNC_DEBUG=1): stop at the first bucket whose chain reports an error
                torch.cuda.synchronize()
                code = int(ch.err.item())
                if code:
                    raise RuntimeError(f"index sync of bucket {bs.bucket_id} (n={n}, k={k}) set status {code}; "
                                       f"state words {self._scratch.state[:16].tolist()}")
            return
        # library / CPU path: same arithmetic, rank-ordered
        mask = KT.topk_rank_local(_score_abs(grad, score), k)
        idx = KT.compact_mask_idx(mask)
        vals = grad[idx.long()].clone()
        grad[idx.long()] = 0.0
        scale = 1.0 / world
        if world > 1 and dist.is_initialized():
            all_idx = [torch.empty_like(idx) for _ in range(world)]
            all_val = [torch.empty_like(vals) for _ in range(world)]
            dist.all_gather(all_idx, idx, group=comm_group)
            dist.all_gather(all_val, vals, group=comm_group)
        else:
            all_idx, all_val = [idx], [vals]
        for ri, rv in zip(all_idx, all_val):
            comm_view.index_add_(0, ri.long(), rv * scale)

    def flush_rank_local(self) -> None:
        """Receive side of every bucket whose push was deferred, in launch order."""
        from ..parallel import p2p

        pending, self._deferred = self._deferred, []
        for token in pending:
            p2p.bucket_index_reduce_(token)

    def configure_rank_local(self, max_bucket_elems: int, max_k: int) -> None:
        """Sizes of the largest bucket and payload; the receive areas of both channels and the work
        memory of the top-k chain are allocated here, at attach, so that no step allocates."""
        self._max_bucket = int(max_bucket_elems)
        self._kcap = int(max_k)
        ddp = self.ddp
        if ddp is not None and ddp.channels and ddp.device.type == "cuda":
            from ..parallel import p2p

            for ci in range(len(ddp.channels)):
                if ci not in self._slots:
                    self._slots[ci] = p2p.IndexSyncSlots(ddp.pool, self._kcap, self._max_bucket)
            if self._scratch is None:
                self._scratch = p2p.IndexSyncScratch(ddp.device, self._max_bucket)
            torch.cuda.synchronize(ddp.device)
