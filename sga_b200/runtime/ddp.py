"""Data-parallel model chunk: the bucketed fp32 gradient arena plus the dense
gradient synchronisation, with per-bucket overlap against the backward pass.

``DataParallel`` is what the engine attaches to (the role Megatron's DDP
wrapper plays for the reference, ``sga/engine.py:318-396``). It owns

* the transport: ``p2p`` (fused CUDA kernels over peer-mapped memory),
  ``nccl`` / ``gloo`` (library collectives through ``torch.distributed``; the
  baseline arm and the CPU path) or ``local`` (one rank);
* a communication stream; a bucket is synchronised there as soon as the model
  reports its last parameter, gated on an event recorded on the compute stream;
* ``finish_grad_sync``: the stock dense all-reduce (average) of every bucket.

The engine installs ``bucket_sync_fn`` for the last micro-batch of a step; the
default is the dense all-reduce.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from .arena import Bucket, FlatArena


class DDPConfig:
    def __init__(self, average_in_collective: bool = True, overlap_grad_reduce: bool = True,
                 comm_max_ctas: int = 0):
        self.average_in_collective = average_in_collective
        self.overlap_grad_reduce = overlap_grad_reduce
        self.comm_max_ctas = comm_max_ctas
        self.use_distributed_optimizer = False
        # dense all-reduce through the NVSwitch's in-switch reduction where the gradient buffer is bound to
        # a multicast object (parallel.symm.McastPool); off unless asked for
        self.nvls_dense = False


class DataParallel:
    def __init__(self, model, *, group=None, transport: str = "auto", ddp_config: Optional[DDPConfig] = None,
                 pool=None):
        self.module = model
        self.arena: FlatArena = model.arena
        self.group = group
        self.ddp_config = ddp_config or DDPConfig()
        self.device = self.arena.device
        if dist.is_available() and dist.is_initialized():
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        cuda = self.device.type == "cuda"
        if transport == "auto":
            if self.world == 1:
                transport = "p2p" if (cuda and pool is not None) else "local"
            elif cuda and pool is not None:
                transport = "p2p"
            else:
                transport = "nccl" if cuda else "gloo"
        if transport == "p2p" and (not cuda or pool is None or self.arena.symm_grad is None):
            raise ValueError("transport 'p2p' needs CUDA and a symmetric memory pool")
        self.transport = transport
        self.pool = pool
        self.gradient_scaling_factor = 1.0 / self.world
        self.channels = []
        self.comm_stream = None
        if cuda:
            # high priority: a bucket's short synchronisation kernels take the SM resources that the
            # long GEMMs of the backward pass leave free as soon as they are launched
            self.comm_stream = torch.cuda.Stream(device=self.device, priority=-1)
        if transport == "p2p":
            from ..parallel.p2p import PeerChannel

            # one channel (flag words, receive slots of the backends) per bucket: a bucket's exchange can
            # then stay open until the end of the backward pass without blocking the next bucket's
            self.channels = [PeerChannel(pool) for _ in range(max(2, len(self.arena.buckets)))]
        # per-step overlap state
        self._pending = {}
        self._synced = set()
        self.bucket_sync_fn: Optional[Callable[[Bucket], None]] = None
        self.after_last_bucket: Optional[Callable[[], None]] = None  # runs on the comm stream once every bucket
        #                                                              of the step has been launched (deferred work)
        self._armed = False
        self._slot_bucket = {id(s): s.bucket for s in self.arena.slots}
        self._bucket_nparams = [len(b.slots) for b in self.arena.buckets]
        self.sync_launches = 0
        self.null_sync = False   # measurement switch: skip the buckets' synchronisation work (see bench.py)

    # ------------------------------------------------------- structure
    @property
    def buckets(self):
        return self.arena.buckets

    def channel_for(self, bucket: Bucket):
        return self.channels[bucket.index % len(self.channels)]

    def named_parameters(self):
        return self.module.named_parameters()

    # ------------------------------------------------- overlap plumbing
    def arm(self, sync_fn: Optional[Callable[[Bucket], None]] = None) -> None:
        """Arm per-bucket synchronisation for the coming backward pass (the last
        micro-batch of a step)."""
        self._pending = {b.index: n for b, n in zip(self.arena.buckets, self._bucket_nparams)}
        self._synced = set()
        self.bucket_sync_fn = sync_fn or self._dense_bucket_sync
        self._armed = self.ddp_config.overlap_grad_reduce

    def disarm(self) -> None:
        self._armed = False

    def on_param_done(self, slot) -> None:
        """Called by the model when ``slot``'s gradient is final for this step."""
        if not self._armed:
            return
        b = self._slot_bucket[id(slot)]
        self._pending[b] -= 1
        if self._pending[b] == 0:
            self._launch_bucket(self.arena.buckets[b])

    def _launch_bucket(self, bucket: Bucket) -> None:
        if bucket.index in self._synced:
            return
        self._synced.add(bucket.index)
        if self.null_sync:
            return
        timed = getattr(self, "time_syncs", False) and self.device.type == "cuda"
        if self.comm_stream is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.comm_stream.wait_event(ev)
            with torch.cuda.stream(self.comm_stream):
                pair = self._timed_pair() if timed else None
                self.bucket_sync_fn(bucket)
                if pair is not None:
                    pair[1].record()
        else:
            pair = self._timed_pair() if timed else None
            self.bucket_sync_fn(bucket)
            if pair is not None:
                pair[1].record()
        self.sync_launches += 1

    def _timed_pair(self):
        """Event pair around one bucket's synchronisation on the stream it runs on (``time_syncs``)."""
        pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        pair[0].record()
        if not hasattr(self, "_sync_events"):
            self._sync_events = []
        self._sync_events.append(pair)
        return pair

    def sync_device_ms(self) -> float:
        """Sum of the device time of the bucket synchronisations recorded since the last call
        (their own kernels and library collectives; overlapped with the backward pass in a step)."""
        torch.cuda.synchronize(self.device)
        total = sum(a.elapsed_time(b) for a, b in getattr(self, "_sync_events", []))
        self._sync_events = []
        return float(total)

    def finish_pending(self) -> None:
        """Synchronise every bucket not yet launched and join the comm stream."""
        fn = self.bucket_sync_fn or self._dense_bucket_sync
        self.bucket_sync_fn = fn
        for b in self.arena.buckets:
            if b.index not in self._synced:
                self._launch_bucket(b)
        self._run_deferred()
        self.join()
        self._armed = False

    def _run_deferred(self) -> None:
        fn, self.after_last_bucket = self.after_last_bucket, None
        if fn is None or self.null_sync:
            return
        timed = getattr(self, "time_syncs", False) and self.device.type == "cuda"
        if self.comm_stream is not None:
            with torch.cuda.stream(self.comm_stream):
                pair = self._timed_pair() if timed else None
                fn()
                if pair is not None:
                    pair[1].record()
        else:
            fn()

    def join(self) -> None:
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)

    # -------------------------------------------------------- dense sync
    def _dense_bucket_sync(self, bucket: Bucket) -> None:
        g = self.arena.main_grad[bucket.start:bucket.end]
        if self.transport == "p2p":
            from ..parallel import p2p

            ch, buf = self.channel_for(bucket), self.arena.symm_grad
            if not (self.ddp_config.nvls_dense and p2p.nvls_allreduce_(
                    ch, buf, 4 * bucket.start, bucket.numel, scale=self.gradient_scaling_factor,
                    max_ctas=self.ddp_config.comm_max_ctas)):
                p2p.allreduce_(ch, buf, 4 * bucket.start, bucket.numel, scale=self.gradient_scaling_factor,
                               max_ctas=self.ddp_config.comm_max_ctas)
        elif self.transport in ("nccl", "gloo"):
            if self.ddp_config.average_in_collective and self.transport == "nccl":
                dist.all_reduce(g, op=dist.ReduceOp.AVG, group=self.group)
            else:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)
                g.mul_(self.gradient_scaling_factor)
        # local: nothing to do

    def finish_grad_sync(self, force_all_reduce: bool = False) -> None:
        """Dense average of every bucket (buckets already launched by the overlap are skipped)."""
        if not self._synced and not self._armed:
            self._synced = set()
        self.bucket_sync_fn = self._dense_bucket_sync
        for b in self.arena.buckets:
            if b.index not in self._synced:
                self._launch_bucket(b)
        self.join()
        self._armed = False

    def begin_step(self) -> None:
        self.after_last_bucket = None
        self._synced = set()
        self._pending = {}
        self._armed = False

    def check(self) -> None:
        for ch in self.channels:
            ch.check()
