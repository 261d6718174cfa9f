"""Flat parameter arena and gradient buckets.

All parameters of a model live in five flat arrays with one shared layout:

  model_param  bf16   what the forward / backward kernels read
  main_param   fp32   master weights
  main_grad    fp32   gradient accumulator; under SGA this buffer *is* the
                      residual (unselected coordinates simply stay in it)
  exp_avg      fp32   Adam first moment
  exp_avg_sq   fp32   Adam second moment

Parameters are laid out in the order their gradients become final during the
backward pass, cut into buckets of about ``bucket_elems`` elements at
parameter boundaries, so bucket ``b`` can be synchronised while the backward
pass is still producing bucket ``b + 1``. ``main_grad`` and ``model_param``
are allocated from symmetric (peer-mapped) memory when a pool is given, which
is what lets the sync kernels read and write other ranks' copies directly.

The reference reaches the equivalent structure through Megatron's DDP bucket
groups (``sga/engine.py:318-396`` walks them); here the framework owns it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

ALIGN = 64  # every parameter starts on a 64-element boundary (256 B fp32, 128 B bf16)


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    group: int = 0            # hyper-parameter group (0 = weight decay, 1 = no weight decay)
    init: str = "normal"      # "normal" (std below) | "ones" | "zeros"
    std: float = 0.02
    tp_duplicate: bool = False  # replicated across tensor-parallel ranks (norm weights)
    tp_full_shape: Optional[tuple] = None  # a tensor-parallel shard: shape of the full tensor ...
    tp_pieces: Optional[list] = None       # ... and the (dim, lo, hi) slices of it, concatenated along dim
    init_order: Optional[int] = None       # position in the random-init stream when it differs from the layout order

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n


@dataclass
class ParamSlot:
    spec: ParamSpec
    start: int
    end: int
    bucket: int = -1
    model: Optional[torch.Tensor] = field(default=None, repr=False)   # bf16 view, spec.shape
    main: Optional[torch.Tensor] = field(default=None, repr=False)    # fp32 view
    grad: Optional[torch.Tensor] = field(default=None, repr=False)    # fp32 view

    @property
    def name(self):
        return self.spec.name


@dataclass
class Bucket:
    index: int
    start: int
    end: int
    slots: list = field(default_factory=list)

    @property
    def numel(self) -> int:
        return self.end - self.start

    def spans(self):
        """Parameter element spans relative to the bucket start."""
        return [(s.start - self.start, s.end - self.start) for s in self.slots]


class FlatArena:
    def __init__(self, specs, *, bucket_elems: int = 16 * 1024 * 1024, device="cpu", pool=None,
                 need_comm_staging: bool = False, split_on_tp_duplicate: bool = False):
        self.device = torch.device(device)
        self.pool = pool
        self.slots: list[ParamSlot] = []
        self.buckets: list[Bucket] = []
        off = 0
        cur = Bucket(0, 0, 0)
        for spec in specs:
            if split_on_tp_duplicate and cur.slots and cur.slots[-1].spec.tp_duplicate != spec.tp_duplicate:
                # a bucket holds either shards or replicated parameters, never both: a per-bucket selection
                # over replicated data is then the same on every tensor-parallel rank
                self.buckets.append(cur)
                cur = Bucket(cur.index + 1, off, off)
            n = spec.numel
            start = off
            end = start + n
            slot = ParamSlot(spec, start, end, bucket=cur.index)
            self.slots.append(slot)
            cur.slots.append(slot)
            off = (end + ALIGN - 1) // ALIGN * ALIGN
            cur.end = off
            if cur.end - cur.start >= bucket_elems:
                self.buckets.append(cur)
                cur = Bucket(cur.index + 1, off, off)
        if cur.slots:
            self.buckets.append(cur)
        self.numel = off
        self.by_name = {s.name: s for s in self.slots}
        n = self.numel
        cuda = self.device.type == "cuda"
        self.symm_grad = self.symm_model = None
        if cuda and pool is not None:
            self.symm_grad = pool.alloc(4 * n)
            self.symm_model = pool.alloc(2 * n)
            self.main_grad = self.symm_grad.view(torch.float32, 0, n)
            self.model_param = self.symm_model.view(torch.bfloat16, 0, n)
        else:
            self.main_grad = torch.zeros(n, dtype=torch.float32, device=self.device)
            self.model_param = torch.zeros(n, dtype=torch.bfloat16, device=self.device)
        self.main_param = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.comm = torch.zeros(n, dtype=torch.float32, device=self.device) if need_comm_staging else None
        for s in self.slots:
            s.model = self.model_param[s.start:s.end].view(s.spec.shape)
            s.main = self.main_param[s.start:s.end].view(s.spec.shape)
            s.grad = self.main_grad[s.start:s.end].view(s.spec.shape)
        self._table = None

    # ------------------------------------------------------------ init
    def init_parameters(self, seed: int = 0, on_device: bool = False) -> None:
        """Random init of the fp32 masters (same values on every data-parallel
        rank for a given seed), then the bf16 copies. ``on_device`` draws with
        the device's generator instead of the host's (fast for large models;
        the values then differ from a host-initialised run of the same seed)."""
        if on_device and self.device.type == "cuda":
            self._init_on_device(seed)
            self.sync_model_from_main()
            return
        # One generator per parameter, keyed by its place in the model's full parameter list: a shard or
        # a pipeline stage that holds only some parameters still draws the values of the whole model.
        order = sorted(range(len(self.slots)), key=lambda i: (
            self.slots[i].spec.init_order if self.slots[i].spec.init_order is not None else i))
        for i in order:
            s = self.slots[i]
            pos = s.spec.init_order if s.spec.init_order is not None else i
            gen = torch.Generator(device="cpu").manual_seed(seed * 1000003 + pos)
            if s.spec.init == "ones":
                s.main.fill_(1.0)
            elif s.spec.init == "zeros":
                s.main.zero_()
            else:
                # generated in chunks on the host: identical bits on CPU and GPU runs
                shape = s.spec.tp_full_shape if s.spec.tp_pieces is not None else s.spec.shape
                full = torch.empty(shape)
                flat = full.view(-1)
                step = 1 << 24
                for lo in range(0, flat.numel(), step):
                    hi = min(flat.numel(), lo + step)
                    flat[lo:hi].copy_(torch.randn(hi - lo, generator=gen) * s.spec.std)
                if s.spec.tp_pieces is not None:
                    dim = s.spec.tp_pieces[0][0]
                    full = torch.cat([full.narrow(dim, lo, hi - lo) for _, lo, hi in s.spec.tp_pieces], dim)
                s.main.copy_(full)
                del full
        self.sync_model_from_main()

    def _init_on_device(self, seed: int) -> None:
        order = sorted(range(len(self.slots)), key=lambda i: (
            self.slots[i].spec.init_order if self.slots[i].spec.init_order is not None else i))
        for i in order:
            s = self.slots[i]
            pos = s.spec.init_order if s.spec.init_order is not None else i
            if s.spec.init == "ones":
                s.main.fill_(1.0)
            elif s.spec.init == "zeros":
                s.main.zero_()
            else:
                # one generator per parameter, keyed by its place in the stream: a shard draws its full tensor
                gen = torch.Generator(device=self.device).manual_seed(seed * 1000003 + pos)
                shape = s.spec.tp_full_shape if s.spec.tp_pieces is not None else s.spec.shape
                full = torch.randn(shape, generator=gen, device=self.device) * s.spec.std
                if s.spec.tp_pieces is not None:
                    dim = s.spec.tp_pieces[0][0]
                    full = torch.cat([full.narrow(dim, lo, hi - lo) for _, lo, hi in s.spec.tp_pieces], dim)
                s.main.copy_(full)
                del full

    def sync_model_from_main(self) -> None:
        if self.device.type == "cuda":
            from .. import kernels as K

            K.cast_bf16(self.main_param, self.model_param)
        else:
            self.model_param.copy_(self.main_param)

    # --------------------------------------------------------- segments
    def segment_table(self):
        """Device table of (start, group) per parameter for the multi-tensor optimizer."""
        if self._table is None:
            starts, groups = [], []
            for s in self.slots:
                starts.append(s.start)
                groups.append(s.spec.group)
            if self.device.type == "cuda":
                from .. import kernels as K

                self._table = K.SegmentTable(starts, groups, self.numel, self.device)
            else:
                self._table = (starts, groups)
        return self._table

    def bucket_view(self, t: torch.Tensor, b: Bucket) -> torch.Tensor:
        return t[b.start:b.end]

    def zero_grad(self) -> None:
        self.main_grad.zero_()

    def state_dict_tensors(self):
        """name -> (w, m, v) fp32 views (torch-Adam layout source)."""
        out = {}
        for s in self.slots:
            sl = slice(s.start, s.end)
            out[s.name] = (self.main_param[sl].view(s.spec.shape), self.exp_avg[sl].view(s.spec.shape),
                           self.exp_avg_sq[sl].view(s.spec.shape))
        return out
