"""Tensor parallelism with sequence-parallel activations.

Outside the linear layers every activation is sharded by rows (tokens) over
the tensor-parallel ranks; a column-parallel linear gathers its input rows and
a row-parallel linear reduce-scatters its output rows. On B200 both run as one
kernel each (``csrc/gemm_tp.cu``): the CTA-pair tcgen05 GEMM pulls the peers'
row chunks over NVLink while it computes the tiles of its own chunk
(all-gather -> GEMM), or stores the partial tiles of the peers' chunks straight
into their receive slots while it computes its own chunk last and adds what the
peers sent (GEMM -> reduce-scatter).

Three transports behind one interface:

* ``fused``   the kernels above (CUDA, one NVSwitch domain, shapes with
  ``rows % (256 * tp) == 0``; anything else falls through to ``library``);
* ``library`` NCCL all-gather / reduce-scatter around the plain GEMM (the
  baseline the fused kernels are measured against);
* CPU tensors: gloo collectives around fp32 matmuls (tests of the host logic).

The reference refuses tensor parallelism for sparse steps
(``sga/runtime.py:50-52``) because gradients of parameters that are replicated
over the tensor-parallel group (norm weights under sequence parallelism) are
summed over that group after the data-parallel machinery has run. Here
``allreduce_replicated`` sums them *before* the gradient becomes final for the
data-parallel layer, so residual accounting only ever sees final gradients.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist


class GatherSlot:
    """An ``[rows, cols]`` bf16 buffer whose row chunk ``r`` is produced by rank
    ``r``. ``local`` is this rank's chunk (write the producer's output there),
    ``full`` the whole buffer, complete after ``ag_linear`` has run on it."""

    def __init__(self, full: torch.Tensor, rank: int, world: int, symm=None, offset_bytes: int = 0):
        self.full = full
        rows = full.shape[0] // world
        self.local = full[rank * rows:(rank + 1) * rows]
        self.symm = symm
        self.offset_bytes = offset_bytes
        self.gathered = False

    def ptr_array(self):
        return self.symm.ptr_array(self.offset_bytes)


class TPContext:
    def __init__(self, group=None, device="cpu", transport: str = "auto", wait_cycles: int = 0,
                 max_ctas: int = 0):
        self.group = group
        self.device = torch.device(device)
        if dist.is_available() and dist.is_initialized():
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        cuda = self.device.type == "cuda"
        if transport == "auto":
            transport = "fused" if cuda and self.world > 1 else "library"
        if transport == "fused" and not cuda:
            raise ValueError("the fused tensor-parallel kernels need a CUDA device")
        self.transport = transport
        self.max_ctas = max_ctas
        self.slots: dict = {}
        self.launches = 0
        self.pool = self.ag_channel = self.rs_channel = None
        self._recv = self._tflag = None
        self._recv_elems = self._tflag_ints = 0
        self._ready = None
        if transport == "fused":
            from .p2p import PeerChannel
            from .symm import SymmPool

            self.pool = SymmPool(group=group, device=self.device)
            self.ag_channel = PeerChannel(self.pool, wait_cycles)
            self.rs_channel = PeerChannel(self.pool, wait_cycles)
            self._ready = torch.zeros(4096, dtype=torch.int32, device=self.device)

    # ---------------------------------------------------------------- slots
    def slot(self, tag, rows: int, cols: int) -> GatherSlot:
        """The gather buffer registered under ``tag`` (allocated on first use; every
        rank of the group must ask for its slots in the same order)."""
        key = (tag, rows, cols)
        s = self.slots.get(key)
        if s is None:
            assert rows % self.world == 0, "token count must divide over the tensor-parallel ranks"
            if self.transport == "fused":
                buf = self.pool.alloc(rows * cols * 2)
                full = buf.view(torch.bfloat16, 0, rows * cols).view(rows, cols)
                s = GatherSlot(full, self.rank, self.world, buf, 0)
            else:
                s = GatherSlot(torch.empty(rows, cols, dtype=torch.bfloat16, device=self.device), self.rank,
                               self.world)
            self.slots[key] = s
        return s

    def _fusable(self, rows: int, k: int = 32, n: int = 32) -> bool:
        return self.transport == "fused" and rows % (256 * self.world) == 0 and k % 32 == 0 and n % 32 == 0

    # ------------------------------------------------------- gather -> GEMM
    def gather(self, slot: GatherSlot) -> torch.Tensor:
        """Plain all-gather of the slot (library collective)."""
        if self.world > 1:
            if self.device.type == "cuda":
                dist.all_gather_into_tensor(slot.full, slot.local.contiguous(), group=self.group)
            else:
                parts = [torch.empty_like(slot.local) for _ in range(self.world)]
                dist.all_gather(parts, slot.local.contiguous(), group=self.group)
                slot.full.copy_(torch.cat(parts, 0))
        return slot.full

    def ag_linear(self, slot: GatherSlot, W: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
        """``gather_rows(slot) @ W^T`` (``W: [N, K]``), or ``@ W`` with ``b_mn``
        (``W: [K, N]``). Leaves the gathered rows in ``slot.full``."""
        M, K = slot.full.shape
        N = W.shape[1] if b_mn else W.shape[0]
        if self.device.type != "cuda":
            full = self.gather(slot).float()
            y = full @ (W.float() if b_mn else W.float().t())
            return y.to(torch.bfloat16)
        from .. import kernels as Kn

        out = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
        if self.world > 1 and self._fusable(M, K):
            from ..csrc import lib
            from ..kernels import _chk, _st

            nblk = M // 256
            if self._ready.numel() < nblk:
                self._ready = torch.zeros(nblk, dtype=torch.int32, device=self.device)
            self._ready[:nblk].zero_()
            d = self.ag_channel.next_desc()
            rc = lib().sga_tp_ag_gemm(ctypes.byref(d), slot.ptr_array(), W.data_ptr(), out.data_ptr(), M, N, K,
                                      int(b_mn), W.stride(0), N, Kn.EPI_BF16, 1.0, self._ready.data_ptr(),
                                      self.max_ctas, _st())
            _chk(rc, "sga_tp_ag_gemm")
            self.launches += 1
            return out
        self.gather(slot)
        self.launches += 1
        return Kn.gemm_bf16(slot.full, W, out, b_mn=b_mn)

    # ------------------------------------------------ GEMM -> reduce-scatter
    def _rs_buffers(self, rows_pc: int, N: int, tiles: int):
        need = self.world * rows_pc * N
        if self._recv is None or self._recv_elems < need:
            self._recv = self.pool.alloc(need * 2)
            self._recv_elems = need
        need_f = self.world * tiles * 8
        if self._tflag is None or self._tflag_ints < need_f:
            self._tflag = self.pool.alloc(need_f * 4)
            self._tflag.raw.zero_()
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
            self._tflag_ints = need_f
        return self._recv, self._tflag

    def linear_rs(self, a: torch.Tensor, W: torch.Tensor, b_mn: bool = False,
                  residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Rows ``[rank * M/tp, (rank+1) * M/tp)`` of ``sum over ranks (a @ W^T)``
        (``W: [N, K]``; ``a @ W`` with ``b_mn``, ``W: [K, N]``), plus ``residual``."""
        M, K = a.shape
        N = W.shape[1] if b_mn else W.shape[0]
        rows_pc = M // self.world
        lo = self.rank * rows_pc
        if self.device.type != "cuda":
            y = a.float() @ (W.float() if b_mn else W.float().t())
            if self.world > 1:
                dist.all_reduce(y, group=self.group)
            y = y[lo:lo + rows_pc]
            if residual is not None:
                y = y + residual.float()
            return y.to(torch.bfloat16)
        from .. import kernels as Kn

        if self.world > 1 and self._fusable(M, 32, N):
            from ..csrc import lib
            from ..kernels import _chk, _p, _st

            tiles = (rows_pc // 256) * ((N + 255) // 256)
            recv, tflag = self._rs_buffers(rows_pc, N, tiles)
            out = torch.empty(rows_pc, N, dtype=torch.bfloat16, device=self.device)
            d = self.rs_channel.next_desc()
            rc = lib().sga_tp_gemm_rs(ctypes.byref(d), a.data_ptr(), W.data_ptr(), out.data_ptr(), _p(residual),
                                      recv.ptr_array(0), tflag.ptr_array(0), M, N, K, 0, int(b_mn), a.stride(0),
                                      W.stride(0), N, Kn.EPI_BF16_ADD if residual is not None else Kn.EPI_BF16,
                                      1.0, self.max_ctas, _st())
            _chk(rc, "sga_tp_gemm_rs")
            self.launches += 1
            return out
        part = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
        Kn.gemm_bf16(a, W, part, b_mn=b_mn)
        self.launches += 1
        if self.world == 1:
            out = part
        else:
            out = torch.empty(rows_pc, N, dtype=torch.bfloat16, device=self.device)
            dist.reduce_scatter_tensor(out, part, group=self.group)
        if residual is not None:
            out += residual
        return out

    # ------------------------------------------------------------- scalars
    def allreduce_replicated(self, grad: torch.Tensor) -> None:
        """Sum over the group of a gradient whose parameter every rank holds."""
        if self.world > 1:
            dist.all_reduce(grad, group=self.group)

    def allreduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def allreduce_(self, t: torch.Tensor, op=None) -> torch.Tensor:
        """In-place all-reduce over the group (sum by default)."""
        if self.world > 1:
            dist.all_reduce(t, op=op if op is not None else dist.ReduceOp.SUM, group=self.group)
        return t

    def reduce_scatter_rows(self, full: torch.Tensor) -> torch.Tensor:
        """Sum of ``full`` ``[rows, cols]`` over the group; this rank keeps its row chunk. Library
        collective (the vocabulary-parallel embedding and output layer use it twice per micro-batch)."""
        if self.world == 1:
            return full
        rows = full.shape[0] // self.world
        if full.is_cuda:
            out = torch.empty(rows, full.shape[1], dtype=full.dtype, device=full.device)
            dist.reduce_scatter_tensor(out, full.contiguous(), group=self.group)
            return out
        acc = full.float()   # gloo: no reduce-scatter, and sums in fp32
        dist.all_reduce(acc, group=self.group)
        return acc[self.rank * rows:(self.rank + 1) * rows].to(full.dtype)

    def check(self) -> None:
        for ch, what in ((self.ag_channel, "all-gather GEMM"), (self.rs_channel, "GEMM reduce-scatter")):
            if ch is not None:
                ch.check(what)

    def close(self) -> None:
        if self.pool is not None:
            self.pool.close()
            self.pool = None
