"""Host side of the fused peer-memory collectives (``csrc/p2p_sync.cu``,
``csrc/dense_sync.cu``).

A :class:`PeerChannel` owns what one in-flight collective needs: the
sequence-numbered flag words in symmetric memory, the grid-barrier counter,
the per-rank norm slots and the device status word. Launches on a channel
must be issued in the same order on every rank (they are: bucket order is
global). ``check()`` reads the status word on the host and raises on every
rank that saw a bounded wait expire.
"""
from __future__ import annotations

import ctypes

import torch

from ..csrc import lib
from ..kernels import _chk, _p, _st
from .symm import SymmBuffer, SymmPool

ERR_BITS = {1: "mbarrier wait expired", 2: "peer flag wait expired", 4: "grid barrier wait expired",
            8: "index outside the owned range", 16: "payload capacity exceeded"}


class PeerTimeout(RuntimeError):
    """A bounded device-side wait expired or a device-side check failed."""


class PeerDesc(ctypes.Structure):
    _fields_ = [("W", ctypes.c_int), ("rank", ctypes.c_int), ("flags", ctypes.c_void_p * 8),
                ("seq", ctypes.c_int), ("prev_seq", ctypes.c_int), ("grid_counter", ctypes.c_void_p),
                ("err", ctypes.c_void_p), ("wait_cycles", ctypes.c_longlong)]


class PeerChannel:
    def __init__(self, pool: SymmPool, wait_cycles: int = 0):
        self.pool = pool
        self.world, self.rank = pool.world, pool.rank
        self.device = pool.device
        # symmetric: int32 flags[16] at 0, float norm_slots[8] at 256
        self.ctrl: SymmBuffer = pool.alloc(512)
        self.grid_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.cta_partials = torch.zeros(2048, dtype=torch.float32, device=self.device)
        self.seq = 0
        self.wait_cycles = int(wait_cycles)

    def next_desc(self) -> PeerDesc:
        d = PeerDesc()
        d.W, d.rank = self.world, self.rank
        for r in range(self.world):
            d.flags[r] = self.ctrl.peer_ptrs[r]
        d.prev_seq = self.seq
        self.seq += 1
        d.seq = self.seq
        d.grid_counter = self.grid_counter.data_ptr()
        d.err = self.err.data_ptr()
        d.wait_cycles = self.wait_cycles
        return d

    def norm_slots(self):
        return self.ctrl.ptr_array(256)

    def check(self, what: str = "peer collective") -> None:
        code = int(self.err.item())
        if code:
            self.err.zero_()
            reasons = [msg for bit, msg in ERR_BITS.items() if code & bit]
            raise PeerTimeout(f"{what}: device status {code} ({'; '.join(reasons)}) on rank {self.rank}")


def _ptrs(bufs_or_buf, offset_bytes=0):
    return bufs_or_buf.ptr_array(offset_bytes)


def allreduce_(ch: PeerChannel, buf: SymmBuffer, offset_bytes: int, n: int, *, scale: float = 1.0, grad=None,
               idx=None, factor: float = 1.0, pack=False, zero_after_pack=False, scatter=False, rs_only=False,
               sumsq_out=None, accumulate=False, max_ctas: int = 0) -> None:
    """In-place two-shot all-reduce of ``n`` fp32 values at ``offset_bytes`` of a
    symmetric buffer, optionally fused with the pack of ``grad[idx]`` before
    and the scatter back after."""
    d = ch.next_desc()
    rc = lib().sga_p2p_allreduce(ctypes.byref(d), _ptrs(buf, offset_bytes), int(n), float(scale), _p(grad), _p(idx),
                                 float(factor), int(pack), int(zero_after_pack), int(scatter), int(rs_only),
                                 ch.norm_slots(), ch.cta_partials.data_ptr(), _p(sumsq_out), int(accumulate),
                                 max_ctas, _st())
    _chk(rc, "sga_p2p_allreduce")


def mask_union_reduce_(ch: PeerChannel, grad: SymmBuffer, grad_off: int, bits: SymmBuffer, bits_off: int,
                       ubits: SymmBuffer, ubits_off: int, n: int, *, scale: float = 1.0, mask_u8=None,
                       sumsq_out=None, accumulate=False, count_out=None, max_ctas: int = 0) -> None:
    d = ch.next_desc()
    rc = lib().sga_p2p_mask_union(ctypes.byref(d), _ptrs(grad, grad_off), _ptrs(bits, bits_off),
                                  _ptrs(ubits, ubits_off), int(n), float(scale), _p(mask_u8), ch.norm_slots(),
                                  ch.cta_partials.data_ptr(), _p(sumsq_out), int(accumulate), _p(count_out),
                                  max_ctas, _st())
    _chk(rc, "sga_p2p_mask_union")


class IndexSyncScratch:
    """Per-device scratch of the fused top-k kernel (histograms kept zero between launches)."""

    def __init__(self, device):
        self.hist1 = torch.zeros(32769, dtype=torch.int32, device=device)
        self.hist2 = torch.zeros(65536, dtype=torch.int32, device=device)
        self.cta_gt = torch.zeros(256, dtype=torch.int32, device=device)
        self.cta_eq = torch.zeros(256, dtype=torch.int32, device=device)
        self.result = torch.zeros(4, dtype=torch.int32, device=device)


def bucket_index_sync_(ch: PeerChannel, scratch: IndexSyncScratch, acc: torch.Tensor, k: int, *, slots: SymmBuffer | None,
                       kcap: int, comm=None, touched: torch.Tensor, scale: float = 1.0, sumsq_out=None,
                       accumulate=False, select_only=False, zero_selected=True, max_ctas: int = 0) -> None:
    """Exact top-``k`` of ``|acc|`` + (index, value) exchange + rank-ordered
    scatter-add into ``comm``. With ``select_only`` only the bit mask of the
    selection is written to ``touched``."""
    d = ch.next_desc()
    rc = lib().sga_bucket_index_sync(ctypes.byref(d), acc.data_ptr(), acc.numel(), int(k), scratch.hist1.data_ptr(),
                                     scratch.hist2.data_ptr(), scratch.cta_gt.data_ptr(), scratch.cta_eq.data_ptr(),
                                     slots.ptr_array(0) if slots is not None else None, int(kcap), _p(comm),
                                     touched.data_ptr(), float(scale), ch.cta_partials.data_ptr(), _p(sumsq_out),
                                     int(accumulate), int(select_only), int(zero_selected), scratch.result.data_ptr(),
                                     max_ctas, _st())
    _chk(rc, "sga_bucket_index_sync")


def dense_adamw_ag_(ch: PeerChannel, w, g, m, v, model: SymmBuffer, bucket_start, bucket_len, table, group_lr,
                    group_wd, *, beta1, beta2, eps, step, coeff=None, adams=False, max_ctas: int = 0) -> None:
    d = ch.next_desc()
    ng = len(group_lr)
    lr_arr = (ctypes.c_float * ng)(*[float(x) for x in group_lr])
    wd_arr = (ctypes.c_float * ng)(*[float(x) for x in group_wd])
    bc1 = 1.0 if adams else 1.0 - beta1 ** step
    bc2 = 1.0 if adams else 1.0 - beta2 ** step
    rc = lib().sga_dense_adamw_ag(ctypes.byref(d), w.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                  model.ptr_array(0), bucket_start.data_ptr(), bucket_len.data_ptr(),
                                  bucket_start.numel(), table.seg_start.data_ptr(), table.seg_group.data_ptr(),
                                  table.nseg, ctypes.cast(lr_arr, ctypes.c_void_p),
                                  ctypes.cast(wd_arr, ctypes.c_void_p), ng, _p(coeff), float(beta1),
                                  float(1.0 - beta1), float(beta2), float(1.0 - beta2), float(bc1), float(bc2),
                                  float(eps), int(adams), max_ctas, _st())
    _chk(rc, "sga_dense_adamw_ag")
