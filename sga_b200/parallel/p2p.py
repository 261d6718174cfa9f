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

    def peek_desc(self) -> PeerDesc:
        """Descriptor for a launch that exchanges nothing (no flag is raised or awaited): the
        channel's sequence number stays where it is."""
        d = self.next_desc()
        self.seq -= 1
        d.seq, d.prev_seq = self.seq, self.seq
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
               sumsq_out=None, accumulate=False, max_ctas: int = 0, block_x: int = 0) -> None:
    """In-place two-shot all-reduce of ``n`` fp32 values at ``offset_bytes`` of a
    symmetric buffer, optionally fused with the pack of ``grad[idx]`` before
    and the scatter back after. With ``block_x`` > 0, ``idx`` holds packed
    ``head | tail_len`` descriptors of ``block_x``-element runs and ``n`` is
    ``len(idx) * block_x``: whole runs are gathered and scattered 16 bytes at a time."""
    d = ch.next_desc()
    rc = lib().sga_p2p_allreduce(ctypes.byref(d), _ptrs(buf, offset_bytes), int(n), float(scale), _p(grad), _p(idx),
                                 float(factor), int(pack), int(zero_after_pack), int(scatter), int(block_x),
                                 int(rs_only),
                                 ch.norm_slots(), ch.cta_partials.data_ptr(), _p(sumsq_out), int(accumulate),
                                 max_ctas, _st())
    _chk(rc, "sga_p2p_allreduce")


def nvls_allreduce_(ch: PeerChannel, buf: SymmBuffer, offset_bytes: int, n: int, *, scale: float = 1.0,
                    rs_only=False, sumsq_out=None, accumulate=False, max_ctas: int = 0) -> bool:
    """The dense all-reduce (or its reduce-scatter form) through the NVSwitch's in-switch reduction, for a
    buffer bound to a multicast object (``buf.mc_ptr``). Returns False, having launched nothing, when the
    buffer has no multicast mapping or the range is not a whole number of 16-byte groups: the caller then
    takes :func:`allreduce_`."""
    if not getattr(buf, "mc_ptr", 0) or n % 4 or offset_bytes % 16:
        return False
    d = ch.next_desc()
    rc = lib().sga_nvls_allreduce(ctypes.byref(d), ctypes.c_void_p(buf.local_ptr + offset_bytes),
                                  ctypes.c_void_p(buf.mc_ptr + offset_bytes), int(n), float(scale), int(rs_only),
                                  ch.norm_slots(), ch.cta_partials.data_ptr(), _p(sumsq_out), int(accumulate),
                                  max_ctas, _st())
    _chk(rc, "sga_nvls_allreduce")
    return True


def mask_union_reduce_(ch: PeerChannel, grad: SymmBuffer, grad_off: int, bits: SymmBuffer, bits_off: int,
                       ubits: SymmBuffer, ubits_off: int, n: int, *, scale: float = 1.0, mask_u8=None,
                       sumsq_out=None, accumulate=False, count_out=None, max_ctas: int = 0) -> None:
    d = ch.next_desc()
    rc = lib().sga_p2p_mask_union(ctypes.byref(d), _ptrs(grad, grad_off), _ptrs(bits, bits_off),
                                  _ptrs(ubits, ubits_off), int(n), float(scale), _p(mask_u8), ch.norm_slots(),
                                  ch.cta_partials.data_ptr(), _p(sumsq_out), int(accumulate), _p(count_out),
                                  max_ctas, _st())
    _chk(rc, "sga_p2p_mask_union")


IS_SEG = 8192           # elements per segment of the candidate arrays (csrc/index_sync.cu)
IS_SEG_PER_RANGE = 4
SCORE_CODES = {"update": 0, "abs_g": 1, "abs_m": 2, "coi": 3}


class ISyncDesc(ctypes.Structure):
    """Mirror of ``SgaISyncDesc`` (csrc/index_sync.cu)."""
    _fields_ = [("acc", ctypes.c_void_p), ("w", ctypes.c_void_p), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("n", ctypes.c_longlong),
                ("k", ctypes.c_int), ("score", ctypes.c_int), ("adams", ctypes.c_int), ("nspan", ctypes.c_int),
                ("beta1", ctypes.c_float), ("omb1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("omb2", ctypes.c_float), ("bc1", ctypes.c_float), ("bc2", ctypes.c_float), ("eps", ctypes.c_float),
                ("scale", ctypes.c_float),
                ("span_start", ctypes.c_void_p), ("span_wd", ctypes.c_void_p),
                ("state", ctypes.c_void_p), ("histA", ctypes.c_void_p), ("histB", ctypes.c_void_p),
                ("cand_idx", ctypes.c_void_p), ("cand_key", ctypes.c_void_p), ("cand_val", ctypes.c_void_p),
                ("segcnt", ctypes.c_void_p), ("segsel", ctypes.c_void_p), ("segeq", ctypes.c_void_p),
                ("roff", ctypes.c_void_p),
                ("partials", ctypes.c_void_p),
                ("slots", ctypes.c_void_p * 8), ("hdr", ctypes.c_void_p * 8),
                ("kcap", ctypes.c_int), ("hstride", ctypes.c_int),
                ("comm", ctypes.c_void_p), ("sumsq_out", ctypes.c_void_p), ("bits", ctypes.c_void_p),
                ("result", ctypes.c_void_p),
                ("cand_capacity", ctypes.c_longlong), ("seg_capacity", ctypes.c_int),
                ("partials_capacity", ctypes.c_int),
                ("accumulate", ctypes.c_int), ("zero_selected", ctypes.c_int), ("mode", ctypes.c_int),
                ("max_ctas", ctypes.c_int), ("phase", ctypes.c_int), ("reduce_ticket", ctypes.c_void_p),
                ("wait_ns", ctypes.c_void_p)]


def _nseg(n: int) -> int:
    return (int(n) + IS_SEG - 1) // IS_SEG


class IndexSyncScratch:
    """Per-device work memory of the fused top-k chain, sized for the largest bucket: the
    candidate arrays hold one entry per bucket element (a segment's candidates live in the
    segment's own slice, so no input can overflow them), the histograms stay zero between
    launches. Launches that share a scratch must be ordered on one stream."""

    def __init__(self, device, max_elems: int = 1 << 20):
        self.device = device
        self.nseg = _nseg(max_elems)
        cap = self.nseg * IS_SEG
        self.capacity = cap
        self.state = torch.zeros(64, dtype=torch.int32, device=device)
        self.histA = torch.zeros(8 * 4096, dtype=torch.int32, device=device)
        self.histB = torch.zeros(8 * 2048 + (1 << 19), dtype=torch.int32, device=device)
        self.cand_idx = torch.empty(cap, dtype=torch.int32, device=device)
        self.cand_key = torch.empty(cap, dtype=torch.int32, device=device)
        self.cand_val = torch.empty(cap, dtype=torch.float32, device=device)
        self.segcnt = torch.zeros(self.nseg, dtype=torch.int32, device=device)
        self.segsel = torch.zeros(self.nseg, dtype=torch.int32, device=device)
        self.segeq = torch.zeros(self.nseg, dtype=torch.int32, device=device)
        self.roff = torch.zeros(self.nseg + 1, dtype=torch.int32, device=device)
        self.nranges = (self.nseg + IS_SEG_PER_RANGE - 1) // IS_SEG_PER_RANGE
        self.partials = torch.zeros(self.nranges, dtype=torch.float32, device=device)
        self.result = torch.zeros(4, dtype=torch.int32, device=device)
        # nanoseconds this rank's exchange kernels stood waiting for peers' flags (accumulates; read and
        # zero it around the steps of interest)
        self.wait_ns = torch.zeros(1, dtype=torch.int64, device=device)

    def ensure(self, n: int) -> None:
        if _nseg(n) > self.nseg:
            self.__init__(self.device, n)


class IndexSyncSlots:
    """Receive area of one channel in symmetric memory: per source rank ``kcap`` (index, value)
    pairs, then per source rank the table of segment offsets into its pairs."""

    def __init__(self, pool: SymmPool, kcap: int, max_elems: int):
        self.kcap = int(kcap)
        self.hstride = _nseg(max_elems) + 1
        self.pairs_bytes = (8 * self.kcap * pool.world + 255) // 256 * 256
        self.buf: SymmBuffer = pool.alloc(self.pairs_bytes + 4 * self.hstride * pool.world)
        self.world = pool.world
        self.ticket = torch.zeros(1, dtype=torch.int32, device=pool.device)  # the reduce kernel's last-CTA ticket

    def pairs(self, src_rank: int, count: int) -> torch.Tensor:
        """``[count, 2]`` int32 view of what rank ``src_rank`` pushed here (index, value bits)."""
        return self.buf.view(torch.int32, 8 * self.kcap * src_rank, 2 * count).view(count, 2)


class ScoreInputs:
    """What the scores other than ``abs_g`` read beside the gradient: the bucket's slices of the
    fp32 weights and moments, the Adam scalars of the coming commit and, for ``update``, the
    weight decay of every parameter span of the bucket."""

    def __init__(self, name: str, *, w=None, m=None, v=None, beta1=0.9, beta2=0.999, eps=1e-8, step=1,
                 adams=False, span_start=None, span_wd=None):
        self.name, self.w, self.m, self.v = name, w, m, v
        self.beta1, self.beta2, self.eps, self.adams = float(beta1), float(beta2), float(eps), bool(adams)
        self.bc1 = 1.0 if adams else 1.0 - self.beta1 ** step
        self.bc2 = 1.0 if adams else 1.0 - self.beta2 ** step
        self.span_start, self.span_wd = span_start, span_wd


def bucket_index_sync_(ch: PeerChannel, scratch: IndexSyncScratch, acc: torch.Tensor, k: int, *,
                       slots: IndexSyncSlots | None = None, comm=None, bits: torch.Tensor | None = None,
                       scale: float = 1.0, sumsq_out=None, accumulate=False, select_only=False, zero_selected=True,
                       score: ScoreInputs | None = None, max_ctas: int = 0, defer_reduce: bool = False):
    """Exact top-``k`` of the score over ``acc`` (default ``|acc|``), exchange of the selected
    (index, value) pairs with every rank of the channel and rank-ordered scatter-add of all ranks'
    pairs, times ``scale``, into ``comm``; the selected coordinates of ``acc`` are zeroed. With
    ``select_only`` nothing is exchanged and the selection's bit mask is written to ``bits``.

    ``defer_reduce`` stops after the push and returns a token for :func:`bucket_index_reduce_`: the
    receive side then runs later (e.g. once every bucket has pushed, when no rank has to wait for a
    slower peer's payload any more). The channel and its slots must not be used in between."""
    n = acc.numel()
    scratch.ensure(n)
    d = ch.peek_desc() if select_only else ch.next_desc()
    s = ISyncDesc()
    s.acc, s.n, s.k = acc.data_ptr(), n, int(k)
    s.score = SCORE_CODES[score.name] if score is not None else 1
    if score is not None:
        s.w, s.m, s.v = _p(score.w), _p(score.m), _p(score.v)
        s.adams = int(score.adams)
        s.beta1, s.omb1, s.beta2, s.omb2 = score.beta1, 1.0 - score.beta1, score.beta2, 1.0 - score.beta2
        s.bc1, s.bc2, s.eps = score.bc1, score.bc2, score.eps
        if score.span_start is not None:
            s.span_start, s.span_wd = score.span_start.data_ptr(), score.span_wd.data_ptr()
            s.nspan = score.span_wd.numel()
    s.scale = float(scale)
    s.state, s.histA, s.histB = scratch.state.data_ptr(), scratch.histA.data_ptr(), scratch.histB.data_ptr()
    s.cand_idx, s.cand_key, s.cand_val = (scratch.cand_idx.data_ptr(), scratch.cand_key.data_ptr(),
                                          scratch.cand_val.data_ptr())
    s.segcnt, s.segsel, s.segeq = scratch.segcnt.data_ptr(), scratch.segsel.data_ptr(), scratch.segeq.data_ptr()
    s.roff = scratch.roff.data_ptr()
    s.partials, s.result = scratch.partials.data_ptr(), scratch.result.data_ptr()
    s.cand_capacity, s.seg_capacity, s.partials_capacity = scratch.capacity, scratch.nseg, scratch.nranges
    if not select_only:
        if slots is None or comm is None:
            raise ValueError("bucket_index_sync_: the exchange needs receive slots and a staging buffer")
        for r in range(slots.world):
            s.slots[r] = slots.buf.peer_ptrs[r]
            s.hdr[r] = slots.buf.peer_ptrs[r] + slots.pairs_bytes
        s.kcap, s.hstride = slots.kcap, slots.hstride
        s.comm = comm.data_ptr()
    else:
        if bits is None:
            raise ValueError("bucket_index_sync_: select_only writes the bit mask to `bits`")
        s.bits = bits.data_ptr()
    s.sumsq_out = _p(sumsq_out)
    s.accumulate, s.zero_selected, s.mode, s.max_ctas = int(accumulate), int(zero_selected), int(select_only), max_ctas
    s.phase = 1 if (defer_reduce and not select_only) else 0
    s.reduce_ticket = slots.ticket.data_ptr() if slots is not None else None
    s.wait_ns = scratch.wait_ns.data_ptr()
    rc = lib().sga_index_sync(ctypes.byref(d), ctypes.byref(s), _st())
    _chk(rc, "sga_index_sync")
    return (d, s, (acc, comm, slots, scratch, sumsq_out)) if s.phase == 1 else None


def bucket_index_reduce_(token) -> None:
    """The receive side of a :func:`bucket_index_sync_` call that was made with ``defer_reduce``."""
    d, s, _keep = token
    s.phase = 2
    rc = lib().sga_index_sync(ctypes.byref(d), ctypes.byref(s), _st())
    _chk(rc, "sga_index_sync (reduce)")


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
