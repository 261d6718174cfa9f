"""Fused, parameter-sharded, multi-configuration replay.

The flat parameter vector is cut into ``world`` contiguous shards (one
process, one GPU each). Every shard streams the window's gradient files once
and advances all R configurations of a group together: per step one pass for
the clip norms, a boundary reselection (exact distributed top-k) where the
calendar asks for it, and one pass that clips, updates residuals, commits Adam
and accumulates the horizon numerators. On CUDA the two passes are the
``csrc/replay.cu`` kernels (one read of ``g`` for all R configurations); on
CPU the same arithmetic runs as PyTorch ops, which is what makes a one-shard
run equal the per-configuration oracle bit for bit.

Cross-shard traffic is small and goes through ``torch.distributed`` (gloo on
CPU, NCCL on GPUs): fp64 partial sums ``[R]`` per pass, int64 radix
histograms and tie counts per selection. Sums are reduced in fp64, so shard
counts only reorder additions ("pure reordering band": sums agree to ~1e-6
relative, everything discrete is exact).

Reference: ``sga/replay_fused.py:97-2404`` (Comms ``:113-227``, shard_select
``:290-402``, GPrefetcher ``:902-1104``, worker ``:1124-2083``).
"""
from __future__ import annotations

import ctypes
import math
import os
import queue
import struct
import threading
import time
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from . import core as RC

# kill switches: unknown values raise so that both arms of an A/B are always reachable
ENV_KERNEL = "REPLAY_FUSED_KERNEL"      # on | off  (off: PyTorch ops even on CUDA)
ENV_SELECT = "REPLAY_FUSED_SELECT"      # auto | cpu  (cpu: the front block's selections run on host tensors)
ENV_FRONT_SORT = "REPLAY_FUSED_FRONT_SORT"  # auto | cpu  (cpu: the front block's ranking sorts run on the host)
ENV_FRONT_RANK_BG = "REPLAY_FUSED_FRONT_RANK_BG"  # on | off  (on: rank 0 ranks the front block on a worker thread)
ENV_P1_READ = "REPLAY_FUSED_P1_READ"    # mmap | load | pread  (mmap and pread: a shard touches only its slice of every gradient file)
ENV_S0_PROFILE = "REPLAY_S0_PROFILE"    # 0 | 1  (1: rank 0 prints per-group counters and the phase times)
ENV_WINDOW_HOST_GIB = "REPLAY_FUSED_WINDOW_HOST_GIB"  # host bytes (GiB, default 8) a shard may spend keeping the
#                                          window's gradients between the dense arm and the stream


def _switch(name, allowed, default):
    v = os.environ.get(name, default)
    if v not in allowed:
        raise ValueError(f"{name} must be one of {allowed} (got {v!r})")
    return v


class Comms:
    """Scalar / histogram plane over one process group (identity for one shard)."""

    def __init__(self, rank=0, world=1, group=None, device="cpu"):
        self.rank, self.world, self.group, self.device = rank, world, group, torch.device(device)
        self.ops = 0

    def sum_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            self.ops += 1
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def min_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            self.ops += 1
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return t

    def gather_i64(self, value: int) -> list:
        if self.world == 1:
            return [int(value)]
        self.ops += 1
        t = torch.tensor([int(value)], dtype=torch.int64, device=self.device)
        out = [torch.zeros_like(t) for _ in range(self.world)]
        dist.all_gather(out, t, group=self.group)
        return [int(x.item()) for x in out]

    def gather_to_root(self, t: torch.Tensor):
        """Variable-length gather of a 1-D tensor; returns the concatenation on rank 0."""
        if self.world == 1:
            return t
        sizes = self.gather_i64(t.numel())
        pad = torch.zeros(max(sizes), dtype=t.dtype, device=t.device)
        pad[:t.numel()] = t
        out = [torch.zeros_like(pad) for _ in range(self.world)]
        self.ops += 1
        dist.all_gather(out, pad, group=self.group)
        return torch.cat([o[:s] for o, s in zip(out, sizes)])


def shard_bounds(n: int, world: int, rank: int):
    per = (n + world - 1) // world
    per = (per + 7) // 8 * 8
    lo = min(n, per * rank)
    return lo, min(n, lo + per)


def _key_float(key: int) -> float:
    """The non-negative fp32 whose bit pattern is ``key``."""
    return struct.unpack("<f", struct.pack("<I", key & 0x7FFFFFFF))[0]


def shard_select(score_loc: torch.Tensor, k: int, comms: Comms, return_threshold: bool = False):
    """Exact distributed top-``k`` by ``|score|`` with ties filled in global
    flat-index order (shards are contiguous and ordered by rank). Two radix
    digits: the 16 high key bits locate the crossing bin, the 16 low bits the
    exact key; no candidate values cross the wire. ``return_threshold`` also
    returns the k-th largest ``|score|``."""
    from ..plugins.selection._histogram import _ops

    ops = _ops(score_loc)
    x = score_loc.contiguous().float()
    hist = torch.zeros(32769, dtype=torch.int64, device=x.device)
    if x.numel():
        ops.hist_top(x, 16, 1, 32769, hist)
    comms.sum_(hist)
    suffix = torch.cumsum(hist.flip(0), 0)
    b = 32768 - int(torch.searchsorted(suffix, k).item())
    above = int(hist[b + 1:].sum().item())
    low = torch.zeros(65536, dtype=torch.int64, device=x.device)
    if x.numel():
        ops.hist_low16(x, b, low)
    comms.sum_(low)
    suffix2 = torch.cumsum(low.flip(0), 0)
    lb = 65535 - int(torch.searchsorted(suffix2, k - above).item())
    T = (b << 16) | lb
    n_gt = above + int(low[lb + 1:].sum().item())
    need = k - n_gt
    key = RC.abs_key(x)
    sel = key > T
    ties = torch.nonzero(key == T, as_tuple=False).view(-1)
    counts = comms.gather_i64(ties.numel())
    before = sum(counts[:comms.rank])
    take = max(0, min(ties.numel(), need - before))
    if take:
        sel[ties[:take]] = True
    return (sel, _key_float(T)) if return_threshold else sel


def _unclip(g: torch.Tensor, gmeta: dict, dev) -> torch.Tensor:
    """The logged (clipped) gradient divided by the clip coefficient its step applied."""
    coef, _flag = RC.coef_dense_for(gmeta)
    return g.to(dev).float() / coef


def shard_stats(flat: torch.Tensor, comms: Comms) -> dict:
    """numel / sum / mean / min / max / fraction of zeros of a sharded vector: shard-partial sums
    combined in fp64, the rest exact (``sga/replay_fused.py:2085-2112``)."""
    n = flat.numel()
    row = torch.tensor([float(n), float(flat.sum()) if n else 0.0, float((flat == 0).sum()) if n else 0.0],
                       dtype=torch.float64, device=comms.device)
    ext = torch.tensor([float(flat.min()) if n else float("inf"), -float(flat.max()) if n else float("inf")],
                       dtype=torch.float64, device=comms.device)
    comms.sum_(row)
    comms.min_(ext)
    total, ssum, nzero = int(row[0]), float(row[1]), int(row[2])
    return {"numel": total, "sum": ssum, "mean": ssum / total if total else 0.0,
            "min": float(ext[0]) if total else 0.0, "max": -float(ext[1]) if total else 0.0,
            "fraction_zero": nzero / total if total else 0.0}


def shard_entries(info, lo: int, hi: int) -> list:
    """This shard's slice of every parameter: ``(local offset, offset inside the parameter, length)``."""
    out = []
    for off, sh in zip(info.offsets, info.shapes):
        n = int(math.prod(sh)) if sh else 1
        a, b = max(off, lo), min(off + n, hi)
        if a < b:
            out.append((a - lo, a - off, b - a))
    return out


def shard_select_balanced(score_loc: torch.Tensor, k: int, comms: Comms, entries, return_threshold: bool = False):
    """The online engine's ``balanced`` histogram selection replayed on a sharded flat vector
    (``sga/replay_fused.py:405-489``): the histogram of the 16 high key bits is built on every 8th
    element of each parameter, on the parameter's own grid (a shard that starts inside a parameter
    continues that grid), the crossing bin is searched at rank ``max(1, round(n_sampled * (n_total -
    k + 1) / n_total))`` and the WHOLE crossing bin is kept, so slightly more than ``k`` coordinates
    are selected. Shard histograms and counts are disjoint partials: their sums are the unsharded
    values and every shard derives the same bin."""
    from ..plugins.selection._histogram import HIST_MODES, _ops, balanced_crossing_bin

    if comms.world > 1 and os.environ.get("SGA_MASTER_ADDR") is not None:
        raise ValueError("--selection-semantics balanced-histogram supports only the single-node engine")
    x = score_loc.contiguous().float()
    if not bool(torch.isfinite(x).all()):
        raise ValueError("shard_select_balanced requires finite scores")
    shift, nbins, stride = HIST_MODES["balanced"]
    ops = _ops(x)
    hist = torch.zeros(nbins, dtype=torch.int64, device=x.device)
    n_tot = n_smp = 0
    for a, p_off, n in entries:
        phase = (-p_off) % stride
        n_tot += n
        if n > phase:
            n_smp += (n - phase + stride - 1) // stride
            ops.hist_top(x[a + phase:a + n], shift, stride, nbins, hist)
    comms.sum_(hist)
    counts = torch.tensor([n_tot, n_smp], dtype=torch.int64, device=x.device)
    comms.sum_(counts)
    b = balanced_crossing_bin(hist, int(counts[0]), int(counts[1]), k, replicas=1)
    sel = (RC.abs_key(x) >> shift) >= b
    return (sel, _key_float(int(b) << shift)) if return_threshold else sel  # threshold: the bin's lower edge


def front_metrics(got_s, got_l, ideal, k: int, threshold, stats, sort_on_host: bool) -> dict:
    """Ranking metrics of one (score, ratio, optimizer) cell from the gathered selections: the
    score's own top-k (``got_s`` scores with their labels ``got_l``) against the label's top-k
    (``ideal``). Pure function of its arguments; runs on whichever device the tensors live on."""
    if sort_on_host:
        got_s, got_l, ideal = got_s.cpu(), got_l.cpu(), ideal.cpu()
    disc = 1.0 / torch.log2(torch.arange(2, k + 2, dtype=torch.float64, device=got_s.device))
    order = torch.argsort(got_s, descending=True, stable=True)
    idl = torch.sort(ideal.double(), descending=True).values
    idcg = float((idl * disc[:idl.numel()]).sum())
    ndcg = float((got_l.double()[order] * disc[:order.numel()]).sum()) / idcg if idcg > 0 else 0.0
    return {"k": k, "threshold": threshold, "ndcg_at_k": ndcg, "recall_at_k": stats[0] / max(k, 1),
            "missed_label_mass": stats[1] / stats[2] if stats[2] > 0 else 0.0,
            "missed_score_mass": stats[3] / stats[4] if stats[4] > 0 else 0.0}


class RankLane:
    """One worker thread that turns gathered selections into ranking metrics while the main thread
    goes on to the next cell's collectives. Work items are closed over plain tensors and numbers:
    the worker never sees a process group and never issues a collective, so every collective stays
    on the main thread, and cells are ranked in submission order by the single writer of
    ``results``, which makes the report identical to the inline path.

    A failure in the worker is kept, not swallowed: ``submit`` refuses to queue behind a dead
    worker (a bounded queue with no consumer would block the main thread for ever) and ``finish``
    re-raises it before the results are used. With ``enabled=False`` the same calls run inline."""

    _STOP = object()

    def __init__(self, enabled: bool, device: torch.device, depth: int = 4):
        self.enabled, self.device = bool(enabled), device
        self.results: dict = {}
        self.rank_s = 0.0      # time spent ranking (worker or inline)
        self.wait_s = 0.0      # time the main thread stood in submit / finish
        self.error: Optional[BaseException] = None
        self.current = "start-up"
        self.thread = None
        # the worker thread starts on the process's default device: give it the creator's one by number
        # (a bare "cuda" device carries no index)
        self.cuda_index = None
        if self.enabled and device.type == "cuda":
            self.cuda_index = device.index if device.index is not None else torch.cuda.current_device()
        if self.enabled:
            self.q = queue.Queue(maxsize=depth)
            self.thread = threading.Thread(target=self._work, name="sga-replay-front-rank", daemon=True)
            self.thread.start()

    def _rank(self, key, args) -> None:
        t0 = time.perf_counter()
        self.current = repr(key)
        self.results[key] = front_metrics(*args)
        self.rank_s += time.perf_counter() - t0

    def _work(self):
        try:
            if self.cuda_index is not None:
                torch.cuda.set_device(self.cuda_index)  # the current device is per thread
            while True:
                item = self.q.get()
                if item is self._STOP:
                    return
                self._rank(*item)
        except BaseException as e:  # kept for the main thread
            self.error = e

    def _fail(self):
        raise RuntimeError(f"front ranking failed at {self.current}") from self.error

    def submit(self, key, *args) -> None:
        if not self.enabled:
            self._rank(key, args)
            return
        t0 = time.perf_counter()
        try:
            while True:
                if self.error is not None:
                    self._fail()
                try:
                    self.q.put((key, args), timeout=0.5)
                    return
                except queue.Full:
                    if not self.thread.is_alive() and self.error is None:
                        raise RuntimeError("front ranking worker exited without a recorded error")
        finally:
            self.wait_s += time.perf_counter() - t0

    def finish(self) -> dict:
        """Drains the lane and returns the results; re-raises a worker failure."""
        if self.enabled and self.thread is not None:
            t0 = time.perf_counter()
            while self.thread.is_alive():
                try:
                    self.q.put(self._STOP, timeout=0.5)
                    break
                except queue.Full:
                    continue
            self.thread.join()
            self.thread = None
            self.wait_s += time.perf_counter() - t0
        if self.error is not None:
            self._fail()
        return self.results


@dataclass
class StepInput:
    si: int
    g: torch.Tensor          # this shard's logged gradient (fp32 or bf16), on the device
    grad_norm: float
    lr: float


READ_ARMS = ("mmap", "load", "pread")


class GPrefetcher:
    """Background reader: produces, step by step, this shard's slice of the logged gradient in
    catalog order, staged in pinned memory when the consumer is a GPU. Depth-bounded; the first
    failure of any of its threads is latched and re-raised by ``get``.

    Read arms (``REPLAY_FUSED_P1_READ``): ``mmap`` maps the step file and copies the slice out of
    the mapping, ``load`` reads the whole file, ``pread`` never opens the file as an archive at
    all: one thread copies the slice's bytes out of the stored zip records with positional reads
    (``ptfile.PtIndex``) while a second thread converts and pins the previous step's bytes, so the
    conversion never sits between two read calls. The pread arm holds up to ``depth`` raw slices
    beside the ``depth`` converted ones. ``index_cache`` (path -> PtIndex) lets several
    prefetchers over the same window parse each file's directory once."""

    def __init__(self, info: RC.TraceInfo, steps, lo, hi, dtype, pin: bool, depth: int = 2, index_cache=None):
        self.info, self.steps, self.lo, self.hi, self.dtype, self.pin = info, list(steps), lo, hi, dtype, pin
        self.mode = _switch(ENV_P1_READ, READ_ARMS, "mmap")
        self.q = queue.Queue(maxsize=depth)
        self.exc: Optional[BaseException] = None
        self.read_s = 0.0
        self.convert_s = 0.0
        self.index_cache = {} if index_cache is None else index_cache
        if self.mode == "pread":
            self.raw_q = queue.Queue(maxsize=depth)
            self.threads = [threading.Thread(target=self._run_pread, name="sga-replay-pread", daemon=True),
                            threading.Thread(target=self._run_convert, name="sga-replay-convert", daemon=True)]
        else:
            self.threads = [threading.Thread(target=self._run, name="sga-replay-prefetch", daemon=True)]
        for t in self.threads:
            t.start()

    def _load(self, t):
        return RC.load_g(self.info, t, mmap=self.mode == "mmap")

    def _run(self):
        try:
            for t in self.steps:
                t0 = time.perf_counter()
                meta, payload = self._load(t)
                flat = RC.flatten(payload, self.info, self.dtype, self.lo, self.hi)
                if self.pin:
                    flat = flat.pin_memory()
                self.read_s += time.perf_counter() - t0
                self.q.put((t, meta, flat))
        except BaseException as e:
            self.exc = e
            self.q.put(None)

    def _run_pread(self):
        from .ptfile import PtIndex

        try:
            for t in self.steps:
                t0 = time.perf_counter()
                path = os.path.join(self.info.dir, f"step_{t:06d}_g.pt")
                idx = self.index_cache.get(path)
                if idx is None:
                    idx = self.index_cache[path] = PtIndex(path)
                meta, stubs = idx.tree["meta"], idx.tree["payload"]
                pieces = []
                fd = os.open(path, os.O_RDONLY)
                try:
                    for name, off, sh in zip(self.info.names, self.info.offsets, self.info.shapes):
                        n = int(math.prod(sh)) if sh else 1
                        a, b = max(off, self.lo), min(off + n, self.hi)
                        if a >= b:
                            continue
                        if name not in stubs:
                            raise KeyError(f"{path}: no gradient for {name}")
                        if stubs[name].numel() != n:
                            raise ValueError(f"{path}: {name} holds {stubs[name].numel()} elements, the catalog says {n}")
                        pieces.append((a - self.lo, idx.read_slice(fd, stubs[name], a - off, b - a)))
                finally:
                    os.close(fd)
                self.read_s += time.perf_counter() - t0
                self.raw_q.put((t, meta, pieces))
            self.raw_q.put(None)
        except BaseException as e:
            self.exc = e
            self.raw_q.put(None)

    def _run_convert(self):
        try:
            while True:
                item = self.raw_q.get()
                if item is None:
                    if self.exc is not None:
                        self.q.put(None)
                    return
                t, meta, pieces = item
                t0 = time.perf_counter()
                flat = torch.empty(self.hi - self.lo, dtype=self.dtype, pin_memory=self.pin)
                for dst, piece in pieces:
                    flat[dst:dst + piece.numel()].copy_(piece)
                self.convert_s += time.perf_counter() - t0
                self.q.put((t, meta, flat))
        except BaseException as e:
            self.exc = e
            self.q.put(None)

    def get(self):
        item = self.q.get()
        if item is None:
            raise RuntimeError(f"gradient prefetch failed: {self.exc!r}") from self.exc
        return item


# score codes of csrc/replay_select.cu: the registry's, plus the replay-only |step gradient|
_SCORE_CODES = {"update": 0, "abs_g": 1, "abs_m": 2, "coi": 3, "abs_g_step": 4}


class _CfgStruct(ctypes.Structure):
    _fields_ = [("boundary", ctypes.c_int), ("fold", ctypes.c_int), ("dual", ctypes.c_int), ("adams", ctypes.c_int),
                ("horizon", ctypes.c_int), ("fold_div", ctypes.c_float), ("coef", ctypes.c_float),
                ("lr", ctypes.c_float), ("lr_inactive", ctypes.c_float), ("bc1", ctypes.c_float),
                ("bc2", ctypes.c_float)]


class FusedGroup:
    """R configurations of one branch point advanced together on one shard."""

    def __init__(self, configs, n_loc, n_total, device, comms: Comms, hp: RC.Hyper, wd_vec, w0, m0, v0, t0, W,
                 horizons, dense_snaps, use_kernel: bool, semantics: str = "topk", entries=None):
        self.cfgs = list(configs)
        self.semantics, self.entries = semantics, entries
        self.R = len(self.cfgs)
        if self.R > 32:
            raise ValueError("at most 32 configurations per fused group")
        self.n, self.n_total, self.device, self.comms, self.hp = n_loc, n_total, torch.device(device), comms, hp
        self.t0, self.Wlen, self.horizons = t0, W, sorted(horizons)
        self.use_kernel = use_kernel and self.device.type == "cuda"
        R, n = self.R, n_loc
        self.W = w0.to(self.device).unsqueeze(0).repeat(R, 1).contiguous()
        self.M = m0.to(self.device).unsqueeze(0).repeat(R, 1).contiguous()
        self.V = v0.to(self.device).unsqueeze(0).repeat(R, 1).contiguous()
        self.RES = torch.zeros(R, n, dtype=torch.float32, device=self.device)
        self.SEL = torch.zeros(R, n, dtype=torch.uint8, device=self.device)
        self.wd = wd_vec.to(self.device)
        self.dense = {h: t.to(self.device) for h, t in dense_snaps.items()}
        self.k = [RC.k_for(n_total, c.ratio_percent) for c in self.cfgs]
        self.numer = {h: [0.0] * R for h in self.horizons}
        self.per_step = []
        self.stats = {"pass1_s": 0.0, "select_s": 0.0, "pass3_s": 0.0, "selects": 0, "h2d_bytes": 0, "host_syncs": 0}
        if self.use_kernel:
            from ..csrc import lib

            L = lib()
            self._nb = L.sga_replay_blocks()
            self._partials = torch.zeros(R * self._nb, dtype=torch.float64, device=self.device)
            self._out = torch.zeros(R, dtype=torch.float64, device=self.device)
            self._cfg_dev = torch.zeros(R * ctypes.sizeof(_CfgStruct), dtype=torch.uint8, device=self.device)

    # -------------------------------------------------------------- selection
    def initial_select(self, branch_grad_loc) -> None:
        """Branch-point supports: the state dump's gradient is post-clip and is scored as is."""
        g = branch_grad_loc.to(self.device).float()
        cache = {}
        for r, c in enumerate(self.cfgs):
            key = (c.score, c.ratio_percent, c.optimizer)
            if key not in cache:
                sc = RC.replay_score(c.score, self.W[r], self.M[r], self.V[r], g, self._hp_dev(), self.t0 + 1,
                                     c.optimizer)
                if self._device_select:
                    cache[key] = self._device_topk([sc.contiguous()], [self.k[r]])[0].clone()
                else:
                    cache[key] = self._select(sc, self.k[r])
            self.SEL[r] = cache[key].to(torch.uint8)

    @property
    def _device_select(self) -> bool:
        """Exact top-k selections run wholly on the device (``csrc/replay_select.cu``) when the
        step kernels do; the balanced-histogram rule keeps its host-driven form."""
        return self.use_kernel and self.semantics == "topk"

    def _select_scratch(self, rows: int):
        if getattr(self, "_sel_rows", 0) < rows:
            dev, n = self.device, self.n
            nblk = (n + 4095) // 4096
            self._h1 = torch.zeros(rows, 32769, dtype=torch.int64, device=dev)
            self._h2 = torch.zeros(rows, 65536, dtype=torch.int64, device=dev)
            self._state = torch.zeros(rows, 8, dtype=torch.int64, device=dev)
            self._blockcnt = torch.zeros(rows, max(nblk, 1), dtype=torch.int32, device=dev)
            self._newsel = torch.zeros(rows, n, dtype=torch.uint8, device=dev)
            self._totals = torch.zeros(self.comms.world * rows, dtype=torch.int64, device=dev)
            self._sel_rows = rows

    def _device_topk(self, scores, ks):
        """Exact distributed top-``ks[j]`` of ``|scores[j]|`` for every row at once, ties in global
        index order: two radix digits whose histograms are summed over the shards (one collective
        per digit for all rows), one gathered tie count, every decision in between taken by kernels.
        Returns uint8 masks (views of a scratch buffer that the next call overwrites)."""
        from .. import kernels as K
        from ..csrc import lib

        L = lib()
        rows, n = len(scores), self.n
        self._select_scratch(rows)
        st = torch.cuda.current_stream().cuda_stream
        h1, h2, state = self._h1[:rows], self._h2[:rows], self._state[:rows]
        h1.zero_()
        h2.zero_()
        state.zero_()
        state[:, 7] = torch.tensor([int(k) for k in ks], dtype=torch.int64).to(self.device, non_blocking=True)
        for j, sc in enumerate(scores):
            if n:
                K.hist_top(sc, 16, 1, 32769, h1[j])
        self.comms.sum_(h1)
        assert L.sga_replay_find_bin(h1.data_ptr(), 32769, state.data_ptr(), 0, rows, st) == 0
        for j, sc in enumerate(scores):
            assert L.sga_replay_hist_low16(sc.data_ptr(), n, state[j].data_ptr(), h2[j].data_ptr(), st) == 0
        self.comms.sum_(h2)
        assert L.sga_replay_find_bin(h2.data_ptr(), 65536, state.data_ptr(), 1, rows, st) == 0
        for j, sc in enumerate(scores):
            assert L.sga_replay_mask(sc.data_ptr(), n, state[j].data_ptr(), self._newsel[j].data_ptr(),
                                     self._blockcnt[j].data_ptr(), st) == 0
        W = self.comms.world
        totals = self._totals[:W * rows]
        mine = state[:, 6].contiguous()
        if W > 1:
            self.comms.ops += 1
            dist.all_gather_into_tensor(totals, mine, group=self.comms.group)
        else:
            totals.copy_(mine)
        for j, sc in enumerate(scores):
            assert L.sga_replay_tie_fill(sc.data_ptr(), n, state[j].data_ptr(), self._blockcnt[j].data_ptr(),
                                         totals.data_ptr(), self.comms.rank, rows, j, self._newsel[j].data_ptr(),
                                         st) == 0
        return [self._newsel[j] for j in range(rows)]

    def _boundary_select_device(self, rs, plan, g_dev, coef_dense, count):
        """Scores of the configurations ``rs`` on their pre-commit state (one kernel each), then the
        batched exact top-k."""
        from ..csrc import lib

        L = lib()
        st = torch.cuda.current_stream().cuda_stream
        self._upload(plan)
        if getattr(self, "_sc", None) is None or self._sc.shape[0] < len(rs):
            self._sc = torch.empty(len(rs), self.n, dtype=torch.float32, device=self.device)
        stride = ctypes.sizeof(_CfgStruct)
        for j, r in enumerate(rs):
            p = plan[r]
            rc = L.sga_replay_score(g_dev.data_ptr(), int(g_dev.dtype == torch.bfloat16), coef_dense,
                                    self.W[r].data_ptr(), self.M[r].data_ptr(), self.V[r].data_ptr(),
                                    self.RES[r].data_ptr(), self.SEL[r].data_ptr(), self.wd.data_ptr(),
                                    self._cfg_dev.data_ptr() + r * stride, _SCORE_CODES[self.cfgs[r].score],
                                    float(self.hp.beta1), float(self.hp.beta2), float(self.hp.eps),
                                    float(p["bc1"]), float(p["bc2"]), self.n, self._sc[j].data_ptr(), st)
            assert rc == 0, rc
        return self._device_topk([self._sc[j] for j in range(len(rs))], [self.k[r] for r in rs])

    def _select(self, sc, k):
        """The trajectory-driving selection: exact top-k, or the online balanced-histogram rule."""
        if self.semantics == "balanced-histogram":
            return shard_select_balanced(sc, k, self.comms, self.entries)
        return shard_select(sc, k, self.comms)

    def _hp_dev(self):
        return RC.Hyper(wd=self.wd, beta1=self.hp.beta1, beta2=self.hp.beta2, eps=self.hp.eps, clip=self.hp.clip)

    # ------------------------------------------------------------------- step
    def _plan(self, si, count, lr):
        plan = []
        for c in self.cfgs:
            adams = c.optimizer == "adams"
            boundary = c.cycle_len > 0 and si % c.cycle_len == 0  # cycle length 0: zerofill, never a boundary
            lr32 = RC.f32(lr)
            plan.append(dict(
                boundary=boundary, fold=bool(c.fold and boundary and si > 0), fold_div=float(max(c.cycle_len, 1)),
                dual=bool(c.dual_lr != 1.0), adams=adams, lr=lr32,
                lr_inactive=RC.f32(lr * c.dual_lr),
                bc1=1.0 if adams else 1.0 - self.hp.beta1 ** count, bc2=1.0 if adams else 1.0 - self.hp.beta2 ** count,
                horizon=(si + 1) in self.dense, coef=1.0))
        return plan

    def _upload(self, plan):
        arr = (_CfgStruct * self.R)()
        for r, p in enumerate(plan):
            a = arr[r]
            a.boundary, a.fold, a.dual, a.adams, a.horizon = int(p["boundary"]), int(p["fold"]), int(p["dual"]), \
                int(p["adams"]), int(p["horizon"])
            a.fold_div, a.coef, a.lr, a.lr_inactive, a.bc1, a.bc2 = p["fold_div"], p["coef"], p["lr"], \
                p["lr_inactive"], p["bc1"], p["bc2"]
        host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
        self._cfg_dev.copy_(host)

    def _q_pre(self, p, g, r):
        if p["boundary"]:
            res = RC._div(self.RES[r], p["fold_div"]) if p["fold"] else self.RES[r]
            return g + res
        return torch.where(self.SEL[r] > 0, g, torch.zeros_like(g))

    def step(self, inp: StepInput) -> None:
        si = inp.si
        count = self.t0 + si + 1
        plan = self._plan(si, count, inp.lr)
        coef_dense = RC.f32(RC.clip_coef(inp.grad_norm ** 2, self.hp.clip)) if self.hp.clip > 0 else 1.0
        g_dev = inp.g.to(self.device, non_blocking=True)
        if self.device.type == "cuda":
            self.stats["h2d_bytes"] += inp.g.numel() * inp.g.element_size()
        st = None
        # ---- pass 1: clip norms
        t0 = time.perf_counter()
        if self.use_kernel:
            from ..csrc import lib

            st = torch.cuda.current_stream().cuda_stream
            self._upload(plan)
            rc = lib().sga_replay_pass1(g_dev.data_ptr(), int(g_dev.dtype == torch.bfloat16), coef_dense,
                                        self.RES.data_ptr(), self.SEL.data_ptr(), self._cfg_dev.data_ptr(), self.R,
                                        self.n, self._partials.data_ptr(), self._out.data_ptr(), st)
            assert rc == 0, rc
            sums = self._out.clone()
            g = None
        else:
            g = RC._div(g_dev.float(), coef_dense)
            sums = torch.stack([(self._q_pre(p, g, r).double() ** 2).sum() for r, p in enumerate(plan)])
        self.comms.sum_(sums)
        sums = sums.tolist()
        self.stats["host_syncs"] += 1
        for p, s in zip(plan, sums):
            p["coef"] = RC.f32(RC.clip_coef(s, self.hp.clip))
        self.stats["pass1_s"] += time.perf_counter() - t0
        # ---- pass 2: boundary reselection on the pre-commit state (the outgoing support stays for pass 3)
        t0 = time.perf_counter()
        new_sel = {}
        reselect = [r for r, p in enumerate(plan) if p["boundary"] and 0 < si < self.Wlen - 1]
        if reselect and self._device_select:
            masks = self._boundary_select_device(reselect, plan, g_dev, coef_dense, count)
            new_sel = dict(zip(reselect, masks))
            self.stats["selects"] += len(reselect)
        elif reselect:
            if g is None:
                g = RC._div(g_dev.float(), coef_dense)
            cache = {}
            for r, (p, c) in enumerate(zip(plan, self.cfgs)):
                if not (p["boundary"] and 0 < si < self.Wlen - 1):
                    continue
                q = self._q_pre(p, g, r) * p["coef"]
                sc = RC.replay_score(c.score, self.W[r], self.M[r], self.V[r], q, self._hp_dev(), count, c.optimizer,
                                     g_step=g)
                new_sel[r] = self._select(sc, self.k[r]).to(torch.uint8)
                self.stats["selects"] += 1
        self.stats["select_s"] += time.perf_counter() - t0
        # ---- pass 3: clip, residual, commit, horizon numerators
        t0 = time.perf_counter()
        h = si + 1
        if self.use_kernel:
            from ..csrc import lib

            self._upload(plan)
            wden = self.dense.get(h)
            rc = lib().sga_replay_pass3(g_dev.data_ptr(), int(g_dev.dtype == torch.bfloat16), coef_dense,
                                        self.W.data_ptr(), self.M.data_ptr(), self.V.data_ptr(), self.RES.data_ptr(),
                                        self.SEL.data_ptr(), self.wd.data_ptr(),
                                        wden.data_ptr() if wden is not None else None, self._cfg_dev.data_ptr(),
                                        self.R, self.n, RC.f32(self.hp.beta1), RC.f32(1.0 - self.hp.beta1),
                                        RC.f32(self.hp.beta2), RC.f32(1.0 - self.hp.beta2), RC.f32(self.hp.eps),
                                        self._partials.data_ptr() if wden is not None else None,
                                        self._out.data_ptr() if wden is not None else None, st)
            assert rc == 0, rc
            if wden is not None:
                num = self.comms.sum_(self._out.clone()).tolist()
                self.stats["host_syncs"] += 1
                self.numer[h] = num
        else:
            for r, (p, c) in enumerate(zip(plan, self.cfgs)):
                q = self._q_pre(p, g, r) * p["coef"]
                sel = self.SEL[r] > 0
                if p["boundary"]:
                    self.RES[r].zero_()
                else:
                    self.RES[r] += torch.where(sel, torch.zeros_like(g), g)
                RC.adam_commit_torch(self.W[r], self.M[r], self.V[r], q, inp.lr, self.wd, self.hp.beta1,
                                     self.hp.beta2, self.hp.eps, count, c.optimizer,
                                     inactive=(~sel if (p["boundary"] and p["dual"]) else None), dual_lr=c.dual_lr)
            if h in self.dense:
                num = torch.stack([((self.W[r].double() - self.dense[h].double()) ** 2).sum() for r in range(self.R)])
                self.numer[h] = self.comms.sum_(num).tolist()
        for r, m in new_sel.items():
            self.SEL[r] = m
        self.stats["pass3_s"] += time.perf_counter() - t0
        self.per_step.append({"si": si, "coef": [p["coef"] for p in plan]})


# --------------------------------------------------------------------- driver
def group_configs(configs, max_configs: int, state_budget_mb: float, n_loc: int):
    """Cut the configuration list into groups of one optimizer that fit ``max_configs`` and,
    when given, a per-shard state budget (17 bytes per element per configuration)."""
    per_cfg = 17.0 * n_loc / (1 << 20)
    cap = max(1, min(32, max_configs))
    if state_budget_mb and state_budget_mb > 0:
        cap = max(1, min(cap, int(state_budget_mb // max(per_cfg, 1e-9))))
    groups = []
    for opt in sorted({c.optimizer for c in configs}):  # a group shares one dense trajectory: one optimizer
        part = [c for c in configs if c.optimizer == opt]
        groups += [part[i:i + cap] for i in range(0, len(part), cap)]
    return groups


def run_shard(rank, world, trace_dir, t0, configs, window, horizons, device, dense_cache, max_configs,
              state_budget_mb, score_names, ratios, group=None, semantics="topk", keep_state=False):
    """One shard's work for one branch point; rank 0 returns the report fragment.
    ``semantics`` picks the rule behind the branch-point and boundary selections; the ranking
    diagnostics of the front block stay on exact top-k under either (``sga/replay_fused.py:1407-1413``).
    ``keep_state`` (single shard) also returns the last group's final weights and supports on the host."""
    t_phase = time.perf_counter()
    phases = {}

    def lap(name):
        nonlocal t_phase
        if torch.device(device).type == "cuda":
            torch.cuda.synchronize(torch.device(device))
        now = time.perf_counter()
        phases[name] = round(phases.get(name, 0.0) + now - t_phase, 4)
        t_phase = now

    # every A/B switch is read once, before any work: an unknown value refuses the run by name
    for name, allowed, dflt in ((ENV_KERNEL, ("on", "off"), "on"), (ENV_SELECT, ("auto", "cpu"), "auto"),
                                (ENV_FRONT_SORT, ("auto", "cpu"), "auto"), (ENV_P1_READ, READ_ARMS, "mmap"), (ENV_FRONT_RANK_BG, ("on", "off"), "on"),
                                (ENV_S0_PROFILE, ("0", "1"), "0")):
        _switch(name, allowed, dflt)
    from .synth import SyntheticSource

    synth = trace_dir if isinstance(trace_dir, SyntheticSource) else None
    info = synth if synth is not None else RC.discover_trace(trace_dir)
    dev = torch.device(device)
    comms = Comms(rank, world, group, dev)
    lo, hi = shard_bounds(info.numel, world, rank)
    steps = info.window(t0, window)
    W = len(steps)
    if W == 0:
        raise ValueError(f"no gradient files at branch point {t0}")
    horizons = sorted(h for h in horizons if h <= W) or [W]
    if synth is not None:
        # generated on the replay device: nothing is read from disk and nothing crosses PCIe
        meta = synth.meta(t0)
        wd_vec = torch.full((hi - lo,), float(meta["param_groups"][0]["weight_decay"]), device=dev)
        w0, m0, v0 = (synth.slice(k_, t0, lo, hi, dev) for k_ in ("w", "m", "v"))
        g0 = synth.slice("g", t0, lo, hi, dev)
    else:
        meta, payload = RC.load_state(info, t0)
        wd_vec = RC.group_vector(info, [g["weight_decay"] for g in meta["param_groups"]], lo, hi)
        w0 = RC.flatten(payload["w"], info, torch.float32, lo, hi)
        m0 = RC.flatten(payload["m"], info, torch.float32, lo, hi)
        v0 = RC.flatten(payload["v"], info, torch.float32, lo, hi)
        g0 = RC.flatten(payload["g"], info, torch.float32, lo, hi)
        del payload
    groups_hp = meta["param_groups"]
    hp = RC.Hyper(wd=None, beta1=groups_hp[0]["adam_beta1"], beta2=groups_hp[0]["adam_beta2"],
                  eps=groups_hp[0]["adam_eps"], clip=meta["clip_grad"])
    use_kernel = dev.type == "cuda" and _switch(ENV_KERNEL, ("on", "off"), "on") == "on"
    gdtype = torch.bfloat16 if info.g_dtype == "bf16" else torch.float32
    # ---- dense arm (element-wise: every shard replays its own slice; cached per shard)
    optimizers = sorted({c.optimizer for c in configs})
    dense, labels = {}, {}
    metas = None
    # the window's gradients, read once for the dense arm, serve the stream below too while they fit the budget
    window_g = None
    keep_bytes = int(float(os.environ.get(ENV_WINDOW_HOST_GIB, "8")) * (1 << 30))
    pt_index = {}  # step file -> parsed archive directory, shared by every prefetcher of this shard (pread arm)
    lap("setup")
    cache_hit = {}
    for opt in optimizers:
        ident = RC.cache_ident(str(trace_dir), t0, W, horizons, "fp32", info.g_dtype, f"fused-v3-{world}-{rank}", opt)
        blob = RC.load_cache(dense_cache, ident) if dense_cache else None
        cache_hit[opt] = blob is not None
        if blob is None and synth is not None:
            logged, metas = synth.gradients(steps, lo, hi, dev), [synth.meta(t) for t in steps]
        elif blob is None:
            pf = GPrefetcher(info, steps, lo, hi, gdtype, pin=dev.type == "cuda", index_cache=pt_index)
            logged, metas = [], []
            for _ in steps:
                _t, gm, flat = pf.get()
                logged.append(flat)
                metas.append(gm)
        if blob is None:
            # the dense arm runs where the sparse arms run (same arithmetic on both sides of the distortion)
            hp_d = RC.Hyper(wd=wd_vec.to(dev), beta1=hp.beta1, beta2=hp.beta2, eps=hp.eps, clip=hp.clip)
            label = torch.zeros_like(w0, device=dev)
            snaps = RC.dense_replay(w0.to(dev), m0.to(dev), v0.to(dev), logged, [gm["lr"][0] for gm in metas], hp_d,
                                    t0, opt, set(horizons), label_out=label)
            # reconstruction check of the logged gradients: the norm of g / coef over the whole vector
            recon = torch.stack([(_unclip(g, gm, dev).double() ** 2).sum() for g, gm in zip(logged, metas)])
            recon = comms.sum_(recon.to(torch.float64)).tolist()
            blob = {"snap_d": snaps, "metas": metas, "label": label, "recon2": recon}  # stays on the replay device
            if dense_cache:
                RC.save_cache(dense_cache, ident, {"snap_d": {h: t.cpu() for h, t in snaps.items()}, "metas": metas,
                                                   "label": label.cpu(), "recon2": recon})
            if synth is None and window_g is None and sum(t.numel() * t.element_size() for t in logged) <= keep_bytes:
                window_g = list(zip(steps, metas, logged))
            del logged
        dense[opt] = blob["snap_d"]
        labels[opt] = blob["label"]
        metas = blob["metas"]
        recon2 = blob["recon2"]
    den = {}
    w0_dev = w0.to(dev)
    for opt in optimizers:
        d = torch.stack([((dense[opt][h].to(dev).double() - w0_dev.double()) ** 2).sum() for h in horizons])
        den[opt] = comms.sum_(d.to(torch.float64)).tolist()
    del w0_dev
    lap("dense_arm")
    # ---- front: branch scores ranked against the label, the window's summed squared gradient-driven step
    # A/B arms of the front block (unknown values raise): selections and / or ranking sorts on host tensors.
    # Radix selection is integer arithmetic and the sorts are stable, so both arms give the same report.
    front_sel = _switch(ENV_SELECT, ("auto", "cpu"), "auto")
    front_sort = _switch(ENV_FRONT_SORT, ("auto", "cpu"), "auto")
    fdev = dev
    if front_sel == "cpu" and dev.type != "cpu":
        if world > 1:
            raise ValueError(f"{ENV_SELECT}=cpu needs a process group that reduces host tensors: one shard, or --device cpu")
        fdev = torch.device("cpu")
    fcomms = comms if fdev == dev else Comms(rank, world, group, fdev)
    hp_dev = RC.Hyper(wd=wd_vec.to(fdev), beta1=hp.beta1, beta2=hp.beta2, eps=hp.eps, clip=hp.clip)
    score_stats, thresholds, label_stats = {}, {}, {}
    entries = shard_entries(info, lo, hi)
    lane = RankLane(rank == 0 and _switch(ENV_FRONT_RANK_BG, ("on", "off"), "on") == "on", fdev)
    for opt in optimizers:
        label_sel = {}
        label_loc = labels[opt].to(fdev)
        label_stats[opt] = shard_stats(label_loc, fcomms)
        for name in score_names:
            sc = RC.replay_score(name, w0.to(fdev), m0.to(fdev), v0.to(fdev), g0.to(fdev), hp_dev, t0 + 1, opt)
            score_stats[(name, opt)] = shard_stats(sc.abs(), fcomms)
            for ratio in ratios:
                k = RC.k_for(info.numel, ratio)
                sel_s, th = shard_select(sc, k, fcomms, return_threshold=True)
                if semantics == "balanced-histogram":  # the trajectory's rule reports the crossing bin's lower edge
                    th = shard_select_balanced(sc, k, fcomms, entries, return_threshold=True)[1]
                thresholds[(name, ratio, opt)] = th
                if ratio not in label_sel:
                    label_sel[ratio] = shard_select(label_loc, k, fcomms)
                sel_l = label_sel[ratio]
                stats = torch.tensor([float((sel_s & sel_l).sum()), float(label_loc[~sel_s].double().sum()),
                                      float(label_loc.double().sum()), float(sc.abs()[~sel_s].double().sum()),
                                      float(sc.abs().double().sum())], dtype=torch.float64, device=fdev)
                fcomms.sum_(stats)
                got_s = fcomms.gather_to_root(sc.abs()[sel_s].float())
                got_l = fcomms.gather_to_root(label_loc[sel_s].float())
                ideal = fcomms.gather_to_root(label_loc[sel_l].float())
                if rank == 0:
                    lane.submit((name, ratio, opt), got_s, got_l, ideal, k, th, stats.tolist(), front_sort == "cpu")
    front = lane.finish()
    del label_sel
    lap("front")
    # ---- stream: groups of configurations, one pass over the window per group
    n_loc = hi - lo
    results, prof = {}, []
    fg = last = None
    for grp in group_configs(configs, max_configs, state_budget_mb, n_loc):
        # one group's state at a time: the previous group is released before the next one is built
        fg = last = None
        if dev.type == "cuda":
            torch.cuda.empty_cache()
        fg = FusedGroup(grp, n_loc, info.numel, dev, comms, hp, wd_vec, w0, m0, v0, t0, W, horizons,
                        dense[grp[0].optimizer],
                        use_kernel, semantics=semantics, entries=entries)
        fg.initial_select(g0)
        lazy = synth.gradients(steps, lo, hi, dev) if synth is not None else None
        pf = None if (window_g is not None or lazy is not None) else GPrefetcher(
            info, steps, lo, hi, gdtype, pin=dev.type == "cuda", index_cache=pt_index)
        for si in range(W):
            if lazy is not None:
                _t, gm, flat = steps[si], synth.meta(steps[si]), lazy[si]
            else:
                _t, gm, flat = window_g[si] if pf is None else pf.get()
            fg.step(StepInput(si, flat, float(gm["grad_norm"]), float(gm["lr"][0])))
        for r, c in enumerate(grp):
            results[c] = {h: math.sqrt(fg.numer[h][r]) / math.sqrt(den[c.optimizer][hi_])
                          if den[c.optimizer][hi_] > 0 else float("nan")
                          for hi_, h in enumerate(horizons)}
        prof.append(dict(fg.stats, configs=len(grp), read_s=pf.read_s if pf is not None else 0.0,
                         comm_ops=comms.ops))
        last = fg
    lap("stream")
    if prof:
        prof[0]["phases_s"] = phases
        prof[0]["arms"] = {"front_sel": front_sel, "front_sort": front_sort, "kernel": "cuda" if use_kernel else "torch",
                           "g_read": _switch(ENV_P1_READ, READ_ARMS, "mmap"),
                           "front_rank_bg": "on" if lane.enabled else "off",
                           "front_rank_s": round(lane.rank_s, 4), "front_rank_wait_s": round(lane.wait_s, 4)}
    if _switch(ENV_S0_PROFILE, ("0", "1"), "0") == "1" and rank == 0:
        for gi, pr in enumerate(prof):
            busy = pr["pass1_s"] + pr["select_s"] + pr["pass3_s"]
            print(f"[fused] S0PROFILE group {gi}: configs={pr['configs']} pass1={pr['pass1_s']:.3f}s "
                  f"select={pr['select_s']:.3f}s ({pr['selects']} selects) pass3={pr['pass3_s']:.3f}s "
                  f"read={pr['read_s']:.3f}s h2d={pr['h2d_bytes'] / 1e9:.3f}GB host_syncs={pr['host_syncs']} "
                  f"comm_ops={pr['comm_ops']} coverage={busy / max(phases.get('stream', 0.0), 1e-9):.2f}", flush=True)
        print(f"[fused] S0PROFILE phases {phases}", flush=True)
    if rank != 0:
        return None
    per_step = []
    for t, gm, r2 in zip(steps, metas, recon2):
        coef, flag = RC.coef_dense_for(gm)
        norm = float(gm.get("grad_norm", float("nan")))
        lrs = [float(x) for x in gm.get("lr", [])]
        mean_lr = sum(lrs) / len(lrs) if lrs else 0.0
        rn = math.sqrt(r2)
        per_step.append({"step": t, "lr": mean_lr, "lr_max_abs_diff": max((abs(x - mean_lr) for x in lrs), default=0.0),
                         "grad_norm": norm, "clip_grad": float(gm.get("clip_grad", 0.0)), "coef_dense": coef,
                         "reconstruct_flag": flag, "recon_grad_norm": rn,
                         "recon_rel_err": (rn - norm) / norm if (math.isfinite(norm) and norm > 0.0) else None})
    return {"t0": t0, "window_len": W, "window_steps": steps, "horizon_steps": horizons, "front": front,
            "score_stats": score_stats, "label_stats": label_stats,
            "label_total": {opt: label_stats[opt]["sum"] for opt in optimizers},
            "per_step": per_step, "dense_cache_hit": cache_hit, "state_meta": meta,
            "results": results, "optimizers": optimizers,
            "den_norm_at_horizon": {opt: {h: math.sqrt(den[opt][i]) for i, h in enumerate(horizons)}
                                    for opt in optimizers},
            "profile": prof, "final_state": (last.W.cpu(), last.SEL.cpu()) if (world == 1 and keep_state) else None}


def _worker(rank, world, port, kwargs, out_path):
    os.environ.update(MASTER_ADDR=os.environ.get("SGA_MASTER_ADDR", "127.0.0.1"),
                      MASTER_PORT=str(os.environ.get("SGA_MASTER_PORT", port)))
    device = kwargs["device"]
    cuda = str(device).startswith("cuda")
    if cuda:
        torch.cuda.set_device(rank % torch.cuda.device_count())
        kwargs = dict(kwargs, device=f"cuda:{rank % torch.cuda.device_count()}")
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    try:
        # the first collective builds the communicator (seconds for NCCL): do it here, so that the
        # engine's phase times, which start in run_shard, are the engine's own
        warm = torch.zeros(1, device=kwargs["device"] if cuda else "cpu")
        dist.all_reduce(warm)
        if cuda:
            torch.cuda.synchronize()
        frag = run_shard(rank, world, **kwargs)
        if rank == 0:
            torch.save(frag, out_path)
    finally:
        dist.destroy_process_group()


def run_fused_branch(trace_dir, t0, configs, window, horizons, world=1, device="cpu", dense_cache=None,
                     max_configs=12, state_budget_mb=0.0, score_names=("abs_g",), ratios=(10.0,),
                     semantics="topk", keep_state=False):
    """Replay one branch point on ``world`` shards; returns rank 0's fragment."""
    kwargs = dict(trace_dir=trace_dir, t0=t0, configs=list(configs), window=window, horizons=list(horizons),
                  device=device, dense_cache=dense_cache, max_configs=max_configs, state_budget_mb=state_budget_mb,
                  score_names=list(score_names), ratios=list(ratios), semantics=semantics, keep_state=keep_state)
    if world == 1:
        return run_shard(0, 1, **kwargs)
    import socket
    import tempfile

    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    fd, out_path = tempfile.mkstemp(suffix=".frag.pt")
    os.close(fd)
    try:
        mp.spawn(_worker, args=(world, port, kwargs, out_path), nprocs=world, join=True)
        return torch.load(out_path, weights_only=False)
    finally:
        if os.path.exists(out_path):
            os.remove(out_path)
