"""Pre-commit trace collector: the data source of the offline replay.

Inside configured windows rank 0 dumps, right before the optimizer commit,
the step's post-clip gradient ``g`` (fp32 or bf16) and, at branch points, the
full fp32 state ``w / m / v / g``. Nothing the training step consumes is ever
written to. Files (all ``torch.save``)::

    catalog.pt             {"meta", "catalog": {name: {shape, dtype, param_group}}, "g_dtype"}
    step_NNNNNN_state.pt   {"meta", "payload": {"w": {name: t}, "m": ..., "v": ..., "g": ...}}
    step_NNNNNN_g.pt       {"meta", "payload": {name: t}}

``NNNNNN`` is the number of commits already applied when the dump is taken
(the first optimizer step dumps as step 0), an absolute number, so a resumed
run continues the sequence instead of overwriting it. Parameter names have
leading ``module.`` wrappers stripped; the flat order is the catalog key
order. A resumed run must match the catalog on disk (names, shapes, dtypes,
groups, ``g_dtype``) or the collector refuses.

Three gradient paths: synchronous (default); ``async`` with ``cpu_snapshot``
(blocking independent CPU copy, background serialisation and write); ``async``
with ``pinned_cuda`` (bf16 cast on the GPU when asked, non-blocking D2H on a
dedicated stream into a bounded pool of reusable pinned slots, stream
synchronised before the optimizer mutates anything, file writes in the
background). The writer enforces a queue depth and a host-memory budget,
writes ``<target>.tmp.<pid>.<seq>`` then renames, latches its first error
(every later call fails closed), removes stale temporaries of dead
processes, keeps per-phase timers and drains at exit with a bound.
Format and behaviour follow ``sga/trace.py:25-1063``.
"""
from __future__ import annotations

import atexit
import os
import threading
import time
from collections import deque
from typing import Optional

import torch

from .config.validation import parse_branch_points  # noqa: F401  (re-exported)

PHASES = ("snapshot", "d2h_submit", "d2h_sync", "slot_wait", "cast", "write", "drain")


def canonical_name(name: str) -> str:
    while name.startswith("module."):
        name = name[len("module."):]
    return name


def _dump_phase(engine) -> str:
    if getattr(engine, "_shadow", False):
        return "shadow"
    return "live_full" if getattr(engine, "_step_full", True) in (True, None) else "live_sparse"


def _catalog_mismatch(old, expected: dict):
    if not isinstance(old, dict):
        return ("catalog", "no catalog dict on disk")
    if list(old.keys()) != list(expected.keys()):
        missing = [k for k in expected if k not in old]
        extra = [k for k in old if k not in expected]
        return ("names", f"missing {missing[:3]} extra {extra[:3]} or a different order")
    for k, want in expected.items():
        have = old[k]
        for field in ("shape", "dtype", "param_group"):
            if field in have and have[field] != want[field]:
                return (k, f"{field} {have[field]} on disk vs {want[field]} this run")
    return None


def _process_alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    return True


def _record_phase(stats: dict, phase: str, elapsed: float) -> None:
    stats[f"{phase}_n"] = stats.get(f"{phase}_n", 0) + 1
    stats[f"{phase}_s"] = stats.get(f"{phase}_s", 0.0) + elapsed
    stats[f"{phase}_max_s"] = max(stats.get(f"{phase}_max_s", 0.0), elapsed)


def _payload_bytes(payload: dict) -> int:
    return sum(t.numel() * t.element_size() for t in payload.values())


class TraceWriterError(RuntimeError):
    """The background writer failed earlier; tracing is closed."""


class _PendingWrite:
    def __init__(self, step, meta, payload, reservation, seq, on_done=None):
        self.step, self.meta, self.payload = step, meta, payload
        self.reservation, self.seq, self.on_done = reservation, seq, on_done


class _AsyncGradWriter:
    def __init__(self, dir: str, queue_depth: int, max_workset_bytes: int, worker_count: int = 1):
        self.dir = dir
        self.queue_depth = int(queue_depth)
        self.max_workset_bytes = int(max_workset_bytes)
        self.worker_count = int(worker_count)
        self._cv = threading.Condition(threading.Lock())
        self._queue = deque()
        self._in_flight = 0          # queued + being written
        self._reserved = 0
        self._error: Optional[BaseException] = None
        self._closing = False
        self._threads = []
        self._seq = 0
        self.stats = {}
        self._started = False

    # ------------------------------------------------------------ lifecycle
    def start(self) -> None:
        if self._started:
            return
        os.makedirs(self.dir, exist_ok=True)
        self._cleanup_stale_tmp()
        for i in range(self.worker_count):
            t = threading.Thread(target=self._writer_loop, name=f"sga-trace-writer-{i}", daemon=True)
            t.start()
            self._threads.append(t)
        atexit.register(self._atexit_close)
        self._started = True

    def _cleanup_stale_tmp(self) -> None:
        """Remove ``*.tmp.<pid>.<seq>`` left by processes that no longer exist."""
        for name in os.listdir(self.dir):
            parts = name.split(".tmp.")
            if len(parts) != 2:
                continue
            try:
                pid = int(parts[1].split(".")[0])
            except ValueError:
                continue
            if pid != os.getpid() and not _process_alive(pid):
                try:
                    os.remove(os.path.join(self.dir, name))
                except OSError:
                    pass

    def check_open(self) -> None:
        if self._error is not None:
            raise TraceWriterError(f"trace writer failed earlier: {self._error!r}") from self._error
        if self._closing:
            raise TraceWriterError("trace writer is closed")

    # --------------------------------------------------------- back-pressure
    def reserve(self, nbytes: int) -> None:
        """Block until one more item of ``nbytes`` fits the depth and byte budgets."""
        if nbytes > self.max_workset_bytes:
            raise ValueError(f"trace: one gradient item needs {nbytes} bytes of host memory, above "
                             f"sga_trace_async_max_workset_gib ({self.max_workset_bytes} bytes)")
        t0 = time.perf_counter()
        with self._cv:
            while True:
                self.check_open()
                if self._in_flight < self.queue_depth and self._reserved + nbytes <= self.max_workset_bytes:
                    self._in_flight += 1
                    self._reserved += nbytes
                    break
                self._cv.wait(0.05)
        _record_phase(self.stats, "slot_wait", time.perf_counter() - t0)

    def release(self, nbytes: int) -> None:
        with self._cv:
            self._in_flight -= 1
            self._reserved -= nbytes
            self._cv.notify_all()

    def submit(self, step, meta, payload, reservation, on_done=None) -> None:
        with self._cv:
            self.check_open()
            self._seq += 1
            self._queue.append(_PendingWrite(step, meta, payload, reservation, self._seq, on_done))
            self._cv.notify_all()

    def existing_matches(self, step: int, payload: dict) -> bool:
        """True when the target file exists and holds bitwise the same payload."""
        path = os.path.join(self.dir, f"step_{step:06d}_g.pt")
        if not os.path.exists(path):
            return False
        try:
            old = torch.load(path, weights_only=False)["payload"]
        except Exception:
            return False
        if list(old.keys()) != list(payload.keys()):
            return False
        return all(old[k].dtype == payload[k].dtype and torch.equal(old[k], payload[k]) for k in payload)

    # -------------------------------------------------------------- workers
    def _writer_loop(self) -> None:
        while True:
            with self._cv:
                while not self._queue and not self._closing:
                    self._cv.wait(0.1)
                if not self._queue and self._closing:
                    return
                item = self._queue.popleft()
            try:
                if self._error is None:
                    self._write_one(item)
            except BaseException as e:  # latch the first failure
                with self._cv:
                    if self._error is None:
                        self._error = e
            finally:
                if item.on_done is not None:
                    try:
                        item.on_done()
                    except Exception:
                        pass
                self.release(item.reservation)

    def _write_one(self, item: _PendingWrite) -> None:
        t0 = time.perf_counter()
        target = os.path.join(self.dir, f"step_{item.step:06d}_g.pt")
        tmp = f"{target}.tmp.{os.getpid()}.{item.seq}"
        try:
            torch.save({"meta": item.meta, "payload": item.payload}, tmp)
            os.replace(tmp, target)
        finally:
            if os.path.exists(tmp):
                try:
                    os.remove(tmp)
                except OSError:
                    pass
        _record_phase(self.stats, "write", time.perf_counter() - t0)

    def close(self, timeout: Optional[float] = None, raise_error: bool = True) -> dict:
        """Drain the queue (bounded by ``timeout``) and stop the workers."""
        t0 = time.perf_counter()
        deadline = None if timeout is None else t0 + timeout
        with self._cv:
            while (self._queue or self._in_flight > 0) and self._error is None:
                if deadline is not None and time.perf_counter() > deadline:
                    break
                self._cv.wait(0.05)
            self._closing = True
            self._cv.notify_all()
        for t in self._threads:
            t.join(None if deadline is None else max(0.0, deadline - time.perf_counter()))
        _record_phase(self.stats, "drain", time.perf_counter() - t0)
        if raise_error and self._error is not None:
            raise TraceWriterError(f"trace writer failed: {self._error!r}") from self._error
        return dict(self.stats)

    def drain(self) -> None:
        """Wait until everything submitted so far is on disk (workers stay up)."""
        t0 = time.perf_counter()
        with self._cv:
            while (self._queue or self._in_flight > 0) and self._error is None:
                self._cv.wait(0.05)
        _record_phase(self.stats, "drain", time.perf_counter() - t0)
        self.check_open()

    def _atexit_close(self) -> None:
        try:
            if not self._closing:
                self.close(timeout=60.0, raise_error=False)
        except Exception:
            pass


class TraceCollector:
    def __init__(self, dir: str, branch_points, window: int, dump_dtype: str = "fp32", async_enabled: bool = False,
                 async_backend: str = "cpu_snapshot", async_queue_depth: int = 2, async_worker_count: int = 1,
                 async_max_workset_gib: float = 16.0):
        if dump_dtype not in ("fp32", "bf16"):
            raise ValueError(f"sga_trace_dump_dtype must be 'fp32' or 'bf16' (got {dump_dtype!r})")
        if async_backend not in ("cpu_snapshot", "pinned_cuda"):
            raise ValueError(f"sga_trace_async_backend must be 'cpu_snapshot' or 'pinned_cuda' (got {async_backend!r})")
        if async_backend == "pinned_cuda" and not async_enabled:
            raise ValueError("sga_trace_async_backend='pinned_cuda' requires sga_trace_async=true")
        if async_worker_count > async_queue_depth:
            raise ValueError("sga_trace_async_worker_count must be <= sga_trace_async_queue_depth")
        self.dir = dir
        self.branch_points = parse_branch_points(branch_points) or []
        self.window = int(window)
        self.dump_dtype = dump_dtype
        self.async_enabled = bool(async_enabled)
        self.async_backend = async_backend
        self.queue_depth = int(async_queue_depth)
        self.worker_count = int(async_worker_count)
        self.max_workset_bytes = int(float(async_max_workset_gib) * (1 << 30))
        self._entries = None            # [(name, record, group index)]
        self._catalog_written = False
        self._writer: Optional[_AsyncGradWriter] = None
        self._drained = False
        self._copy_stream = None
        self._slot_cv = threading.Condition(threading.Lock())
        self._pinned_slots = []
        self._free_slots = deque()
        self.stats = {}

    # ------------------------------------------------------------- calendar
    def wants(self, step: int):
        """``(want_state, want_g)`` for a dump step (= commits applied so far)."""
        want_state = step in self.branch_points
        want_g = want_state or any(t0 <= step < t0 + self.window for t0 in self.branch_points)
        return want_state, want_g

    @property
    def _last_g_step(self) -> Optional[int]:
        return self.branch_points[-1] + self.window - 1 if self.branch_points else None

    # ----------------------------------------------------------------- bind
    def _bind(self, records) -> None:
        entries, seen = [], set()
        for rec in records:
            name = canonical_name(rec.name)
            if name in seen:
                raise ValueError(f"trace: duplicate canonical parameter name '{name}'")
            seen.add(name)
            entries.append((name, rec, int(rec.group)))
        self._entries = entries

    def _meta(self, optimizer, step: int, grad_norm, phase) -> dict:
        cfg = optimizer.config
        groups = []
        for g in optimizer.param_groups:
            betas = g.get("betas", (0.9, 0.999))
            groups.append({"lr": float(g.get("lr", 0.0)), "weight_decay": float(g.get("weight_decay", 0.0)),
                           "adam_beta1": float(betas[0]), "adam_beta2": float(betas[1]),
                           "adam_eps": float(g.get("eps", 1e-8))})
        return {"step": step, "phase": phase, "lr": [g["lr"] for g in groups],
                "grad_norm": float(grad_norm) if grad_norm is not None else float("nan"),
                "clip_grad": float(getattr(cfg, "clip_grad", 0.0) or 0.0),
                "weight_decay": float(getattr(cfg, "weight_decay", 0.0)),
                "adam_beta1": float(getattr(cfg, "adam_beta1", 0.9)),
                "adam_beta2": float(getattr(cfg, "adam_beta2", 0.999)),
                "adam_eps": float(getattr(cfg, "adam_eps", 1e-8)), "param_groups": groups}

    # ------------------------------------------------------------ dump slot
    @torch.no_grad()
    def maybe_dump(self, engine, optimizer, step: int, grad_norm) -> None:
        want_state, want_g = self.wants(step)
        if not (want_state or want_g):
            self._final_drain(step)
            return
        if engine._rank != 0:
            return
        records = engine._refresh_records(optimizer)
        if self._entries is None:
            self._bind(records)
        else:
            self._entries = [(n, r, gi) for (n, _old, gi), r in zip(self._entries, records)]
        os.makedirs(self.dir, exist_ok=True)
        meta = self._meta(optimizer, step, grad_norm, _dump_phase(engine))
        if not self._catalog_written:
            self._write_or_verify_catalog(meta)
        if want_state:
            self._dump_state(step, meta)
        if want_g:
            if not self.async_enabled:
                self._dump_grad(step, meta)
            elif self.async_backend == "pinned_cuda" and self._entries[0][1].grad.is_cuda:
                self._dump_grad_pinned_cuda(step, meta)
            else:
                self._dump_grad_async(step, meta)
        self._final_drain(step)

    def _write_or_verify_catalog(self, meta) -> None:
        path = os.path.join(self.dir, "catalog.pt")
        catalog = {name: {"shape": list(rec.main_param.shape), "dtype": str(rec.main_param.dtype), "param_group": gi}
                   for name, rec, gi in self._entries}
        if os.path.exists(path):
            on_disk = torch.load(path, weights_only=False)
            old = on_disk.get("catalog") if isinstance(on_disk, dict) else None
            mismatch = _catalog_mismatch(old, catalog)
            if mismatch is None and on_disk.get("g_dtype", "fp32") != self.dump_dtype:
                mismatch = ("g_dtype", f"{on_disk.get('g_dtype', 'fp32')} on disk vs {self.dump_dtype} this run")
            if mismatch is not None:
                raise ValueError(f"trace: existing catalog.pt in {self.dir} does not match this run "
                                 f"({mismatch[1]} for {mismatch[0]})")
        else:
            torch.save({"meta": meta, "catalog": catalog, "g_dtype": self.dump_dtype}, path)
        self._catalog_written = True

    def _cast(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(torch.bfloat16) if self.dump_dtype == "bf16" else t

    def _dump_state(self, step: int, meta: dict) -> None:
        payload = {"w": {}, "m": {}, "v": {}, "g": {}}
        for name, rec, _gi in self._entries:
            payload["w"][name] = rec.main_param.detach().float().cpu().clone()
            payload["m"][name] = rec.m.detach().float().cpu().clone()
            payload["v"][name] = rec.v.detach().float().cpu().clone()
            payload["g"][name] = rec.grad.detach().float().cpu().clone()
        m = dict(meta)
        m["state_absent"] = False
        path = os.path.join(self.dir, f"step_{step:06d}_state.pt")
        tmp = f"{path}.tmp.{os.getpid()}.0"
        torch.save({"meta": m, "payload": payload}, tmp)
        os.replace(tmp, path)

    def _dump_grad(self, step: int, meta: dict) -> None:
        payload = {name: self._cast(rec.grad.detach()).cpu().clone() for name, rec, _gi in self._entries}
        path = os.path.join(self.dir, f"step_{step:06d}_g.pt")
        tmp = f"{path}.tmp.{os.getpid()}.0"
        torch.save({"meta": meta, "payload": payload}, tmp)
        os.replace(tmp, path)

    # ---------------------------------------------------------- async paths
    def _ensure_writer(self) -> _AsyncGradWriter:
        if self._writer is None:
            self._writer = _AsyncGradWriter(self.dir, self.queue_depth, self.max_workset_bytes, self.worker_count)
            self._writer.start()
        self._writer.check_open()
        return self._writer

    def _item_bytes(self) -> int:
        per = 2 if self.dump_dtype == "bf16" else 4
        return sum(rec.grad.numel() for _n, rec, _g in self._entries) * per

    def _dump_grad_async(self, step: int, meta: dict) -> None:
        """cpu_snapshot: reserve 2x the payload (snapshot + serialisation transient),
        take a blocking independent CPU copy, hand it to the writer."""
        w = self._ensure_writer()
        nbytes = 2 * self._item_bytes()
        w.reserve(nbytes)
        try:
            t0 = time.perf_counter()
            payload = {name: self._cast(rec.grad.detach()).cpu().clone() for name, rec, _gi in self._entries}
            _record_phase(w.stats, "snapshot", time.perf_counter() - t0)
            if w.existing_matches(step, payload):
                w.release(nbytes)
                return
            if os.path.exists(os.path.join(self.dir, f"step_{step:06d}_g.pt")):
                raise ValueError(f"trace: step_{step:06d}_g.pt exists with different contents; refusing to overwrite")
        except BaseException:
            w.release(nbytes)
            raise
        w.submit(step, meta, payload, nbytes)

    def _acquire_pinned_slot(self, writer):
        """A reusable pinned buffer holding one whole gradient item; the pool is
        sized on first use against the host-memory cap."""
        item = self._item_bytes()
        if not self._pinned_slots:
            n = min(self.queue_depth, max(0, self.max_workset_bytes // max(item, 1)))
            if n < self.worker_count:
                raise ValueError(f"trace: sga_trace_async_max_workset_gib allows {n} pinned slot(s) of {item} bytes, "
                                 f"fewer than the {self.worker_count} writer(s)")
            dt = torch.bfloat16 if self.dump_dtype == "bf16" else torch.float32
            total = sum(rec.grad.numel() for _n, rec, _g in self._entries)
            for _ in range(n):
                buf = torch.empty(total, dtype=dt, pin_memory=True)
                self._pinned_slots.append(buf)
                self._free_slots.append(buf)
        t0 = time.perf_counter()
        with self._slot_cv:
            while not self._free_slots:
                writer.check_open()
                self._slot_cv.wait(0.05)
            slot = self._free_slots.popleft()
        _record_phase(writer.stats, "slot_wait", time.perf_counter() - t0)
        return slot

    def _release_pinned_slot(self, slot) -> None:
        with self._slot_cv:
            self._free_slots.append(slot)
            self._slot_cv.notify_all()

    def _dump_grad_pinned_cuda(self, step: int, meta: dict) -> None:
        w = self._ensure_writer()
        dev = self._entries[0][1].grad.device
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=dev)
        slot = self._acquire_pinned_slot(w)
        w.reserve(0)
        t0 = time.perf_counter()
        self._copy_stream.wait_stream(torch.cuda.current_stream(dev))
        payload, off = {}, 0
        with torch.cuda.stream(self._copy_stream):
            for name, rec, _gi in self._entries:
                n = rec.grad.numel()
                view = slot[off:off + n].view(rec.grad.shape)
                view.copy_(self._cast(rec.grad.detach()), non_blocking=True)
                payload[name] = view
                off += n
        _record_phase(w.stats, "d2h_submit", time.perf_counter() - t0)
        t0 = time.perf_counter()
        self._copy_stream.synchronize()   # the optimizer may mutate the gradients after this point
        _record_phase(w.stats, "d2h_sync", time.perf_counter() - t0)
        w.submit(step, meta, payload, 0, on_done=lambda s=slot: self._release_pinned_slot(s))

    # ---------------------------------------------------------------- drain
    def _final_drain(self, step: int) -> None:
        last = self._last_g_step
        if self._writer is None or self._drained or last is None or step < last:
            return
        self._writer.drain()
        self._drained = True

    def close(self, timeout: Optional[float] = None) -> dict:
        if self._writer is not None:
            self.stats.update(self._writer.close(timeout=timeout))
        return dict(self.stats)

    def diagnostics(self) -> dict:
        out = dict(self.stats)
        if self._writer is not None:
            out.update(self._writer.stats)
        return out
