"""Isolated timing of the communication regions: a breakdown instrument, never
a throughput number.

``--sga-backend-timer <dir>`` switches it on. A timed region is a ``with``
block::

    with backend_timer.region("sparse", backend=name, bucket=i, k=k):
        ... launch the bucket's synchronisation ...

Entering drains the device (so the region starts on an idle GPU), leaving
records a CUDA event on the calling stream and waits for it; one JSON line per
region is appended to ``<dir>/backend_timer_rank{R}.jsonl``::

    {"phase": "sparse" | "prescale" | "fullsync", "wall_ms", "rank", "iter",
     "seq", "ts", ["error"], "backend", ... , ["device_ms"]}

which is the record of ``sga/backend_timer.py:116-155`` plus ``device_ms``, the
CUDA-event duration of the region on its stream. The brackets serialise the
step and destroy every overlap on purpose. Switched off (the default) a region
costs one ``None`` test. Dense full syncs are timed by wrapping the
data-parallel chunk class's ``finish_grad_sync`` (``time_full_syncs``), which
is refused together with overlapped gradient reduction: an overlapped sync
never passes through that method.
"""
from __future__ import annotations

import contextlib
import functools
import json
import os
import time

import torch


class BackendTimer:
    """One rank's recorder: the open JSONL file, the current step and the running sequence number."""

    def __init__(self, out_dir: str, rank: int):
        if not isinstance(out_dir, str) or not out_dir.strip():
            raise ValueError(f"sga_backend_timer must be a non-empty output directory path (got {out_dir!r})")
        os.makedirs(out_dir, exist_ok=True)
        self.out_dir, self.rank = out_dir, rank
        self.step = None
        self.seq = 0
        self.path = os.path.join(out_dir, f"backend_timer_rank{rank}.jsonl")
        self._fh = open(self.path, "a", buffering=1)

    def close(self) -> None:
        self._fh.close()

    @contextlib.contextmanager
    def region(self, phase: str, **fields):
        cuda = torch.cuda.is_available()
        start = None
        if cuda:
            torch.cuda.synchronize()
            start = torch.cuda.Event(enable_timing=True)
            start.record(torch.cuda.current_stream())
        t0 = time.perf_counter()
        failed = False
        try:
            yield
        except BaseException:
            failed = True
            raise
        finally:
            device_ms = None
            if start is not None:
                stop = torch.cuda.Event(enable_timing=True)
                stop.record(torch.cuda.current_stream())
                stop.synchronize()
                device_ms = round(start.elapsed_time(stop), 6)
            rec = {"phase": phase, "wall_ms": round((time.perf_counter() - t0) * 1e3, 6), "rank": self.rank,
                   "iter": self.step, "seq": self.seq, "ts": round(time.time(), 6)}
            if device_ms is not None:
                rec["device_ms"] = device_ms
            if failed:
                rec["error"] = True
            rec.update(fields)
            self.seq += 1
            self._fh.write(json.dumps(rec, sort_keys=True) + "\n")


_timer: BackendTimer | None = None
_NO_REGION = contextlib.nullcontext()


def enabled() -> bool:
    return _timer is not None


def enable(out_dir, rank) -> None:
    global _timer
    if _timer is not None:
        raise RuntimeError(f"sga_backend_timer already configured for rank {_timer.rank} ({_timer.out_dir!r})")
    _timer = BackendTimer(out_dir, rank)
    print(f"[SGA] backend_timer active: rank {rank} -> {_timer.path} (isolated comm timing; not e2e numbers)",
          flush=True)


def disable() -> None:
    global _timer
    if _timer is not None:
        _timer.close()
        _timer = None


def at_step(step) -> None:
    if _timer is not None:
        _timer.step = step


def region(phase: str, **fields):
    """Context manager around one communication region; a no-op while the timer is off."""
    return _NO_REGION if _timer is None else _timer.region(phase, **fields)


def time_full_syncs(chunk_cls=None) -> None:
    """Time the dense full sync of ``chunk_cls`` (default: this framework's ``DataParallel``) as the
    ``fullsync`` phase by wrapping its ``finish_grad_sync`` once. Does nothing while the timer is off."""
    if _timer is None:
        return
    if chunk_cls is None:
        from ..runtime.ddp import DataParallel as chunk_cls
    inner = chunk_cls.finish_grad_sync
    if getattr(inner, "_timed_as_fullsync", False):
        return

    @functools.wraps(inner)
    def finish_grad_sync(self, *args, **kwargs):
        if _timer is None:
            return inner(self, *args, **kwargs)
        if getattr(getattr(self, "ddp_config", None), "overlap_grad_reduce", False):
            raise RuntimeError("sga_backend_timer refuses overlap_grad_reduce=true: overlapped grad sync bypasses "
                               "finish_grad_sync, so the fullsync phase would record nothing real")
        with _timer.region("fullsync", backend="ddp", bucket=None):
            return inner(self, *args, **kwargs)

    finish_grad_sync._timed_as_fullsync = True
    chunk_cls.finish_grad_sync = finish_grad_sync
