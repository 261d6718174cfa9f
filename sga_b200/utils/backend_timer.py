"""Isolated timing of the communication regions (a breakdown instrument).

Off (the default) costs one ``None`` check per call site. On, every region is
bracketed by a device synchronisation at ``begin`` and an event synchronise on
the calling stream at ``end``, and one JSON line per region goes to
``<dir>/backend_timer_rank{R}.jsonl``::

    {"phase": "sparse"|"prescale"|"fullsync", "wall_ms", "device_ms", "rank",
     "iter", "seq", "ts", ["error"], "backend", ...}

``device_ms`` is the CUDA-event time of the region on the calling stream (not
in the reference's schema; ``wall_ms`` is). The brackets serialise the step
and destroy overlap on purpose: these are isolated durations, never
throughput. Refused with overlapped gradient reduction.
Schema and discipline: ``sga/backend_timer.py:1-200``.
"""
from __future__ import annotations

import functools
import json
import os
import sys
import time

import torch

_STATE = None


class _TimerState:
    def __init__(self, out_dir, rank):
        self.out_dir = out_dir
        self.rank = rank
        self.iter = None
        self.seq = 0
        os.makedirs(out_dir, exist_ok=True)
        self.fh = open(os.path.join(out_dir, f"backend_timer_rank{rank}.jsonl"), "a", buffering=1)

    def write(self, record):
        self.seq += 1
        self.fh.write(json.dumps(record, sort_keys=True) + "\n")


def active() -> bool:
    return _STATE is not None


def configure(out_dir, rank) -> None:
    global _STATE
    if _STATE is not None:
        raise RuntimeError(f"sga_backend_timer already configured for rank {_STATE.rank} ({_STATE.out_dir!r})")
    if not isinstance(out_dir, str) or not out_dir.strip():
        raise ValueError(f"sga_backend_timer must be a non-empty output directory path (got {out_dir!r})")
    _STATE = _TimerState(out_dir, rank)
    print(f"[SGA] backend_timer active: rank {rank} -> {_STATE.fh.name} (isolated comm timing; not e2e numbers)",
          flush=True)


def set_iter(step) -> None:
    if _STATE is not None:
        _STATE.iter = step


def reset() -> None:
    global _STATE
    if _STATE is not None:
        _STATE.fh.close()
        _STATE = None


def begin():
    if _STATE is None:
        return None
    ev = None
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream())
    return (time.perf_counter(), ev)


def end(token, phase, **fields) -> None:
    if token is None or _STATE is None:
        return
    t0, ev0 = token
    device_ms = None
    if ev0 is not None:
        ev1 = torch.cuda.Event(enable_timing=True)
        ev1.record(torch.cuda.current_stream())
        ev1.synchronize()
        device_ms = round(ev0.elapsed_time(ev1), 6)
    record = {"phase": phase, "wall_ms": round((time.perf_counter() - t0) * 1e3, 6), "rank": _STATE.rank,
              "iter": _STATE.iter, "seq": _STATE.seq, "ts": round(time.time(), 6)}
    if device_ms is not None:
        record["device_ms"] = device_ms
    if sys.exc_info()[0] is not None:
        record["error"] = True
    record.update(fields)
    _STATE.write(record)


def wrap_finish_grad_sync(chunk_cls) -> None:
    """Class-level wrap of ``finish_grad_sync`` (the ``fullsync`` phase). Idempotent."""
    marker = "_sga_backend_timer"
    orig = getattr(chunk_cls, "finish_grad_sync")
    if getattr(orig, marker, False):
        return

    @functools.wraps(orig)
    def finish_grad_sync(self, *args, **kwargs):
        if _STATE is None:
            return orig(self, *args, **kwargs)
        cfg = getattr(self, "ddp_config", None)
        if getattr(cfg, "overlap_grad_reduce", False):
            raise RuntimeError("sga_backend_timer refuses overlap_grad_reduce=true: overlapped grad sync bypasses "
                               "finish_grad_sync, so the fullsync phase would record nothing real")
        token = begin()
        try:
            return orig(self, *args, **kwargs)
        finally:
            end(token, "fullsync", backend="ddp", bucket=None)

    setattr(finish_grad_sync, marker, True)
    chunk_cls.finish_grad_sync = finish_grad_sync


def install_fullsync_wrap() -> None:
    if _STATE is None:
        return
    from ..runtime.ddp import DataParallel

    wrap_finish_grad_sync(DataParallel)
