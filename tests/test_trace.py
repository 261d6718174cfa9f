"""Trace capture: file set, numbering, formats, async writer behaviour and
failure latching, catalog identity on resume, bf16 conversion."""
import os
import threading
import time

import pytest
import torch

from sga_b200 import trace as T
from sga_b200.runtime.trainer import Trainer, default_args
from sga_b200.trace_convert import convert_trace


def _trainer(tmp, **kw):
    base = dict(model="test_tiny", micro_batch_size=2, global_batch_size=2, train_iters=8, device="cpu", lr=1e-3,
                sga_bucket_elems=30000, log_interval=0, sga_enabled=True, sga_shadow=True, sga_score="abs_g",
                sga_selection_method="histogram", sga_selection_histogram_mode="balanced",
                sga_selection_ratio_percent=10.0, sga_backend="torch_pipelined_index", sga_cycle_period=2,
                sga_trace_dir=str(tmp), sga_trace_branch_points="2", sga_trace_window=3)
    base.update(kw)
    return Trainer(default_args(**base), quiet=True)


def _run(tr, n=7):
    for s in range(n):
        tr.train_step(tr.host_batch(s))
    tr.close()


def test_sync_trace_files_and_format(tmp_path):
    tr = _trainer(tmp_path)
    _run(tr)
    names = sorted(os.listdir(tmp_path))
    assert names == ["catalog.pt", "step_000002_g.pt", "step_000002_state.pt", "step_000003_g.pt", "step_000004_g.pt"]
    cat = torch.load(tmp_path / "catalog.pt", weights_only=False)
    assert cat["g_dtype"] == "fp32"
    keys = list(cat["catalog"].keys())
    assert keys == [s.name for s in tr.model.arena.slots]
    ent = cat["catalog"][keys[0]]
    assert set(ent) == {"shape", "dtype", "param_group"} and ent["dtype"] == "torch.float32"
    st = torch.load(tmp_path / "step_000002_state.pt", weights_only=False)
    assert set(st["payload"]) == {"w", "m", "v", "g"} and st["meta"]["state_absent"] is False
    assert st["meta"]["step"] == 2 and st["meta"]["phase"] == "shadow"
    assert len(st["meta"]["param_groups"]) == 2
    g = torch.load(tmp_path / "step_000003_g.pt", weights_only=False)
    assert list(g["payload"].keys()) == keys and g["payload"][keys[0]].dtype == torch.float32
    # the state's g equals the g file of the same step
    g2 = torch.load(tmp_path / "step_000002_g.pt", weights_only=False)
    assert all(torch.equal(st["payload"]["g"][k], g2["payload"][k]) for k in keys)
    # two commits were applied before the step-2 dump
    assert float(st["payload"]["m"][keys[0]].abs().sum()) > 0


def test_trace_numbering_is_commits_applied(tmp_path):
    tr = _trainer(tmp_path, sga_trace_branch_points="0", sga_trace_window=1)
    _run(tr, 2)
    st = torch.load(tmp_path / "step_000000_state.pt", weights_only=False)
    assert all(float(v.abs().sum()) == 0.0 for v in st["payload"]["m"].values()), "step 0 = no commit applied yet"


@pytest.mark.parametrize("workers,depth", [(1, 2), (2, 2)])
def test_async_cpu_snapshot_matches_sync(tmp_path, workers, depth):
    a, b = tmp_path / "sync", tmp_path / "async"
    _run(_trainer(a))
    _run(_trainer(b, sga_trace_async=True, sga_trace_async_queue_depth=depth,
                  sga_trace_async_worker_count=workers))
    for name in sorted(os.listdir(a)):
        if name.endswith("_g.pt"):
            x = torch.load(a / name, weights_only=False)["payload"]
            y = torch.load(b / name, weights_only=False)["payload"]
            assert all(torch.equal(x[k], y[k]) for k in x)
    assert not [n for n in os.listdir(b) if ".tmp." in n]


def test_bf16_dump_equals_converted_fp32(tmp_path):
    a, b, c = tmp_path / "fp32", tmp_path / "bf16", tmp_path / "conv"
    _run(_trainer(a))
    _run(_trainer(b, sga_trace_dump_dtype="bf16"))
    res = convert_trace(str(a), str(c))
    assert res["g_files"] == 3 and res["state_files"] == 1
    assert torch.load(c / "catalog.pt", weights_only=False)["g_dtype"] == "bf16"
    for name in ("step_000002_g.pt", "step_000004_g.pt"):
        x = torch.load(b / name, weights_only=False)["payload"]
        y = torch.load(c / name, weights_only=False)["payload"]
        assert all(x[k].dtype == torch.bfloat16 and torch.equal(x[k], y[k]) for k in x)
    # a destination that holds files is refused; --overwrite purges its trace files first; ranges are half-open
    with pytest.raises(ValueError, match="not empty"):
        convert_trace(str(a), str(c))
    with pytest.raises(ValueError, match="must differ"):
        convert_trace(str(a), str(a))
    res = convert_trace(str(a), str(c), overwrite=True, from_step=3, to_step=4)
    assert res["g_files"] == 1 and res["state_files"] == 0
    assert sorted(os.listdir(c)) == ["catalog.pt", "step_000003_g.pt"]
    again = convert_trace(str(c), str(tmp_path / "twice"))  # already bf16: an identical copy, with a warning
    assert again["g_files"] == 1


def test_resume_catalog_identity(tmp_path):
    _run(_trainer(tmp_path))
    with pytest.raises(ValueError, match="g_dtype"):
        _run(_trainer(tmp_path, sga_trace_dump_dtype="bf16"))
    with pytest.raises(ValueError, match="does not match"):
        _run(_trainer(tmp_path, model="test_tiny_qk"))


def test_writer_backpressure_and_error_latch(tmp_path):
    w = T._AsyncGradWriter(str(tmp_path), queue_depth=1, max_workset_bytes=1000, worker_count=1)
    gate = threading.Event()
    orig = w._write_one

    def slow(item):
        gate.wait(5)
        orig(item)

    w._write_one = slow
    w.start()
    w.reserve(400)
    w.submit(0, {"step": 0}, {"a": torch.zeros(4)}, 400)
    blocked = []

    def second():
        w.reserve(400)   # depth 1: must wait for the first item
        blocked.append(time.perf_counter())
        w.submit(1, {"step": 1}, {"a": torch.ones(4)}, 400)

    t = threading.Thread(target=second)
    t0 = time.perf_counter()
    t.start()
    time.sleep(0.3)
    assert not blocked, "the second reservation must block while the queue is full"
    gate.set()
    t.join(5)
    assert blocked and blocked[0] - t0 >= 0.25
    w.drain()
    assert sorted(n for n in os.listdir(tmp_path)) == ["step_000000_g.pt", "step_000001_g.pt"]
    with pytest.raises(ValueError):
        w.reserve(2000)  # above the byte budget
    # failure injection: the first error is latched and every later call fails closed

    def boom(item):
        raise OSError("disk full")

    w._write_one = boom
    w.reserve(10)
    w.submit(2, {}, {"a": torch.zeros(1)}, 10)
    with pytest.raises(T.TraceWriterError):
        w.drain()
    with pytest.raises(T.TraceWriterError):
        w.reserve(10)
    with pytest.raises(T.TraceWriterError):
        w.close(timeout=2)
    assert not [n for n in os.listdir(tmp_path) if ".tmp." in n]


def test_stale_tmp_cleanup(tmp_path):
    dead = tmp_path / "step_000009_g.pt.tmp.999999.1"
    dead.write_bytes(b"x")
    mine = tmp_path / f"step_000009_g.pt.tmp.{os.getpid()}.1"
    mine.write_bytes(b"x")
    w = T._AsyncGradWriter(str(tmp_path), 1, 1000, 1)
    w.start()
    assert not dead.exists() and mine.exists()
    w.close(timeout=2)


@pytest.mark.gpu
def test_pinned_cuda_backend_matches_sync(tmp_path):
    a, b = tmp_path / "sync", tmp_path / "pinned"
    _run(_trainer(a, device="cuda:0"))
    tr = _trainer(b, device="cuda:0", sga_trace_async=True, sga_trace_async_backend="pinned_cuda",
                  sga_trace_dump_dtype="fp32")
    _run(tr)
    for name in sorted(os.listdir(a)):
        if name.endswith("_g.pt"):
            x = torch.load(a / name, weights_only=False)["payload"]
            y = torch.load(b / name, weights_only=False)["payload"]
            assert all(torch.equal(x[k], y[k]) for k in x)
    d = tr.engine._trace.diagnostics()
    assert d.get("d2h_submit_n", 0) == 3 and d.get("write_n", 0) == 3
