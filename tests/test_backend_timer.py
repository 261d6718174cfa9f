"""Backend timer: off by default (no records, one None check), on it writes one
JSON line per bracketed region with the documented schema, refuses a second
configuration and overlapped gradient reduction, marks regions that raised,
and the trainer wires it end to end on CPU.
Reference behaviour: ``sga/backend_timer.py:1-200``."""
import json
import os

import pytest

from sga_b200.utils import backend_timer as BT


@pytest.fixture(autouse=True)
def _clean():
    BT.disable()
    yield
    BT.disable()


def _records(d, rank=0):
    with open(os.path.join(d, f"backend_timer_rank{rank}.jsonl")) as fh:
        return [json.loads(line) for line in fh if line.strip()]


def test_off_is_inert(tmp_path):
    assert not BT.enabled()
    with BT.region("sparse", backend="x"):  # no state, no file, no error
        pass
    BT.at_step(3)
    BT.time_full_syncs()
    assert not os.listdir(tmp_path)


def test_records_schema_and_sequence(tmp_path):
    d = str(tmp_path / "timer")
    BT.enable(d, 2)
    assert BT.enabled()
    BT.at_step(7)
    with BT.region("sparse", backend="torch_pipelined_index", bucket=4, nbytes=128):
        pass
    with BT.region("prescale", backend="torch_pipelined_index", bucket=4):
        pass
    recs = _records(d, rank=2)
    assert [r["phase"] for r in recs] == ["sparse", "prescale"]
    assert [r["seq"] for r in recs] == [0, 1]
    for r in recs:
        assert r["rank"] == 2 and r["iter"] == 7 and r["wall_ms"] >= 0 and "ts" in r and "error" not in r
    assert recs[0]["nbytes"] == 128 and recs[0]["bucket"] == 4


def test_enable_twice_and_bad_path_refused(tmp_path):
    with pytest.raises(ValueError):
        BT.enable("  ", 0)
    BT.enable(str(tmp_path), 0)
    with pytest.raises(RuntimeError, match="already configured"):
        BT.enable(str(tmp_path), 0)


def test_error_inside_region_is_marked_and_propagates(tmp_path):
    BT.enable(str(tmp_path), 0)
    with pytest.raises(OSError, match="link down"):
        with BT.region("sparse", backend="x"):
            raise OSError("link down")
    assert _records(str(tmp_path))[0]["error"] is True


def test_fullsync_wrap_refuses_overlap_and_is_idempotent(tmp_path):
    class Cfg:
        overlap_grad_reduce = True

    class Chunk:
        ddp_config = Cfg()
        calls = 0

        def finish_grad_sync(self, force_all_reduce=False):
            Chunk.calls += 1
            return "done"

    plain = Chunk.finish_grad_sync
    BT.time_full_syncs(Chunk)
    assert Chunk.finish_grad_sync is plain  # timer off: the class is left alone
    BT.enable(str(tmp_path), 0)
    BT.time_full_syncs(Chunk)
    first = Chunk.finish_grad_sync
    BT.time_full_syncs(Chunk)
    assert Chunk.finish_grad_sync is first and first is not plain  # wrapped once
    c = Chunk()
    with pytest.raises(RuntimeError, match="overlap_grad_reduce"):
        c.finish_grad_sync()
    Cfg.overlap_grad_reduce = False
    assert c.finish_grad_sync() == "done"
    recs = _records(str(tmp_path))
    assert len(recs) == 1 and recs[0]["phase"] == "fullsync" and recs[0]["backend"] == "ddp"
    BT.disable()
    assert c.finish_grad_sync() == "done"  # switched off again: straight through, nothing recorded
    assert len(_records(str(tmp_path))) == 1


def test_trainer_writes_sparse_and_fullsync_regions(tmp_path):
    from sga_b200.runtime.trainer import Trainer, default_args

    d = str(tmp_path / "t")
    tr = Trainer(default_args(model="test_tiny", micro_batch_size=2, global_batch_size=2, device="cpu", lr=1e-3,
                              sga_bucket_elems=30000, log_interval=0, sga_enabled=True, sga_score="abs_g",
                              sga_selection_method="histogram", sga_selection_histogram_mode="balanced",
                              sga_selection_ratio_percent=10.0, sga_backend="torch_pipelined_index",
                              sga_cycle_period=2, sga_backend_timer=d),
                 quiet=True)
    for s in range(4):
        tr.train_step(tr.host_batch(s))
    tr.close()
    phases = {r["phase"] for r in _records(d)}
    assert "fullsync" in phases and ("sparse" in phases or "prescale" in phases), phases
