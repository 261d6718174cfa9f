"""A dense run never touches the SGA machinery.

Without ``sga_enabled`` the trainer builds no engine and no plugin, reserves no staging memory for the sparse
exchange, and takes the dense step; the gate is ``sga_enabled`` alone, so a namespace that carries no ``sga_*``
attribute at all (a trainer driven by a foreign argument parser) trains densely too, and with equal
arithmetic. Counterpart of the reference's ``tests/test_waist_inert.py`` (the three call sites of the
external training stack are inert without the flag).
"""
import argparse

import torch

import sga_b200.runtime.trainer as T
from sga_b200.runtime.trainer import Trainer, default_args

KW = dict(model="test_tiny", micro_batch_size=2, global_batch_size=4, device="cpu", lr=1e-3, log_interval=0)


def _run(args, steps=3):
    tr = Trainer(args, quiet=True)
    losses = [float(tr.train_step(tr.host_batch(s))) for s in range(steps)]
    return tr, losses


def test_dense_run_builds_no_engine_and_no_plugins(monkeypatch, capsys):
    def boom(*a, **k):
        raise AssertionError("a dense run must not build the SGA engine")

    monkeypatch.setattr(T, "build_engine", boom)
    tr, losses = _run(default_args(**KW))
    assert tr.engine is None and tr.sga is False
    assert tr.model.arena.comm is None, "no staging buffer for the sparse exchange in a dense run"
    assert all(l == l for l in losses) and losses[-1] < losses[0] + 1.0
    assert "[SGA]" not in capsys.readouterr().out
    tr.close()


def test_namespace_without_any_sga_attribute_trains_densely(monkeypatch):
    monkeypatch.setattr(T, "build_engine", lambda *a, **k: (_ for _ in ()).throw(AssertionError("engine built")))
    full = default_args(**KW)
    bare = argparse.Namespace(**{k: v for k, v in vars(full).items() if not k.startswith("sga_")})
    assert not any(k.startswith("sga_") for k in vars(bare))
    tr_a, la = _run(full)
    tr_b, lb = _run(bare)
    assert tr_b.engine is None
    assert la == lb, "the same dense arithmetic with and without the sga_* attributes"
    assert torch.equal(tr_a.model.arena.main_param, tr_b.model.arena.main_param)
    tr_a.close()
    tr_b.close()


def test_the_gate_is_sga_enabled_alone():
    # every other sga_* attribute present and set, the switch off: still inert
    args = default_args(**KW, sga_score="abs_m", sga_selection_method="exact", sga_selection_ratio_percent=5.0,
                        sga_backend="torch_pipelined_index", sga_selection_locality="rank_local", sga_cycle_period=3)
    assert not args.sga_enabled
    tr, _ = _run(args, steps=1)
    assert tr.engine is None and tr.model.arena.comm is None
    tr.close()
    on = default_args(**KW, sga_enabled=True, sga_score="abs_g", sga_selection_method="exact",
                      sga_selection_ratio_percent=5.0, sga_backend="torch_pipelined_index",
                      sga_selection_locality="rank_local", sga_cycle_period=3)
    tr, _ = _run(on, steps=1)
    assert tr.engine is not None
    tr.close()
