"""Resume guard against stub checkpoints (``iter_0000500/mp_rank_00/model_optim_rng.pt``)
and the checkpoint writer's torch-Adam optimizer layout."""
import argparse
import os

import pytest
import torch

from sga_b200 import config as C
from sga_b200.runtime import checkpoint as ck
from sga_b200.runtime.trainer import Trainer, default_args


def _args(load, **kw):
    base = dict(sga_enabled=True, sga_score="abs_g", sga_selection_method="histogram",
                sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=10.0,
                sga_backend="torch_pipelined_index", sga_cycle_period=4)
    base.update(kw)
    ns = C.make_args(**base)
    ns.load = load
    ns.sga_allow_config_override = False
    ns.train_iters = 100
    return ns


def _stub(root, saved_args, iteration=500, tracker=True):
    d = os.path.join(root, f"iter_{iteration:07d}", "mp_rank_00")
    os.makedirs(d, exist_ok=True)
    torch.save({"args": saved_args, "iteration": iteration}, os.path.join(d, "model_optim_rng.pt"))
    if tracker:
        with open(os.path.join(root, ck.TRACKER), "w") as fh:
            fh.write(str(iteration))


def test_same_config_passes(tmp_path):
    _stub(str(tmp_path), _args(None))
    ck.sga_resume_guard(_args(str(tmp_path)))


def test_missing_tracker_is_a_cold_start(tmp_path):
    ck.sga_resume_guard(_args(str(tmp_path)))
    _stub(str(tmp_path), _args(None), tracker=False)
    ck.sga_resume_guard(_args(str(tmp_path), sga_cycle_period=8))


@pytest.mark.parametrize("change", [dict(sga_cycle_period=8), dict(sga_selection_ratio_percent=20.0),
                                    dict(sga_score="abs_m"), dict(sga_selection_locality="rank_local")])
def test_differing_config_refuses(tmp_path, change):
    _stub(str(tmp_path), _args(None))
    with pytest.raises(SystemExit):
        ck.sga_resume_guard(_args(str(tmp_path), **change), log=lambda m: None)


def test_comparison_is_spelling_faithful(tmp_path):
    _stub(str(tmp_path), _args(None, sga_selection_ratio_percent=10))     # int 10 vs float 10.0
    with pytest.raises(SystemExit):
        ck.sga_resume_guard(_args(str(tmp_path)), log=lambda m: None)
    saved = _args(None, sga_cycle_start_iter_percent=40.0)
    _stub(str(tmp_path), saved)
    cur = _args(str(tmp_path), sga_cycle_start_iter_percent=40.0)
    ck.sga_resume_guard(cur)
    cur.train_iters = 200                                                 # the percent's context changed
    with pytest.raises(SystemExit):
        ck.sga_resume_guard(cur, log=lambda m: None)


def test_override_and_non_sga_runs_skip_the_guard(tmp_path):
    _stub(str(tmp_path), _args(None))
    ns = _args(str(tmp_path), sga_cycle_period=8)
    ns.sga_allow_config_override = True
    ck.sga_resume_guard(ns)
    dense = _args(str(tmp_path), sga_cycle_period=8)
    dense.sga_enabled = False
    ck.sga_resume_guard(dense)
    timer = _args(str(tmp_path), sga_backend_timer="/tmp/timer")          # plumbing key: not identity
    ck.sga_resume_guard(timer)


def test_fail_closed_cases(tmp_path, monkeypatch):
    msgs = []
    _stub(str(tmp_path), argparse.Namespace(lr=1.0))                      # a dense checkpoint
    with pytest.raises(SystemExit):
        ck.sga_resume_guard(_args(str(tmp_path)), log=msgs.append)
    assert "no saved sga arguments" in msgs[-1]
    _stub(str(tmp_path), argparse.Namespace(sga_config='{"a": 1}'))       # the retired JSON era
    with pytest.raises(SystemExit):
        ck.sga_resume_guard(_args(str(tmp_path)), log=msgs.append)
    assert "predates the flat sga arguments" in msgs[-1]
    old = _args(None)
    old.sga_topk_ratio = 0.1                                              # a retired key
    _stub(str(tmp_path), old)
    with pytest.raises(SystemExit):
        ck.sga_resume_guard(_args(str(tmp_path)), log=msgs.append)
    assert "retired sga keys ['sga_topk_ratio']" in msgs[-1]
    with open(os.path.join(tmp_path, "iter_0000500", "mp_rank_00", "model_optim_rng.pt"), "wb") as fh:
        fh.write(b"garbage")
    with pytest.raises(SystemExit):
        ck.sga_resume_guard(_args(str(tmp_path)), log=msgs.append)
    assert "could not verify" in msgs[-1]
    import shutil

    shutil.rmtree(os.path.join(tmp_path, "iter_0000500", "mp_rank_00"))
    with pytest.raises(SystemExit):
        ck.sga_resume_guard(_args(str(tmp_path)), log=msgs.append)
    assert "no model_optim_rng.pt rank shard" in msgs[-1]
    monkeypatch.setenv("RANK", "3")                                       # only rank 0 pays the load
    ck.sga_resume_guard(_args(str(tmp_path)))


def test_checkpoint_layout_and_bit_continuous_dense_resume(tmp_path):
    kw = dict(model="test_tiny", micro_batch_size=2, global_batch_size=2, device="cpu", lr=1e-3, log_interval=0,
              sga_bucket_elems=30000)
    a = Trainer(default_args(train_iters=6, **kw), quiet=True)
    for s in range(3):
        a.train_step(a.host_batch(s))
    path = ck.save_checkpoint(str(tmp_path), 3, a.args, a.model, a.optimizer)
    assert path.endswith("iter_0000003/mp_rank_00/model_optim_rng.pt")
    assert open(tmp_path / ck.TRACKER).read() == "3"
    st = torch.load(path, weights_only=False)
    assert st["iteration"] == 3 and hasattr(st["args"], "sga_enabled")
    osd = st["optimizer"]["optimizer"]
    assert set(osd["state"][0]) == {"exp_avg", "exp_avg_sq"}
    assert [g["step"] for g in osd["param_groups"]] == [3, 3]
    assert osd["state"][0]["exp_avg"].dtype == torch.float32
    adam = torch.optim.Adam([torch.nn.Parameter(torch.zeros_like(osd["state"][i]["exp_avg"]))
                             for i in sorted(osd["state"])])
    assert set(adam.state_dict()) == {"state", "param_groups"}             # same top-level layout
    for s in range(3, 6):
        a.train_step(a.host_batch(s))
    b = Trainer(default_args(train_iters=6, **kw), quiet=True)
    assert ck.load_checkpoint(str(tmp_path), b.model, b.optimizer) == 3
    b.iteration = 3
    for s in range(3, 6):
        b.train_step(b.host_batch(s))
    assert torch.equal(a.model.arena.main_param, b.model.arena.main_param)
    assert torch.equal(a.model.arena.exp_avg_sq, b.model.arena.exp_avg_sq)
