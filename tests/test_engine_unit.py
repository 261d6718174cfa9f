"""Engine unit tests on CPU: calendar, frozen step order, full/sparse contract,
always-sync layers, dual lr, shadow invariants, consistency layers under a
mutating all-reduce, failed steps, logging."""
import json
import os

import pytest
import torch
import torch.distributed as dist

from sga_b200 import config as C
from sga_b200.runtime import engine as E
from sga_b200.runtime.arena import FlatArena, ParamSpec
from sga_b200.runtime.builder import build_engine
from sga_b200.runtime.ddp import DataParallel, DDPConfig
from sga_b200.runtime.optimizer import FlatOptimizer, OptimizerConfig


class _Model:
    def __init__(self, sizes=(3000, 64, 5000, 128), bucket=4000, groups=(0, 1, 0, 1)):
        names = ["layers.1.fc.weight", "layers.1.norm.weight", "layers.0.fc.weight", "layers.0.norm.weight"]
        specs = [ParamSpec(n, (s,), g, "normal", 0.02) for n, s, g in zip(names, sizes, groups)]
        self.arena = FlatArena(specs, bucket_elems=bucket, device="cpu")
        self.arena.init_parameters(0)

    def named_parameters(self):
        for s in self.arena.slots:
            yield s.name, s.model


def _build(monkeypatch=None, clip=1.0, **kw):
    os.environ["SGA_ALLOW_FROZEN_SELECTION"] = "1"
    base = dict(sga_enabled=True, sga_score="abs_g", sga_selection_method="histogram",
                sga_selection_histogram_mode="exact", sga_selection_ratio_percent=10.0,
                sga_backend="torch_pipelined_index", sga_cycle_period=4)
    base.update(kw)
    C.set_args(C.make_args(**base))
    model = _Model()
    ddp = DataParallel(model, transport="local", ddp_config=DDPConfig(overlap_grad_reduce=False))
    opt = FlatOptimizer(model.arena, OptimizerConfig(lr=1e-3, clip_grad=clip))
    eng = build_engine(quiet=True)
    eng.log_interval = 0
    eng.attach(ddp)
    return model, ddp, opt, eng


def _feed(model, step, scale=1e-2):
    g = torch.Generator().manual_seed(step)
    for s in model.arena.slots:
        s.grad += torch.randn(s.grad.shape, generator=g) * scale


def _step(model, ddp, opt, eng, step, force=False):
    _feed(model, step)
    eng.begin_step(ddp, step, force_all_reduce=force)
    assert eng.grad_sync(ddp, force)
    return eng.optimizer_step(opt, [ddp], step)


# ---------------------------------------------------------------- calendar
def test_cycle_manager_calendar():
    cm = E.CycleManager(20, 8, False, None)
    full = [s for s in range(1, 50) if cm.is_full(s)]
    assert full == list(range(1, 21)) + [28, 36, 44]
    assert [s for s in range(1, 50) if cm.reselect_boundary(s)] == [28, 36, 44]
    assert cm.fold_window == 8 and cm.is_full(30, force=True)
    dc = E.CycleManager(0, 8, True, 4)
    assert [s for s in range(1, 20) if dc.is_full(s)] == [4, 8, 12, 16]
    assert [s for s in range(1, 20) if dc.reselect_boundary(s)] == [8, 16] and dc.fold_window == 4
    with pytest.raises(AssertionError):
        E.CycleManager(0, 8, True, 3)
    with pytest.raises(AssertionError):
        E.CycleManager(0, 8, False, 4)
    never = E.CycleManager(2, 0, False, None, allow_zero=True)
    assert [s for s in range(1, 9) if never.is_full(s)] == [1, 2]


def test_phases_follow_calendar_and_support():
    model, ddp, opt, eng = _build(sga_cycle_start_iter=1)
    phases = []
    for step in range(1, 12):
        _feed(model, step)
        eng.begin_step(ddp, step)
        eng.grad_sync(ddp, False)
        phases.append("F" if eng._step_full else "S")
        eng.optimizer_step(opt, [ddp], step)
    # start 1, period 4: boundaries 5, 9; no support before the first reselection at 5
    assert "".join(phases) == "FFFFFSSSFSS"
    assert opt.step_count == 11


def test_forced_full_advances_cycle_but_never_reselects():
    model, ddp, opt, eng = _build()
    for step in range(1, 5):
        _step(model, ddp, opt, eng, step)
    sup = eng._active_support
    assert sup is not None
    for step in range(5, 8):
        _step(model, ddp, opt, eng, step)
    _step(model, ddp, opt, eng, 8, force=True)       # boundary, but forced
    assert eng._active_support is sup, "a forced full step must not reselect"


# ------------------------------------------------------------------- order
def test_frozen_step_order(monkeypatch):
    model, ddp, opt, eng = _build(sga_trace_dir=None)
    calls = []

    def spy(obj, name, label=None):
        orig = getattr(obj, name)

        def wrapped(*a, **k):
            calls.append(label or name)
            return orig(*a, **k)

        monkeypatch.setattr(obj, name, wrapped)

    class _Trace:
        def wants(self, step):
            return (False, False)

        def maybe_dump(self, *a):
            calls.append("trace_dump")

        def close(self):
            pass

    eng._trace = _Trace()
    opt.config.log_num_zeros_in_grad = True
    spy(opt, "prepare_grads")
    spy(eng, "_masked_clip_grad_norm", "clip")
    spy(eng, "_count_zeros", "count_zeros")
    spy(eng.opt, "full_step")
    spy(eng.opt, "sparse_step")
    spy(eng, "_check_norm_spread", "norm_spread")
    spy(eng, "_run_selection", "selection")
    spy(eng.opt, "reset")
    spy(eng, "_activate_support", "activate")
    spy(eng, "_check_counts", "count_guard")
    spy(eng, "_log_step", "log")
    for step in range(1, 4):
        _step(model, ddp, opt, eng, step)
    calls.clear()
    _step(model, ddp, opt, eng, 4)                    # boundary: full + reselection
    assert calls == ["prepare_grads", "clip", "count_zeros", "trace_dump", "full_step", "norm_spread", "selection",
                     "reset", "activate", "count_guard", "log"]
    calls.clear()
    _step(model, ddp, opt, eng, 5)                    # sparse
    assert calls == ["prepare_grads", "clip", "count_zeros", "trace_dump", "sparse_step", "reset", "log"]


# ------------------------------------------------------- full/sparse contract
def test_sparse_step_keeps_residual_and_clears_support():
    model, ddp, opt, eng = _build(clip=0.0)
    arena = model.arena
    for step in range(1, 5):
        _step(model, ddp, opt, eng, step)
    assert float(arena.main_grad.abs().sum()) == 0.0, "a full step ends with zeroed grad buffers"
    mask = eng._active_mask_arena().clone()
    sel = int(mask.sum())
    real = sum(s.end - s.start for s in arena.slots)
    assert abs(sel / real - 0.10) < 0.01
    _feed(model, 5)
    before = arena.main_grad.clone()
    w0, m0 = arena.main_param.clone(), arena.exp_avg.clone()
    eng.begin_step(ddp, 5)
    eng.grad_sync(ddp, False)
    assert not eng._step_full
    vals = list(eng._compact_values.values())
    assert vals and all(isinstance(v, torch.Tensor) for v in vals), "compact emission hands back the values"
    eng.optimizer_step(opt, [ddp], 5)
    on = mask > 0
    assert float(arena.main_grad[on].abs().sum()) == 0.0
    assert torch.equal(arena.main_grad[~on], before[~on])
    assert torch.equal(arena.exp_avg[~on], m0[~on] * 0.9 + torch.zeros(1) * (1.0 - 0.9)), "m decays where g = 0"
    assert not torch.equal(arena.main_param[on], w0[on])
    assert torch.equal(arena.model_param.float(), arena.main_param.to(torch.bfloat16).float())


def test_residual_mean_fold_on_pre_boundary_step():
    model, ddp, opt, eng = _build(clip=0.0, sga_optimizer_residual_mean=True)
    for step in range(1, 7):
        _step(model, ddp, opt, eng, step)
    mask = eng._active_mask_arena().clone()
    _feed(model, 7)
    before = model.arena.main_grad.clone()
    eng.begin_step(ddp, 7)
    eng.grad_sync(ddp, False)
    eng.optimizer_step(opt, [ddp], 7)                # step 8 is a boundary: fold by the window (4)
    off = mask == 0
    assert torch.equal(model.arena.main_grad[off], before[off] / torch.tensor(4.0))


def test_writeback_and_mask_backends_agree_with_index_backend():
    finals = []
    for kw in (dict(), dict(sga_backend_emission="writeback"), dict(sga_backend="torch_pipelined_mask"),
               dict(sga_backend="nccl_pipelined_index")):
        model, ddp, opt, eng = _build(**kw)
        for step in range(1, 9):
            _step(model, ddp, opt, eng, step)
        finals.append(model.arena.main_param.clone())
    assert all(torch.equal(finals[0], f) for f in finals[1:])


def test_block_layouts_run_and_select_whole_blocks():
    for kw in (dict(sga_backend_emission="writeback"), dict(sga_backend_layout="eb"),
               dict(sga_backend="torch_pipelined_mask"), dict(sga_backend="nccl_pipelined_index")):
        model, ddp, opt, eng = _build(sga_selection_block_size=8, sga_selection_histogram_mode="balanced", **kw)
        for step in range(1, 7):
            _step(model, ddp, opt, eng, step)
        sup = eng._active_support.buckets[0]
        assert sup.block_size == 8 and sup.block_idx.numel() > 0
        assert int(sup.mask_u8.sum()) >= sup.block_idx.numel()


def test_always_sync_layers_forced_and_out_of_the_pool():
    model, ddp, opt, eng = _build(sga_always_sync_layers="norm")
    for step in range(1, 5):
        _step(model, ddp, opt, eng, step)
    mask = eng._active_mask_arena()
    for s in model.arena.slots:
        m = mask[s.start:s.end]
        if "norm" in s.name:
            assert int(m.sum()) == m.numel()
    eligible = sum(s.end - s.start for s in model.arena.slots if "norm" not in s.name)
    picked = sum(int(mask[s.start:s.end].sum()) for s in model.arena.slots if "norm" not in s.name)
    assert abs(picked / eligible - 0.10) < 0.01
    with pytest.raises(E.SGAEngineError, match="matched no parameter"):
        _build(sga_always_sync_layers="does_not_exist")
    with pytest.raises(E.SGAEngineError, match="every parameter"):
        _build(sga_always_sync_layers="layers")


def test_dual_lr_applies_scaled_step_outside_outgoing_support():
    a = _build(clip=0.0)
    b = _build(clip=0.0, sga_optimizer_full_sync_inactive_lr_scale=0.0)
    for step in range(1, 8):
        _step(*a, step)
        _step(*b, step)
    assert torch.equal(a[0].arena.main_param, b[0].arena.main_param), "identical until the next boundary"
    mask = b[3]._active_mask_arena().clone()
    w_before = b[0].arena.main_param.clone()
    _step(*a, 8)
    _step(*b, 8)
    off = mask == 0
    assert torch.equal(b[0].arena.main_param[off], w_before[off]), "scale 0 freezes the never-communicated tail"
    assert torch.equal(b[0].arena.main_param[~off], a[0].arena.main_param[~off])
    assert torch.equal(a[0].arena.exp_avg, b[0].arena.exp_avg), "the commit is mask-blind"


# ------------------------------------------------------------------ shadow
def test_shadow_equals_dense_and_only_reads_state():
    shadow = _build(sga_shadow=True, sga_score="update", sga_cycle_period=2)
    C.set_args(C.make_args())
    dense_model = _Model()
    dense_opt = FlatOptimizer(dense_model.arena, OptimizerConfig(lr=1e-3, clip_grad=1.0))
    from sga_b200.plugins.optimizer.reference import grad_correct_torch

    for step in range(1, 6):
        _feed(shadow[0], step)
        _feed(dense_model, step)
        model, ddp, opt, eng = shadow
        eng.begin_step(ddp, step)
        assert eng.grad_sync(ddp, False) is False, "shadow leaves the dense sync to the caller"
        ddp.finish_grad_sync()
        eng.optimizer_step(opt, [ddp], step)
        ar = dense_model.arena
        norm = float((ar.main_grad.double() ** 2).sum().sqrt())
        c = 1.0 / (norm + 1e-6)
        coeff = float(torch.tensor(c, dtype=torch.float32)) if c < 1.0 else 1.0
        for s in ar.slots:
            sl = slice(s.start, s.end)
            grp = dense_opt.param_groups[s.spec.group]
            grad_correct_torch(ar.main_param[sl], ar.main_grad[sl], ar.exp_avg[sl], ar.exp_avg_sq[sl], grp["lr"], 0.9,
                               0.95, 1e-8, grp["weight_decay"], 1 - 0.9 ** step, 1 - 0.95 ** step, None, None,
                               coeff=coeff)
        ar.main_grad.zero_()
    assert torch.equal(shadow[0].arena.main_param, dense_model.arena.main_param)
    assert shadow[3]._active_support is not None and float(shadow[0].arena.main_grad.abs().sum()) == 0.0


def test_shadow_rng_bracket_detects_consumption(monkeypatch):
    model, ddp, opt, eng = _build(sga_shadow=True, sga_cycle_period=1)
    orig = eng._run_selection

    def noisy(views, meta):
        torch.rand(1)
        return orig(views, meta)

    monkeypatch.setattr(eng, "_run_selection", noisy)
    _feed(model, 1)
    ddp.finish_grad_sync()
    with pytest.raises(RuntimeError, match="consumed CPU RNG"):
        eng.optimizer_step(opt, [ddp], 1)


# ------------------------------------------------------ consistency layers
class _MutatingAllReduce:
    """Stands in for a two-rank world whose other rank holds different values:
    MIN and MAX see the local tensor shifted in opposite directions."""

    def __init__(self, monkeypatch, shift=True):
        self.shift = shift
        monkeypatch.setattr(dist, "is_initialized", lambda: True)
        monkeypatch.setattr(dist, "all_reduce", self)

    def __call__(self, t, op=None, group=None, async_op=False):
        if self.shift and t.numel() and op in (dist.ReduceOp.MIN, dist.ReduceOp.MAX):
            t += (-1 if op == dist.ReduceOp.MIN else 1) * (t.abs().max() * 1e-3 + 1).to(t.dtype)
        elif self.shift and op == dist.ReduceOp.MAX:
            pass
        return None


def test_support_checksum_and_norm_spread_abort_on_divergence(monkeypatch):
    model, ddp, opt, eng = _build()
    ddp.group = object()
    for bs in eng._bucket_states:
        bs.dp_group = ddp.group
    _MutatingAllReduce(monkeypatch)
    masks = [torch.ones(8, dtype=torch.uint8)]
    with pytest.raises(E.SGAEngineError, match="checksum mismatch"):
        eng._verify_support_consistency(masks)
    with pytest.raises(E.SGAEngineError, match="norm spread"):
        eng._check_norm_spread([torch.ones(8)])


def test_count_guard_refuses_mismatched_counts(monkeypatch):
    model, ddp, opt, eng = _build()
    for step in range(1, 5):
        _step(model, ddp, opt, eng, step)
    ddp.group = object()

    def fake(t, op=None, group=None, async_op=False):
        t[1] += 1       # the cluster minimum of bucket 0 differs from its maximum

    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "all_reduce", fake)
    with pytest.raises(E.SGAEngineError, match="count mismatch"):
        eng._check_counts()


def test_checks_master_switch_silences_layers(capsys):
    model, ddp, opt, eng = _build(sga_checks=False)
    assert not (eng._count_guard or eng._support_consistency or eng._norm_spread)
    assert "escape hatch active" in capsys.readouterr().out


# ----------------------------------------------------------- failed steps, log
def test_found_inf_clears_everything_and_consumes_the_step(monkeypatch):
    model, ddp, opt, eng = _build()
    _feed(model, 1)
    monkeypatch.setattr(opt, "prepare_grads", lambda: True)
    eng.begin_step(ddp, 1)
    eng.grad_sync(ddp, False)
    ok, gn, nz = eng.optimizer_step(opt, [ddp], 1)
    assert ok is False and gn is None
    assert float(model.arena.main_grad.abs().sum()) == 0.0 and opt.step_count == 0 and eng._iter == 1


def test_step_accounting_assert():
    model, ddp, opt, eng = _build()
    _step(model, ddp, opt, eng, 1)
    _feed(model, 3)
    eng.grad_sync(ddp, False)
    with pytest.raises(AssertionError, match="step accounting"):
        eng.optimizer_step(opt, [ddp], 3)


def test_resume_seeds_the_counter_and_cold_starts():
    model, ddp, opt, eng = _build()
    ok, _, _ = _step(model, ddp, opt, eng, 501)
    assert ok and eng._iter == 501 and eng._active_support is None


def test_log_line_and_metrics_file(tmp_path, capsys, monkeypatch):
    monkeypatch.setenv("SGA_METRICS_FILE", str(tmp_path / "m.jsonl"))
    model, ddp, opt, eng = _build()
    eng.log_interval = 1
    for step in range(1, 6):
        _step(model, ddp, opt, eng, step)
    out = capsys.readouterr().out
    import re

    assert "[SGA] step=1 phase=full ratio=-1.0000 grad_norm=" in out, "no support yet"
    m4 = re.search(r"\[SGA\] step=4 phase=full ratio=(0\.\d{4}) sel_thresh=\d\.\d{3}e[-+]\d+ grad_norm=\d+\.\d{3}\n", out)
    assert m4 and abs(float(m4.group(1)) - 0.10) < 0.01, "the boundary line already shows the new support"
    m = re.search(r"\[SGA\] step=5 phase=sparse ratio=(0\.\d+) sel_thresh=\S+ grad_norm=\d", out)
    assert m and abs(float(m.group(1)) - 0.10) < 0.01
    recs = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert [r["step"] for r in recs] == [1, 2, 3, 4, 5]
    assert set(recs[0]) == {"step", "phase", "ratio", "grad_norm", "reselected"}
    assert recs[3]["reselected"] is True and recs[4]["phase"] == "sparse"


def test_attach_contract():
    model, ddp, opt, eng = _build()
    with pytest.raises(TypeError, match="attaches to DataParallel"):
        eng.attach(object())
    eng.attach(ddp)  # idempotent
    other = DataParallel(_Model(), transport="local")
    with pytest.raises(E.SGAEngineError, match="one model chunk"):
        eng.attach(other)
    assert eng.grad_sync(other, False) is False
