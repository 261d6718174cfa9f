"""Bit-for-bit parity with the reference's own Python modules, where a plain
copy of the reference package is present under ``baseline/_ref`` (it is not
part of the repository; without it every test here is skipped).

Covered: the score registry, the torch optimizer references (AdamW and AdamS,
every fusion knob), mask compaction and the block forms, the cycle calendar,
the flag surface and its validation, the three histogram selection modes, the
exact selection, the adaptive threshold controller over a sequence of steps,
and the replay CLI on a trace written by this framework's own trace collector.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "sga")),
                                reason="no copy of the reference package under baseline/_ref")


@pytest.fixture(scope="module")
def ref():
    """Imports reference modules by name with Triton hidden from them (their replay kernels refuse
    every Triton release but one; without Triton the reference takes its torch paths)."""
    saved = sys.modules.get("triton", "absent")
    sys.modules["triton"] = None
    sys.path.insert(0, REF)
    try:
        yield lambda name: importlib.import_module(name)
    finally:
        sys.path.remove(REF)
        if saved == "absent":
            sys.modules.pop("triton", None)
        else:
            sys.modules["triton"] = saved


def _same_masks(a, b):
    return all(torch.equal(x.view(-1).to(torch.uint8), y.view(-1).to(torch.uint8)) for x, y in zip(a, b))


def test_scores_bitwise(ref):
    RS = ref("sga.plugins.scores")
    from sga_b200.plugins import scores as MS

    RS.register_default_scores()
    MS.register_default_scores()
    assert sorted(RS.score_names()) == sorted(MS.score_names())
    torch.manual_seed(0)
    n = 4000
    w, m, g = torch.randn(n) * 0.02, torch.randn(n) * 1e-3, torch.randn(n) * 1e-2
    v = (torch.randn(n) * 1e-3) ** 2
    for step in (1, 7, 300):
        bc1, bc2 = 1 - 0.9 ** step, 1 - 0.95 ** step
        for name in RS.score_names():
            for inc in (True, False):
                want = RS.get_score_spec(name).formula(w, m, v, g, 0.9, 0.95, 1e-8, 0.1, bc1, bc2, update_includes_wd=inc)
                got = MS.compute_score(name, w, m, v, g, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, bc1=bc1,
                                       bc2=bc2, update_includes_wd=inc)
                assert torch.equal(want, got), (name, step, inc)


def test_optimizer_references_bitwise(ref):
    R_w = ref("sga.plugins.optimizer.adamw_torch").grad_correct_torch
    R_s = ref("sga.plugins.optimizer.adams_torch").adams_grad_correct_torch
    from sga_b200.plugins.optimizer.reference import grad_correct_torch as M

    torch.manual_seed(1)
    n = 3000
    w, m, g = torch.randn(n) * 0.02, torch.randn(n) * 1e-3, torch.randn(n) * 1e-2
    v = (torch.randn(n) * 1e-3) ** 2
    mask = (torch.rand(n) < 0.1).to(torch.uint8)
    cases = [dict(mask=None, emit_score=s) for s in ("abs_g", "update", "coi", "abs_m")] + [
        dict(mask=mask, emit_score=None), dict(mask=mask, emit_score=None, coeff=0.37, clear=True),
        dict(mask=mask, emit_score=None, clear=True, fold=True, interval=4.0),
        dict(mask=mask, emit_score="update", inactive_lr_scale=0.25)]
    bc1, bc2 = 1 - 0.9 ** 7, 1 - 0.95 ** 7
    for opt in ("adamw", "adams"):
        for kw in cases:
            a = [t.clone() for t in (w, g, m, v)]
            b = [t.clone() for t in (w, g, m, v)]
            if opt == "adamw":
                R_w(*a, 3e-4, 0.9, 0.95, 1e-8, 0.1, bc1, bc2, **kw)
            else:
                R_s(*a, 3e-4, 0.9, 0.95, 1e-8, 0.1, **kw)
            M(*b, 3e-4, 0.9, 0.95, 1e-8, 0.1, bc1, bc2, optimizer=opt, **kw)
            assert all(torch.equal(x, y) for x, y in zip(a, b)), (opt, {k: v for k, v in kw.items() if k != "mask"})


def test_support_forms_bitwise(ref):
    R = ref("sga.support")
    from sga_b200 import support as M

    torch.manual_seed(2)
    n = 16384
    mk = (torch.rand(n) < 0.13).to(torch.uint8)
    assert torch.equal(R.compact_mask_u8(mk), M.compact_mask_u8(mk))
    spans = [(0, 4096), (4096, 4160), (4160, 12288), (12288, 16384)]
    for x in (4, 8, 64):
        heads = R.block_idx_from_mask(mk, spans, x)
        assert torch.equal(heads, M.block_idx_from_mask(mk, spans, x))
        full = torch.zeros(n, dtype=torch.uint8)
        for h in heads.tolist():
            end = next(e for s, e in spans if s <= h < e)
            full[h:min(h + x, end)] = 1
        assert torch.equal(R.block_desc_from_mask(full, spans, x), M.block_desc_from_mask(full, spans, x))


def test_cycle_calendar(ref):
    R = ref("sga.engine").CycleManager
    from sga_b200.runtime.engine import CycleManager as M

    for cfg in [(0, 4, False, None), (20, 8, False, None), (5, 8, True, 4), (1, 1, False, None), (3, 6, True, 2)]:
        a, b = R(*cfg), M(*cfg)
        assert a.fold_window == b.fold_window
        for step in range(1, 90):
            for force in (False, True):
                assert (a.is_full(step, force), a.reselect_boundary(step), a.extra_full(step)) == \
                       (b.is_full(step, force), b.reselect_boundary(step), b.extra_full(step)), (cfg, step, force)


def test_flag_surface_and_validation(ref):
    R_add = ref("sga.config.arguments").add_sga_args
    R_val = ref("sga.config.validation").validate_sga_args
    from sga_b200.config.arguments import add_sga_args as M_add
    from sga_b200.config.validation import validate_sga_args as M_val

    pr, pm = argparse.ArgumentParser(), argparse.ArgumentParser()
    R_add(pr)
    M_add(pm)
    ra = {a.dest: a for a in pr._actions if a.dest.startswith("sga_")}
    ma = {a.dest: a for a in pm._actions if a.dest.startswith("sga_")}
    assert not set(ra) - set(ma)
    assert set(ma) - set(ra) == {"sga_backend_transport", "sga_bucket_elems", "sga_selection_locality"}
    for d, x in ra.items():
        y = ma[d]
        assert x.default == y.default and x.option_strings == y.option_strings, d
        assert (x.choices is None) == (y.choices is None) and (x.choices is None or list(x.choices) == list(y.choices)), d

    base = ["--sga-enabled", "true", "--sga-score", "abs_g", "--sga-backend", "torch_pipelined_index",
            "--sga-selection-ratio-percent", "10", "--sga-cycle-period", "8", "--sga-selection-method", "histogram",
            "--sga-selection-histogram-mode", "balanced"]
    trials = [[], ["--sga-cycle-start-iter", "20"], ["--sga-cycle-start-iter-percent", "10"],
              ["--sga-selection-method", "exact"], ["--sga-selection-histogram-mode", "fast"],
              ["--sga-selection-block-size", "8"], ["--sga-selection-block-size", "3"],
              ["--sga-backend", "torch_pipelined_mask"], ["--sga-optimizer", "adams"], ["--sga-score", "coi"],
              ["--sga-selection-ratio-percent", "0"], ["--sga-selection-ratio-percent", "100"],
              ["--sga-trace-dir", "/tmp/x", "--sga-trace-branch-points", "3,1,2"], ["--sga-shadow", "true"],
              ["--sga-always-sync-layers", "embedding,final"], ["--sga-backend-index-slices", "3"],
              ["--sga-cycle-decouple-full-sync-interval-and-period", "true", "--sga-cycle-full-sync-interval", "4"],
              ["--sga-cycle-full-sync-interval", "4"], ["--sga-optimizer-full-sync-inactive-lr-scale", "0.5"],
              ["--sga-optimizer-residual-mean", "true"], ["--sga-checks", "false"],
              ["--sga-backend-layout", "bb", "--sga-selection-block-size", "8"], ["--sga-backend-emission", "writeback"],
              ["--sga-selection-method", "adaptive"]]

    def run(add, val, argv):
        p = argparse.ArgumentParser()
        add(p)
        ns = p.parse_args(argv)
        ns.train_iters, ns.pipeline_model_parallel_size, ns.tensor_model_parallel_size = 100, 1, 1
        try:
            val(ns)
        except ValueError:
            return "refused", None
        return "ok", {k: v for k, v in vars(ns).items() if k.startswith("sga_")}

    for t in trials:
        a, b = run(R_add, R_val, base + t), run(M_add, M_val, base + t)
        assert a[0] == b[0], (t, a[0], b[0])
        if a[0] == "ok":
            assert not {k for k in a[1] if a[1][k] != b[1].get(k)}, t


def test_validation_differential_fuzz(ref, monkeypatch):
    """Seeded random configurations (one to six keys drawn from legal, boundary and illegal values on
    top of a valid base) through both validators: the same accept / refuse decision every time, and
    the same namespace after the write-backs of an accepted configuration."""
    import random

    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")
    RV = ref("sga.config.validation")
    import sga_b200.config.validation as OV

    dom = {
        "sga_score": [None, "update", "abs_g", "abs_m", "coi"],
        "sga_backend": ["dense", "torch_pipelined_index", "torch_pipelined_mask", "nccl_pipelined_index", "bogus"],
        "sga_selection": ["topk", "bogus"], "sga_optimizer": ["adamw", "adams"], "sga_checks": [True, False],
        "sga_cycle_start_iter": [0, 5], "sga_cycle_start_iter_percent": [None, 10.0, 150.0],
        "sga_cycle_period": [1, 4, 6, 0], "sga_cycle_decouple_full_sync_interval_and_period": [False, True],
        "sga_cycle_full_sync_interval": [None, 2, 3, 4, 6], "sga_trace_dir": [None, "/tmp/x", ""],
        "sga_trace_branch_points": [None, "2,4", "a", "-1"], "sga_trace_window": [100, 0, 5],
        "sga_trace_dump_dtype": ["fp32", "bf16"], "sga_trace_async": [False, True],
        "sga_trace_async_backend": ["cpu_snapshot", "pinned_cuda"], "sga_trace_async_queue_depth": [1, 4],
        "sga_trace_async_worker_count": [2, 8], "sga_shadow": [False, True], "sga_shadow_score": [True, False],
        "sga_always_sync_layers": [None, "embedding", "a,,b", "null"],
        "sga_optimizer_full_sync_inactive_lr_scale": [1.0, 0.5, 0.0, -1.0],
        "sga_optimizer_residual_mean": [False, True], "sga_backend_emission": ["compact", "writeback"],
        "sga_selection_method": [None, "histogram", "exact", "adaptive", "bogus"],
        "sga_selection_histogram_mode": ["fast", "balanced", "exact"], "sga_selection_block_size": [1, 8, 3],
        "sga_selection_ratio_percent": [None, 1.0, 0.0, 100.0, 101.0], "sga_backend_index_slices": [1, 3, 0],
        "sga_backend_mask_slices": [2, 0], "sga_optimizer_compact_search": ["table", "bisect", "bogus"],
        "train_iters": [None, 100], "pipeline_model_parallel_size": [1, 2],
    }
    rd, od = RV.sga_defaults(), OV.sga_defaults()
    assert all(k in rd for k in dom if k.startswith("sga_"))
    rng = random.Random(0)
    accepted = refused = 0
    for _ in range(2500):
        over = {"sga_enabled": True, "sga_score": "update", "sga_backend": "torch_pipelined_index",
                "sga_selection_method": "histogram", "sga_selection_ratio_percent": 1.0}
        for k in rng.sample(sorted(dom), rng.choice([1, 2, 3, 4, 6])):
            over[k] = rng.choice(dom[k])
        sides = []
        for defaults, V in ((rd, RV), (od, OV)):
            ns = argparse.Namespace(**{"train_iters": None, "pipeline_model_parallel_size": 1, **defaults, **over})
            try:
                V.validate_sga_args(ns)
                sides.append(ns)
            except (ValueError, TypeError):
                sides.append(None)
        assert (sides[0] is None) == (sides[1] is None), over
        if sides[0] is None:
            refused += 1
        else:
            accepted += 1
            assert not {k for k in rd if getattr(sides[0], k) != getattr(sides[1], k)}, over
    assert accepted > 300 and refused > 300


def test_selection_plugins_bitwise(ref):
    R_hist = ref("sga.plugins.selection._histogram").select_masks_histogram
    R_ex = ref("sga.plugins.selection._exact").select_masks_exact_kthvalue
    RA = ref("sga.plugins.selection._adaptive").AdaptiveTau
    from sga_b200.plugins.selection.threshold import AdaptiveThresholdSelect as MA
    from sga_b200.plugins.selection._exact import select_masks_exact_kthvalue as M_ex
    from sga_b200.plugins.selection._histogram import select_masks_histogram as M_hist

    torch.manual_seed(3)
    views = [torch.randn(40000) * 1e-3, torch.randn(7), torch.randn(123457) * 3e-2, torch.zeros(1000),
             (torch.randn(5000) * 1e-3).abs()]
    views[2][::13] = 0.05  # a tie layer
    total = sum(v.numel() for v in views)
    for mode in ("exact", "balanced", "fast"):
        for k in (1, 17, 1000, 50000, total - 5):
            tr, mr = R_hist([v.clone() for v in views], k, None, mode=mode, global_allreduce=False)
            tm, mm = M_hist([v.clone() for v in views], k, None, mode=mode, global_allreduce=False)
            assert float(tr) == float(tm) and _same_masks(mr, mm), (mode, k)
    small = [views[0][:4000], views[1], views[2][:12345]]
    for k in (1, 17, 900, 8000):
        tr, mr = R_ex([v.clone() for v in small], k, None)
        tm, mm = M_ex([v.clone() for v in small], k, None)
        assert float(tr) == float(tm) and _same_masks(mr, mm), k
    for wm in ("balanced", "fast", "exact"):
        for ws in (1, 3):
            a, b = RA(5.0, ws, wm, False), MA(5.0, ws, wm, False)
            gen = torch.Generator().manual_seed(5)
            for it in range(14):
                scale = 1e-3 * (1 + 0.3 * ((it * 7) % 5))
                gs = [torch.randn(20000, generator=gen) * scale, torch.randn(10000, generator=gen) * scale * 2]
                wa, wb = a.warmup_sync_target(0, 4), b.warmup_sync_target(0, 4)
                ra = a.select([x.clone() for x in gs], 1500, None, wa)
                rb = b.select([x.clone() for x in gs], 1500, None, wb)
                assert wa == wb and float(ra[0]) == float(rb[0]) and _same_masks(ra[1], rb[1]), (wm, ws, it)


@pytest.mark.timeout(600)
def test_reference_replay_reads_our_trace_and_agrees(tmp_path):
    """A trace written by this framework's collector during a real (CPU) training run is consumed by
    the reference's replay CLI, and both replays report the same distortions and ranking metrics."""
    from sga_b200.replay import cli
    from sga_b200.runtime.trainer import Trainer, default_args

    tdir = str(tmp_path / "trace")
    tr = Trainer(default_args(model="test_tiny", micro_batch_size=2, global_batch_size=2, train_iters=12, device="cpu",
                              lr=1e-3, sga_bucket_elems=30000, log_interval=0, sga_enabled=True, sga_shadow=True,
                              sga_score="abs_g", sga_selection_method="histogram",
                              sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=10.0,
                              sga_backend="torch_pipelined_index", sga_cycle_period=2, sga_trace_dir=tdir,
                              sga_trace_branch_points="2", sga_trace_window=6), quiet=True)
    for s in range(10):
        tr.train_step(tr.host_batch(s))
    tr.close()
    hide = tmp_path / "hide" / "triton"
    hide.mkdir(parents=True)
    (hide / "__init__.py").write_text('raise ImportError("hidden")\n')
    common = ["--trace-dir", tdir, "--branch-point", "2", "--ratios", "5,10", "--replay-mode", "cycle", "--cycle-lens",
              "1,2", "--score-names", "abs_g,update", "--window", "6", "--device", "cpu"]
    ref_out, our_out = str(tmp_path / "ref.json"), str(tmp_path / "our.json")
    env = dict(os.environ, PYTHONPATH=str(tmp_path / "hide") + os.pathsep + REF)
    res = subprocess.run([sys.executable, "-m", "sga.replay"] + common + ["--dense-cache", str(tmp_path / "cache"), "--out",
                         ref_out], env=env, capture_output=True, text=True, cwd=str(tmp_path))
    assert res.returncode == 0, res.stderr[-2000:]
    assert cli.main(common + ["--out", our_out]) == 0
    a = json.load(open(ref_out))["branch_results"]["2"]["per_ratio"]
    b = json.load(open(our_out))["branch_results"]["2"]["per_ratio"]
    for r in a:
        for key, want in a[r]["scores"].items():
            got = b[r]["scores"][key]
            if not key.endswith("T1"):
                assert abs(got["distortion"]["6"] - want["distortion"]["6"]) < 5e-8, (r, key)
            for mname in ("ndcg_at_k", "recall_at_k", "missed_label_mass", "missed_score_mass"):
                assert abs(got[mname] - want[mname]) < 5e-8, (r, key, mname, got[mname], want[mname])


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "tests", "ref_engine_harness.py")),
                    reason="no copy of the reference's engine test harness under baseline/_ref/tests")
def test_engine_flow_matches_reference_engine(ref, monkeypatch):
    """The reference engine, driven by its own fake data-parallel chunk and optimizer wrapper
    (``tests/test_engine_unit.py:647-730`` there), against this framework's engine on the same
    parameters and the same per-step gradients, for mask- and index-consuming backends across scores,
    both optimizers, the residual fold, the boundary dual lr, every selection method and histogram
    mode, sliced and block transports, always-synchronised parameters, the decoupled calendar and failed (non-finite) steps: same full / sparse calendar, bit-identical
    residual buffer, weights and gradient norms equal to fp32 rounding (the reference's dense steps
    run ``torch.optim.Adam``, whose operation order differs from the fused form by an ulp)."""
    import copy
    import types

    from sga_b200 import config as C
    from sga_b200.runtime.arena import FlatArena, ParamSpec
    from sga_b200.runtime.builder import build_engine
    from sga_b200.runtime.ddp import DataParallel, DDPConfig
    from sga_b200.runtime.optimizer import FlatOptimizer, OptimizerConfig

    # the two helper predicates the reference engine imports from its external training stack
    mods = {n: types.ModuleType(n) for n in ("megatron", "megatron.core", "megatron.core.tensor_parallel",
                                             "megatron.core.transformer", "megatron.core.transformer.module")}
    mods["megatron.core.tensor_parallel"].param_is_not_tensor_parallel_duplicate = lambda p, g=None: True
    mods["megatron.core.transformer.module"].param_is_not_shared = lambda p: True
    for n, m in mods.items():
        monkeypatch.setitem(sys.modules, n, m)
    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")  # the harness builds without the validation gate
    monkeypatch.syspath_prepend(os.path.join(REF, "tests"))
    ref("sga.engine")
    H = importlib.import_module("ref_engine_harness")

    def run_reference(combo, steps, seed, extra, bad_steps=()):
        torch.manual_seed(seed)
        chunk = H._FakeChunk(n_params=3, numel_per=64)
        mp = H._FakeMPOpt(chunk)
        now = {"step": 0}
        stock_prepare = mp.prepare_grads
        mp.prepare_grads = lambda: (stock_prepare() or True) if now["step"] in bad_steps else stock_prepare()
        p0 = [p.detach().clone() for p in chunk.params]
        eng = H._build_engine(combo, extra)
        eng.attach(chunk)
        grads, log = [], []
        gen = torch.Generator().manual_seed(seed + 1)
        with H._ReplicaWorld(world=1):
            for step in range(1, steps + 1):
                now["step"] = step
                g = torch.randn(chunk.bucket.grad_data.numel(), generator=gen)
                grads.append(g.clone())
                chunk.bucket.grad_data += g
                assert eng.grad_sync(chunk, force_all_reduce=False) is True
                full = bool(eng._step_full)
                ok, gn, _nz = eng.optimizer_step(mp, [chunk], step)
                log.append((step, (full, bool(ok)), float(gn) if gn is not None else float("nan")))
        return p0, grads, log, [m.detach().clone() for m in mp.main_params], chunk.bucket.grad_data.clone()

    def run_ours(combo, p0, grads, extra, bad_steps=()):
        kw = {**combo["config"], **combo["selection_params"], **combo["opt_params"], **combo.get("backend_params", {}),
              "sga_score": combo["score"], "sga_selection": combo["selection"], "sga_optimizer": combo["opt"],
              "sga_backend": combo["backend"], "sga_enabled": True, **(extra or {})}
        C.set_args(C.make_args(**kw))
        model = types.SimpleNamespace()
        model.arena = FlatArena([ParamSpec(f"p{i}", tuple(p.shape), 0, "zeros") for i, p in enumerate(p0)],
                                bucket_elems=10 ** 9, device="cpu")
        model.named_parameters = lambda: [(s.name, s.model) for s in model.arena.slots]
        for s, p in zip(model.arena.slots, p0):
            s.main.copy_(p)
        model.arena.sync_model_from_main()
        ddp = DataParallel(model, transport="local",
                           ddp_config=DDPConfig(average_in_collective=False, overlap_grad_reduce=False))
        opt = FlatOptimizer(model.arena, OptimizerConfig(lr=1e-3, weight_decay=1e-2, adam_beta1=0.9, adam_beta2=0.95,
                                                         adam_eps=1e-8, clip_grad=1.0))
        now = {"step": 0}
        own_prepare = opt.prepare_grads
        opt.prepare_grads = lambda: True if now["step"] in bad_steps else own_prepare()
        eng = build_engine(quiet=True)
        eng.log_interval = 0
        eng.attach(ddp)
        log = []
        for step, g in enumerate(grads, 1):
            now["step"] = step
            off = 0
            for s in model.arena.slots:
                n = s.end - s.start
                model.arena.main_grad[s.start:s.end] += g[off:off + n]
                off += n
            ddp.begin_step()
            eng.begin_step(ddp, step)
            if not eng.grad_sync(ddp, False):
                ddp.finish_grad_sync()
            full = bool(eng._step_full)
            ok, gn, _nz = eng.optimizer_step(opt, [ddp], step)
            log.append((step, (full, bool(ok)), float(gn) if gn is not None else float("nan")))
        return (log, [s.main.clone() for s in model.arena.slots],
                torch.cat([model.arena.main_grad[s.start:s.end] for s in model.arena.slots]))

    U, M = H._UPDATE, H._ABS_M
    ratio = {"sga_selection_ratio_percent": 30.0}
    cases = [(c, e) for c in (U, M) for e in (None, {"sga_optimizer_residual_mean": True})] + [
        ({**M, "score": "abs_g"}, {"sga_backend_emission": "writeback"}),
        ({**M, "score": "abs_g"}, {"sga_backend_index_slices": 3}),
        ({**U, "score": "coi"}, None),
        ({**M, "score": "update"}, None),
        ({**U, "score": "abs_m", "opt": "adams"}, None),
        ({**M, "score": "abs_g", "opt": "adams"}, None),
        (U, {"sga_optimizer_full_sync_inactive_lr_scale": 0.5}),
        (U, {"sga_optimizer_full_sync_inactive_lr_scale": 0.25, "sga_optimizer_residual_mean": True}),
        ({**M, "opt": "adams"}, {"sga_optimizer_full_sync_inactive_lr_scale": 0.0}),
        (M, {"sga_selection_histogram_mode": "balanced"}),
        (M, {"sga_selection_histogram_mode": "fast"}),
        ({**M, "selection_params": {"sga_selection_method": "exact", **ratio}}, None),
        ({**M, "selection_params": {"sga_selection_method": "adaptive", **ratio}}, None),
        ({**U, "config": {"sga_cycle_start_iter": 0, "sga_cycle_period": 6, "sga_cycle_full_sync_interval": 3,
                          "sga_cycle_decouple_full_sync_interval_and_period": True}}, None),
        (U, {"sga_always_sync_layers": ["p1"]}),
        (M, {"sga_always_sync_layers": ["p0", "p2"], "sga_optimizer_residual_mean": True}),
        (U, {"sga_checks": False}),
        ({**M, "score": "abs_g"}, {"sga_selection_block_size": 8, "sga_selection_histogram_mode": "exact",
                                   "sga_backend_emission": "writeback"}),
    ]
    # a failed step (the optimizer wrapper reports non-finite gradients) on a sparse step and on a boundary:
    # full clear, the cycle position is consumed, nothing is committed (sga/engine.py:512-521)
    cases = [(c, e, ()) for c, e in cases] + [(U, None, (5, 9)), (M, None, (5, 9)),
                                              (M, {"sga_optimizer_residual_mean": True}, (4, 8))]
    for combo, extra, bad_steps in cases:
        c = copy.deepcopy(combo)
        tag = (combo["score"], combo["backend"], combo["opt"], extra, bad_steps)
        p0, grads, rlog, rfinal, rres = run_reference(c, 14, 7, extra, bad_steps)
        olog, ofinal, ores = run_ours(c, p0, grads, extra, bad_steps)
        assert [(s, f) for s, f, _ in rlog] == [(s, f) for s, f, _ in olog], tag
        assert [ok for _, (_, ok), _ in rlog].count(False) == len(bad_steps), tag
        assert torch.equal(rres, ores), ("residual buffer differs", tag)
        for (_, _, a), (_, _, b) in zip(rlog, olog):
            assert (a != a and b != b) or abs(a - b) <= 5e-7 * max(a, 1e-9), tag
        for a, b in zip(rfinal, ofinal):
            assert float((a - b).abs().max()) <= 3e-7, tag


@pytest.mark.parametrize("world", [2, 3])
def test_engine_flow_matches_reference_engine_multirank(world):
    """``world`` gloo ranks with different gradients per rank: see ``tests/ref_parity_worker.py``."""
    import socket

    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", str(port),
                          os.path.join(ROOT, "tests", "ref_parity_worker.py")], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert res.returncode == 0 and "PARITY OK" in res.stdout, (res.stdout[-1500:], res.stderr[-1500:])


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "tests", "ref_engine_harness.py")),
                    reason="no copy of the reference's engine test harness under baseline/_ref/tests")
def test_replay_reports_equal_on_a_trace_written_by_the_reference(ref, monkeypatch, tmp_path):
    """The other direction of the trace format: the reference engine and its trace collector write a
    trace (CPU, the reference's own fakes), then both replay CLIs run every per-configuration axis on it
    (two optimizers, fold off / on, plain and T-relative dual lr, two cycle lengths, default
    balanced-histogram semantics) and the zerofill mode (frozen exact top-k support) on it. The whole report must agree: same keys and nesting, every number
    (distortions, thresholds, ranking metrics, score and label statistics, the per-step reconstruction
    check) to 5e-8; this framework adds ``step`` / ``phase`` to ``meta`` and a ``profile`` block."""
    import copy
    import types

    from sga_b200.replay import cli

    mods = {n: types.ModuleType(n) for n in ("megatron", "megatron.core", "megatron.core.tensor_parallel",
                                             "megatron.core.transformer", "megatron.core.transformer.module")}
    mods["megatron.core.tensor_parallel"].param_is_not_tensor_parallel_duplicate = lambda p, g=None: True
    mods["megatron.core.transformer.module"].param_is_not_shared = lambda p: True
    for n, m in mods.items():
        monkeypatch.setitem(sys.modules, n, m)
    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")
    monkeypatch.syspath_prepend(os.path.join(REF, "tests"))
    ref("sga.engine")
    H = importlib.import_module("ref_engine_harness")
    tdir = str(tmp_path / "trace")
    torch.manual_seed(3)
    chunk = H._FakeChunk(n_params=3, numel_per=4096)
    mp = H._FakeMPOpt(chunk)
    eng = H._build_engine(copy.deepcopy(H._ABS_M), {"sga_trace_dir": tdir, "sga_trace_branch_points": [3],
                                                    "sga_trace_window": 6})
    eng.attach(chunk)
    gen = torch.Generator().manual_seed(4)
    with H._ReplicaWorld(world=1):
        for step in range(1, 12):
            chunk.bucket.grad_data += torch.randn(chunk.bucket.grad_data.numel(), generator=gen)
            eng.grad_sync(chunk, force_all_reduce=False)
            eng.optimizer_step(mp, [chunk], step)
    assert os.path.exists(os.path.join(tdir, "step_000003_state.pt"))
    hide = tmp_path / "hide" / "triton"
    hide.mkdir(parents=True)
    (hide / "__init__.py").write_text('raise ImportError("hidden")\n')
    env = dict(os.environ, PYTHONPATH=str(tmp_path / "hide") + os.pathsep + REF)
    allowed = {"/config/dense_cache", "/branch_results/3/meta/step", "/branch_results/3/meta/phase",
               "/branch_results/3/replay/profile"}

    def walk(x, y, path, diffs):
        if isinstance(x, dict):
            if not isinstance(y, dict):
                return diffs.append((path, "type"))
            for k in x:
                if k not in y:
                    diffs.append((path + "/" + k, "missing"))
                else:
                    walk(x[k], y[k], path + "/" + k, diffs)
            diffs.extend((path + "/" + k, "extra") for k in y if k not in x)
        elif isinstance(x, list):
            if not isinstance(y, list) or len(x) != len(y):
                return diffs.append((path, "list"))
            for i, (p, q) in enumerate(zip(x, y)):
                walk(p, q, f"{path}[{i}]", diffs)
        elif isinstance(x, float) or isinstance(y, float):
            if x is None or y is None or abs(x - y) > 6e-8 * max(1.0, abs(x)):
                diffs.append((path, x, y))
        elif x != y:
            diffs.append((path, x, y))

    # the bf16 screening copy: both converters on that trace, same file set, same contents
    from sga_b200 import trace_convert as TC

    ca, cb = str(tmp_path / "conv_ref"), str(tmp_path / "conv_ours")
    res = subprocess.run([sys.executable, "-m", "sga.trace_convert", "--src", tdir, "--dst", ca, "--from-step", "4"], env=env,
                         capture_output=True, text=True, cwd=str(tmp_path))
    assert res.returncode == 0, res.stderr[-2000:]
    assert TC.main(["--src", tdir, "--dst", cb, "--from-step", "4"]) == 0
    assert sorted(os.listdir(ca)) == sorted(os.listdir(cb)) and len(os.listdir(ca)) == 6

    def same(x, y):
        if isinstance(x, dict):
            return isinstance(y, dict) and x.keys() == y.keys() and all(same(x[k], y[k]) for k in x)
        if torch.is_tensor(x):
            return torch.is_tensor(y) and x.dtype == y.dtype and torch.equal(x, y)
        if isinstance(x, (list, tuple)):
            return len(x) == len(y) and all(same(p, q) for p, q in zip(x, y))
        return x == y

    for f in os.listdir(ca):
        assert same(torch.load(os.path.join(ca, f), weights_only=False), torch.load(os.path.join(cb, f), weights_only=False)), f

    base = ["--trace-dir", tdir, "--branch-point", "3", "--window", "6", "--device", "cpu", "--fused-shards", "1"]
    runs = {"cycle": (["--ratios", "5", "--replay-mode", "cycle", "--cycle-lens", "2,3", "--score-names", "abs_g,update",
                       "--optimizer", "adamw,adams", "--fold", "off,on", "--dual-lr", "1,T/4"], 32),
            "zerofill": (["--ratios", "5,20", "--replay-mode", "zerofill", "--score-names", "abs_g,abs_m,coi",
                          "--selection-semantics", "topk"], 3)}
    for tag, (extra, arms) in runs.items():
        ref_out, our_out = str(tmp_path / f"ref_{tag}.json"), str(tmp_path / f"our_{tag}.json")
        res = subprocess.run([sys.executable, "-m", "sga.replay"] + base + extra + ["--dense-cache", str(tmp_path / f"rc_{tag}"),
                             "--out", ref_out], env=env, capture_output=True, text=True, cwd=str(tmp_path))
        assert res.returncode == 0, res.stderr[-2000:]
        assert cli.main(base + extra + ["--dense-cache", str(tmp_path / f"oc_{tag}"), "--out", our_out]) == 0
        a, b = json.load(open(ref_out)), json.load(open(our_out))
        diffs = []
        walk(a, b, "", diffs)
        assert not [d for d in diffs if d[0] not in allowed], (tag, diffs[:10])
        assert len(a["branch_results"]["3"]["per_ratio"]["5.0"]["scores"]) == arms


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "tests", "ref_engine_harness.py")),
                    reason="no copy of the reference's engine test harness under baseline/_ref/tests")
def test_shadow_flow_matches_reference_engine(ref, monkeypatch):
    """Shadow mode on both engines: the stock dense step (decoupled AdamW behind the wrapper surface the
    reference's shadow step calls, ``sga/engine.py:612-744``) plus the read-only boundary scoring. Same
    gradient norms, the same support after every boundary (the score reads the post-clip gradient and
    the upcoming commit's bias corrections), the same cleared gradient buffer, weights to rounding."""
    import copy
    import types

    from sga_b200 import config as C
    from sga_b200.runtime.arena import FlatArena, ParamSpec
    from sga_b200.runtime.builder import build_engine
    from sga_b200.runtime.ddp import DataParallel, DDPConfig
    from sga_b200.runtime.optimizer import FlatOptimizer, OptimizerConfig

    mods = {n: types.ModuleType(n) for n in ("megatron", "megatron.core", "megatron.core.tensor_parallel",
                                             "megatron.core.transformer", "megatron.core.transformer.module")}
    mods["megatron.core.tensor_parallel"].param_is_not_tensor_parallel_duplicate = lambda p, g=None: True
    mods["megatron.core.transformer.module"].param_is_not_shared = lambda p: True
    for n, m in mods.items():
        monkeypatch.setitem(sys.modules, n, m)
    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")
    monkeypatch.syspath_prepend(os.path.join(REF, "tests"))
    ref("sga.engine")
    H = importlib.import_module("ref_engine_harness")

    class StockOpt(H._FakeMPOpt):
        def __init__(self, chunk):
            super().__init__(chunk)
            self.config = types.SimpleNamespace(clip_grad=1.0, log_num_zeros_in_grad=False)
            self.optimizer = torch.optim.AdamW(self.main_params, lr=1e-3, betas=(0.9, 0.95), eps=1e-8,
                                               weight_decay=1e-2)

        def clip_grad_norm(self, clip_grad):
            total = float(torch.sqrt(sum((mp.grad.float() ** 2).sum() for mp in self.main_params)))
            c = min(1.0, clip_grad / (total + 1e-6))
            if c < 1.0:
                for mp in self.main_params:
                    mp.grad.data.mul_(c)
            return total

        def count_zeros(self):
            return sum(int((mp.grad == 0).sum()) for mp in self.main_params)

        def step_with_ready_grads(self):
            self.optimizer.step()
            self._copy_main_params_to_model_params()
            return True

    def run_reference(combo, extra, steps=14, seed=21):
        torch.manual_seed(seed)
        chunk = H._FakeChunk(n_params=3, numel_per=64)
        mp = StockOpt(chunk)
        p0 = [p.detach().clone() for p in chunk.params]
        eng = H._build_engine(combo, extra)
        eng._dp_cp_group = lambda: None
        eng.attach(chunk)
        gen = torch.Generator().manual_seed(seed + 1)
        grads, log = [], []
        with H._ReplicaWorld(world=1):
            for step in range(1, steps + 1):
                g = torch.randn(chunk.bucket.grad_data.numel(), generator=gen)
                grads.append(g.clone())
                chunk.bucket.grad_data += g
                if not eng.grad_sync(chunk, force_all_reduce=False):
                    chunk.finish_grad_sync()
                _ok, gn, _nz = eng.optimizer_step(mp, [chunk], step)
                mk = eng._bucket_states[0].active_mask_u8
                log.append((float(gn), None if mk is None else mk.view(-1).to(torch.uint8).clone(),
                            chunk.bucket.grad_data.clone()))
                chunk.bucket.grad_data.zero_()  # the stock loop zeroes the buffer between steps
        return p0, grads, log, torch.cat([m.reshape(-1) for m in mp.main_params])

    def run_ours(combo, extra, p0, grads):
        kw = {**combo["config"], **combo["selection_params"], **combo["opt_params"], **combo.get("backend_params", {}),
              "sga_score": combo["score"], "sga_selection": combo["selection"], "sga_optimizer": combo["opt"],
              "sga_backend": combo["backend"], "sga_enabled": True, **extra}
        C.set_args(C.make_args(**kw))
        model = types.SimpleNamespace()
        model.arena = FlatArena([ParamSpec(f"p{i}", tuple(p.shape), 0, "zeros") for i, p in enumerate(p0)],
                                bucket_elems=10 ** 9, device="cpu")
        model.named_parameters = lambda: [(s.name, s.model) for s in model.arena.slots]
        for s, p in zip(model.arena.slots, p0):
            s.main.copy_(p)
        model.arena.sync_model_from_main()
        ddp = DataParallel(model, transport="local",
                           ddp_config=DDPConfig(average_in_collective=False, overlap_grad_reduce=False))
        opt = FlatOptimizer(model.arena, OptimizerConfig(lr=1e-3, weight_decay=1e-2, adam_beta1=0.9, adam_beta2=0.95,
                                                         adam_eps=1e-8, clip_grad=1.0))
        eng = build_engine(quiet=True)
        eng.log_interval = 0
        eng.attach(ddp)
        log = []
        slots = model.arena.slots
        for step, g in enumerate(grads, 1):
            off = 0
            for s in slots:
                n = s.end - s.start
                model.arena.main_grad[s.start:s.end] += g[off:off + n]
                off += n
            ddp.begin_step()
            eng.begin_step(ddp, step)
            if not eng.grad_sync(ddp, False):
                ddp.finish_grad_sync()
            _ok, gn, _nz = eng.optimizer_step(opt, [ddp], step)
            mk = eng._active_mask_arena() if eng._active_support is not None else None
            log.append((float(gn), None if mk is None else torch.cat([mk[s.start:s.end] for s in slots]).clone(),
                        torch.cat([model.arena.main_grad[s.start:s.end] for s in slots]).clone()))
            model.arena.main_grad.zero_()
        return log, torch.cat([s.main.reshape(-1) for s in slots])

    cases = [(H._UPDATE, {"sga_shadow": True}), (H._ABS_M, {"sga_shadow": True}),
             ({**H._UPDATE, "score": "coi"}, {"sga_shadow": True}), ({**H._ABS_M, "score": "abs_g"}, {"sga_shadow": True}),
             (H._ABS_M, {"sga_shadow": True, "sga_shadow_score": False})]
    for combo, extra in cases:
        c = copy.deepcopy(combo)
        tag = (combo["score"], combo["backend"], extra)
        p0, grads, rlog, rw = run_reference(c, extra)
        olog, ow = run_ours(c, extra, p0, grads)
        for (gn, mk, gb), (gn2, mk2, gb2) in zip(rlog, olog):
            assert abs(gn - gn2) <= 1e-6 * max(gn, 1e-9), tag
            assert (mk is None) == (mk2 is None) and (mk is None or torch.equal(mk, mk2)), tag
            assert torch.equal(gb, gb2), tag
        assert float((rw - ow).abs().max()) <= 5e-6, tag  # torch.optim.AdamW folds the bias corrections differently


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "tests", "ref_engine_harness.py")),
                    reason="no copy of the reference's engine test harness under baseline/_ref/tests")
@pytest.mark.parametrize("async_writer", [False, True])
def test_trace_files_equal_reference_collector(ref, monkeypatch, tmp_path, async_writer):
    """Both engines with their trace collectors on over the same run (two branch points, windows that
    span full and sparse steps): the same file names (the step number is the engine's own step), the
    same phase tags, bit-identical gradient payloads, weights and moments to an ulp."""
    import copy
    import types

    from sga_b200 import config as C
    from sga_b200.runtime.arena import FlatArena, ParamSpec
    from sga_b200.runtime.builder import build_engine
    from sga_b200.runtime.ddp import DataParallel, DDPConfig
    from sga_b200.runtime.optimizer import FlatOptimizer, OptimizerConfig

    mods = {n: types.ModuleType(n) for n in ("megatron", "megatron.core", "megatron.core.tensor_parallel",
                                             "megatron.core.transformer", "megatron.core.transformer.module")}
    mods["megatron.core.tensor_parallel"].param_is_not_tensor_parallel_duplicate = lambda p, g=None: True
    mods["megatron.core.transformer.module"].param_is_not_shared = lambda p: True
    for n, m in mods.items():
        monkeypatch.setitem(sys.modules, n, m)
    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")
    monkeypatch.syspath_prepend(os.path.join(REF, "tests"))
    ref("sga.engine")
    H = importlib.import_module("ref_engine_harness")
    ta, tb = str(tmp_path / "ref"), str(tmp_path / "ours")
    combo = copy.deepcopy(H._ABS_M)
    extra = {"sga_trace_branch_points": [3, 7], "sga_trace_window": 3, "sga_trace_async": async_writer}

    torch.manual_seed(3)
    chunk = H._FakeChunk(n_params=3, numel_per=256)
    mp = H._FakeMPOpt(chunk)
    p0 = [p.detach().clone() for p in chunk.params]
    eng = H._build_engine(combo, {**extra, "sga_trace_dir": ta})
    eng.attach(chunk)
    gen = torch.Generator().manual_seed(4)
    grads = []
    with H._ReplicaWorld(world=1):
        for step in range(1, 13):  # the step past the last window drains the asynchronous writer
            g = torch.randn(chunk.bucket.grad_data.numel(), generator=gen)
            grads.append(g.clone())
            chunk.bucket.grad_data += g
            eng.grad_sync(chunk, force_all_reduce=False)
            eng.optimizer_step(mp, [chunk], step)

    kw = {**combo["config"], **combo["selection_params"], **combo["opt_params"], **combo.get("backend_params", {}),
          "sga_score": combo["score"], "sga_selection": combo["selection"], "sga_optimizer": combo["opt"],
          "sga_backend": combo["backend"], "sga_enabled": True, **extra, "sga_trace_dir": tb}
    C.set_args(C.make_args(**kw))
    model = types.SimpleNamespace()
    model.arena = FlatArena([ParamSpec(f"p{i}", tuple(p.shape), 0, "zeros") for i, p in enumerate(p0)],
                            bucket_elems=10 ** 9, device="cpu")
    model.named_parameters = lambda: [(s.name, s.model) for s in model.arena.slots]
    for s, p in zip(model.arena.slots, p0):
        s.main.copy_(p)
    model.arena.sync_model_from_main()
    ddp = DataParallel(model, transport="local",
                       ddp_config=DDPConfig(average_in_collective=False, overlap_grad_reduce=False))
    opt = FlatOptimizer(model.arena, OptimizerConfig(lr=1e-3, weight_decay=1e-2, adam_beta1=0.9, adam_beta2=0.95,
                                                     adam_eps=1e-8, clip_grad=1.0))
    ours = build_engine(quiet=True)
    ours.log_interval = 0
    ours.attach(ddp)
    for step, g in enumerate(grads, 1):
        off = 0
        for s in model.arena.slots:
            n = s.end - s.start
            model.arena.main_grad[s.start:s.end] += g[off:off + n]
            off += n
        ddp.begin_step()
        ours.begin_step(ddp, step)
        if not ours.grad_sync(ddp, False):
            ddp.finish_grad_sync()
        ours.optimizer_step(opt, [ddp], step)
    ours._trace.close()

    names = sorted(os.listdir(ta))
    assert names == sorted(os.listdir(tb))
    assert names == ["catalog.pt"] + sorted([f"step_{t:06d}_g.pt" for t in (3, 4, 5, 7, 8, 9)]
                                            + [f"step_{t:06d}_state.pt" for t in (3, 7)])
    for name in names[1:]:
        a = torch.load(os.path.join(ta, name), weights_only=False)
        b = torch.load(os.path.join(tb, name), weights_only=False)
        assert (a["meta"]["step"], a["meta"]["phase"]) == (b["meta"]["step"], b["meta"]["phase"]), name
        assert abs(a["meta"]["grad_norm"] - b["meta"]["grad_norm"]) <= 1e-6 * a["meta"]["grad_norm"], name
        if name.endswith("_g.pt"):
            assert all(torch.equal(a["payload"][k], b["payload"][k]) for k in a["payload"]), name
        else:
            assert all(torch.equal(a["payload"]["g"][k], b["payload"]["g"][k]) for k in a["payload"]["g"]), name
            for part, tol in (("w", 1e-7), ("m", 4e-9), ("v", 4e-9)):  # the reference's dense steps run torch.optim.Adam
                assert all(float((a["payload"][part][k] - b["payload"][part][k]).abs().max()) <= tol
                           for k in a["payload"][part]), (name, part)


def test_resume_guard_decisions_equal(ref, monkeypatch, tmp_path):
    """The reference's resume guard (``sga/train_gpt.py:49-194``; the modules of its external training
    stack are empty stand-ins, the two checkpoint-path helpers it calls spell Megatron's layout) and this
    framework's, over stub checkpoints: the same pass / refuse decision in every scenario."""
    import types

    from sga_b200.config.validation import sga_defaults as our_defaults
    from sga_b200.runtime import checkpoint as ck

    torch.serialization.add_safe_globals([argparse.Namespace])

    def stand_in(name, **attrs):
        m = types.ModuleType(name)
        for k, v in attrs.items():
            setattr(m, k, v)
        monkeypatch.setitem(sys.modules, name, m)

    for name in ("pretrain_gpt", "megatron", "megatron.core"):
        stand_in(name)
    stand_in("megatron.core.enums", ModelType=None)
    stand_in("megatron.training", inprocess_restart=None, pretrain=None)
    stand_in("megatron.training.argument_utils", pretrain_cfg_container_from_args=None)
    stand_in("megatron.training.arguments", parse_and_validate_args=None)
    stand_in("gpt_builders", gpt_builder=None)
    stand_in("model_provider", model_provider=None)
    stand_in("megatron.training.checkpointing",
             get_checkpoint_tracker_filename=lambda load: os.path.join(load, "latest_checkpointed_iteration.txt"),
             get_checkpoint_name=lambda load, it, return_base_dir=False: os.path.join(load, f"iter_{it:07d}"))
    R = ref("sga.train_gpt")
    ref_defaults = ref("sga.config.validation").sga_defaults

    def namespace(defaults, **over):
        a = argparse.Namespace(**defaults)
        a.train_iters, a.load, a.sga_allow_config_override = 100, None, False
        for k, v in over.items():
            setattr(a, k, v)
        return a

    def save(root, it, saved_args, tracker=True, shard=True, raw=None):
        os.makedirs(root, exist_ok=True)
        if tracker:
            with open(os.path.join(root, "latest_checkpointed_iteration.txt"), "w") as fh:
                fh.write(str(it) if tracker is True else tracker)
        if shard:
            d = os.path.join(root, f"iter_{it:07d}", "mp_rank_00")
            os.makedirs(d, exist_ok=True)
            torch.save(raw if raw is not None else {"args": saved_args, "iteration": it},
                       os.path.join(d, "model_optim_rng.pt"))

    base = dict(sga_enabled=True, sga_score="abs_g", sga_backend="torch_pipelined_index",
                sga_selection_method="histogram", sga_selection_ratio_percent=10.0, sga_cycle_period=4)
    pct = {**base, "sga_cycle_start_iter_percent": 10.0}
    scenarios = {
        "no tracker": (dict(saved=base, cur=base, tracker=False), "pass"),
        "same": (dict(saved=base, cur=base), "pass"),
        "value differs": (dict(saved=base, cur={**base, "sga_cycle_period": 8}), "refuse"),
        "10 vs 10.0": (dict(saved={**base, "sga_selection_ratio_percent": 10}, cur=base), "refuse"),
        "release tracker": (dict(saved=base, cur={**base, "sga_cycle_period": 8}, tracker="release"), "pass"),
        "no shard": (dict(saved=base, cur=base, shard=False), "refuse"),
        "no saved sga attrs": (dict(saved=None, cur=base), "refuse"),
        "legacy json era": (dict(saved={**base, "sga_config": "{}"}, cur=base), "refuse"),
        "retired key": (dict(saved={**base, "sga_old_knob": 3}, cur=base), "refuse"),
        "override": (dict(saved=base, cur={**base, "sga_cycle_period": 8, "sga_allow_config_override": True}), "pass"),
        "sga off": (dict(saved=base, cur={**base, "sga_enabled": False, "sga_cycle_period": 8}), "pass"),
        "percent same": (dict(saved=pct, cur=pct), "pass"),
        "percent, train_iters changed": (dict(saved={**pct, "train_iters": 50}, cur=pct), "refuse"),
        "list reordered": (dict(saved={**base, "sga_always_sync_layers": "a,b"},
                                cur={**base, "sga_always_sync_layers": "b,a"}), "refuse"),
        "older checkpoint lacks a key": (dict(saved=base, cur=base, drop=["sga_backend_index_slices"]), "pass"),
        "corrupt shard": (dict(saved=base, cur=base, raw=[1, 2, 3]), "refuse"),
        "newest iteration decides": (dict(saved=base, cur=base, older={**base, "sga_cycle_period": 8}), "pass"),
    }
    for name, (sc, want) in scenarios.items():
        got = []
        for side, (defaults, guard) in enumerate(((ref_defaults(), R._sga_resume_guard),
                                                  (our_defaults(), ck.sga_resume_guard))):
            root = str(tmp_path / f"{abs(hash(name))}_{side}")
            saved = argparse.Namespace(train_iters=100) if sc["saved"] is None else namespace(defaults, **sc["saved"])
            for k in sc.get("drop", []):
                delattr(saved, k)
            if "older" in sc:
                save(root, 100, namespace(defaults, **sc["older"]))
                save(root, 500, saved, tracker="100\n500")
            else:
                save(root, 500, saved, tracker=sc.get("tracker", True), shard=sc.get("shard", True), raw=sc.get("raw"))
            cur = namespace(defaults, **sc["cur"])
            cur.load = root
            try:
                guard(cur)
                got.append("pass")
            except SystemExit:
                got.append("refuse")
        assert got == [want, want], (name, got)
