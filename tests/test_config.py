"""Flag surface, validation rules and write-backs of the ``sga_*`` configuration."""
import argparse
import os

import pytest

from sga_b200 import config as C
from sga_b200.config.arguments import add_sga_args, sga_bool, sga_int_or_null

# name -> (type name, default): the reference surface, reproduced exactly
GOLDEN = {
    "sga_enabled": ("sga_bool", False), "sga_shadow": ("sga_bool", False), "sga_shadow_score": ("sga_bool", True),
    "sga_always_sync_layers": ("str", None), "sga_cycle_start_iter": ("int", 0),
    "sga_cycle_start_iter_percent": ("float", None), "sga_cycle_period": ("int", 1),
    "sga_cycle_decouple_full_sync_interval_and_period": ("sga_bool", False),
    "sga_cycle_full_sync_interval": ("int", None), "sga_checks": ("sga_bool", True),
    "sga_checks_count_guard": ("sga_bool", True), "sga_checks_support_consistency": ("sga_bool", True),
    "sga_checks_norm_spread": ("sga_bool", True), "sga_checks_rng_bracket": ("sga_bool", True),
    "sga_trace_dir": ("str", None), "sga_trace_branch_points": ("str", None), "sga_trace_window": ("int", 100),
    "sga_trace_dump_dtype": ("str", "fp32"), "sga_trace_async": ("sga_bool", False),
    "sga_trace_async_backend": ("str", "cpu_snapshot"), "sga_trace_async_queue_depth": ("int", 2),
    "sga_trace_async_worker_count": ("int", 1), "sga_trace_async_max_workset_gib": ("float", 16.0),
    "sga_score": ("str", None), "sga_selection": ("str", "topk"), "sga_selection_method": ("str", None),
    "sga_selection_ratio_percent": ("float", None), "sga_selection_histogram_mode": ("str", "exact"),
    "sga_selection_topk_histogram_add_global_allreduce": ("sga_bool", False),
    "sga_selection_adaptive_warmup_syncs": ("sga_int_or_null", 5),
    "sga_selection_adaptive_warmup_mode": ("str", "fast"), "sga_selection_block_size": ("int", 1),
    "sga_selection_block_reduce": ("str", "mean"), "sga_optimizer": ("str", "adamw"),
    "sga_optimizer_residual_mean": ("sga_bool", False),
    "sga_optimizer_full_sync_inactive_lr_scale": ("float", 1.0), "sga_optimizer_compact_search": ("str", "table"),
    "sga_backend": ("str", "dense"), "sga_backend_emission": ("str", "auto"), "sga_backend_layout": ("str", "auto"),
    "sga_backend_high_priority_group": ("sga_bool", False), "sga_backend_index_slices": ("int", 2),
    "sga_backend_mask_slices": ("int", 2), "sga_backend_timer": ("str", None),
}
EXTENSIONS = {"sga_selection_locality", "sga_backend_transport", "sga_bucket_elems"}


def _enabled(**kw):
    base = dict(sga_enabled=True, sga_score="abs_g", sga_selection_method="histogram",
                sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=10.0,
                sga_backend="torch_pipelined_index")
    base.update(kw)
    return C.make_args(**base)


def test_golden_flag_table():
    acts = C.sga_actions()
    assert set(acts) == set(GOLDEN) | EXTENSIONS
    assert len(GOLDEN) == 44
    for dest, (tname, default) in GOLDEN.items():
        a = acts[dest]
        assert a.default == default, dest
        assert a.type.__name__ == tname, (dest, a.type.__name__)
        assert a.option_strings == ["--" + dest.replace("_", "-")]


def test_bool_and_null_types():
    assert sga_bool("TRUE") is True and sga_bool("false") is False and sga_bool(True) is True
    with pytest.raises(argparse.ArgumentTypeError):
        sga_bool("yes")
    assert sga_int_or_null("null") is None and sga_int_or_null("7") == 7 and sga_int_or_null(None) is None


def test_flag_and_namespace_equivalence():
    p = argparse.ArgumentParser()
    add_sga_args(p)
    ns = p.parse_args(["--sga-enabled", "true", "--sga-score", "abs_m", "--sga-selection-method", "histogram",
                       "--sga-selection-histogram-mode", "balanced", "--sga-selection-ratio-percent", "40",
                       "--sga-backend", "torch_pipelined_index", "--sga-cycle-period", "4",
                       "--sga-selection-adaptive-warmup-syncs", "null", "--sga-always-sync-layers", "b,a,,"[:3]])
    ns.train_iters, ns.pipeline_model_parallel_size = 100, 1
    C.validate_sga_args(ns)
    assert ns.sga_selection_ratio_percent == 40.0 and ns.sga_selection_adaptive_warmup_syncs is None
    assert ns.sga_always_sync_layers == ["a", "b"]
    assert ns.sga_backend_layout == "er"
    with pytest.raises(SystemExit):
        p.parse_args(["--sga-score", "nonsense"])


def test_disabled_runs_zero_checks():
    ns = C.make_args(sga_score=None, sga_cycle_period=-5, sga_backend="dense")
    C.validate_sga_args(ns)  # nothing is validated while disabled


def test_required_when_enabled():
    with pytest.raises(ValueError, match="sga_score is required"):
        C.validate_sga_args(_enabled(sga_score=None))
    with pytest.raises(ValueError, match="still 'dense'"):
        C.validate_sga_args(_enabled(sga_backend="dense"))
    with pytest.raises(ValueError, match="sga_selection_method is required"):
        C.validate_sga_args(_enabled(sga_selection_method=None))
    with pytest.raises(ValueError, match="ratio_percent is required"):
        C.validate_sga_args(_enabled(sga_selection_ratio_percent=None))
    with pytest.raises(ValueError, match="Unknown SGA backend"):
        C.validate_sga_args(_enabled(sga_backend="bogus"))
    for bad in (0.0, 100.0, float("nan"), float("inf"), 10):
        with pytest.raises(ValueError, match="ratio_percent"):
            C.validate_sga_args(_enabled(sga_selection_ratio_percent=bad))


def test_checks_master_forces_subflags_off():
    ns = _enabled(sga_checks=False)
    C.validate_sga_args(ns)
    assert not any(getattr(ns, d) for d in vars(ns) if d.startswith("sga_checks_"))


def test_percent_resolution_and_exclusivity():
    ns = _enabled(sga_cycle_start_iter_percent=40.0, train_iters=50)
    C.validate_sga_args(ns)
    assert ns.sga_cycle_start_iter == 20 and ns.sga_cycle_start_iter_percent is None
    with pytest.raises(ValueError, match="not both"):
        C.validate_sga_args(_enabled(sga_cycle_start_iter_percent=40.0, sga_cycle_start_iter=3, train_iters=50))
    with pytest.raises(ValueError, match="train_iters"):
        C.validate_sga_args(_enabled(sga_cycle_start_iter_percent=40.0))
    with pytest.raises(ValueError, match=r"\[0, 100\]"):
        C.validate_sga_args(_enabled(sga_cycle_start_iter_percent=140.0, train_iters=50))


def test_cycle_rules():
    with pytest.raises(ValueError, match="period must be >= 1"):
        C.validate_sga_args(_enabled(sga_cycle_period=0))
    with pytest.raises(ValueError, match="decouple switch is false"):
        C.validate_sga_args(_enabled(sga_cycle_period=8, sga_cycle_full_sync_interval=4))
    with pytest.raises(ValueError, match="is unset"):
        C.validate_sga_args(_enabled(sga_cycle_period=8, sga_cycle_decouple_full_sync_interval_and_period=True))
    for bad in (8, 3, 0):
        with pytest.raises(ValueError, match="must satisfy"):
            C.validate_sga_args(_enabled(sga_cycle_period=8, sga_cycle_decouple_full_sync_interval_and_period=True,
                                         sga_cycle_full_sync_interval=bad))
    C.validate_sga_args(_enabled(sga_cycle_period=8, sga_cycle_decouple_full_sync_interval_and_period=True,
                                 sga_cycle_full_sync_interval=4))


def test_trace_rules():
    with pytest.raises(ValueError, match="sga_trace_dir is required"):
        C.validate_sga_args(_enabled(sga_trace_window=5))
    ns = _enabled(sga_trace_dir="/tmp/x", sga_trace_branch_points="30,10,10")
    C.validate_sga_args(ns)
    assert ns.sga_trace_branch_points == [10, 30]
    with pytest.raises(ValueError, match="branch_points"):
        C.validate_sga_args(_enabled(sga_trace_dir="/tmp/x", sga_trace_branch_points="null"))
    with pytest.raises(ValueError, match="requires sga_trace_async=true"):
        C.validate_sga_args(_enabled(sga_trace_dir="/tmp/x", sga_trace_async_backend="pinned_cuda"))
    with pytest.raises(ValueError, match="worker_count must be <="):
        C.validate_sga_args(_enabled(sga_trace_dir="/tmp/x", sga_trace_async=True, sga_trace_async_worker_count=3))
    with pytest.raises(ValueError, match="max_workset_gib"):
        C.validate_sga_args(_enabled(sga_trace_dir="/tmp/x", sga_trace_async_max_workset_gib=0.0))
    with pytest.raises(ValueError, match="sga_trace_window"):
        C.validate_sga_args(_enabled(sga_trace_dir="/tmp/x", sga_trace_window=0))


def test_shadow_rules():
    with pytest.raises(ValueError, match="sga_shadow_score is set"):
        C.validate_sga_args(_enabled(sga_shadow_score=False))
    with pytest.raises(ValueError, match="adams"):
        C.validate_sga_args(_enabled(sga_shadow=True, sga_optimizer="adams"))
    C.validate_sga_args(_enabled(sga_shadow=True, sga_shadow_score=False))


def test_always_sync_rules():
    with pytest.raises(ValueError, match="non-empty"):
        C.validate_sga_args(_enabled(sga_always_sync_layers="a,,b"))
    with pytest.raises(ValueError, match="null"):
        C.validate_sga_args(_enabled(sga_always_sync_layers="null"))
    with pytest.raises(ValueError, match="pipeline_model_parallel_size == 1"):
        C.validate_sga_args(_enabled(sga_always_sync_layers="norm", pipeline_model_parallel_size=2))
    ns = _enabled(sga_always_sync_layers="  ")
    C.validate_sga_args(ns)
    assert ns.sga_always_sync_layers is None
    ns = _enabled(sga_always_sync_layers=["z", "a", "z"])
    C.validate_sga_args(ns)
    assert ns.sga_always_sync_layers == ["a", "z"]


def test_dual_lr_rules():
    with pytest.raises(ValueError, match="finite float >= 0"):
        C.validate_sga_args(_enabled(sga_cycle_period=4, sga_optimizer_full_sync_inactive_lr_scale=-1.0))
    with pytest.raises(ValueError, match="finite float >= 0"):
        C.validate_sga_args(_enabled(sga_cycle_period=4, sga_optimizer_full_sync_inactive_lr_scale=float("nan")))
    with pytest.raises(ValueError, match="sga_shadow true"):
        C.validate_sga_args(_enabled(sga_cycle_period=4, sga_shadow=True,
                                     sga_optimizer_full_sync_inactive_lr_scale=0.5))
    with pytest.raises(ValueError, match="period 1"):
        C.validate_sga_args(_enabled(sga_optimizer_full_sync_inactive_lr_scale=0.5))
    C.validate_sga_args(_enabled(sga_cycle_period=4, sga_optimizer_full_sync_inactive_lr_scale=0.0))


def test_selection_freeze_and_escape(monkeypatch):
    monkeypatch.delenv("SGA_ALLOW_FROZEN_SELECTION", raising=False)
    with pytest.raises(ValueError, match="frozen to histogram balanced"):
        C.validate_sga_args(_enabled(sga_selection_method="exact", sga_selection_histogram_mode="exact"))
    with pytest.raises(ValueError, match="frozen"):
        C.validate_sga_args(_enabled(sga_selection_histogram_mode="fast"))
    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")
    C.validate_sga_args(_enabled(sga_selection_method="adaptive"))


def test_block_and_layout_rules(monkeypatch):
    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")
    for bad in (0, 3, 2048, True):
        with pytest.raises(ValueError, match="power of two"):
            C.validate_sga_args(_enabled(sga_selection_block_size=bad, sga_backend_emission="writeback"))
    with pytest.raises(ValueError, match="only applies to the histogram"):
        C.validate_sga_args(_enabled(sga_selection_method="exact", sga_selection_block_size=8))
    with pytest.raises(ValueError, match="'fast'"):
        C.validate_sga_args(_enabled(sga_selection_histogram_mode="fast", sga_selection_block_size=8,
                                     sga_backend_emission="writeback"))
    with pytest.raises(ValueError, match="'er'"):
        C.validate_sga_args(_enabled(sga_selection_block_size=8, sga_backend_layout="er"))
    with pytest.raises(ValueError, match="block_size == 1"):
        C.validate_sga_args(_enabled(sga_backend_layout="bb"))
    with pytest.raises(ValueError, match="torch_pipelined_mask"):
        C.validate_sga_args(_enabled(sga_backend="torch_pipelined_mask", sga_selection_block_size=8,
                                     sga_backend_layout="eb"))
    with pytest.raises(ValueError, match="needs sga_backend_emission 'writeback'"):
        C.validate_sga_args(_enabled(sga_selection_block_size=8))
    ns = _enabled(sga_selection_block_size=8, sga_backend_emission="writeback")
    C.validate_sga_args(ns)
    assert ns.sga_backend_layout == "bb"
    C.validate_sga_args(_enabled(sga_selection_block_size=8, sga_backend_layout="eb"))
    with pytest.raises(ValueError, match=r"\[4, 64\]"):
        C.validate_sga_args(_enabled(sga_backend="nccl_pipelined_index", sga_selection_block_size=128))
    with pytest.raises(ValueError, match="'compact' is only supported"):
        C.validate_sga_args(_enabled(sga_backend="torch_pipelined_mask", sga_backend_emission="compact"))


def test_rank_local_rules():
    ok = _enabled(sga_selection_locality="rank_local", sga_selection_method="exact", sga_cycle_period=0)
    C.validate_sga_args(ok)
    # every score runs inside the fused index kernel; the mask backend keeps |grad + residual|
    for score in ("abs_m", "update", "coi"):
        C.validate_sga_args(_enabled(sga_selection_locality="rank_local", sga_score=score,
                                     sga_selection_method="exact"))
    with pytest.raises(ValueError, match="rank_local"):
        C.validate_sga_args(_enabled(sga_selection_locality="rank_local", sga_score="abs_m",
                                     sga_selection_method="exact", sga_backend="torch_pipelined_mask"))
    with pytest.raises(ValueError, match="sga_shadow"):
        C.validate_sga_args(_enabled(sga_selection_locality="rank_local", sga_shadow=True,
                                     sga_selection_method="exact"))


def test_validation_is_idempotent():
    ns = _enabled(sga_trace_dir="/tmp/x", sga_trace_branch_points="5,1", sga_always_sync_layers="b,a")
    C.validate_sga_args(ns)
    snap = dict(vars(ns))
    C.validate_sga_args(ns)
    assert dict(vars(ns)) == snap


def test_singleton_and_config_attrs():
    ns = _enabled(sga_backend_timer="/tmp/t")
    C.set_args(ns)
    assert C.get_args() is ns
    attrs = C.sga_config_attrs(ns)
    assert "sga_backend_timer" not in attrs and attrs["sga_score"] == "abs_g"
    assert all(k.startswith("sga_") for k in attrs)


def test_arguments_module_only_declares():
    """``config/arguments.py`` holds declarations: imports, constants, the two value-type helpers,
    group functions whose bodies are ``add_argument_group`` / ``add_argument`` calls, and the entry
    that calls them. No rule, no cross-flag logic, no I/O (those belong to ``validation.py``)."""
    import ast
    import inspect

    from sga_b200.config import arguments as A

    tree = ast.parse(inspect.getsource(A))
    types = {"sga_bool", "sga_int_or_null"}
    for node in tree.body:
        if isinstance(node, (ast.Import, ast.ImportFrom)):
            continue
        if isinstance(node, ast.Expr) and isinstance(node.value, ast.Constant):  # docstring
            continue
        if isinstance(node, ast.Assign):
            assert all(isinstance(t, ast.Name) and t.id.isupper() for t in node.targets), ast.dump(node)
            continue
        assert isinstance(node, ast.FunctionDef), f"unexpected top-level statement: {ast.dump(node)[:80]}"
        if node.name in types:
            continue
        for stmt in node.body:
            if isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Constant):
                continue
            if isinstance(stmt, ast.Return):
                continue
            call = stmt.value if isinstance(stmt, (ast.Expr, ast.Assign)) else None
            if isinstance(stmt, ast.For):  # the entry point: for group in (...): group(parser)
                assert all(isinstance(x, ast.Expr) and isinstance(x.value, ast.Call) for x in stmt.body)
                continue
            assert isinstance(call, ast.Call), f"{node.name}: only calls are allowed, found {ast.dump(stmt)[:80]}"
            fn = call.func
            name = fn.attr if isinstance(fn, ast.Attribute) else getattr(fn, "id", "")
            assert name in {"add_argument", "add_argument_group"} or name.startswith("_"), f"{node.name}: call to {name}"


def test_every_flag_has_a_consumer():
    """Every declared ``sga_*`` destination is read somewhere outside its declaration, so a flag can
    never silently do nothing. The flags that select nothing in this framework are listed here with
    the reason, and nothing may read them (or they must leave the list)."""
    import os
    import re

    no_effect = {
        # chooses between two bracket searches of the reference's compact merge-join kernel; here the
        # reduced values are read from the dense bucket, so there is no search. Accepted, part of the
        # saved configuration identity, selects nothing.
        "sga_optimizer_compact_search",
    }
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "sga_b200")
    text = {}
    for d, _s, files in os.walk(root):
        for f in files:
            if f.endswith(".py") and not (d.endswith("config") and f == "arguments.py"):
                text[os.path.join(d, f)] = open(os.path.join(d, f)).read()
    blob = "\n".join(text.values())
    dests = sorted(C.sga_defaults())
    assert len(dests) >= 44
    unread = [k for k in dests if not re.search(rf"\b{k}\b", blob)]
    assert sorted(unread) == sorted(no_effect), f"flags nobody reads: {sorted(set(unread) - no_effect)}; " \
                                                f"listed as without effect but read: {sorted(no_effect - set(unread))}"

