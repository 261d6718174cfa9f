"""``python -m sga_b200.replay`` -- offline evaluation of score / ratio / cycle
configurations against a captured trace.

For every requested branch point the fused engine replays the dense arm and
every configuration of the grid ``scores x ratios x cycle lengths x optimizers
x fold x dual-lr`` over the window, and reports the branch-point ranking
quality of each score (NDCG@k, recall@k, missed masses against the realised
dense displacement) and each configuration's distortion at the horizons.

Report JSON (shape of ``sga/replay.py:1387-1416,2022-2070``)::

    {"trace_dir", "config": {...},
     "branch_results": {t0: {"t0", "state_absent", "window_len", "window_steps", "cycle_lens",
                             "horizon_steps", "meta", "replay": {...}, "scores": {...},
                             "per_ratio": {r: {"k", "scores": {key: {"distortion": {h: d}, "ndcg_at_k", ...}}}}}}}

Arm keys carry ``@T{t}``, ``@{opt}``, ``@fold``, ``@dl{g}`` suffixes only for
axes with more than one value. CLI surface: ``sga/replay.py:1609-1797``.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

from . import core as RC
from . import fused as RF


def _floats(s):
    return [float(x) for x in str(s).split(",") if x.strip()]


def _ints(s):
    return [int(x) for x in str(s).split(",") if x.strip()]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("sga_b200.replay", description=__doc__.splitlines()[0])
    p.add_argument("--trace-dir", required=True)
    p.add_argument("--branch-point", default="all", help="comma ints or 'all'")
    p.add_argument("--self-check", nargs=2, type=int, metavar=("FROM", "TO"), default=None,
                   help="replay the dense arm from state FROM to state TO and compare with the dumped state")
    p.add_argument("--ratios", default="10,20")
    p.add_argument("--horizons", default=None, help="comma ints (default: the window length)")
    p.add_argument("--out", default=None)
    p.add_argument("--device", default="cpu")
    p.add_argument("--chunk-mb", type=int, default=256)
    p.add_argument("--replay-dtype", choices=("fp32", "fp64"), default="fp32")
    p.add_argument("--norm-dtype", choices=("fp32", "fp64"), default="fp64")
    p.add_argument("--trace-dtype", choices=("fp32", "bf16"), default=None)
    p.add_argument("--dense-cache", default=None)
    p.add_argument("--replay-mode", choices=("zerofill", "cycle"), default="cycle")
    p.add_argument("--cycle-len", type=int, default=None)
    p.add_argument("--cycle-lens", default=None)
    p.add_argument("--optimizer", default="adamw", help="comma set of {adamw, adams}")
    p.add_argument("--fold", default="off", help="comma set of {off, on}")
    p.add_argument("--dual-lr", default="1", help="comma floats")
    p.add_argument("--fused", action="store_true", help="accepted for compatibility; the fused engine is the only one")
    p.add_argument("--fused-shards", type=int, default=1)
    p.add_argument("--selection-semantics", choices=("topk", "balanced-histogram"), default=None,
                   help="rule behind the branch-point and boundary selections: balanced-histogram (the default of "
                        "single-node cycle replay: the online engine's stride-8, whole-crossing-bin histogram "
                        "mode) or topk (exact global top-k with index-ordered ties; the default with --nodes and "
                        "for zerofill)")
    p.add_argument("--fused-max-configs", type=int, default=12)
    p.add_argument("--fused-state-budget-mb", type=float, default=0.0)
    p.add_argument("--nodes", default=None, help="comma host list for a multi-node replay")
    p.add_argument("--ssh-key", default=None)
    p.add_argument("--preflight-timeout", type=float, default=600.0)
    p.add_argument("--run-deadline", type=float, default=0.0)
    p.add_argument("--launch-log-dir", default=None)
    p.add_argument("--fused-g-residency", action="store_true")
    p.add_argument("--fused-dev-reduce", action="store_true")
    p.add_argument("--score-names", default="abs_g,abs_m,coi,update")
    p.add_argument("--window", type=int, default=100)
    p.add_argument("--seed", type=int, default=1234)
    p.add_argument("--verbose", action="store_true")
    return p


def build_configs(ns):
    from ..plugins.scores import score_names

    scores = [s for s in str(ns.score_names).split(",") if s]
    for s in scores:
        if s not in score_names():
            raise ValueError(f"unknown score '{s}' (registered: {score_names()})")
    ratios = _floats(ns.ratios)
    if ns.cycle_len is not None and ns.cycle_lens is not None:
        raise ValueError("give --cycle-len or --cycle-lens, not both")
    Ts = [ns.cycle_len] if ns.cycle_len is not None else (_ints(ns.cycle_lens) if ns.cycle_lens else [1])
    # the reference's defaults (sga/replay.py:1703-1715, 1876-1882): single-node cycle replay selects by
    # the online balanced-histogram rule; zerofill and multi-node replays need exact top-k
    if ns.selection_semantics is None:
        ns.selection_semantics = "balanced-histogram" if (ns.replay_mode == "cycle" and not ns.nodes) else "topk"
    if ns.selection_semantics == "balanced-histogram" and (ns.replay_mode != "cycle" or ns.nodes):
        raise ValueError("--selection-semantics balanced-histogram requires --replay-mode cycle on a single node")
    if ns.replay_mode == "zerofill":
        Ts = [10 ** 9]  # never a second boundary: unselected gradient mass just accumulates
    opts = [o for o in str(ns.optimizer).split(",") if o]
    for o in opts:
        if o not in ("adamw", "adams"):
            raise ValueError(f"unknown optimizer '{o}'")
    folds = [f == "on" for f in str(ns.fold).split(",") if f]
    duals = _floats(ns.dual_lr)
    multi = {"cycle_len": len(Ts) > 1, "optimizer": len(opts) > 1, "fold": len(folds) > 1, "dual_lr": len(duals) > 1}
    cfgs = [RC.CycleConfig(s, r, T, o, f, d) for o in opts for f in folds for d in duals for T in Ts for r in ratios
            for s in scores]
    return cfgs, scores, ratios, Ts, multi


def self_check(trace_dir, t_from, t_to, device="cpu") -> dict:
    """Dense-replay the logged gradients from one dumped state to the next and
    compare with what the run itself dumped there."""
    info = RC.discover_trace(trace_dir)
    meta, p0 = RC.load_state(info, t_from)
    _, p1 = RC.load_state(info, t_to)
    w, m, v = (RC.flatten(p0[k], info) for k in ("w", "m", "v"))
    steps = info.window(t_from, t_to - t_from)
    if len(steps) != t_to - t_from:
        raise ValueError(f"gradient files between {t_from} and {t_to} are not contiguous")
    wd = RC.group_vector(info, [g["weight_decay"] for g in meta["param_groups"]])
    hp = RC.Hyper(wd=wd, beta1=meta["param_groups"][0]["adam_beta1"], beta2=meta["param_groups"][0]["adam_beta2"],
                  eps=meta["param_groups"][0]["adam_eps"], clip=meta["clip_grad"])
    logged, lrs = [], []
    for t in steps:
        gm, gp = RC.load_g(info, t)
        logged.append(RC.flatten(gp, info))
        lrs.append(gm["lr"][0])
    snaps = RC.dense_replay(w, m, v, logged, lrs, hp, t_from, "adamw", {len(steps)})
    want = RC.flatten(p1["w"], info)
    err = float((snaps[len(steps)] - want).abs().max())
    return {"from": t_from, "to": t_to, "max_abs_err": err, "scale": float(want.abs().max())}


def sanitize(obj):
    if isinstance(obj, dict):
        return {str(k): sanitize(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [sanitize(v) for v in obj]
    if isinstance(obj, float) and (math.isnan(obj) or math.isinf(obj)):
        return None
    if isinstance(obj, torch.Tensor):
        return obj.tolist()
    return obj


def run(ns) -> dict:
    info = RC.discover_trace(ns.trace_dir)
    if ns.trace_dtype and ns.trace_dtype != info.g_dtype:
        raise ValueError(f"--trace-dtype {ns.trace_dtype} but the trace stores {info.g_dtype}")
    cfgs, scores, ratios, Ts, multi = build_configs(ns)
    bps = info.branch_points if ns.branch_point == "all" else _ints(ns.branch_point)
    report = {"trace_dir": os.path.abspath(ns.trace_dir),
              "config": {k: v for k, v in vars(ns).items() if k not in ("out",)}, "branch_results": {}}
    if ns.self_check:
        report["self_check"] = self_check(ns.trace_dir, ns.self_check[0], ns.self_check[1], ns.device)
    for t0 in bps:
        if t0 not in info.branch_points:
            report["branch_results"][t0] = {"t0": t0, "state_absent": True}
            continue
        W = len(info.window(t0, ns.window))
        horizons = _ints(ns.horizons) if ns.horizons else [W]
        if ns.nodes:
            from . import launch

            frag = launch.run_fused_branch_multinode(ns, t0, cfgs, horizons, scores, ratios)
        else:
            frag = RF.run_fused_branch(ns.trace_dir, t0, cfgs, ns.window, horizons, world=ns.fused_shards,
                                       device=ns.device, dense_cache=ns.dense_cache,
                                       max_configs=ns.fused_max_configs, state_budget_mb=ns.fused_state_budget_mb,
                                       score_names=scores, ratios=ratios, semantics=ns.selection_semantics)
        meta, _ = RC.load_state(info, t0)
        per_ratio = {}
        for r in ratios:
            entry = {"k": RC.k_for(info.numel, r), "scores": {}}
            for c in cfgs:
                if c.ratio_percent != r:
                    continue
                key = c.key(multi)
                rank = frag["front"].get((c.score, r), {})
                entry["scores"][key] = dict({"distortion": frag["results"][c]},
                                            **{k: v for k, v in rank.items() if k != "k"})
            per_ratio[r] = entry
        report["branch_results"][t0] = {
            "t0": t0, "state_absent": False, "window_len": frag["window_len"], "window_steps": frag["window_steps"],
            "cycle_lens": Ts, "horizon_steps": frag["horizon_steps"],
            "meta": {k: meta[k] for k in ("step", "phase", "clip_grad", "lr", "grad_norm") if k in meta},
            "replay": {"dtype": ns.replay_dtype, "trace_dtype": info.g_dtype, "dense_cache_hit": None,
                       "g_residency": bool(ns.fused_g_residency), "dev_reduce": bool(ns.fused_dev_reduce),
                       "den_norm_at_horizon": frag["den_norm_at_horizon"], "profile": frag["profile"]},
            "scores": {s: {"ranked": True} for s in scores}, "per_ratio": per_ratio}
    return sanitize(report)


def print_summary(report) -> None:
    for t0, br in report["branch_results"].items():
        if br.get("state_absent"):
            print(f"branch {t0}: state absent")
            continue
        print(f"branch {t0}: window {br['window_len']} horizons {br['horizon_steps']}")
        for r, entry in br["per_ratio"].items():
            print(f"  ratio {r}% (k={entry['k']})")
            for key, s in sorted(entry["scores"].items()):
                d = ", ".join(f"H{h}={v:.5f}" if v is not None else f"H{h}=nan" for h, v in s["distortion"].items())
                extra = f" ndcg={s['ndcg_at_k']:.4f} recall={s['recall_at_k']:.4f}" if "ndcg_at_k" in s else ""
                print(f"    {key:32s} distortion {d}{extra}")


def main(argv=None) -> int:
    ns = build_parser().parse_args(argv)
    report = run(ns)
    if ns.out:
        tmp = ns.out + ".tmp"
        with open(tmp, "w") as fh:
            json.dump(report, fh, indent=1)
        os.replace(tmp, ns.out)
    print_summary(report)
    return 0


if __name__ == "__main__":
    sys.exit(main())
