"""``python -m sga_b200.replay`` -- offline evaluation of score / ratio / cycle
configurations against a captured trace.

For every requested branch point the fused engine replays the dense arm and
every configuration of the grid ``scores x ratios x cycle lengths x optimizers
x fold x dual-lr`` over the window, and reports the branch-point ranking
quality of each score (NDCG@k, recall@k, missed masses against the realised
dense displacement) and each configuration's distortion at the horizons.

Report JSON (keys and value forms of ``sga/replay.py:2022-2070`` and ``sga/replay_fused.py:1985-2075``; floats
rounded to 8 decimals)::

    {"trace_dir", "config": {"branch_points", "ratios", "horizons", "device", ..., "score_names", "window", "seed"},
     "branch_results": {t0: {"t0", "state_absent", "window_len", "window_steps", "cycle_lens",
                             "horizon_steps": {h: steps replayed}, "meta": {lr, grad_norm, clip_grad, ...},
                             "replay": {"dtype", "trace_dtype", "dense_cache_hit", "per_step": [reconstruction
                                        check of every logged gradient], "den_norm_at_horizon", "label_total",
                                        "label_stats", "profile"},
                             "scores": {name: {numel, sum, mean, min, max, fraction_zero}},
                             "per_ratio": {r: {"k", "scores": {key: {"threshold", "distortion": {h: d},
                                                                      "ndcg_at_k", "recall_at_k", ...}}}}}}}

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
    p.add_argument("--norm-dtype", choices=("fp32", "fp64"), default="fp32")
    p.add_argument("--trace-dtype", choices=("fp32", "bf16"), default=None)
    p.add_argument("--dense-cache", default=None)
    p.add_argument("--replay-mode", choices=("zerofill", "cycle"), default="zerofill",
                   help="zerofill (default): frozen support, the gradient zero-filled outside it on every step of "
                        "the window, re-clipped on its own norm, AdamW. cycle: residual accumulation, boundary "
                        "merge (and fold) and re-selection every --cycle-len steps")
    p.add_argument("--cycle-len", type=int, default=None)
    p.add_argument("--cycle-lens", default=None)
    p.add_argument("--optimizer", default=None, help="comma set of {adamw, adams} (cycle mode; default adamw)")
    p.add_argument("--fold", default=None, help="comma set of {off, on} (cycle mode; default off)")
    p.add_argument("--dual-lr", default=None,
                   help="comma set of boundary inactive-lr scales: floats, or T-relative multiples of each "
                        "configuration's cycle length ('T', 'T/2')")
    p.add_argument("--fused", action="store_true", help="accepted for compatibility; the fused engine is the only one")
    p.add_argument("--fused-shards", type=int, default=None,
                   help="parameter shards, one process (and GPU) each; default: min(8, visible GPUs) on cuda "
                        "(the reference's 8 on an 8-GPU node), 1 on cpu")
    p.add_argument("--selection-semantics", choices=("topk", "balanced-histogram"), default="balanced-histogram",
                   help="rule behind the branch-point and boundary selections: balanced-histogram (default: the "
                        "online engine's stride-8, whole-crossing-bin histogram mode; single-node cycle replay "
                        "only) or topk (exact global top-k with index-ordered ties; zerofill and --nodes need it "
                        "spelled out)")
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


def resolve_dual_lr_token(tok: str, T: int) -> float:
    """One ``--dual-lr`` token against a cycle length: a plain float, ``T`` (the cycle length) or ``T/k``
    (``sga/replay.py:299-331``)."""
    s_ = tok.strip()
    if s_ in ("T", "t"):
        return float(T)
    if s_[:2] in ("T/", "t/"):
        try:
            k = float(s_[2:])
        except ValueError:
            raise ValueError(f"--dual-lr token {tok!r}: the divisor after 'T/' must be a number") from None
        if not (math.isfinite(k) and k > 0.0):
            raise ValueError(f"--dual-lr token {tok!r}: the divisor after 'T/' must be finite > 0")
        return float(T) / k
    try:
        return float(s_)
    except ValueError:
        raise ValueError(f"--dual-lr token {tok!r} is neither a number nor a T-relative multiple ('T', 'T/2', ...)") \
            from None


def parse_dual_lr_set(spec: str, Ts) -> list:
    """Validated token list ordered by the scale at the largest cycle length; tokens must resolve to scales
    that are finite, >= 0 and distinct (also in the report key's %g form) at every cycle length
    (``sga/replay.py:342-378``)."""
    toks = [t for t in str(spec).replace(" ", "").split(",") if t]
    if not toks:
        raise ValueError(f"--dual-lr {spec!r} names no dual-lr value")
    if len(set(toks)) != len(toks):
        raise ValueError(f"--dual-lr {spec!r} carries duplicate tokens")
    at_max = {}
    for tok in toks:
        at_max[tok] = resolve_dual_lr_token(tok, max(Ts))
        if not (math.isfinite(at_max[tok]) and at_max[tok] >= 0.0):
            raise ValueError(f"--dual-lr token {tok!r} resolves to {at_max[tok]!r}; scales must be finite >= 0")
    for T in Ts:
        scales = [resolve_dual_lr_token(tok, T) for tok in toks]
        if len({f"{x:g}" for x in scales}) != len(scales):
            raise ValueError(f"--dual-lr {spec!r}: tokens collide at T={T} (resolved scales {scales})")
    return sorted(toks, key=lambda tok: at_max[tok])


def build_configs(ns):
    from ..plugins.scores import score_names

    scores = [s for s in str(ns.score_names).split(",") if s]
    for s in scores:
        if s not in score_names() and s not in RC.REPLAY_ONLY_SCORES:
            raise ValueError(f"unknown score '{s}' (registered: {score_names()}; replay only: "
                             f"{list(RC.REPLAY_ONLY_SCORES)})")
    ratios = _floats(ns.ratios)
    if ns.cycle_len is not None and ns.cycle_lens:
        raise ValueError("give --cycle-len or --cycle-lens, not both")
    # sga/replay.py:1813-1835: --cycle-lens is a comma set, --cycle-len its single spelling (default 20, echoed
    # into the report even where zerofill does not use it)
    if ns.cycle_lens:
        Ts = sorted(set(_ints(ns.cycle_lens)))
    else:
        if ns.cycle_len is None:
            ns.cycle_len = 20
        Ts = [ns.cycle_len]
    if any(t < 1 for t in Ts):
        raise ValueError(f"cycle lengths must be >= 1 (got {Ts})")
    # sga/replay.py:1840-1882: the per-configuration axes exist in cycle mode only; balanced-histogram is the
    # default everywhere and is refused, not silently replaced, where only exact top-k exists (a dense
    # --self-check selects nothing and needs no override)
    if (ns.optimizer is not None or ns.fold is not None or ns.dual_lr is not None) and ns.replay_mode != "cycle":
        raise ValueError("--optimizer/--fold/--dual-lr are only supported with --replay-mode cycle")
    if ns.replay_mode == "cycle" and ns.self_check is not None:
        raise ValueError("--replay-mode cycle cannot be combined with --self-check")
    if ns.nodes and ns.replay_mode != "cycle":
        raise ValueError("--nodes is only supported with --replay-mode cycle")
    if ns.self_check is None and ns.selection_semantics != "topk" and (ns.replay_mode != "cycle" or ns.nodes):
        raise ValueError("--selection-semantics balanced-histogram requires --replay-mode cycle on a single node "
                         "(zerofill and --nodes require an explicit --selection-semantics topk)")
    ns.report_cycle_lens = list(Ts)
    if ns.replay_mode == "zerofill":
        Ts = [0]  # never a boundary: frozen support, zero-filled gradient on every step
    opts = sorted({o for o in str(ns.optimizer or "adamw").replace(" ", "").split(",") if o})
    for o in opts:
        if o not in ("adamw", "adams"):
            raise ValueError(f"unknown optimizer '{o}'")
    fold_toks = [f for f in str(ns.fold or "off").replace(" ", "").split(",") if f]
    if any(f not in ("off", "on") for f in fold_toks) or len(set(fold_toks)) != len(fold_toks):
        raise ValueError(f"--fold {ns.fold!r}: a comma set of off / on")
    folds = sorted({f == "on" for f in fold_toks})
    ns.optimizer_set, ns.fold_set = opts, folds
    duals = parse_dual_lr_set(ns.dual_lr, Ts) if ns.dual_lr is not None else ["1"]
    ns.dual_lr_set = duals
    multi = {"cycle_len": len(Ts) > 1, "optimizer": len(opts) > 1, "fold": len(folds) > 1, "dual_lr": len(duals) > 1}
    cfgs = [RC.CycleConfig(s, r, T, o, f, resolve_dual_lr_token(d, T)) for o in opts for f in folds for d in duals
            for T in Ts for r in ratios for s in scores]
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


def sanitize(obj, nd=8):
    """JSON-safe copy with floats rounded to ``nd`` decimals (``sga/replay.py:1544-1561``, called with 8)."""
    if isinstance(obj, dict):
        return {str(k): sanitize(v, nd) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [sanitize(v, nd) for v in obj]
    if isinstance(obj, float):
        return None if (math.isnan(obj) or math.isinf(obj)) else round(obj, nd)
    if isinstance(obj, torch.Tensor):
        return sanitize(obj.tolist(), nd)
    return obj


def report_config(ns, bps, scores, ratios, Ts) -> dict:
    """The ``config`` block of the report, keys and value forms of ``sga/replay.py:2022-2070``: the
    per-configuration axes and the selection rule are echoed only when they differ from the defaults."""
    cfg = {"branch_points": list(bps), "ratios": list(ratios), "horizons": _ints(ns.horizons) if ns.horizons else None,
           "device": ns.device, "chunk_mb": ns.chunk_mb, "replay_dtype": ns.replay_dtype,
           "trace_dtype": ns.trace_dtype, "norm_dtype": ns.norm_dtype, "dense_cache": ns.dense_cache,
           "replay_mode": ns.replay_mode, "cycle_len": ns.cycle_len,
           "cycle_lens": list(getattr(ns, "report_cycle_lens", Ts)), "fused": bool(ns.fused),
           "fused_effective": bool(ns.fused) or ns.replay_mode == "cycle", "fused_shards": ns.fused_shards, "fused_max_configs": ns.fused_max_configs,
           "nodes": ns.nodes, "fused_g_residency": bool(ns.fused_g_residency),
           "fused_dev_reduce": bool(ns.fused_dev_reduce), "score_names": list(scores), "window": ns.window,
           "seed": ns.seed}
    if ns.fused_state_budget_mb and ns.fused_state_budget_mb > 0:
        cfg["fused_state_budget_mb"] = ns.fused_state_budget_mb
    if getattr(ns, "optimizer_set", ["adamw"]) != ["adamw"]:
        cfg["optimizer"] = list(ns.optimizer_set)
    if getattr(ns, "fold_set", [False]) != [False]:
        cfg["fold"] = ["on" if f else "off" for f in ns.fold_set]
    if getattr(ns, "dual_lr_set", ["1"]) != ["1"]:
        cfg["dual_lr"] = list(ns.dual_lr_set)
    if ns.selection_semantics != "topk":
        cfg["selection_semantics"] = ns.selection_semantics
    return cfg


def run(ns) -> dict:
    info = RC.discover_trace(ns.trace_dir)
    if ns.trace_dtype and ns.trace_dtype != info.g_dtype:
        raise ValueError(f"--trace-dtype {ns.trace_dtype} but the trace stores {info.g_dtype}")
    cfgs, scores, ratios, Ts, multi = build_configs(ns)
    bps = info.branch_points if ns.branch_point == "all" else _ints(ns.branch_point)
    ns.trace_dtype = ns.trace_dtype or info.g_dtype
    if ns.fused_shards is None:
        ns.fused_shards = min(8, torch.cuda.device_count()) if str(ns.device).startswith("cuda") else 1
        ns.fused_shards = max(1, ns.fused_shards)
    report = {"trace_dir": os.path.abspath(ns.trace_dir), "config": report_config(ns, bps, scores, ratios, Ts),
              "branch_results": {}}
    if ns.self_check:
        report["self_check"] = self_check(ns.trace_dir, ns.self_check[0], ns.self_check[1], ns.device)
    for t0 in bps:
        if t0 not in info.branch_points:
            report["branch_results"][t0] = {"t0": t0, "state_absent": True}
            continue
        W = len(info.window(t0, ns.window))
        horizons = _ints(ns.horizons) if ns.horizons else [W]
        if report["config"]["horizons"] is None:
            report["config"]["horizons"] = list(horizons)
        if ns.nodes:
            from . import launch

            frag = launch.run_fused_branch_multinode(ns, t0, cfgs, horizons, scores, ratios)
        else:
            frag = RF.run_fused_branch(ns.trace_dir, t0, cfgs, ns.window, horizons, world=ns.fused_shards,
                                       device=ns.device, dense_cache=ns.dense_cache,
                                       max_configs=ns.fused_max_configs, state_budget_mb=ns.fused_state_budget_mb,
                                       score_names=scores, ratios=ratios, semantics=ns.selection_semantics)
        meta = frag.get("state_meta") or RC.load_state(info, t0)[0]
        per_ratio = {}
        for r in ratios:
            entry = {"k": RC.k_for(info.numel, r), "scores": {}}
            for c in cfgs:
                if c.ratio_percent != r:
                    continue
                key = c.key(multi)
                rank = frag["front"].get((c.score, r, c.optimizer), {})
                entry["scores"][key] = dict({"threshold": rank.get("threshold"), "distortion": frag["results"][c]},
                                            **{k: v for k, v in rank.items() if k not in ("k", "threshold")})
            per_ratio[r] = entry
        Wl = frag["window_len"]
        lr = meta.get("lr", [])
        # one optimizer keeps the flat views; several nest them under the optimizer's name and key the score
        # statistics "name@optimizer" (sga/replay_fused.py:2025-2038, 2066-2068)
        fopts = frag.get("optimizers") or ["adamw"]
        one = len(fopts) == 1

        def view(d):
            d = d or {}
            return d.get(fopts[0]) if one else {o: d.get(o) for o in fopts}
        report["branch_results"][t0] = {
            "t0": t0, "state_absent": False, "window_len": Wl, "window_steps": frag["window_steps"],
            "cycle_lens": list(ns.report_cycle_lens), "horizon_steps": {str(h): max(1, min(h, Wl)) for h in horizons},
            # the state dump's scalars, with the reference's defaults where a trace carries its
            # hyper-parameters per parameter group only (sga/replay_fused.py:2047-2056)
            "meta": {"lr": [float(x) for x in (lr if isinstance(lr, (list, tuple)) else [lr])],
                     "grad_norm": float(meta.get("grad_norm", float("nan"))),
                     "clip_grad": float(meta.get("clip_grad", 0.0)),
                     "weight_decay": float(meta.get("weight_decay", 0.0)),
                     "adam_beta1": float(meta.get("adam_beta1", 0.9)), "adam_beta2": float(meta.get("adam_beta2", 0.999)),
                     "adam_eps": float(meta.get("adam_eps", 1e-8)),
                     **{k: meta[k] for k in ("step", "phase") if k in meta}},
            "replay": {"dtype": ns.replay_dtype, "trace_dtype": info.g_dtype,
                       "dense_cache_hit": view(frag.get("dense_cache_hit")),
                       "g_residency": bool(ns.fused_g_residency), "dev_reduce": bool(ns.fused_dev_reduce),
                       "per_step": frag.get("per_step", []),
                       "den_norm_at_horizon": view(frag["den_norm_at_horizon"]),
                       "label_total": view(frag.get("label_total")), "label_stats": view(frag.get("label_stats")),
                       "profile": frag["profile"]},
            "scores": {(s if one else f"{s}@{o}"): frag.get("score_stats", {}).get((s, o), {})
                       for s in scores for o in fopts},
            "per_ratio": per_ratio}
        if ns.replay_mode == "zerofill":  # the cycle engine's echoes do not exist in this mode
            br = report["branch_results"][t0]
            del br["cycle_lens"], br["replay"]["g_residency"], br["replay"]["dev_reduce"]
    return sanitize(report)


def print_summary(report) -> None:
    for t0, br in report["branch_results"].items():
        if br.get("state_absent"):
            print(f"branch {t0}: state absent")
            continue
        print(f"branch {t0}: window {br['window_len']} horizons {sorted(int(h) for h in br['horizon_steps'])}")
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
