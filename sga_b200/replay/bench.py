"""Replay benchmark on a synthetic trace: ``python -m sga_b200.replay.bench
--elems 50331648 --steps 12 --shards 1 --device cuda``.

Writes a synthetic trace (the generator of ``synth.py``: heavy-tailed bf16
gradient dumps plus an AdamW snapshot), replays the 18-config grid of the
headline replay workload (scores |g| and |g + residual| x ratios {0.1, 1, 5} % x cycle lengths
{1, 4, 16}) in one fused pass over ``--shards`` GPUs with exact distributed
top-k, and prints one JSON line: wall seconds of the replay, the engine's own
seconds (what the shards spend after their process group is up: set-up, dense
arm, front block, stream), milliseconds per trace step, and replayed
element-configs per second.

``--generate`` replaces the files by the on-device generator of
``synth.SyntheticSource`` (same distribution, produced block by block from the
seed wherever a pass needs a step), which is how the full-size workload
(``--elems 1240000000 --steps 64``: 159 GB of dumps) runs without writing them.
``--state-budget-mb`` bounds the per-shard state of a configuration group.

``--impl reference`` runs the unmodified reference replay (``python -m
sga.replay`` from ``baseline/_ref``, its public CLI and stock code path) on the
same trace and grid in a child process and prints the same line with
``"impl": "reference"``. The reference's Triton kernels refuse every Triton
release but the one they were written against, so the child sees no Triton and
takes the reference's own torch-eager path (its documented fallback,
``sga/replay_kernels.py:48-58``). ``--impl both`` runs the two arms on one
trace and also reports the largest difference between their distortions.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--elems", type=int, default=48 * 1024 * 1024)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--shards", type=int, default=1)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--trace-dir", default=None)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference", "both"))
    ap.add_argument("--generate", action="store_true", help="generate the trace on the replay device, no files")
    ap.add_argument("--state-budget-mb", type=float, default=0.0)
    ap.add_argument("--scores", default=None,
                    help="comma list (default abs_g_step,abs_g: |g| and |g + residual|; with the reference arm "
                         "abs_g,abs_m, since abs_g_step exists only in this framework's replay)")
    ns = ap.parse_args(argv)
    if ns.scores is None:
        ns.scores = "abs_g_step,abs_g" if ns.impl == "ours" else "abs_g,abs_m"
    from . import core as RC
    from . import fused as RF
    from .synth import SyntheticSource, make_synthetic_trace

    t_gen = time.perf_counter()
    if ns.generate:
        if ns.impl != "ours":
            ap.error("--generate has no files for the reference arm to read")
        tdir = SyntheticSource(ns.elems, steps=ns.steps, seed=0)
    else:
        tdir = ns.trace_dir or tempfile.mkdtemp(prefix="sga_replay_bench_")
        third = ns.elems // 3
        make_synthetic_trace(tdir, sizes=(third, third, ns.elems - 2 * third), steps=ns.steps, g_dtype="bf16", seed=0)
    t_gen = time.perf_counter() - t_gen
    # the replay scores the accumulated gradient q = g + residual: "abs_g" is |g + residual| here, and
    # "abs_g_step" the step's own |g|
    scores, ratios, Ts = [x for x in ns.scores.split(",") if x], [0.1, 1.0, 5.0], [1, 4, 16]
    cfgs = [RC.CycleConfig(score=s, ratio_percent=r, cycle_len=T) for s in scores for r in ratios for T in Ts]
    ref = None
    if ns.impl in ("reference", "both"):
        ref = _reference_arm(ns, tdir, scores, ratios, Ts)
        print(json.dumps({k: v for k, v in ref.items() if k != "distortions"}, default=str), flush=True)
        if ns.impl == "reference":
            return 0
    t0 = time.perf_counter()
    frag = RF.run_fused_branch(tdir, 0, cfgs, ns.steps, [ns.steps], world=ns.shards, device=ns.device,
                               max_configs=len(cfgs), state_budget_mb=ns.state_budget_mb, score_names=scores,
                               ratios=ratios, semantics="topk")
    wall = time.perf_counter() - t0
    prof = frag.get("profile") or [{}]
    engine_s = sum((prof[0].get("phases_s") or {}).values())
    stream_s = (prof[0].get("phases_s") or {}).get("stream")
    rec = {"bench": "fused replay", "elems": ns.elems, "steps": ns.steps, "configs": len(cfgs), "shards": ns.shards,
           "device": ns.device, "scores": scores, "source": "generated on the device" if ns.generate else "trace files",
           "trace_gen_s": round(t_gen, 2), "replay_wall_s": round(wall, 3), "engine_s": round(engine_s, 3),
           "stream_s": stream_s, "host_syncs_per_step": round(sum(p.get("host_syncs", 0) for p in prof) /
                                                             max(ns.steps * len(prof), 1), 2),
           "ms_per_step": round(1e3 * wall / ns.steps, 2),
           "elem_configs_per_s": round(ns.elems * len(cfgs) * ns.steps / wall / 1e9, 3),
           "unit": "1e9 element-configs/s (wall clock, includes trace reads and process start)",
           "profile": frag.get("profile")}
    if ref is not None and "distortions" in ref and "unavailable" not in ref:
        worst = 0.0
        for c in cfgs:
            mine = frag["results"][c][ns.steps]
            theirs = ref["distortions"].get((c.score, c.ratio_percent, c.cycle_len))
            if theirs is not None and c.cycle_len > 1:
                worst = max(worst, abs(mine - theirs))
        rec["max_abs_distortion_diff_vs_reference"] = worst
        rec["speedup_vs_reference_wall"] = round(ref["replay_wall_s"] / wall, 2)
    print(json.dumps(rec, default=str), flush=True)
    return 0


def _reference_arm(ns, tdir, scores, ratios, Ts) -> dict:
    """The reference CLI on the same trace and grid (exact top-k semantics on both arms), timed by wall clock."""
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ref_root = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "sga")):
        return {"impl": "reference", "unavailable": "baseline/_ref/sga is not present on this machine"}
    hide = tempfile.mkdtemp(prefix="sga_no_triton_")
    os.makedirs(os.path.join(hide, "triton"))
    with open(os.path.join(hide, "triton", "__init__.py"), "w") as fh:
        fh.write('raise ImportError("hidden: the reference replay kernels pin another Triton release")\n')
    out = os.path.join(tempfile.mkdtemp(prefix="sga_ref_out_"), "report.json")
    cache = tempfile.mkdtemp(prefix="sga_ref_cache_")
    dev = "cuda" if ns.device.startswith("cuda") else "cpu"  # the reference maps shards to local GPU indices itself
    cmd = [sys.executable, "-m", "sga.replay", "--trace-dir", tdir, "--branch-point", "0", "--ratios",
           ",".join(str(r) for r in ratios), "--replay-mode", "cycle", "--cycle-lens", ",".join(str(t) for t in Ts),
           "--score-names", ",".join(scores), "--window", str(ns.steps), "--device", dev, "--dense-cache", cache,
           "--trace-dtype", "bf16", "--selection-semantics", "topk", "--fused-shards", str(ns.shards),
           "--fused-max-configs", str(len(scores) * len(ratios) * len(Ts)), "--out", out]
    env = dict(os.environ, PYTHONPATH=hide + os.pathsep + ref_root)
    t0 = time.perf_counter()
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, cwd=tempfile.gettempdir())
    wall = time.perf_counter() - t0
    if res.returncode != 0 or not os.path.exists(out):
        why = (res.stderr or res.stdout).strip().splitlines()[-1][:300] if (res.stderr or res.stdout) else "failed"
        return {"bench": "fused replay", "impl": "reference", "unavailable": why}
    rec = {"bench": "fused replay", "impl": "reference", "elems": ns.elems, "steps": ns.steps,
           "configs": len(scores) * len(ratios) * len(Ts), "shards": ns.shards, "device": dev,
           "replay_wall_s": round(wall, 3), "ms_per_step": round(1e3 * wall / ns.steps, 2),
           "elem_configs_per_s": round(ns.elems * len(scores) * len(ratios) * len(Ts) * ns.steps / wall / 1e9, 3),
           "kernels": "torch eager (the reference's fallback when Triton is not importable)",
           "unit": "wall clock of the child process: interpreter start, imports, dense cache, replay"}
    per_ratio = json.load(open(out))["branch_results"]["0"]["per_ratio"]
    dist = {}
    for r, entry in per_ratio.items():
        for key, sc in entry["scores"].items():
            name, _, t = key.partition("@T")
            dist[(name, float(r), int(t) if t else Ts[0])] = float(sc["distortion"][str(ns.steps)])
    rec["distortions"] = dist
    return rec


if __name__ == "__main__":
    sys.exit(main())
