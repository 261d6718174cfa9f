"""Replay benchmark on a synthetic trace: ``python -m sga_b200.replay.bench
--elems 50331648 --steps 12 --shards 1 --device cuda``.

Writes a synthetic trace (the generator of ``synth.py``: heavy-tailed bf16
gradient dumps plus an AdamW snapshot), replays the 18-config grid of the
headline replay workload (scores |g + residual| and |m| x ratios {0.1, 1, 5} % x cycle lengths
{1, 4, 16}) in one fused pass over ``--shards`` GPUs with exact distributed
top-k, and prints one JSON line: wall seconds of the replay, milliseconds per
trace step, and replayed element-configs per second.
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
    ns = ap.parse_args(argv)
    from . import core as RC
    from . import fused as RF
    from .synth import make_synthetic_trace

    tdir = ns.trace_dir or tempfile.mkdtemp(prefix="sga_replay_bench_")
    third = ns.elems // 3
    t_gen = time.perf_counter()
    make_synthetic_trace(tdir, sizes=(third, third, ns.elems - 2 * third), steps=ns.steps, g_dtype="bf16", seed=0)
    t_gen = time.perf_counter() - t_gen
    # the replay scores the accumulated gradient q = g + residual: "abs_g" is |g + residual| here
    scores, ratios, Ts = ["abs_g", "abs_m"], [0.1, 1.0, 5.0], [1, 4, 16]
    cfgs = [RC.CycleConfig(score=s, ratio_percent=r, cycle_len=T) for s in scores for r in ratios for T in Ts]
    t0 = time.perf_counter()
    frag = RF.run_fused_branch(tdir, 0, cfgs, ns.steps, [ns.steps], world=ns.shards, device=ns.device,
                               max_configs=len(cfgs), score_names=scores, ratios=ratios)
    wall = time.perf_counter() - t0
    rec = {"bench": "fused replay", "elems": ns.elems, "steps": ns.steps, "configs": len(cfgs), "shards": ns.shards,
           "device": ns.device, "trace_gen_s": round(t_gen, 2), "replay_wall_s": round(wall, 3),
           "ms_per_step": round(1e3 * wall / ns.steps, 2),
           "elem_configs_per_s": round(ns.elems * len(cfgs) * ns.steps / wall / 1e9, 3),
           "unit": "1e9 element-configs/s (wall clock, includes trace reads and process start)",
           "profile": frag.get("profile")}
    print(json.dumps(rec, default=str), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
