"""Pick the replay configuration with the smallest distortion at the last horizon.

    python experiments/example/select_best.py outputs/example/replay.json [--ratio 10]

Prints the winning arm key and the ``sga:`` overrides to paste into the sparse
run's yaml. Counterpart of ``experiments/example/select_best.py:56-97``.
"""
import argparse
import json
import re
import sys


def best_arm(report: dict, ratio=None):
    best = None
    for t0, br in report["branch_results"].items():
        if br.get("state_absent"):
            continue
        h = str(max(int(x) for x in br["horizon_steps"]))  # {horizon: steps replayed} (a list in older reports)
        for r, entry in br["per_ratio"].items():
            if ratio is not None and float(r) != float(ratio):
                continue
            for key, s in entry["scores"].items():
                d = s["distortion"].get(h)
                if d is None:
                    continue
                if best is None or d < best[0]:
                    best = (d, key, float(r), t0)
    return best


def overrides_for(key: str, ratio: float) -> dict:
    out = {"sga_score": key.split("@")[0], "sga_selection_ratio_percent": ratio}
    m = re.search(r"@T(\d+)", key)
    if m:
        out["sga_cycle_period"] = int(m.group(1))
    if "@adams" in key:
        out["sga_optimizer"] = "adams"
    if "@fold" in key:
        out["sga_optimizer_residual_mean"] = True
    m = re.search(r"@dl([0-9.eE+-]+)", key)
    if m:
        out["sga_optimizer_full_sync_inactive_lr_scale"] = float(m.group(1))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("report")
    ap.add_argument("--ratio", type=float, default=None)
    ns = ap.parse_args(argv)
    best = best_arm(json.load(open(ns.report)), ns.ratio)
    if best is None:
        print("no replayed configuration found", file=sys.stderr)
        return 1
    d, key, ratio, t0 = best
    print(f"best arm: {key} at ratio {ratio}% (branch {t0}), distortion {d:.6f}")
    for k, v in overrides_for(key, ratio).items():
        print(f"  sga.{k}={v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
