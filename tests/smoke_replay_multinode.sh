#!/bin/bash
# Cross-node fused replay smoke on CPU: a tiny synthetic trace, a two-node world=2 replay through the
# multi-node launcher (cold dense cache on the first node, bounded preflight, one node-worker per node),
# then the one-shard replay of the same grid, and a comparison inside the pure-reordering band
# (sums to 1e-6 relative, everything else exact).
#
#   bash tests/smoke_replay_multinode.sh <node0> <node1> <workdir>
#
# <workdir> must be visible under the same path on both nodes (a shared file system), as must this
# checkout. With SGA_LAUNCH_EXECUTOR=local the node-workers are local subprocesses and the two node names
# are only labels, so the whole smoke runs on one machine:
#
#   SGA_LAUNCH_EXECUTOR=local bash tests/smoke_replay_multinode.sh nodeA nodeB /tmp/replay_smoke
#
# Counterpart of the reference's tests/smoke_replay_multinode.sh.
set -euo pipefail

NODE0="${1:?first node}"
NODE1="${2:?second node}"
WORK="${3:?work directory shared by both nodes}"
ROOT="$(cd "$(dirname "$0")/.." && pwd)"
cd "$ROOT"
export PYTHONPATH="$ROOT${PYTHONPATH:+:$PYTHONPATH}"
SSH_KEY_OPT=()
if [ -n "${SGA_SSH_KEY:-}" ]; then SSH_KEY_OPT=(--ssh-key "$SGA_SSH_KEY"); fi

ARGS=(--trace-dir "$WORK/trace" --branch-point 0 --window 6 --horizons 6 --ratios 20,30
      --score-names abs_g,update --replay-mode cycle --cycle-len 2 --dense-cache "$WORK/cache"
      --selection-semantics topk --device cpu)

echo "== [1/4] tiny synthetic trace -> $WORK/trace =="
rm -rf "$WORK"
mkdir -p "$WORK"
python - <<PYEOF
from sga_b200.replay.synth import make_synthetic_trace
make_synthetic_trace("$WORK/trace", sizes=(4000, 3000, 1700), steps=8, g_dtype="fp32", seed=3)
print("fixture ok")
PYEOF

echo "== [2/4] world=2 over $NODE0 + $NODE1, cold cache =="
PYTHONUNBUFFERED=1 python -m sga_b200.replay "${ARGS[@]}" --fused-shards 2 --nodes "$NODE0,$NODE1" \
  --launch-log-dir "$WORK/logs" --preflight-timeout 120 "${SSH_KEY_OPT[@]}" --out "$WORK/report_w2.json"

echo "== [3/4] world=1 on this node =="
PYTHONUNBUFFERED=1 python -m sga_b200.replay "${ARGS[@]}" --fused-shards 1 --out "$WORK/report_w1.json"

echo "== [4/4] pure-reordering band: world=2 against world=1 =="
python - <<PYEOF
import json
w1 = json.load(open("$WORK/report_w1.json"))["branch_results"]["0"]
w2 = json.load(open("$WORK/report_w2.json"))["branch_results"]["0"]
assert json.load(open("$WORK/report_w2.json"))["config"]["nodes"] in ("$NODE0,$NODE1", ["$NODE0", "$NODE1"])
worst = 0.0
for r, entry in w1["per_ratio"].items():
    assert entry["k"] == w2["per_ratio"][r]["k"]
    for key, a in entry["scores"].items():
        b = w2["per_ratio"][r]["scores"][key]
        assert a["recall_at_k"] == b["recall_at_k"] and a["threshold"] == b["threshold"], (r, key)
        for h, d in a["distortion"].items():
            rel = abs(d - b["distortion"][h]) / max(abs(d), 1e-12)
            worst = max(worst, rel)
            assert rel <= 1e-6, (r, key, h, d, b["distortion"][h])
        for m in ("ndcg_at_k", "missed_label_mass", "missed_score_mass"):
            assert abs(a[m] - b[m]) <= 1e-6 * max(abs(a[m]), 1e-12), (r, key, m)
print(f"SMOKE PASS: cross-node world=2 matches world=1 within the band (worst relative difference {worst:.2e})")
PYEOF
echo "== smoke done: logs and reports under $WORK =="
