#!/bin/bash
# Three-step walkthrough on one GPU (or CPU with DEVICE=cpu):
#   1. shadow run of a toy llama that captures a trace
#   2. fused replay of a grid of configurations against that trace
#   3. sparse run with the configuration that distorted least
set -euo pipefail
cd "$(dirname "$0")/../.."
DEVICE=${DEVICE:-cuda}
OUT=${OUT:-outputs/example}
mkdir -p "$OUT"

echo "== step 1: shadow trace =="
python -m sga_b200.train_gpt --model llama_tiny --seq-length 512 --micro-batch-size 4 --global-batch-size 8 \
  --train-iters 32 --device "$DEVICE" --sga-enabled true --sga-shadow true --sga-score abs_g \
  --sga-selection-method histogram --sga-selection-histogram-mode balanced --sga-selection-ratio-percent 10 \
  --sga-cycle-period 4 --sga-backend torch_pipelined_index --sga-trace-dir "$OUT/trace" \
  --sga-trace-branch-points 8 --sga-trace-window 16

echo "== step 2: fused replay (4 scores x 2 ratios x 3 cycle lengths x fold on/off = 48 cells) =="
python -m sga_b200.replay --trace-dir "$OUT/trace" --branch-point all --ratios 5,10 --replay-mode cycle --cycle-lens 2,4,8 \
  --dense-cache "$OUT/dense_cache" \
  --score-names abs_g,abs_m,coi,update --fold off,on --window 16 --device "$DEVICE" --fused-max-configs 24 \
  --out "$OUT/replay.json"
python experiments/example/select_best.py "$OUT/replay.json" | tee "$OUT/best.txt"

echo "== step 3: sparse run with the selected score =="
SCORE=$(grep -o 'sga.sga_score=[a-z_]*' "$OUT/best.txt" | cut -d= -f2)
SGA_ALLOW_FROZEN_SELECTION=1 python -m sga_b200.train_gpt --model llama_tiny --seq-length 512 --micro-batch-size 4 \
  --global-batch-size 8 --train-iters 32 --device "$DEVICE" --sga-enabled true --sga-score "$SCORE" \
  --sga-selection-method histogram --sga-selection-histogram-mode balanced --sga-selection-ratio-percent 10 \
  --sga-cycle-period 4 --sga-cycle-start-iter 4 --sga-backend torch_pipelined_index
