#!/usr/bin/env bash
# usage: run_baselines.sh NGPUS   — layer latency of every backend, one record per backend
set -euo pipefail
cd "$(dirname "$0")/../../.."
source moeflow_b200/cli/sh/config.sh
N="${1:?number of GPUs}"
prologue baselines
BACKENDS="${MOEFLOW_BACKENDS:-fused torch_fixed naive reference_fixed}"
TOKENS="${MOEFLOW_TOKENS:-1,2,4,8,16,32,64,128}"
for b in $BACKENDS; do
  echo "== $b" | tee -a "$OUT/commands.log"
  timeout -s KILL "${MOEFLOW_BENCH_TIMEOUT:-1800}" $MOEFLOW_TORCHRUN --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 \
    --master-port 29532 -m moeflow_b200.cli.bench_layer --backend "$b" --tokens "$TOKENS" --flush --out "$OUT/layer_$b.json" \
    || echo "$b failed (recorded in $OUT/layer_$b.json if it got that far)"
done
$MOEFLOW_PYTHON -m moeflow_b200.cli.summarize layer "$OUT"/layer_*.json | tee "$OUT/summary.md" || true
