#!/usr/bin/env bash
# usage: e2e_bench.sh MODEL DP OUTDIR [modes] [workloads] [extra server args...]
# One server per mode (native_agrs | moeflow_fixed | native_default); per mode: health poll, greedy gate
# against the native reference, optional raw-logits gate, then the serving workloads, each validated.
set -euo pipefail
cd "$(dirname "$0")/../../.."
source moeflow_b200/cli/sh/config.sh
MODEL="${1:?model}"; DP="${2:?dp}"; OUTDIR="${3:?outdir}"; MODES="${4:-native_agrs moeflow_fixed}"; WORKLOADS="${5:-W1 W1c64}"; shift 5 || true
mkdir -p "$OUTDIR"
declare -A WL=( [W1]="1024 1024 4 16" [W1c64]="1024 1024 64 128" [W2]="1024 1024 128 256" [W3]="1024 8192 4 16" [W4]="1024 8192 64 128" [W5]="8192 1024 4 16" [W6]="8192 1024 64 128" )
for mode in $MODES; do
  if nvidia-smi --query-compute-apps=pid --format=csv,noheader | grep -q .; then echo "GPUs busy; refusing to start $mode"; exit 1; fi
  case "$mode" in
    native_agrs)    ENVS=(VLLM_ALL2ALL_BACKEND=allgather_reducescatter) ;;
    native_default) ENVS=() ;;
    moeflow_fixed)  ENVS=(MOEFLOW_RUNNER=1 MOEFLOW_MODE=fixed MOEFLOW_COMBINE_MODE="${MOEFLOW_COMBINE_MODE:-fp32}" MOEFLOW_SMOKE_DIR="$OUTDIR/$mode/runner") ;;
    *) echo "unknown mode $mode"; exit 1 ;;
  esac
  mkdir -p "$OUTDIR/$mode"
  env "${ENVS[@]}" $MOEFLOW_VLLM serve "$MODEL" --served-model-name smoke --port 8000 --data-parallel-size "$DP" --enable-expert-parallel \
    --max-model-len 32768 --kv-cache-dtype fp8 "$@" > "$OUTDIR/$mode/server.log" 2>&1 &
  SERVER=$!
  ready=0
  for _ in $(seq "${MOEFLOW_SERVER_TIMEOUT:-1800}"); do
    curl -sf http://127.0.0.1:8000/health > /dev/null && { ready=1; break; }
    kill -0 "$SERVER" 2>/dev/null || break
    sleep 1
  done
  [ "$ready" = 1 ] || { echo "$mode: server not ready"; kill "$SERVER" 2>/dev/null || true; exit 1; }
  $MOEFLOW_PYTHON -m moeflow_b200.cli.smoke_client run --port 8000 --out "$OUTDIR/$mode/greedy.json" --max-tokens "${MOEFLOW_GREEDY_TOKENS:-32}"
  REF="${MOEFLOW_REFERENCE_JSON:-$OUTDIR/native_agrs/greedy.json}"
  if [ "$mode" != native_agrs ] && [ -f "$REF" ]; then
    $MOEFLOW_PYTHON -m moeflow_b200.cli.smoke_client compare "$REF" "$OUTDIR/$mode/greedy.json" ${MOEFLOW_EXACT_GREEDY:+--exact-logprobs}
  fi
  if [ -n "${MOEFLOW_LOGITS_VOCAB:-}" ]; then
    $MOEFLOW_PYTHON -m moeflow_b200.cli.logits_client run --port 8000 --vocab "$MOEFLOW_LOGITS_VOCAB" --steps "${MOEFLOW_LOGITS_STEPS:-8}" --out "$OUTDIR/$mode/logits.npz"
  fi
  for w in $WORKLOADS; do
    read -r ISL OSL CONC NPROMPTS <<< "${WL[$w]}"
    $MOEFLOW_VLLM bench serve --model smoke --port 8000 --dataset-name random --random-input-len "$ISL" --random-output-len "$OSL" --ignore-eos \
      --max-concurrency "$CONC" --num-prompts "$NPROMPTS" --save-result --save-detailed --result-filename "$OUTDIR/$mode/$w.json" > "$OUTDIR/$mode/$w.log" 2>&1
    $MOEFLOW_PYTHON -m moeflow_b200.cli.validate_serving_result "$OUTDIR/$mode/$w.json" --requests "$NPROMPTS" --input-len "$ISL" --output-len "$OSL" --concurrency "$CONC"
  done
  kill "$SERVER"; wait "$SERVER" || true
done
