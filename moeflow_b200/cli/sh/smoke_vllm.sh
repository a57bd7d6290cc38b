#!/usr/bin/env bash
# usage: smoke_vllm.sh MODEL DP   — native engine vs MoEFlowRunner on a (trimmed) checkpoint: the plugin must
# intercept every MoE call, the route sets must match, and greedy outputs must be identical.
set -euo pipefail
cd "$(dirname "$0")/../../.."
source moeflow_b200/cli/sh/config.sh
MODEL="${1:-$MOEFLOW_TRIMMED_MODEL_PATH}"; DP="${2:-2}"
prologue smoke
serve() {  # serve NAME [ENV=VALUE ...]
  local name="$1"; shift
  env "$@" $MOEFLOW_VLLM serve "$MODEL" --served-model-name smoke --port 8000 --data-parallel-size "$DP" \
    --enable-expert-parallel --enforce-eager --max-model-len 4096 > "$OUT/server_$name.log" 2>&1 &
  SERVER=$!
  for _ in $(seq "${MOEFLOW_SMOKE_TIMEOUT:-900}"); do
    curl -sf http://127.0.0.1:8000/health > /dev/null && return 0
    kill -0 "$SERVER" 2>/dev/null || { echo "server $name died"; return 1; }
    sleep 1
  done
  return 1
}
serve native && $MOEFLOW_PYTHON -m moeflow_b200.cli.smoke_client run --port 8000 --out "$OUT/native.json"; kill "$SERVER"; wait "$SERVER" || true
serve moeflow MOEFLOW_RUNNER=1 MOEFLOW_MODE="${MOEFLOW_MODE:-route_check}" MOEFLOW_SMOKE_DIR="$OUT/runner" \
  && $MOEFLOW_PYTHON -m moeflow_b200.cli.smoke_client run --port 8000 --out "$OUT/moeflow.json"; kill "$SERVER"; wait "$SERVER" || true
$MOEFLOW_PYTHON -m moeflow_b200.cli.smoke_client compare "$OUT/native.json" "$OUT/moeflow.json"
$MOEFLOW_PYTHON - "$OUT/runner" <<'PY'
import json, sys, pathlib
rows = [json.loads(l) for p in pathlib.Path(sys.argv[1]).glob("runner_pid*.jsonl") for l in p.read_text().splitlines()]
hit = [r for r in rows if r.get("intercepted")]
miss = [r for r in rows if r.get("intercepted") is False]
match = [r["token_expert_set_match"] for r in hit if "token_expert_set_match" in r]
print(json.dumps({"intercepted": len(hit), "not_intercepted": len(miss), "min_route_set_match": min(match) if match else None}))
sys.exit(0 if hit and not miss and all(m == 1.0 for m in match) else 1)
PY
