#!/usr/bin/env bash
# CPU tests, then (with a GPU) the single-GPU and multi-GPU tests; junit XML next to the logs.
set -euo pipefail
cd "$(dirname "$0")/../../.."
source moeflow_b200/cli/sh/config.sh
prologue tests
$MOEFLOW_PYTHON -m pytest tests -q -m "not gpu" --junitxml "$OUT/cpu.xml"
if $MOEFLOW_PYTHON -c "import torch,sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  timeout -s KILL 1800 $MOEFLOW_PYTHON -m pytest tests -q -m gpu --junitxml "$OUT/gpu.xml"
fi
