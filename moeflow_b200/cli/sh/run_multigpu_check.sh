#!/usr/bin/env bash
# usage: run_multigpu_check.sh NGPUS [extra args of tests/multigpu/fixed_peer_check.py]
set -euo pipefail
cd "$(dirname "$0")/../../.."
source moeflow_b200/cli/sh/config.sh
N="${1:?number of GPUs}"; shift || true
NCCL_NVLS_ENABLE=0 timeout -s KILL "${MOEFLOW_CHECK_TIMEOUT:-600}" $MOEFLOW_TORCHRUN --nnodes=1 --nproc-per-node "$N" \
  --master-addr 127.0.0.1 --master-port "${MOEFLOW_PORT:-29531}" tests/multigpu/fixed_peer_check.py "$@"
