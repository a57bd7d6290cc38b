#!/usr/bin/env bash
# usage (as the torchrun entry point, --no-python): profile_rank.sh <command...>
# Rank 0 runs under Nsight Compute (launch list: one pass, every kernel with its device time); all other ranks
# run the command plainly.  Clocks are left alone (--clock-control none).
set -euo pipefail
if [ "${RANK:-0}" = "0" ]; then
  exec ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file "${MOEFLOW_TRACE_OUT:-launches_rank0.csv}" "$@"
else
  exec "$@"
fi
