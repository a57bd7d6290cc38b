#!/usr/bin/env bash
# Build the native library and run the CPU test suite.  No network access is needed.
set -euo pipefail
cd "$(dirname "$0")/../../.."
source moeflow_b200/cli/sh/config.sh
$MOEFLOW_PYTHON -m moeflow_b200.build
$MOEFLOW_PYTHON -m pytest tests -q -m "not gpu"
