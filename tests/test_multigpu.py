"""Multi-GPU checks, launched as child processes with torch.distributed.run on 127.0.0.1."""

import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(n: int, script: str, *extra: str, timeout: int = 600) -> dict:
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "multigpu" / script), *extra]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert res.returncode == 0 and lines, f"rc={res.returncode}\n{res.stdout[-3000:]}\n{res.stderr[-3000:]}"
    return json.loads(lines[-1])


def test_fused_layer_over_peer_memory_with_the_multi_cta_metadata_pass():
    """Capacity 1024 x top-8: more than 8192 received slot words per rank, so the metadata pass runs as its two
    chained multi-CTA launches behind real peers' dispatch flags."""
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    out = _launch(n, "fixed_peer_check.py", "--dist", "uniform", "--iters", "4", "--replays", "20", "--capacity", "1024",
                  "--top-k", "8", "--experts", "64")
    assert out["ok"], out


@pytest.mark.parametrize("dist_name", ["uniform", "hotspot"])
def test_fused_layer_over_peer_memory(dist_name):
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    out = _launch(n, "fixed_peer_check.py", "--dist", dist_name, "--iters", "12", "--replays", "120")
    assert out["ok"], out


def test_graph_gate_interleaved_capacities_shared_buffers_one_gpu():
    """The 1000-replay gate (capacities 1, 8, 64, 128 side by side, two weight sets on one buffer set, bitwise
    against an eager layer) on a single GPU: stale-buffer contamination between graphs needs no second rank."""
    out = _launch(1, "fixed_graph_gate.py", "--replays", "1000", timeout=900)
    assert out["ok"] and out["replays"] == 1000, out


def test_graph_gate_interleaved_capacities_shared_buffers_over_peers():
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    out = _launch(n, "fixed_graph_gate.py", "--replays", "1000", timeout=900)
    assert out["ok"] and out["replays"] == 1000, out


def _launch_module(n: int, module: str, *extra: str, timeout: int = 900) -> str:
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), "-m", module, *extra]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert res.returncode == 0, f"rc={res.returncode}\n{res.stdout[-3000:]}\n{res.stderr[-3000:]}"
    return res.stdout


@pytest.mark.parametrize("arm_b", ["fused", "fixed_vllm_experts"])
def test_native_allgather_reducescatter_arm_against_the_fixed_layer(arm_b, tmp_path):
    """The paired native-vs-fixed driver end to end at a small shape: both arms pass the oracle gate on every rank,
    each arm's graph replays equal its eager runs byte for byte, and a complete record is written."""
    pytest.importorskip("vllm")
    n = min(torch.cuda.device_count(), 2)
    out = tmp_path / "ab.json"
    text = _launch_module(n, "moeflow_b200.cli.ab_native_fixed", "--small", "--tokens", "1,8", "--reps", "3", "--inner", "5",
                          "--check-graph-replays", "20", "--b", arm_b, "--out", str(out))
    assert "T=8:" in text
    record = json.loads(out.read_text())
    points = record["results"]["points"]
    assert [p["tokens"] for p in points] == [1, 8]
    for p in points:
        assert p["gate"]["a"]["passed"] and p["gate"]["b"]["passed"] and all(p["replays_ok"].values())
