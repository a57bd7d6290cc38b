"""Real multi-process runs on CPU (gloo): EP data path and failure detection without any GPU."""

import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world: int, *extra: str, timeout: int = 240):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "multiproc" / "cpu_ep_check.py"), *extra]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    rows = [json.loads(line) for line in res.stdout.splitlines() if line.startswith("{")]
    return res, rows


@pytest.mark.parametrize("world", [2, 4])
def test_fixed_and_variable_pipelines_over_gloo(world):
    res, rows = _run(world)
    assert res.returncode == 0 and rows, res.stdout[-2000:] + res.stderr[-2000:]
    assert rows[-1]["ok"] and rows[-1]["world"] == world and rows[-1]["max_err"] < 1e-5


def test_a_rank_that_leaves_is_detected_by_a_collective_timeout():
    res, rows = _run(2, "--drop-rank", "1")
    left = [r for r in rows if r.get("left")]
    noticed = [r for r in rows if r.get("peer_loss_detected")]
    assert left and noticed, res.stdout[-2000:] + res.stderr[-2000:]
    assert noticed[0]["ok"]


def _bootstrap(world: int, *extra: str):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "multiproc" / "peer_bootstrap_check.py"),
           *extra]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=env, cwd=ROOT)
    rows = [json.loads(line) for line in res.stdout.splitlines() if line.startswith("{")]
    assert res.returncode == 0 and rows, res.stdout[-2000:] + res.stderr[-2000:]
    return rows[-1]


def test_peer_bootstrap_accepts_matching_ranks():
    out = _bootstrap(2)
    assert out["raised"] == [False, False]


@pytest.mark.parametrize("flag", ["--bad-size-rank", "--bad-handle-rank"])
def test_peer_bootstrap_mismatch_is_raised_on_every_rank(flag):
    """A rank that asks for a different region size (a different capacity) or sends a malformed IPC handle:
    all ranks raise before any peer memory would be mapped, nobody is left waiting."""
    out = _bootstrap(2, flag, "1")
    assert out["raised"] == [True, True] and "symmetric allocation" in out["error"]
