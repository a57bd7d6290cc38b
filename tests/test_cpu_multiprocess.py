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
