"""Stack probes as tests: one GPU (device + native library) and several GPUs (NCCL all-to-all incl. graph capture
and orderly teardown; peer-memory ping incl. the bounded wait that runs out).  Counterpart of the reference's
``tests/test_probes.py``."""

import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _last_json(text: str) -> dict:
    lines = [ln for ln in text.splitlines() if ln.startswith("{")]
    assert lines, text[-2000:]
    return json.loads(lines[-1])


def _probe(what: str, nproc: int = 0, timeout: int = 300) -> dict:
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    if nproc:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port()), "-m", "moeflow_b200.cli.probes", what]
    else:
        cmd = [sys.executable, "-m", "moeflow_b200.cli.probes", what]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert res.returncode == 0, f"rc={res.returncode}\n{res.stdout[-2000:]}\n{res.stderr[-3000:]}"
    return _last_json(res.stdout)


def _ranks() -> int:
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    return n


def test_native_probe_runs_a_kernel_of_the_library():
    info = _probe("native")
    assert info["sm_100_or_newer"] and info["sms"] > 0 and info["library"].endswith(".so")
    assert info["rmsnorm_max_err"] < 0.05


@pytest.mark.multigpu
def test_nccl_all_to_all_even_uneven_graph_and_teardown():
    info = _probe("a2a", _ranks())
    assert info["ok"] and info["teardown"] == "clean", info


@pytest.mark.multigpu
def test_peer_memory_ping_and_bounded_wait():
    """Every rank stores into every peer and sees all flags; then nobody stores and the wait must run out with
    the time-out status (code 8) while the context stays usable (the probe goes on to gather and tear down)."""
    info = _probe("peer", _ranks())
    assert info["ok"], info
    assert all(r["timeout_code"] == 8 for r in info["ranks"])
