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


def test_peer_ping_bounded_wait_on_one_gpu():
    """Two simulated ranks on one GPU, their kernels launched one after the other (never concurrently): rank 0
    pings first and its wait for rank 1's word runs out with the time-out status; rank 1 then finds both words;
    a second ping of rank 0 succeeds, i.e. the context survived the time-out."""
    from moeflow_b200.ops._lib import decode_status
    from moeflow_b200.parallel.peer import PeerGroup, ping

    regions = PeerGroup.local(2, 4096)
    status = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(2)]
    ping(regions[0], 0, 1, status[0], wait_ns=20_000_000)
    ping(regions[1], 0, 1, status[1], wait_ns=20_000_000)
    torch.cuda.synchronize()
    first, second = decode_status(int(status[0].item())), decode_status(int(status[1].item()))
    assert first["code"] == 8 and first["who"] == 1, first
    assert second["code"] == 0, second
    status[0].zero_()
    ping(regions[0], 0, 1, status[0], wait_ns=20_000_000)
    torch.cuda.synchronize()
    assert decode_status(int(status[0].item()))["code"] == 0


def test_a_missing_peer_is_reported_by_the_layer_status_word_and_nothing_hangs():
    """Rank 0 of a simulated pair runs a whole forward alone: rank 1 never dispatches, so the metadata kernel's
    bounded wait for its flag runs out (50 ms), the layer records who was missing and carries on to the end.
    A fresh pair of layers then runs normally on the same context."""
    from conftest import SMALL_GPU
    from moeflow_b200.ep_moe import shard_experts
    from moeflow_b200.fixed import FixedEPLayer, simulate_fixed
    from moeflow_b200.parallel.peer import PeerGroup
    from moeflow_b200.testing import make_bias, make_hidden, make_logits, make_weights

    cfg, cap = SMALL_GPU, 8
    w13, w2 = make_weights(cfg, 0, device="cuda")
    bias = make_bias(cfg, 1, device="cuda")

    def pair():
        regions = PeerGroup.local(2, FixedEPLayer.peer_bytes(cfg, 2, cap))
        return [FixedEPLayer(cfg, r, 2, *shard_experts(w13, w2, r, 2), capacity=cap, backend="cuda",
                             peer_region=regions[r], wait_ns=50_000_000) for r in range(2)]

    xs = [make_hidden(cap, cfg, 5 + r, device="cuda") for r in range(2)]
    lgs = [make_logits(cap, cfg, 50 + r, device="cuda") for r in range(2)]
    lonely = pair()[0]
    hit = lonely.stage_pack(xs[0], lgs[0], bias)
    lonely.stage_experts()
    out = lonely.stage_combine(hit, xs[0].dtype)
    torch.cuda.synchronize()
    st = lonely.check_status()
    assert st["code"] == 1 and st["who"] == 1, st  # dispatch flag of source rank 1 never arrived
    assert out.shape == (cap, cfg.hidden_size)
    fresh = pair()
    outs = simulate_fixed(fresh, xs, lgs, bias)
    torch.cuda.synchronize()
    assert all(ly.check_status()["code"] == 0 for ly in fresh)
    assert all(torch.isfinite(o.float()).all() for o in outs)
