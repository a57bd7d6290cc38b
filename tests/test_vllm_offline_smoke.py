"""Offline serving smoke: the comparison logic on CPU, and the two-arm run through the installed vLLM on a GPU."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from moeflow_b200.cli import vllm_offline_smoke as smoke

ROOT = Path(__file__).resolve().parent.parent


def _req(tokens, tops):
    return {"tokens": tokens, "steps": [{"token": t, "top": top} for t, top in zip(tokens, tops)]}


def test_compare_accepts_small_logprob_noise_and_near_tie_flips():
    native = {"requests": [_req([5, 7, 9], [[(5, -1.0), (6, -2.0)], [(7, -1.00), (8, -1.01)], [(9, -1.0), (3, -3.0)]])]}
    ours = {"requests": [_req([5, 8, 2], [[(5, -1.01), (6, -2.0)], [(8, -1.00), (7, -1.02)], [(2, -1.0), (3, -3.0)]])]}
    res = smoke.compare(native, ours, margin=0.1, logprob_tol=0.05)
    # step 2 is a near tie (margin 0.01): the flip is allowed and ends the comparison of that request
    assert res["passed"] and res["steps_compared"] == 2 and res["decisive_steps"] == 1
    assert abs(res["max_abs_logprob_diff"] - 0.02) < 1e-9


def test_compare_rejects_a_decisive_disagreement_and_large_logprob_error():
    native = {"requests": [_req([5], [[(5, -1.0), (6, -2.0)]])]}
    flipped = {"requests": [_req([6], [[(6, -1.0), (5, -2.0)]])]}
    assert not smoke.compare(native, flipped, 0.1, 5.0)["passed"]
    drift = {"requests": [_req([5], [[(5, -1.2), (6, -2.0)]])]}
    assert not smoke.compare(native, drift, 0.1, 0.05)["passed"]
    assert not smoke.compare({"requests": []}, {"requests": []}, 0.1, 0.05)["passed"]  # nothing compared


def test_model_dir_prompts_and_seeded_init_are_deterministic(tmp_path):
    cfg = json.loads((smoke.write_model_dir(tmp_path / "m", {"num_hidden_layers": 2}) / "config.json").read_text())
    assert cfg["architectures"] == ["Glm4MoeForCausalLM"] and cfg["num_hidden_layers"] == 2
    assert cfg["hidden_size"] % 128 == 0 and cfg["moe_intermediate_size"] % 128 == 0
    p = smoke.prompts(3, 10, 4096)
    assert p == smoke.prompts(3, 10, 4096) and all(2 <= t < 4096 for row in p for t in row) and p[0] != p[1]

    def make():
        m = torch.nn.Sequential(torch.nn.Linear(64, 32, bias=False), torch.nn.LayerNorm(32))
        smoke.seeded_init(m)
        return m

    a, b = make(), make()
    assert torch.equal(a[0].weight, b[0].weight) and torch.equal(a[1].weight, torch.ones(32))
    assert 0.08 < a[0].weight.std().item() < 0.17  # 1/sqrt(64) = 0.125


@pytest.mark.gpu
@pytest.mark.slow
def test_two_arm_serving_smoke_through_the_installed_engine(tmp_path):
    """Decode steps of a tiny GLM-4-MoE model run through MoEFlowRunner + the tcgen05 experts and agree with
    the engine's own path.  An engine that does not come up in time is a skip, not a failure of this framework."""
    pytest.importorskip("vllm")
    outs = {}
    for arm in ("moeflow", "native"):
        outs[arm] = tmp_path / f"{arm}.json"
        cmd = [sys.executable, "-m", "moeflow_b200.cli.vllm_offline_smoke", "--arm", arm, "--out", str(outs[arm]),
               "--log-dir", str(tmp_path / "log")]
        try:
            res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
        except subprocess.TimeoutExpired:
            pytest.skip(f"{arm} arm: the engine did not finish within 300 s")
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    ours = json.loads(outs["moeflow"].read_text())
    assert ours["runner_log"]["fixed_intercepted"] > 0 and ours["runner_log"]["experts"] == ["native-bf16"]
    verdict = smoke.compare(json.loads(outs["native"].read_text()), ours, 0.1, 0.05)
    assert verdict["passed"], verdict
