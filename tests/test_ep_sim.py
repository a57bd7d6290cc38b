"""Expert parallelism without a cluster: every rank's stages in one process, exchanges simulated."""

import pytest
import torch

from conftest import SMALL
from moeflow_b200.ep_moe import EPMoELayer, shard_experts, simulate_ep
from moeflow_b200.reference import moe_reference
from moeflow_b200.testing import DISTRIBUTIONS, make_bias, make_hidden, make_logits, make_weights
from moeflow_b200.tolerances import bitwise_equal, gemm_tolerance, normwise_rel_err


def _run(world, dist, tokens, combine_dtype=torch.bfloat16, seed=0):
    cfg = SMALL
    w13, w2 = make_weights(cfg, seed)
    bias = make_bias(cfg, seed + 1)
    xs = [make_hidden(tokens[r], cfg, seed + 10 + r) for r in range(world)]
    lgs = [make_logits(tokens[r], cfg, seed + 20 + r, dist=dist) for r in range(world)]
    layers = [EPMoELayer(cfg, r, world, *shard_experts(w13, w2, r, world), combine_dtype=combine_dtype) for r in range(world)]
    return cfg, w13, w2, bias, xs, lgs, simulate_ep(layers, xs, lgs, bias)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("dist", DISTRIBUTIONS)
def test_matches_oracle(world, dist):
    tokens = [5, 0, 9, 2, 1, 7, 3, 4][:world]
    cfg, w13, w2, bias, xs, lgs, outs = _run(world, dist, tokens)
    for r in range(world):
        assert outs[r].shape == xs[r].shape
        if tokens[r]:
            ref = moe_reference(xs[r], lgs[r], bias, w13, w2, cfg)
            assert normwise_rel_err(outs[r], ref) < gemm_tolerance()


def test_deterministic():
    a = _run(4, "zipf", [6, 6, 6, 6])[-1]
    b = _run(4, "zipf", [6, 6, 6, 6])[-1]
    assert all(bitwise_equal(x, y) for x, y in zip(a, b))


def test_all_ranks_empty():
    outs = _run(2, "uniform", [0, 0])[-1]
    assert all(o.shape == (0, SMALL.hidden_size) for o in outs)


def test_result_does_not_depend_on_world_size_with_exact_transport():
    """With fp32 partial rows and one token per call the EP degree changes only the summation tree."""
    tokens = [4] * 8
    base = None
    for world in (1, 2, 4, 8):
        cfg, w13, w2, bias, xs, lgs, outs = _run(world, "uniform", tokens, combine_dtype=torch.float32, seed=3)
        ref = moe_reference(xs[0], lgs[0], bias, w13, w2, cfg)
        err = normwise_rel_err(outs[0], ref)
        assert err < gemm_tolerance()
        base = err if base is None else base
