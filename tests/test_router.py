"""The PyTorch router (twin of the ``router_topk`` kernel): agreement with the loop oracle at the full
288-expert shape, and properties that must hold whatever the logits are."""

import pytest
import torch

from moeflow_b200 import GLM53_FLASH, MoEConfig
from moeflow_b200.reference import route_reference
from moeflow_b200.router import expert_scores, route
from moeflow_b200.testing import DISTRIBUTIONS, make_bias, make_logits

GROUPED = MoEConfig(n_routed_experts=32, top_k=4, n_group=4, topk_group=2, scoring_func="softmax")
SHAPES = {
    "glm": GLM53_FLASH,
    "grouped_softmax": GROUPED,
    "no_renorm": MoEConfig(n_routed_experts=24, top_k=3, norm_topk_prob=False, routed_scaling_factor=2.5),
}


def _agrees_with_oracle(logits, bias, cfg, saturated=False):
    """``saturated``: the fp32 sigmoid of the hot experts is exactly 1.0, so among them the fp32 router orders
    by id while the fp64 oracle still sees differences; then only the set of picks is comparable."""
    weights, ids = route(logits, bias, cfg)
    assert (weights.dtype, ids.dtype) == (torch.float32, torch.int32)
    assert weights.shape == ids.shape == (logits.shape[0], cfg.top_k)
    for t, picks in enumerate(route_reference(logits, bias, cfg)):
        if saturated:
            assert sorted(ids[t].tolist()) == sorted(expert for expert, _ in picks), f"token {t}"
            continue
        assert ids[t].tolist() == [expert for expert, _ in picks], f"token {t}"
        want = torch.tensor([w for _, w in picks], dtype=torch.float64)
        torch.testing.assert_close(weights[t].to(torch.float64), want, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("profile", DISTRIBUTIONS)
@pytest.mark.parametrize("biased", [True, False])
def test_oracle_agreement_at_the_served_shape(profile, biased):
    cfg = GLM53_FLASH
    _agrees_with_oracle(make_logits(10, cfg, 5, dist=profile), make_bias(cfg, 6) if biased else None, cfg,
                        saturated=profile == "hotspot")


@pytest.mark.parametrize("shape", ["grouped_softmax", "no_renorm"])
@pytest.mark.parametrize("biased", [True, False])
def test_oracle_agreement_with_groups_softmax_and_without_renormalisation(shape, biased):
    cfg = SHAPES[shape]
    _agrees_with_oracle(make_logits(9, cfg, 1), make_bias(cfg, 2) if biased else None, cfg)


@pytest.mark.parametrize("shape", list(SHAPES))
def test_invariants(shape):
    cfg = SHAPES[shape]
    logits, bias = make_logits(64, cfg, 9), make_bias(cfg, 10)
    weights, ids = route(logits, bias, cfg)
    # K distinct experts per token, slots ordered by descending selection key
    assert all(len(set(row)) == cfg.top_k for row in ids.tolist())
    key = expert_scores(logits, cfg) + bias
    picked = key.gather(1, ids.to(torch.int64))
    assert bool((picked[:, :-1] >= picked[:, 1:]).all())
    # weights are the unbiased scores of the picks, renormalised and scaled
    raw = expert_scores(logits, cfg).gather(1, ids.to(torch.int64))
    if cfg.norm_topk_prob:
        torch.testing.assert_close(weights.sum(dim=1), torch.full((64,), float(cfg.routed_scaling_factor)), rtol=1e-5, atol=0)
        raw = raw / raw.sum(dim=1, keepdim=True)
    torch.testing.assert_close(weights, raw * cfg.routed_scaling_factor, rtol=1e-5, atol=1e-8)
    # with groups, every pick comes from one of topk_group groups
    if cfg.n_group > 1:
        group_of = ids // (cfg.n_routed_experts // cfg.n_group)
        assert all(len(set(row)) <= cfg.topk_group for row in group_of.tolist())


def test_equal_scores_go_to_the_lowest_ids():
    cfg = MoEConfig(n_routed_experts=16, top_k=4)
    _, ids = route(torch.full((3, 16), 0.25), None, cfg)
    assert ids.tolist() == [[0, 1, 2, 3]] * 3
    partly = torch.zeros(1, 16)
    partly[0, [5, 9]] = 1.0  # two clear winners, then a tie among all the rest
    assert route(partly, None, cfg)[1].tolist() == [[5, 9, 0, 1]]
    _agrees_with_oracle(partly, None, cfg)


def test_selection_uses_the_bias_but_weights_do_not():
    cfg = MoEConfig(n_routed_experts=8, top_k=2, norm_topk_prob=False, routed_scaling_factor=1.0)
    logits = torch.zeros(1, 8)
    bias = torch.zeros(8)
    bias[6], bias[3] = 0.3, 0.2
    weights, ids = route(logits, bias, cfg)
    assert ids.tolist() == [[6, 3]]
    assert weights.tolist() == [[0.5, 0.5]]  # sigmoid(0), bias not included


def test_hotspot_profile_keeps_every_token_on_the_hot_experts():
    cfg = GLM53_FLASH
    _, ids = route(make_logits(40, cfg, 3, dist="hotspot"), make_bias(cfg, 4), cfg)
    assert torch.equal(ids.sort(dim=1).values, torch.arange(cfg.top_k, dtype=torch.int32).expand(40, -1))


def test_empty_batch_and_unknown_scoring():
    cfg = GLM53_FLASH
    weights, ids = route(torch.empty(0, cfg.n_routed_experts), None, cfg)
    assert weights.shape == ids.shape == (0, cfg.top_k)
    with pytest.raises(ValueError):
        expert_scores(torch.zeros(1, 4), MoEConfig(n_routed_experts=4, top_k=1, scoring_func="tanh"))
