"""The oracle has to be right by inspection, so it is tested against cases small enough to do by hand and
against a dense restatement (one big matrix product per expert) that shares nothing with its loops."""

import math

import pytest
import torch

from moeflow_b200 import MoEConfig
from moeflow_b200.reference import (
    ep_dispatch_reference,
    expert_forward,
    moe_reference,
    route_reference,
    route_token,
    swiglu_clamp,
)


def sigma(v: float) -> float:
    return 1.0 / (1.0 + math.exp(-v))


# ---- routing ---------------------------------------------------------------------------------------------
def test_a_bias_changes_who_is_picked_but_not_the_weights():
    cfg = MoEConfig(n_routed_experts=5, top_k=2, routed_scaling_factor=3.0)
    logits = torch.tensor([2.0, 0.0, 1.0, -2.0, 0.5])
    assert [e for e, _ in route_token(logits, None, cfg)] == [0, 2]
    lifted = route_token(logits, torch.tensor([0.0, 0.0, 0.0, 0.85, 0.0]), cfg)
    # keys: .881, .5, .731, .119 + .85 = .969, .622 -> expert 3 first, then expert 0
    assert [e for e, _ in lifted] == [3, 0]
    norm = sigma(-2.0) + sigma(2.0)  # = 1: the two scores are complementary
    assert math.isclose(norm, 1.0, rel_tol=1e-15)
    assert math.isclose(lifted[0][1], 3.0 * sigma(-2.0) / norm, rel_tol=1e-12)
    assert math.isclose(lifted[1][1], 3.0 * sigma(2.0) / norm, rel_tol=1e-12)
    assert math.isclose(sum(w for _, w in lifted), 3.0, rel_tol=1e-12)


def test_equal_keys_are_taken_in_id_order():
    cfg = MoEConfig(n_routed_experts=7, top_k=3)
    assert [e for e, _ in route_token(torch.full((7,), -1.5), None, cfg)] == [0, 1, 2]
    logits = torch.tensor([0.0, 4.0, 0.0, 4.0, 0.0, 0.0, 0.0])
    assert [e for e, _ in route_token(logits, None, cfg)] == [1, 3, 0]


def test_groups_are_rated_by_two_best_keys_with_a_bias_and_by_the_best_key_without():
    cfg = MoEConfig(n_routed_experts=6, top_k=2, n_group=3, topk_group=1)
    # group 0: one strong and one hopeless expert; group 1: two good ones; group 2: mediocre
    logits = torch.tensor([4.0, -8.0, 2.0, 2.0, 0.0, 0.0])
    assert 2 * sigma(2.0) > sigma(4.0) + sigma(-8.0) > sigma(2.0)
    assert sorted(e for e, _ in route_token(logits, torch.zeros(6), cfg)) == [2, 3]
    assert sorted(e for e, _ in route_token(logits, None, cfg)) == [0, 1]
    two_groups = MoEConfig(n_routed_experts=6, top_k=3, n_group=3, topk_group=2)
    picks = [e for e, _ in route_token(logits, torch.zeros(6), two_groups)]
    # ratings: group 0 = .982 + .0003, group 1 = 2 * .881, group 2 = 2 * .5: groups 1 and 2 stay eligible and
    # group 0 is closed although it holds the single best expert
    assert picks == [2, 3, 4]


def test_softmax_scores_without_renormalisation():
    cfg = MoEConfig(n_routed_experts=4, top_k=2, scoring_func="softmax", norm_topk_prob=False, routed_scaling_factor=1.0)
    logits = torch.tensor([0.5, 2.5, 1.5, -1.0])
    whole = sum(math.exp(v) for v in logits.tolist())
    picks = route_token(logits, None, cfg)
    assert [e for e, _ in picks] == [1, 2]
    assert math.isclose(picks[0][1], math.exp(2.5) / whole, rel_tol=1e-12)
    assert math.isclose(picks[1][1], math.exp(1.5) / whole, rel_tol=1e-12)
    shifted = route_token(logits + 1000.0, None, cfg)  # softmax is shift invariant, and must not overflow
    assert [e for e, _ in shifted] == [1, 2] and math.isclose(shifted[0][1], picks[0][1], rel_tol=1e-9)


def test_route_reference_is_route_token_per_row():
    cfg = MoEConfig(n_routed_experts=8, top_k=2)
    logits = torch.randn(5, 8, generator=torch.Generator().manual_seed(2))
    assert route_reference(logits, None, cfg) == [route_token(logits[t], None, cfg) for t in range(5)]
    with pytest.raises(ValueError):
        route_token(logits[0], None, MoEConfig(n_routed_experts=8, top_k=2, scoring_func="relu"))


# ---- experts ------------------------------------------------------------------------------------------------
def test_the_clamp_caps_the_gate_from_above_only():
    gate = torch.tensor([-30.0, 30.0, 1.0])
    up = torch.tensor([-30.0, 30.0, 0.5])
    got = swiglu_clamp(gate, up, 7.0)
    want = torch.tensor([-30.0 * sigma(-30.0) * -7.0, 7.0 * sigma(7.0) * 7.0, 1.0 * sigma(1.0) * 0.5])
    torch.testing.assert_close(got, want)
    free = swiglu_clamp(gate, up, None)
    torch.testing.assert_close(free[1], torch.tensor(30.0 * sigma(30.0) * 30.0))


def test_one_expert_by_hand():
    x = torch.tensor([2.0, -1.0])
    w13 = torch.tensor([[1.0, 1.0], [0.5, 0.0], [0.0, 3.0], [1.0, 0.0]])  # gate rows, then up rows
    w2 = torch.tensor([[1.0, -1.0], [2.0, 0.0]])
    gate, up = torch.tensor([1.0, 1.0]), torch.tensor([-3.0, 2.0])
    act = torch.tensor([sigma(1.0) * -3.0, sigma(1.0) * 2.0])
    torch.testing.assert_close(swiglu_clamp(gate, up, None), act)
    torch.testing.assert_close(expert_forward(x, w13, w2, None), torch.tensor([act[0] - act[1], 2 * act[0]]))


def test_layer_equals_a_dense_restatement():
    cfg = MoEConfig(hidden_size=6, moe_intermediate_size=4, n_routed_experts=5, top_k=2, swiglu_limit=1.5)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(7, 6, generator=g)
    logits = torch.randn(7, 5, generator=g)
    w13, w2 = torch.randn(5, 8, 6, generator=g), torch.randn(5, 6, 4, generator=g)
    got = moe_reference(x, logits, None, w13, w2, cfg)
    # dense: every expert on every token, then a [T, E] weight matrix that is zero off the route
    hidden = torch.einsum("efh,th->tef", w13, x)
    act = swiglu_clamp(hidden[..., :4], hidden[..., 4:], 1.5)
    everyone = torch.einsum("ehi,tei->teh", w2, act)
    mix = torch.zeros(7, 5)
    for t, picks in enumerate(route_reference(logits, None, cfg)):
        for e, w in picks:
            mix[t, e] = w
    torch.testing.assert_close(got, torch.einsum("te,teh->th", mix, everyone), rtol=1e-5, atol=1e-5)


def test_given_routes_replace_the_routing_and_output_keeps_the_input_dtype():
    cfg = MoEConfig(hidden_size=4, moe_intermediate_size=2, n_routed_experts=3, top_k=1, swiglu_limit=None)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 4, generator=g).to(torch.bfloat16)
    w13, w2 = torch.randn(3, 4, 4, generator=g), torch.randn(3, 4, 2, generator=g)
    out = moe_reference(x, torch.zeros(2, 3), None, w13, w2, cfg, routes=[[(2, 0.25)], [(0, -1.0)]])
    assert out.dtype == torch.bfloat16
    torch.testing.assert_close(out[0].float(), 0.25 * expert_forward(x[0], w13[2], w2[2], None), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(out[1].float(), -expert_forward(x[1], w13[0], w2[0], None), rtol=1e-2, atol=1e-2)
    assert moe_reference(x[:0], torch.zeros(0, 3), None, w13, w2, cfg).shape == (0, 4)


# ---- dispatch contract ------------------------------------------------------------------------------------------
def test_one_copy_per_token_and_destination():
    rank0 = [[(4, 0.1), (1, 0.2)], [(0, 0.3), (1, 0.4)], [(5, 0.5), (4, 0.6)]]
    rank1 = [[(2, 0.7), (3, 0.8)]]
    got = ep_dispatch_reference([rank0, rank1, []], experts_per_rank=2)
    assert got[0] == [(0, 0, [(1, 0.2)]), (0, 1, [(0, 0.3), (1, 0.4)])]
    assert got[1] == [(1, 0, [(0, 0.7), (1, 0.8)])]
    assert got[2] == [(0, 0, [(0, 0.1)]), (0, 2, [(1, 0.5), (0, 0.6)])]  # slot order kept, ids local to rank 2
