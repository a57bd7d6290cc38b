"""The loop-level oracle against closed-form cases."""

import math

import torch

from moeflow_b200 import MoEConfig
from moeflow_b200.reference import ep_dispatch_reference, expert_forward, moe_reference, route_token, swiglu_clamp


def _sig(v):
    return 1.0 / (1.0 + math.exp(-v))


def test_bias_moves_the_selection_not_the_weight():
    cfg = MoEConfig(n_routed_experts=4, top_k=2, routed_scaling_factor=2.5)
    logits = torch.tensor([0.0, 1.0, -1.0, 2.0])
    bias = torch.tensor([0.0, 0.0, 0.9, 0.0])
    picked = route_token(logits, bias, cfg)
    # biased scores: .5, .731, .269 + .9, .881 -> experts 2 then 3
    assert [e for e, _ in picked] == [2, 3]
    total = _sig(-1.0) + _sig(2.0)
    assert math.isclose(picked[0][1], 2.5 * _sig(-1.0) / total, rel_tol=1e-12)
    assert math.isclose(picked[1][1], 2.5 * _sig(2.0) / total, rel_tol=1e-12)


def test_equal_scores_go_to_the_lower_id():
    cfg = MoEConfig(n_routed_experts=6, top_k=3)
    assert [e for e, _ in route_token(torch.zeros(6), None, cfg)] == [0, 1, 2]


def test_group_limited_routing_uses_top2_sum_with_bias_and_max_without():
    cfg = MoEConfig(n_routed_experts=8, top_k=2, n_group=4, topk_group=1)
    logits = torch.tensor([3.0, -9.0, 2.5, 2.5, 0.0, 0.0, 0.0, 0.0])
    with_bias = route_token(logits, torch.zeros(8), cfg)
    assert sorted(e for e, _ in with_bias) == [2, 3]  # 2*s(2.5) beats s(3)+s(-9)
    no_bias = route_token(logits, None, cfg)
    assert sorted(e for e, _ in no_bias) == [0, 1]  # best single score wins the group


def test_softmax_scoring_and_no_renorm():
    cfg = MoEConfig(n_routed_experts=3, top_k=2, scoring_func="softmax", norm_topk_prob=False, routed_scaling_factor=1.0)
    logits = torch.tensor([1.0, 3.0, 2.0])
    z = sum(math.exp(v) for v in (1.0, 3.0, 2.0))
    picked = route_token(logits, None, cfg)
    assert [e for e, _ in picked] == [1, 2]
    assert math.isclose(picked[0][1], math.exp(3.0) / z, rel_tol=1e-12)


def test_clamp_is_one_sided_for_the_gate():
    out = swiglu_clamp(torch.tensor([-20.0, 20.0]), torch.tensor([-20.0, 20.0]), 10.0)
    expect = torch.tensor([-20.0 * _sig(-20.0) * -10.0, 10.0 * _sig(10.0) * 10.0])
    assert torch.allclose(out, expect)


def test_expert_forward_closed_form():
    x = torch.tensor([1.0, 2.0, -1.0])
    w13 = torch.tensor([[1.0, 0, 0], [0, 1.0, 0], [0, 0, 1.0], [1.0, 1.0, 1.0]])
    w2 = torch.tensor([[1.0, 0], [0, 1.0], [1.0, 1.0]])
    gate, up = torch.tensor([1.0, 2.0]), torch.tensor([-1.0, 2.0])
    act = gate * torch.sigmoid(gate) * up
    assert torch.allclose(expert_forward(x, w13, w2, None), w2 @ act)


def test_routes_override():
    cfg = MoEConfig(hidden_size=4, moe_intermediate_size=2, n_routed_experts=2, top_k=1, swiglu_limit=None)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 4, generator=g)
    w13, w2 = torch.randn(2, 4, 4, generator=g), torch.randn(2, 4, 2, generator=g)
    out = moe_reference(x, torch.zeros(2, 2), None, w13, w2, cfg, routes=[[(1, 0.5)], [(0, 2.0)]])
    assert torch.allclose(out[0], 0.5 * expert_forward(x[0], w13[1], w2[1], None))
    assert torch.allclose(out[1], 2.0 * expert_forward(x[1], w13[0], w2[0], None))


def test_dispatch_reference_sends_one_copy_per_rank():
    routes = [[[(0, 1.0), (1, 2.0)], [(3, 1.0), (0, 0.5)]], [[(2, 1.0), (3, 1.0)]]]
    recv = ep_dispatch_reference(routes, experts_per_rank=2)
    assert recv[0] == [(0, 0, [(0, 1.0), (1, 2.0)]), (0, 1, [(0, 0.5)])]
    assert recv[1] == [(0, 1, [(1, 1.0)]), (1, 0, [(0, 1.0), (1, 1.0)])]
