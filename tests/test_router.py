"""Vectorised router against the oracle at the full 288-expert shape."""

import pytest
import torch

from moeflow_b200 import GLM53_FLASH, MoEConfig
from moeflow_b200.reference import route_reference
from moeflow_b200.router import route
from moeflow_b200.testing import DISTRIBUTIONS, make_bias, make_logits


def _check(logits, bias, cfg):
    w, ids = route(logits, bias, cfg)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32
    for t, r in enumerate(route_reference(logits, bias, cfg)):
        assert ids[t].tolist() == [e for e, _ in r]
        torch.testing.assert_close(w[t].double(), torch.tensor([v for _, v in r], dtype=torch.float64), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dist", DISTRIBUTIONS)
def test_full_shape(dist):
    _check(make_logits(12, GLM53_FLASH, 5, dist=dist), make_bias(GLM53_FLASH, 6), GLM53_FLASH)


def test_groups_softmax_and_no_bias():
    cfg = MoEConfig(n_routed_experts=32, top_k=4, n_group=4, topk_group=2, scoring_func="softmax")
    lg = make_logits(9, cfg, 1)
    _check(lg, make_bias(cfg, 2), cfg)
    _check(lg, None, cfg)


def test_ties_go_to_lower_ids():
    cfg = MoEConfig(n_routed_experts=16, top_k=4)
    _, ids = route(torch.zeros(3, 16), None, cfg)
    assert ids.tolist() == [[0, 1, 2, 3]] * 3


def test_hotspot_selects_the_hot_experts():
    lg = make_logits(20, GLM53_FLASH, 3, dist="hotspot")
    _, ids = route(lg, make_bias(GLM53_FLASH, 4), GLM53_FLASH)
    assert ids.max() < GLM53_FLASH.top_k
