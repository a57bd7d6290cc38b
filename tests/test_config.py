"""MoEConfig: defaults, divisibility, HuggingFace config parsing."""

import json

import pytest

from moeflow_b200 import GLM53_FLASH, GLM53_FLASH_I1536, MoEConfig


def test_defaults_describe_glm53_flash():
    c = GLM53_FLASH
    assert (c.hidden_size, c.n_routed_experts, c.n_shared_experts, c.top_k) == (4096, 288, 1, 8)
    assert c.scoring_func == "sigmoid" and c.topk_method == "noaux_tc" and c.norm_topk_prob
    assert c.routed_scaling_factor == 2.5 and c.swiglu_limit == 10.0
    assert GLM53_FLASH_I1536.moe_intermediate_size == 1536


@pytest.mark.parametrize("ep,per", [(1, 288), (2, 144), (4, 72), (8, 36)])
def test_experts_per_rank(ep, per):
    assert GLM53_FLASH.experts_per_rank(ep) == per


def test_uneven_placement_is_rejected():
    with pytest.raises(ValueError):
        GLM53_FLASH.experts_per_rank(5)
    with pytest.raises(ValueError):
        GLM53_FLASH.experts_per_rank(0)


def test_frozen_and_round_trip():
    with pytest.raises(Exception):
        GLM53_FLASH.top_k = 4  # type: ignore[misc]
    assert MoEConfig.from_dict(GLM53_FLASH.to_dict()) == GLM53_FLASH


@pytest.mark.parametrize("nested", [False, True])
def test_from_hf_config(tmp_path, nested):
    text = {
        "hidden_size": 128, "moe_intermediate_size": 64, "n_routed_experts": 16, "n_shared_experts": 1,
        "num_experts_per_tok": 4, "n_group": 2, "topk_group": 1, "norm_topk_prob": False,
        "routed_scaling_factor": 1, "scoring_func": "softmax", "topk_method": "noaux_tc",
    }
    cfg = {"text_config": text, "hidden_size": 999} if nested else text
    p = tmp_path / "config.json"
    p.write_text(json.dumps(cfg))
    c = MoEConfig.from_hf_config(p)
    assert c.hidden_size == 128 and c.top_k == 4 and c.n_group == 2 and not c.norm_topk_prob
    assert isinstance(c.routed_scaling_factor, float) and c.swiglu_limit is None
