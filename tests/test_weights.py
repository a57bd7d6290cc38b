"""Checkpoint reader (FP8 block scaling) and the trimmed-checkpoint builder on synthetic checkpoints."""

import json

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from moeflow_b200.cli.make_trimmed_checkpoint import trim
from moeflow_b200.weights import CheckpointReader, dequant_block_fp8, quant_block_fp8


def test_dequant_is_the_elementwise_definition_including_edge_blocks():
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(200, 130, generator=g) * 4).to(torch.float8_e4m3fn)
    s = torch.rand(2, 2, generator=g) + 0.5
    out = dequant_block_fp8(w, s)
    for i, j in [(0, 0), (127, 127), (128, 0), (0, 128), (199, 129)]:
        assert out[i, j].item() == (w[i, j].float() * s[i // 128, j // 128]).item()


def test_quant_round_trip_error_is_e4m3_sized():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(256, 384, generator=g) * 0.02
    q, s = quant_block_fp8(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 3)
    back = dequant_block_fp8(q, s)
    assert ((back - w).norm() / w.norm()).item() < 0.04
    assert back.abs().max() <= w.abs().max() * 1.0001


def _write_checkpoint(root, layer=3, hidden=256, inter=128, experts=2, fp8=True):
    p = f"model.language_model.layers.{layer}.mlp"
    t = {}
    for e in range(experts):
        for proj, shape in (("gate_proj", (inter, hidden)), ("up_proj", (inter, hidden)), ("down_proj", (hidden, inter))):
            full = torch.full(shape, float(e + 1) * (2.0 if proj == "up_proj" else 1.0))
            if fp8:
                t[f"{p}.experts.{e}.{proj}.weight"] = full.to(torch.float8_e4m3fn)
                t[f"{p}.experts.{e}.{proj}.weight_scale_inv"] = torch.full((shape[0] // 128, shape[1] // 128), 0.5)
            else:
                t[f"{p}.experts.{e}.{proj}.weight"] = full.bfloat16()
    t[f"{p}.gate.weight"] = torch.ones(experts, hidden, dtype=torch.bfloat16)
    t[f"{p}.gate.e_score_correction_bias"] = torch.zeros(experts)
    save_file(t, root / "m.safetensors")
    (root / "model.safetensors.index.json").write_text(json.dumps({"weight_map": dict.fromkeys(t, "m.safetensors")}))
    (root / "config.json").write_text(json.dumps({"quantization_config": {"weight_block_size": [128, 128]}}))


def test_reader_layouts(tmp_path):
    _write_checkpoint(tmp_path)
    r = CheckpointReader(tmp_path)
    w13, w2 = r.expert_weights(3, range(1, 2))
    assert w13.shape == (1, 256, 256) and w2.shape == (1, 256, 128) and w13.dtype == torch.bfloat16
    assert torch.all(w13[0, :128] == 1.0) and torch.all(w13[0, 128:] == 2.0) and torch.all(w2 == 1.0)  # value * 0.5
    gate, bias = r.router(3)
    assert gate.dtype == torch.float32 and gate.shape == (2, 256) and bias.shape == (2,)
    q13, s13, q2, s2 = r.expert_weights_fp8(3, range(0, 2))
    assert q13.dtype == torch.float8_e4m3fn and q13.shape == (2, 256, 256) and s13.shape == (2, 2, 2)
    assert q2.shape == (2, 256, 128) and s2.shape == (2, 2, 1)
    assert torch.equal(dequant_block_fp8(q13[1], s13[1]).bfloat16(), w13[0])


def test_reader_passes_unquantised_weights_through(tmp_path):
    _write_checkpoint(tmp_path, fp8=False)
    w13, w2 = CheckpointReader(tmp_path).expert_weights(3, range(0, 1))
    assert torch.all(w13[0, 128:] == 2.0) and torch.all(w2 == 1.0)


def test_trimmed_checkpoint(tmp_path):
    src, dst = tmp_path / "src", tmp_path / "dst"
    src.mkdir()
    tensors = {
        "model.language_model.embed_tokens.weight": torch.ones(4, 2),
        "model.language_model.norm.weight": torch.ones(2),
        "lm_head.weight": torch.ones(4, 2),
        "model.visual.patch_embed.weight": torch.ones(2, 2),
    }
    for layer in range(6):
        tensors[f"model.language_model.layers.{layer}.mlp.gate.weight"] = torch.full((2, 2), float(layer))
    save_file({k: v for k, v in tensors.items() if "layers.5" not in k}, src / "a.safetensors")
    save_file({k: v for k, v in tensors.items() if "layers.5" in k}, src / "b.safetensors")
    index = {k: ("b.safetensors" if "layers.5" in k else "a.safetensors") for k in tensors}
    (src / "model.safetensors.index.json").write_text(json.dumps({"weight_map": index}))
    cfg = {"text_config": {"num_hidden_layers": 6, "num_nextn_predict_layers": 1, "layer_types": list("abcdef"),
                           "mlp_layer_types": list("dddsss"), "linear_attn_config": {"kda_layers": [0, 1, 2, 4], "full_attn_layers": [3, 5]}}}
    (src / "config.json").write_text(json.dumps(cfg))
    (src / "tokenizer.json").write_text("{}")
    trim(src, dst, 4, verbose=False)
    out_cfg = json.loads((dst / "config.json").read_text())["text_config"]
    assert out_cfg["num_hidden_layers"] == 4 and out_cfg["num_nextn_predict_layers"] == 0
    assert out_cfg["layer_types"] == list("abcd") and out_cfg["mlp_layer_types"] == list("ddds")
    assert out_cfg["linear_attn_config"] == {"kda_layers": [0, 1, 2], "full_attn_layers": [3]}
    new_index = json.loads((dst / "model.safetensors.index.json").read_text())["weight_map"]
    assert set(new_index) == {k for k in tensors if "layers.4" not in k and "layers.5" not in k}
    assert (dst / "tokenizer.json").is_symlink()
    assert set(new_index.values()) == {"model-00001.safetensors"}
    with safe_open(dst / "model-00001.safetensors", framework="pt") as h:
        assert h.get_tensor("model.language_model.layers.3.mlp.gate.weight")[0, 0] == 3.0
    assert json.loads((dst / "TRIMMED_FROM.json").read_text())["num_layers"] == 4


def test_trim_plan_and_config_rules():
    from moeflow_b200.cli.make_trimmed_checkpoint import keeps, layer_of, plan_shards, trim_config

    assert layer_of("model.language_model.layers.12.mlp.gate.weight") == 12 and layer_of("lm_head.weight") is None
    assert keeps("model.visual.blocks.30.attn.qkv.weight", 2)  # a vision block is not a decoder layer
    weight_map = {"model.language_model.layers.0.a": "s2", "model.language_model.layers.9.a": "s1", "lm_head.weight": "s3",
                  "model.language_model.layers.1.a": "s2"}
    assert plan_shards(weight_map, 2) == [
        ("s2", "model-00001.safetensors", ["model.language_model.layers.0.a", "model.language_model.layers.1.a"]),
        ("s3", "model-00002.safetensors", ["lm_head.weight"]),
    ]
    flat = trim_config({"num_hidden_layers": 3, "layer_types": ["x", "y", "z"]}, 2)  # no nested text_config
    assert flat == {"num_hidden_layers": 2, "num_nextn_predict_layers": 0, "layer_types": ["x", "y"]}
    for bad in (0, 4):
        with pytest.raises(ValueError):
            trim_config({"num_hidden_layers": 3}, bad)
