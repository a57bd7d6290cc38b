"""Shared expert, MoE block and the decode model on one GPU at small shapes."""

import pytest
import torch

from moeflow_b200 import MoEConfig
from moeflow_b200.experts import swiglu_clamp
from moeflow_b200.tolerances import normwise_rel_err

pytestmark = pytest.mark.gpu

CFG = MoEConfig(hidden_size=512, moe_intermediate_size=256, n_routed_experts=16, n_shared_experts=1, top_k=4)


@pytest.mark.parametrize("capacity,tokens", [(8, 5), (128, 128)])
def test_shared_expert_matches_fp32(capacity, tokens):
    from moeflow_b200.models.glm_moe import SharedExpert

    g = torch.Generator().manual_seed(0)
    w13 = (torch.randn(512, 512, generator=g) * 2 / 512**0.5).bfloat16().cuda()
    w2 = (torch.randn(512, 256, generator=g) / 16).bfloat16().cuda()
    x = torch.randn(tokens, 512, generator=g).bfloat16().cuda()
    shared = SharedExpert(w13, w2, capacity, 10.0)
    out = shared(x).clone()
    torch.cuda.synchronize()
    assert int(shared.status.item()) == 0
    ref = swiglu_clamp(x.float() @ w13.float().t(), 10.0) @ w2.float().t()
    assert normwise_rel_err(out, ref) < 4 * 2.0**-8


def test_decode_model_steps_and_matches_eager():
    from moeflow_b200.models.glm_moe import AttentionConfig, DecodeModel

    model = DecodeModel(CFG, 0, 1, batch=4, n_layers=3, device="cuda", acfg=AttentionConfig(n_heads=8, n_kv_heads=2, head_dim=64, max_seq=64))
    model.prefill_standin(16)
    model.x.copy_(torch.randn(4, CFG.hidden_size, generator=torch.Generator().manual_seed(1)).bfloat16())
    eager = model.step().clone()
    assert int(model.pos) == 17 and torch.isfinite(eager.float()).all()
    # replay the same step from a graph: same position and cache contents give the same numbers
    model.prefill_standin(16)
    model.capture()
    model.prefill_standin(16)
    replay = model.step().clone()
    torch.cuda.synchronize()
    assert model.routed.check_status()["code"] == 0
    assert normwise_rel_err(replay, eager.float()) < 1e-2
    for _ in range(5):
        out = model.step()
    assert int(model.pos) == 22 and torch.isfinite(out.float()).all()
    model.close()


@pytest.mark.parametrize("experts,hidden,capacity,tokens", [(288, 512, 8, 5), (16, 512, 128, 128), (130, 1024, 64, 64)])
def test_router_logits_on_the_grouped_kernel_match_fp32(experts, hidden, capacity, tokens):
    """fp32 logits from the tcgen05 down-projection kernel (bf16 operands, fp32 accumulation, fp32 store, expert
    count not a multiple of 128) against an fp32 matmul of the same bf16 values."""
    from moeflow_b200.models.glm_moe import RouterLogits

    g = torch.Generator().manual_seed(3)
    gate = (torch.randn(experts, hidden, generator=g) / hidden**0.5).cuda()
    h = torch.randn(tokens, hidden, generator=g).bfloat16().cuda()
    router = RouterLogits(gate, capacity)
    guard = router.logits.clone()
    out = router(h).clone()
    torch.cuda.synchronize()
    assert int(router.status.item()) == 0
    assert out.dtype == torch.float32 and tuple(out.shape) == (tokens, experts)
    ref = h.float() @ gate.bfloat16().float().t()
    assert (out - ref).abs().max() <= 1e-3 * ref.abs().max() + 1e-4
    assert torch.equal(router.logits[tokens:], guard[tokens:])  # rows past the batch are not touched


def test_decode_model_with_fp8_experts_steps():
    from moeflow_b200.models.glm_moe import AttentionConfig, DecodeModel

    acfg = AttentionConfig(n_heads=8, n_kv_heads=2, head_dim=64, max_seq=64)
    bf16 = DecodeModel(CFG, 0, 1, batch=4, n_layers=2, device="cuda", acfg=acfg, seed=5)
    fp8 = DecodeModel(CFG, 0, 1, batch=4, n_layers=2, device="cuda", acfg=acfg, seed=5, fp8=True)
    x = torch.randn(4, CFG.hidden_size, generator=torch.Generator().manual_seed(2)).bfloat16()
    outs = []
    for model in (bf16, fp8):
        model.prefill_standin(16)
        model.x.copy_(x)
        model.capture()
        model.prefill_standin(16)
        outs.append(model.step().clone())
        torch.cuda.synchronize()
        assert model.routed.check_status()["code"] == 0
        model.close()
    # same random weights, e4m3 experts and activations: each MoE block is a few percent off and a token near a
    # routing tie may change experts in the second layer, so the streams agree only roughly
    assert torch.isfinite(outs[1].float()).all()
    assert normwise_rel_err(outs[1], outs[0].float()) < 0.35
