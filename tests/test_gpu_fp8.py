"""Block-scaled FP8 path: the 1x128 quantiser and the two tcgen05 e4m3 GEMMs against their PyTorch definition."""

import pytest
import torch

from moeflow_b200.experts import swiglu_clamp
from moeflow_b200.tolerances import normwise_rel_err
from moeflow_b200.weights import dequant_block_fp8, quant_block_fp8

pytestmark = pytest.mark.gpu


def _ok(status):
    from moeflow_b200.ops._lib import decode_status

    st = decode_status(int(status.item()))
    assert st["code"] == 0, st


@pytest.mark.parametrize("rows,hidden", [(1, 128), (7, 4096), (33, 1536)])
def test_quantiser_matches_definition(rows, hidden):
    from moeflow_b200.ops.fp8 import dequant_rows, quant_rows_1x128, quant_rows_reference

    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, hidden, generator=g) * 3).bfloat16().cuda()
    x[0, :128] = 0  # an all-zero group must not divide by zero
    q, s = quant_rows_1x128(x)
    q_ref, s_ref = quant_rows_reference(x)
    torch.cuda.synchronize()
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    # 1/scale is computed once per group on the device: allow a one-code difference at rounding ties
    same = (q.view(torch.uint8) == q_ref.view(torch.uint8)).float().mean().item()
    assert same > 0.999, same
    assert normwise_rel_err(dequant_rows(q, s), x.float()) < 0.04


def test_quantiser_gather_valid_flag_and_row_bound():
    from moeflow_b200.ops.fp8 import quant_rows_1x128, quant_rows_reference

    g = torch.Generator().manual_seed(0)
    store = torch.zeros(6, 256 + 8, dtype=torch.bfloat16, device="cuda")  # rows with a tail: [256 lanes | flag | pad]
    store[:, :256] = torch.randn(6, 256, generator=g).bfloat16().cuda()
    flags = store[:, 256:258].view(torch.int32)
    flags[:, 0] = torch.tensor([1, 0, 1, 1, 0, 1], dtype=torch.int32, device="cuda")
    q = torch.full((6, 256), 7, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    s = torch.full((6, 2), -1.0, device="cuda")
    quant_rows_1x128(store, rows=6, out_q=q, out_s=s, valid_off=512, hidden=256)
    torch.cuda.synchronize()
    q_ref, s_ref = quant_rows_reference(store[:, :256].contiguous())
    for r, live in enumerate([1, 0, 1, 1, 0, 1]):
        if live:
            torch.testing.assert_close(s[r], s_ref[r], rtol=1e-6, atol=0)
        else:
            assert (s[r] == -1).all() and (q[r].view(torch.uint8) == 7).all()  # untouched
    idx = torch.tensor([5, 0, 3], dtype=torch.int32, device="cuda")
    bound = torch.tensor(2, dtype=torch.int32, device="cuda")
    q2, s2 = quant_rows_1x128(store, row_index=idx, hidden=256, n_rows_dev=bound)
    torch.cuda.synchronize()
    torch.testing.assert_close(s2[:2], s_ref[[5, 0]], rtol=1e-6, atol=0)
    assert (s2[2] == 0).all()  # beyond the device-side row count


def _fp8_problem(counts, hidden, inter, seed):
    g = torch.Generator().manual_seed(seed)
    n = sum(counts)
    w13 = torch.randn(len(counts), 2 * inter, hidden, generator=g) * (2.0 / hidden**0.5)
    w2 = torch.randn(len(counts), hidden, inter, generator=g) / inter**0.5
    q13, s13, q2, s2 = [], [], [], []
    for e in range(len(counts)):
        a, b = quant_block_fp8(w13[e])
        c, d = quant_block_fp8(w2[e])
        q13.append(a.view(torch.uint8)), s13.append(b), q2.append(c.view(torch.uint8)), s2.append(d)
    f8 = lambda ts: torch.stack(ts).view(torch.float8_e4m3fn).cuda()  # noqa: E731
    x = torch.randn(n + 3, hidden, generator=g).bfloat16().cuda()
    idx = torch.randint(0, n + 3, (n,), generator=g).int().cuda()
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    scale = (torch.rand(n, generator=g) + 0.5).cuda()
    return f8(q13), torch.stack(s13).cuda(), f8(q2), torch.stack(s2).cuda(), x, idx, offsets, scale


@pytest.mark.parametrize("counts,hidden,inter,block_m", [([1], 256, 128, 64), ([3, 0, 17, 5], 512, 256, 64),
                                                          ([70, 2, 33], 1024, 384, 64), ([9, 30], 512, 256, 32),
                                                          ([128], 256, 128, 128), ([300, 5, 129], 512, 256, 128),
                                                          ([100, 20, 64], 1024, 384, 128)])
@pytest.mark.parametrize("split", [0, 1, 2])
def test_fp8_gemms_match_dequantised_definition(counts, hidden, inter, block_m, split):
    """K cuts 1 and 2, and 0 = stream-K; token tiles of 32, 64 and 128 rows (128: two promotion warp groups)."""
    from moeflow_b200.ops.fp8 import dequant_rows, down_proj_fp8, gate_up_swiglu_fp8, quant_rows_1x128
    from moeflow_b200.ops.grouped_gemm import plan_from_offsets

    if split and (inter // 128) % split:
        pytest.skip("split does not divide the K blocks of the down GEMM")
    q13, s13, q2, s2, x, idx, offsets, scale = _fp8_problem(counts, hidden, inter, seed=hidden + len(counts))
    n = offsets[-1]
    tp = plan_from_offsets(offsets, block_m, x.device)
    status = torch.zeros(1, dtype=torch.int64, device="cuda")
    xq, xs = quant_rows_1x128(x)
    act = gate_up_swiglu_fp8(xq, xs, q13, s13, tp, row_index=idx, limit=10.0, split=split, status=status, wait_ns=50_000_000)
    torch.cuda.synchronize()
    _ok(status)
    x_dq = dequant_rows(xq, xs)[idx.long()]
    ref_act = torch.zeros(n, inter, device="cuda")
    for e, (lo, hi) in enumerate(zip(offsets[:-1], offsets[1:])):
        if hi > lo:
            w = dequant_block_fp8(q13[e], s13[e])
            ref_act[lo:hi] = swiglu_clamp(x_dq[lo:hi] @ w.t(), 10.0)
    assert normwise_rel_err(act, ref_act) < 4 * 2.0**-8, normwise_rel_err(act, ref_act)

    aq, a_s = quant_rows_1x128(act.contiguous())
    y = down_proj_fp8(aq, a_s, q2, s2, tp, row_scale=scale, split=split, status=status, wait_ns=50_000_000)
    y_gather = down_proj_fp8(aq, a_s, q2, s2, tp, row_scale=scale, split=split, status=status, wait_ns=50_000_000, b_tma=False)
    torch.cuda.synchronize()
    _ok(status)
    assert torch.equal(y.view(torch.int16), y_gather.view(torch.int16)), "token tiles by TMA and by gather differ"
    a_dq = dequant_rows(aq, a_s)
    ref_y = torch.zeros(n, hidden, device="cuda")
    for e, (lo, hi) in enumerate(zip(offsets[:-1], offsets[1:])):
        if hi > lo:
            ref_y[lo:hi] = (a_dq[lo:hi] @ dequant_block_fp8(q2[e], s2[e]).t()) * scale[lo:hi, None]
    assert normwise_rel_err(y, ref_y) < 4 * 2.0**-8, normwise_rel_err(y, ref_y)


@pytest.mark.parametrize("world", [1, 2])
def test_layer_with_fp8_weights_matches_dequantised_oracle(world):
    """Whole layer with block-scaled e4m3 experts against the fp32 oracle on the dequantised weights."""
    from moeflow_b200 import MoEConfig
    from moeflow_b200.fixed import FixedEPLayer, simulate_fixed
    from moeflow_b200.parallel.peer import PeerGroup
    from moeflow_b200.reference import moe_reference
    from moeflow_b200.testing import make_bias, make_hidden, make_logits, make_weights

    cfg = MoEConfig(hidden_size=512, moe_intermediate_size=256, n_routed_experts=16, top_k=4)
    cap = 16
    w13, w2 = make_weights(cfg, 0, dtype=torch.float32)
    packs = [(quant_block_fp8(w13[e]), quant_block_fp8(w2[e])) for e in range(cfg.n_routed_experts)]
    w13_dq = torch.stack([dequant_block_fp8(*p[0]) for p in packs])
    w2_dq = torch.stack([dequant_block_fp8(*p[1]) for p in packs])
    bias = make_bias(cfg, 1, device="cuda")
    per = cfg.experts_per_rank(world)
    regions = PeerGroup.local(world, FixedEPLayer.peer_bytes(cfg, world, cap))
    layers = []
    for r in range(world):
        ly = FixedEPLayer(cfg, r, world, None, None, capacity=cap, backend="cuda", device="cuda", peer_region=regions[r],
                          wait_ns=50_000_000)
        sel = packs[r * per:(r + 1) * per]
        stack8 = lambda ts: torch.stack([t.view(torch.uint8) for t in ts]).view(torch.float8_e4m3fn).cuda()  # noqa: E731
        ly.set_weights_fp8(stack8([p[0][0] for p in sel]), torch.stack([p[0][1] for p in sel]).cuda(),
                           stack8([p[1][0] for p in sel]), torch.stack([p[1][1] for p in sel]).cuda())
        layers.append(ly)
    tokens = [cap, 7][:world]
    xs = [make_hidden(t, cfg, 30 + r, device="cuda") for r, t in enumerate(tokens)]
    lgs = [make_logits(t, cfg, 40 + r, device="cuda") for r, t in enumerate(tokens)]
    outs = simulate_fixed(layers, xs, lgs, bias)
    torch.cuda.synchronize()
    for r in range(world):
        assert layers[r].check_status()["code"] == 0
        t = tokens[r]
        ref = moe_reference(xs[r].cpu(), lgs[r].cpu(), bias.cpu(), w13_dq, w2_dq, cfg)
        err = normwise_rel_err(outs[r][:t].cpu(), ref)
        # activations are e4m3 (3 mantissa bits) per 128-wide group: a few percent is the format, not a bug
        assert err < 0.06, err
        assert outs[r][t:].abs().sum() == 0


@pytest.mark.parametrize("shape", [(128, 128), (3, 256, 512), (2, 384, 1536)])
def test_expand_block_fp8_equals_definition(shape):
    """e4m3 x block scale -> bf16 in one pass equals the PyTorch dequantisation rounded once to bf16."""
    from moeflow_b200.ops.fp8 import expand_block_fp8

    g = torch.Generator().manual_seed(5)
    w = torch.randn(*shape, generator=g) * 0.05
    flat = w.reshape(-1, shape[-2], shape[-1])
    qs, ss = zip(*(quant_block_fp8(m) for m in flat))
    q = torch.stack([t.view(torch.uint8) for t in qs]).view(torch.float8_e4m3fn).reshape(shape).cuda()
    s = torch.stack(list(ss)).cuda()
    out = expand_block_fp8(q, s)
    torch.cuda.synchronize()
    ref = torch.stack([dequant_block_fp8(a, b) for a, b in zip(qs, ss)]).reshape(shape).to(torch.bfloat16)
    assert torch.equal(out.cpu(), ref)


def test_layer_expands_fp8_weights_on_256_row_tiles():
    """A layer built with 256-row token tiles and e4m3 weights expands them to bf16 in every forward and then equals,
    bit for bit, the same layer bound to the dequantised bf16 weights."""
    from moeflow_b200 import MoEConfig
    from moeflow_b200.fixed import FixedEPLayer, simulate_fixed
    from moeflow_b200.parallel.peer import PeerGroup
    from moeflow_b200.testing import make_bias, make_hidden, make_logits, make_weights

    cfg = MoEConfig(hidden_size=512, moe_intermediate_size=256, n_routed_experts=4, top_k=2)
    cap = 600
    w13, w2 = make_weights(cfg, 0, dtype=torch.float32)
    packs = [(quant_block_fp8(w13[e]), quant_block_fp8(w2[e])) for e in range(cfg.n_routed_experts)]
    w13_dq = torch.stack([dequant_block_fp8(*p[0]) for p in packs]).to(torch.bfloat16).cuda()
    w2_dq = torch.stack([dequant_block_fp8(*p[1]) for p in packs]).to(torch.bfloat16).cuda()
    bias = make_bias(cfg, 1, device="cuda")
    stack8 = lambda ts: torch.stack([t.view(torch.uint8) for t in ts]).view(torch.float8_e4m3fn).cuda()  # noqa: E731
    outs = []
    for fp8 in (True, False):
        region = PeerGroup.local(1, FixedEPLayer.peer_bytes(cfg, 1, cap))[0]
        ly = FixedEPLayer(cfg, 0, 1, None if fp8 else w13_dq, None if fp8 else w2_dq, capacity=cap, backend="cuda",
                          device="cuda", peer_region=region, wait_ns=50_000_000, gemm_kwargs={"block_m": 256})
        if fp8:
            ly.set_weights_fp8(stack8([p[0][0] for p in packs]), torch.stack([p[0][1] for p in packs]).cuda(),
                               stack8([p[1][0] for p in packs]), torch.stack([p[1][1] for p in packs]).cuda())
        x = make_hidden(cap, cfg, 30, device="cuda")
        lg = make_logits(cap, cfg, 40, device="cuda")
        for _ in range(2):  # the second forward re-expands into the same scratch
            out = simulate_fixed([ly], [x], [lg], bias)[0].clone()
        torch.cuda.synchronize()
        assert ly.check_status()["code"] == 0
        outs.append(out)
    assert torch.isfinite(outs[0].float()).all() and outs[0].abs().sum() > 0
    assert torch.equal(outs[0], outs[1])
