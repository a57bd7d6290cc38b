"""FixedEPLayer on the torch backend (CPU): fixed == variable-size pipeline bitwise, zero padding,
static buffers, stage prefixes, external expert hooks, direct expert output."""

import pytest
import torch

from conftest import SMALL, replace
from moeflow_b200 import MoEConfig
from moeflow_b200.ep_moe import EPMoELayer, shard_experts, simulate_ep
from moeflow_b200.fixed import STAGES, FixedEPLayer, meta_lanes, row_pitch_lanes, simulate_fixed
from moeflow_b200.reference import ep_dispatch_reference, moe_reference, route_reference
from moeflow_b200.testing import DISTRIBUTIONS, make_bias, make_hidden, make_logits, make_weights
from moeflow_b200.tolerances import bitwise_equal, normwise_rel_err


def _setup(cfg, world, cap, tokens, dtype=torch.bfloat16, dist="uniform", seed=0):
    w13, w2 = make_weights(cfg, seed, dtype=dtype)
    bias = make_bias(cfg, seed + 1)
    xs = [make_hidden(tokens[r], cfg, seed + 10 + r, dtype=dtype) for r in range(world)]
    lgs = [make_logits(tokens[r], cfg, seed + 20 + r, dist=dist) for r in range(world)]
    fixed = [FixedEPLayer(cfg, r, world, *shard_experts(w13, w2, r, world), capacity=cap, backend="torch") for r in range(world)]
    naive = [EPMoELayer(cfg, r, world, *shard_experts(w13, w2, r, world), combine_dtype=dtype) for r in range(world)]
    return w13, w2, bias, xs, lgs, fixed, naive


def test_row_geometry():
    assert meta_lanes(8) == 34 and meta_lanes(8, 4) == 17
    assert row_pitch_lanes(4096, 8) == 4136 and (row_pitch_lanes(4096, 8) * 2) % 16 == 0
    assert row_pitch_lanes(64, 2, 4) % 4 == 0


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("dist", DISTRIBUTIONS)
def test_fixed_equals_variable_pipeline_bitwise(world, dist):
    cap = 8
    tokens = [8, 3, 0, 5, 1, 8, 2, 7][:world]
    w13, w2, bias, xs, lgs, fixed, naive = _setup(SMALL, world, cap, tokens, dist=dist)
    out_f = simulate_fixed(fixed, xs, lgs, bias)
    out_n = simulate_ep(naive, xs, lgs, bias)
    for r in range(world):
        t = tokens[r]
        assert bitwise_equal(out_f[r][:t], out_n[r])
        assert out_f[r][t:].abs().sum() == 0


def test_cpu_plumbing_configuration_fp32_softmax():
    """hidden 64, 8 experts, top-2, intermediate 128, fp32, softmax scoring, 16 tokens/rank, EP=2."""
    cfg = MoEConfig(hidden_size=64, moe_intermediate_size=128, n_routed_experts=8, n_shared_experts=1, top_k=2,
                    scoring_func="softmax")
    w13, w2, bias, xs, lgs, fixed, naive = _setup(cfg, 2, 16, [16, 16], dtype=torch.float32)
    out = simulate_fixed(fixed, xs, lgs, None)
    ref_n = simulate_ep(naive, xs, lgs, None)
    for r in range(2):
        assert bitwise_equal(out[r], ref_n[r])
        assert normwise_rel_err(out[r], moe_reference(xs[r], lgs[r], None, w13, w2, cfg)) < 1e-5
    # dispatch: what every owner received equals the oracle's one-copy-per-rank list, bit for bit
    want = ep_dispatch_reference([route_reference(lg, None, cfg) for lg in lgs], cfg.experts_per_rank(2))
    for d, ly in enumerate(fixed):
        x_rows, local, wts = ly.received_routing()
        got = []
        for s in range(2):
            for t in range(16):
                row = s * 16 + t
                hits = [(int(i), float(w)) for i, w in zip(local[row].tolist(), wts[row].tolist()) if i >= 0]
                if hits:
                    got.append((s, t, hits))
                    assert torch.equal(x_rows[row], xs[s][t])
        assert [(s, t, [e for e, _ in h]) for s, t, h in got] == [(s, t, [e for e, _ in h]) for s, t, h in want[d]]
        for (_, _, hg), (_, _, hw) in zip(got, want[d]):
            for (_, a), (_, b) in zip(hg, hw):
                assert abs(a - b) <= 1e-6 * abs(b)  # oracle scores in float64, the router in fp32


def test_num_valid_masks_rows():
    world, cap = 2, 8
    w13, w2, bias, xs, lgs, fixed, naive = _setup(SMALL, world, cap, [8, 8])
    nv = [torch.tensor(3), torch.tensor(0)]
    out = simulate_fixed(fixed, xs, lgs, bias, nv)
    ref = simulate_ep(naive, [xs[0][:3], xs[1][:0]], [lgs[0][:3], lgs[1][:0]], bias)
    assert bitwise_equal(out[0][:3], ref[0]) and out[0][3:].abs().sum() == 0 and out[1].abs().sum() == 0


def test_buffers_are_static():
    w13, w2, bias, xs, lgs, fixed, _ = _setup(SMALL, 2, 8, [8, 4])
    before = [(ly._send_store.data_ptr(), ly._recv_store.data_ptr(), ly.ret_send.data_ptr(), ly.ret_recv.data_ptr()) for ly in fixed]
    for _ in range(3):
        simulate_fixed(fixed, xs, lgs, bias)
    after = [(ly._send_store.data_ptr(), ly._recv_store.data_ptr(), ly.ret_send.data_ptr(), ly.ret_recv.data_ptr()) for ly in fixed]
    assert before == after


def test_stage_prefixes_world1():
    cfg = SMALL
    w13, w2 = make_weights(cfg, 0)
    ly = FixedEPLayer(cfg, 0, 1, w13, w2, capacity=4, backend="torch")
    x, lg = make_hidden(4, cfg, 1), make_logits(4, cfg, 2)
    shapes = {}
    for st in STAGES:
        shapes[st] = tuple(ly.forward(x, lg, None, stop_after=st).shape)
    assert shapes["ROUTER"] == (4, cfg.top_k) and shapes["DISPATCH"] == (4, 1)
    assert shapes["A2A_FORWARD"] == (1, 4, ly.row_width) and shapes["EXPERT"] == (1, 4, cfg.hidden_size)
    assert shapes["COMBINE"] == (4, cfg.hidden_size)
    full = ly.forward(x, lg, None)
    assert bitwise_equal(full, ly.forward(x, lg, None, stop_after="COMBINE"))
    with pytest.raises(ValueError):
        ly.forward(x, lg, None, stop_after="NOPE")


def test_flags_are_accepted_and_validated():
    cfg = SMALL
    w13, w2 = make_weights(cfg, 0)
    with pytest.raises(ValueError, match="metadata_kernel"):
        FixedEPLayer(cfg, 0, 1, w13, w2, capacity=4, fused_reduce=True, backend="torch")
    ly = FixedEPLayer(cfg, 0, 1, w13, w2, capacity=4, metadata_kernel=True, fused_reduce=True, fused_combine=True,
                      fused_dispatch=True, backend="torch")
    x, lg = make_hidden(4, cfg, 1), make_logits(4, cfg, 2)
    base = FixedEPLayer(cfg, 0, 1, w13, w2, capacity=4, backend="torch").forward(x, lg, None)
    assert bitwise_equal(ly.forward(x, lg, None), base)
    with pytest.raises(ValueError, match="capacity"):
        ly.forward(make_hidden(5, cfg, 1), make_logits(5, cfg, 2), None)


def test_external_expert_function_and_prepare_hook():
    cfg = replace(SMALL, top_k=2)
    world, cap = 2, 4
    w13, w2, bias, xs, lgs, fixed, _ = _setup(cfg, world, cap, [4, 4])
    base = simulate_fixed(fixed, xs, lgs, bias)
    seen = {}

    def expert_fn(x_rows, local, wts):
        seen["shapes"] = (tuple(x_rows.shape), tuple(local.shape), tuple(wts.shape))
        return x_rows.to(torch.float32).mul(2.0).to(x_rows.dtype).contiguous()

    ly = fixed[0]
    ly.stage_experts(expert_fn)
    assert seen["shapes"] == ((world * cap, cfg.hidden_size), (world * cap, cfg.top_k), (world * cap, cfg.top_k))
    assert bitwise_equal(ly.ret_send.view(world * cap, -1), (ly.recv[:, :, : cfg.hidden_size].reshape(world * cap, -1).float() * 2).to(ly.dtype))

    def prepare_fn(rows):
        assert rows.shape == (world * cap, ly.row_width)
        return (rows[:, : cfg.hidden_size].contiguous(),)

    out = ly.stage_experts(lambda h: h.clone(), prepare_fn=prepare_fn)
    assert out is None
    assert bitwise_equal(ly.ret_send.view(world * cap, -1), ly.recv[:, :, : cfg.hidden_size].reshape(world * cap, -1).contiguous())
    del base


def test_direct_expert_output_aliases_and_validates():
    cfg = SMALL
    w13, w2 = make_weights(cfg, 0)
    ly = FixedEPLayer(cfg, 0, 1, w13, w2, capacity=4, backend="torch")
    x, lg = make_hidden(4, cfg, 1), make_logits(4, cfg, 2)
    ly.stage_pack(x, lg, None)
    ly._recv_store.copy_(ly._send_store)
    prepare = lambda rows: (rows[:, : cfg.hidden_size],)  # noqa: E731
    produced = torch.full((4, cfg.hidden_size), 3.0, dtype=ly.dtype)
    got = ly.stage_experts(lambda h: produced, prepare_fn=prepare, direct_output=True)
    assert got.data_ptr() == produced.data_ptr() and got.shape == (1, 4, cfg.hidden_size)
    with pytest.raises(ValueError, match="requires custom input preparation"):
        ly.stage_experts(lambda h: produced, direct_output=True)
    with pytest.raises(ValueError, match="external expert function"):
        ly.stage_experts(None, prepare_fn=prepare)
    for bad in (
        torch.zeros(3, cfg.hidden_size, dtype=ly.dtype),
        torch.zeros(4, cfg.hidden_size, dtype=torch.float32),
        torch.zeros(cfg.hidden_size, 4, dtype=ly.dtype).t(),
    ):
        with pytest.raises(ValueError, match="Direct expert output"):
            ly.stage_experts(lambda h, bad=bad: bad, prepare_fn=prepare, direct_output=True)


def test_forward_routed_with_custom_combine():
    cfg = SMALL
    w13, w2 = make_weights(cfg, 0)
    ly = FixedEPLayer(cfg, 0, 1, w13, w2, capacity=4, backend="torch")
    x, lg = make_hidden(3, cfg, 1), make_logits(3, cfg, 2)
    w, ids = ly.stage_route(lg, None)
    base = ly.forward_routed(x, w, ids)
    calls = []

    def combine_fn(ret_recv, hit):
        calls.append((tuple(ret_recv.shape), tuple(hit.shape)))
        return ret_recv[0].clone()

    out = ly.forward_routed(x, w, ids, combine_fn=combine_fn)
    assert calls == [((1, 4, cfg.hidden_size), (4, 1))] and out.shape == (3, cfg.hidden_size)
    assert bitwise_equal(out, base)
