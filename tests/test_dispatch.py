"""Dispatch and restore move data only, so they are checked bit for bit against the loop oracle."""

import pytest
import torch

from moeflow_b200 import dispatch as D
from moeflow_b200.comm import pack_meta, simulated_exchange, unpack_meta
from moeflow_b200.reference import ep_dispatch_reference

E, K, H = 32, 4, 8


def _as_routes(ids, w):
    return [list(zip(map(int, ids[t].tolist()), map(float, w[t].tolist()))) for t in range(ids.shape[0])]


def _distinct_ids(n_tokens, n_experts, gen):
    if n_tokens == 0:
        return torch.empty(0, K, dtype=torch.int32)
    return torch.stack([torch.randperm(n_experts, generator=gen)[:K] for _ in range(n_tokens)]).to(torch.int32)


def _case(kind, n_tokens, gen):
    w = torch.rand(n_tokens, K, generator=gen)
    if kind == "spread":
        return _distinct_ids(n_tokens, E, gen), w
    if kind == "identical":
        return torch.arange(K, dtype=torch.int32).repeat(n_tokens, 1), w
    if kind == "first_quarter":
        return _distinct_ids(n_tokens, E // 4, gen), w
    raise AssertionError(kind)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("kind", ["spread", "identical", "first_quarter"])
@pytest.mark.parametrize("tokens", [[0, 3, 1, 5, 2, 0, 7, 4], [1] * 8, [16] * 8])
def test_received_rows_match_the_oracle(world, kind, tokens):
    per_rank_experts = E // world
    gen = torch.Generator().manual_seed(1000 * world + len(kind) + tokens[1])
    routed = [_case(kind, tokens[r], gen) for r in range(world)]
    xs = [torch.randn(tokens[r], H, generator=gen).bfloat16() for r in range(world)]

    plans = [D.plan_dispatch(ids, w, world, per_rank_experts) for ids, w in routed]
    counts = [p.send_counts for p in plans]
    recv_x, recv_counts = simulated_exchange([D.pack_send(x, p) for x, p in zip(xs, plans)], counts)
    recv_meta, _ = simulated_exchange([pack_meta(p.slot_local_id, p.slot_weight) for p in plans], counts)

    want = ep_dispatch_reference([_as_routes(ids, w) for ids, w in routed], per_rank_experts)
    for dst in range(world):
        assert recv_x[dst].shape[0] == len(want[dst])
        local_id, weight = unpack_meta(recv_meta[dst])
        for row, (src, t, hits) in enumerate(want[dst]):
            assert torch.equal(recv_x[dst][row], xs[src][t])
            got = [(i, w) for i, w in zip(local_id[row].tolist(), weight[row].tolist()) if i != D.INVALID]
            assert got == [(e, torch.tensor(w, dtype=torch.float32).item()) for e, w in hits]
        per_src = [sum(1 for s, _, _ in want[dst] if s == src) for src in range(world)]
        assert recv_counts[dst].tolist() == per_src


def test_layout_is_expert_major_stable_and_complete():
    local_id = torch.tensor([[2, -1, 0], [0, 0, -1], [-1, -1, -1], [1, 2, 2]], dtype=torch.int32)
    lay = D.build_expert_layout(local_id, num_local_experts=3)
    assert lay.expert_offsets.tolist() == [0, 3, 4, 7]
    assert list(zip(lay.entry_row.tolist(), lay.entry_slot.tolist())) == [
        (0, 2), (1, 0), (1, 1), (3, 0), (0, 0), (3, 1), (3, 2)
    ]


def test_identity_experts_restore_the_input_bitwise():
    world, per, hidden, n = 4, 2, 16, 9
    gen = torch.Generator().manual_seed(7)
    ids = torch.randint(0, world * per, (n, 1), generator=gen, dtype=torch.int32)
    x = torch.randn(n, hidden, generator=gen).bfloat16()
    x[0, 0] = -0.0
    plan = D.plan_dispatch(ids, torch.ones(n, 1), world, per)
    out = D.combine(D.pack_send(x, plan), plan, n, world, torch.bfloat16)
    # -0.0 + (+0.0 start) is +0.0: everything else is bit-exact
    assert torch.equal(out[1:], x[1:]) and torch.equal(out[0, 1:], x[0, 1:]) and out[0, 0] == 0


def _layout(local_id):
    return D.build_expert_layout(local_id, int(local_id.max()) + 1)


def test_garbage_in_an_empty_slot_is_never_read():
    local_id = torch.tensor([[0, -1]], dtype=torch.int32)
    y = torch.tensor([[3.0]], dtype=torch.bfloat16)
    out = D.reduce_local(y, _layout(local_id), torch.tensor([[0.5, float("nan")]]), torch.bfloat16)
    assert out.item() == 3.0


def test_sums_start_from_positive_zero():
    local_id = torch.tensor([[0]], dtype=torch.int32)
    neg_zero = torch.tensor([[-0.0]], dtype=torch.bfloat16)
    out = D.reduce_local(neg_zero, _layout(local_id), torch.tensor([[1.0]]), torch.bfloat16)
    assert not torch.signbit(out).item()
    plan = D.plan_dispatch(torch.tensor([[1]], dtype=torch.int32), torch.ones(1, 1), world=2, experts_per_rank=1)
    assert not torch.signbit(D.combine(neg_zero, plan, 1, 2, torch.bfloat16)).item()


def test_no_tokens():
    plan = D.plan_dispatch(torch.empty(0, 4, dtype=torch.int32), torch.empty(0, 4), world=4, experts_per_rank=2)
    assert plan.send_counts.tolist() == [0, 0, 0, 0] and plan.send_token.numel() == 0


def test_reduce_only_adds_preweighted_branches():
    local_id = torch.tensor([[1, -1, 0]], dtype=torch.int32)
    lay = _layout(local_id)
    y = torch.tensor([[0.25], [3.0]], dtype=torch.bfloat16)
    w = torch.tensor([[7.0, float("nan"), 9.0]])
    assert D.reduce_local(y, lay, w, torch.float32).item() == 3.25
    assert D.entry_weights(lay, w).tolist() == [9.0, 7.0]


def test_meta_round_trip_keeps_weight_bits():
    ids = torch.tensor([[3, -1]], dtype=torch.int32)
    w = torch.tensor([[-0.0, 1.5]])
    got_ids, got_w = unpack_meta(pack_meta(ids, w))
    assert torch.equal(got_ids, ids) and torch.equal(got_w.view(torch.int32), w.view(torch.int32))
