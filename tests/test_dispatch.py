"""Variable-size dispatch / restore.  These stages only move data, so everything is compared bit for bit:
against the loop oracle of ``reference.py``, and against brute-force restatements written here."""

from dataclasses import dataclass

import pytest
import torch

from moeflow_b200 import dispatch as D
from moeflow_b200.comm import pack_meta, simulated_exchange, unpack_meta
from moeflow_b200.reference import ep_dispatch_reference

EXPERTS, TOP_K, HIDDEN = 32, 4, 8
TOKEN_PROFILES = {"ragged": (0, 3, 1, 5, 2, 0, 7, 4), "one_each": (1,) * 8, "sixteen_each": (16,) * 8}


def _routing(profile: str, n: int, gen) -> tuple[torch.Tensor, torch.Tensor]:
    """ids [n, K] int32 with distinct experts per token, weights [n, K] fp32."""
    pool = {"anywhere": EXPERTS, "low_quarter": EXPERTS // 4}.get(profile)
    if profile == "all_alike":
        ids = torch.arange(TOP_K).expand(n, TOP_K)
    else:
        ids = torch.stack([torch.randperm(pool, generator=gen)[:TOP_K] for _ in range(n)]) if n else torch.empty(0, TOP_K)
    return ids.to(torch.int32).contiguous(), torch.rand(n, TOP_K, generator=gen)


@dataclass
class Exchanged:
    """All ranks' dispatch run inside one process."""

    xs: list
    routed: list
    rows: list          # per destination: received hidden rows
    slot_ids: list      # per destination: [S, K] local ids (-1 = not here)
    slot_w: list
    per_source: list    # per destination: rows received from each source

    @classmethod
    def run(cls, world: int, tokens, profile: str, seed: int) -> "Exchanged":
        gen = torch.Generator().manual_seed(seed)
        routed = [_routing(profile, tokens[r], gen) for r in range(world)]
        xs = [torch.randn(tokens[r], HIDDEN, generator=gen).to(torch.bfloat16) for r in range(world)]
        plans = [D.plan_dispatch(ids, w, world, EXPERTS // world) for ids, w in routed]
        counts = [p.send_counts for p in plans]
        rows, per_source = simulated_exchange([D.pack_send(x, p) for x, p in zip(xs, plans)], counts)
        meta, _ = simulated_exchange([pack_meta(p.slot_local_id, p.slot_weight) for p in plans], counts)
        unpacked = [unpack_meta(m) for m in meta]
        return cls(xs, routed, rows, [u[0] for u in unpacked], [u[1] for u in unpacked], per_source)

    def oracle(self, world: int):
        as_lists = [[[(int(e), float(w)) for e, w in zip(i.tolist(), ww.tolist())] for i, ww in zip(ids, wts)]
                    for ids, wts in self.routed]
        return ep_dispatch_reference(as_lists, EXPERTS // world)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("profile", ["anywhere", "all_alike", "low_quarter"])
@pytest.mark.parametrize("tokens", list(TOKEN_PROFILES))
def test_every_rank_receives_what_the_loop_oracle_says(world, profile, tokens):
    ex = Exchanged.run(world, TOKEN_PROFILES[tokens], profile, seed=97 * world + len(profile) + len(tokens))
    expected = ex.oracle(world)
    for dst in range(world):
        want_rows = expected[dst]
        assert ex.rows[dst].shape[0] == len(want_rows)
        sources_seen = [0] * world
        for r, (src, token, hits) in enumerate(want_rows):
            sources_seen[src] += 1
            assert torch.equal(ex.rows[dst][r], ex.xs[src][token]), (dst, r)
            here = [(int(i), w) for i, w in zip(ex.slot_ids[dst][r].tolist(), ex.slot_w[dst][r].tolist()) if i != D.INVALID]
            assert here == [(e, torch.tensor(w).item()) for e, w in hits]  # weights travel as fp32 bits
        assert ex.per_source[dst].tolist() == sources_seen


@pytest.mark.parametrize("world", [2, 4])
def test_one_row_per_token_and_destination_in_token_order(world):
    """Independent of the oracle: a token contributes exactly one row to every rank that owns one of its
    experts, and a source's rows for one destination are in token order."""
    per = EXPERTS // world
    ids, w = _routing("anywhere", 11, torch.Generator().manual_seed(3))
    plan = D.plan_dispatch(ids, w, world, per)
    owners = [sorted({int(e) // per for e in row}) for row in ids.tolist()]
    expect_tokens = [t for dst in range(world) for t, own in enumerate(owners) if dst in own]
    assert plan.send_token.tolist() == expect_tokens
    assert plan.send_counts.tolist() == [sum(dst in own for own in owners) for dst in range(world)]


def test_expert_major_layout_equals_a_stable_sort():
    gen = torch.Generator().manual_seed(12)
    local = torch.randint(-1, 5, (13, 3), generator=gen, dtype=torch.int32)
    lay = D.build_expert_layout(local, num_local_experts=5)
    triples = sorted((int(e), r, s) for r, row in enumerate(local.tolist()) for s, e in enumerate(row) if e >= 0)
    assert list(zip(lay.entry_row.tolist(), lay.entry_slot.tolist())) == [(r, s) for _, r, s in triples]
    per_expert = [sum(1 for e, _, _ in triples if e == k) for k in range(5)]
    assert lay.expert_offsets.tolist() == [sum(per_expert[:k]) for k in range(6)]


def test_a_row_without_local_slots_takes_no_entries():
    lay = D.build_expert_layout(torch.tensor([[1, -1], [-1, -1], [0, 1]], dtype=torch.int32), num_local_experts=2)
    assert lay.expert_offsets.tolist() == [0, 1, 3] and 1 not in lay.entry_row.tolist()


def test_single_hit_identity_round_trip_is_bit_exact_except_negative_zero():
    world, per, n = 4, 2, 9
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(n, 16, generator=gen).to(torch.bfloat16)
    x[3, 5] = -0.0
    ids = torch.randint(0, world * per, (n, 1), generator=gen, dtype=torch.int32)
    plan = D.plan_dispatch(ids, torch.ones(n, 1), world, per)
    restored = D.combine(D.pack_send(x, plan), plan, n, world, torch.bfloat16)  # identity experts, weight 1
    same = restored.view(torch.int16) == x.view(torch.int16)
    same[3, 5] = True
    assert bool(same.all())
    assert restored[3, 5] == 0 and not torch.signbit(restored[3, 5])  # the sum starts at +0.0


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_owner_reduce_reads_neither_empty_slots_nor_weights(out_dtype):
    """Expert outputs arrive already weighted: the reduce adds them in slot order and touches nothing else,
    so NaN in an empty slot's weight (or any weight) cannot leak."""
    local = torch.tensor([[1, -1, 0]], dtype=torch.int32)
    lay = D.build_expert_layout(local, num_local_experts=2)
    weighted = torch.tensor([[0.25], [3.0]], dtype=torch.bfloat16)  # expert-major: expert 0 (slot 2), expert 1 (slot 0)
    poison = torch.tensor([[7.0, float("nan"), 9.0]])
    assert D.reduce_local(weighted, lay, poison, out_dtype).item() == 3.25
    assert D.entry_weights(lay, poison).tolist() == [9.0, 7.0]


def test_sums_of_negative_zero_come_out_positive():
    lay = D.build_expert_layout(torch.tensor([[0]], dtype=torch.int32), num_local_experts=1)
    minus_zero = torch.tensor([[-0.0]], dtype=torch.bfloat16)
    assert not torch.signbit(D.reduce_local(minus_zero, lay, torch.ones(1, 1), torch.bfloat16)).item()
    plan = D.plan_dispatch(torch.tensor([[1]], dtype=torch.int32), torch.ones(1, 1), world=2, experts_per_rank=1)
    assert not torch.signbit(D.combine(minus_zero, plan, 1, 2, torch.bfloat16)).item()


def test_an_empty_batch_plans_nothing():
    plan = D.plan_dispatch(torch.empty(0, TOP_K, dtype=torch.int32), torch.empty(0, TOP_K), world=4, experts_per_rank=2)
    assert plan.send_counts.tolist() == [0] * 4 and plan.send_token.numel() == 0


def test_metadata_packing_preserves_every_weight_bit():
    ids = torch.tensor([[3, -1], [0, 7]], dtype=torch.int32)
    w = torch.tensor([[-0.0, 1.5], [float("inf"), 1e-40]])  # signed zero, infinity, a subnormal
    ids2, w2 = unpack_meta(pack_meta(ids, w))
    assert torch.equal(ids2, ids) and torch.equal(w2.view(torch.int32), w.view(torch.int32))
