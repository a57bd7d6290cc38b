"""The variable-size pipeline with every rank inside one process: against the loop oracle, against itself
(run-to-run), and against a re-sharding of the same problem (the EP degree must not change which experts run,
only how the partial sums are grouped)."""

from dataclasses import dataclass, field

import pytest
import torch

from conftest import SMALL
from moeflow_b200.ep_moe import EPMoELayer, shard_experts, simulate_ep
from moeflow_b200.reference import moe_reference
from moeflow_b200.testing import DISTRIBUTIONS, make_bias, make_hidden, make_logits, make_weights
from moeflow_b200.tolerances import bitwise_equal, gemm_tolerance, normwise_rel_err

RAGGED = (5, 0, 9, 2, 1, 7, 3, 4)


@dataclass
class Problem:
    """One layer's weights and the tokens of every rank, all derived from one seed."""

    world: int
    tokens: tuple
    profile: str = "uniform"
    seed: int = 0
    xs: list = field(init=False)
    logits: list = field(init=False)

    def __post_init__(self):
        self.w13, self.w2 = make_weights(SMALL, self.seed)
        self.bias = make_bias(SMALL, self.seed + 1)
        self.xs = [make_hidden(n, SMALL, self.seed + 10 + r) for r, n in enumerate(self.tokens[: self.world])]
        self.logits = [make_logits(n, SMALL, self.seed + 20 + r, dist=self.profile) for r, n in enumerate(self.tokens[: self.world])]

    def solve(self, world: int | None = None, wire_dtype=torch.bfloat16, xs=None, logits=None):
        world = world or self.world
        layers = [EPMoELayer(SMALL, r, world, *shard_experts(self.w13, self.w2, r, world), combine_dtype=wire_dtype)
                  for r in range(world)]
        return simulate_ep(layers, xs or self.xs, logits or self.logits, self.bias)

    def oracle(self, rank: int) -> torch.Tensor:
        return moe_reference(self.xs[rank], self.logits[rank], self.bias, self.w13, self.w2, SMALL)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("profile", DISTRIBUTIONS)
def test_every_rank_is_within_tolerance_of_the_oracle(world, profile):
    p = Problem(world, RAGGED, profile)
    for rank, out in enumerate(p.solve()):
        assert out.shape == p.xs[rank].shape and out.dtype == p.xs[rank].dtype
        if out.numel():
            assert normwise_rel_err(out, p.oracle(rank)) < gemm_tolerance()


def test_two_runs_agree_bit_for_bit():
    first = Problem(4, (6, 6, 6, 6), "zipf", seed=5).solve()
    second = Problem(4, (6, 6, 6, 6), "zipf", seed=5).solve()
    assert all(bitwise_equal(a, b) for a, b in zip(first, second))


def test_ranks_without_tokens():
    nobody = Problem(2, (0, 0)).solve()
    assert [tuple(o.shape) for o in nobody] == [(0, SMALL.hidden_size)] * 2
    one_sided = Problem(4, (7, 0, 0, 0), seed=2)
    outs = one_sided.solve()
    assert outs[1].numel() == 0 and normwise_rel_err(outs[0], one_sided.oracle(0)) < gemm_tolerance()


def test_resharding_only_regroups_the_sum():
    """The same 12 tokens on rank 0 at EP = 1, 2, 4, 8 with fp32 partial rows on the wire: every expert output is
    computed identically, only the grouping of the K terms into per-rank partial sums differs, so the results agree
    to a few fp32 roundings of a bf16-sized value."""
    p = Problem(1, (12,), seed=3)
    whole = p.solve(wire_dtype=torch.float32)[0].float()
    for world in (2, 4, 8):
        nothing = [p.xs[0][:0]] * (world - 1)
        no_logits = [p.logits[0][:0]] * (world - 1)
        split = p.solve(world, torch.float32, xs=[p.xs[0], *nothing], logits=[p.logits[0], *no_logits])[0].float()
        assert (split - whole).abs().max() <= 2.0**-7 * whole.abs().max()


def test_bf16_and_fp32_wire_formats_stay_close():
    p = Problem(4, (5, 3, 0, 6), "zipf", seed=11)
    for narrow, wide in zip(p.solve(wire_dtype=torch.bfloat16), p.solve(wire_dtype=torch.float32)):
        if wide.numel():
            assert normwise_rel_err(narrow, wide) < gemm_tolerance()
