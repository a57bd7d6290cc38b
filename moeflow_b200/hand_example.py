"""A worked example small enough for pencil and paper, pushed through the real variable-size stages.

Two EP ranks, four experts (two per rank), top-2, hidden size 2.  Expert ``g`` is the stand-in
``x -> (g + 1) * x`` (``testing.ScaleExperts``), so every intermediate is a short sum one can verify by hand:

    rank 0   token a = ( 1,  2  )  ->  expert 0 (w 1.5),  expert 1 (w 1.0)
             token b = ( 3, -1  )  ->  expert 1 (w 2.0),  expert 3 (w 0.5)
             token c = ( 2,  0.5)  ->  expert 2 (w 1.25), expert 3 (w 1.25)
    rank 1   token d = ( 0.5, 4 )  ->  expert 3 (w 2.0),  expert 0 (w 0.5)

``trace()`` records what every stage produced on every rank; ``expected_outputs()`` computes the final rows
from the table above alone (no stage code), so the two can be held against each other.  The same scenario
and numbers as ``moeflow/hand_example.py:13-48`` of the reference, so that its documented walk-through
applies here too.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field

import torch

from .comm import simulated_exchange, unpack_meta
from .config import MoEConfig
from .dispatch import build_expert_layout
from .ep_moe import EPMoELayer
from .testing import ScaleExperts

WORLD = 2
CFG = MoEConfig(hidden_size=2, moe_intermediate_size=1, n_routed_experts=4, top_k=2)

#: per rank: (token vector, ((expert, routing weight), (expert, routing weight)))
SCENARIO = (
    (
        ((1.0, 2.0), ((0, 1.5), (1, 1.0))),
        ((3.0, -1.0), ((1, 2.0), (3, 0.5))),
        ((2.0, 0.5), ((2, 1.25), (3, 1.25))),
    ),
    (
        ((0.5, 4.0), ((3, 2.0), (0, 0.5))),
    ),
)


def _tensors(rank: int):
    tokens = SCENARIO[rank]
    x = torch.tensor([list(vec) for vec, _ in tokens])
    ids = torch.tensor([[e for e, _ in routes] for _, routes in tokens], dtype=torch.int32)
    weights = torch.tensor([[w for _, w in routes] for _, routes in tokens])
    return x, ids, weights


# Module-level views of the scenario (names kept for callers of the reference's module).
X = [_tensors(r)[0] for r in range(WORLD)]
TOPK_IDS = [_tensors(r)[1] for r in range(WORLD)]
TOPK_W = [_tensors(r)[2] for r in range(WORLD)]


def expected_outputs() -> list[list[list[float]]]:
    """Final rows straight from the scenario table: ``sum_k w_k * (expert_k + 1) * x``."""
    return [
        [[sum(w * (e + 1) for e, w in routes) * v for v in vec] for vec, routes in SCENARIO[rank]]
        for rank in range(WORLD)
    ]


@dataclass
class StageTrace:
    """Everything the stages produced, one list entry per rank."""

    send_counts: list = field(default_factory=list)
    send_token: list = field(default_factory=list)
    send_slots: list = field(default_factory=list)
    recv_counts: list = field(default_factory=list)
    recv_x: list = field(default_factory=list)
    recv_slots: list = field(default_factory=list)
    recv_weights: list = field(default_factory=list)
    expert_offsets: list = field(default_factory=list)
    expert_entries: list = field(default_factory=list)
    partials: list = field(default_factory=list)
    returned: list = field(default_factory=list)
    out: list = field(default_factory=list)


def trace(dtype: torch.dtype = torch.bfloat16) -> StageTrace:
    experts_here = CFG.experts_per_rank(WORLD)
    placeholder = torch.zeros(experts_here, 1, 1)  # the stand-in experts never read weights
    ranks = range(WORLD)
    layer = {
        r: EPMoELayer(CFG, r, WORLD, placeholder, placeholder, experts=ScaleExperts(r * experts_here), combine_dtype=dtype)
        for r in ranks
    }
    t = StageTrace()

    # source side: group rows by destination rank
    sent = {r: layer[r].stage_dispatch(X[r].to(dtype), TOPK_W[r], TOPK_IDS[r]) for r in ranks}
    for r in ranks:
        t.send_counts.append(sent[r].plan.send_counts.tolist())
        t.send_token.append(sent[r].plan.send_token.tolist())
        t.send_slots.append(unpack_meta(sent[r].send_meta)[0].tolist())

    # the exchange (in one process): rows and their metadata travel with the same counts
    counts = [sent[r].plan.send_counts for r in ranks]
    got_x, got_counts = simulated_exchange([sent[r].send_x for r in ranks], counts)
    got_meta, _ = simulated_exchange([sent[r].send_meta for r in ranks], counts)

    # owner side: expert-major layout, experts, one partial row per received row
    partial = {}
    for r in ranks:
        slots, weights = unpack_meta(got_meta[r])
        layout = build_expert_layout(slots, experts_here)
        partial[r] = layer[r].stage_experts(got_x[r], got_meta[r])
        t.recv_counts.append(got_counts[r].tolist())
        t.recv_x.append(got_x[r].float().tolist())
        t.recv_slots.append(slots.tolist())
        t.recv_weights.append(weights.tolist())
        t.expert_offsets.append(layout.expert_offsets.tolist())
        t.expert_entries.append([(int(a), int(b)) for a, b in zip(layout.entry_row.tolist(), layout.entry_slot.tolist())])
        t.partials.append(partial[r].float().tolist())

    # way back and source-side merge
    home, _ = simulated_exchange([partial[r] for r in ranks], got_counts)
    for r in ranks:
        t.returned.append(home[r].float().tolist())
        t.out.append(layer[r].stage_combine(home[r], sent[r], dtype).float().tolist())
    return t


def run(dtype: torch.dtype = torch.bfloat16) -> dict:
    """``trace()`` as a plain dict (stage name -> per-rank lists)."""
    return asdict(trace(dtype))


def main() -> None:
    record = run()
    for stage, per_rank in record.items():
        for rank, value in enumerate(per_rank):
            print(f"{stage:>15s}  rank {rank}: {json.dumps(value)}")
    print(f"{'closed form':>15s}        : {json.dumps(expected_outputs())}")


if __name__ == "__main__":
    main()
