"""Per-rank, communication-free stages of the variable-size ("naive") expert-parallel pipeline.

Contract
  * every rank owns the tokens of its own data-parallel shard;
  * experts are placed in contiguous blocks: rank r owns experts ``[r*L, (r+1)*L)``;
  * a token travels to a destination rank at most once, however many of its experts live there, and
    carries K slots (local expert id or -1, routing weight or 0);
  * send rows are ordered by destination rank, then by token index;
  * the destination sums a row's local hits in slot order k = 0..K-1 in fp32 starting from +0.0 and
    returns one partial row per received row;
  * the source sums the partial rows of a token over destination ranks in ascending rank order, in
    fp32 starting from +0.0.

This path needs the per-destination counts on the host, so it is not CUDA-graph capturable; it is
the bitwise oracle of the fixed-capacity path on valid rows.  Behavioural counterpart of the
reference's ``moeflow/dispatch.py:21-124``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

INVALID = -1


@dataclass
class DispatchPlan:
    """Source-side plan; send row i goes to ``send_rank[i]`` and carries token ``send_token[i]``."""

    send_token: torch.Tensor  # [S] int64
    send_rank: torch.Tensor  # [S] int64, non-decreasing
    send_counts: torch.Tensor  # [world] int64
    slot_local_id: torch.Tensor  # [S, K] int32, INVALID where the slot lives elsewhere
    slot_weight: torch.Tensor  # [S, K] fp32, 0 where INVALID


def plan_dispatch(
    topk_ids: torch.Tensor, topk_weights: torch.Tensor, world: int, experts_per_rank: int
) -> DispatchPlan:
    n_tokens, _ = topk_ids.shape
    ids = topk_ids.to(torch.int64)
    owner = torch.div(ids, experts_per_rank, rounding_mode="floor")  # [T, K]
    ranks = torch.arange(world, device=ids.device)
    touches = (owner[:, None, :] == ranks[None, :, None]).any(dim=-1)  # [T, world]
    # Enumerate (rank, token) pairs rank-major: transposing first makes nonzero() do the ordering.
    rank_idx, token_idx = touches.transpose(0, 1).nonzero(as_tuple=True)
    counts = touches.sum(dim=0).to(torch.int64)

    here = owner[token_idx] == rank_idx[:, None]  # [S, K]
    local = ids[token_idx] - rank_idx[:, None] * experts_per_rank
    slot_local_id = torch.where(here, local, torch.full_like(local, INVALID)).to(torch.int32)
    w = topk_weights.to(torch.float32)[token_idx]
    slot_weight = torch.where(here, w, torch.zeros_like(w))
    del n_tokens
    return DispatchPlan(token_idx, rank_idx, counts, slot_local_id, slot_weight)


def pack_send(x: torch.Tensor, plan: DispatchPlan) -> torch.Tensor:
    return x[plan.send_token]


@dataclass
class ExpertLayout:
    """Destination-side expert-major order over the (received row, slot) entries."""

    entry_row: torch.Tensor  # [N] int64
    entry_slot: torch.Tensor  # [N] int64
    expert_offsets: torch.Tensor  # [L + 1] int64; expert e owns entries [off[e], off[e+1])


def build_expert_layout(recv_local_id: torch.Tensor, num_local_experts: int) -> ExpertLayout:
    _, top_k = recv_local_id.shape
    flat = recv_local_id.reshape(-1).to(torch.int64)
    live = torch.nonzero(flat != INVALID).reshape(-1)  # ascending (row, slot)
    experts = flat[live]
    # A stable sort keeps (row, slot) ascending inside every expert, so the layout is deterministic.
    by_expert = torch.sort(experts, stable=True).indices
    entries = live[by_expert]
    counts = torch.bincount(experts, minlength=num_local_experts)
    offsets = torch.zeros(num_local_experts + 1, dtype=torch.int64, device=flat.device)
    torch.cumsum(counts, dim=0, out=offsets[1:])
    return ExpertLayout(torch.div(entries, top_k, rounding_mode="floor"), entries % top_k, offsets)


def gather_expert_input(recv_x: torch.Tensor, layout: ExpertLayout) -> torch.Tensor:
    return recv_x[layout.entry_row]


def entry_weights(layout: ExpertLayout, recv_weight: torch.Tensor) -> torch.Tensor:
    """Routing weight of every expert-major entry, ``[N]`` fp32."""
    return recv_weight.to(torch.float32)[layout.entry_row, layout.entry_slot]


def _ordered_masked_sum(values: torch.Tensor, present: torch.Tensor) -> torch.Tensor:
    """fp32 sum over dim 1 in index order, starting from +0.0, skipping absent terms.

    ``values [N, S, H]``, ``present [N, S]``.  Skipped terms are not added at all (adding a zero could
    turn a -0.0 running sum into +0.0, and garbage in absent slots must never be read as a number).
    """
    n, steps, width = values.shape
    acc = torch.zeros(n, width, dtype=torch.float32, device=values.device)
    for i in range(steps):
        acc = torch.where(present[:, i, None], acc + values[:, i].to(torch.float32), acc)
    return acc


def reduce_local(
    expert_out: torch.Tensor, layout: ExpertLayout, recv_weight: torch.Tensor, out_dtype: torch.dtype
) -> torch.Tensor:
    """Per received row: sum the local hits in slot order (fp32, from +0.0), cast to ``out_dtype``.

    ``expert_out`` already holds ``bf16(weight * fp32 accumulator)``: the routing weight is applied in
    the down-projection epilogue, only the sum happens here.
    """
    n_rows, top_k = recv_weight.shape
    width = expert_out.shape[1]
    slots = torch.zeros(n_rows, top_k, width, dtype=expert_out.dtype, device=expert_out.device)
    present = torch.zeros(n_rows, top_k, dtype=torch.bool, device=expert_out.device)
    slots[layout.entry_row, layout.entry_slot] = expert_out
    present[layout.entry_row, layout.entry_slot] = True
    return _ordered_masked_sum(slots, present).to(out_dtype)


def combine(
    partials: torch.Tensor, plan: DispatchPlan, num_tokens: int, world: int, out_dtype: torch.dtype
) -> torch.Tensor:
    """Per owned token: sum the returned partial rows in ascending destination-rank order."""
    width = partials.shape[1]
    by_rank = torch.zeros(num_tokens, world, width, dtype=torch.float32, device=partials.device)
    present = torch.zeros(num_tokens, world, dtype=torch.bool, device=partials.device)
    by_rank[plan.send_token, plan.send_rank] = partials.to(torch.float32)
    present[plan.send_token, plan.send_rank] = True
    return _ordered_masked_sum(by_rank, present).to(out_dtype)
