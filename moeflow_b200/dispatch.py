"""The local stages of the variable-size ("naive") expert-parallel pipeline; nothing here communicates.

The rules these functions implement (and ``fixed.py`` must reproduce bit for bit on valid rows):

placement    experts live in contiguous blocks, rank r owns ``[r * L, (r + 1) * L)``; tokens stay with the rank
             of their data-parallel shard.
one copy     a token is sent to a destination rank once, however many of its K experts live there.  The row
             carries K slots: the expert id local to the destination (``INVALID`` where the slot belongs to
             another rank) and the routing weight (0 there).
send order   rows are grouped by destination rank; inside a group tokens are in ascending order.
owner sum    the destination adds the (already weighted) expert outputs of a row's local slots in slot order
             0..K-1, in fp32, starting from +0.0, and returns one partial row per received row.
source sum   the source adds a token's partial rows in ascending destination-rank order, again fp32 from +0.0.

A term that is absent is *skipped*, not added as zero: adding +0.0 would turn a -0.0 running sum into +0.0,
and whatever sits in an absent slot must never be read as a number.

Per-destination counts are needed on the host, so this pipeline cannot be captured in a CUDA graph.
Behavioural counterpart of ``moeflow/dispatch.py:21-124`` of the reference (same names).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

INVALID = -1


@dataclass
class DispatchPlan:
    send_token: torch.Tensor     # [S] int64: the local token each send row carries
    send_rank: torch.Tensor      # [S] int64: its destination rank (non-decreasing)
    send_counts: torch.Tensor    # [world] int64: rows per destination
    slot_local_id: torch.Tensor  # [S, K] int32: expert id local to the destination, INVALID elsewhere
    slot_weight: torch.Tensor    # [S, K] fp32: routing weight, 0 where INVALID


def plan_dispatch(topk_ids: torch.Tensor, topk_weights: torch.Tensor, world: int, experts_per_rank: int) -> DispatchPlan:
    tokens, top_k = topk_ids.shape
    expert = topk_ids.to(torch.int64)
    owner = torch.div(expert, experts_per_rank, rounding_mode="floor")
    # Every (token, slot) names a (destination, token) pair; numbering the pairs destination-major and keeping
    # each number once gives the send rows already in their order.
    token_of = torch.arange(tokens, device=expert.device)[:, None].expand(tokens, top_k)
    pair = torch.unique(owner * max(tokens, 1) + token_of)  # sorted ascending
    send_rank = torch.div(pair, max(tokens, 1), rounding_mode="floor")
    send_token = pair - send_rank * max(tokens, 1)
    send_counts = torch.bincount(send_rank, minlength=world)[:world].to(torch.int64)

    lives_there = owner[send_token] == send_rank[:, None]
    local_id = (expert[send_token] - send_rank[:, None] * experts_per_rank).to(torch.int32)
    weight = topk_weights.to(torch.float32)[send_token]
    return DispatchPlan(
        send_token=send_token,
        send_rank=send_rank,
        send_counts=send_counts,
        slot_local_id=local_id.masked_fill(~lives_there, INVALID),
        slot_weight=weight.masked_fill(~lives_there, 0.0),
    )


def pack_send(x: torch.Tensor, plan: DispatchPlan) -> torch.Tensor:
    """The hidden rows in send order."""
    return x.index_select(0, plan.send_token)


@dataclass
class ExpertLayout:
    """Expert-major order of the live (received row, slot) entries on the destination."""

    entry_row: torch.Tensor       # [N] int64
    entry_slot: torch.Tensor      # [N] int64
    expert_offsets: torch.Tensor  # [L + 1] int64: local expert e owns entries [off[e], off[e + 1])


def build_expert_layout(recv_local_id: torch.Tensor, num_local_experts: int) -> ExpertLayout:
    rows, top_k = recv_local_id.shape
    expert = recv_local_id.reshape(-1).to(torch.int64)
    position = torch.arange(rows * top_k, device=expert.device)
    live = expert != INVALID
    # (expert, position) as one number: all keys differ, so a plain sort orders the entries by expert and,
    # inside an expert, by (row, slot); this makes the layout unique without relying on sort stability.
    ordered = torch.sort(expert[live] * max(rows * top_k, 1) + position[live]).values
    ordered_expert = torch.div(ordered, max(rows * top_k, 1), rounding_mode="floor")
    where = ordered - ordered_expert * max(rows * top_k, 1)
    boundaries = torch.arange(num_local_experts + 1, device=expert.device)
    return ExpertLayout(
        entry_row=torch.div(where, top_k, rounding_mode="floor"),
        entry_slot=where % top_k,
        expert_offsets=torch.searchsorted(ordered_expert, boundaries),
    )


def gather_expert_input(recv_x: torch.Tensor, layout: ExpertLayout) -> torch.Tensor:
    """One input row per entry, in expert-major order."""
    return recv_x.index_select(0, layout.entry_row)


def entry_weights(layout: ExpertLayout, recv_weight: torch.Tensor) -> torch.Tensor:
    """fp32 routing weight of every entry, in expert-major order."""
    return recv_weight.to(torch.float32)[layout.entry_row, layout.entry_slot]


def _ordered_masked_sum(values: torch.Tensor, present: torch.Tensor) -> torch.Tensor:
    """``values [N, S, H]``, ``present [N, S]`` -> fp32 ``[N, H]``: terms added in order s = 0..S-1 onto +0.0,
    absent terms skipped."""
    total = torch.zeros(values.shape[0], values.shape[2], dtype=torch.float32, device=values.device)
    for term, there in zip(values.unbind(dim=1), present.unbind(dim=1)):
        total = torch.where(there[:, None], total + term.to(torch.float32), total)
    return total


def _dense_terms(rows: int, steps: int, at_row: torch.Tensor, at_step: torch.Tensor, terms: torch.Tensor):
    """Terms addressed by (row, step) laid out densely as ``[rows, steps, H]`` plus the mask of filled places.
    The dense block is built by a gather through an index table, so unfilled places hold a copy of term 0 (or
    nothing at all when there are no terms) and are masked out."""
    table = torch.full((rows, steps), -1, dtype=torch.int64, device=terms.device)
    table[at_row, at_step] = torch.arange(terms.shape[0], device=terms.device)
    filled = table >= 0
    if terms.shape[0] == 0:
        return terms.new_zeros(rows, steps, terms.shape[1]), filled
    return terms[table.clamp(min=0)], filled


def reduce_local(expert_out: torch.Tensor, layout: ExpertLayout, recv_weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """One partial row per received row.  ``expert_out`` is in expert-major order and already carries the
    routing weight (it is applied to the fp32 accumulator of the down projection, before the single cast), so
    ``recv_weight`` only supplies the shape here."""
    rows, top_k = recv_weight.shape
    terms, filled = _dense_terms(rows, top_k, layout.entry_row, layout.entry_slot, expert_out)
    return _ordered_masked_sum(terms, filled).to(out_dtype)


def combine(partials: torch.Tensor, plan: DispatchPlan, num_tokens: int, world: int, out_dtype: torch.dtype) -> torch.Tensor:
    """The final rows of this rank's tokens from the partial rows that came back (in send order)."""
    terms, filled = _dense_terms(num_tokens, world, plan.send_token, plan.send_rank, partials)
    return _ordered_masked_sum(terms, filled).to(out_dtype)
