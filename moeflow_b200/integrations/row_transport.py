"""The variable-size row transport behind the engine-facing Prepare/Finalize, free of any engine import.

``scatter`` sends every token's row to the ranks that own one of its experts and hands back what this rank
received, already in the form an expert kernel with an expert map wants: global expert ids per slot (slots
that are not for this rank point at a *filler* expert this rank does not own, with weight 0) and the number
of rows per local expert.  ``gather`` takes one partial row per received row, sends it home and merges the
partials of every token in ascending rank order.

Keeping this apart from the engine adapter (``vllm_pf.MoEFlowPrepareAndFinalize``) means the data path runs
under test on CPU ranks (gloo) or with a loop-back exchange.  One call may be in flight at a time.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import dispatch as D
from ..comm import RowExchange, pack_meta, unpack_meta
from .vllm_runner_ops import filler_expert


@dataclass(frozen=True)
class ReceivedRows:
    hidden: torch.Tensor          # [S, H] rows this rank received, grouped by source rank
    expert_ids: torch.Tensor      # [S, K] global ids; the filler expert where a slot is not for this rank
    weights: torch.Tensor         # [S, K] fp32 routing weights; 0 where the slot is not for this rank
    rows_per_local_expert: torch.Tensor  # [L] int32


class VariableRowTransport:
    def __init__(self, comm: RowExchange, num_local_experts: int):
        self.comm = comm
        self.num_local_experts = num_local_experts
        self.first_expert = comm.rank * num_local_experts
        self._pending: tuple[D.DispatchPlan, torch.Tensor, int] | None = None

    @property
    def busy(self) -> bool:
        return self._pending is not None

    def scatter(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, num_experts: int,
                ids_dtype: torch.dtype | None = None) -> ReceivedRows:
        if self.busy:
            raise RuntimeError("scatter() called again before gather(): this transport is not re-entrant")
        plan = D.plan_dispatch(topk_ids, topk_weights, self.comm.world, self.num_local_experts)
        arriving = self.comm.exchange_counts(plan.send_counts)

        def ship(rows: torch.Tensor) -> torch.Tensor:
            return self.comm.exchange(rows, plan.send_counts, arriving)

        hidden = ship(D.pack_send(x, plan))
        slot_expert, slot_weight = unpack_meta(ship(pack_meta(plan.slot_local_id, plan.slot_weight)))
        self._pending = (plan, arriving, int(x.shape[0]))

        mine = slot_expert != D.INVALID
        elsewhere = filler_expert(self.first_expert, num_experts)
        ids = torch.where(mine, slot_expert + self.first_expert, elsewhere).to(ids_dtype or topk_ids.dtype)
        per_expert = torch.zeros(self.num_local_experts, dtype=torch.int32, device=slot_expert.device)
        per_expert.scatter_add_(0, slot_expert[mine].to(torch.int64), torch.ones_like(slot_expert[mine], dtype=torch.int32))
        return ReceivedRows(hidden, ids, slot_weight, per_expert)

    def gather(self, partial_rows: torch.Tensor, out_dtype: torch.dtype, wire_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        if not self.busy:
            raise RuntimeError("gather() without a matching scatter()")
        (plan, arrived, tokens), self._pending = self._pending, None
        home = self.comm.exchange(partial_rows.to(wire_dtype), arrived, plan.send_counts)
        return D.combine(home, plan, tokens, self.comm.world, out_dtype)
