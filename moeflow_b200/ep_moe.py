"""Variable-size expert-parallel pipeline (the "naive" arm): every rank sends exactly the rows its tokens
need, so the row counts differ per step and travel over a count-then-rows exchange.

    route -> pack rows by destination -> exchange -> expert-major layout -> experts
          -> slot-ordered reduce per received row -> exchange back -> merge per token

One driver (``_pipeline``) walks these steps for a list of ranks.  What differs between a real SPMD run and
the in-process simulation is only the *wire* that carries rows between ranks: ``_TransportWire`` moves one
rank's rows through a ``RowExchange`` (NCCL / gloo), ``_LoopbackWire`` swaps the rows of all ranks held in one
process.  That is how the dispatch and combine logic is tested without GPUs.  Behavioural counterpart of
``moeflow/ep_moe.py:30-102`` of the reference (same class, method and function names).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from . import dispatch as D
from .comm import RowExchange, pack_meta, simulated_exchange, unpack_meta
from .config import MoEConfig
from .experts import ExpertCompute, TorchLoopExperts
from .router import route


@dataclass
class DispatchState:
    """What the source side keeps between dispatch and combine."""

    plan: D.DispatchPlan
    send_x: torch.Tensor
    send_meta: torch.Tensor
    num_tokens: int


class EPMoELayer:
    """One EP rank's expert shard (``w13 [L, 2I, H]``, ``w2 [L, H, I]``) and the three local stages."""

    def __init__(
        self,
        cfg: MoEConfig,
        rank: int,
        world: int,
        w13_local: torch.Tensor,
        w2_local: torch.Tensor,
        experts: ExpertCompute | None = None,
        combine_dtype: torch.dtype = torch.bfloat16,
    ):
        owned = cfg.experts_per_rank(world)
        for name, w in (("w13", w13_local), ("w2", w2_local)):
            if w.shape[0] != owned:
                raise ValueError(f"{name} shard holds {w.shape[0]} experts, this rank owns {owned}")
        self.cfg, self.rank, self.world, self.num_local = cfg, rank, world, owned
        self.w13, self.w2 = w13_local, w2_local
        self.experts: ExpertCompute = TorchLoopExperts() if experts is None else experts
        #: dtype of the partial rows that travel back (bf16: half the bytes; fp32: exact transport)
        self.combine_dtype = combine_dtype

    # ---- local stages ------------------------------------------------------------------------------
    def stage_dispatch(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> DispatchState:
        """Source side: one row per (token, destination rank) with its per-slot metadata."""
        plan = D.plan_dispatch(topk_ids, topk_weights, self.world, self.num_local)
        rows = D.pack_send(x, plan)
        return DispatchState(plan=plan, send_x=rows, send_meta=pack_meta(plan.slot_local_id, plan.slot_weight),
                             num_tokens=int(x.shape[0]))

    def stage_experts(self, recv_x: torch.Tensor, recv_meta: torch.Tensor) -> torch.Tensor:
        """Owner side: received rows -> one partial row each (its local slots summed in slot order)."""
        slot_expert, slot_weight = unpack_meta(recv_meta)
        layout = D.build_expert_layout(slot_expert, self.num_local)
        per_entry = self.experts(
            D.gather_expert_input(recv_x, layout),
            layout.expert_offsets,
            self.w13,
            self.w2,
            self.cfg.swiglu_limit,
            D.entry_weights(layout, slot_weight),
        )
        return D.reduce_local(per_entry, layout, slot_weight, self.combine_dtype)

    def stage_combine(self, partials: torch.Tensor, state: DispatchState, out_dtype: torch.dtype) -> torch.Tensor:
        """Source side again: merge the returned partial rows of every token."""
        return D.combine(partials, state.plan, state.num_tokens, self.world, out_dtype)

    # ---- SPMD entry points ---------------------------------------------------------------------------
    def forward(self, x, router_logits, bias, comm: RowExchange) -> torch.Tensor:
        return self.forward_routed(x, *route(router_logits, bias, self.cfg), comm)

    def forward_routed(self, x, topk_weights, topk_ids, comm: RowExchange) -> torch.Tensor:
        return _pipeline([self], [x], [(topk_weights, topk_ids)], _TransportWire(comm))[0]


class _TransportWire:
    """Carries the rows of the one local rank through a real ``RowExchange``."""

    def __init__(self, comm: RowExchange):
        self.comm = comm

    def forward(self, states: Sequence[DispatchState]):
        (st,) = states
        out_counts = st.plan.send_counts
        in_counts = self.comm.exchange_counts(out_counts)
        rows = self.comm.exchange(st.send_x, out_counts, in_counts)
        meta = self.comm.exchange(st.send_meta, out_counts, in_counts)
        return [rows], [meta], [in_counts]

    def backward(self, partials: Sequence[torch.Tensor], in_counts, states: Sequence[DispatchState]):
        return [self.comm.exchange(partials[0], in_counts[0], states[0].plan.send_counts)]


class _LoopbackWire:
    """Swaps the rows of all ranks inside one process."""

    def forward(self, states: Sequence[DispatchState]):
        out_counts = [st.plan.send_counts for st in states]
        rows, in_counts = simulated_exchange([st.send_x for st in states], out_counts)
        meta, _ = simulated_exchange([st.send_meta for st in states], out_counts)
        return rows, meta, in_counts

    def backward(self, partials: Sequence[torch.Tensor], in_counts, states: Sequence[DispatchState]):
        return simulated_exchange(list(partials), list(in_counts))[0]


def _pipeline(layers: Sequence[EPMoELayer], xs: Sequence[torch.Tensor], routed, wire) -> list[torch.Tensor]:
    states = [layer.stage_dispatch(x, w, ids) for layer, x, (w, ids) in zip(layers, xs, routed)]
    rows, meta, in_counts = wire.forward(states)
    partials = [layer.stage_experts(r, m) for layer, r, m in zip(layers, rows, meta)]
    returned = wire.backward(partials, in_counts, states)
    return [layer.stage_combine(back, st, x.dtype) for layer, back, st, x in zip(layers, returned, states, xs)]


def simulate_ep(layers: list[EPMoELayer], xs, logits, bias) -> list[torch.Tensor]:
    """All ranks in lock-step inside one process (``layers[r]`` is rank r)."""
    cfg = layers[0].cfg
    return _pipeline(layers, xs, [route(lg, bias, cfg) for lg in logits], _LoopbackWire())


def shard_experts(w13: torch.Tensor, w2: torch.Tensor, rank: int, world: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Contiguous placement: rank r owns experts ``[r * L, (r + 1) * L)`` with ``L = E / world``."""
    if w13.shape[0] % world or w13.shape[0] != w2.shape[0]:
        raise ValueError("the expert count must be the same for both weights and divisible by the world size")
    return w13.chunk(world, dim=0)[rank], w2.chunk(world, dim=0)[rank]
