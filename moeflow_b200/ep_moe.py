"""Variable-size expert-parallel pipeline: route -> rank-packed dispatch -> exchange ->
expert-major layout -> experts -> slot-ordered local reduce -> exchange back -> combine.

Every stage but the exchanges is local, so the same stage code runs over a real transport
(``EPMoELayer.forward``) or inside one process for all ranks (``simulate_ep``) — that is how the
dispatch/combine logic is tested without GPUs.  Behavioural counterpart of ``moeflow/ep_moe.py:30-102``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import dispatch as D
from .comm import RowExchange, pack_meta, simulated_exchange, unpack_meta
from .config import MoEConfig
from .experts import ExpertCompute, TorchLoopExperts
from .router import route


@dataclass
class DispatchState:
    plan: D.DispatchPlan
    send_x: torch.Tensor
    send_meta: torch.Tensor
    num_tokens: int


class EPMoELayer:
    """The local expert shard of one EP rank: ``w13 [L, 2I, H]``, ``w2 [L, H, I]``."""

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
        self.cfg, self.rank, self.world = cfg, rank, world
        self.num_local = cfg.experts_per_rank(world)
        if w13_local.shape[0] != self.num_local or w2_local.shape[0] != self.num_local:
            raise ValueError("weight shard does not hold experts_per_rank experts")
        self.w13, self.w2 = w13_local, w2_local
        self.experts = experts if experts is not None else TorchLoopExperts()
        # dtype of the partial rows on the way back (bf16 halves the bytes, fp32 is exact transport)
        self.combine_dtype = combine_dtype

    def stage_dispatch(self, x, topk_weights, topk_ids) -> DispatchState:
        plan = D.plan_dispatch(topk_ids, topk_weights, self.world, self.num_local)
        meta = pack_meta(plan.slot_local_id, plan.slot_weight)
        return DispatchState(plan, D.pack_send(x, plan), meta, x.shape[0])

    def stage_experts(self, recv_x: torch.Tensor, recv_meta: torch.Tensor) -> torch.Tensor:
        local_id, weight = unpack_meta(recv_meta)
        layout = D.build_expert_layout(local_id, self.num_local)
        rows = D.gather_expert_input(recv_x, layout)
        y = self.experts(
            rows, layout.expert_offsets, self.w13, self.w2, self.cfg.swiglu_limit, D.entry_weights(layout, weight)
        )
        return D.reduce_local(y, layout, weight, self.combine_dtype)

    def stage_combine(self, partials, state: DispatchState, out_dtype) -> torch.Tensor:
        return D.combine(partials, state.plan, state.num_tokens, self.world, out_dtype)

    def forward(self, x, router_logits, bias, comm: RowExchange) -> torch.Tensor:
        weights, ids = route(router_logits, bias, self.cfg)
        return self.forward_routed(x, weights, ids, comm)

    def forward_routed(self, x, topk_weights, topk_ids, comm: RowExchange) -> torch.Tensor:
        st = self.stage_dispatch(x, topk_weights, topk_ids)
        recv_counts = comm.exchange_counts(st.plan.send_counts)
        recv_x = comm.exchange(st.send_x, st.plan.send_counts, recv_counts)
        recv_meta = comm.exchange(st.send_meta, st.plan.send_counts, recv_counts)
        partials = self.stage_experts(recv_x, recv_meta)
        back = comm.exchange(partials, recv_counts, st.plan.send_counts)
        return self.stage_combine(back, st, x.dtype)


def simulate_ep(layers: list[EPMoELayer], xs, logits, bias) -> list[torch.Tensor]:
    """All ranks in lock-step inside one process."""
    cfg = layers[0].cfg
    states = []
    for layer, x, lg in zip(layers, xs, logits):
        w, ids = route(lg, bias, cfg)
        states.append(layer.stage_dispatch(x, w, ids))
    counts = [s.plan.send_counts for s in states]
    recv_x, recv_counts = simulated_exchange([s.send_x for s in states], counts)
    recv_meta, _ = simulated_exchange([s.send_meta for s in states], counts)
    partials = [layer.stage_experts(rx, rm) for layer, rx, rm in zip(layers, recv_x, recv_meta)]
    back, _ = simulated_exchange(partials, recv_counts)
    return [layer.stage_combine(b, s, x.dtype) for layer, b, s, x in zip(layers, back, states, xs)]


def shard_experts(w13: torch.Tensor, w2: torch.Tensor, rank: int, world: int):
    """Contiguous placement: rank r owns experts ``[r*L, (r+1)*L)``."""
    per = w13.shape[0] // world
    lo = rank * per
    return w13[lo : lo + per], w2[lo : lo + per]
