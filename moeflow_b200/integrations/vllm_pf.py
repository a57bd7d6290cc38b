"""The variable-size moeflow transport as a vLLM modular-kernel Prepare/Finalize.

vLLM's own fused expert kernels (chosen by its oracle: Triton, FP8, NVFP4, ...) run unchanged between
``prepare`` and ``finalize``, so an end-to-end comparison isolates the communication path.  The top-k
ids handed to the experts follow the convention of vLLM's high-throughput all-to-all: one row per
(token, destination rank), local hits mapped back to global ids, empty slots pointed at an expert
this rank does not own so that the expert map turns them into "skip".

This class uses the host-synchronising collective transport (``CollectiveRowExchange``), so it is a
baseline, not the product path; the product path is ``MoEFlowRunner`` in ``fixed`` mode.
Not re-entrant (one call in flight), no asynchronous mode.  Importing this module imports vLLM.
Counterpart of ``moeflow/integrations/vllm_pf.py:30-131``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import vllm.model_executor.layers.fused_moe.modular_kernel as mk
from vllm.model_executor.layers.fused_moe.topk_weight_and_reduce import (
    TopKWeightAndReduceContiguous,
    TopKWeightAndReduceDelegate,
)
from vllm.model_executor.layers.fused_moe.utils import moe_kernel_quantize_input

from .. import dispatch as D
from ..comm import CollectiveRowExchange, pack_meta, unpack_meta
from .vllm_runner_ops import filler_expert


@dataclass
class _InFlight:
    plan: D.DispatchPlan
    recv_counts: torch.Tensor
    num_tokens: int


class MoEFlowPrepareAndFinalize(mk.FusedMoEPrepareAndFinalizeModular):
    def __init__(self, ep_group: torch.distributed.ProcessGroup, num_local_experts: int, comm=None):
        super().__init__()
        self.comm = comm if comm is not None else CollectiveRowExchange(ep_group)
        self.num_local_experts = num_local_experts
        self.rank_expert_offset = self.comm.rank * num_local_experts
        self._inflight: _InFlight | None = None

    @property
    def activation_format(self):
        return mk.FusedMoEActivationFormat.Standard

    def topk_indices_dtype(self):
        return None

    def max_num_tokens_per_rank(self):
        return None

    def num_dispatchers(self) -> int:
        return self.comm.world

    def output_is_reduced(self) -> bool:
        return True

    def supports_async(self) -> bool:
        return False

    def prepare(self, a1, topk_weights, topk_ids, num_experts, expert_map, apply_router_weight_on_input,
                quant_config, defer_input_quant=False):
        if apply_router_weight_on_input:
            raise NotImplementedError("moeflow applies router weights after the experts")
        if self._inflight is not None:
            raise RuntimeError("prepare() called again before finalize(): this transport is not re-entrant")
        plan = D.plan_dispatch(topk_ids, topk_weights, self.comm.world, self.num_local_experts)
        recv_counts = self.comm.exchange_counts(plan.send_counts)
        recv_x = self.comm.exchange(D.pack_send(a1, plan), plan.send_counts, recv_counts)
        recv_meta = self.comm.exchange(pack_meta(plan.slot_local_id, plan.slot_weight), plan.send_counts, recv_counts)
        self._inflight = _InFlight(plan, recv_counts, a1.shape[0])

        local_id, weight = unpack_meta(recv_meta)
        empty = local_id == D.INVALID
        filler = filler_expert(self.rank_expert_offset, num_experts)
        global_ids = torch.where(empty, filler, local_id + self.rank_expert_offset).to(topk_ids.dtype)
        counts = torch.bincount(local_id[~empty].to(torch.int64), minlength=self.num_local_experts).to(torch.int32)
        tokens_meta = mk.ExpertTokensMetadata(expert_num_tokens=counts, expert_num_tokens_cpu=None)

        scale = None
        if quant_config.quant_dtype is not None and not defer_input_quant and recv_x.numel():
            recv_x, scale = moe_kernel_quantize_input(
                recv_x, quant_config.a1_scale, quant_dtype=quant_config.quant_dtype,
                per_act_token_quant=quant_config.per_act_token_quant, block_shape=quant_config.block_shape,
            )
        return recv_x, scale, tokens_meta, global_ids, weight

    def finalize(self, output, fused_expert_output, topk_weights, topk_ids, apply_router_weight_on_input,
                 weight_and_reduce_impl) -> None:
        state, self._inflight = self._inflight, None
        if state is None:
            raise RuntimeError("finalize() without a matching prepare()")
        if fused_expert_output.numel():
            if isinstance(weight_and_reduce_impl, TopKWeightAndReduceDelegate):
                weight_and_reduce_impl = TopKWeightAndReduceContiguous()
            partial = weight_and_reduce_impl.apply(
                output=None, fused_expert_output=fused_expert_output, topk_weights=topk_weights, topk_ids=topk_ids,
                apply_router_weight_on_input=apply_router_weight_on_input,
            )
        else:
            partial = fused_expert_output.new_empty((0, output.shape[-1]))
        back = self.comm.exchange(partial.to(torch.bfloat16), state.recv_counts, state.plan.send_counts)
        output.copy_(D.combine(back, state.plan, state.num_tokens, self.comm.world, output.dtype))
