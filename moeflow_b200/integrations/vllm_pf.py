"""The variable-size moeflow transport as a vLLM modular-kernel Prepare/Finalize.

vLLM's own fused expert kernels (whatever its oracle picks: Triton, FP8, NVFP4, ...) run unchanged between
``prepare`` and ``finalize``, so an end-to-end comparison against the engine's transports isolates the
communication path.  The data path itself is ``row_transport.VariableRowTransport``; this class only
translates to and from the engine's types: the per-expert row counts become ``ExpertTokensMetadata``, the
received rows are quantised the way the chosen expert kernel asks for, and the expert output is weighted
and reduced per received row with the engine's ``TopKWeightAndReduce`` before it travels home.

Host-synchronising collective transport, so a baseline and not the product path (that is ``MoEFlowRunner``
in ``fixed`` mode).  Not re-entrant, no asynchronous mode.  Importing this module imports vLLM.
Counterpart of ``moeflow/integrations/vllm_pf.py:30-131`` of the reference.
"""

from __future__ import annotations

import torch
import vllm.model_executor.layers.fused_moe.modular_kernel as mk
from vllm.model_executor.layers.fused_moe.topk_weight_and_reduce import (
    TopKWeightAndReduceContiguous,
    TopKWeightAndReduceDelegate,
)
from vllm.model_executor.layers.fused_moe.utils import moe_kernel_quantize_input

from ..comm import CollectiveRowExchange
from .row_transport import VariableRowTransport

# Answers to the engine's capability questions: rows in the standard (non-batched) format, no preferred id
# dtype, no per-rank token ceiling, the output of finalize() is complete (no later reduction), synchronous.
_CAPABILITIES = {"topk_indices_dtype": None, "max_num_tokens_per_rank": None, "output_is_reduced": True,
                 "supports_async": False}


def _quantise_for_experts(rows: torch.Tensor, quant_config, defer: bool):
    """Activation quantisation the expert kernel expects of its Prepare step (none for bf16 kernels)."""
    if quant_config.quant_dtype is None or defer or rows.numel() == 0:
        return rows, None
    return moe_kernel_quantize_input(rows, quant_config.a1_scale, quant_dtype=quant_config.quant_dtype,
                                     per_act_token_quant=quant_config.per_act_token_quant,
                                     block_shape=quant_config.block_shape)


class MoEFlowPrepareAndFinalize(mk.FusedMoEPrepareAndFinalizeModular):
    def __init__(self, ep_group: torch.distributed.ProcessGroup, num_local_experts: int, comm=None):
        super().__init__()
        self.comm = CollectiveRowExchange(ep_group) if comm is None else comm
        self.transport = VariableRowTransport(self.comm, num_local_experts)
        self.num_local_experts = num_local_experts
        self.rank_expert_offset = self.transport.first_expert

    # ---- capability questions ----------------------------------------------------------------------
    @property
    def activation_format(self):
        return mk.FusedMoEActivationFormat.Standard

    def num_dispatchers(self) -> int:
        return self.comm.world

    def topk_indices_dtype(self):
        return _CAPABILITIES["topk_indices_dtype"]

    def max_num_tokens_per_rank(self):
        return _CAPABILITIES["max_num_tokens_per_rank"]

    def output_is_reduced(self) -> bool:
        return _CAPABILITIES["output_is_reduced"]

    def supports_async(self) -> bool:
        return _CAPABILITIES["supports_async"]

    # ---- data path -----------------------------------------------------------------------------------
    def prepare(self, a1, topk_weights, topk_ids, num_experts, expert_map, apply_router_weight_on_input,
                quant_config, defer_input_quant=False):
        if apply_router_weight_on_input:
            raise NotImplementedError("moeflow applies router weights after the experts")
        got = self.transport.scatter(a1, topk_weights, topk_ids, num_experts)
        rows, scale = _quantise_for_experts(got.hidden, quant_config, defer_input_quant)
        counts = mk.ExpertTokensMetadata(expert_num_tokens=got.rows_per_local_expert, expert_num_tokens_cpu=None)
        return rows, scale, counts, got.expert_ids, got.weights

    def finalize(self, output, fused_expert_output, topk_weights, topk_ids, apply_router_weight_on_input,
                 weight_and_reduce_impl) -> None:
        if not self.transport.busy:
            raise RuntimeError("finalize() without a matching prepare()")
        if fused_expert_output.numel() == 0:
            per_row = fused_expert_output.new_empty((0, output.shape[-1]))
        else:
            reducer = weight_and_reduce_impl
            if isinstance(reducer, TopKWeightAndReduceDelegate):  # "ask the Prepare/Finalize": plain contiguous sum
                reducer = TopKWeightAndReduceContiguous()
            per_row = reducer.apply(output=None, fused_expert_output=fused_expert_output, topk_weights=topk_weights,
                                    topk_ids=topk_ids, apply_router_weight_on_input=apply_router_weight_on_input)
        output.copy_(self.transport.gather(per_row, output.dtype))
