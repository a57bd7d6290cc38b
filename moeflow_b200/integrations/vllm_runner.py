"""``MoEFlowRunner``: a vLLM ``MoERunner`` subclass that routes decode steps through ``FixedEPLayer``.

Modes (``MOEFLOW_MODE``):

``route_check`` (default; a smoke test): the project's router replaces vLLM's and is cross-checked
    against it on the first calls of every layer, then vLLM's own modular kernel runs (its dispatch and
    combine included).

``fixed``: expert-parallel execution through the fixed-capacity, CUDA-graph-capturable layer while the
    largest per-DP-rank token count of the step is at most ``MOEFLOW_MAX_TOKENS``; the capacity is the
    next power of two.  Larger steps (prefill) are handed to vLLM's native runner as a whole, routing
    included, and monolithic expert kernels are never intercepted.  The decision uses the host-side
    ``num_tokens_across_dp_cpu`` that is identical on all ranks, so every rank takes the same branch.

    Experts (``MOEFLOW_EXPERTS``): ``native`` runs the layer's bf16 weights through the tcgen05 grouped
    GEMMs of this package, fully fused with dispatch and return; ``vllm`` runs this layer's own vLLM
    fused-experts object (FP8 or BF16) between the fused dispatch and the return push; ``auto`` picks
    ``native`` when the layer's weights are bf16 of a supported shape.

One ``FixedEPLayer`` (communication buffers, metadata, scratch) is shared by all compatible MoE layers
of the process, keyed by ``(cfg, rank, world, capacity, device, group, fused_dispatch)``: layers run one
at a time.  The logic lives in ``RunnerCore`` so that it can be unit-tested with stand-ins; the class
``MoEFlowRunner`` that derives from vLLM's ``MoERunner`` is created on first access.
Counterpart of ``moeflow/integrations/vllm_runner.py:29-320``.
"""

from __future__ import annotations

import json
import os

import torch

from ..config import MoEConfig
from ..router import route
from ..utils.env import RunnerSettings
from .vllm_runner_ops import (
    compare_routing,
    fixed_capacity,
    local_to_global_ids,
    make_combine_fn,
    make_prepare_fn,
)

MAX_LOGGED_CALLS_PER_LAYER = 8
MAX_TRACED_CALLS = 32
MAX_TRACED_TOKENS = 128
_BUFFER_POOL: dict = {}


def shared_fixed_layer(cfg: MoEConfig, rank: int, world: int, capacity: int, device, group, fused_dispatch=False,
                       backend: str | None = None):
    """The process-wide buffer set for this (shape, rank, capacity); created on first use."""
    from ..fixed import FixedEPLayer

    key = (cfg, rank, world, capacity, str(device), group, fused_dispatch)
    layer = _BUFFER_POOL.get(key)
    if layer is None:
        layer = FixedEPLayer(cfg, rank, world, None, None, capacity=capacity, group=group, device=device,
                             fused_dispatch=fused_dispatch, backend=backend)
        _BUFFER_POOL[key] = layer
    return layer


def cfg_from_hf_text_config(hf) -> MoEConfig:
    return MoEConfig(
        hidden_size=hf.hidden_size,
        moe_intermediate_size=hf.moe_intermediate_size,
        n_routed_experts=hf.n_routed_experts,
        n_shared_experts=getattr(hf, "n_shared_experts", 0) or 0,
        top_k=hf.num_experts_per_tok,
        n_group=getattr(hf, "n_group", 1) or 1,
        topk_group=getattr(hf, "topk_group", 1) or 1,
        norm_topk_prob=bool(getattr(hf, "norm_topk_prob", True)),
        routed_scaling_factor=float(getattr(hf, "routed_scaling_factor", 1.0) or 1.0),
        # GLM-4-MoE configurations do not spell these out; the family routes with sigmoid scores and a
        # selection bias
        scoring_func=getattr(hf, "scoring_func", "sigmoid"),
        topk_method=getattr(hf, "topk_method", "noaux_tc"),
        swiglu_limit=getattr(hf, "swiglu_limit", None),
    )


class RunnerCore:
    """MoEFlow behaviour of the runner, independent of vLLM's base class.

    The host class provides vLLM's runner attributes: ``routed_experts``, ``router``, ``gate``,
    ``_quant_method``, ``_shared_experts``, ``layer_name``, ``_maybe_apply_shared_experts`` and the native
    ``_apply_quant_method`` reachable through ``_native_apply``.
    """

    _moeflow_runner = True

    def _moeflow_setup(self, cfg: MoEConfig, settings: RunnerSettings | None = None) -> None:
        self.moeflow_cfg = cfg
        self.moeflow = settings if settings is not None else RunnerSettings.from_env()
        # attribute names of the reference, kept for scripts that read them
        self.moeflow_mode = self.moeflow.mode
        self.moeflow_max_tokens = self.moeflow.max_tokens
        self.moeflow_combine_mode = self.moeflow.combine_mode
        self._moeflow_calls = 0
        self._moeflow_fixed_calls = 0
        self._routing_trace_calls = 0
        self._local_kernel = None
        self._router_takes_dtype = None
        self._native_tmaps = None
        self._fixed_probe = None
        if self.moeflow.validate_fixed:
            from .vllm_diagnostics import FixedLayerProbe

            self._fixed_probe = FixedLayerProbe(self.moeflow.routing_trace_dir)
        log_dir = self.moeflow.smoke_dir
        self._moeflow_log = log_dir / f"runner_pid{os.getpid()}.jsonl" if log_dir else None

    # ---- logging -------------------------------------------------------------------------------
    def _record(self, entry: dict) -> None:
        calls = self._moeflow_fixed_calls if entry.get("mode") == "fixed" else self._moeflow_calls
        if self._moeflow_log is None or calls > MAX_LOGGED_CALLS_PER_LAYER:
            return
        entry.update(layer=getattr(self, "layer_name", None), call=self._moeflow_calls)
        self._moeflow_log.parent.mkdir(parents=True, exist_ok=True)
        with open(self._moeflow_log, "a") as sink:
            sink.write(json.dumps(entry) + "\n")

    def _ep(self):
        from vllm.distributed import get_ep_group

        return get_ep_group()

    def _forward_context(self):
        from vllm.forward_context import get_forward_context

        return get_forward_context()

    def _record_routing_trace(self, ids: torch.Tensor, weights: torch.Tensor) -> None:
        """Sample real eager requests, only after the launcher switched collection on."""
        directory = self.moeflow.routing_trace_dir
        if directory is None or self._routing_trace_calls >= MAX_TRACED_CALLS or not (directory / "enabled").is_file():
            return
        if ids.shape[0] == 0 or (ids.is_cuda and torch.cuda.is_current_stream_capturing()):
            return
        group = self._ep()
        rows = ids.shape[0]
        padding = self._forward_context().is_padding
        if padding is not None:
            if tuple(padding.shape) != (rows,):
                raise ValueError("Routing trace padding mask does not match local rows")
            ids, weights = ids[~padding], weights[~padding]
        kept = min(ids.shape[0], MAX_TRACED_TOKENS)
        line = {
            "layer": getattr(self, "layer_name", None),
            "call": self._moeflow_calls,
            "mode": self.moeflow.mode,
            "ep_rank": group.rank_in_group,
            "world": group.world_size,
            "execution_rows": rows,
            "padding_known": padding is not None,
            "tokens": int(ids.shape[0]),
            "tokens_recorded": kept,
            "expert_ids": ids[:kept].detach().cpu().tolist(),
            "weights": weights[:kept].detach().float().cpu().tolist(),
        }
        with (directory / f"routes_pid{os.getpid()}.jsonl").open("a") as sink:
            sink.write(json.dumps(line) + "\n")
        self._routing_trace_calls += 1

    # ---- path decision ---------------------------------------------------------------------------
    def _fixed_capacity(self, local_tokens: int) -> int | None:
        dp = self._forward_context().dp_metadata
        across = dp.num_tokens_across_dp_cpu if dp is not None else None
        return fixed_capacity(local_tokens, None if across is None else across.tolist(), self.moeflow.max_tokens)

    def _is_monolithic(self) -> bool:
        method = getattr(self.routed_experts, "quant_method", None) or self._quant_method
        return bool(method.is_monolithic)

    def _select_experts(self, hidden_states, router_logits, input_ids):
        """The engine's own router.  Engines differ in whether ``select_experts`` takes the id dtype."""
        import inspect

        dtype = self._quant_method.topk_indices_dtype
        if self._router_takes_dtype is None:
            try:
                params = inspect.signature(self.router.select_experts).parameters
                self._router_takes_dtype = "topk_indices_dtype" in params or any(
                    p.kind is p.VAR_KEYWORD for p in params.values())
            except (TypeError, ValueError):
                self._router_takes_dtype = True
        if self._router_takes_dtype:
            return self.router.select_experts(hidden_states=hidden_states, router_logits=router_logits,
                                              topk_indices_dtype=dtype, input_ids=input_ids)
        weights, ids = self.router.select_experts(hidden_states=hidden_states, router_logits=router_logits,
                                                  input_ids=input_ids)
        return weights, (ids if dtype is None else ids.to(dtype))

    def _run_modular(self, hidden_states, weights, ids, shared_experts_input):
        """The engine's modular expert path with routing already decided."""
        experts = self.routed_experts
        if hasattr(experts, "forward_modular"):
            return experts.forward_modular(x=hidden_states, topk_weights=weights, topk_ids=ids,
                                           shared_experts=self._shared_experts, shared_experts_input=shared_experts_input)
        return self._quant_method.apply(layer=experts, x=hidden_states, topk_weights=weights, topk_ids=ids,
                                        shared_experts=self._shared_experts, shared_experts_input=shared_experts_input)

    def _late_shared_experts(self) -> None:
        """Hook for engines that run the shared experts after the routed ones on a second stream."""

    def _apply_quant_method(self, hidden_states, router_logits, shared_experts_input, input_ids=None,
                            shared_experts_overlapping=False):
        self._moeflow_calls += 1
        monolithic = self._is_monolithic()
        if self.moeflow.mode == "fixed" and not monolithic:
            cap = self._fixed_capacity(hidden_states.shape[0])
            if cap is not None:
                return self._apply_fixed(hidden_states, router_logits, shared_experts_input, input_ids,
                                         shared_experts_overlapping, cap)
        if self.moeflow.mode == "fixed" or monolithic:
            # the fixed mode declines large prefills as a whole, routing included
            self._record({"intercepted": False, "reason": "monolithic expert kernel" if monolithic else "fixed token limit"})
            return self._native_apply(hidden_states, router_logits, shared_experts_input, input_ids,
                                      shared_experts_overlapping)
        return self._apply_route_check(hidden_states, router_logits, shared_experts_input, input_ids,
                                       shared_experts_overlapping)

    def _shared_output(self, overlapping: bool, routed_out):
        if overlapping:
            self._shared_experts.wait()
        else:
            self._late_shared_experts()
        shared = self._shared_experts.output if self._shared_experts is not None else None
        return shared, routed_out

    # ---- route_check -----------------------------------------------------------------------------
    def _apply_route_check(self, hidden_states, router_logits, shared_experts_input, input_ids, overlapping):
        self._maybe_apply_shared_experts(shared_experts_input, _no_overlap_order())
        gate = getattr(self, "gate", None)
        bias = getattr(gate, "e_score_correction_bias", None) if gate is not None else None
        weights, ids = route(router_logits, bias, self.moeflow_cfg)
        self._record_routing_trace(ids, weights)
        if self._moeflow_log is not None and self._moeflow_calls <= MAX_LOGGED_CALLS_PER_LAYER:
            v_w, v_ids = self._select_experts(hidden_states, router_logits, input_ids)
            self._record(compare_routing(ids, weights, v_ids, v_w))
        ids = ids.to(self._quant_method.topk_indices_dtype or torch.int32)
        out = self._run_modular(hidden_states, weights, ids, shared_experts_input)
        return self._shared_output(overlapping, out)

    # ---- fixed -------------------------------------------------------------------------------------
    def _local_experts_kernel(self):
        """This layer's own fused experts behind a Prepare/Finalize that does no communication."""
        if self._local_kernel is None:
            import vllm.model_executor.layers.fused_moe.modular_kernel as mk
            from vllm.model_executor.layers.fused_moe.prepare_finalize.no_dp_ep import (
                MoEPrepareAndFinalizeNoDPEPModular,
            )

            experts = self._quant_method.moe_kernel.fused_experts
            self._local_kernel = mk.FusedMoEKernel(MoEPrepareAndFinalizeNoDPEPModular(), experts)
        return self._local_kernel

    def _use_native_experts(self, layer) -> str | None:
        """Which of this framework's own expert kernels can run the layer's weights: ``"bf16"``, ``"fp8"`` (e4m3
        weights with one fp32 ``weight_scale_inv`` per 128x128 block, the GLM-5.3-Flash FP8 checkpoint layout:
        activations are quantised per 1x128 group on the device) or None (the engine's fused experts run)."""
        choice = self.moeflow.experts
        if choice == "vllm" or layer.backend != "cuda":
            return None
        experts = self.routed_experts
        w13 = getattr(experts, "w13_weight", None)
        w2 = getattr(experts, "w2_weight", None)
        shapes = (
            w13 is not None and w2 is not None
            and tuple(w13.shape) == (layer.L, 2 * layer.I, layer.H) and tuple(w2.shape) == (layer.L, layer.H, layer.I)
        )
        kind = None
        if shapes and w13.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16:
            kind = "bf16"
        elif shapes and w13.dtype == torch.float8_e4m3fn and w2.dtype == torch.float8_e4m3fn:
            s13 = getattr(experts, "w13_weight_scale_inv", None)
            s2 = getattr(experts, "w2_weight_scale_inv", None)
            if (
                s13 is not None and s2 is not None and layer.H <= 4096 and layer.I <= 4096
                and tuple(s13.shape) == (layer.L, 2 * layer.I // 128, layer.H // 128)
                and tuple(s2.shape) == (layer.L, layer.H // 128, layer.I // 128)
            ):
                kind = "fp8"
        if choice == "native" and kind is None:
            raise ValueError("MOEFLOW_EXPERTS=native needs bf16 expert weights w13 [L, 2I, H] / w2 [L, H, I], or e4m3 "
                             "weights of those shapes with fp32 weight_scale_inv per 128x128 block")
        return kind

    def _apply_fixed(self, hidden_states, router_logits, shared_experts_input, input_ids, overlapping, capacity):
        self._moeflow_fixed_calls += 1
        self._maybe_apply_shared_experts(shared_experts_input, _no_overlap_order())
        weights, ids = self._select_experts(hidden_states, router_logits, input_ids)
        self._record_routing_trace(ids, weights)
        group = self._ep()
        layer = shared_fixed_layer(self.moeflow_cfg, group.rank_in_group, group.world_size, capacity,
                                   hidden_states.device, group.device_group, fused_dispatch=self.moeflow.fused_dispatch)
        experts = self.routed_experts
        offset = group.rank_in_group * layer.L
        if self.moeflow.combine_mode != "fp32" and hidden_states.dtype != torch.bfloat16:
            raise ValueError("BF16 Ring compatibility requires BF16 hidden states")
        combine_fn = make_combine_fn(self.moeflow.combine_mode, group.rank_in_group)
        native = self._use_native_experts(layer)
        if native == "fp8":
            # the block-scaled e4m3 weights stay as the engine loaded them; descriptors are built once per MoE layer
            if self._native_tmaps is None:
                self._native_tmaps = layer.make_fp8_pack(experts.w13_weight, experts.w13_weight_scale_inv,
                                                         experts.w2_weight, experts.w2_weight_scale_inv)
            layer.bind_weights_fp8(self._native_tmaps)
            out = layer.forward_routed(hidden_states, weights, ids, combine_fn=combine_fn)
        elif native:
            if self._native_tmaps is None:
                self._native_tmaps = layer.make_weight_maps(experts.w13_weight, experts.w2_weight)
            layer.bind_weights(experts.w13_weight, experts.w2_weight, *self._native_tmaps)
            out = layer.forward_routed(hidden_states, weights, ids, combine_fn=combine_fn)
        else:
            kernel = self._local_experts_kernel()
            prep = self.moeflow.fused_expert_prep

            def compute_local_experts(hidden_rows, expert_ids, routing_weights):
                if prep:
                    gids, local_w = expert_ids, routing_weights
                else:
                    gids, local_w = local_to_global_ids(expert_ids, routing_weights, offset, experts.global_num_experts)
                return kernel.apply(hidden_rows, experts.w13_weight, experts.w2_weight, local_w, gids.to(ids.dtype),
                                    activation=experts.activation, global_num_experts=experts.global_num_experts,
                                    expert_map=experts.expert_map, apply_router_weight_on_input=False)

            out = layer.forward_routed(
                hidden_states, weights, ids, expert_fn=compute_local_experts, combine_fn=combine_fn,
                prepare_fn=make_prepare_fn(self.moeflow_cfg, offset, experts.global_num_experts, ids.dtype) if prep else None,
                direct_expert_output=self.moeflow.direct_expert_output,
            )
        if self._fixed_probe is not None:
            self._fixed_probe.compare(experts, hidden_states, weights, ids, out, getattr(self, "layer_name", None), capacity,
                                      owner_partials=layer.ret_recv, experts_per_rank=layer.L)
        capturing = hidden_states.is_cuda and torch.cuda.is_current_stream_capturing()
        if self._moeflow_log is not None and self._moeflow_fixed_calls <= MAX_LOGGED_CALLS_PER_LAYER and not capturing:
            self._record({
                "intercepted": True, "mode": "fixed", "tokens": int(hidden_states.shape[0]), "capacity": capacity,
                "combine_mode": self.moeflow.combine_mode, "fused_dispatch": self.moeflow.fused_dispatch,
                "fused_expert_prep": self.moeflow.fused_expert_prep,
                "direct_expert_output": self.moeflow.direct_expert_output,
                "experts": f"native-{native}" if native else "vllm",
            })
        return self._shared_output(overlapping, out)


def _no_overlap_order():
    from vllm.model_executor.layers.fused_moe.runner.shared_experts import SharedExpertsOrder

    return SharedExpertsOrder.NO_OVERLAP


_RUNNER_CLASS = None


def _build_runner_class():
    """Subclass the installed engine's ``MoERunner``.

    Two generations of the runner interface are supported.  The older one calls
    ``_apply_quant_method(hidden_states, router_logits, shared_experts_input, input_ids, overlapping)`` and keeps
    the expert layer in ``self.routed_experts``.  The newer one (vLLM 0.22) passes the expert layer as the first
    argument ``layer``, has no overlap flag and runs multi-stream shared experts after the routed ones.
    """
    import inspect

    from vllm.config import get_current_vllm_config
    from vllm.model_executor.layers.fused_moe.runner.moe_runner import MoERunner

    takes_layer = "layer" in inspect.signature(MoERunner._apply_quant_method).parameters

    class MoEFlowRunner(RunnerCore, MoERunner):
        def __init__(self, *args, **kwargs):
            MoERunner.__init__(self, *args, **kwargs)
            self._moeflow_setup(cfg_from_hf_text_config(get_current_vllm_config().model_config.hf_text_config))

        if takes_layer:

            def _apply_quant_method(self, layer, hidden_states, router_logits, shared_experts_input, input_ids=None):
                # kept out of the module registry on purpose: the layer owns this runner, not the reverse
                self.__dict__["routed_experts"] = layer
                self.__dict__["_late_shared_input"] = shared_experts_input
                return RunnerCore._apply_quant_method(self, hidden_states, router_logits, shared_experts_input, input_ids,
                                                      False)

            def _native_apply(self, hidden_states, router_logits, shared_experts_input, input_ids=None, *_):
                return MoERunner._apply_quant_method(self, self.routed_experts, hidden_states, router_logits,
                                                     shared_experts_input, input_ids)

            def _late_shared_experts(self):
                from vllm.model_executor.layers.fused_moe.runner.shared_experts import SharedExpertsOrder

                order = getattr(SharedExpertsOrder, "MULTI_STREAM_OVERLAPPED", None)
                if order is not None:
                    self._maybe_apply_shared_experts(self.__dict__.get("_late_shared_input"), order)

        else:

            def _native_apply(self, *args, **kwargs):
                return MoERunner._apply_quant_method(self, *args, **kwargs)

    MoEFlowRunner.__qualname__ = "MoEFlowRunner"
    return MoEFlowRunner


def __getattr__(name: str):
    """``MoEFlowRunner`` is built on first access, so importing this module does not import vLLM."""
    global _RUNNER_CLASS
    if name == "MoEFlowRunner":
        if _RUNNER_CLASS is None:
            _RUNNER_CLASS = _build_runner_class()
        return _RUNNER_CLASS
    raise AttributeError(name)
