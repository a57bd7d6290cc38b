"""vLLM general plugin (entry point group ``vllm.general_plugins``, name ``moeflow``).

It never edits the vLLM installation; it only rebinds names in already importable modules.

* ``MOEFLOW_RUNNER=1``: MoE layers are built with ``MoEFlowRunner``.  Where vLLM has a
  ``FusedMoEFactory(..., runner_cls=...)`` the factory is wrapped (in the defining module, the package
  re-export and any model module that imported it earlier) and ``runner_cls`` is injected only when the
  caller left it unset.  Older vLLM builds construct ``MoERunner`` directly inside
  ``fused_moe/layer.py``; there the module's ``MoERunner`` binding is replaced by the subclass.
* ``MOEFLOW_ALL2ALL=1``: ``maybe_make_prepare_finalize`` is wrapped in every module that bound it by name,
  and returns ``MoEFlowPrepareAndFinalize`` for EP all-to-all configurations that are not monolithic.

Both registrations are idempotent.  Counterpart of ``moeflow/integrations/vllm_plugin.py:20-129``.
"""

from __future__ import annotations

import importlib
import logging
import os
import sys

logger = logging.getLogger("moeflow")

FACTORY_MODULES = ("vllm.model_executor.layers.fused_moe.layer", "vllm.model_executor.layers.fused_moe")
#: model modules that may have imported the factory before the plugin ran
LATE_BINDING_MODULES = ("vllm.models.glm5next.common.model",)
#: modules that bind ``maybe_make_prepare_finalize`` by name at import time
PREPARE_FINALIZE_MODULES = (
    "vllm.model_executor.layers.fused_moe.all2all_utils",
    "vllm.model_executor.layers.fused_moe.oracle.fp8",
    "vllm.model_executor.layers.fused_moe.oracle.unquantized",
    "vllm.model_executor.layers.fused_moe.oracle.nvfp4",
    "vllm.model_executor.layers.fused_moe.oracle.mxfp4",
    "vllm.model_executor.layers.fused_moe.oracle.int8",
    "vllm.model_executor.layers.fused_moe.oracle.int_wna16",
    "vllm.model_executor.layers.fused_moe.oracle.w4a8",
    "vllm.model_executor.layers.fused_moe.oracle.w4a8_int8",
    "vllm.model_executor.layers.fused_moe.eep_reconfigure",
    "vllm.model_executor.layers.quantization.modelopt_block_quant",
)


def _runner_class():
    from .vllm_runner import MoEFlowRunner

    return MoEFlowRunner


def wrap_factory(original):
    """A factory that passes ``runner_cls=MoEFlowRunner`` unless the caller chose a runner."""

    def FusedMoEFactory(*args, **kwargs):  # noqa: N802 - keeps vLLM's name
        if kwargs.get("runner_cls") is None:
            kwargs["runner_cls"] = _runner_class()
        return original(*args, **kwargs)

    FusedMoEFactory._moeflow_wrapped = True
    FusedMoEFactory._moeflow_original = original
    return FusedMoEFactory


def register_runner() -> str:
    """Returns which hook was used: ``"factory"``, ``"runner_binding"`` or ``"already"``."""
    base = importlib.import_module(FACTORY_MODULES[0])
    original = getattr(base, "FusedMoEFactory", None)
    if original is not None:
        if getattr(original, "_moeflow_wrapped", False):
            return "already"
        wrapped = wrap_factory(original)
        for name in FACTORY_MODULES:
            mod = importlib.import_module(name)
            if getattr(mod, "FusedMoEFactory", None) is original:
                mod.FusedMoEFactory = wrapped
        for name in LATE_BINDING_MODULES:
            mod = sys.modules.get(name)
            if mod is not None and getattr(mod, "FusedMoEFactory", None) is original:
                mod.FusedMoEFactory = wrapped
        logger.warning("moeflow: FusedMoEFactory wrapped (runner_cls=MoEFlowRunner)")
        return "factory"
    # No factory in this vLLM: the layer module instantiates its ``MoERunner`` binding directly.
    current = getattr(base, "MoERunner", None)
    if current is None:
        raise RuntimeError("this vLLM has neither FusedMoEFactory nor a MoERunner binding to hook")
    if getattr(current, "_moeflow_runner", False):
        return "already"
    base.MoERunner = _runner_class()
    logger.warning("moeflow: fused_moe.layer.MoERunner rebound to MoEFlowRunner (no FusedMoEFactory in this vLLM)")
    return "runner_binding"


def wrap_prepare_finalize(original):
    def maybe_make_prepare_finalize(moe, quant_config, *args, **kwargs):
        use_monolithic = kwargs.get("use_monolithic", False)
        parallel = moe.moe_parallel_config
        if parallel.use_all2all_kernels and not use_monolithic:
            from vllm.distributed import get_ep_group

            from .vllm_pf import MoEFlowPrepareAndFinalize

            logger.info("moeflow: MoEFlowPrepareAndFinalize (ep_size=%d, local experts=%d)", parallel.ep_size,
                        moe.num_local_experts)
            return MoEFlowPrepareAndFinalize(get_ep_group().device_group, moe.num_local_experts)
        return original(moe, quant_config, *args, **kwargs)

    maybe_make_prepare_finalize._moeflow_wrapped_pf = True
    maybe_make_prepare_finalize._moeflow_original = original
    return maybe_make_prepare_finalize


def register_prepare_finalize() -> list[str]:
    """Returns the short names of the modules whose binding now points at the wrapper."""
    base = importlib.import_module(PREPARE_FINALIZE_MODULES[0])
    original = base.maybe_make_prepare_finalize
    if getattr(original, "_moeflow_wrapped_pf", False):
        return []
    wrapped = wrap_prepare_finalize(original)
    patched = []
    for name in PREPARE_FINALIZE_MODULES:
        try:
            mod = importlib.import_module(name)
        except ImportError:
            continue
        bound = getattr(mod, "maybe_make_prepare_finalize", None)
        if bound is original:
            mod.maybe_make_prepare_finalize = wrapped
            bound = wrapped
        if bound is wrapped:
            patched.append(name.rsplit(".", 1)[-1])
    logger.warning("moeflow: patched maybe_make_prepare_finalize in %s", ", ".join(patched))
    return patched


def register() -> None:
    """Plugin entry point; does nothing unless a switch is set."""
    if os.environ.get("MOEFLOW_RUNNER") == "1":
        register_runner()
    if os.environ.get("MOEFLOW_ALL2ALL") == "1":
        register_prepare_finalize()
