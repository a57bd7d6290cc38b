"""The ``MOEFLOW_*`` environment switches (stable public surface) in one place.

Runner switches (read once per ``MoEFlowRunner``):
  MOEFLOW_RUNNER=1                wrap the MoE layer factory so layers are built with ``MoEFlowRunner``
  MOEFLOW_ALL2ALL=1               swap the modular Prepare/Finalize for ``MoEFlowPrepareAndFinalize``
  MOEFLOW_MODE                    ``route_check`` (default) | ``fixed``
  MOEFLOW_MAX_TOKENS              token ceiling of the fixed path (default 256)
  MOEFLOW_COMBINE_MODE            ``fp32`` (default) | ``bf16_ring`` | ``bf16_ring_fused``
  MOEFLOW_FUSED_DISPATCH=1        accepted for compatibility (dispatch is always fused on the cuda backend)
  MOEFLOW_FUSED_EXPERT_PREP=1     unpack received rows to global ids before the external experts run
  MOEFLOW_DIRECT_EXPERT_OUTPUT=1  use the external experts' output tensor as the return buffer (needs PREP)
  MOEFLOW_EXPERTS                 ``auto`` (default) | ``native`` (tcgen05 grouped GEMMs) | ``vllm`` (the engine's experts)
  MOEFLOW_ROUTING_TRACE_DIR       directory of the routing trace (collection starts when ``<dir>/enabled`` exists)
  MOEFLOW_VALIDATE_FIXED=1        eager comparison against the engine's native path (needs the trace dir)
  MOEFLOW_SMOKE_DIR               directory of the per-process JSONL call log
Site / harness switches: MOEFLOW_MODEL_PATH, MOEFLOW_TRIMMED_MODEL_PATH, MOEFLOW_PYTHON, MOEFLOW_TORCHRUN,
MOEFLOW_VLLM, MOEFLOW_JOBID, MOEFLOW_RESULTS_ROOT and the MOEFLOW_GREEDY_* / MOEFLOW_LOGITS_* /
MOEFLOW_*_TIMEOUT knobs of the shell drivers.  Counterpart of the reference's switch table
(``moeflow/integrations/vllm_runner.py:67-89``, ``vllm_plugin.py:105-109``).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path

MODES = ("route_check", "fixed")
COMBINE_MODES = ("fp32", "bf16_ring", "bf16_ring_fused")
EXPERT_ENGINES = ("auto", "native", "vllm")


def flag(name: str, env=None) -> bool:
    return (env if env is not None else os.environ).get(name) == "1"


@dataclass(frozen=True)
class RunnerSettings:
    mode: str = "route_check"
    max_tokens: int = 256
    combine_mode: str = "fp32"
    fused_dispatch: bool = False
    fused_expert_prep: bool = False
    direct_expert_output: bool = False
    experts: str = "auto"
    routing_trace_dir: Path | None = None
    validate_fixed: bool = False
    smoke_dir: Path | None = None

    @classmethod
    def from_env(cls, env=None) -> "RunnerSettings":
        env = env if env is not None else os.environ
        s = cls(
            mode=env.get("MOEFLOW_MODE", "route_check"),
            max_tokens=int(env.get("MOEFLOW_MAX_TOKENS", "256")),
            combine_mode=env.get("MOEFLOW_COMBINE_MODE", "fp32"),
            fused_dispatch=flag("MOEFLOW_FUSED_DISPATCH", env),
            fused_expert_prep=flag("MOEFLOW_FUSED_EXPERT_PREP", env),
            direct_expert_output=flag("MOEFLOW_DIRECT_EXPERT_OUTPUT", env),
            experts=env.get("MOEFLOW_EXPERTS", "auto"),
            routing_trace_dir=Path(env["MOEFLOW_ROUTING_TRACE_DIR"]) if env.get("MOEFLOW_ROUTING_TRACE_DIR") else None,
            validate_fixed=flag("MOEFLOW_VALIDATE_FIXED", env),
            smoke_dir=Path(env["MOEFLOW_SMOKE_DIR"]) if env.get("MOEFLOW_SMOKE_DIR") else None,
        )
        s.validate()
        return s

    def validate(self) -> None:
        if self.mode not in MODES:
            raise ValueError(f"MOEFLOW_MODE must be one of {MODES}")
        if self.combine_mode not in COMBINE_MODES:
            raise ValueError("MOEFLOW_COMBINE_MODE must be fp32, bf16_ring or bf16_ring_fused")
        if self.experts not in EXPERT_ENGINES:
            raise ValueError(f"MOEFLOW_EXPERTS must be one of {EXPERT_ENGINES}")
        if self.direct_expert_output and not self.fused_expert_prep:
            raise ValueError("Direct expert output requires MOEFLOW_FUSED_EXPERT_PREP=1")
        if self.validate_fixed and self.routing_trace_dir is None:
            raise ValueError("Fixed diagnostics require MOEFLOW_ROUTING_TRACE_DIR and eager execution")
