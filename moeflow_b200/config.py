"""Configuration of one Mixture-of-Experts layer.

``MoEConfig`` carries everything the router, the dispatch layout and the expert GEMMs need to know
about a layer.  The defaults describe GLM-5.3-Flash (hidden 4096, 288 routed experts + 1 shared,
top-8, sigmoid scoring with the "noaux_tc" correction bias).  The expert intermediate size is a free
parameter: the public checkpoint uses 2048, benchmark configurations may use others.

Same public surface as the reference's ``moeflow/config.py:10-55``.
"""

from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Any

_HF_KEYS = {
    "hidden_size": "hidden_size",
    "moe_intermediate_size": "moe_intermediate_size",
    "n_routed_experts": "n_routed_experts",
    "n_shared_experts": "n_shared_experts",
    "top_k": "num_experts_per_tok",
    "n_group": "n_group",
    "topk_group": "topk_group",
    "norm_topk_prob": "norm_topk_prob",
    "routed_scaling_factor": "routed_scaling_factor",
    "scoring_func": "scoring_func",
    "topk_method": "topk_method",
}


@dataclasses.dataclass(frozen=True)
class MoEConfig:
    hidden_size: int = 4096
    moe_intermediate_size: int = 2048
    n_routed_experts: int = 288
    n_shared_experts: int = 1
    top_k: int = 8
    n_group: int = 1
    topk_group: int = 1
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 2.5
    scoring_func: str = "sigmoid"
    topk_method: str = "noaux_tc"
    #: SwiGLU clamp: the gate is clamped from above only, the up projection to [-limit, limit].
    swiglu_limit: float | None = 10.0

    def experts_per_rank(self, ep_size: int) -> int:
        """Local expert count under contiguous placement; the expert count must divide evenly."""
        if ep_size < 1 or self.n_routed_experts % ep_size != 0:
            raise ValueError(f"{self.n_routed_experts} experts not divisible by ep_size={ep_size}")
        return self.n_routed_experts // ep_size

    def to_dict(self) -> dict[str, Any]:
        return dataclasses.asdict(self)

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "MoEConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    @classmethod
    def from_hf_dict(cls, cfg: dict[str, Any]) -> "MoEConfig":
        """Build from a parsed HuggingFace config (uses ``text_config`` when there is one)."""
        text = cfg.get("text_config", cfg)
        kwargs = {field: text[key] for field, key in _HF_KEYS.items()}
        kwargs["routed_scaling_factor"] = float(kwargs["routed_scaling_factor"])
        kwargs["swiglu_limit"] = text.get("swiglu_limit")
        return cls(**kwargs)

    @classmethod
    def from_hf_config(cls, path: str | Path) -> "MoEConfig":
        """Build from a HuggingFace ``config.json`` file."""
        return cls.from_hf_dict(json.loads(Path(path).read_text()))


GLM53_FLASH = MoEConfig()
#: The benchmark shape: GLM-5.3-Flash routing with expert intermediate size 1536.
GLM53_FLASH_I1536 = dataclasses.replace(GLM53_FLASH, moe_intermediate_size=1536)
