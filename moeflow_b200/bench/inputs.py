"""Weights for benchmarks: ``"synthetic"`` or ``"real:<layer>"`` from the checkpoint reader.
Counterpart of ``scripts/bench/inputs.py:8-23``.
"""

from __future__ import annotations

from ..config import MoEConfig
from ..testing import make_bias, make_weights


def load_weights(spec: str, cfg: MoEConfig, device, seed: int = 0, experts: range | None = None):
    """Returns ``(w13 [E|len(experts), 2I, H], w2, bias [E])`` on ``device``."""
    if spec == "synthetic":
        w13, w2 = make_weights(cfg, seed, device=device, experts=experts)
        return w13, w2, make_bias(cfg, seed + 1, device=device)
    if spec.startswith("real:"):
        from ..weights import CheckpointReader

        layer = int(spec.split(":", 1)[1])
        reader = CheckpointReader()
        rng = experts if experts is not None else range(cfg.n_routed_experts)
        w13, w2 = reader.expert_weights(layer, rng)
        _, bias = reader.router(layer)
        return w13.to(device), w2.to(device), bias.to(device)
    raise ValueError(f"unknown weight spec {spec!r} (use 'synthetic' or 'real:<layer>')")
