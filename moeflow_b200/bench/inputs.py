"""Where a benchmark's expert weights come from.

A weight source is written as a short spec string so that it fits in a record's configuration:

    synthetic          seeded random weights of the configured shape (``testing.make_weights``)
    real:<layer>       the experts of checkpoint layer <layer>, through ``weights.CheckpointReader``

``WeightSource.parse`` turns the string into an object; ``load`` materialises ``(w13, w2, bias)`` on a device,
optionally only for a range of experts (one EP rank's shard), so that a rank never holds more than it owns.
Same two sources as ``scripts/bench/inputs.py:8-23`` of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..config import MoEConfig


@dataclass(frozen=True)
class WeightSource:
    kind: str                  # "synthetic" | "real"
    layer: int | None = None   # checkpoint layer of a "real" source

    @classmethod
    def parse(cls, spec: str) -> "WeightSource":
        head, _, tail = spec.partition(":")
        if head == "synthetic" and not tail:
            return cls("synthetic")
        if head == "real" and tail.isdigit():
            return cls("real", int(tail))
        raise ValueError(f"unknown weight spec {spec!r} (use 'synthetic' or 'real:<layer>')")

    def load(self, cfg: MoEConfig, device, seed: int = 0, experts: range | None = None):
        """``(w13 [n, 2I, H], w2 [n, H, I], bias [E])`` on ``device``; n = all experts or ``len(experts)``."""
        if self.kind == "synthetic":
            from ..testing import make_bias, make_weights

            return (*make_weights(cfg, seed, device=device, experts=experts), make_bias(cfg, seed + 1, device=device))
        from ..weights import CheckpointReader

        reader = CheckpointReader()
        wanted = range(cfg.n_routed_experts) if experts is None else experts
        w13, w2 = reader.expert_weights(self.layer, wanted)
        selection_bias = reader.router(self.layer)[1]
        return w13.to(device), w2.to(device), selection_bias.to(device)


def load_weights(spec: str, cfg: MoEConfig, device, seed: int = 0, experts: range | None = None):
    """``WeightSource.parse(spec).load(...)``."""
    return WeightSource.parse(spec).load(cfg, device, seed=seed, experts=experts)
