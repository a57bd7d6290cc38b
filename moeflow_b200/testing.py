"""Seeded synthetic inputs for tests and benchmarks: expert weights, hidden rows, a selection bias, and router
logits whose top-k choice follows a chosen popularity profile.

Everything is drawn on the CPU from a ``torch.Generator`` seeded by the caller and only then moved to the
target device, so every rank and every backend sees the same numbers whatever hardware it runs on.

Popularity profiles (``make_logits(dist=...)``); each is an additive offset on i.i.d. normal logits:

    uniform   no offset
    zipf      the expert of popularity rank r gets ``-2 s ln r``; ranks are a random permutation of the experts,
              or follow the expert id (``hot_first``), which puts all popular experts on the first EP rank
    hotspot   the first ``hot_experts`` experts (default: top_k) get +20, all others -20, so they win every token

Counterpart of ``moeflow/testing.py:14-80`` of the reference.
"""

from __future__ import annotations

import math
from typing import Callable

import torch

from .config import MoEConfig


def _generator(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


# ---- weights, hidden rows, bias -----------------------------------------------------------------------
def _gate_up_and_down(cfg: MoEConfig, experts: int, gen: torch.Generator):
    """fp32 ``w13 [experts, 2I, H]`` with std ``2/sqrt(H)`` and ``w2 [experts, H, I]`` with std ``1/sqrt(I)``:
    activations stay O(1) and the SwiGLU clamp bites now and then."""
    hidden, inter = cfg.hidden_size, cfg.moe_intermediate_size
    w13 = torch.randn(experts, 2 * inter, hidden, generator=gen).mul_(2.0 / math.sqrt(hidden))
    w2 = torch.randn(experts, hidden, inter, generator=gen).mul_(1.0 / math.sqrt(inter))
    return w13, w2


def make_weights(cfg: MoEConfig, seed: int, device="cpu", dtype=torch.bfloat16, experts: range | None = None):
    """All experts from one stream, or (``experts`` given) only those, each from its own stream
    ``seed * 1_000_003 + e`` so that expert e gets the same numbers whichever slice asks for it."""
    if experts is None:
        w13, w2 = _gate_up_and_down(cfg, cfg.n_routed_experts, _generator(seed))
        return w13.to(device=device, dtype=dtype), w2.to(device=device, dtype=dtype)
    if len(experts) == 0:
        empty13, empty2 = _gate_up_and_down(cfg, 0, _generator(seed))
        return empty13.to(device=device, dtype=dtype), empty2.to(device=device, dtype=dtype)
    gate_up, down = [], []
    for e in experts:  # converted one expert at a time, so the fp32 draw of a large shard never exists whole
        w13, w2 = _gate_up_and_down(cfg, 1, _generator(seed * 1_000_003 + e))
        gate_up.append(w13.to(device=device, dtype=dtype))
        down.append(w2.to(device=device, dtype=dtype))
    return torch.cat(gate_up), torch.cat(down)


def make_hidden(num_tokens: int, cfg: MoEConfig, seed: int, device="cpu", dtype=torch.bfloat16):
    return torch.randn(num_tokens, cfg.hidden_size, generator=_generator(seed)).to(device=device, dtype=dtype)


def make_bias(cfg: MoEConfig, seed: int, device="cpu"):
    """A small selection bias (std 0.05), enough to reorder close scores."""
    draw = torch.randn(cfg.n_routed_experts, generator=_generator(seed))
    return draw.mul_(0.05).to(device=device, dtype=torch.float32)


# ---- router logits --------------------------------------------------------------------------------------
def _no_offset(cfg, gen, **_):
    return 0.0


def _zipf_offset(cfg, gen, zipf_s: float, hot_first: bool, **_):
    by_popularity = torch.randperm(cfg.n_routed_experts, generator=gen)  # drawn even when unused: keeps streams aligned
    if hot_first:
        by_popularity = torch.arange(cfg.n_routed_experts)
    rank = torch.empty(cfg.n_routed_experts)
    rank[by_popularity] = torch.arange(1, cfg.n_routed_experts + 1, dtype=torch.float32)
    return -2.0 * zipf_s * rank.log()


def _hotspot_offset(cfg, gen, hot_experts: int | None, **_):
    hot = cfg.top_k if hot_experts is None else hot_experts
    offset = torch.full((cfg.n_routed_experts,), -20.0)
    offset[:hot] = 20.0
    return offset


_PROFILES: dict[str, Callable] = {"uniform": _no_offset, "zipf": _zipf_offset, "hotspot": _hotspot_offset}
DISTRIBUTIONS = tuple(_PROFILES)


def make_logits(num_tokens: int, cfg: MoEConfig, seed: int, dist: str = "uniform", device="cpu", zipf_s: float = 1.2,
                hot_experts: int | None = None, hot_first: bool = False):
    """fp32 router logits ``[T, E]``: i.i.d. normal plus the profile's per-expert offset."""
    if dist not in _PROFILES:
        raise ValueError(f"unknown routing distribution {dist!r}")
    gen = _generator(seed)
    noise = torch.randn(num_tokens, cfg.n_routed_experts, generator=gen)
    offset = _PROFILES[dist](cfg, gen, zipf_s=zipf_s, hot_first=hot_first, hot_experts=hot_experts)
    return (noise + offset).to(device=device, dtype=torch.float32)


# ---- a stand-in expert backend ----------------------------------------------------------------------------
class ScaleExperts:
    """Expert backend one can check by hand: global expert ``g`` maps a row ``x`` to ``(g + 1) * x``
    (times the row's routing weight when one is passed).  Takes the expert-major rows and offsets of the
    variable-size pipeline like every ``ExpertCompute``; the weights are ignored."""

    name = "scale"

    def __init__(self, rank_expert_offset: int):
        self.offset = rank_expert_offset

    def __call__(self, a, expert_offsets, w13, w2, swiglu_limit, row_weight=None):
        rows_per_expert = expert_offsets[1:] - expert_offsets[:-1]
        local_expert = torch.repeat_interleave(torch.arange(rows_per_expert.numel(), device=a.device),
                                               rows_per_expert.to(torch.int64), output_size=a.shape[0])
        gain = (local_expert + (self.offset + 1)).to(torch.float32)
        scaled = a.to(torch.float32) * gain[:, None]
        if row_weight is not None:
            scaled = scaled * row_weight[:, None]
        return scaled.to(a.dtype)
