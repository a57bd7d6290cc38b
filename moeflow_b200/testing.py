"""Deterministic synthetic inputs: expert weights, hidden states, routing distributions.

All generators draw on the CPU from a seeded ``torch.Generator`` so that every rank and every
backend sees the same numbers.  Counterpart of the reference's ``moeflow/testing.py:14-80``.
"""

from __future__ import annotations

import math

import torch

from .config import MoEConfig

DISTRIBUTIONS = ("uniform", "zipf", "hotspot")


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def make_weights(cfg: MoEConfig, seed: int, device="cpu", dtype=torch.bfloat16, experts: range | None = None):
    """``w13 [E, 2I, H]`` ~ N(0, (2/sqrt(H))^2), ``w2 [E, H, I]`` ~ N(0, (1/sqrt(I))^2).

    The scales keep activations O(1) and make the SwiGLU clamp bite now and then.  With ``experts``
    only that slice is materialised (expert e always gets the same numbers, whatever the slice).
    """
    n_exp, hidden, inter = cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size
    if experts is None:
        g = _gen(seed)
        w13 = torch.randn(n_exp, 2 * inter, hidden, generator=g) * (2.0 / math.sqrt(hidden))
        w2 = torch.randn(n_exp, hidden, inter, generator=g) * (1.0 / math.sqrt(inter))
        return w13.to(device=device, dtype=dtype), w2.to(device=device, dtype=dtype)
    w13 = torch.empty(len(experts), 2 * inter, hidden, dtype=dtype, device=device)
    w2 = torch.empty(len(experts), hidden, inter, dtype=dtype, device=device)
    for i, e in enumerate(experts):
        g = _gen(seed * 1_000_003 + e)
        w13[i] = (torch.randn(2 * inter, hidden, generator=g) * (2.0 / math.sqrt(hidden))).to(dtype)
        w2[i] = (torch.randn(hidden, inter, generator=g) * (1.0 / math.sqrt(inter))).to(dtype)
    return w13, w2


def make_hidden(num_tokens: int, cfg: MoEConfig, seed: int, device="cpu", dtype=torch.bfloat16):
    return torch.randn(num_tokens, cfg.hidden_size, generator=_gen(seed)).to(device=device, dtype=dtype)


def make_logits(
    num_tokens: int,
    cfg: MoEConfig,
    seed: int,
    dist: str = "uniform",
    device="cpu",
    zipf_s: float = 1.2,
    hot_experts: int | None = None,
    hot_first: bool = False,
):
    """Router logits ``[T, E]`` fp32 whose top-k choice follows a popularity profile.

    ``uniform``: i.i.d. normal.  ``zipf``: expert with popularity rank r gets an offset
    ``-2 * s * log(r)``; ranks are a random permutation of the experts, or 1..E in id order with
    ``hot_first`` (the popular experts then share one EP rank).  ``hotspot``: the first
    ``hot_experts`` (default ``top_k``) experts win every token.
    """
    g = _gen(seed)
    n_exp = cfg.n_routed_experts
    logits = torch.randn(num_tokens, n_exp, generator=g)
    if dist == "uniform":
        pass
    elif dist == "zipf":
        order = torch.randperm(n_exp, generator=g)
        if hot_first:
            order = torch.arange(n_exp)
        rank_of = torch.empty(n_exp)
        rank_of[order] = torch.arange(1, n_exp + 1, dtype=torch.float32)
        logits = logits - 2.0 * zipf_s * torch.log(rank_of)
    elif dist == "hotspot":
        hot = cfg.top_k if hot_experts is None else hot_experts
        logits[:, :hot] += 20.0
        logits[:, hot:] -= 20.0
    else:
        raise ValueError(f"unknown routing distribution {dist!r}")
    return logits.to(device=device, dtype=torch.float32)


def make_bias(cfg: MoEConfig, seed: int, device="cpu"):
    return (0.05 * torch.randn(cfg.n_routed_experts, generator=_gen(seed))).to(device=device, dtype=torch.float32)


class ScaleExperts:
    """Hand-checkable expert backend: global expert ``g`` maps ``x`` to ``(g + 1) * x``."""

    name = "scale"

    def __init__(self, rank_expert_offset: int):
        self.offset = rank_expert_offset

    def __call__(self, a, expert_offsets, w13, w2, swiglu_limit, row_weight=None):
        bounds = expert_offsets.tolist()
        out = torch.empty_like(a)
        for e, (lo, hi) in enumerate(zip(bounds[:-1], bounds[1:])):
            y = a[lo:hi].to(torch.float32) * float(self.offset + e + 1)
            if row_weight is not None:
                y = y * row_weight[lo:hi].unsqueeze(1)
            out[lo:hi] = y.to(a.dtype)
        return out
