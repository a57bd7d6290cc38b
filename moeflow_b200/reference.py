"""Loop-level oracle for one routed MoE layer.

Boundary: hidden states ``x [T, H]``, router logits ``[T, E]`` (fp32) and the optional selection bias
``[E]`` go in; the weighted sum of the selected routed experts (routed scaling factor included)
comes out in ``x.dtype``.  Gate GEMM, shared expert and norms are outside.

Everything here is written one token and one expert at a time with plain Python loops and scalar
float64 scoring.  It shares no indexing code with the router, dispatch or GEMM implementations it is
used to check.  Behavioural counterpart of the reference's ``moeflow/reference.py:21-127``.
"""

from __future__ import annotations

import math

import torch

from .config import MoEConfig

Route = list[tuple[int, float]]


def _scores(logit_row: torch.Tensor, kind: str) -> list[float]:
    raw = logit_row.detach().to(torch.float64).cpu().tolist()
    if kind == "sigmoid":
        return [1.0 / (1.0 + math.exp(-v)) for v in raw]
    if kind == "softmax":
        top = max(raw)
        expd = [math.exp(v - top) for v in raw]
        total = math.fsum(expd)
        return [v / total for v in expd]
    raise ValueError(f"unknown scoring function {kind!r}")


def route_token(logits: torch.Tensor, bias: torch.Tensor | None, cfg: MoEConfig) -> Route:
    """Route one token; returns ``[(expert, weight)]`` in selection order (best biased score first).

    The selection uses ``score + bias``; the returned weight is the *unbiased* score, renormalised by
    ``sum + 1e-20`` when ``norm_topk_prob`` and multiplied by ``routed_scaling_factor``.  With expert
    groups, a group's rank is the sum of its two best biased scores when a bias is given and its best
    score otherwise, and only ``topk_group`` groups stay eligible.  Equal scores go to the lower id.
    """
    n_experts = logits.numel()
    score = _scores(logits, cfg.scoring_func)
    shift = [0.0] * n_experts if bias is None else bias.detach().to(torch.float64).cpu().tolist()
    key = [score[e] + shift[e] for e in range(n_experts)]

    width = n_experts // cfg.n_group
    ranked_groups = []
    for g in range(cfg.n_group):
        best_first = sorted(key[g * width : (g + 1) * width], reverse=True)
        strength = best_first[0] + best_first[1] if bias is not None else best_first[0]
        ranked_groups.append((-strength, g))
    ranked_groups.sort()
    open_groups = {g for _, g in ranked_groups[: cfg.topk_group]}

    order = sorted((e for e in range(n_experts) if e // width in open_groups), key=lambda e: (-key[e], e))
    picked = order[: cfg.top_k]
    w = [score[e] for e in picked]
    if cfg.norm_topk_prob:
        denom = sum(w) + 1e-20
        w = [v / denom for v in w]
    return [(e, v * cfg.routed_scaling_factor) for e, v in zip(picked, w)]


def route_reference(logits: torch.Tensor, bias: torch.Tensor | None, cfg: MoEConfig) -> list[Route]:
    return [route_token(logits[t], bias, cfg) for t in range(logits.shape[0])]


def swiglu_clamp(gate: torch.Tensor, up: torch.Tensor, limit: float | None) -> torch.Tensor:
    """``silu(gate) * up`` with the gate clamped from above and the up branch clamped both ways."""
    if limit is not None:
        gate = gate.clamp(max=limit)
        up = up.clamp(min=-limit, max=limit)
    return gate * torch.sigmoid(gate) * up


def expert_forward(
    x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, limit: float | None, acc_dtype: torch.dtype = torch.float32
) -> torch.Tensor:
    """One token through one expert: ``x [H]``, ``w13 [2I, H] = [gate; up]``, ``w2 [H, I]`` -> ``[H]``."""
    inter = w2.shape[1]
    hidden = torch.mv(w13.to(acc_dtype), x.to(acc_dtype))
    act = swiglu_clamp(hidden[:inter], hidden[inter:], limit)
    return torch.mv(w2.to(acc_dtype), act)


def moe_reference(
    x: torch.Tensor,
    logits: torch.Tensor,
    bias: torch.Tensor | None,
    w13: torch.Tensor,
    w2: torch.Tensor,
    cfg: MoEConfig,
    acc_dtype: torch.dtype = torch.float32,
    routes: list[Route] | None = None,
) -> torch.Tensor:
    """Whole layer: ``w13 [E, 2I, H]``, ``w2 [E, H, I]`` -> ``[T, H]`` in ``x.dtype``.

    ``routes`` replaces the routing, so that the expert/combine path can be judged on exactly the
    expert choice of the implementation under test.
    """
    n_tokens, hidden = x.shape
    out = torch.zeros(n_tokens, hidden, dtype=acc_dtype, device=x.device)
    for t in range(n_tokens):
        chosen = route_token(logits[t], bias, cfg) if routes is None else routes[t]
        total = torch.zeros(hidden, dtype=acc_dtype, device=x.device)
        for expert, weight in chosen:
            total = total + weight * expert_forward(x[t], w13[expert], w2[expert], cfg.swiglu_limit, acc_dtype)
        out[t] = total
    return out.to(x.dtype)


def ep_dispatch_reference(routes_per_rank: list[list[Route]], experts_per_rank: int) -> list[list]:
    """What every destination rank must receive: one copy per (token, destination rank).

    ``routes_per_rank[src][t]`` is the route of token ``t`` owned by rank ``src``.  The result
    ``recv[dst]`` lists ``(src, t, [(local_expert, weight), ...])`` ordered by source rank, then token;
    the hits keep the top-k slot order and carry ids local to ``dst``.
    """
    world = len(routes_per_rank)
    inbox: list[list] = [[] for _ in range(world)]
    for src, routes in enumerate(routes_per_rank):
        for t, route in enumerate(routes):
            for dst in range(world):
                lo = dst * experts_per_rank
                hits = [(e - lo, w) for e, w in route if lo <= e < lo + experts_per_rank]
                if hits:
                    inbox[dst].append((src, t, hits))
    return inbox
