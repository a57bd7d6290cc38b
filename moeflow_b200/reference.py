"""The oracle: one routed MoE layer computed the slowest and most obvious way.

In:  hidden rows ``x [T, H]``, router logits ``[T, E]``, optionally the selection bias ``[E]``, and the expert
weights ``w13 [E, 2I, H]`` (gate rows, then up rows) and ``w2 [E, H, I]``.
Out: for every token the sum over its K chosen experts of ``weight * expert(x)``, the routed scaling factor
included, in ``x.dtype``.  The gate projection that produces the logits, the shared expert and the norms are
not part of this boundary.

Nothing here is vectorised over tokens or experts and nothing is sorted: scores are Python floats (fp64),
"the best k" is found by scanning k times for the largest remaining value (a strict ``>`` keeps the lower
index on ties), and every (token, expert) pair is one pair of matrix-vector products.  The module shares no
indexing code with the router, the dispatch stages or the kernels, which is what makes it usable as their
judge.  Same semantics as ``moeflow/reference.py:21-127`` of the reference.
"""

from __future__ import annotations

import math

import torch

from .config import MoEConfig

Route = list[tuple[int, float]]


# ---- routing ----------------------------------------------------------------------------------------------
def _sigmoid_scores(z: list[float]) -> list[float]:
    return [1.0 / (1.0 + math.exp(-v)) for v in z]


def _softmax_scores(z: list[float]) -> list[float]:
    peak = max(z)
    grown = [math.exp(v - peak) for v in z]
    whole = math.fsum(grown)
    return [g / whole for g in grown]


_SCORING = {"sigmoid": _sigmoid_scores, "softmax": _softmax_scores}


def _scan_best(values: list[float], how_many: int, allowed=None) -> list[int]:
    """Indices of the ``how_many`` largest values, best first; among equals the lower index comes first."""
    taken: list[int] = []
    for _ in range(min(how_many, len(values))):
        best = None
        for i, v in enumerate(values):
            if i in taken or (allowed is not None and i not in allowed):
                continue
            if best is None or v > values[best]:
                best = i
        if best is None:
            break
        taken.append(best)
    return taken


def route_token(logits: torch.Tensor, bias: torch.Tensor | None, cfg: MoEConfig) -> Route:
    """``[(expert, weight), ...]`` of one token, best selection key first.

    key = score + bias decides who is picked; the weight is the *unbiased* score, divided by the picks' sum
    (+1e-20) under ``norm_topk_prob``, times ``routed_scaling_factor``.  With expert groups only the
    ``topk_group`` best groups are eligible; a group is rated by its two best keys added up when there is a
    bias and by its best key when there is none.
    """
    if cfg.scoring_func not in _SCORING:
        raise ValueError(f"unknown scoring function {cfg.scoring_func!r}")
    score = _SCORING[cfg.scoring_func](logits.detach().to(torch.float64).cpu().tolist())
    experts = len(score)
    if bias is None:
        key = list(score)
    else:
        key = [s + b for s, b in zip(score, bias.detach().to(torch.float64).cpu().tolist())]

    per_group = experts // cfg.n_group
    rating = []
    for g in range(cfg.n_group):
        members = key[g * per_group:(g + 1) * per_group]
        first = _scan_best(members, 1)[0]
        if bias is None:
            rating.append(members[first])
        else:
            second = _scan_best(members, 2)[1]
            rating.append(members[first] + members[second])
    eligible_groups = set(_scan_best(rating, cfg.topk_group))
    eligible = {e for e in range(experts) if e // per_group in eligible_groups}

    picks = _scan_best(key, cfg.top_k, allowed=eligible)
    weights = [score[e] for e in picks]
    if cfg.norm_topk_prob:
        whole = sum(weights) + 1e-20
        weights = [w / whole for w in weights]
    return [(e, w * cfg.routed_scaling_factor) for e, w in zip(picks, weights)]


def route_reference(logits: torch.Tensor, bias: torch.Tensor | None, cfg: MoEConfig) -> list[Route]:
    return [route_token(row, bias, cfg) for row in logits]


# ---- experts ------------------------------------------------------------------------------------------------
def swiglu_clamp(gate: torch.Tensor, up: torch.Tensor, limit: float | None) -> torch.Tensor:
    """``silu(gate) * up``; with a limit the gate is capped from above and the up branch on both sides."""
    if limit is not None:
        gate, up = gate.clamp(max=limit), up.clamp(min=-limit, max=limit)
    return gate * torch.sigmoid(gate) * up


def expert_forward(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, limit: float | None,
                   acc_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """One token ``x [H]`` through one expert (``w13 [2I, H]``, ``w2 [H, I]``) -> ``[H]`` in ``acc_dtype``."""
    gate_and_up = torch.mv(w13.to(acc_dtype), x.to(acc_dtype))
    inter = w2.shape[1]
    return torch.mv(w2.to(acc_dtype), swiglu_clamp(gate_and_up[:inter], gate_and_up[inter:], limit))


def moe_reference(x: torch.Tensor, logits: torch.Tensor, bias: torch.Tensor | None, w13, w2, cfg: MoEConfig,
                  acc_dtype: torch.dtype = torch.float32, routes: list[Route] | None = None) -> torch.Tensor:
    """The whole layer.  ``routes`` (one per token) replaces the routing step, so that the expert and combine
    path of an implementation can be judged on exactly the experts that implementation chose.
    ``w13`` / ``w2`` only need ``__getitem__`` by expert id (a tensor, or a lookup of the few experts needed)."""
    rows = []
    for t in range(x.shape[0]):
        route = routes[t] if routes is not None else route_token(logits[t], bias, cfg)
        acc = torch.zeros(x.shape[1], dtype=acc_dtype, device=x.device)
        for expert, weight in route:
            acc = acc + weight * expert_forward(x[t], w13[expert], w2[expert], cfg.swiglu_limit, acc_dtype)
        rows.append(acc)
    if not rows:
        return torch.zeros(0, x.shape[1], dtype=x.dtype, device=x.device)
    return torch.stack(rows).to(x.dtype)


# ---- dispatch contract ------------------------------------------------------------------------------------------
def ep_dispatch_reference(routes_per_rank: list[list[Route]], experts_per_rank: int) -> list[list]:
    """What every rank has to receive: one copy of a token per destination rank that owns one of its experts.

    ``routes_per_rank[src][t]`` is the route of token t of rank src.  ``result[dst]`` lists
    ``(src, t, [(expert local to dst, weight), ...])`` by source rank, then token; the hits keep their slot order.
    """
    world = len(routes_per_rank)
    received = []
    for dst in range(world):
        first, beyond = dst * experts_per_rank, (dst + 1) * experts_per_rank
        rows = []
        for src in range(world):
            for t, route in enumerate(routes_per_rank[src]):
                here = [(expert - first, weight) for expert, weight in route if first <= expert < beyond]
                if here:
                    rows.append((src, t, here))
        received.append(rows)
    return received
