"""The noaux_tc router in PyTorch, written the way the ``router_topk`` CUDA kernel works: the K experts of a
token are picked in K rounds of "take the best remaining key", not by sorting.

Among equal keys the lowest expert id is taken, which is the tie rule of
the loop oracle (``reference.route_token``) and of the kernel's warp reduction; slots therefore come out in
descending order of the selection key.  Scores and weights are fp32 throughout.

    key    = score (+ selection bias)           score = sigmoid(logit) or softmax(logits)
    groups : with n_group > 1 only the topk_group best groups stay eligible; a group is rated by the sum
             of its two best keys when a bias is given, else by its best key
    weight = unbiased score of the picked expert, renormalised over the K picks (+1e-20) if configured,
             times routed_scaling_factor

Behavioural counterpart of ``moeflow/router.py:10-42`` of the reference.
"""

from __future__ import annotations

import torch

from .config import MoEConfig

_NEVER = float("-inf")


def expert_scores(logits: torch.Tensor, cfg: MoEConfig) -> torch.Tensor:
    """fp32 ``[T, E]`` gate scores."""
    z = logits.to(torch.float32)
    if cfg.scoring_func == "sigmoid":
        return z.sigmoid()
    if cfg.scoring_func == "softmax":
        return z.softmax(dim=-1)
    raise ValueError(f"unknown scoring function {cfg.scoring_func!r}")


def _take_best(keys: torch.Tensor, rounds: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``rounds`` times: index and value of the largest remaining key of every row (first one on ties)."""
    remaining = keys.clone()
    rows = torch.arange(keys.shape[0], device=keys.device)
    picked = torch.empty(keys.shape[0], rounds, dtype=torch.int64, device=keys.device)
    values = torch.empty(keys.shape[0], rounds, dtype=keys.dtype, device=keys.device)
    lane = torch.arange(keys.shape[1], device=keys.device).expand_as(keys)
    for r in range(rounds):
        top = remaining.amax(dim=-1, keepdim=True)
        # lowest index among the maxima, spelled out so that the tie rule does not rest on a backend's argmax
        best = torch.where(remaining == top, lane, keys.shape[1]).amin(dim=-1).clamp_(max=keys.shape[1] - 1)
        picked[:, r] = best
        values[:, r] = top[:, 0]
        remaining[rows, best] = _NEVER
    return picked, values


def _eligible_groups(keys: torch.Tensor, cfg: MoEConfig, rated_by_two_best: bool) -> torch.Tensor:
    """bool ``[T, n_group]``: the ``topk_group`` best-rated groups of every token."""
    tokens = keys.shape[0]
    by_group = keys.reshape(tokens, cfg.n_group, -1)
    if rated_by_two_best:
        rating = _take_best(by_group.reshape(tokens * cfg.n_group, -1), 2)[1].sum(dim=-1).reshape(tokens, cfg.n_group)
    else:
        rating = by_group.amax(dim=-1)
    winners, _ = _take_best(rating, cfg.topk_group)
    eligible = torch.zeros(tokens, cfg.n_group, dtype=torch.bool, device=keys.device)
    eligible[torch.arange(tokens, device=keys.device)[:, None], winners] = True
    return eligible


def route(logits: torch.Tensor, bias: torch.Tensor | None, cfg: MoEConfig) -> tuple[torch.Tensor, torch.Tensor]:
    """``logits [T, E]`` -> ``(weights [T, K] fp32, ids [T, K] int32)``, slots by descending selection key."""
    tokens, experts = logits.shape
    score = expert_scores(logits, cfg)
    keys = score if bias is None else score + bias.to(torch.float32)
    if cfg.n_group > 1:
        eligible = _eligible_groups(keys, cfg, rated_by_two_best=bias is not None)
        per_expert = eligible.repeat_interleave(experts // cfg.n_group, dim=1)
        keys = keys.masked_fill(~per_expert, _NEVER)
    ids, _ = _take_best(keys, cfg.top_k)
    weights = score.gather(1, ids)
    if cfg.norm_topk_prob:
        weights = weights / (weights.sum(dim=-1, keepdim=True) + 1e-20)
    return (weights * cfg.routed_scaling_factor).to(torch.float32), ids.to(torch.int32)
