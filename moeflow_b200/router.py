"""Vectorised noaux_tc router in PyTorch (CPU/GPU twin of the ``router_topk`` CUDA kernel).

Semantics are fixed by ``moeflow_b200.reference.route_token``; the reference's counterpart is
``moeflow/router.py:10-42``.
"""

from __future__ import annotations

import torch

from .config import MoEConfig


def route(logits: torch.Tensor, bias: torch.Tensor | None, cfg: MoEConfig) -> tuple[torch.Tensor, torch.Tensor]:
    """``logits [T, E]`` -> ``(weights [T, K] fp32, ids [T, K] int32)``, slots by descending biased score.

    Equal scores resolve to the lower expert id (stable sort).
    """
    n_tokens, n_experts = logits.shape
    z = logits.to(torch.float32)
    if cfg.scoring_func == "sigmoid":
        score = z.sigmoid()
    elif cfg.scoring_func == "softmax":
        score = z.softmax(dim=-1)
    else:
        raise ValueError(f"unknown scoring function {cfg.scoring_func!r}")
    key = score if bias is None else score + bias.to(torch.float32)[None, :]

    if cfg.n_group > 1:
        per_group = key.reshape(n_tokens, cfg.n_group, n_experts // cfg.n_group)
        if bias is None:
            strength = per_group.amax(dim=-1)
        else:
            strength = per_group.topk(2, dim=-1).values.sum(dim=-1)
        keep = strength.sort(dim=-1, descending=True, stable=True).indices[:, : cfg.topk_group]
        open_mask = torch.zeros(n_tokens, cfg.n_group, dtype=torch.bool, device=logits.device)
        open_mask.scatter_(1, keep, True)
        key = torch.where(open_mask[:, :, None], per_group, per_group.new_full((), float("-inf"))).reshape(
            n_tokens, n_experts
        )

    ids = key.sort(dim=-1, descending=True, stable=True).indices[:, : cfg.top_k]
    weights = torch.gather(score, 1, ids)
    if cfg.norm_topk_prob:
        weights = weights / (weights.sum(dim=-1, keepdim=True) + 1e-20)
    weights = weights * cfg.routed_scaling_factor
    return weights.to(torch.float32), ids.to(torch.int32)
