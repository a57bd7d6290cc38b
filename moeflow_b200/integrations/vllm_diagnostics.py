"""Opt-in eager diagnostics of the fixed path inside a serving engine.  These comparisons synchronise
and are never performance samples.  Counterpart of ``moeflow/integrations/vllm_diagnostics.py:14-113``.
"""

from __future__ import annotations

import json
import os
from itertools import permutations
from pathlib import Path

import torch
import torch.distributed as dist

from ..tolerances import bitwise_equal, normwise_rel_err


def compare_outputs(fixed: torch.Tensor, native: torch.Tensor, is_padding: torch.Tensor | None = None) -> dict:
    """Routed outputs of two paths on identical inputs; rows known to be padding are left out."""
    if fixed.shape != native.shape:
        raise ValueError("Layer output shapes differ")
    if is_padding is not None:
        if tuple(is_padding.shape) != (fixed.shape[0],):
            raise ValueError("Padding mask does not match local rows")
        keep = ~is_padding
        fixed, native = fixed[keep], native[keep]
    finite = bool(torch.isfinite(fixed).all()) and bool(torch.isfinite(native).all())
    measurable = finite and fixed.numel() > 0 and fixed.dtype == native.dtype
    return {
        "padding_known": is_padding is not None,
        "rows_compared": int(fixed.shape[0]),
        "finite": finite,
        "bitwise_equal": bitwise_equal(fixed, native),
        "equality_check": "bytes",
        "normwise_vs_native": normwise_rel_err(fixed, native) if measurable else None,
        "max_abs_diff": (fixed.float() - native.float()).abs().max().item() if finite and fixed.numel() else None,
    }


def compare_reduction_orders(partials: torch.Tensor, native: torch.Tensor) -> dict:
    """Which rounding order of the owner partials ``[R, T, H]`` reproduces ``native`` exactly?

    Tries fp32-sum-then-round, every sequential bf16 order, and (for four owners) the pairwise trees.
    An exact match is diagnostic evidence about the native collective's arithmetic.
    """
    partials, native = partials.detach().cpu(), native.detach().cpu()
    owners = partials.shape[0]
    usable = owners <= 4 and native.numel() > 0 and bool(torch.isfinite(partials).all()) and bool(torch.isfinite(native).all())
    if not usable:
        return {"tested": 0, "exact_matches": []}
    dt = native.dtype
    tried = {"fp32_then_bf16": partials.to(torch.float32).sum(dim=0).to(dt)}
    for order in permutations(range(owners)):
        acc = torch.zeros_like(native)
        for owner in order:
            acc = (acc.to(torch.float32) + partials[owner].to(torch.float32)).to(dt)
        tried["bf16_order_" + "".join(str(o) for o in order)] = acc
    if owners == 4:
        for a, b, c, d in ((0, 1, 2, 3), (0, 2, 1, 3), (0, 3, 1, 2)):
            left = (partials[a].float() + partials[b].float()).to(dt)
            right = (partials[c].float() + partials[d].float()).to(dt)
            tried[f"bf16_pairs_{a}{b}_{c}{d}"] = (left.float() + right.float()).to(dt)
    err = {name: normwise_rel_err(val, native) for name, val in tried.items()}
    best = min(err, key=err.get)
    return {
        "tested": len(tried),
        "exact_matches": [name for name, val in tried.items() if bitwise_equal(val, native)],
        "best_candidate": best,
        "best_normwise_vs_native": err[best],
    }


class FixedLayerProbe:
    """Re-runs the engine's native routed experts on cloned inputs for the first two samples of a
    layer, after all EP ranks agreed (all-reduce MIN over a sentinel file ``<dir>/enabled``) that
    diagnostics are on, and appends one JSON line per sample."""

    def __init__(self, directory: Path, max_samples: int = 2):
        self.directory, self.calls, self.max_samples = Path(directory), 0, max_samples

    def compare(self, experts, hidden, weights, ids, fixed_output, layer_name, capacity, owner_partials=None,
                experts_per_rank=None, ep_group=None, is_padding=None):
        if self.calls >= self.max_samples:
            return
        if hidden.is_cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Fixed layer diagnostics require eager execution")
        if ep_group is None:
            from vllm.distributed import get_ep_group
            from vllm.forward_context import get_forward_context

            ep_group = get_ep_group()
            is_padding = get_forward_context().is_padding
        on = torch.tensor(int((self.directory / "enabled").is_file()), device=hidden.device)
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(on, op=dist.ReduceOp.MIN, group=ep_group.device_group)
        if not int(on.item()):
            return
        self.calls += 1  # ranks without tokens count too: every rank spends the same collective budget
        fixed = fixed_output.clone()
        native = experts.forward_modular(x=hidden.clone(), topk_weights=weights.clone(), topk_ids=ids.clone())
        row = {"layer": layer_name, "ep_rank": ep_group.rank_in_group, "sample": self.calls,
               "execution_rows": int(hidden.shape[0]), "capacity": capacity, **compare_outputs(fixed, native, is_padding)}
        if owner_partials is not None:
            part = owner_partials[:, : hidden.shape[0]].detach().cpu().clone()
            owner_of = torch.div(ids.detach().cpu().to(torch.int64), experts_per_rank, rounding_mode="floor")
            for owner in range(part.shape[0]):
                part[owner].masked_fill_(~(owner_of == owner).any(dim=-1, keepdim=True), 0)
            native_cpu = native.detach().cpu()
            if is_padding is not None:
                keep = ~is_padding.detach().cpu()
                part, native_cpu = part[:, keep], native_cpu[keep]
            row["reduction_candidates"] = compare_reduction_orders(part, native_cpu)
        with (self.directory / f"layer_comparison_pid{os.getpid()}.jsonl").open("a") as sink:
            sink.write(json.dumps(row, allow_nan=False) + "\n")
