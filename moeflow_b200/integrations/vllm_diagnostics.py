"""Opt-in eager diagnostics of the fixed path inside a serving engine.

Everything here synchronises with the host and re-runs work, so it never produces performance samples; it
answers two questions about a layer whose fixed-path output differs from the engine's own:

* how far apart are they (``compare_outputs``: byte equality, norm-wise error, largest difference, with rows
  the engine marked as padding left out), and
* which order of rounding would reproduce the engine's result from the owner ranks' partial rows
  (``compare_reduction_orders``: the hypotheses are written as small expression trees and evaluated with a
  rounding step at every node).

``FixedLayerProbe`` does this for the first samples of every layer once all EP ranks agree that diagnostics
are switched on.  Same record fields as ``moeflow/integrations/vllm_diagnostics.py:14-113`` of the reference.
"""

from __future__ import annotations

import json
import os
from itertools import permutations
from pathlib import Path

import torch
import torch.distributed as dist

from ..tolerances import bitwise_equal, normwise_rel_err

ZERO = "zero"  # leaf of a reduction tree: an accumulator that starts at +0.0


def _without_padding(is_padding, rows: int, *tensors):
    if is_padding is None:
        return tensors
    if tuple(is_padding.shape) != (rows,):
        raise ValueError("Padding mask does not match local rows")
    live = torch.logical_not(is_padding)
    return tuple(t[live] for t in tensors)


def compare_outputs(fixed: torch.Tensor, native: torch.Tensor, is_padding: torch.Tensor | None = None) -> dict:
    """Two routed outputs computed from identical inputs."""
    if fixed.shape != native.shape:
        raise ValueError("Layer output shapes differ")
    fixed, native = _without_padding(is_padding, fixed.shape[0], fixed, native)
    report = {"padding_known": is_padding is not None, "rows_compared": int(fixed.shape[0]), "equality_check": "bytes"}
    report["finite"] = all(bool(torch.isfinite(t).all()) for t in (fixed, native))
    report["bitwise_equal"] = bitwise_equal(fixed, native)
    comparable = report["finite"] and fixed.numel() > 0
    report["normwise_vs_native"] = (
        normwise_rel_err(fixed, native) if comparable and fixed.dtype == native.dtype else None
    )
    report["max_abs_diff"] = float((fixed.to(torch.float32) - native.to(torch.float32)).abs().max()) if comparable else None
    return report


def _reduction_hypotheses(owners: int) -> dict:
    """name -> expression tree over owner indices; a tuple node means "add in fp32, round to the output dtype"."""
    trees = {}
    for order in permutations(range(owners)):
        tree = ZERO
        for owner in order:  # a running accumulator: ((((0 + a) + b) + c) + d)
            tree = (tree, owner)
        trees["bf16_order_" + "".join(str(o) for o in order)] = tree
    if owners == 4:  # the three ways to pair four owners (a two-level tree, as a recursive-halving collective adds)
        for a, b, c, d in ((0, 1, 2, 3), (0, 2, 1, 3), (0, 3, 1, 2)):
            trees[f"bf16_pairs_{a}{b}_{c}{d}"] = ((a, b), (c, d))
    return trees


def _evaluate(tree, partials: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if tree == ZERO:
        return torch.zeros(partials.shape[1:], dtype=dtype)
    if isinstance(tree, int):
        return partials[tree].to(dtype)
    left, right = (_evaluate(branch, partials, dtype).to(torch.float32) for branch in tree)
    return (left + right).to(dtype)


def compare_reduction_orders(partials: torch.Tensor, native: torch.Tensor) -> dict:
    """Which rounding order of the owner partials ``[R, T, H]`` gives exactly ``native [T, H]``?

    Candidates: one fp32 sum rounded once, every running-accumulator order, and for four owners the pairwise
    trees.  Only attempted for up to four owners and finite data (runs on the CPU).
    """
    partials, native = partials.detach().to("cpu"), native.detach().to("cpu")
    owners = int(partials.shape[0])
    if owners > 4 or native.numel() == 0 or not (torch.isfinite(partials).all() and torch.isfinite(native).all()):
        return {"tested": 0, "exact_matches": []}
    results = {"fp32_then_bf16": partials.to(torch.float32).sum(dim=0).to(native.dtype)}
    for name, tree in _reduction_hypotheses(owners).items():
        results[name] = _evaluate(tree, partials, native.dtype)
    distance = {name: normwise_rel_err(value, native) for name, value in results.items()}
    closest = min(distance, key=distance.get)
    return {
        "tested": len(results),
        "exact_matches": [name for name, value in results.items() if bitwise_equal(value, native)],
        "best_candidate": closest,
        "best_normwise_vs_native": distance[closest],
    }


class FixedLayerProbe:
    """Per layer, compares the fixed path with the engine's native routed experts on cloned inputs for the
    first ``max_samples`` calls made while the sentinel file ``<directory>/enabled`` exists on *every* EP rank,
    and appends one JSON line per sample to ``<directory>/layer_comparison_pid<pid>.jsonl``."""

    def __init__(self, directory: Path, max_samples: int = 2):
        self.directory = Path(directory)
        self.max_samples = max_samples
        self.calls = 0

    # The decision is collective (MIN over the ranks' own view of the sentinel) so that every rank spends the
    # same number of collectives whether or not it holds tokens.
    def _switched_on_everywhere(self, device, ep_group) -> bool:
        flag = torch.tensor(1 if (self.directory / "enabled").is_file() else 0, device=device)
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=ep_group.device_group)
        return bool(flag.item())

    @staticmethod
    def _engine_context():
        from vllm.distributed import get_ep_group
        from vllm.forward_context import get_forward_context

        return get_ep_group(), get_forward_context().is_padding

    @staticmethod
    def _partials_of_these_tokens(owner_partials, ids, rows: int, experts_per_rank: int) -> torch.Tensor:
        """Owner partial rows of the live tokens, zeroed where an owner holds none of the token's experts (the
        return buffer keeps stale rows there)."""
        part = owner_partials[:, :rows].detach().to("cpu").clone()
        owner_of_slot = torch.div(ids.detach().to("cpu", torch.int64), experts_per_rank, rounding_mode="floor")
        for owner in range(part.shape[0]):
            untouched = (owner_of_slot != owner).all(dim=-1, keepdim=True)
            part[owner].masked_fill_(untouched, 0)
        return part

    def compare(self, experts, hidden, weights, ids, fixed_output, layer_name, capacity, owner_partials=None,
                experts_per_rank=None, ep_group=None, is_padding=None) -> None:
        if self.calls >= self.max_samples:
            return
        if hidden.is_cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Fixed layer diagnostics require eager execution")
        if ep_group is None:
            ep_group, is_padding = self._engine_context()
        if not self._switched_on_everywhere(hidden.device, ep_group):
            return
        self.calls += 1
        mine = fixed_output.clone()
        theirs = experts.forward_modular(x=hidden.clone(), topk_weights=weights.clone(), topk_ids=ids.clone())
        record = {"layer": layer_name, "ep_rank": ep_group.rank_in_group, "sample": self.calls,
                  "execution_rows": int(hidden.shape[0]), "capacity": capacity}
        record.update(compare_outputs(mine, theirs, is_padding))
        if owner_partials is not None:
            part = self._partials_of_these_tokens(owner_partials, ids, hidden.shape[0], experts_per_rank)
            theirs_cpu = theirs.detach().to("cpu")
            if is_padding is not None:
                live = torch.logical_not(is_padding.detach().to("cpu"))
                part, theirs_cpu = part[:, live], theirs_cpu[live]
            record["reduction_candidates"] = compare_reduction_orders(part, theirs_cpu)
        with (self.directory / f"layer_comparison_pid{os.getpid()}.jsonl").open("a") as sink:
            sink.write(json.dumps(record, allow_nan=False) + "\n")
