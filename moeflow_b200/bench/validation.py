"""Gates that run before any performance sample is taken.

* ``check_reference``: output vs the loop oracle under the frozen GEMM tolerance, finiteness included.
* ``require_matching_variants``: two variants must agree bit for bit **on every rank** (and be finite:
  identical NaNs do not pass) before either is timed.
* ``require_matching_graphs``: the same under CUDA-graph replay with inputs changing between replays.

Counterpart of ``scripts/bench/validation.py:11-72``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..tolerances import bitwise_equal, calc_diff, gemm_tolerance, normwise_rel_err


def check_reference(out: torch.Tensor, ref: torch.Tensor) -> dict:
    empty = ref.numel() == 0
    err = 0.0 if empty else normwise_rel_err(out, ref)
    finite = bool(torch.isfinite(out).all()) and bool(torch.isfinite(ref).all())
    tol = gemm_tolerance()
    return {
        "tokens_checked": int(ref.shape[0]) if ref.dim() else 0,
        "normwise_rel_err": err,
        "max_abs_err": 0.0 if empty else float((out.float() - ref.float()).abs().max()),
        "calc_diff": 0.0 if empty else calc_diff(out, ref),
        "finite": finite,
        "tolerance": tol,
        "passed": finite and err <= tol,
    }


def all_ranks_agree(flag: bool, device=None, group=None) -> bool:
    if not (dist.is_available() and dist.is_initialized()):
        return flag
    t = torch.tensor(int(flag), device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return bool(t.item())


def require_matching_variants(a: torch.Tensor, b: torch.Tensor, group=None) -> None:
    same = bitwise_equal(a, b) and bool(torch.isfinite(a).all())
    if not all_ranks_agree(same, a.device, group):
        raise RuntimeError("A/B outputs differ on at least one rank; performance measurement rejected")


def require_matching_graphs(fn_a, fn_b, update, replays: int, group=None) -> None:
    """Capture both functions, then compare their outputs after every input update."""
    from .timing import capture

    holder: dict[str, torch.Tensor] = {}

    def recorder(key, fn):
        def run():
            holder[key] = fn()

        return run

    graph_a = capture(recorder("a", fn_a), group=group)
    graph_b = capture(recorder("b", fn_b), group=group)
    try:
        for step in range(replays):
            update(step)
            graph_a.replay()
            graph_b.replay()
            require_matching_variants(holder["a"], holder["b"], group)
    finally:
        del graph_a, graph_b
        holder.clear()
        if torch.cuda.is_available():
            torch.cuda.synchronize()


def check_backend_pair(a: torch.Tensor, b: torch.Tensor, ref: torch.Tensor) -> dict:
    """Backends with different reduction orders may round differently: judge each against the oracle."""
    return {"a": check_reference(a, ref), "b": check_reference(b, ref), "bitwise_equal": bitwise_equal(a, b),
            "equality_check": "bytes"}
