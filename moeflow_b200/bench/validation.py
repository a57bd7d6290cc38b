"""Gates a measurement has to pass before a single timing sample is taken.

``check_reference``             an output against the loop oracle: finite, and within the GEMM tolerance in the
                                norm-wise metric (the record also carries the largest absolute error and the
                                similarity metric other EP libraries report).
``require_matching_variants``   two variants that are meant to be interchangeable must agree byte for byte on
                                *every* rank; identical NaNs do not count as agreement.
``require_matching_graphs``     the same after CUDA-graph capture, checked again after every change of the
                                captured inputs: a graph that silently reads a stale buffer is caught here.
``check_backend_pair``          two backends with different (legitimate) reduction orders: each is held to the
                                oracle separately and their byte equality is only reported.

Same gates as ``scripts/bench/validation.py:11-72`` of the reference.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from ..tolerances import bitwise_equal, calc_diff, gemm_tolerance, normwise_rel_err

REJECTED = "A/B outputs differ on at least one rank; performance measurement rejected"


def _is_finite(*tensors: torch.Tensor) -> bool:
    return all(bool(torch.isfinite(t).all()) for t in tensors)


def check_reference(out: torch.Tensor, ref: torch.Tensor) -> dict:
    tolerance = gemm_tolerance()
    report = {"tokens_checked": int(ref.shape[0]) if ref.dim() > 0 else 0, "tolerance": tolerance,
              "finite": _is_finite(out, ref), "normwise_rel_err": 0.0, "max_abs_err": 0.0, "calc_diff": 0.0}
    if ref.numel() > 0:
        report["normwise_rel_err"] = normwise_rel_err(out, ref)
        report["max_abs_err"] = float((out.to(torch.float32) - ref.to(torch.float32)).abs().max())
        report["calc_diff"] = calc_diff(out, ref)
    report["passed"] = report["finite"] and report["normwise_rel_err"] <= tolerance
    return report


def all_ranks_agree(mine: bool, device=None, group=None) -> bool:
    """Logical AND of ``mine`` over the ranks of ``group`` (just ``mine`` outside a distributed run)."""
    if not (dist.is_available() and dist.is_initialized()):
        return mine
    vote = torch.ones((), dtype=torch.int32, device=device or "cpu") * int(mine)
    dist.all_reduce(vote, op=dist.ReduceOp.MIN, group=group)
    return int(vote) == 1


def require_matching_variants(a: torch.Tensor, b: torch.Tensor, group=None) -> None:
    here = _is_finite(a) and bitwise_equal(a, b)
    if not all_ranks_agree(here, a.device, group):
        raise RuntimeError(REJECTED)


class _CapturedVariant:
    """One variant under graph replay; ``output`` is the tensor its captured call returned."""

    def __init__(self, fn: Callable[[], torch.Tensor], group):
        from .timing import capture

        self.output: torch.Tensor | None = None

        def call_and_keep() -> None:
            self.output = fn()

        self.graph = capture(call_and_keep, group=group)

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.output

    def release(self) -> None:
        self.graph = None  # graphs are dropped before anything else that may own communicator state
        self.output = None


def require_matching_graphs(fn_a, fn_b, update: Callable[[int], None], replays: int, group=None) -> None:
    """Capture both variants; for ``replays`` steps call ``update(step)`` (which rewrites the static input
    buffers in place), replay both graphs and require byte-equal outputs on every rank."""
    variants = [_CapturedVariant(fn_a, group), _CapturedVariant(fn_b, group)]
    try:
        for step in range(replays):
            update(step)
            first, second = (v.replay() for v in variants)
            require_matching_variants(first, second, group)
    finally:
        for v in variants:
            v.release()
        if torch.cuda.is_available():
            torch.cuda.synchronize()


def check_backend_pair(a: torch.Tensor, b: torch.Tensor, ref: torch.Tensor) -> dict:
    verdicts = {name: check_reference(out, ref) for name, out in (("a", a), ("b", b))}
    return {**verdicts, "bitwise_equal": bitwise_equal(a, b), "equality_check": "bytes"}
