"""Acceptance criteria.

* Pure data movement (dispatch, restore, metadata) must be bitwise equal, signed zeros and NaN
  payloads included.
* The expert GEMM path is compared with the fp32 oracle by the normwise relative error
  ``|out - ref|_2 / |ref|_2`` and must stay under ``max(2 * err_baseline, 4 * 2**-8)`` where
  ``err_baseline`` is the error of a trusted bf16 implementation on the same inputs, if known.
* Reductions are deterministic, so two runs on the same input are bitwise equal.

Counterpart of the reference's ``moeflow/tolerances.py:17-44``.
"""

from __future__ import annotations

import torch

BF16_U = 2.0**-8  # unit roundoff of bfloat16
FLOOR_ULPS = 4
K_FACTOR = 2.0


def bitwise_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """True iff both tensors have the same shape, dtype, device and exactly the same bytes."""
    if a.shape != b.shape or a.dtype != b.dtype or a.device != b.device:
        return False
    if a.numel() == 0:
        return True
    raw_a = a.contiguous().view(-1).view(torch.uint8)
    raw_b = b.contiguous().view(-1).view(torch.uint8)
    return bool(torch.equal(raw_a, raw_b))


def normwise_rel_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    r = ref.detach().to(torch.float64)
    diff = (out.detach().to(torch.float64) - r).norm().item()
    scale = r.norm().item()
    return diff if scale == 0.0 else diff / scale


def gemm_tolerance(err_baseline: float | None = None) -> float:
    floor = FLOOR_ULPS * BF16_U
    if err_baseline is None:
        return floor
    return max(floor, K_FACTOR * err_baseline)


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """Similarity metric ``1 - 2<x+1, y+1> / (|x+1|^2 + |y+1|^2)`` (0 means identical)."""
    a = x.to(torch.float64) + 1.0
    b = y.to(torch.float64) + 1.0
    return float(1.0 - 2.0 * (a * b).sum() / ((a * a).sum() + (b * b).sum()))
