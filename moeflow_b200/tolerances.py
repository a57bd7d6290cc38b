"""What counts as "equal" and "close enough" in this project.

Three kinds of acceptance, from strictest to loosest:

``bitwise_equal``   data movement (dispatch, restore, metadata, combine of identical partials) must reproduce
                    every bit: +0.0 and -0.0 differ, NaNs compare by payload, and so do dtype, shape and device.
                    Deterministic reductions are held to the same standard between two runs.
``gemm_tolerance``  the expert GEMM path is compared with the fp32 oracle by the norm-wise relative error
                    ``|out - ref|_2 / |ref|_2`` (``normwise_rel_err``).  The bound is four bf16 unit roundoffs,
                    or twice the error a trusted bf16 implementation makes on the same inputs if that is larger.
``calc_diff``       a cosine-like similarity used by other EP libraries' tests (0 = identical), kept for
                    cross-checking against their numbers.

``first_difference`` tells where two tensors that should be bitwise equal start to differ.
Same criteria and constants as ``moeflow/tolerances.py:17-44`` of the reference.
"""

from __future__ import annotations

import torch

BF16_U = 2.0**-8   # unit roundoff of bfloat16 (8 significand bits)
FLOOR_ULPS = 4     # the bound never drops below this many roundoffs
K_FACTOR = 2.0     # allowed multiple of the trusted implementation's own error

_SAME_SIZE_INT = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}


def _bits(t: torch.Tensor) -> torch.Tensor:
    """The tensor's storage reinterpreted as integers of the element size (no value conversion)."""
    flat = t.detach().contiguous().reshape(-1)
    return flat.view(_SAME_SIZE_INT[flat.element_size()]) if flat.dtype != torch.bool else flat.to(torch.uint8)


def bitwise_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    same_kind = a.dtype == b.dtype and a.shape == b.shape and a.device == b.device
    return bool(same_kind and (a.numel() == 0 or torch.equal(_bits(a), _bits(b))))


def first_difference(a: torch.Tensor, b: torch.Tensor) -> dict | None:
    """``None`` if bitwise equal, else the reason or the first differing flat index with both values."""
    if a.dtype != b.dtype or a.shape != b.shape or a.device != b.device:
        return {"reason": "dtype, shape or device differ", "a": (str(a.dtype), tuple(a.shape)), "b": (str(b.dtype), tuple(b.shape))}
    if a.numel() == 0:
        return None
    unequal = (_bits(a) != _bits(b)).nonzero()
    if unequal.numel() == 0:
        return None
    at = int(unequal[0])
    return {"index": at, "count": int(unequal.shape[0]), "a": a.reshape(-1)[at].item(), "b": b.reshape(-1)[at].item()}


def normwise_rel_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    """``|out - ref|_2 / |ref|_2`` in fp64 (the absolute error when the reference is all zero)."""
    exact = ref.detach().to(torch.float64)
    miss = float(torch.linalg.vector_norm(out.detach().to(torch.float64) - exact))
    size = float(torch.linalg.vector_norm(exact))
    return miss / size if size > 0.0 else miss


def gemm_tolerance(err_baseline: float | None = None) -> float:
    bound = FLOOR_ULPS * BF16_U
    if err_baseline is not None:
        bound = max(bound, K_FACTOR * err_baseline)
    return bound


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """``1 - 2 <x+1, y+1> / (|x+1|^2 + |y+1|^2)``."""
    u = x.detach().to(torch.float64).add(1.0).reshape(-1)
    v = y.detach().to(torch.float64).add(1.0).reshape(-1)
    return float(1.0 - 2.0 * torch.dot(u, v) / (torch.dot(u, u) + torch.dot(v, v)))
