"""Strict parsing and comparison of raw full-vocabulary logits returned by a serving endpoint.
Counterpart of ``scripts/bench/logits.py:8-50``.
"""

from __future__ import annotations

import hashlib
import math

import numpy as np


def parse_raw_logits(payload, vocab_size: int) -> np.ndarray:
    """``payload``: a list of floats (or of per-step lists) -> float32 array ``[steps, vocab]``.

    Rejects anything that is not exactly ``vocab_size`` finite numbers per step.
    """
    steps = payload if payload and isinstance(payload[0], (list, tuple)) else [payload]
    rows = []
    for i, row in enumerate(steps):
        if len(row) != vocab_size:
            raise ValueError(f"step {i}: expected {vocab_size} logits, got {len(row)}")
        arr = np.asarray(row, dtype=np.float64)
        if not np.all(np.isfinite(arr)):
            raise ValueError(f"step {i}: non-finite logits")
        rows.append(arr.astype(np.float32))
    return np.stack(rows) if rows else np.zeros((0, vocab_size), dtype=np.float32)


def digest(logits: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(logits).tobytes()).hexdigest()


def compare_logits(a: np.ndarray, b: np.ndarray) -> dict:
    """Byte-level comparison plus the usual distances."""
    if a.shape != b.shape:
        return {"bitwise_equal": False, "shape_a": list(a.shape), "shape_b": list(b.shape)}
    same = a.tobytes() == b.tobytes()
    diff = np.abs(a.astype(np.float64) - b.astype(np.float64))
    return {
        "bitwise_equal": same,
        "max_abs_diff": float(diff.max()) if diff.size else 0.0,
        "argmax_equal": bool((a.argmax(-1) == b.argmax(-1)).all()) if a.size else True,
        "sha256_a": digest(a),
        "sha256_b": digest(b),
        "rms_diff": float(math.sqrt((diff**2).mean())) if diff.size else 0.0,
    }
