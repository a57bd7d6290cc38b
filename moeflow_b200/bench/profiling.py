"""Profiler bracket: cudaProfilerStart/Stop plus an NVTX range around a validated timing region, so
that an external profiler started with a "capture range = cudaProfilerApi" option records only that.
Counterpart of ``scripts/bench/profiling.py:10-22``.
"""

from __future__ import annotations

from contextlib import contextmanager

import torch


@contextmanager
def profile_layer(label: str, enabled: bool = True):
    if not (enabled and torch.cuda.is_available()):
        yield
        return
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    torch.cuda.nvtx.range_push(label)
    try:
        yield
    finally:
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_pop()
        torch.cuda.cudart().cudaProfilerStop()
