"""A profiler window around exactly the region one wants to see.

External profilers can be told to record only between ``cudaProfilerStart`` and ``cudaProfilerStop`` (their
"capture range = CUDA profiler API" mode).  ``ProfilerWindow`` opens that range after a device synchronise,
names it with an NVTX range, and closes both again behind a second synchronise, so weight loading, warm-up and
validation stay out of the capture.  On a machine without CUDA, or when disabled, it does nothing.
Counterpart of ``scripts/bench/profiling.py:10-22`` of the reference.
"""

from __future__ import annotations

import torch


class ProfilerWindow:
    def __init__(self, label: str, enabled: bool = True):
        self.label = label
        self.active = bool(enabled) and torch.cuda.is_available()

    def __enter__(self) -> "ProfilerWindow":
        if self.active:
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStart()
            torch.cuda.nvtx.range_push(self.label)
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        if self.active:
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()
            torch.cuda.cudart().cudaProfilerStop()
        return False


def profile_layer(label: str, enabled: bool = True) -> ProfilerWindow:
    """``with profile_layer("LAYER:fused:T=8", args.profile): ...``"""
    return ProfilerWindow(label, enabled)
