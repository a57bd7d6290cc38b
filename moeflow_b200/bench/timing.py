"""Multi-rank latency measurement: barrier-aligned start, device-side timing, slowest rank wins.

Each repetition: barrier on all ranks -> CUDA events around ``inner`` back-to-back calls -> per-rank
mean per call -> ``all_reduce(MAX)``.  Graph mode captures ``inner`` calls into one CUDA graph once
and replays it per repetition; a function that cannot be captured is reported as such, never timed
eagerly behind the caller's back.  Optionally an L2 flush (a write larger than L2) precedes every
repetition, outside the timed interval.  Counterpart of ``scripts/bench/timing.py:27-127``.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class TimingResult:
    mode: str
    per_call_us: list[float] = field(default_factory=list)  # one sample per repetition, max over ranks
    inner: int = 1
    capturable: bool = True
    error: str | None = None


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


def max_over_ranks(value: float, group=None) -> float:
    if not _dist_on():
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def aligned_start(group=None) -> None:
    if _dist_on():
        dist.barrier(group=group, device_ids=[torch.cuda.current_device()])
    torch.cuda.synchronize()


class L2Flush:
    """Writes a buffer larger than the 126 MB L2 so that the next kernel starts from HBM."""

    def __init__(self, nbytes: int = 256 << 20, device=None):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device or "cuda")

    def __call__(self) -> None:
        self.buf.zero_()


def _one_sample(run: Callable[[], None], inner: int, group, flush) -> float:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if flush is not None:
        flush()
    aligned_start(group)
    start.record()
    run()
    end.record()
    end.synchronize()
    return max_over_ranks(start.elapsed_time(end) * 1e3 / inner, group)


def time_eager(fn, reps: int = 10, inner: int = 20, warmup: int = 5, group=None, flush=None) -> TimingResult:
    for _ in range(warmup):
        fn()

    def run():
        for _ in range(inner):
            fn()

    return TimingResult("eager", [_one_sample(run, inner, group, flush) for _ in range(reps)], inner)


def capture(fn, warmup: int = 3, inner: int = 1, group=None) -> torch.cuda.CUDAGraph:
    """Capture ``inner`` back-to-back calls (raises when the function cannot be captured)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    aligned_start(group)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(inner):
            fn()
    aligned_start(group)
    return graph


def time_graph(fn, reps: int = 10, inner: int = 20, warmup: int = 3, group=None, flush=None) -> TimingResult:
    try:
        graph = capture(fn, warmup, inner, group)
    except Exception as exc:  # "not capturable" is a result of its own
        torch.cuda.synchronize()
        return TimingResult("graph", [], inner, capturable=False, error=f"{type(exc).__name__}: {exc}"[:500])
    graph.replay()
    samples = [_one_sample(graph.replay, inner, group, flush) for _ in range(reps)]
    del graph  # graphs must go before the process group does
    torch.cuda.synchronize()
    return TimingResult("graph", samples, inner)


def time_graphs_alternating(fn_a, fn_b, reps: int = 10, inner: int = 20, group=None, flush=None):
    """A/B timing: both variants captured, then replayed A, B, A, B, ...; samples are paired by index."""
    graph_a = capture(fn_a, inner=inner, group=group)
    graph_b = capture(fn_b, inner=inner, group=group)
    graph_a.replay()
    graph_b.replay()
    a, b = [], []
    for _ in range(reps):
        a.append(_one_sample(graph_a.replay, inner, group, flush))
        b.append(_one_sample(graph_b.replay, inner, group, flush))
    del graph_a, graph_b
    torch.cuda.synchronize()
    return a, b
