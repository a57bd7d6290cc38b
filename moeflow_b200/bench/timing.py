"""Latency of a multi-rank step, measured on the device.

One *sample* is taken like this (``Stopwatch.sample``): optionally flush L2 (a write larger than the cache, so
the step starts from HBM), line all ranks up at a barrier and drain the device, record a CUDA event, run the
work (``inner`` back-to-back calls, or one replay of a graph that holds them), record the second event, wait
for it, divide by ``inner`` and take the MAX over the ranks: the slowest rank is the step time.  The flush and
the barrier are outside the timed interval.

``time_eager`` calls the function; ``time_graph`` captures ``inner`` calls into one CUDA graph and replays it.
A function that cannot be captured is reported as such (``capturable=False`` with the error text) and is never
silently timed eagerly.  ``time_graphs_alternating`` replays two captured variants A, B, A, B, ... so that
their samples pair up by index for the paired A/B rule.  Graphs are always released before returning, since a
live graph that holds communicator work must not outlive the process group.
Counterpart of ``scripts/bench/timing.py:27-127`` of the reference.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class TimingResult:
    mode: str                                                 # "eager" | "graph"
    per_call_us: list[float] = field(default_factory=list)    # one value per repetition, max over ranks
    inner: int = 1
    capturable: bool = True
    error: str | None = None


def _in_a_group() -> bool:
    return dist.is_available() and dist.is_initialized()


def max_over_ranks(value: float, group=None) -> float:
    if not _in_a_group():
        return value
    box = torch.full((1,), value, dtype=torch.float64, device="cuda")
    dist.all_reduce(box, op=dist.ReduceOp.MAX, group=group)
    return float(box[0])


def aligned_start(group=None) -> None:
    """All ranks at the same point, nothing pending on this device."""
    if _in_a_group():
        dist.barrier(group=group, device_ids=[torch.cuda.current_device()])
    torch.cuda.synchronize()


class L2Flush:
    """Overwrites a buffer larger than the 126 MB L2, then reads a second one of the same size.

    The write evicts whatever ran before.  It also leaves the L2 full of dirty lines, and their write-back would
    compete with the first tens of microseconds of the timed work (measured on B200: cold loads at the start of a
    layer took five times longer right after a plain memset); the read pass replaces them with clean lines, so the
    timed region starts with a cold cache and an idle memory system.
    """

    def __init__(self, nbytes: int = 256 << 20, device=None):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device or "cuda")
        self.clean = torch.zeros(nbytes // 4, dtype=torch.int32, device=device or "cuda")
        self.sink = torch.zeros((), dtype=torch.int32, device=device or "cuda")

    def __call__(self) -> None:
        self.buf.zero_()
        torch.sum(self.clean, dim=0, dtype=torch.int32, out=self.sink)


class Stopwatch:
    """Takes samples of one piece of work under fixed conditions (group, flush, calls per sample)."""

    def __init__(self, inner: int, group=None, flush: Callable[[], None] | None = None):
        self.inner, self.group, self.flush = inner, group, flush
        self.begin = torch.cuda.Event(enable_timing=True)
        self.finish = torch.cuda.Event(enable_timing=True)

    def sample(self, work: Callable[[], None]) -> float:
        """Microseconds per call, slowest rank."""
        if self.flush is not None:
            self.flush()
        aligned_start(self.group)
        self.begin.record()
        work()
        self.finish.record()
        self.finish.synchronize()
        return max_over_ranks(self.begin.elapsed_time(self.finish) * 1000.0 / self.inner, self.group)

    def samples(self, work: Callable[[], None], count: int) -> list[float]:
        return [self.sample(work) for _ in range(count)]


def _repeat(fn: Callable[[], object], times: int) -> Callable[[], None]:
    def run() -> None:
        for _ in range(times):
            fn()

    return run


def time_eager(fn, reps: int = 10, inner: int = 20, warmup: int = 5, group=None, flush=None) -> TimingResult:
    _repeat(fn, warmup)()
    return TimingResult("eager", Stopwatch(inner, group, flush).samples(_repeat(fn, inner), reps), inner)


def capture(fn, warmup: int = 3, inner: int = 1, group=None) -> torch.cuda.CUDAGraph:
    """``inner`` back-to-back calls as one CUDA graph, after ``warmup`` calls on a side stream (lazy
    initialisation must not happen during capture).  Raises whatever the capture raises."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        _repeat(fn, warmup)()
    torch.cuda.current_stream().wait_stream(side)
    aligned_start(group)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        _repeat(fn, inner)()
    aligned_start(group)
    return graph


def time_graph(fn, reps: int = 10, inner: int = 20, warmup: int = 3, group=None, flush=None) -> TimingResult:
    try:
        graph = capture(fn, warmup, inner, group)
    except Exception as problem:  # not being capturable is a finding, not a crash
        torch.cuda.synchronize()
        return TimingResult("graph", [], inner, capturable=False, error=f"{type(problem).__name__}: {problem}"[:500])
    graph.replay()  # one untimed replay
    result = TimingResult("graph", Stopwatch(inner, group, flush).samples(graph.replay, reps), inner)
    del graph
    torch.cuda.synchronize()
    return result


def time_graphs_alternating(fn_a, fn_b, reps: int = 10, inner: int = 20, group=None, flush=None):
    """``(samples of A, samples of B)``, taken in the order A, B, A, B, ..."""
    graphs = [capture(fn, inner=inner, group=group) for fn in (fn_a, fn_b)]
    for graph in graphs:
        graph.replay()
    watch = Stopwatch(inner, group, flush)
    taken: tuple[list[float], list[float]] = ([], [])
    for _ in range(reps):
        for arm, graph in zip(taken, graphs):
            arm.append(watch.sample(graph.replay))
    del graph
    graphs.clear()
    torch.cuda.synchronize()
    return taken
