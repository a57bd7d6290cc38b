"""Timeline of one fused layer forward from the kernels' own ``globaltimer`` stamps (no profiler needed).

    python -m moeflow_b200.cli.trace_layer --tokens 128 --experts 36

Every kernel of the forward takes an optional trace buffer: the two grouped GEMMs stamp eleven events per CTA
(entry, dependencies met, first weight tile requested, first operand stage complete, first accumulator
complete, last epilogue done, exit, and for the first unit: epilogue done, first 16-column group loaded from
tensor memory, first group stored, all groups stored), the transport kernels stamp CTA 0 (dispatch: entry, routed, rows stored,
fenced, arrivals sent, last CTA done; metadata: entry, dispatch complete, flags seen, histogram, plan written,
entries placed; reduce + push: entry, GEMM complete, row stored, fenced, -, last CTA done; combine: entry,
predecessor complete, return flags seen, row written).  The layer is captured in a CUDA graph, replayed with a
cold L2, and the stamps are printed in microseconds relative to the first one, so the gaps between kernels
(launch chain, grid dependencies, fences) can be read directly.  One GPU; ``--experts`` sets the local expert
count so that a rank's share of a larger EP group can be reproduced.
"""

from __future__ import annotations

import argparse
import dataclasses

import torch

from ..bench.timing import L2Flush
from ..config import GLM53_FLASH_I1536
from ..fixed import FixedEPLayer
from ..testing import make_bias, make_hidden, make_logits

GEMM_EVENTS = ("entry", "deps met", "first weight tile", "first stage full", "first accumulator", "last epilogue", "exit",
               "first epilogue done", "first chunk loaded", "first chunk stored", "first unit stored")
SMALL_EVENTS = {
    "dispatch": ("entry", "routed", "rows stored", "fenced", "arrivals sent", "last CTA done"),
    "metadata": ("entry", "dispatch complete", "flags seen", "histogram", "plan written", "entries placed",
                 "counters cleared", "warp 0 histogram"),
    "reduce+push": ("entry", "GEMM complete", "row stored", "fenced", "-", "last CTA done"),
    "combine": ("entry", "predecessor complete", "flags seen", "row written"),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--experts", type=int, default=288)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--fuse-return", type=int, default=0)
    ap.add_argument("--gemm-kwargs", default="", help="extra FixedEPLayer gemm_kwargs as key=int pairs, comma separated")
    args = ap.parse_args()
    cfg = dataclasses.replace(GLM53_FLASH_I1536, n_routed_experts=args.experts)
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    H, I, E, T = cfg.hidden_size, cfg.moe_intermediate_size, args.experts, args.tokens
    w13 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=dev)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16, device=dev)
    for e in range(E):
        w13[e] = (torch.randn(2 * I, H, generator=g, device=dev) * (2.0 / H**0.5)).bfloat16()
        w2[e] = (torch.randn(H, I, generator=g, device=dev) / I**0.5).bfloat16()
    bias = make_bias(cfg, 1, device=dev)
    extra = {k: int(v) for k, v in (kv.split("=") for kv in args.gemm_kwargs.split(",") if kv)}
    layer = FixedEPLayer(cfg, 0, 1, w13, w2, capacity=T, backend="cuda", gemm_kwargs={"fuse_return": bool(args.fuse_return), **extra})
    n_sms = layer.n_sms
    tr_g1 = torch.zeros(n_sms, 16, dtype=torch.int64, device=dev)
    tr_g2 = torch.zeros_like(tr_g1)
    small = {name: torch.zeros(8, dtype=torch.int64, device=dev) for name in SMALL_EVENTS}
    layer._a_gemm1.trace, layer._a_gemm2.trace = tr_g1.data_ptr(), tr_g2.data_ptr()
    layer._a_dispatch.trace, layer._a_meta.trace = small["dispatch"].data_ptr(), small["metadata"].data_ptr()
    layer._a_reduce.trace, layer._a_combine.trace = small["reduce+push"].data_ptr(), small["combine"].data_ptr()
    x = make_hidden(T, cfg, 3, device=dev)
    lg = make_logits(T, cfg, 4, device=dev)
    flush = L2Flush(device=dev)  # write pass, then a read pass: cold cache, no write-back pending
    for _ in range(3):
        layer.forward(x, lg, bias)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer.forward(x, lg, bias)
    for _ in range(args.reps):
        flush()
        for t in (tr_g1, tr_g2, *small.values()):
            t.zero_()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
    st = layer.check_status()
    print(f"tokens {T}, local experts {E}, plan {layer.plan.tolist()[:6]}, meta CTAs {layer.meta_ctas}, "
          f"status {st['name']}, event time {s.elapsed_time(e) * 1e3:.1f} us")
    stamps = [t[t > 0] for t in (tr_g1, tr_g2, *small.values())]
    base = min(float(t.min()) for t in stamps if t.numel())

    def us(v) -> float:
        return (float(v) - base) / 1e3

    for name, events in SMALL_EVENTS.items():
        t = small[name].cpu()
        row = "  ".join(f"{ev} {us(t[i]):.2f}" for i, ev in enumerate(events) if ev != "-" and int(t[i]) > 0)
        print(f"{name:12s} {row}")
    for name, t in (("gate/up GEMM", tr_g1.cpu().double()), ("down GEMM", tr_g2.cpu().double())):
        print(name)
        for i, ev in enumerate(GEMM_EVENTS):
            col = t[:, i]
            col = col[col > 0]
            if len(col):
                print(f"  {ev:18s} min {us(col.min()):8.2f}  median {us(col.median()):8.2f}  max {us(col.max()):8.2f}  ({len(col)} CTAs)")


if __name__ == "__main__":
    main()
