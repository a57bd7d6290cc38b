"""Stage breakdown without a profiler: time CUDA-graph prefixes of the layer and difference them.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m moeflow_b200.cli.bench_stages \
        --tokens 1,8,128 --out results/stages.json

For every capacity T the layer is captured up to each stage (``forward(stop_after=...)``); the time of a
stage is the difference between consecutive prefixes (max over ranks, median over repetitions).  The
padding cost of the fixed layout is the full-layer time with one valid row versus T valid rows.
Counterpart of ``scripts/bench_stages.py:30-93``.
"""

from __future__ import annotations

import argparse
import statistics

import torch
import torch.distributed as dist

from ..bench.backends import init_dist
from ..bench.record import make_record, write_record
from ..bench.timing import L2Flush, time_graph
from ..config import GLM53_FLASH_I1536, MoEConfig
from ..fixed import CUDA_SUBSTAGES, STAGES, FixedEPLayer
from ..testing import make_bias, make_hidden, make_logits


def _weights(cfg: MoEConfig, rank: int, world: int, dev):
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    L, H, I = cfg.experts_per_rank(world), cfg.hidden_size, cfg.moe_intermediate_size
    w13 = torch.empty(L, 2 * I, H, dtype=torch.bfloat16, device=dev)
    w2 = torch.empty(L, H, I, dtype=torch.bfloat16, device=dev)
    for e in range(L):
        w13[e] = (torch.randn(2 * I, H, generator=g, device=dev) * (2.0 / H**0.5)).bfloat16()
        w2[e] = (torch.randn(H, I, generator=g, device=dev) / I**0.5).bfloat16()
    return w13, w2


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,8,128")
    ap.add_argument("--dist", default="uniform")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--inner", type=int, default=1)
    ap.add_argument("--backend", default="cuda", choices=["cuda", "torch"])
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--small", action="store_true", help="small layer shape (smoke runs)")
    ap.add_argument("--experts", type=int, default=None, help="override the routed expert count (keeps hidden/intermediate)")
    ap.add_argument("--only-full", action="store_true", help="time only the whole layer (profiling runs)")
    ap.add_argument("--block-m", type=int, default=None, help="token rows per GEMM tile (32, 64, 128, 256); default: chosen by the layer")
    ap.add_argument("--meta-ctas", type=int, default=None, help="CTAs of the metadata pass (1 = single-CTA kernel); default: by size")
    ap.add_argument("--permute-rows", action="store_true",
                    help="copy received rows into expert-major order so the gate/up GEMM reads token tiles by TMA")
    ap.add_argument("--fuse-return", type=int, default=None, help="1/0: owner reduce + return push inside the down GEMM or as its own kernel")
    ap.add_argument("--tile-handover", type=int, default=None, help="1/0: the down GEMM starts a tile when its activations are final, or after the whole gate/up grid")
    ap.add_argument("--stream-k", type=int, default=None, help="1/0: allow the stream-K cut of the GEMMs' K steps or K splits only")
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 expert weights (quantised from the bf16 ones)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    info = init_dist()
    cfg = MoEConfig(hidden_size=512, moe_intermediate_size=256, n_routed_experts=32, top_k=4) if args.small else GLM53_FLASH_I1536
    if args.experts is not None:
        import dataclasses

        cfg = dataclasses.replace(cfg, n_routed_experts=args.experts)
    w13, w2 = _weights(cfg, info.rank, info.world, info.device)
    bias = make_bias(cfg, 1, device=info.device)
    fp8_pack = None
    if args.fp8:
        from ..weights import quant_block_fp8

        def pack(w):
            qs, ss = zip(*(quant_block_fp8(w[e]) for e in range(w.shape[0])))
            return torch.stack([q.view(torch.uint8) for q in qs]).view(torch.float8_e4m3fn), torch.stack(ss)

        q13, s13 = pack(w13)
        q2, s2 = pack(w2)
        fp8_pack = (q13, s13, q2, s2)
    flush = None if args.no_flush else L2Flush(device=info.device)
    stages = list(STAGES)
    if args.only_full:
        stages = ["COMBINE"]
    elif args.backend == "cuda":
        at = stages.index("EXPERT")
        stages = stages[:at] + list(CUDA_SUBSTAGES) + stages[at:]
    points = []
    for T in [int(t) for t in args.tokens.split(",")]:
        layer = FixedEPLayer(cfg, info.rank, info.world, w13, w2, capacity=T, backend=args.backend,
                             gemm_kwargs={**({"block_m": args.block_m} if args.block_m else {}),
                                          **({"fp8_weights": True} if args.fp8 else {}),
                                          **({"meta_ctas": args.meta_ctas} if args.meta_ctas else {}),
                                          **({"permute_rows": True} if args.permute_rows else {}),
                                          **({"stream_k": args.stream_k} if args.stream_k is not None else {}),
                                          **({"tile_handover": bool(args.tile_handover)} if args.tile_handover is not None else {}),
                                          **({"fuse_return": bool(args.fuse_return)} if args.fuse_return is not None else {})})
        if args.fp8:
            layer.set_weights_fp8(*fp8_pack)
        x = make_hidden(T, cfg, 300 + T + info.rank, device=info.device)
        lg = make_logits(T, cfg, 400 + T + info.rank, dist=args.dist, device=info.device)
        prefix_us = {}
        for st in stages:
            res = time_graph(lambda st=st: layer.forward(x, lg, bias, stop_after=st), reps=args.reps, inner=args.inner,
                             flush=flush)
            prefix_us[st] = statistics.median(res.per_call_us) if res.capturable else None
        one = torch.ones((), dtype=torch.int32, device=info.device)
        full = torch.full((), T, dtype=torch.int32, device=info.device)
        pad = {}
        for name, nv in (("valid_1", one), ("valid_T", full)):
            res = time_graph(lambda nv=nv: layer.forward(x, lg, bias, num_valid=nv), reps=args.reps, inner=args.inner, flush=flush)
            pad[name] = statistics.median(res.per_call_us) if res.capturable else None
        stage_us, prev = {}, 0.0
        for st in stages:
            if prefix_us[st] is not None:
                stage_us[st] = prefix_us[st] - prev
                prev = prefix_us[st]
        status = layer.check_status() if args.backend == "cuda" else {"code": 0}
        points.append({"tokens": T, "prefix_us": prefix_us, "stage_us": stage_us, "padding": pad, "status": status})
        if info.rank == 0:
            print(f"T={T}: " + "  ".join(f"{k}={v:.1f}" for k, v in stage_us.items()) + f"  | full {prefix_us['COMBINE']:.1f} us, one valid row {pad['valid_1']:.1f} us", flush=True)
        del layer
        torch.cuda.synchronize()
    if info.rank == 0 and args.out:
        write_record(args.out, make_record("bench_stages", {"cfg": cfg.to_dict(), "world": info.world, "backend": args.backend,
                                                             "dist": args.dist, "flush": not args.no_flush}, {"points": points}))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
