"""Layer latency versus tokens per rank for one backend, with the oracle gate before every timing.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m moeflow_b200.cli.bench_layer \
        --backend fused --tokens 1,2,4,8,16,32,64,128 --weights synthetic --out results/layer_fused.json

Per capacity T: build the backend, run it once, compare the first min(T, 8) tokens of every rank with
the loop oracle (all ranks must pass; a failure is recorded and that point is not timed), then time it
eagerly and under CUDA-graph replay (barrier-aligned, device events, max over ranks).  The record is
rewritten after every point (``complete: false`` until the end) so that a later hang loses nothing.
Inputs are seeded ``seed * 1000003 + T * 101 + rank``.  Counterpart of ``scripts/bench_layer.py:41-194``.
"""

from __future__ import annotations

import argparse
import dataclasses
import faulthandler
import statistics

import torch
import torch.distributed as dist

from ..bench.backends import BACKENDS, init_dist, make_backend
from ..bench.profiling import profile_layer
from ..bench.record import make_record, write_record
from ..bench.stats import summarize
from ..bench.timing import L2Flush, time_eager, time_graph
from ..bench.validation import check_reference
from ..config import GLM53_FLASH, GLM53_FLASH_I1536, MoEConfig
from ..reference import moe_reference
from ..testing import make_bias, make_hidden, make_logits


def local_weights(cfg: MoEConfig, rank: int, world: int, dev, seed: int):
    """Per-expert seeded weights: expert e gets the same numbers whatever the EP degree."""
    per = cfg.experts_per_rank(world)
    H, I = cfg.hidden_size, cfg.moe_intermediate_size
    w13 = torch.empty(per, 2 * I, H, dtype=torch.bfloat16, device=dev)
    w2 = torch.empty(per, H, I, dtype=torch.bfloat16, device=dev)
    for i in range(per):
        g = torch.Generator(device=dev).manual_seed(seed * 1_000_003 + rank * per + i)
        w13[i] = (torch.randn(2 * I, H, generator=g, device=dev) * (2.0 / H**0.5)).bfloat16()
        w2[i] = (torch.randn(H, I, generator=g, device=dev) / I**0.5).bfloat16()
    return w13, w2


def gather_expert_weights(w13_local, w2_local, ids: set[int], cfg, rank, world):
    """All ranks exchange only the experts the oracle check needs (CPU copies)."""
    per = cfg.experts_per_rank(world)
    mine = {e: (w13_local[e - rank * per].cpu(), w2_local[e - rank * per].cpu()) for e in ids if e // per == rank}
    if world == 1:
        return mine
    wanted = [None] * world
    dist.all_gather_object(wanted, sorted(ids))
    need_from_me = {e for lst in wanted for e in lst if e // per == rank}
    have = {e: (w13_local[e - rank * per].cpu(), w2_local[e - rank * per].cpu()) for e in need_from_me}
    everything = [None] * world
    dist.all_gather_object(everything, have)
    merged = {}
    for part in everything:
        merged.update(part)
    return {e: merged[e] for e in ids}


def oracle_check(cfg, out, x, logits, bias, w13_local, w2_local, rank, world, n_check: int) -> dict:
    from ..reference import route_reference

    n = min(n_check, x.shape[0])
    routes = route_reference(logits[:n].cpu(), None if bias is None else bias.cpu(), cfg)
    ids = {e for r in routes for e, _ in r}
    table = gather_expert_weights(w13_local, w2_local, ids, cfg, rank, world)
    E, H, I = cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size
    sparse13 = {e: t[0] for e, t in table.items()}
    sparse2 = {e: t[1] for e, t in table.items()}

    class _Lookup:
        def __init__(self, d):
            self.d = d

        def __getitem__(self, e):
            return self.d[e]

    ref = moe_reference(x[:n].cpu(), logits[:n].cpu(), None, _Lookup(sparse13), _Lookup(sparse2), cfg, routes=routes)
    del E, H, I
    return check_reference(out[:n].cpu(), ref)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="fused", choices=BACKENDS)
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64,128")
    ap.add_argument("--dist", default="uniform")
    ap.add_argument("--weights", default="synthetic")
    ap.add_argument("--intermediate", type=int, default=1536)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--inner", type=int, default=20)
    ap.add_argument("--flush", action="store_true", help="flush L2 before every repetition")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    info = init_dist()
    cfg = dataclasses.replace(GLM53_FLASH, moe_intermediate_size=args.intermediate)
    if args.small:
        cfg = MoEConfig(hidden_size=512, moe_intermediate_size=256, n_routed_experts=32, top_k=4)
    elif args.intermediate == 1536:
        cfg = GLM53_FLASH_I1536
    if args.weights == "synthetic":
        w13, w2 = local_weights(cfg, info.rank, info.world, info.device, args.seed)
        bias = make_bias(cfg, args.seed + 1, device=info.device)
    else:
        from ..bench.inputs import load_weights

        per = cfg.experts_per_rank(info.world)
        w13, w2, bias = load_weights(args.weights, cfg, info.device, experts=range(info.rank * per, (info.rank + 1) * per))
    flush = L2Flush(device=info.device) if args.flush else None
    points, failed = [], False
    for T in [int(t) for t in args.tokens.split(",")]:
        faulthandler.dump_traceback_later(600, exit=True)
        seed = args.seed * 1_000_003 + T * 101 + info.rank
        x = make_hidden(T, cfg, seed, device=info.device)
        lg = make_logits(T, cfg, seed + 7, dist=args.dist, device=info.device)
        backend = make_backend(args.backend, cfg, info, w13, w2, bias, T)
        out = backend.run(x, lg)
        torch.cuda.synchronize()
        check = oracle_check(cfg, out, x, lg, bias, w13, w2, info.rank, info.world, 8)
        gathered = [check]
        if info.world > 1:
            gathered = [None] * info.world
            dist.all_gather_object(gathered, check)
        point = {"tokens": T, "reference": gathered, "passed": all(c["passed"] for c in gathered)}
        if point["passed"]:
            with profile_layer(f"LAYER:{args.backend}:T={T}", args.profile):
                eager = time_eager(lambda: backend.run(x, lg), reps=args.reps, inner=args.inner, flush=flush)
                graph = time_graph(lambda: backend.run(x, lg), reps=args.reps, inner=args.inner, flush=flush)
            point["eager_us"] = summarize(eager.per_call_us).to_dict()
            point["graph_capturable"] = graph.capturable
            point["graph_us"] = summarize(graph.per_call_us).to_dict() if graph.capturable else None
            point["graph_error"] = graph.error
            if info.rank == 0:
                g = f"{statistics.median(graph.per_call_us):.1f}" if graph.capturable else "not capturable"
                print(f"{args.backend} T={T}: eager {statistics.median(eager.per_call_us):.1f} us, graph {g} us", flush=True)
        else:
            failed = True
            if info.rank == 0:
                print(f"{args.backend} T={T}: REFERENCE CHECK FAILED {gathered}", flush=True)
        points.append(point)
        if info.rank == 0 and args.out:
            write_record(args.out, make_record("bench_layer", {"backend": args.backend, "cfg": cfg.to_dict(), "world": info.world,
                                                               "dist": args.dist, "weights": args.weights, "reps": args.reps, "inner": args.inner,
                                                               "flush": args.flush}, {"points": points}, seed=args.seed, complete=False))
        del backend
        torch.cuda.synchronize()
        if failed:
            break
    faulthandler.cancel_dump_traceback_later()
    if info.rank == 0 and args.out:
        write_record(args.out, make_record("bench_layer", {"backend": args.backend, "cfg": cfg.to_dict(), "world": info.world,
                                                           "dist": args.dist, "weights": args.weights, "reps": args.reps, "inner": args.inner,
                                                           "flush": args.flush}, {"points": points}, seed=args.seed, complete=not failed))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    raise SystemExit(1 if failed else 0)


if __name__ == "__main__":
    main()
