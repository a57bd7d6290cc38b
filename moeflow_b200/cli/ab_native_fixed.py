"""Paired comparison of the serving engine's native expert-parallel path with the fixed-capacity layer.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m moeflow_b200.cli.ab_native_fixed \
        --tokens 1,2,4,8,16,32,64,128 --check-graph-replays 1000 --out results/native_vs_fixed.json

Arm A (``--a``, default ``vllm_agrs``): all-gather of hidden rows and routing, the engine's fused experts on the
gathered batch, reduce-scatter (NCCL).  Arm B (``--b``, default ``fused``): the fused peer-memory layer with the
tcgen05 experts; ``--b fixed_vllm_experts`` keeps the engine's expert kernel and changes only the transport, the
pairing the reference publishes.  The two arms use different (legitimate) reduction orders, so they are not
compared with each other bit for bit: each is held to the loop oracle on every rank, and with
``--check-graph-replays N`` each arm's CUDA graph is replayed N times on changing inputs and every replay must
equal an eager run of the same arm on the same inputs byte for byte on every rank, before any timing sample is
taken.  Timing alternates A, B, A, B ... graph replays; the verdict is the paired rule of ``bench.stats``.
Counterpart of ``scripts/ab_native_fixed.py:36-190``.
"""

from __future__ import annotations

import argparse
import statistics

import torch
import torch.distributed as dist

from ..bench.backends import BACKENDS, init_dist, make_backend
from ..bench.record import make_record, write_record
from ..bench.stats import paired_ab, summarize
from ..bench.timing import L2Flush, capture, time_graphs_alternating
from ..bench.validation import all_ranks_agree, check_backend_pair
from ..config import GLM53_FLASH_I1536, MoEConfig
from ..testing import make_bias, make_hidden, make_logits
from ..tolerances import bitwise_equal
from .bench_layer import local_weights, oracle_check


def replay_check(arm, x, lg, update, replays: int) -> bool:
    """Replay ``arm``'s graph ``replays`` times on changing inputs; every replay must equal an eager run of the
    same arm on the same inputs byte for byte (this rank's verdict)."""
    kept = {}

    def call():
        kept["out"] = arm.run(x, lg)

    graph = capture(call)
    ok = True
    try:
        for step in range(replays):
            update(step)
            graph.replay()
            got = kept["out"].clone()
            want = arm.run(x, lg).clone()
            torch.cuda.synchronize()
            if not (bool(torch.isfinite(got.float()).all()) and bitwise_equal(got, want)):
                ok = False
                break
    finally:
        graph = None
        torch.cuda.synchronize()
    return ok


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--a", default="vllm_agrs", choices=BACKENDS)
    ap.add_argument("--b", default="fused", choices=BACKENDS)
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64,128")
    ap.add_argument("--dist", default="uniform")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--inner", type=int, default=20)
    ap.add_argument("--flush", action="store_true", help="flush L2 before every repetition")
    ap.add_argument("--check-graph-replays", type=int, default=0)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    info = init_dist()
    cfg = MoEConfig(hidden_size=512, moe_intermediate_size=256, n_routed_experts=32, top_k=4) if args.small else GLM53_FLASH_I1536
    w13, w2 = local_weights(cfg, info.rank, info.world, info.device, 0)
    bias = make_bias(cfg, 1, device=info.device)
    flush = L2Flush(device=info.device) if args.flush else None
    points = []
    for T in [int(t) for t in args.tokens.split(",")]:
        x = make_hidden(T, cfg, 300 + T + info.rank, device=info.device)
        lg = make_logits(T, cfg, 400 + T + info.rank, dist=args.dist, device=info.device)
        arms = {"a": make_backend(args.a, cfg, info, w13, w2, bias, T), "b": make_backend(args.b, cfg, info, w13, w2, bias, T)}
        outs = {k: arm.run(x, lg).clone() for k, arm in arms.items()}
        torch.cuda.synchronize()
        gate = {k: oracle_check(cfg, outs[k], x, lg, bias, w13, w2, info.rank, info.world, 8) for k in arms}
        if not all_ranks_agree(all(g["passed"] for g in gate.values()), info.device):
            raise SystemExit(f"T={T}: an arm failed the oracle gate: {gate}")
        replays_ok = None
        if args.check_graph_replays:
            def update(step, x=x, lg=lg, T=T):
                x.copy_(make_hidden(T, cfg, 9000 + step * 13 + info.rank, device=info.device))
                lg.copy_(make_logits(T, cfg, 9500 + step * 13 + info.rank, dist=args.dist, device=info.device))

            replays_ok = {}
            for k, arm in arms.items():
                replays_ok[k] = all_ranks_agree(replay_check(arm, x, lg, update, args.check_graph_replays), info.device)
            if not all(replays_ok.values()):
                raise SystemExit(f"T={T}: graph replays differ from eager runs: {replays_ok}")
        a, b = time_graphs_alternating(lambda: arms["a"].run(x, lg), lambda: arms["b"].run(x, lg), reps=args.reps,
                                       inner=args.inner, flush=flush)
        verdict = paired_ab(a, b)
        points.append({"tokens": T, "gate": gate, "graph_replays": args.check_graph_replays, "replays_ok": replays_ok,
                       "pair": check_backend_pair(outs["a"], outs["b"], outs["a"]), "a_us": summarize(a).to_dict(),
                       "b_us": summarize(b).to_dict(), "paired": verdict.to_dict()})
        if info.rank == 0:
            print(f"T={T}: {args.a} {statistics.median(a):.1f} us  {args.b} {statistics.median(b):.1f} us  "
                  f"gain {verdict.median_improvement:+.1f} us  significant={verdict.significant} beneficial={verdict.beneficial}",
                  flush=True)
        arms.clear()
        torch.cuda.synchronize()
    if info.rank == 0 and args.out:
        write_record(args.out, make_record("ab_native_fixed", {"a": args.a, "b": args.b, "cfg": cfg.to_dict(), "world": info.world,
                                                               "dist": args.dist, "reps": args.reps, "inner": args.inner,
                                                               "flush": args.flush, "graph_replays": args.check_graph_replays},
                                           {"points": points}))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
