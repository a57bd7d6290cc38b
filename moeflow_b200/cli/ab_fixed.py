"""Paired A/B comparison of two layer backends under alternating CUDA-graph replays.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m moeflow_b200.cli.ab_fixed \
        --a reference_fixed --b fused --tokens 1,8,128 --out results/ab.json

Both arms get the same weights and inputs.  Before timing, each arm must pass the oracle gate on every
rank; arms that are meant to be bitwise equal (``--require-bitwise``, e.g. ``torch_fixed`` with two flag
sets) must also match byte for byte on every rank, also under graph replay with changing inputs
(``--graph-check N``).  Timing alternates A, B, A, B ...; the verdict uses the paired rule of
``bench.stats.paired_ab`` (95 % CI of the differences excludes 0 and the median gain exceeds the noise).
Counterpart of ``scripts/ab_fixed.py:33-89`` and ``scripts/ab_native_fixed.py:36-190``.
"""

from __future__ import annotations

import argparse
import statistics

import torch
import torch.distributed as dist

from ..bench.backends import BACKENDS, init_dist, make_backend
from ..bench.record import make_record, write_record
from ..bench.stats import paired_ab, summarize
from ..bench.timing import L2Flush, time_graphs_alternating
from ..bench.validation import check_backend_pair, require_matching_graphs, require_matching_variants
from ..config import GLM53_FLASH_I1536, MoEConfig
from ..testing import make_bias, make_hidden, make_logits
from .bench_layer import local_weights, oracle_check


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--a", required=True, choices=BACKENDS)
    ap.add_argument("--b", required=True, choices=BACKENDS)
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64,128")
    ap.add_argument("--dist", default="uniform")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--inner", type=int, default=20)
    ap.add_argument("--flush", action="store_true")
    ap.add_argument("--require-bitwise", action="store_true")
    ap.add_argument("--graph-check", type=int, default=0, help="replays with changing inputs compared bit for bit")
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
        arm_a = make_backend(args.a, cfg, info, w13, w2, bias, T)
        arm_b = make_backend(args.b, cfg, info, w13, w2, bias, T)
        out_a, out_b = arm_a.run(x, lg).clone(), arm_b.run(x, lg).clone()
        torch.cuda.synchronize()
        gate = {"a": oracle_check(cfg, out_a, x, lg, bias, w13, w2, info.rank, info.world, 8),
                "b": oracle_check(cfg, out_b, x, lg, bias, w13, w2, info.rank, info.world, 8)}
        ok = gate["a"]["passed"] and gate["b"]["passed"]
        if info.world > 1:
            flag = torch.tensor(int(ok), device=info.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(flag.item())
        if not ok:
            raise SystemExit(f"T={T}: an arm failed the oracle gate: {gate}")
        if args.require_bitwise:
            require_matching_variants(out_a, out_b)
            if args.graph_check:
                def update(step, x=x, lg=lg, T=T):
                    x.copy_(make_hidden(T, cfg, 9000 + step * 13 + info.rank, device=info.device))
                    lg.copy_(make_logits(T, cfg, 9500 + step * 13 + info.rank, dist=args.dist, device=info.device))

                require_matching_graphs(lambda: arm_a.run(x, lg), lambda: arm_b.run(x, lg), update, args.graph_check)
        a, b = time_graphs_alternating(lambda: arm_a.run(x, lg), lambda: arm_b.run(x, lg), reps=args.reps, inner=args.inner, flush=flush)
        verdict = paired_ab(a, b)
        points.append({"tokens": T, "gate": gate, "pair": check_backend_pair(out_a, out_b, out_a), "a_us": summarize(a).to_dict(),
                       "b_us": summarize(b).to_dict(), "paired": verdict.to_dict()})
        if info.rank == 0:
            print(f"T={T}: {args.a} {statistics.median(a):.1f} us  {args.b} {statistics.median(b):.1f} us  "
                  f"gain {verdict.median_improvement:+.1f} us  significant={verdict.significant} beneficial={verdict.beneficial}", flush=True)
        del arm_a, arm_b
        torch.cuda.synchronize()
    if info.rank == 0 and args.out:
        write_record(args.out, make_record("ab_fixed", {"a": args.a, "b": args.b, "cfg": cfg.to_dict(), "world": info.world, "dist": args.dist,
                                                        "reps": args.reps, "inner": args.inner, "flush": args.flush}, {"points": points}))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
