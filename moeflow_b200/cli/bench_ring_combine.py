"""Micro A/B of the source-side combine alone: PyTorch ring loop versus the fused combine kernel.

    python -m moeflow_b200.cli.bench_ring_combine --world 4 --tokens 1,8,128 [--out results/ring.json]

Both arms must agree bit for bit before they are timed.  Counterpart of ``scripts/bench_ring_combine.py:19-68``.
"""

from __future__ import annotations

import argparse
import statistics

import torch

from ..bench.record import make_record, write_record
from ..bench.stats import paired_ab
from ..bench.timing import time_graphs_alternating
from ..bench.validation import require_matching_variants
from ..integrations.vllm_runner_ops import combine_bf16_ring, combine_bf16_ring_fused


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--tokens", default="1,8,128")
    ap.add_argument("--rank", type=int, default=1)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--inner", type=int, default=20)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    points = []
    for T in [int(t) for t in args.tokens.split(",")]:
        g = torch.Generator(device="cuda").manual_seed(T)
        part = torch.randn(args.world, T, args.hidden, generator=g, device="cuda").bfloat16()
        hit = torch.rand(T, args.world, generator=g, device="cuda") > 0.3
        out = torch.empty(T, args.hidden, dtype=torch.bfloat16, device="cuda")
        hit_u8 = hit.to(torch.uint8)
        require_matching_variants(combine_bf16_ring(part, hit, args.rank), combine_bf16_ring_fused(part, hit_u8, args.rank, out))
        a, b = time_graphs_alternating(lambda: combine_bf16_ring(part, hit, args.rank),
                                       lambda: combine_bf16_ring_fused(part, hit_u8, args.rank, out), reps=args.reps, inner=args.inner)
        verdict = paired_ab(a, b)
        points.append({"tokens": T, "torch_us": statistics.median(a), "fused_us": statistics.median(b), "paired": verdict.to_dict()})
        print(f"T={T}: torch {statistics.median(a):.2f} us  fused {statistics.median(b):.2f} us  beneficial={verdict.beneficial}")
    if args.out:
        write_record(args.out, make_record("bench_ring_combine", vars(args), {"points": points}))


if __name__ == "__main__":
    main()
