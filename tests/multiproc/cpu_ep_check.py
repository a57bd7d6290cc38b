"""CPU plumbing check on real processes (gloo): fixed layer and variable-size pipeline, EP = world.

One MoE layer, hidden 64, 8 routed experts + 1 shared, top-2, SwiGLU intermediate 128, fp32, weights
N(0, 0.02), softmax scoring with renormalised top-k, 16 tokens per rank.  Every rank checks that
  * the fixed layer over gloo all-to-alls equals the in-process simulation of all ranks bit for bit,
  * the variable-size pipeline over the collective transport does too,
  * both stay within fp32 noise of the loop oracle,
  * a rank that stops participating is noticed by the others through a short collective time-out.
Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from moeflow_b200 import MoEConfig  # noqa: E402
from moeflow_b200.comm import CollectiveRowExchange  # noqa: E402
from moeflow_b200.ep_moe import EPMoELayer, shard_experts, simulate_ep  # noqa: E402
from moeflow_b200.fixed import FixedEPLayer, simulate_fixed  # noqa: E402
from moeflow_b200.reference import moe_reference  # noqa: E402
from moeflow_b200.tolerances import bitwise_equal, normwise_rel_err  # noqa: E402

CFG = MoEConfig(hidden_size=64, moe_intermediate_size=128, n_routed_experts=8, n_shared_experts=1, top_k=2,
                scoring_func="softmax", norm_topk_prob=True)


def make_all(world: int, tokens: int):
    g = torch.Generator().manual_seed(0)
    w13 = torch.randn(CFG.n_routed_experts, 2 * CFG.moe_intermediate_size, CFG.hidden_size, generator=g) * 0.02
    w2 = torch.randn(CFG.n_routed_experts, CFG.hidden_size, CFG.moe_intermediate_size, generator=g) * 0.02
    xs = [torch.randn(tokens, CFG.hidden_size, generator=g) for _ in range(world)]
    lgs = [torch.randn(tokens, CFG.n_routed_experts, generator=g) for _ in range(world)]
    return w13, w2, xs, lgs


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16)
    ap.add_argument("--drop-rank", type=int, default=-1, help="this rank leaves before the last collective")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    w13, w2, xs, lgs = make_all(world, args.tokens)
    mine13, mine2 = shard_experts(w13, w2, rank, world)
    fails = []

    fixed = FixedEPLayer(CFG, rank, world, mine13, mine2, capacity=args.tokens, backend="torch")
    out_fixed = fixed.forward(xs[rank], lgs[rank], None)
    sim_layers = [FixedEPLayer(CFG, r, world, *shard_experts(w13, w2, r, world), capacity=args.tokens, backend="torch")
                  for r in range(world)]
    sim = simulate_fixed(sim_layers, xs, lgs, None)
    if not bitwise_equal(out_fixed, sim[rank]):
        fails.append("fixed over gloo differs from the in-process simulation")
    if not bitwise_equal(fixed.recv.contiguous(), sim_layers[rank].recv.contiguous()):
        fails.append("received rows differ from the simulation")

    naive = EPMoELayer(CFG, rank, world, mine13, mine2, combine_dtype=torch.float32)
    out_naive = naive.forward(xs[rank], lgs[rank], None, CollectiveRowExchange())
    sim_naive = simulate_ep([EPMoELayer(CFG, r, world, *shard_experts(w13, w2, r, world), combine_dtype=torch.float32)
                             for r in range(world)], xs, lgs, None)
    if not bitwise_equal(out_naive, sim_naive[rank]):
        fails.append("variable-size pipeline over gloo differs from the simulation")
    if not bitwise_equal(out_naive, out_fixed):
        fails.append("fixed and variable-size outputs differ")
    err = normwise_rel_err(out_fixed, moe_reference(xs[rank], lgs[rank], None, w13, w2, CFG))
    if err > 1e-5:
        fails.append(f"oracle error {err:.2e}")

    # The engine-facing transport core with stand-in experts (global expert g scales by g + 1): what comes back
    # must equal the closed form sum_k w_k * (id_k + 1) * x, and foreign slots must point at the filler expert.
    from moeflow_b200.integrations.row_transport import VariableRowTransport
    from moeflow_b200.router import route

    transport = VariableRowTransport(CollectiveRowExchange(), CFG.experts_per_rank(world))
    tw, tids = route(lgs[rank], None, CFG)
    got = transport.scatter(xs[rank], tw, tids, CFG.n_routed_experts)
    lo, hi = transport.first_expert, transport.first_expert + transport.num_local_experts
    mine = (got.expert_ids >= lo) & (got.expert_ids < hi)
    if not bool(((got.weights == 0) | mine).all()):
        fails.append("a slot of another rank kept a non-zero weight")
    if int(got.rows_per_local_expert.sum()) != int(mine.sum()):
        fails.append("rows per local expert do not add up to the local slots")
    gain = (torch.where(mine, got.expert_ids + 1, 0).to(torch.float32) * got.weights).sum(dim=1, keepdim=True)
    back = transport.gather(gain * got.hidden, torch.float32, wire_dtype=torch.float32)
    want = ((tids + 1).to(torch.float32) * tw).sum(dim=1, keepdim=True) * xs[rank]
    if not torch.allclose(back, want, rtol=1e-5, atol=1e-6) or transport.busy:
        fails.append("row transport round trip differs from the closed form")

    detected = None
    if args.drop_rank >= 0:
        # The leaving rank exits between steps; the others learn of it when their next collective times out.
        if rank == args.drop_rank:
            print(json.dumps({"rank": rank, "left": True}), flush=True)
            os._exit(0)
        try:
            fixed.forward(xs[rank], lgs[rank], None)
            detected = False
        except Exception as exc:  # the failure is reported on the host, nothing hangs
            detected = True
            print(json.dumps({"rank": rank, "ok": not fails, "fails": fails, "peer_loss_detected": True,
                              "error": type(exc).__name__}), flush=True)
            os._exit(0 if not fails else 1)
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "fails": fails, "err": err})
    dist.destroy_process_group()
    if rank == 0:
        bad = [g for g in gathered if g["fails"]]
        print(json.dumps({"ok": not bad, "world": world, "bad": bad, "max_err": max(g["err"] for g in gathered),
                          "peer_loss_detected": detected}))
        return 1 if bad else 0
    return 0


if __name__ == "__main__":
    sys.exit(main())
