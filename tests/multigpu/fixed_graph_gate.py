"""Graph-replay gate of the fused layer over real peer memory (launch with torch.distributed.run).

What a serving engine does to the layer, at the strength of the reference's own gate
(``tests/multigpu/fixed_graph_check.py:57-205`` there): several capacities are captured side by side and
replayed in a random interleaving for many steps, every rank with its own random number of valid rows, and
one buffer set is shared by two weight sets (as a decoder shares one layer object between its MoE blocks).

  G1  every rank replays the same sequence of (capacity, weight set) graphs (the sequences are gathered
      and compared at the end; a rank that took another branch would leave its peers waiting);
  G2  buffers keep their addresses;
  G3  after every replay the output is **bitwise** equal to an eager forward of a second cuda-backend layer
      of the same capacity on the same inputs (same kernels, so the bits must match: a replay that picked
      up a stale row of another capacity's or another weight set's forward would not), padding rows are
      exactly zero;
  G4  every 50th replay is also held to the torch twin (NCCL all-to-all) within the GEMM tolerance;
  G5  graphs are dropped before the process group is destroyed.

Rank 0 prints one JSON line and exits non-zero on any failure.
"""

from __future__ import annotations

import argparse
import faulthandler
import json
import os
import sys
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from moeflow_b200 import MoEConfig  # noqa: E402
from moeflow_b200.fixed import FixedEPLayer  # noqa: E402
from moeflow_b200.testing import make_bias, make_hidden, make_logits, make_weights  # noqa: E402
from moeflow_b200.tolerances import bitwise_equal, normwise_rel_err  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--capacities", default="1,8,64,128")
    ap.add_argument("--replays", type=int, default=1000)
    ap.add_argument("--hidden", type=int, default=512)
    ap.add_argument("--inter", type=int, default=256)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--watchdog", type=int, default=500)
    args = ap.parse_args()

    faulthandler.dump_traceback_later(args.watchdog, exit=True)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=timedelta(seconds=args.watchdog))
    cfg = MoEConfig(hidden_size=args.hidden, moe_intermediate_size=args.inter, n_routed_experts=args.experts,
                    top_k=args.top_k)
    L = cfg.experts_per_rank(world)
    bias = make_bias(cfg, 1, device=dev)
    shards = []
    for seed in (0, 7):  # two weight sets sharing every buffer set
        w13, w2 = make_weights(cfg, seed)
        shards.append((w13[rank * L:(rank + 1) * L].to(dev).contiguous(), w2[rank * L:(rank + 1) * L].to(dev).contiguous()))
    caps = [int(c) for c in args.capacities.split(",")]
    failures: list[str] = []
    worst = 0.0

    class Arm:
        def __init__(self, cap: int):
            self.cap = cap
            self.graphed = FixedEPLayer(cfg, rank, world, *shards[0], capacity=cap, backend="cuda", wait_ns=5_000_000_000)
            self.eager = FixedEPLayer(cfg, rank, world, *shards[0], capacity=cap, backend="cuda", wait_ns=5_000_000_000)
            self.twin = FixedEPLayer(cfg, rank, world, *shards[0], capacity=cap, backend="torch")
            self.maps = [self.graphed.make_weight_maps(*sh) for sh in shards]
            self.x = torch.zeros(cap, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
            self.lg = torch.zeros(cap, cfg.n_routed_experts, device=dev)
            self.nv = torch.full((), cap, dtype=torch.int32, device=dev)
            self.addrs = self._addresses()
            self.graphs, self.outs = [], []

        def _addresses(self):
            g = self.graphed
            return (g._recv_store.data_ptr(), g.ret_recv.data_ptr(), g.out.data_ptr())

        def capture(self):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for w in range(len(shards)):
                    self.graphed.bind_weights(*shards[w], *self.maps[w])
                    self.graphed.forward(self.x, self.lg, bias, self.nv)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            dist.barrier()
            for w in range(len(shards)):
                self.graphed.bind_weights(*shards[w], *self.maps[w])
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    out = self.graphed.forward(self.x, self.lg, bias, self.nv)
                self.graphs.append(g)
                self.outs.append(out)
                torch.cuda.synchronize()
                dist.barrier()

    arms = {c: Arm(c) for c in caps}
    for c in caps:  # all graphs exist side by side before the first replay
        arms[c].capture()

    shared = torch.Generator().manual_seed(4242)       # the same schedule on every rank
    private = torch.Generator().manual_seed(100 + rank)  # this rank's own valid prefixes
    sequence = []
    for step in range(args.replays):
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
        cap = caps[int(torch.randint(0, len(caps), (1,), generator=shared))]
        wset = int(torch.randint(0, len(shards), (1,), generator=shared))
        arm = arms[cap]
        sequence.append((cap, wset))
        t = int(torch.randint(0, cap + 1, (1,), generator=private))
        arm.x.copy_(make_hidden(cap, cfg, 50_000 + 17 * step + rank, device=dev))
        arm.lg.copy_(make_logits(cap, cfg, 90_000 + 17 * step + rank, device=dev))
        arm.nv.fill_(t)
        arm.graphs[wset].replay()
        got = arm.outs[wset]
        arm.eager.bind_weights(*shards[wset])
        want = arm.eager.forward(arm.x, arm.lg, bias, arm.nv)
        torch.cuda.synchronize()
        if not bitwise_equal(got, want):
            failures.append(f"replay {step} (capacity {cap}, weights {wset}): differs from the eager forward")
        if got[t:].abs().sum() != 0:
            failures.append(f"replay {step}: padding rows not zero")
        if step % 50 == 0 or step == args.replays - 1:
            arm.twin.bind_weights(*shards[wset])
            ref = arm.twin.forward(arm.x, arm.lg, bias, arm.nv)
            torch.cuda.synchronize()
            if t:
                err = normwise_rel_err(got[:t], ref[:t].float())
                worst = max(worst, err)
                if err > 4 * 2.0**-8:
                    failures.append(f"replay {step}: error vs twin {err:.3e}")
        if len(failures) > 8:
            break
    torch.cuda.synchronize()
    for c in caps:
        for ly in (arms[c].graphed, arms[c].eager):
            st = ly.check_status()
            if st["code"] != 0:
                failures.append(f"capacity {c}: status {st}")
        if arms[c].addrs != arms[c]._addresses():
            failures.append(f"capacity {c}: buffer addresses moved")

    # G5: graphs go first
    for c in caps:
        arms[c].graphs.clear()
        arms[c].outs.clear()
    torch.cuda.synchronize()
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "failures": failures[:5], "worst": worst, "sequence": sequence})
    dist.barrier()
    dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()
    if rank == 0:
        bad = [{"rank": g["rank"], "failures": g["failures"]} for g in gathered if g["failures"]]
        same = all(g["sequence"] == gathered[0]["sequence"] for g in gathered)
        if not same:
            bad.append({"rank": -1, "failures": ["ranks replayed different graph sequences"]})
        print(json.dumps({"ok": not bad, "world": world, "replays": len(sequence), "capacities": caps,
                          "worst_err": max(g["worst"] for g in gathered), "bad": bad}))
        return 1 if bad else 0
    return 0


if __name__ == "__main__":
    sys.exit(main())
