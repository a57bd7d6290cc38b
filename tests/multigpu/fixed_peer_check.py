"""Multi-GPU check of the cuda backend over real peer memory (launch with torch.distributed.run).

Every rank builds the fused layer (peer-memory dispatch/return) and a torch-backend twin that moves
the same rows with NCCL all_to_all_single, then checks, on every rank:

  G1  dispatch: routing metadata of all received rows and the hidden lanes of valid rows are
      bitwise equal to the twin's receive buffer;
  G2  buffers keep their addresses across forwards;
  G3  outputs are within the GEMM tolerance of the twin and of the loop oracle (first tokens), padding
      rows are exactly zero, for eager forwards with changing inputs and per-rank valid prefixes;
  G4  the same under CUDA-graph replay (hundreds of replays, inputs and valid prefixes changing);
  G5  graphs are dropped before the process group is destroyed.

Results are gathered on rank 0, which prints one JSON line and exits non-zero on any failure.
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
from moeflow_b200.reference import moe_reference  # noqa: E402
from moeflow_b200.testing import make_bias, make_hidden, make_logits, make_weights  # noqa: E402
from moeflow_b200.tolerances import bitwise_equal, normwise_rel_err  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--capacity", type=int, default=16)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--replays", type=int, default=200)
    ap.add_argument("--dist", default="uniform")
    ap.add_argument("--hidden", type=int, default=512)
    ap.add_argument("--inter", type=int, default=256)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--watchdog", type=int, default=240)
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
    w13, w2 = make_weights(cfg, 0)
    bias = make_bias(cfg, 1, device=dev)
    w13_l, w2_l = w13[rank * L:(rank + 1) * L].to(dev).contiguous(), w2[rank * L:(rank + 1) * L].to(dev).contiguous()
    cap = args.capacity
    fused = FixedEPLayer(cfg, rank, world, w13_l, w2_l, capacity=cap, backend="cuda", wait_ns=5_000_000_000,
                         gemm_kwargs={"skip_payload": 0})
    twin = FixedEPLayer(cfg, rank, world, w13_l, w2_l, capacity=cap, backend="torch")
    failures: list[str] = []
    worst = 0.0
    addrs = (fused._recv_store.data_ptr(), fused.ret_recv.data_ptr(), fused.out.data_ptr())
    gen = torch.Generator().manual_seed(100 + rank)

    def inputs(step: int):
        t = int(torch.randint(0, cap + 1, (1,), generator=gen)) if step % 3 else cap
        x = make_hidden(t, cfg, 1000 * step + rank, device=dev)
        lg = make_logits(t, cfg, 2000 * step + rank, dist=args.dist, device=dev)
        return t, x, lg

    # G1..G3: eager forwards
    for step in range(args.iters):
        t, x, lg = inputs(step)
        # one routing decision for both layers, so that the received rows can be compared bit for bit
        w, ids = fused.stage_route(lg, bias)
        w, ids = w.clone(), ids.clone()
        out = fused.forward_routed(x, w, ids)
        out = torch.cat([out, fused.out[t:]]).clone()
        ref = twin.forward_routed(x, w, ids)
        ref = torch.cat([ref, ref.new_zeros(cap - t, cfg.hidden_size)])
        torch.cuda.synchronize()
        st = fused.check_status()
        if st["code"] != 0:
            failures.append(f"step {step}: status {st}")
            break
        meta_f = fused._meta_view(fused._recv_store)
        meta_t = twin._meta_view(twin._recv_store)
        if not torch.equal(meta_f, meta_t):
            failures.append(f"step {step}: received metadata differs")
        valid = meta_t[:, :, 2 * cfg.top_k] != 0
        if not bitwise_equal(fused.recv[:, :, : cfg.hidden_size][valid], twin.recv[:, :, : cfg.hidden_size][valid]):
            failures.append(f"step {step}: received hidden rows differ")
        if out[t:].abs().sum() != 0:
            failures.append(f"step {step}: padding rows not zero")
        if t:
            err = normwise_rel_err(out[:t], ref[:t].float())
            worst = max(worst, err)
            if err > 4 * 2.0**-8:
                failures.append(f"step {step}: error vs twin {err:.3e}")
        if step == 0 and t:
            n = min(t, 4)
            w13_all, w2_all = w13.float(), w2.float()
            oracle = moe_reference(x[:n].cpu(), lg[:n].cpu(), bias.cpu(), w13_all, w2_all, cfg)
            err = normwise_rel_err(out[:n].cpu(), oracle)
            if err > 4 * 2.0**-8:
                failures.append(f"oracle error {err:.3e}")
    if addrs != (fused._recv_store.data_ptr(), fused.ret_recv.data_ptr(), fused.out.data_ptr()):
        failures.append("buffer addresses moved")

    # G4: graph replay with changing inputs and valid prefixes
    xs = torch.zeros(cap, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
    lgs = torch.zeros(cap, cfg.n_routed_experts, device=dev)
    nv = torch.full((), cap, dtype=torch.int32, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fused.forward(xs, lgs, bias, nv)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g_out = fused.forward(xs, lgs, bias, nv)
    torch.cuda.synchronize()
    dist.barrier()
    for step in range(args.replays):
        t, x, lg = inputs(10_000 + step)
        xs[:t].copy_(x)
        lgs[:t].copy_(lg)
        nv.fill_(t)
        graph.replay()
        if step % 10 == 0 or step == args.replays - 1:
            ref = twin.forward(xs, lgs, bias, nv)
            torch.cuda.synchronize()
            if g_out[t:].abs().sum() != 0:
                failures.append(f"replay {step}: padding rows not zero")
            if t:
                err = normwise_rel_err(g_out[:t], ref[:t].float())
                worst = max(worst, err)
                if err > 4 * 2.0**-8:
                    failures.append(f"replay {step}: error vs twin {err:.3e}")
        else:
            # the twin's collectives must still run on every rank in the same order: skip both sides alike
            pass
    torch.cuda.synchronize()
    st = fused.check_status()
    if st["code"] != 0:
        failures.append(f"after replays: status {st}")

    # G5: teardown order
    del graph
    torch.cuda.synchronize()
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "failures": failures[:5], "worst": worst})
    dist.barrier()
    dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()
    if rank == 0:
        bad = [g for g in gathered if g["failures"]]
        print(json.dumps({"ok": not bad, "world": world, "worst_err": max(g["worst"] for g in gathered), "bad": bad}))
        return 1 if bad else 0
    return 0


if __name__ == "__main__":
    sys.exit(main())
