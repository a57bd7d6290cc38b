"""Stack probes: is the machine able to run the framework at all?

    python -m moeflow_b200.cli.probes native                      # device capability, native library, one kernel
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m moeflow_b200.cli.probes a2a
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m moeflow_b200.cli.probes peer

``a2a`` runs even, uneven and CUDA-graph-captured ``all_to_all_single`` on NCCL and logs an orderly
teardown (graphs dropped before the process group).  ``peer`` allocates a symmetric region, lets every
rank store into every peer and wait (bounded) for all flags, then exercises the time-out path by
skipping the stores once.  Counterpart of ``scripts/probes/nccl_a2a.py:16-87`` and ``triton_min.py:11-35``.
"""

from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist


def probe_native() -> dict:
    from ..ops import _lib
    from ..ops.kernels import rmsnorm, sm_count

    cap = torch.cuda.get_device_capability()
    x = torch.randn(4, 256, device="cuda").bfloat16()
    out = rmsnorm(x, torch.ones(256, device="cuda").bfloat16())
    torch.cuda.synchronize()
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    return {"capability": list(cap), "sm_100_or_newer": cap >= (10, 0), "sms": sm_count(0), "library": str(_lib.LIB_PATH),
            "rmsnorm_max_err": float((out.float() - ref).abs().max())}


def probe_a2a() -> dict:
    from ..bench.backends import init_dist

    info = init_dist()
    w, dev = info.world, info.device
    send = torch.arange(w * 4096, dtype=torch.float32, device=dev) + info.rank * 1e6
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send)
    even_ok = all(float(recv[s * 4096]) == s * 1e6 + info.rank * 4096 for s in range(w))
    splits_in = [info.rank + 1] * w
    splits_out = [s + 1 for s in range(w)]
    usend = torch.full((sum(splits_in),), float(info.rank), device=dev)
    urecv = torch.empty(sum(splits_out), device=dev)
    dist.all_to_all_single(urecv, usend, splits_out, splits_in)
    uneven_ok = urecv.tolist() == [float(s) for s in range(w) for _ in range(s + 1)]
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        dist.all_to_all_single(recv, send)
    torch.cuda.synchronize()
    dist.barrier()
    with torch.cuda.graph(graph):
        dist.all_to_all_single(recv, send)
    for _ in range(10):
        graph.replay()
    torch.cuda.synchronize()
    graph_ok = all(float(recv[s * 4096]) == s * 1e6 + info.rank * 4096 for s in range(w))
    del graph  # graphs first, then the group
    torch.cuda.synchronize()
    gathered = [None] * w
    dist.all_gather_object(gathered, {"rank": info.rank, "even": even_ok, "uneven": uneven_ok, "graph": graph_ok})
    dist.barrier()
    dist.destroy_process_group()
    return {"ranks": gathered, "ok": all(g["even"] and g["uneven"] and g["graph"] for g in gathered), "teardown": "clean"} if info.rank == 0 else {}


def probe_peer() -> dict:
    from ..bench.backends import init_dist
    from ..ops._lib import decode_status
    from ..parallel.peer import PeerGroup, ping

    info = init_dist()
    group = PeerGroup(info.rank, info.world, None, info.device)
    region = group.allocate(4096)
    status = torch.zeros(1, dtype=torch.int64, device=info.device)
    for value in (1, 2, 3):
        ping(region, 0, value, status, wait_ns=5_000_000_000)
        torch.cuda.synchronize()
        dist.barrier()
    ok = decode_status(int(status.item()))["code"] == 0
    status.zero_()
    dist.barrier()
    ping(region, 0, 99, status, wait_ns=200_000_000, skip_store=True)  # nobody stores: the wait must run out cleanly
    torch.cuda.synchronize()
    timed_out = decode_status(int(status.item()))
    gathered = [None] * info.world
    dist.all_gather_object(gathered, {"rank": info.rank, "ping_ok": ok, "timeout_code": timed_out["code"]})
    dist.barrier()
    region.close()
    dist.destroy_process_group()
    return {"ranks": gathered, "ok": all(g["ping_ok"] and g["timeout_code"] == 8 for g in gathered)} if info.rank == 0 else {}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("what", choices=["native", "a2a", "peer"])
    args = ap.parse_args()
    out = {"native": probe_native, "a2a": probe_a2a, "peer": probe_peer}[args.what]()
    if out:
        print(json.dumps(out))
        raise SystemExit(0 if out.get("ok", True) else 1)


if __name__ == "__main__":
    main()
