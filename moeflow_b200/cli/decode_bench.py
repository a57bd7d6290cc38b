"""Decode throughput of the GLM-5.3-Flash-shaped model: time per output token and tokens per second.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m moeflow_b200.cli.decode_bench \
        --layers 42 --concurrency 64 --input-len 1024 --output-len 1024 --out results/decode_c64.json

DP = EP = N: the ``concurrency`` sequences are spread over the ranks (each rank decodes
``concurrency / N`` sequences per step), every layer's experts are sharded over the ranks, attention runs
per rank (TP=1).  Weights are random-initialised at the named shape, token inputs are synthetic; a
stand-in prefill fills the KV cache for ``input-len`` positions, then ``output-len`` decode steps are
replayed from one CUDA graph per step and timed on the device (barrier-aligned, max over ranks).

TPOT = time of one decode step; tokens/s = concurrency / TPOT.
"""

from __future__ import annotations

import argparse
import dataclasses

import torch
import torch.distributed as dist

from ..bench.backends import init_dist
from ..bench.record import make_record, write_record
from ..bench.stats import summarize
from ..bench.timing import aligned_start, max_over_ranks
from ..config import GLM53_FLASH_I1536
from ..models.glm_moe import AttentionConfig, DecodeModel


def routed_weights_factory(cfg, rank: int, world: int, device, fp8: bool):
    """Per-layer routed-expert weights, generated once and kept, so that several models (one per concurrency)
    share them.  Returns ``factory(layer) -> (w13, w2)`` for bf16 or ``(None, None, pack_args)`` for fp8."""
    import math

    from ..weights import quant_block_fp8

    cache: dict = {}
    H, I, L = cfg.hidden_size, cfg.moe_intermediate_size, cfg.experts_per_rank(world)

    def factory(layer: int):
        if layer not in cache:
            g = torch.Generator(device=device).manual_seed(7919 * layer + rank)
            w13 = torch.empty(L, 2 * I, H, dtype=torch.bfloat16, device=device)
            w2 = torch.empty(L, H, I, dtype=torch.bfloat16, device=device)
            for e in range(L):
                w13[e] = (torch.randn(2 * I, H, generator=g, device=device) * (2.0 / math.sqrt(H))).to(torch.bfloat16)
                w2[e] = (torch.randn(H, I, generator=g, device=device) / math.sqrt(I)).to(torch.bfloat16)
            if fp8:
                def quantise(w):
                    qs, ss = zip(*(quant_block_fp8(w[e]) for e in range(w.shape[0])))
                    return torch.stack([q.view(torch.uint8) for q in qs]).view(torch.float8_e4m3fn), torch.stack(ss)

                cache[layer] = (*quantise(w13), *quantise(w2))
            else:
                cache[layer] = (w13, w2)
        return cache[layer]

    return factory


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=42)
    ap.add_argument("--concurrency", default="4", help="total sequences in flight; a comma-separated list runs one "
                    "measurement per value on the same weights")
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=1024)
    ap.add_argument("--intermediate", type=int, default=1536)
    ap.add_argument("--chunk", type=int, default=64, help="decode steps per timing sample")
    ap.add_argument("--no-attention", action="store_true")
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 routed experts (128x128 weight blocks, 1x128 activation groups)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    info = init_dist()
    cfg = dataclasses.replace(GLM53_FLASH_I1536, moe_intermediate_size=args.intermediate)
    factory = routed_weights_factory(cfg, info.rank, info.world, info.device, args.fp8)
    results = []
    for concurrency in [int(c) for c in str(args.concurrency).split(",")]:
        results.append(measure(args, info, cfg, factory, concurrency))
    if info.rank == 0 and args.out:
        write_record(args.out, make_record("decode_bench", {**vars(args), "world": info.world, "cfg": cfg.to_dict()},
                                           {"points": results}))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def measure(args, info, cfg, factory, concurrency: int) -> dict:
    batch = max(1, (concurrency + info.world - 1) // info.world)
    acfg = AttentionConfig(max_seq=args.input_len + args.output_len + 8)
    model = DecodeModel(cfg, info.rank, info.world, batch, args.layers, info.device, acfg, attention=not args.no_attention,
                        fp8=args.fp8, weights_factory=factory)
    model.prefill_standin(args.input_len)
    model.x.copy_(torch.randn(batch, cfg.hidden_size, device=info.device).bfloat16())
    model.capture()
    for _ in range(3):
        model.step()
    samples = []
    done = 0
    while done < args.output_len:
        n = min(args.chunk, args.output_len - done)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        aligned_start()
        start.record()
        for _ in range(n):
            model.step()
        end.record()
        end.synchronize()
        samples.append(max_over_ranks(start.elapsed_time(end) / n))
        done += n
    status = model.routed.check_status()
    tpot = summarize(samples)
    result = {"concurrency": concurrency, "tpot_ms": tpot.to_dict(), "tokens_per_second": concurrency / (tpot.median / 1e3),
              "batch_per_rank": batch, "status": status, "finite": bool(torch.isfinite(model.out.float()).all())}
    if info.rank == 0:
        print(f"layers={args.layers} EP={info.world} concurrency={concurrency} {'fp8' if args.fp8 else 'bf16'}: TPOT median "
              f"{tpot.median:.3f} ms (p95 {tpot.p95:.3f}), {result['tokens_per_second']:.1f} tokens/s, status {status['name']}",
              flush=True)
    model.close()
    del model
    torch.cuda.synchronize()
    return result


if __name__ == "__main__":
    main()
