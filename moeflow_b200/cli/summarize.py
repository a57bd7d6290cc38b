"""Turn benchmark records into Markdown tables; refuses records that are incomplete or unvalidated.

    python -m moeflow_b200.cli.summarize layer  results/layer_*.json
    python -m moeflow_b200.cli.summarize ab     results/ab_*.json        # ab_fixed and ab_native_fixed records
    python -m moeflow_b200.cli.summarize stages results/stages_*.json
    python -m moeflow_b200.cli.summarize logits native.json candidate.json
    python -m moeflow_b200.cli.summarize serving w1_native.json w1_moeflow.json --requests 16 --input-len 1024 --output-len 1024 --concurrency 4
    python -m moeflow_b200.cli.summarize decode  results/decode_*.json   # self-contained decoder (cli/decode_bench.py)
    python -m moeflow_b200.cli.summarize launches launches.csv      # kernels per forward from an ncu launch list

Counterpart of the reference's ``scripts/summarize_{ablations,backend_pair,logits,replay_trace,stage1,w1}.py``.
"""

from __future__ import annotations

import argparse
import csv
import hashlib
import json
from collections import Counter
from pathlib import Path


def load(path: str, kind: str | tuple[str, ...] | None = None) -> dict:
    rec = json.loads(Path(path).read_text())
    kinds = (kind,) if isinstance(kind, str) else kind
    if kinds is not None and rec.get("kind") not in kinds:
        raise SystemExit(f"{path}: expected a {' or '.join(kinds)} record, found {rec.get('kind')!r}")
    if rec.get("complete") is False:
        raise SystemExit(f"{path}: record is incomplete; refusing to summarise it")
    return rec


def layer_table(paths: list[str]) -> str:
    rows = ["| backend | EP | T | graph median us | graph p95 us | eager median us | oracle err |", "|---|---:|---:|---:|---:|---:|---:|"]
    for p in paths:
        rec = load(p, "bench_layer")
        for pt in rec["results"]["points"]:
            if not pt["passed"]:
                raise SystemExit(f"{p}: T={pt['tokens']} failed its reference check; no table")
            g = pt.get("graph_us")
            err = max(c["normwise_rel_err"] for c in pt["reference"])
            rows.append(f"| {rec['config']['backend']} | {rec['config']['world']} | {pt['tokens']} | "
                        f"{g['median']:.1f} | {g['p95']:.1f} | {pt['eager_us']['median']:.1f} | {err:.2e} |" if g else
                        f"| {rec['config']['backend']} | {rec['config']['world']} | {pt['tokens']} | not capturable | | {pt['eager_us']['median']:.1f} | {err:.2e} |")
    return "\n".join(rows)


def ab_table(paths: list[str]) -> str:
    rows = ["| A | B | EP | T | A median us | B median us | gain us | 95% CI of (B-A) | significant | beneficial |", "|---|---|---:|---:|---:|---:|---:|---|---|---|"]
    for p in paths:
        rec = load(p, ("ab_fixed", "ab_native_fixed"))  # same shape: fused variants, or native transport vs fused
        c = rec["config"]
        for pt in rec["results"]["points"]:
            if not (pt["gate"]["a"]["passed"] and pt["gate"]["b"]["passed"]):
                raise SystemExit(f"{p}: an arm failed its oracle gate; no table")
            pr = pt["paired"]
            rows.append(f"| {c['a']} | {c['b']} | {c['world']} | {pt['tokens']} | {pt['a_us']['median']:.1f} | {pt['b_us']['median']:.1f} | "
                        f"{pr['median_improvement']:+.1f} | [{pr['ci95'][0]:+.1f}, {pr['ci95'][1]:+.1f}] | {pr['significant']} | {pr['beneficial']} |")
    return "\n".join(rows)


def stages_table(paths: list[str]) -> str:
    rows = []
    for p in paths:
        rec = load(p, "bench_stages")
        pts = rec["results"]["points"]
        names = list(pts[0]["stage_us"])
        rows += [f"EP={rec['config']['world']} backend={rec['config']['backend']} flush={rec['config']['flush']}", "",
                 "| T | " + " | ".join(names) + " | full | one valid row |", "|---:|" + "---:|" * (len(names) + 2)]
        for pt in pts:
            if pt["status"]["code"] != 0:
                raise SystemExit(f"{p}: device status {pt['status']}; no table")
            rows.append(f"| {pt['tokens']} | " + " | ".join(f"{pt['stage_us'][n]:.1f}" for n in names) +
                        f" | {pt['prefix_us']['COMBINE']:.1f} | {pt['padding']['valid_1']:.1f} |")
        rows.append("")
    return "\n".join(rows)


def logits_summary(a: str, b: str) -> str:
    import numpy as np

    from ..bench.logits import compare_logits

    res = compare_logits(np.load(a)["logits"], np.load(b)["logits"])
    return json.dumps(res, indent=1)


def serving_table(paths: list[str], requests, input_len, output_len, concurrency) -> str:
    from .validate_serving_result import validate_result

    rows = ["| run | tokens/s | median TPOT ms | p99 TPOT ms | median TTFT ms |", "|---|---:|---:|---:|---:|"]
    for p in paths:
        rec = json.loads(Path(p).read_text())
        v = validate_result(rec, requests, input_len, output_len, concurrency)
        rows.append(f"| {Path(p).stem} | {v['tokens_per_second']:.1f} | {rec['median_tpot_ms']:.3f} | {rec['p99_tpot_ms']:.3f} | {rec['median_ttft_ms']:.2f} |")
    return "\n".join(rows)


def decode_table(paths: list[str]) -> str:
    """TPOT / throughput of the self-contained decoder (``cli/decode_bench.py`` records); a point whose layer status
    is not ok or whose output is not finite makes the whole table refuse."""
    rows = ["| layers | EP | experts | concurrency | sequences per rank | TPOT median ms | p95 ms | tokens/s |",
            "|---:|---:|---|---:|---:|---:|---:|---:|"]
    for p in paths:
        rec = load(p, "decode_bench")
        c = rec["config"]
        for pt in rec["results"]["points"]:
            if pt["status"]["code"] != 0 or not pt["finite"]:
                raise SystemExit(f"{p}: a point ended with status {pt['status']['name']!r} or a non-finite output; no table")
            rows.append(f"| {c['layers']} | {c['world']} | {'e4m3' if c.get('fp8') else 'bf16'} | {pt['concurrency']} | "
                        f"{pt['batch_per_rank']} | {pt['tpot_ms']['median']:.3f} | {pt['tpot_ms']['p95']:.3f} | "
                        f"{pt['tokens_per_second']:.0f} |")
    return "\n".join(rows)


def launches_summary(path: str, forwards: int | None = None) -> str:
    """Kernel launches per forward from a launch list written by
    ``ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file <path> <command>`` (one pass per
    launch; ``--clock-control none`` keeps the profiler from locking the clocks of a shared GPU)."""
    lines = [ln for ln in Path(path).read_text().splitlines() if not ln.startswith("==")]
    names = Counter()
    total = Counter()
    for row in csv.DictReader(lines):
        name = row["Kernel Name"].split("(")[0]
        names[name] += 1
        total[name] += float(row["Metric Value"].replace(",", ""))
    ours = {k: v for k, v in names.items() if "mf::" in k or k.startswith("mf")}
    n_fwd = forwards or (min(ours.values()) if ours else 1)
    out = [f"sha256 {hashlib.sha256(Path(path).read_bytes()).hexdigest()}", f"forwards assumed: {n_fwd}", "",
           "| kernel | launches | per forward | total us |", "|---|---:|---:|---:|"]
    for k, v in sorted(names.items(), key=lambda kv: -total[kv[0]]):
        out.append(f"| {k[:70]} | {v} | {v / n_fwd:.2f} | {total[k] / 1e3:.1f} |")
    helper = sum(v for k, v in names.items() if "at::native" in k)
    out += ["", f"library helper kernels (at::native): {helper} ({helper / n_fwd:.2f} per forward)"]
    return "\n".join(out)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("what", choices=["layer", "ab", "stages", "logits", "serving", "decode", "launches"])
    ap.add_argument("paths", nargs="+")
    ap.add_argument("--requests", type=int)
    ap.add_argument("--input-len", type=int)
    ap.add_argument("--output-len", type=int)
    ap.add_argument("--concurrency", type=int)
    ap.add_argument("--forwards", type=int)
    args = ap.parse_args()
    if args.what == "layer":
        print(layer_table(args.paths))
    elif args.what == "ab":
        print(ab_table(args.paths))
    elif args.what == "stages":
        print(stages_table(args.paths))
    elif args.what == "logits":
        print(logits_summary(*args.paths[:2]))
    elif args.what == "decode":
        print(decode_table(args.paths))
    elif args.what == "serving":
        print(serving_table(args.paths, args.requests, args.input_len, args.output_len, args.concurrency))
    else:
        print(launches_summary(args.paths[0], args.forwards))


if __name__ == "__main__":
    main()
