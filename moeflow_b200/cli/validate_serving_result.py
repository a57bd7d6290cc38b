"""Refuse incomplete serving measurements before they are accepted as performance results.

    python -m moeflow_b200.cli.validate_serving_result result.json --requests 16 --input-len 1024 \
        --output-len 1024 --concurrency 4

The input is the detailed JSON a serving benchmark writes (per-request input/output lengths, errors,
TTFTs, latencies, inter-token latencies, and the mean/median/std/p50/p90/p95/p99 of TTFT, TPOT, ITL and
E2EL).  Every request must have completed with exactly the requested token counts, every statistic
must be a finite non-negative number, and the throughputs must equal completed work / duration.
Counterpart of ``scripts/validate_serving_result.py:19-64``.
"""

from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

STATS = ("mean", "median", "std", "p50", "p90", "p95", "p99")
QUANTITIES = ("ttft", "tpot", "itl", "e2el")
METRICS = [f"{stat}_{q}_ms" for q in QUANTITIES for stat in STATS]


def _number(v) -> bool:
    return type(v) in (int, float) and math.isfinite(v) and v >= 0


def validate_result(record: dict, requests: int, input_len: int, output_len: int, concurrency: int) -> dict:
    if requests < 1 or input_len < 1 or concurrency < 1 or output_len < 2:
        raise ValueError("Requests, input length and concurrency must be positive; output length must exceed one")
    exact = {"num_prompts": requests, "completed": requests, "failed": 0, "max_concurrency": concurrency,
             "total_input_tokens": requests * input_len, "total_output_tokens": requests * output_len}
    for key, want in exact.items():
        got = record.get(key)
        if type(got) is not int or got != want:
            raise ValueError(f"{key}: expected {want}, got {got!r}")
    if record.get("input_lens") != [input_len] * requests:
        raise ValueError(f"input_lens: every request must contain exactly {input_len} tokens")
    if record.get("output_lens") != [output_len] * requests:
        raise ValueError(f"output_lens: every request must contain exactly {output_len} tokens")
    if record.get("errors") != [""] * requests:
        raise ValueError("Missing or failed per-request error records; save the detailed result")
    for key in ("ttfts", "latencies"):
        vals = record.get(key)
        if not isinstance(vals, list) or len(vals) != requests or not all(_number(v) for v in vals):
            raise ValueError(f"Missing or invalid per-request {key}")
    itls = record.get("itls")
    ok = isinstance(itls, list) and len(itls) == requests and all(
        isinstance(row, list) and row and all(_number(v) for v in row) for row in itls)
    if not ok:
        raise ValueError("Missing or invalid inter-token latencies")
    for key in (*METRICS, "duration", "request_throughput", "output_throughput"):
        if not _number(record.get(key)):
            raise ValueError(f"Missing or nonfinite metric: {key}")
    if record["duration"] <= 0 or record["output_throughput"] <= 0:
        raise ValueError("Duration and output throughput must be positive")
    for key, work in (("request_throughput", requests), ("output_throughput", requests * output_len)):
        if not math.isclose(record[key], work / record["duration"], rel_tol=1e-6):
            raise ValueError(f"{key} does not match completed work / duration")
    return {"passed": True, "requests": requests, "total_output_tokens": requests * output_len,
            "metrics": {k: record[k] for k in METRICS},
            "tokens_per_second": record["output_throughput"], "median_tpot_ms": record["median_tpot_ms"]}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("path", type=Path)
    for name in ("requests", "input-len", "output-len", "concurrency"):
        ap.add_argument(f"--{name}", required=True, type=int)
    args = ap.parse_args()
    try:
        out = validate_result(json.loads(args.path.read_text()), args.requests, args.input_len, args.output_len, args.concurrency)
    except (OSError, ValueError) as err:
        print(json.dumps({"passed": False, "error": str(err)}))
        raise SystemExit(1) from err
    print(json.dumps(out, indent=2))


if __name__ == "__main__":
    main()
