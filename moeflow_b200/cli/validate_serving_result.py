"""Gate for serving measurements: a result file is accepted as a performance number only if it is complete.

    python -m moeflow_b200.cli.validate_serving_result result.json --requests 16 --input-len 1024 \
        --output-len 1024 --concurrency 4

The input is the detailed JSON a serving benchmark writes.  The checks are a list of named rules applied in
order; the first rule that does not hold is reported (as ``{"passed": false, "error": ...}`` and exit status 1
on the command line, as ``ValueError`` from ``validate_result``):

1. the run was the requested one: request count, concurrency and the total token counts are exact integers;
2. every request ran to the end: per-request input and output lengths equal the requested ones, no error text;
3. per-request timings exist for every request and are finite and non-negative (TTFT, end-to-end latency, and
   a non-empty list of inter-token latencies each);
4. every summary statistic (mean / median / std / p50 / p90 / p95 / p99 of TTFT, TPOT, ITL, E2EL) and the
   duration and throughputs are finite, non-negative numbers, duration and output throughput positive;
5. the throughputs are what the completed work and the duration imply.

Same acceptance conditions as ``scripts/validate_serving_result.py:19-64`` of the reference.
"""

from __future__ import annotations

import argparse
import json
import math
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

QUANTITIES = ("ttft", "tpot", "itl", "e2el")
STATS = ("mean", "median", "std", "p50", "p90", "p95", "p99")
METRICS = [f"{stat}_{quantity}_ms" for quantity in QUANTITIES for stat in STATS]
SCALARS = (*METRICS, "duration", "request_throughput", "output_throughput")


def _is_measurement(value) -> bool:
    """A real, finite, non-negative int or float (bools and strings are not measurements)."""
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value) and value >= 0


def _all_measurements(values, count: int) -> bool:
    return isinstance(values, list) and len(values) == count and all(_is_measurement(v) for v in values)


@dataclass(frozen=True)
class Workload:
    requests: int
    input_len: int
    output_len: int
    concurrency: int

    def __post_init__(self):
        if self.requests < 1 or self.input_len < 1 or self.concurrency < 1 or self.output_len < 2:
            raise ValueError("Requests, input length and concurrency must be positive; output length must exceed one")

    @property
    def output_tokens(self) -> int:
        return self.requests * self.output_len


@dataclass(frozen=True)
class Rule:
    holds: Callable[[dict, Workload], bool]
    complaint: Callable[[dict, Workload], str]


def _exact_int(key: str, want: Callable[[Workload], int]) -> Rule:
    return Rule(
        lambda rec, w: type(rec.get(key)) is int and rec[key] == want(w),
        lambda rec, w: f"{key}: expected {want(w)}, got {rec.get(key)!r}",
    )


def _uniform_lengths(key: str, want: Callable[[Workload], int]) -> Rule:
    return Rule(
        lambda rec, w: rec.get(key) == [want(w)] * w.requests,
        lambda rec, w: f"{key}: every request must contain exactly {want(w)} tokens",
    )


def _scalar(key: str) -> Rule:
    return Rule(lambda rec, w: _is_measurement(rec.get(key)), lambda rec, w: f"Missing or nonfinite metric: {key}")


def _throughput(key: str, work: Callable[[Workload], int]) -> Rule:
    return Rule(
        lambda rec, w: math.isclose(rec[key], work(w) / rec["duration"], rel_tol=1e-6),
        lambda rec, w: f"{key} does not match completed work / duration",
    )


RULES: tuple[Rule, ...] = (
    _exact_int("num_prompts", lambda w: w.requests),
    _exact_int("completed", lambda w: w.requests),
    _exact_int("failed", lambda w: 0),
    _exact_int("max_concurrency", lambda w: w.concurrency),
    _exact_int("total_input_tokens", lambda w: w.requests * w.input_len),
    _exact_int("total_output_tokens", lambda w: w.output_tokens),
    _uniform_lengths("input_lens", lambda w: w.input_len),
    _uniform_lengths("output_lens", lambda w: w.output_len),
    Rule(lambda rec, w: rec.get("errors") == [""] * w.requests,
         lambda rec, w: "Missing or failed per-request error records; save the detailed result"),
    Rule(lambda rec, w: _all_measurements(rec.get("ttfts"), w.requests), lambda rec, w: "Missing or invalid per-request ttfts"),
    Rule(lambda rec, w: _all_measurements(rec.get("latencies"), w.requests),
         lambda rec, w: "Missing or invalid per-request latencies"),
    Rule(lambda rec, w: isinstance(rec.get("itls"), list) and len(rec["itls"]) == w.requests
         and all(isinstance(row, list) and len(row) > 0 and _all_measurements(row, len(row)) for row in rec["itls"]),
         lambda rec, w: "Missing or invalid inter-token latencies"),
    *(_scalar(key) for key in SCALARS),
    Rule(lambda rec, w: rec["duration"] > 0 and rec["output_throughput"] > 0,
         lambda rec, w: "Duration and output throughput must be positive"),
    _throughput("request_throughput", lambda w: w.requests),
    _throughput("output_throughput", lambda w: w.output_tokens),
)


def validate_result(record: dict, requests: int, input_len: int, output_len: int, concurrency: int) -> dict:
    """Raises ``ValueError`` naming the first rule that does not hold; returns the accepted summary otherwise."""
    workload = Workload(requests, input_len, output_len, concurrency)
    for rule in RULES:
        if not rule.holds(record, workload):
            raise ValueError(rule.complaint(record, workload))
    return {
        "passed": True,
        "requests": requests,
        "total_output_tokens": workload.output_tokens,
        "tokens_per_second": record["output_throughput"],
        "median_tpot_ms": record["median_tpot_ms"],
        "metrics": {key: record[key] for key in METRICS},
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("path", type=Path)
    for flag in ("--requests", "--input-len", "--output-len", "--concurrency"):
        ap.add_argument(flag, required=True, type=int)
    args = ap.parse_args(argv)
    try:
        accepted = validate_result(json.loads(args.path.read_text()), args.requests, args.input_len, args.output_len,
                                   args.concurrency)
    except (OSError, ValueError) as problem:
        print(json.dumps({"passed": False, "error": str(problem)}))
        return 1
    print(json.dumps(accepted, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
