"""Greedy completions against a local OpenAI-compatible server, and strict comparison of two runs.

    python -m moeflow_b200.cli.smoke_client run --port 8000 --out greedy.json [--dp-rank 0 | --dp-ranks 0,1]
    python -m moeflow_b200.cli.smoke_client compare reference.json candidate.json [--exact-logprobs]

Requests are pinned to a data-parallel rank with the ``X-data-parallel-rank`` header so that both runs
exercise the same engine.  ``compare`` demands identical token sequences (and, optionally, bitwise
identical log-probabilities).  Counterpart of ``scripts/smoke_client.py:42-133``.
"""

from __future__ import annotations

import argparse
import json
import math
import sys
import urllib.request

PROMPTS = [
    "The capital of France is",
    "def fibonacci(n):",
    "Mixture-of-experts models route each token to",
    "1, 2, 3, 4, 5,",
]


def validate_prompts(prompts) -> list:
    """Text or token-id prompts; never an empty or ambiguous batch."""
    if not isinstance(prompts, list) or not prompts:
        raise ValueError("Prompts must be a nonempty JSON list")
    for p in prompts:
        text_ok = isinstance(p, str) and p != ""
        ids_ok = isinstance(p, list) and p and all(type(t) is int and t >= 0 for t in p)
        if not (text_ok or ids_ok):
            raise ValueError("Each prompt must be nonempty text or a nonempty list of nonnegative integer token IDs")
    return prompts


def has_complete_logprobs(record: dict) -> bool:
    toks, lps = record["tokens"], record["logprobs"]
    return bool(toks) and len(lps) == len(toks) and all(type(v) in (int, float) and math.isfinite(v) for v in lps)


def _post(port: int, payload: dict, dp_rank: int | None, timeout: float) -> dict:
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", data=json.dumps(payload).encode(),
                                 headers={"Content-Type": "application/json"})
    if dp_rank is not None:
        req.add_header("X-data-parallel-rank", str(dp_rank))
    with urllib.request.urlopen(req, timeout=timeout) as resp:
        return json.loads(resp.read())


def run(port: int, out: str, model: str = "smoke", max_tokens: int = 16, dp_ranks: list[int | None] | None = None,
        requests: int | None = None, prompts: list | None = None, timeout: float = 600.0) -> list[dict]:
    prompts = validate_prompts(PROMPTS if prompts is None else prompts)
    ranks = dp_ranks if dp_ranks else [None]
    if any(r is not None and (type(r) is not int or r < 0) for r in ranks):
        raise ValueError("DP ranks must be nonnegative integers")
    n = len(prompts) if requests is None else requests
    records = []
    for rank in ranks:
        for i in range(n):
            prompt = prompts[i % len(prompts)]
            body = _post(port, {"model": model, "prompt": prompt, "max_tokens": max_tokens, "temperature": 0.0, "logprobs": 1},
                         rank, timeout)
            choice = body["choices"][0]
            lp = choice.get("logprobs") or {}
            rec = {"dp_rank": rank, "prompt": prompt, "text": choice.get("text", ""), "tokens": lp.get("tokens") or [],
                   "logprobs": lp.get("token_logprobs") or [], "finish_reason": choice.get("finish_reason")}
            rec["complete"] = has_complete_logprobs(rec)
            records.append(rec)
    with open(out, "w") as sink:
        json.dump({"port": port, "model": model, "max_tokens": max_tokens, "records": records}, sink, indent=1)
    return records


def compare(a: dict, b: dict, exact_logprobs: bool = False) -> dict:
    ra, rb = a["records"], b["records"]
    if len(ra) != len(rb) or not ra:
        return {"passed": False, "error": "record counts differ or are empty"}
    mismatches = []
    for i, (x, y) in enumerate(zip(ra, rb)):
        if x["prompt"] != y["prompt"] or x.get("dp_rank") != y.get("dp_rank"):
            return {"passed": False, "error": f"record {i}: prompts or DP ranks differ"}
        if not (x.get("complete") and y.get("complete")):
            return {"passed": False, "error": f"record {i}: incomplete output or log-probabilities"}
        if x["tokens"] != y["tokens"] or x["text"] != y["text"]:
            mismatches.append(i)
        elif exact_logprobs and x["logprobs"] != y["logprobs"]:
            mismatches.append(i)
    return {"passed": not mismatches, "records": len(ra), "mismatching_records": mismatches,
            "exact_logprobs": exact_logprobs}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run")
    r.add_argument("--port", type=int, required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--model", default="smoke")
    r.add_argument("--max-tokens", type=int, default=16)
    r.add_argument("--dp-rank", type=int)
    r.add_argument("--dp-ranks")
    r.add_argument("--requests", type=int)
    r.add_argument("--prompts-json")
    c = sub.add_parser("compare")
    c.add_argument("reference")
    c.add_argument("candidate")
    c.add_argument("--exact-logprobs", action="store_true")
    args = ap.parse_args()
    if args.cmd == "run":
        if args.dp_rank is not None and args.dp_ranks:
            raise SystemExit("Specify one DP rank or a list of DP ranks, not both")
        ranks = [args.dp_rank] if args.dp_rank is not None else ([int(v) for v in args.dp_ranks.split(",")] if args.dp_ranks else None)
        prompts = json.load(open(args.prompts_json)) if args.prompts_json else None
        recs = run(args.port, args.out, args.model, args.max_tokens, ranks, args.requests, prompts)
        print(json.dumps({"records": len(recs), "complete": all(r["complete"] for r in recs)}))
        return
    result = compare(json.load(open(args.reference)), json.load(open(args.candidate)), args.exact_logprobs)
    print(json.dumps(result))
    sys.exit(0 if result["passed"] else 1)


if __name__ == "__main__":
    main()
