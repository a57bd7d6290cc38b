"""Full-vocabulary raw logits from a serving endpoint, stored as NPZ with a SHA-256, and compared bitwise.

    python -m moeflow_b200.cli.logits_client run --port 8000 --vocab 154880 --steps 8 --out native.npz [--dp-rank 0]
    python -m moeflow_b200.cli.logits_client compare native.npz candidate.npz

``run`` asks the server for the raw logits of every generated step (the endpoint must be started with its
raw-logits option), checks that each step carries exactly ``vocab`` finite numbers, and stores them.
Counterpart of ``scripts/logits_client.py:39-117``.
"""

from __future__ import annotations

import argparse
import json
import sys
import urllib.request

import numpy as np

from ..bench.logits import compare_logits, digest, parse_raw_logits


def fetch(port: int, prompt, steps: int, dp_rank: int | None, model: str, timeout: float = 600.0):
    body = {"model": model, "prompt": prompt, "max_tokens": steps, "temperature": 0.0, "return_raw_logits": True}
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    if dp_rank is not None:
        req.add_header("X-data-parallel-rank", str(dp_rank))
    with urllib.request.urlopen(req, timeout=timeout) as resp:
        choice = json.loads(resp.read())["choices"][0]
    if "raw_logits" not in choice:
        raise ValueError("the server did not return raw logits")
    return choice["raw_logits"], choice.get("token_ids")


def run(port: int, out: str, vocab: int, steps: int, prompt="The capital of France is", dp_rank=None, model="smoke") -> dict:
    payload, token_ids = fetch(port, prompt, steps, dp_rank, model)
    logits = parse_raw_logits(payload, vocab)
    if logits.shape[0] != steps:
        raise ValueError(f"expected {steps} steps of logits, got {logits.shape[0]}")
    np.savez(out, logits=logits, token_ids=np.asarray(token_ids if token_ids is not None else [], dtype=np.int64))
    return {"steps": int(logits.shape[0]), "vocab": vocab, "sha256": digest(logits), "dp_rank": dp_rank}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run")
    r.add_argument("--port", type=int, required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--vocab", type=int, required=True)
    r.add_argument("--steps", type=int, default=8)
    r.add_argument("--dp-rank", type=int)
    r.add_argument("--model", default="smoke")
    c = sub.add_parser("compare")
    c.add_argument("a")
    c.add_argument("b")
    args = ap.parse_args()
    if args.cmd == "run":
        print(json.dumps(run(args.port, args.out, args.vocab, args.steps, dp_rank=args.dp_rank, model=args.model)))
        return
    result = compare_logits(np.load(args.a)["logits"], np.load(args.b)["logits"])
    print(json.dumps(result))
    sys.exit(0 if result.get("bitwise_equal") else 1)


if __name__ == "__main__":
    main()
