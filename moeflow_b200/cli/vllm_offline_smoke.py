"""Offline serving smoke: a tiny random-weight GLM-4-MoE model through the installed vLLM, in process.

    python -m moeflow_b200.cli.vllm_offline_smoke --arm moeflow --out smoke_moeflow.json
    python -m moeflow_b200.cli.vllm_offline_smoke --arm native  --out smoke_native.json
    python -m moeflow_b200.cli.vllm_offline_smoke --compare smoke_native.json smoke_moeflow.json

No checkpoint and no tokenizer are needed: the model directory holds only a ``config.json``, the weights are
the engine's seeded dummy initialisation and the prompts are token ids.  The engine core runs inside this
process (``VLLM_ENABLE_V1_MULTIPROCESSING=0``) so that the plugin can be registered by a plain call; a
deployment installs the package and lets vLLM load the entry point instead.

The ``moeflow`` arm builds every MoE layer with ``MoEFlowRunner`` in ``fixed`` mode and records the runner's
call log; the run fails unless at least one decode step was intercepted and, with ``MOEFLOW_EXPERTS=native``
(the default here), computed by this framework's grouped GEMMs.  ``--compare`` checks that both arms
produced the same greedy tokens wherever the native arm's top-1 margin exceeds the tolerance, and that the
logprobs of the chosen tokens agree.  Counterpart of the reference's serving smoke
(``scripts/smoke_client.py``, ``scripts/validate_serving_result.py``) for a box without a model checkpoint.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
from pathlib import Path

TINY_GLM4_MOE = {
    "architectures": ["Glm4MoeForCausalLM"],
    "model_type": "glm4_moe",
    "hidden_size": 512,
    "intermediate_size": 1024,
    "moe_intermediate_size": 256,
    "n_routed_experts": 32,
    "n_shared_experts": 1,
    "num_experts_per_tok": 4,
    "n_group": 1,
    "topk_group": 1,
    "first_k_dense_replace": 1,
    "norm_topk_prob": True,
    "routed_scaling_factor": 1.0,
    "num_hidden_layers": 3,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "vocab_size": 4096,
    "max_position_embeddings": 1024,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "partial_rotary_factor": 0.5,
    "use_qk_norm": False,
    "attention_bias": False,
    "hidden_act": "silu",
    "tie_word_embeddings": False,
    "torch_dtype": "bfloat16",
    "pad_token_id": 0,
    "eos_token_id": 1,
}


def write_model_dir(path: Path, overrides: dict | None = None) -> Path:
    path.mkdir(parents=True, exist_ok=True)
    cfg = dict(TINY_GLM4_MOE, **(overrides or {}))
    (path / "config.json").write_text(json.dumps(cfg, indent=1))
    return path


def prompts(n: int, length: int, vocab: int) -> list[list[int]]:
    """Deterministic token-id prompts (a multiplicative hash, ids 2..vocab-1)."""
    return [[2 + (7919 * (i + 1) * (j + 3) + 104729 * j) % (vocab - 2) for j in range(length)] for i in range(n)]


def seeded_init(model) -> int:
    """Replace the engine's dummy weights (about 1e-3, which makes every logit a near-tie) by seeded
    values of a realistic scale, the same in every process: matrices N(0, 1/fan_in), norm weights 1, the
    router's selection bias small.  The seed of a parameter is a hash of its name."""
    import zlib

    import torch

    n = 0
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            g = torch.Generator(device="cpu").manual_seed(zlib.crc32(name.encode()))
            if name.endswith("e_score_correction_bias"):
                v = torch.randn(p.shape, generator=g) * 0.05
            elif p.dim() == 1:
                v = torch.ones(p.shape)
            else:
                v = torch.randn(p.shape, generator=g) * (float(p.shape[-1]) ** -0.5)
            p.copy_(v.to(device=p.device, dtype=p.dtype))
            n += 1
    return n


def run_arm(args) -> dict:
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    # FlashInfer's sampler, attention and MoE kernels compile or fetch binaries on first use; the smoke run
    # keeps to kernels that ship with the engine (Triton), which is also the modular path the runner intercepts
    os.environ.setdefault("VLLM_USE_FLASHINFER_SAMPLER", "0")
    smoke_dir = Path(args.log_dir or tempfile.mkdtemp(prefix="moeflow_smoke_"))
    hook = None
    if args.arm == "moeflow":
        os.environ["MOEFLOW_RUNNER"] = "1"
        os.environ.setdefault("MOEFLOW_MODE", "fixed")
        os.environ.setdefault("MOEFLOW_MAX_TOKENS", str(args.max_fixed_tokens))
        os.environ.setdefault("MOEFLOW_EXPERTS", "native")
        os.environ["MOEFLOW_SMOKE_DIR"] = str(smoke_dir)
        from ..integrations import vllm_plugin

        hook = vllm_plugin.register_runner()
    from vllm import LLM, SamplingParams

    model_dir = write_model_dir(Path(args.model_dir or tempfile.mkdtemp(prefix="tiny_glm4_moe_")))
    llm = LLM(model=str(model_dir), load_format="dummy", skip_tokenizer_init=True, enforce_eager=not args.graphs,
              max_model_len=512, gpu_memory_utilization=args.gpu_memory_utilization, seed=0, dtype="bfloat16",
              enable_expert_parallel=True, max_num_seqs=args.requests, moe_backend=args.moe_backend,
              attention_backend=args.attention_backend)
    n_params = llm.apply_model(seeded_init)[0] if not args.dummy_weights else 0
    sp = SamplingParams(max_tokens=args.max_tokens, temperature=0.0, logprobs=args.logprobs, detokenize=False,
                        ignore_eos=True)
    reqs = [{"prompt_token_ids": p} for p in prompts(args.requests, args.prompt_len, TINY_GLM4_MOE["vocab_size"])]
    outs = llm.generate(reqs, sp)
    result = {"arm": args.arm, "hook": hook, "seeded_parameters": n_params, "requests": []}
    for o in outs:
        c = o.outputs[0]
        steps = []
        for tok, lp in zip(c.token_ids, c.logprobs or []):
            ranked = sorted(((int(t), float(v.logprob)) for t, v in lp.items()), key=lambda kv: -kv[1])
            steps.append({"token": int(tok), "top": ranked})
        result["requests"].append({"tokens": [int(t) for t in c.token_ids], "steps": steps})
    if args.arm == "moeflow":
        entries = []
        for f in sorted(smoke_dir.glob("runner_pid*.jsonl")):
            entries += [json.loads(line) for line in f.read_text().splitlines() if line.strip()]
        fixed = [e for e in entries if e.get("mode") == "fixed" and e.get("intercepted")]
        result["runner_log"] = {
            "entries": len(entries), "fixed_intercepted": len(fixed),
            "experts": sorted({e.get("experts") for e in fixed if e.get("experts")}),
            "declined": sorted({e.get("reason") for e in entries if e.get("intercepted") is False}),
        }
        if not fixed:
            raise SystemExit(f"moeflow arm: no MoE call was intercepted by the fixed path ({result['runner_log']})")
    return result


def compare(native: dict, ours: dict, margin: float, logprob_tol: float) -> dict:
    """Step by step while both arms have generated the same tokens (so both condition on the same history):
    the logprobs of every token that both arms list must agree within ``logprob_tol``, and where the native
    arm's top-1 margin exceeds ``margin`` both arms must pick the same token."""
    steps = decisive = decisive_agree = values = 0
    worst = 0.0
    for a, b in zip(native["requests"], ours["requests"]):
        for sa, sb in zip(a["steps"], b["steps"]):
            steps += 1
            theirs = dict(sb["top"])
            for tok, lp in sa["top"]:
                if tok in theirs:
                    values += 1
                    worst = max(worst, abs(lp - theirs[tok]))
            top = sa["top"]
            if len(top) < 2 or top[0][1] - top[1][1] > margin:
                decisive += 1
                decisive_agree += int(sa["token"] == sb["token"])
            if sa["token"] != sb["token"]:
                break  # later steps condition on different histories
    ok = values > 0 and decisive_agree == decisive and worst <= logprob_tol
    return {"passed": ok, "steps_compared": steps, "logprobs_compared": values, "max_abs_logprob_diff": worst,
            "decisive_steps": decisive, "decisive_steps_agreeing": decisive_agree, "margin": margin,
            "logprob_tol": logprob_tol}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--arm", choices=["native", "moeflow"], default="moeflow")
    ap.add_argument("--compare", nargs=2, metavar=("NATIVE_JSON", "MOEFLOW_JSON"))
    ap.add_argument("--out", default=None)
    ap.add_argument("--model-dir", default=None)
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--requests", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=24)
    ap.add_argument("--max-tokens", type=int, default=8)
    ap.add_argument("--logprobs", type=int, default=5)
    ap.add_argument("--max-fixed-tokens", type=int, default=64)
    ap.add_argument("--moe-backend", default="triton",
                    help="engine expert kernels; a monolithic backend (FlashInfer TRT-LLM) is never intercepted")
    ap.add_argument("--attention-backend", default="TRITON_ATTN")
    ap.add_argument("--dummy-weights", action="store_true", help="keep the engine's dummy initialisation")
    ap.add_argument("--graphs", action="store_true", help="let the engine capture CUDA graphs (default: eager)")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.2)
    ap.add_argument("--margin", type=float, default=0.1)
    ap.add_argument("--logprob-tol", type=float, default=0.05)
    args = ap.parse_args(argv)
    if args.compare:
        res = compare(json.loads(Path(args.compare[0]).read_text()), json.loads(Path(args.compare[1]).read_text()),
                      args.margin, args.logprob_tol)
    else:
        res = run_arm(args)
    text = json.dumps(res)
    if args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(text)
    summary = {k: v for k, v in res.items() if k != "requests"}
    print(json.dumps(summary))
    return 0 if res.get("passed", True) else 1


if __name__ == "__main__":
    sys.exit(main())
