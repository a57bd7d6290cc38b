"""Cut a checkpoint down to its first N decoder layers (width unchanged).

    python -m moeflow_b200.cli.make_trimmed_checkpoint --src <snapshot> --dst <dir> --num-layers 4

Keeps decoder layers ``[0, N)`` and everything that is not a decoder layer (embeddings, final norm,
lm_head, vision tower); drops the other layers and the multi-token-prediction layer; trims the
per-layer lists of the config; links tokenizer/processor files instead of copying them.
Counterpart of ``scripts/make_trimmed_checkpoint.py:21-77``.
"""

from __future__ import annotations

import argparse
import json
import os
import re
from pathlib import Path

LAYER_NAME = re.compile(r"^model\.language_model\.layers\.(\d+)\.")
PER_LAYER_LISTS = ("layer_types", "indexer_types", "mlp_layer_types")
LAYER_INDEX_LISTS = ("kda_layers", "full_attn_layers")


def keeps(name: str, num_layers: int) -> bool:
    m = LAYER_NAME.match(name)
    return m is None or int(m.group(1)) < num_layers


def trim_config(cfg: dict, num_layers: int) -> dict:
    text = cfg.get("text_config", cfg)
    if num_layers > text["num_hidden_layers"]:
        raise ValueError(f"checkpoint has only {text['num_hidden_layers']} layers")
    text["num_hidden_layers"] = num_layers
    text["num_nextn_predict_layers"] = 0
    for key in PER_LAYER_LISTS:
        if isinstance(text.get(key), list):
            text[key] = text[key][:num_layers]
    linear = text.get("linear_attn_config") or {}
    for key in LAYER_INDEX_LISTS:
        if key in linear:
            linear[key] = [i for i in linear[key] if i < num_layers]
    return cfg


def trim(src: Path, dst: Path, num_layers: int, verbose: bool = True) -> None:
    from safetensors import safe_open
    from safetensors.torch import save_file

    dst.mkdir(parents=True, exist_ok=True)
    cfg = trim_config(json.loads((src / "config.json").read_text()), num_layers)
    (dst / "config.json").write_text(json.dumps(cfg, indent=2))

    weight_map = json.loads((src / "model.safetensors.index.json").read_text())["weight_map"]
    per_shard: dict[str, list[str]] = {}
    for name, shard in weight_map.items():
        if keeps(name, num_layers):
            per_shard.setdefault(shard, []).append(name)
    new_map: dict[str, str] = {}
    for i, shard in enumerate(sorted(per_shard), start=1):
        with safe_open(src / shard, framework="pt") as handle:
            tensors = {name: handle.get_tensor(name) for name in per_shard[shard]}
        out_name = f"model-{i:05d}.safetensors"
        save_file(tensors, dst / out_name, metadata={"format": "pt"})
        new_map.update(dict.fromkeys(tensors, out_name))
        if verbose:
            print(f"{shard} -> {out_name}: {len(tensors)} tensors", flush=True)
    (dst / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": new_map}, indent=1))

    skip = {"config.json", "model.safetensors.index.json"}
    for p in src.iterdir():
        if p.suffix == ".safetensors" or p.name in skip:
            continue
        link = dst / p.name
        if not link.exists():
            os.symlink(p.resolve(), link)
    (dst / "TRIMMED_FROM.json").write_text(json.dumps({"src": str(src), "num_layers": num_layers}, indent=1))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--num-layers", type=int, default=4)
    args = ap.parse_args()
    trim(Path(args.src), Path(args.dst), args.num_layers)


if __name__ == "__main__":
    main()
