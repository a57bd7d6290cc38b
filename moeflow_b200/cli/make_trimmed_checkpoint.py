"""A shallower copy of a checkpoint: the first N decoder layers at full width.

    python -m moeflow_b200.cli.make_trimmed_checkpoint --src <snapshot> --dst <dir> --num-layers 4

Serving experiments that only need "a model of the right layer shape" load in seconds from such a copy.
What is kept: decoder layers ``0 .. N-1`` and every tensor that does not belong to a decoder layer
(embeddings, final norm, output head, vision tower).  What goes: the deeper layers and the multi-token-
prediction layer.  The configuration is cut to match (layer count, per-layer type lists, the layer-index
lists of the linear-attention block), the kept tensors are re-packed shard by shard and re-indexed, and the
tokenizer / processor files are linked rather than copied.  A ``TRIMMED_FROM.json`` records the origin.

The work is planned first (``plan_shards``: which tensors of which source shard survive) and then carried
out, so the plan can be inspected or tested without touching tensor data.
Same result as ``scripts/make_trimmed_checkpoint.py:21-77`` of the reference.
"""

from __future__ import annotations

import argparse
import json
import os
import re
from pathlib import Path

INDEX_FILE = "model.safetensors.index.json"
CONFIG_FILE = "config.json"
_DECODER_LAYER = re.compile(r"model\.language_model\.layers\.(?P<layer>\d+)\.")
_LISTS_WITH_ONE_ENTRY_PER_LAYER = ("layer_types", "indexer_types", "mlp_layer_types")
_LISTS_OF_LAYER_INDICES = ("kda_layers", "full_attn_layers")  # inside linear_attn_config


def layer_of(tensor_name: str) -> int | None:
    """Decoder layer a tensor belongs to, or ``None`` for tensors outside the decoder stack."""
    found = _DECODER_LAYER.match(tensor_name)
    return int(found["layer"]) if found else None


def keeps(tensor_name: str, num_layers: int) -> bool:
    layer = layer_of(tensor_name)
    return layer is None or layer < num_layers


def trim_config(cfg: dict, num_layers: int) -> dict:
    """Cut the (text) configuration to ``num_layers`` layers, in place; returns ``cfg``."""
    text = cfg["text_config"] if "text_config" in cfg else cfg
    depth = text["num_hidden_layers"]
    if not 0 < num_layers <= depth:
        raise ValueError(f"cannot keep {num_layers} layers of a checkpoint with {depth}")
    text.update(num_hidden_layers=num_layers, num_nextn_predict_layers=0)
    for key in _LISTS_WITH_ONE_ENTRY_PER_LAYER:
        if isinstance(text.get(key), list):
            del text[key][num_layers:]
    linear_attention = text.get("linear_attn_config")
    if isinstance(linear_attention, dict):
        for key in _LISTS_OF_LAYER_INDICES:
            if key in linear_attention:
                linear_attention[key] = [layer for layer in linear_attention[key] if layer < num_layers]
    return cfg


def plan_shards(weight_map: dict[str, str], num_layers: int) -> list[tuple[str, str, list[str]]]:
    """``[(source shard, new shard name, surviving tensor names)]``; source shards with nothing left are
    dropped and the new shards are numbered from 1 in source-name order."""
    survivors: dict[str, list[str]] = {}
    for tensor_name, shard in weight_map.items():
        if keeps(tensor_name, num_layers):
            survivors.setdefault(shard, []).append(tensor_name)
    return [(shard, f"model-{number:05d}.safetensors", survivors[shard])
            for number, shard in enumerate(sorted(survivors), start=1)]


def _repack(src: Path, dst: Path, plan, say) -> dict[str, str]:
    from safetensors import safe_open
    from safetensors.torch import save_file

    where: dict[str, str] = {}
    for old_shard, new_shard, names in plan:
        with safe_open(src / old_shard, framework="pt") as reader:
            kept = {name: reader.get_tensor(name) for name in names}
        save_file(kept, dst / new_shard, metadata={"format": "pt"})
        where.update((name, new_shard) for name in names)
        say(f"{old_shard} -> {new_shard}: {len(names)} tensors")
    return where


def _link_everything_else(src: Path, dst: Path) -> None:
    for entry in src.iterdir():
        is_model_data = entry.suffix == ".safetensors" or entry.name in (CONFIG_FILE, INDEX_FILE)
        if not is_model_data and not (dst / entry.name).exists():
            os.symlink(entry.resolve(), dst / entry.name)


def trim(src: Path, dst: Path, num_layers: int, verbose: bool = True) -> None:
    src, dst = Path(src), Path(dst)
    say = (lambda line: print(line, flush=True)) if verbose else (lambda line: None)
    config = trim_config(json.loads((src / CONFIG_FILE).read_text()), num_layers)  # validates before anything is written
    plan = plan_shards(json.loads((src / INDEX_FILE).read_text())["weight_map"], num_layers)
    dst.mkdir(parents=True, exist_ok=True)
    (dst / CONFIG_FILE).write_text(json.dumps(config, indent=2))
    new_map = _repack(src, dst, plan, say)
    (dst / INDEX_FILE).write_text(json.dumps({"metadata": {}, "weight_map": new_map}, indent=1))
    _link_everything_else(src, dst)
    (dst / "TRIMMED_FROM.json").write_text(json.dumps({"src": str(src), "num_layers": num_layers}, indent=1))


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--src", required=True, type=Path, help="checkpoint directory (config, index, shards)")
    ap.add_argument("--dst", required=True, type=Path, help="directory to create")
    ap.add_argument("--num-layers", type=int, default=4)
    args = ap.parse_args(argv)
    trim(args.src, args.dst, args.num_layers)


if __name__ == "__main__":
    main()
