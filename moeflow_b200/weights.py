"""Expert weights from a GLM-5.3-Flash style checkpoint (safetensors shards + index).

Tensor names: ``model.language_model.layers.{L}.mlp.experts.{e}.{gate_proj,up_proj,down_proj}.weight``
(+ ``.weight_scale_inv`` for block-scaled float8_e4m3fn weights), ``...mlp.gate.weight [E, H]`` and
``...mlp.gate.e_score_correction_bias [E]``.  FP8 weights are scaled per 128x128 block
(``quantization_config.weight_block_size``): ``w[i, j] * scale_inv[i // 128, j // 128]``; partial edge
blocks use the scale of the block they fall into.

Two ways to read a layer's experts:

* ``expert_weights`` dequantises to bf16: ``w13 [n, 2I, H] = [gate; up]``, ``w2 [n, H, I]`` (what the
  bf16 tcgen05 path consumes);
* ``expert_weights_fp8`` keeps e4m3 bytes and fp32 block scales side by side for the block-scaled
  GEMM: ``(w13_q [n, 2I, H] e4m3, w13_s [n, 2I/128, H/128] fp32, w2_q, w2_s)``.

The checkpoint root comes from ``MOEFLOW_MODEL_PATH``.  Counterpart of ``moeflow/weights.py:19-77``.
"""

from __future__ import annotations

import json
import os
from pathlib import Path

import torch

DEFAULT_SNAPSHOT = Path(os.environ.get("MOEFLOW_MODEL_PATH", "checkpoints/GLM-5.3-Flash"))
PREFIX = "model.language_model.layers.{layer}.mlp"
PROJECTIONS = ("gate_proj", "up_proj", "down_proj")


def dequant_block_fp8(w: torch.Tensor, scale_inv: torch.Tensor, block: tuple[int, int] = (128, 128)) -> torch.Tensor:
    """Block-scaled FP8 -> fp32 (one fp32 product per element)."""
    rows, cols = w.shape
    row_block = torch.arange(rows, device=w.device) // block[0]
    col_block = torch.arange(cols, device=w.device) // block[1]
    scale = scale_inv.to(torch.float32)[row_block][:, col_block]
    return w.to(torch.float32) * scale


def quant_block_fp8(w: torch.Tensor, block: tuple[int, int] = (128, 128)) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32/bf16 ``[rows, cols]`` -> ``(e4m3 [rows, cols], scale_inv [ceil(rows/128), ceil(cols/128)] fp32)``.

    ``scale_inv`` is ``amax / 448`` per block (448 is the largest e4m3 value), so that
    ``dequant_block_fp8`` undoes it up to the e4m3 rounding.  Used to build synthetic FP8 checkpoints
    and benchmark weights.
    """
    rows, cols = w.shape
    br, bc = block
    pr, pc = (rows + br - 1) // br, (cols + bc - 1) // bc
    padded = torch.zeros(pr * br, pc * bc, dtype=torch.float32, device=w.device)
    padded[:rows, :cols] = w.to(torch.float32)
    tiles = padded.view(pr, br, pc, bc)
    amax = tiles.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale_inv = amax / 448.0
    q = (tiles / scale_inv[:, None, :, None]).view(pr * br, pc * bc)[:rows, :cols].to(torch.float8_e4m3fn)
    return q, scale_inv


class CheckpointReader:
    """Reads tensors by name through the shard index, and a layer's experts in the two layouts above."""

    def __init__(self, snapshot: str | Path = DEFAULT_SNAPSHOT):
        self.root = Path(snapshot)
        self.index: dict[str, str] = json.loads((self.root / "model.safetensors.index.json").read_text())["weight_map"]
        quant = json.loads((self.root / "config.json").read_text()).get("quantization_config") or {}
        rows, cols = quant.get("weight_block_size", (128, 128))
        self.block: tuple[int, int] = (int(rows), int(cols))

    # ---- raw access ------------------------------------------------------------------------------------
    def get(self, names: list[str]) -> dict[str, torch.Tensor]:
        """The named tensors; every shard file that holds one of them is opened once."""
        from safetensors import safe_open

        by_shard: dict[str, list[str]] = {}
        for name in names:
            by_shard.setdefault(self.index[name], []).append(name)
        found: dict[str, torch.Tensor] = {}
        for shard, wanted in by_shard.items():
            with safe_open(self.root / shard, framework="pt") as handle:
                found.update((name, handle.get_tensor(name)) for name in wanted)
        return found

    def _projections(self, layer: int, experts: range):
        """For every requested expert: ``{projection: (weight as stored, block scales or None)}``."""
        stem = PREFIX.format(layer=layer) + ".experts.{expert}.{projection}"
        weight_of = {(e, p): stem.format(expert=e, projection=p) + ".weight" for e in experts for p in PROJECTIONS}
        scale_of = {key: name + "_scale_inv" for key, name in weight_of.items() if name + "_scale_inv" in self.index}
        raw = self.get([*weight_of.values(), *scale_of.values()])
        for e in experts:
            yield {p: (raw[weight_of[e, p]], raw[scale_of[e, p]] if (e, p) in scale_of else None) for p in PROJECTIONS}

    def _as_fp32(self, weight: torch.Tensor, scales: torch.Tensor | None) -> torch.Tensor:
        if weight.dtype == torch.float8_e4m3fn:
            return dequant_block_fp8(weight, scales, self.block)
        return weight.to(torch.float32)

    # ---- a layer's experts ---------------------------------------------------------------------------------
    def expert_weights(self, layer: int, experts: range, dtype=torch.bfloat16) -> tuple[torch.Tensor, torch.Tensor]:
        """Dequantised: ``w13 [n, 2I, H]`` (gate rows, then up rows) and ``w2 [n, H, I]`` in ``dtype``."""
        gate_up, down = [], []
        for projections in self._projections(layer, experts):
            dense = {name: self._as_fp32(*stored) for name, stored in projections.items()}
            gate_up.append(torch.cat((dense["gate_proj"], dense["up_proj"])).to(dtype))
            down.append(dense["down_proj"].to(dtype))
        return torch.stack(gate_up), torch.stack(down)

    def expert_weights_fp8(self, layer: int, experts: range):
        """As stored: ``(w13 e4m3 [n, 2I, H], its scales fp32 [n, 2I/128, H/128], w2 e4m3 [n, H, I], its scales)``."""
        def as_bytes(t: torch.Tensor) -> torch.Tensor:  # cat / stack are not defined for float8 tensors
            return t.view(torch.uint8)

        columns: tuple[list, list, list, list] = ([], [], [], [])
        for projections in self._projections(layer, experts):
            for name, (weight, scales) in projections.items():
                if weight.dtype != torch.float8_e4m3fn or scales is None:
                    raise ValueError(f"layer {layer}: {name} is stored as {weight.dtype}, not block-scaled float8_e4m3fn")
            (gate, gate_s), (up, up_s), (down, down_s) = (projections[name] for name in PROJECTIONS)
            if gate.shape[0] % self.block[0]:
                raise ValueError("gate/up rows must be a multiple of the scale block to be stacked")
            columns[0].append(torch.cat((as_bytes(gate), as_bytes(up))))
            columns[1].append(torch.cat((gate_s, up_s)).to(torch.float32))
            columns[2].append(as_bytes(down))
            columns[3].append(down_s.to(torch.float32))
        w13, s13, w2, s2 = (torch.stack(column) for column in columns)
        return w13.view(torch.float8_e4m3fn), s13, w2.view(torch.float8_e4m3fn), s2

    def router(self, layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Gate weight ``[E, H]`` and selection bias ``e_score_correction_bias [E]``, both fp32."""
        gate = PREFIX.format(layer=layer) + ".gate."
        raw = self.get([gate + "weight", gate + "e_score_correction_bias"])
        return raw[gate + "weight"].to(torch.float32), raw[gate + "e_score_correction_bias"].to(torch.float32)
