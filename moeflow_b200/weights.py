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
    def __init__(self, snapshot: str | Path = DEFAULT_SNAPSHOT):
        self.root = Path(snapshot)
        self.index: dict[str, str] = json.loads((self.root / "model.safetensors.index.json").read_text())["weight_map"]
        cfg = json.loads((self.root / "config.json").read_text())
        quant = cfg.get("quantization_config") or {}
        self.block: tuple[int, int] = tuple(quant.get("weight_block_size", (128, 128)))  # type: ignore[assignment]

    def get(self, names: list[str]) -> dict[str, torch.Tensor]:
        """Read the named tensors, opening every shard file once."""
        from safetensors import safe_open

        wanted: dict[str, list[str]] = {}
        for name in names:
            wanted.setdefault(self.index[name], []).append(name)
        out: dict[str, torch.Tensor] = {}
        for shard, shard_names in wanted.items():
            with safe_open(self.root / shard, framework="pt") as handle:
                for name in shard_names:
                    out[name] = handle.get_tensor(name)
        return out

    def _expert_names(self, layer: int, experts: range) -> list[str]:
        base = PREFIX.format(layer=layer)
        names = []
        for e in experts:
            for proj in PROJECTIONS:
                stem = f"{base}.experts.{e}.{proj}"
                names.append(f"{stem}.weight")
                if f"{stem}.weight_scale_inv" in self.index:
                    names.append(f"{stem}.weight_scale_inv")
        return names

    def _dense(self, stem: str, raw: dict[str, torch.Tensor]) -> torch.Tensor:
        w = raw[f"{stem}.weight"]
        if w.dtype == torch.float8_e4m3fn:
            return dequant_block_fp8(w, raw[f"{stem}.weight_scale_inv"], self.block)
        return w.to(torch.float32)

    def expert_weights(self, layer: int, experts: range, dtype=torch.bfloat16) -> tuple[torch.Tensor, torch.Tensor]:
        raw = self.get(self._expert_names(layer, experts))
        base = PREFIX.format(layer=layer)
        w13, w2 = [], []
        for e in experts:
            stem = f"{base}.experts.{e}"
            gate, up = self._dense(f"{stem}.gate_proj", raw), self._dense(f"{stem}.up_proj", raw)
            w13.append(torch.cat([gate, up], dim=0).to(dtype))
            w2.append(self._dense(f"{stem}.down_proj", raw).to(dtype))
        return torch.stack(w13), torch.stack(w2)

    def expert_weights_fp8(self, layer: int, experts: range):
        """Keep e4m3 weights and their fp32 128x128 block scales un-dequantised."""
        raw = self.get(self._expert_names(layer, experts))
        base = PREFIX.format(layer=layer)
        q13, s13, q2, s2 = [], [], [], []
        for e in experts:
            stem = f"{base}.experts.{e}"
            parts = {}
            for proj in PROJECTIONS:
                w = raw[f"{stem}.{proj}.weight"]
                if w.dtype != torch.float8_e4m3fn:
                    raise ValueError(f"{stem}.{proj} is {w.dtype}, not float8_e4m3fn")
                parts[proj] = (w, raw[f"{stem}.{proj}.weight_scale_inv"].to(torch.float32))
            if parts["gate_proj"][0].shape[0] % self.block[0]:
                raise ValueError("gate/up rows must be a multiple of the scale block to be stacked")
            q13.append(torch.cat([parts["gate_proj"][0].view(torch.uint8), parts["up_proj"][0].view(torch.uint8)]).view(torch.float8_e4m3fn))
            s13.append(torch.cat([parts["gate_proj"][1], parts["up_proj"][1]]))
            q2.append(parts["down_proj"][0])
            s2.append(parts["down_proj"][1])
        stack8 = lambda ts: torch.stack([t.view(torch.uint8) for t in ts]).view(torch.float8_e4m3fn)  # noqa: E731
        return stack8(q13), torch.stack(s13), stack8(q2), torch.stack(s2)

    def router(self, layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Gate weight ``[E, H]`` and ``e_score_correction_bias [E]``, both fp32."""
        base = PREFIX.format(layer=layer)
        raw = self.get([f"{base}.gate.weight", f"{base}.gate.e_score_correction_bias"])
        return raw[f"{base}.gate.weight"].to(torch.float32), raw[f"{base}.gate.e_score_correction_bias"].to(torch.float32)
