"""Expert compute backends over an expert-major row layout (PyTorch implementations).

``a [N, H]`` holds the gathered token rows ordered by local expert; ``expert_offsets [L+1]`` delimits
them.  Each backend returns ``[N, H]`` in ``a.dtype``; with ``row_weight`` the routing weight multiplies
the fp32 down-projection sum before the single cast.  The CUDA (tcgen05) path lives in
``moeflow_b200.ops.grouped_gemm``.  Behavioural counterpart of ``moeflow/experts.py:10-78``.
"""

from __future__ import annotations

from typing import Protocol

import torch
import torch.nn.functional as F


def swiglu_clamp(h: torch.Tensor, limit: float | None) -> torch.Tensor:
    """``h [..., 2I]`` holding the gate half and then the up half -> ``silu(gate) * up`` as ``[..., I]``.
    With a limit the gate is capped from above and the up half on both sides.  fp32 math, ``h.dtype`` out."""
    gate, up = (half.to(torch.float32) for half in h.chunk(2, dim=-1))
    if limit is not None:
        gate, up = gate.clamp(max=limit), up.clamp(min=-limit, max=limit)
    return F.silu(gate).mul(up).to(h.dtype)


class ExpertCompute(Protocol):
    """``a [N, H]`` rows in expert-major order, ``expert_offsets [L + 1]``, ``w13 [L, 2I, H]``, ``w2 [L, H, I]``
    -> ``[N, H]`` in ``a.dtype``.  ``row_weight [N]`` (fp32), when given, multiplies the fp32 result of the
    down projection before its only cast."""

    name: str

    def __call__(self, a: torch.Tensor, expert_offsets: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor,
                 swiglu_limit: float | None, row_weight: torch.Tensor | None = None) -> torch.Tensor: ...


def _segments(expert_offsets: torch.Tensor):
    """``(expert, first row, one past the last row)`` of every expert that has rows (reads the offsets on the host)."""
    edges = [int(v) for v in expert_offsets.tolist()]
    for expert in range(len(edges) - 1):
        if edges[expert + 1] > edges[expert]:
            yield expert, edges[expert], edges[expert + 1]


def _one_expert(rows: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, limit: float | None,
                weight: torch.Tensor | None) -> torch.Tensor:
    """The MLP of one expert on its rows.  Without a weight both projections run in the rows' dtype; with one
    the down projection is computed in fp32, scaled per row and cast once."""
    act = swiglu_clamp(F.linear(rows, gate_up), limit)
    if weight is None:
        return F.linear(act, down)
    exact = F.linear(act.to(torch.float32), down.to(torch.float32))
    return exact.mul(weight[:, None]).to(rows.dtype)


class TorchLoopExperts:
    """A pair of library GEMMs per expert that has rows."""

    name = "torch_loop"

    def __call__(self, a, expert_offsets, w13, w2, swiglu_limit, row_weight=None):
        out = torch.empty_like(a)
        for expert, lo, hi in _segments(expert_offsets):
            weight = None if row_weight is None else row_weight[lo:hi]
            out[lo:hi] = _one_expert(a[lo:hi], w13[expert], w2[expert], swiglu_limit, weight)
        return out


class BatchedTorchExperts:
    """No host round trip: every row fetches its own expert's matrices and the projections are batched
    row by row.  Memory-hungry (a weight copy per row), so for small shapes, tests and CPU runs only."""

    name = "torch_bmm"

    def __call__(self, a, expert_offsets, w13, w2, swiglu_limit, row_weight=None):
        if a.shape[0] == 0:
            return torch.empty_like(a)
        row = torch.arange(a.shape[0], device=a.device)
        ends = expert_offsets.to(torch.int64)[1:].contiguous()
        expert_of_row = torch.searchsorted(ends, row, right=True).clamp(max=w13.shape[0] - 1)
        x = a.to(torch.float32)[:, None, :]                                                  # [N, 1, H]
        h = torch.bmm(x, w13[expert_of_row].to(torch.float32).transpose(1, 2))[:, 0].to(a.dtype)  # [N, 2I]
        act = swiglu_clamp(h, swiglu_limit).to(torch.float32)[:, None, :]                    # [N, 1, I]
        y = torch.bmm(act, w2[expert_of_row].to(torch.float32).transpose(1, 2))[:, 0]        # [N, H]
        if row_weight is not None:
            y = y * row_weight[:, None]
        return y.to(a.dtype)


class Tcgen05GroupedExperts:
    """The sm_100a grouped GEMMs (gate/up + SwiGLU, down + routing weight) behind the ExpertCompute
    protocol of the variable-size pipeline.  The tile plan is built from the offsets on the host (this
    pipeline synchronises with the host anyway); ``FixedEPLayer`` drives the same kernels with a
    device-side plan instead."""

    name = "tcgen05_grouped"

    def __init__(self, block_m: int = 64):
        self.block_m = block_m

    def __call__(self, a, expert_offsets, w13, w2, swiglu_limit, row_weight=None):
        from .ops.grouped_gemm import down_proj, gate_up_swiglu, plan_from_offsets

        if a.shape[0] == 0:
            return torch.empty_like(a)
        tp = plan_from_offsets(expert_offsets, self.block_m, a.device)
        act = gate_up_swiglu(a.contiguous(), w13, tp, limit=swiglu_limit)
        scale = None if row_weight is None else row_weight.to(torch.float32).contiguous()
        return down_proj(act, w2, tp, row_scale=scale)


EXPERT_BACKENDS = {"torch_loop": TorchLoopExperts, "torch_bmm": BatchedTorchExperts, "tcgen05_grouped": Tcgen05GroupedExperts}
