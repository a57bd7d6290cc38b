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
    """``h [N, 2I] = [gate | up]`` -> ``[N, I]``; fp32 math, result in ``h.dtype``."""
    inter = h.shape[-1] // 2
    gate = h[..., :inter].to(torch.float32)
    up = h[..., inter:].to(torch.float32)
    if limit is not None:
        gate = gate.clamp(max=limit)
        up = up.clamp(min=-limit, max=limit)
    return (F.silu(gate) * up).to(h.dtype)


class ExpertCompute(Protocol):
    name: str

    def __call__(
        self,
        a: torch.Tensor,
        expert_offsets: torch.Tensor,
        w13: torch.Tensor,
        w2: torch.Tensor,
        swiglu_limit: float | None,
        row_weight: torch.Tensor | None = None,
    ) -> torch.Tensor: ...


class TorchLoopExperts:
    """One GEMM pair per non-empty local expert (reads the offsets on the host)."""

    name = "torch_loop"

    def __call__(self, a, expert_offsets, w13, w2, swiglu_limit, row_weight=None):
        bounds = [int(v) for v in expert_offsets.tolist()]
        out = torch.empty_like(a)
        for e, (lo, hi) in enumerate(zip(bounds[:-1], bounds[1:])):
            if hi == lo:
                continue
            act = swiglu_clamp(a[lo:hi] @ w13[e].transpose(0, 1), swiglu_limit)
            if row_weight is None:
                out[lo:hi] = act @ w2[e].transpose(0, 1)
            else:
                y = act.to(torch.float32) @ w2[e].to(torch.float32).transpose(0, 1)
                out[lo:hi] = (y * row_weight[lo:hi, None]).to(a.dtype)
        return out


class BatchedTorchExperts:
    """Device-only variant (no host sync): pads every expert segment to the longest one via bmm.

    Only meant for small shapes in tests and CPU runs.
    """

    name = "torch_bmm"

    def __call__(self, a, expert_offsets, w13, w2, swiglu_limit, row_weight=None):
        n = a.shape[0]
        if n == 0:
            return torch.empty_like(a)
        offs = expert_offsets.to(torch.int64)
        pos = torch.arange(n, device=a.device)
        expert_of = torch.searchsorted(offs[1:].contiguous(), pos, right=True).clamp(max=w13.shape[0] - 1)
        h = torch.einsum("nh,nfh->nf", a.to(torch.float32), w13[expert_of].to(torch.float32)).to(a.dtype)
        act = swiglu_clamp(h, swiglu_limit)
        y = torch.einsum("ni,nhi->nh", act.to(torch.float32), w2[expert_of].to(torch.float32))
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
