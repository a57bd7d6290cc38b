"""Python entry points of the standalone sm_100a kernels (router top-k, RMSNorm) and helpers shared by
the fused layer (tensor maps for the weight stream, SM count).  Each call launches on the current
CUDA stream, allocates only its outputs, and raises if the native library is missing.
"""

from __future__ import annotations

import ctypes as C
from functools import lru_cache

import torch

from ..config import MoEConfig
from . import _lib


def _need_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{what} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous")


@lru_cache(maxsize=8)
def sm_count(device_index: int) -> int:
    out = C.c_int()
    with torch.cuda.device(device_index):
        _lib.check(_lib.lib().mf_device_sm_count(C.byref(out)), "sm count")
    return out.value


def router_topk(
    logits: torch.Tensor,
    bias: torch.Tensor | None,
    cfg: MoEConfig,
    out_weights: torch.Tensor | None = None,
    out_ids: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """``logits [T, E]`` fp32 -> ``(weights [T, K] fp32, ids [T, K] int32)`` (see ``router.route``)."""
    _need_cuda(logits, "logits")
    if logits.dtype != torch.float32:
        raise ValueError("router_topk takes fp32 logits")
    n_tokens, n_experts = logits.shape
    if bias is not None:
        _need_cuda(bias, "bias")
        if bias.dtype != torch.float32 or bias.numel() != n_experts:
            raise ValueError("bias must be fp32 [E]")
    if cfg.scoring_func not in ("sigmoid", "softmax"):
        raise ValueError(f"unknown scoring function {cfg.scoring_func!r}")
    w = out_weights if out_weights is not None else torch.empty(n_tokens, cfg.top_k, dtype=torch.float32, device=logits.device)
    ids = out_ids if out_ids is not None else torch.empty(n_tokens, cfg.top_k, dtype=torch.int32, device=logits.device)
    _lib.check(
        _lib.lib().mf_router_topk(
            logits.data_ptr(), _lib.ptr(bias), w.data_ptr(), ids.data_ptr(), n_tokens, n_experts, cfg.top_k,
            cfg.n_group, cfg.topk_group, int(cfg.scoring_func == "sigmoid"), int(cfg.norm_topk_prob),
            float(cfg.routed_scaling_factor), _lib.stream_ptr(),
        ),
        "router_topk",
    )
    return w, ids


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out = x * rsqrt(mean(x^2) + eps) * gamma`` per row; bf16 in/out, fp32 math, one rounding."""
    _need_cuda(x, "x")
    _need_cuda(gamma, "gamma")
    if x.dtype != torch.bfloat16 or gamma.dtype != torch.bfloat16:
        raise ValueError("rmsnorm takes bf16 tensors")
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    out = out if out is not None else torch.empty_like(x)
    _lib.check(
        _lib.lib().mf_rmsnorm(x.data_ptr(), gamma.data_ptr(), out.data_ptr(), rows, hidden, float(eps), _lib.stream_ptr()),
        "rmsnorm",
    )
    return out


def make_tile_tmap(x: torch.Tensor, box_rows: int) -> C.Array:
    """128-byte TMA descriptor over a contiguous ``x [rows, K]`` with boxes of ``box_rows`` rows x 128 bytes.

    Used for the token operand of the down GEMM (its rows are contiguous in expert-major order), with
    ``box_rows`` equal to the kernel's token-tile width.  The buffer must outlive every launch that uses it.
    """
    _need_cuda(x, "token operand")
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError("the token operand must be a contiguous [rows, K] tensor")
    buf = (C.c_ubyte * 128)()
    _lib.check(_lib.lib().mf_make_tile_tmap(buf, x.data_ptr(), x.shape[0], x.shape[1], x.element_size(), box_rows),
               "tensor map")
    return buf


def make_weight_tmap(w: torch.Tensor) -> C.Array:
    """128-byte TMA descriptor over ``w`` viewed as ``[rows, K]`` (K innermost, 128 B x 128 row boxes)."""
    _need_cuda(w, "weight")
    k_elems = w.shape[-1]
    rows = w.numel() // k_elems
    buf = (C.c_ubyte * 128)()
    _lib.check(_lib.lib().mf_make_weight_tmap(buf, w.data_ptr(), rows, k_elems, w.element_size()), "tensor map")
    return buf
