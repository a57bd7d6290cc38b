"""Block-scaled FP8 (e4m3) expert path: activation quantiser and the two grouped GEMMs.

Format (GLM-5.3-Flash FP8 checkpoint): weights ``float8_e4m3fn`` with one fp32 ``weight_scale_inv`` per
128x128 block; activations quantised on the fly with one fp32 scale per row and 128-wide group:
``scale = max(amax, 1e-10) / 448``, ``q = e4m3(x / scale)``.  The GEMM kernels accumulate every 128-wide
K block on the tensor cores (``tcgen05 kind::f8f6f4``) and promote it into fp32 registers with
``w_scale * x_scale``; see ``csrc/grouped_gemm_fp8.cu``.

``quant_rows_reference`` / ``dequant_rows`` are the PyTorch definition the kernels are tested against.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .grouped_gemm import TilePlan, _scratch
from .kernels import make_tile_tmap, make_weight_tmap, sm_count

E4M3_MAX = 448.0


def quant_rows_reference(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``x [N, K]`` -> ``(q [N, K] e4m3, scales [N, K/128] fp32)`` in PyTorch."""
    n, k = x.shape
    g = x.to(torch.float32).view(n, k // 128, 128)
    scale = g.abs().amax(dim=-1).clamp(min=1e-10) / E4M3_MAX
    q = (g / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(n, k), scale


def dequant_rows(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    n, k = q.shape
    return (q.to(torch.float32).view(n, k // 128, 128) * scale[..., None]).view(n, k)


def quant_rows_1x128(x: torch.Tensor, row_index: torch.Tensor | None = None, rows: int | None = None,
                     out_q: torch.Tensor | None = None, out_s: torch.Tensor | None = None, valid_off: int = -1,
                     n_rows_dev: torch.Tensor | None = None, hidden: int | None = None):
    """Quantise bf16 rows on the device.  ``x`` may be a row store with a larger pitch (``hidden`` given)."""
    if x.dtype != torch.bfloat16 or x.stride(-1) != 1:
        raise ValueError("bf16 rows with unit inner stride expected")
    k = hidden if hidden is not None else x.shape[-1]
    n = rows if rows is not None else (row_index.numel() if row_index is not None else x.shape[0])
    q = out_q if out_q is not None else torch.zeros(n, k, dtype=torch.float8_e4m3fn, device=x.device)
    s = out_s if out_s is not None else torch.zeros(n, k // 128, dtype=torch.float32, device=x.device)
    _lib.check(
        _lib.lib().mf_quant_rows_1x128(x.data_ptr(), x.stride(0) * 2, _lib.ptr(row_index), n, k, q.data_ptr(), s.data_ptr(),
                                       valid_off, _lib.ptr(n_rows_dev), _lib.stream_ptr()),
        "quant_rows_1x128",
    )
    return q, s


def _gemm_fp8(gate_up: bool, xq, xs, wq, ws, tp: TilePlan, out, row_index, row_scale, limit, split, status, wait_ns, grid,
              b_tma: bool = False):
    n_exp, rows, k = wq.shape
    if xq.dtype != torch.float8_e4m3fn or wq.dtype != torch.float8_e4m3fn:
        raise ValueError("e4m3 operands expected")
    if k % 128 or rows % 128 or k > 4096:
        raise ValueError("K must be a multiple of 128 and at most 4096; weight rows a multiple of 128")
    dev = xq.device
    wq = wq.contiguous()
    ws = ws.to(torch.float32).contiguous()
    if tuple(ws.shape) != (n_exp, rows // 128, k // 128):
        raise ValueError(f"weight scales must be [{n_exp}, {rows // 128}, {k // 128}]")
    tmap = make_weight_tmap(wq.view(torch.uint8))
    inter = rows // 2 if gate_up else rows
    m_blocks = inter // 128
    word = _lib.PLAN_SPLIT1 if gate_up else _lib.PLAN_SPLIT2
    tp.plan[word] = split
    grid = grid or sm_count(dev.index or 0)
    partial, counters, slots = _scratch(tp, m_blocks, split, dev, grid)
    status = status if status is not None else torch.zeros(1, dtype=torch.int64, device=dev)
    args = _lib.GemmArgs(
        b_base=xq.data_ptr(), b_pitch=xq.stride(0), b_index=_lib.ptr(row_index), tile_e=tp.tile_e.data_ptr(),
        tile_s=tp.tile_s.data_ptr(), tile_n=tp.tile_n.data_ptr(), plan=tp.plan.data_ptr(), split_word=word,
        m_blocks=m_blocks, k_blocks=k // 128, rows_per_expert=rows, up_row_offset=inter if gate_up else 0,
        out=out.data_ptr(), out_pitch=out.shape[1], row_scale=_lib.ptr(row_scale), partial=partial.data_ptr(),
        counters=counters.data_ptr(), max_split_slots=slots, limit=float(limit) if limit is not None else 0.0, round_h=0,
        status=status.data_ptr(), wait_ns=wait_ns, w_scale=ws.data_ptr(), b_scale=xs.data_ptr(), b_scale_pitch=xs.stride(0),
        partial_floats=partial.numel(), n_counters=counters.numel(), max_tiles=tp.tile_e.numel(),
    )
    tmap_b = None
    if b_tma:
        if row_index is not None or not xq.is_contiguous():
            raise ValueError("token tiles by TMA need contiguous rows and no row index")
        xq8 = xq.view(torch.uint8)
        if xq8.shape[0] < tp.block_m:  # the tensor map needs at least one box of rows
            xq8 = torch.cat([xq8, xq8.new_zeros(tp.block_m - xq8.shape[0], k)])
            args.b_base = xq8.data_ptr()
        tmap_b = make_tile_tmap(xq8, tp.block_m)
        args.b_tmap = C.addressof(tmap_b)
        xq = xq8
    fn = _lib.lib().mf_gemm_gate_up_fp8 if gate_up else _lib.lib().mf_gemm_down_fp8
    _lib.check(fn(tmap, C.byref(args), tp.block_m, grid, _lib.stream_ptr()), "fp8 gemm")
    out._keep = (wq, ws, partial, counters, status, xq, xs, row_index, row_scale)
    return out


def gate_up_swiglu_fp8(xq, xs, w13_q, w13_s, tp: TilePlan, row_index=None, limit=10.0, split=1, status=None,
                       wait_ns=2_000_000_000, grid=None) -> torch.Tensor:
    """``act [N, I]`` bf16 from e4m3 rows ``xq`` (scales ``xs [rows, K/128]``) and ``w13_q [E, 2I, H]``."""
    inter = w13_q.shape[1] // 2
    act = torch.zeros(max(tp.n_entries, 1), inter, dtype=torch.bfloat16, device=xq.device)
    return _gemm_fp8(True, xq, xs, w13_q, w13_s, tp, act, row_index, None, limit, split, status, wait_ns, grid)[: tp.n_entries]


def down_proj_fp8(aq, a_s, w2_q, w2_s, tp: TilePlan, row_scale=None, split=1, status=None, wait_ns=2_000_000_000, grid=None,
                  b_tma: bool = True):
    """``y [N, H]`` bf16 = ``row_scale * (dequant(aq) . dequant(w2)^T)``; ``b_tma``: token tiles by TMA or by the
    16-byte gather."""
    hidden = w2_q.shape[1]
    y = torch.zeros(max(tp.n_entries, 1), hidden, dtype=torch.bfloat16, device=aq.device)
    return _gemm_fp8(False, aq, a_s, w2_q, w2_s, tp, y, None, row_scale, None, split, status, wait_ns, grid,
                     b_tma=b_tma)[: tp.n_entries]


def expand_block_fp8(w_q: torch.Tensor, w_s: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Block-scaled e4m3 weights ``[..., rows, K]`` with fp32 scales ``[..., rows/128, K/128]`` -> bf16, one pass.

    ``out`` (bf16, same shape, contiguous) is overwritten when given.  Used by layers that hold e4m3 experts and run
    the bf16 grouped GEMMs on long-prefill tiles.
    """
    if w_q.dtype not in (torch.float8_e4m3fn, torch.uint8) or not w_q.is_contiguous():
        raise ValueError("contiguous e4m3 weights expected")
    K = w_q.shape[-1]
    rows = w_q.numel() // K
    if rows % 128 or K % 128:
        raise ValueError("rows and K must be multiples of 128")
    w_s = w_s.to(torch.float32).contiguous()
    if w_s.numel() != (rows // 128) * (K // 128):
        raise ValueError("one fp32 scale per 128x128 block expected")
    if out is None:
        out = torch.empty(w_q.shape, dtype=torch.bfloat16, device=w_q.device)
    elif out.dtype != torch.bfloat16 or out.numel() != w_q.numel() or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 tensor of the weights' shape")
    _lib.check(_lib.lib().mf_dequant_block_fp8(w_q.data_ptr(), w_s.data_ptr(), out.data_ptr(), rows, K, _lib.stream_ptr()),
               "expand e4m3 weights")
    return out
