"""Stand-alone entry points of the tcgen05 grouped expert GEMMs.

``FixedEPLayer`` drives the same kernels through pre-built argument blocks and a device-side plan; the
functions here build the plan from host-known expert offsets, which is convenient for tests, the
shared expert (one "expert" holding every token) and experiments.

    act = gate_up_swiglu(x, w13, offsets, row_index=None, limit=10.0)     # [N, I]
    y   = down_proj(act, w2, offsets, row_scale=None)                      # [N, H]

``x`` rows may be gathered by ``row_index`` (entry -> row of ``x``) inside the kernel; ``x`` rows then only
need a 16-byte aligned pitch.  Replaces ``moeflow/kernels/grouped_gemm.py:101-161`` of the reference.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from .kernels import make_tile_tmap, make_weight_tmap, sm_count


@dataclass
class TilePlan:
    tile_e: torch.Tensor
    tile_s: torch.Tensor
    tile_n: torch.Tensor
    plan: torch.Tensor
    n_tiles: int
    n_entries: int
    block_m: int


def plan_from_offsets(offsets, block_m: int, device, split1: int = 1, split2: int = 1) -> TilePlan:
    """Token tiles ``(expert, first entry, count <= block_m)`` from host-side expert offsets."""
    offs = [int(v) for v in (offsets.tolist() if torch.is_tensor(offsets) else offsets)]
    te, ts, tn = [], [], []
    for e, (lo, hi) in enumerate(zip(offs[:-1], offs[1:])):
        for s in range(lo, hi, block_m):
            te.append(e)
            ts.append(s)
            tn.append(min(block_m, hi - s))
    i32 = dict(dtype=torch.int32, device=device)
    plan = torch.zeros(_lib.PLAN_WORDS, **i32)
    plan[_lib.PLAN_N_TILES] = len(te)
    plan[_lib.PLAN_SPLIT1] = split1
    plan[_lib.PLAN_SPLIT2] = split2
    plan[_lib.PLAN_N_ENTRIES] = offs[-1]
    pad = [0]
    return TilePlan(
        torch.tensor(te or pad, **i32), torch.tensor(ts or pad, **i32), torch.tensor(tn or pad, **i32), plan, len(te),
        offs[-1], block_m,
    )


def _scratch(tp: TilePlan, m_blocks: int, split: int, device, grid: int):
    """Partial-sum tiles and arrival counters for a K cut: ``split`` segments per unit, or (``split == 0``,
    stream-K) two tiles per CTA."""
    slots = max(1, 2 * grid if split == 0 else tp.n_tiles * m_blocks * split)
    partial = torch.empty(slots * 2 * tp.block_m * 128 if split != 1 else 1, dtype=torch.float32, device=device)
    counters = torch.zeros(max(1, tp.n_tiles) * m_blocks * 8, dtype=torch.int32, device=device)  # x2: fp8 column groups
    return partial, counters, slots


def gate_up_swiglu(
    x: torch.Tensor,
    w13: torch.Tensor,
    tp: TilePlan,
    row_index: torch.Tensor | None = None,
    limit: float | None = 10.0,
    round_h: bool = False,
    split: int = 1,
    status: torch.Tensor | None = None,
    wait_ns: int = 2_000_000_000,
    grid: int | None = None,
    b_tma: bool = False,
) -> torch.Tensor:
    """``act[n] = silu(min(x[i_n] . Wg^T, lim)) * clamp(x[i_n] . Wu^T, +-lim)`` per expert segment.

    ``b_tma`` (only without ``row_index``, contiguous ``x``): fetch the token tiles by TMA instead of the
    16-byte gather."""
    n_exp, two_i, hidden = w13.shape
    inter = two_i // 2
    if x.dtype != torch.bfloat16 or w13.dtype != torch.bfloat16:
        raise ValueError("bf16 only")
    if hidden % 64 or inter % 128:
        raise ValueError("hidden must be a multiple of 64 and intermediate a multiple of 128")
    if x.stride(-1) != 1 or (x.stride(0) * 2) % 16 or x.data_ptr() % 16:
        raise ValueError("x rows must be 16-byte aligned with unit inner stride")
    dev = x.device
    w13 = w13.contiguous()
    tmap = make_weight_tmap(w13)
    act = torch.zeros(max(tp.n_entries, 1), inter, dtype=torch.bfloat16, device=dev)
    tp.plan[_lib.PLAN_SPLIT1] = split
    grid = grid or sm_count(dev.index or 0)
    partial, counters, slots = _scratch(tp, inter // 128, split, dev, grid)
    status = status if status is not None else torch.zeros(1, dtype=torch.int64, device=dev)
    args = _lib.GemmArgs(
        b_base=x.data_ptr(), b_pitch=x.stride(0) * 2, b_index=_lib.ptr(row_index), tile_e=tp.tile_e.data_ptr(),
        tile_s=tp.tile_s.data_ptr(), tile_n=tp.tile_n.data_ptr(), plan=tp.plan.data_ptr(), split_word=_lib.PLAN_SPLIT1,
        m_blocks=inter // 128, k_blocks=hidden // 64, rows_per_expert=two_i, up_row_offset=inter, out=act.data_ptr(),
        out_pitch=inter, row_scale=None, partial=partial.data_ptr(), counters=counters.data_ptr(),
        max_split_slots=slots, limit=float(limit) if limit is not None else 0.0, round_h=int(round_h),
        status=status.data_ptr(), wait_ns=wait_ns, partial_floats=partial.numel(), n_counters=counters.numel(),
        max_tiles=tp.tile_e.numel(),
    )
    tmap_b = None
    if b_tma:
        if row_index is not None or not x.is_contiguous():
            raise ValueError("token tiles by TMA need contiguous rows and no row index")
        if x.shape[0] < tp.block_m:  # the tensor map needs at least one box of rows
            x = torch.cat([x, x.new_zeros(tp.block_m - x.shape[0], hidden)])
            args.b_base = x.data_ptr()
        tmap_b = make_tile_tmap(x, tp.block_m)
        args.b_tmap = C.addressof(tmap_b)
    _lib.check(_lib.lib().mf_gemm_gate_up(tmap, C.byref(args), tp.block_m, grid, _lib.stream_ptr()), "gate/up gemm")
    act._keep = (w13, partial, counters, status, row_index, x)
    return act[: tp.n_entries]


def down_proj(
    act: torch.Tensor,
    w2: torch.Tensor,
    tp: TilePlan,
    row_scale: torch.Tensor | None = None,
    split: int = 1,
    status: torch.Tensor | None = None,
    wait_ns: int = 2_000_000_000,
    grid: int | None = None,
    b_tma: bool = True,
    two_blocks: bool = False,
) -> torch.Tensor:
    """``y[n] = bf16(row_scale[n] * (act[n] . W2[e_n]^T))`` per expert segment.

    ``two_blocks``: a work unit covers two adjacent 128-row weight blocks (hidden must be a multiple of 256).

    ``b_tma``: fetch the token tiles of ``act`` by TMA (its rows are contiguous); ``False`` gathers them
    16 bytes at a time like the gate/up GEMM does for indexed rows.
    """
    n_exp, hidden, inter = w2.shape
    if act.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16:
        raise ValueError("bf16 only")
    if hidden % 128 or inter % 64:
        raise ValueError("hidden must be a multiple of 128 and intermediate a multiple of 64")
    dev = act.device
    act = act.contiguous()
    w2 = w2.contiguous()
    tmap = make_weight_tmap(w2)
    y = torch.zeros(max(tp.n_entries, 1), hidden, dtype=torch.bfloat16, device=dev)
    tp.plan[_lib.PLAN_SPLIT2] = split
    grid = grid or sm_count(dev.index or 0)
    partial, counters, slots = _scratch(tp, hidden // 128, split, dev, grid)
    status = status if status is not None else torch.zeros(1, dtype=torch.int64, device=dev)
    if two_blocks and hidden % 256:
        raise ValueError("two_blocks needs a hidden size that is a multiple of 256")
    args = _lib.GemmArgs(
        b_base=act.data_ptr(), b_pitch=inter * 2, b_index=None, tile_e=tp.tile_e.data_ptr(), tile_s=tp.tile_s.data_ptr(),
        tile_n=tp.tile_n.data_ptr(), plan=tp.plan.data_ptr(), split_word=_lib.PLAN_SPLIT2,
        m_blocks=hidden // 256 if two_blocks else hidden // 128, two_blocks=int(two_blocks),
        k_blocks=inter // 64, rows_per_expert=hidden, up_row_offset=128 if two_blocks else 0, out=y.data_ptr(), out_pitch=hidden,
        row_scale=_lib.ptr(row_scale), partial=partial.data_ptr(), counters=counters.data_ptr(), max_split_slots=slots,
        limit=0.0, round_h=0, status=status.data_ptr(), wait_ns=wait_ns, partial_floats=partial.numel(),
        n_counters=counters.numel(), max_tiles=tp.tile_e.numel(),
    )
    tmap_b = None
    if b_tma:
        tmap_b = make_tile_tmap(act, tp.block_m)
        args.b_tmap = C.addressof(tmap_b)
    _lib.check(_lib.lib().mf_gemm_down(tmap, C.byref(args), tp.block_m, grid, _lib.stream_ptr()), "down gemm")
    y._keep = (w2, partial, counters, status, row_scale, act)
    return y[: tp.n_entries]
