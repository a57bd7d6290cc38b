"""The allocation-free down projection (``mf_gemm_down_static_scratch``) against ``mf_gemm_down``.

Some callers cannot obtain device memory when they call into the library (a plain C host, or serving
code running after the engine gave all free GPU memory to its cache pool), so this entry point keeps
its split-K scratch in a device array that belongs to the loaded library.  The test drives it through
the exported C symbol, twice in a row on different inputs — the second call meets the first call's
leftovers in the shared array — and expects the same bits as the ordinary entry point, which computes
with the same kernel and summation order.  Sizes beyond the array must be refused.

This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(counts, hidden, inter, seed):
    g = torch.Generator().manual_seed(seed)
    n = sum(counts)
    w2 = (torch.randn(len(counts), hidden, inter, generator=g) / inter**0.5).bfloat16().cuda()
    act = torch.randn(n, inter, generator=g).bfloat16().cuda()
    scale = (torch.rand(n, generator=g) + 0.5).float().cuda()
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    return w2, act, scale, offsets


def _static_scratch_call(act, w2, tp, scale, split, max_tiles=None):
    from moeflow_b200.ops import _lib
    from moeflow_b200.ops.kernels import make_weight_tmap, sm_count

    handle = _lib.lib()
    fn = handle.mf_gemm_down_static_scratch  # the exported C symbol
    fn.argtypes = [C.c_void_p, C.POINTER(_lib.GemmArgs), C.c_int, C.c_int, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    n_exp, hidden, inter = w2.shape
    y = torch.zeros(tp.n_entries, hidden, dtype=torch.bfloat16, device=act.device)
    status = torch.zeros(1, dtype=torch.int64, device=act.device)
    tp.plan[_lib.PLAN_SPLIT2] = split
    tmap = make_weight_tmap(w2)
    args = _lib.GemmArgs(
        b_base=act.data_ptr(), b_pitch=inter * 2, b_index=None, tile_e=tp.tile_e.data_ptr(), tile_s=tp.tile_s.data_ptr(),
        tile_n=tp.tile_n.data_ptr(), plan=tp.plan.data_ptr(), split_word=_lib.PLAN_SPLIT2, m_blocks=hidden // 128,
        k_blocks=inter // 64, rows_per_expert=hidden, up_row_offset=0, out=y.data_ptr(), out_pitch=hidden,
        row_scale=scale.data_ptr(), partial=None, counters=None, max_split_slots=0, limit=0.0, round_h=0,
        status=status.data_ptr(), wait_ns=50_000_000,
    )
    code = fn(tmap, C.byref(args), tp.n_tiles if max_tiles is None else max_tiles, split, sm_count(0), _lib.stream_ptr())
    return code, y, status


def test_matches_the_allocating_entry_point_twice_in_a_row():
    from moeflow_b200.ops._lib import decode_status
    from moeflow_b200.ops.grouped_gemm import down_proj, plan_from_offsets

    for seed, counts, split in ((1, [5, 0, 40, 9], 2), (2, [64, 3, 17, 1], 4)):
        w2, act, scale, offsets = _problem(counts, 512, 256, seed)
        tp = plan_from_offsets(offsets, 64, act.device)
        code, y, status = _static_scratch_call(act, w2, tp, scale, split)
        assert code == 0, code
        ref = down_proj(act, w2, tp, row_scale=scale, split=split)
        torch.cuda.synchronize()
        assert decode_status(int(status.item()))["code"] == 0
        assert torch.equal(y.view(torch.int16), ref.view(torch.int16))
        fp32 = torch.zeros_like(y, dtype=torch.float32)
        for e, (lo, hi) in enumerate(zip(offsets[:-1], offsets[1:])):
            fp32[lo:hi] = (act[lo:hi].float() @ w2[e].float().t()) * scale[lo:hi, None]
        assert ((y.float() - fp32).norm() / fp32.norm()).item() < 4 * 2.0**-8


def test_sizes_beyond_the_static_array_are_refused():
    from moeflow_b200.ops.grouped_gemm import plan_from_offsets

    w2, act, scale, offsets = _problem([3, 3], 512, 256, 3)
    tp = plan_from_offsets(offsets, 64, act.device)
    code, _, _ = _static_scratch_call(act, w2, tp, scale, 4, max_tiles=1000)  # 1000 * 4 * 4 slots
    assert code == -20
    code, _, _ = _static_scratch_call(act, w2, tp, scale, 1, max_tiles=2000)  # fits the slots? no: counters
    assert code in (-20, -21)
    code, _, _ = _static_scratch_call(act, w2, tp, scale, 3)
    assert code == -2


def test_a_plan_word_larger_than_declared_is_refused_on_the_device_and_nothing_is_written():
    """The caller declares ``max_tiles`` and ``split`` on the host, but the kernel reads the plan from device
    memory.  When the plan holds more tiles than declared, or tiles wider than the 64 rows this entry point
    supports, the kernel must report 'bad argument' and leave the output untouched instead of running past
    the static array."""
    from moeflow_b200.ops import _lib
    from moeflow_b200.ops.grouped_gemm import plan_from_offsets

    w2, act, scale, offsets = _problem([5, 0, 40, 9], 512, 256, 5)
    tp = plan_from_offsets(offsets, 64, act.device)
    true_tiles = tp.n_tiles
    tp.plan[_lib.PLAN_N_TILES] = true_tiles + 400  # the lie: (tiles + 400) * 4 blocks * 4 splits would overrun the array
    code, y, status = _static_scratch_call(act, w2, tp, scale, 4, max_tiles=true_tiles)
    torch.cuda.synchronize()
    assert code == 0  # the host-side check saw only the declared sizes
    assert _lib.decode_status(int(status.item()))["code"] == 7
    assert float(y.float().abs().sum()) == 0.0
    # tiles of 128 rows in a kernel built for 64: skipped and reported, the 64-row tiles still computed
    tp = plan_from_offsets(offsets, 64, act.device)
    tp.tile_n[0] = 100
    code, y, status = _static_scratch_call(act, w2, tp, scale, 2)
    torch.cuda.synchronize()
    assert code == 0 and _lib.decode_status(int(status.item()))["code"] == 7
    # and a correct call afterwards works on the same array
    tp = plan_from_offsets(offsets, 64, act.device)
    from moeflow_b200.ops.grouped_gemm import down_proj

    code, y, status = _static_scratch_call(act, w2, tp, scale, 2)
    ref = down_proj(act, w2, tp, row_scale=scale, split=2)
    torch.cuda.synchronize()
    assert code == 0 and _lib.decode_status(int(status.item()))["code"] == 0
    assert torch.equal(y.view(torch.int16), ref.view(torch.int16))
