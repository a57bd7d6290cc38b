"""tcgen05 grouped GEMMs (gate/up + SwiGLU, down + row scale) against plain fp32 PyTorch."""

import pytest
import torch

from moeflow_b200.experts import swiglu_clamp
from moeflow_b200.tolerances import normwise_rel_err

pytestmark = pytest.mark.gpu


def _status_ok(status):
    from moeflow_b200.ops._lib import decode_status

    st = decode_status(int(status.item()))
    assert st["code"] == 0, st


def _problem(counts, hidden, inter, seed=0, scale_x=1.0):
    g = torch.Generator().manual_seed(seed)
    n_exp = len(counts)
    n = sum(counts)
    w13 = (torch.randn(n_exp, 2 * inter, hidden, generator=g) * (2.0 / hidden**0.5)).bfloat16().cuda()
    w2 = (torch.randn(n_exp, hidden, inter, generator=g) / inter**0.5).bfloat16().cuda()
    n_src = max(n, 1) + 5
    x = (torch.randn(n_src, hidden, generator=g) * scale_x).bfloat16().cuda()
    row_index = torch.randint(0, n_src, (max(n, 1),), generator=g).int().cuda()
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    scale = torch.rand(max(n, 1), generator=g).float().cuda() + 0.5
    return w13, w2, x, row_index, offsets, scale


def _ref_gate_up(x, row_index, w13, offsets, limit):
    rows = x[row_index.long()].float()
    out = torch.zeros(offsets[-1], w13.shape[1] // 2, device=x.device)
    for e, (lo, hi) in enumerate(zip(offsets[:-1], offsets[1:])):
        if hi > lo:
            h = rows[lo:hi] @ w13[e].float().t()
            out[lo:hi] = swiglu_clamp(h, limit)
    return out


def _ref_down(act, w2, offsets, scale):
    out = torch.zeros(offsets[-1], w2.shape[1], device=act.device)
    for e, (lo, hi) in enumerate(zip(offsets[:-1], offsets[1:])):
        if hi > lo:
            out[lo:hi] = (act[lo:hi].float() @ w2[e].float().t()) * scale[lo:hi, None]
    return out


CASES = [
    ([1], 256, 128, 64),
    ([3, 0, 17, 5], 512, 256, 64),
    ([16, 64, 1, 0, 33], 1024, 384, 64),
    ([70, 2, 130], 512, 128, 64),  # experts longer than one tile
    ([5, 9], 512, 256, 32),
    ([100, 20], 512, 256, 128),
    ([128], 256, 128, 128),  # one full 128-row tile: UMMA N = 128, both 128-column accumulators of a stage
    ([300, 5, 129], 512, 256, 128),  # experts spanning several 128-row tiles, a one-row remainder
    ([128, 128, 64], 256, 128, 128),
    ([256], 256, 128, 256),  # 256-row tiles: UMMA N = 256, the gate/up accumulators fill all 512 tensor-memory columns
    ([300, 5, 600], 512, 256, 256),
]


@pytest.mark.parametrize("counts,hidden,inter,block_m", CASES)
@pytest.mark.parametrize("split", [0, 1, 2, 4])
def test_gate_up_and_down(counts, hidden, inter, block_m, split):
    """``split`` 1, 2, 4: equal K segments per unit; 0: the stream-K cut (every CTA one contiguous share of all
    K steps, units cut at CTA boundaries)."""
    from moeflow_b200.ops.grouped_gemm import down_proj, gate_up_swiglu, plan_from_offsets

    if split and (inter // 64) % split:
        pytest.skip("split does not divide the K blocks of the down GEMM")
    w13, w2, x, row_index, offsets, scale = _problem(counts, hidden, inter, seed=len(counts) + hidden)
    n = offsets[-1]
    tp = plan_from_offsets(offsets, block_m, x.device)
    status = torch.zeros(1, dtype=torch.int64, device=x.device)
    act = gate_up_swiglu(x, w13, tp, row_index=row_index[:n], limit=10.0, split=split, status=status, wait_ns=50_000_000)
    torch.cuda.synchronize()
    _status_ok(status)
    ref_act = _ref_gate_up(x, row_index[:n], w13, offsets, 10.0)
    assert normwise_rel_err(act, ref_act) < 4 * 2.0**-8, normwise_rel_err(act, ref_act)

    y = down_proj(act, w2, tp, row_scale=scale[:n], split=split, status=status, wait_ns=50_000_000)
    torch.cuda.synchronize()
    _status_ok(status)
    ref_y = _ref_down(act, w2, offsets, scale[:n])
    assert normwise_rel_err(y, ref_y) < 4 * 2.0**-8, normwise_rel_err(y, ref_y)
    # bf16 rounding of an fp32 result: element-wise within one bf16 ulp plus fp32 summation noise
    assert (y.float() - ref_y).abs().max() <= 2.0**-7 * ref_y.abs().max() + 1e-3


def test_clamp_is_exercised_and_identity_rows():
    from moeflow_b200.ops.grouped_gemm import gate_up_swiglu, plan_from_offsets

    w13, _, x, _, offsets, _ = _problem([20, 12], 256, 128, seed=5, scale_x=8.0)
    tp = plan_from_offsets(offsets, 64, x.device)
    status = torch.zeros(1, dtype=torch.int64, device=x.device)
    ident = torch.arange(offsets[-1], dtype=torch.int32, device=x.device)
    act = gate_up_swiglu(x, w13, tp, row_index=None, limit=2.0, status=status, wait_ns=50_000_000)
    torch.cuda.synchronize()
    _status_ok(status)
    ref = _ref_gate_up(x, ident, w13, offsets, 2.0)
    h = x[: offsets[-1]].float() @ w13[0].float().t()
    assert (h.abs() > 2.0).any(), "inputs do not reach the clamp"
    assert normwise_rel_err(act, ref) < 4 * 2.0**-8
    act_r = gate_up_swiglu(x, w13, tp, row_index=None, limit=2.0, round_h=True, status=status, wait_ns=50_000_000)
    ref_r = torch.zeros_like(ref)
    for e, (lo, hi) in enumerate(zip(offsets[:-1], offsets[1:])):
        ref_r[lo:hi] = swiglu_clamp((x[lo:hi].float() @ w13[e].float().t()).bfloat16(), 2.0).float()
    torch.cuda.synchronize()
    assert normwise_rel_err(act_r, ref_r) < 4 * 2.0**-8


@pytest.mark.parametrize("split", [4, 0])
def test_split_k_is_deterministic(split):
    from moeflow_b200.ops.grouped_gemm import gate_up_swiglu, plan_from_offsets

    w13, _, x, row_index, offsets, _ = _problem([9, 30, 4], 1024, 256, seed=9)
    tp = plan_from_offsets(offsets, 64, x.device)
    runs = [gate_up_swiglu(x, w13, tp, row_index=row_index[: offsets[-1]], split=split).clone() for _ in range(5)]
    torch.cuda.synchronize()
    for r in runs[1:]:
        assert torch.equal(r.view(torch.int16), runs[0].view(torch.int16))


@pytest.mark.slow
def test_glm_shape_one_expert_tile():
    from moeflow_b200.ops.grouped_gemm import down_proj, gate_up_swiglu, plan_from_offsets

    w13, w2, x, row_index, offsets, scale = _problem([7, 0, 21], 4096, 1536, seed=2)
    n = offsets[-1]
    tp = plan_from_offsets(offsets, 64, x.device)
    status = torch.zeros(1, dtype=torch.int64, device=x.device)
    act = gate_up_swiglu(x, w13, tp, row_index=row_index[:n], status=status, split=2)
    y = down_proj(act, w2, tp, row_scale=scale[:n], status=status, split=2)
    torch.cuda.synchronize()
    _status_ok(status)
    ref_act = _ref_gate_up(x, row_index[:n], w13, offsets, 10.0)
    assert normwise_rel_err(act, ref_act) < 4 * 2.0**-8
    assert normwise_rel_err(y, _ref_down(act, w2, offsets, scale[:n])) < 4 * 2.0**-8


@pytest.mark.parametrize("weighted", [False, True])
def test_expert_compute_backend_matches_the_torch_loop(weighted):
    """The ExpertCompute adapter of the variable-size pipeline: same call, tcgen05 kernels inside."""
    from moeflow_b200.experts import EXPERT_BACKENDS

    w13, w2, x, _, offsets, scale = _problem([5, 0, 70, 17], 512, 256, seed=11)
    n = offsets[-1]
    a = x[:n].contiguous() if x.shape[0] >= n else x
    offs = torch.tensor(offsets, dtype=torch.int64, device=x.device)
    rw = scale[:n] if weighted else None
    got = EXPERT_BACKENDS["tcgen05_grouped"]()(a, offs, w13, w2, 10.0, rw)
    ref = EXPERT_BACKENDS["torch_loop"]()(a.float(), offs, w13.float(), w2.float(), 10.0, rw)
    torch.cuda.synchronize()
    assert got.shape == a.shape and got.dtype == a.dtype
    assert normwise_rel_err(got, ref) < 6 * 2.0**-8, normwise_rel_err(got, ref)


@pytest.mark.parametrize("counts,block_m,split", [([3, 0, 17, 5], 64, 1), ([70, 2, 130], 64, 2), ([100, 20], 128, 1), ([5, 9], 32, 4)])
def test_down_proj_token_tiles_by_tma_equal_the_gather_bitwise(counts, block_m, split):
    """The token operand of the down GEMM fetched by TMA (box of block_m rows) or gathered by cp.async."""
    from moeflow_b200.ops.grouped_gemm import down_proj, plan_from_offsets

    _, w2, _, _, offsets, scale = _problem(counts, 512, 256, seed=21)
    n = offsets[-1]
    g = torch.Generator().manual_seed(3)
    act = torch.randn(n, 256, generator=g).bfloat16().cuda()
    tp = plan_from_offsets(offsets, block_m, act.device)
    status = torch.zeros(1, dtype=torch.int64, device=act.device)
    a = down_proj(act, w2, tp, row_scale=scale[:n], split=split, status=status, wait_ns=50_000_000, b_tma=True).clone()
    b = down_proj(act, w2, tp, row_scale=scale[:n], split=split, status=status, wait_ns=50_000_000, b_tma=False).clone()
    torch.cuda.synchronize()
    _status_ok(status)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert normwise_rel_err(a, _ref_down(act, w2, offsets, scale[:n])) < 4 * 2.0**-8


@pytest.mark.parametrize("counts,hidden,inter,block_m,split", [([3, 0, 17, 5], 512, 256, 64, 1), ([70, 2, 130], 512, 128, 64, 2),
                                                          ([128], 256, 128, 128, 1), ([300, 5, 129], 512, 256, 128, 1),
                                                          ([127, 131, 3, 128], 256, 128, 128, 1), ([5, 9], 512, 256, 32, 4),
                                                          ([256, 700, 1], 512, 256, 256, 1), ([256], 256, 128, 256, 2)])
def test_gate_up_token_tiles_by_tma_equal_the_gather_bitwise_and_the_oracle(counts, hidden, inter, block_m, split):
    """Gate/up GEMM with its token tiles fetched by TMA (contiguous rows) or gathered by cp.async: same bits,
    and both within tolerance of fp32 PyTorch.  Includes full 128-row tiles."""
    from moeflow_b200.ops.grouped_gemm import gate_up_swiglu, plan_from_offsets

    w13, _, x, _, offsets, _ = _problem(counts, hidden, inter, seed=31)
    n = offsets[-1]
    x = x[:n].contiguous()
    tp = plan_from_offsets(offsets, block_m, x.device)
    status = torch.zeros(1, dtype=torch.int64, device=x.device)
    ident = torch.arange(n, dtype=torch.int32, device=x.device)
    a = gate_up_swiglu(x, w13, tp, limit=10.0, split=split, status=status, wait_ns=50_000_000, b_tma=True).clone()
    b = gate_up_swiglu(x, w13, tp, row_index=ident, limit=10.0, split=split, status=status, wait_ns=50_000_000).clone()
    torch.cuda.synchronize()
    _status_ok(status)
    ref = _ref_gate_up(x, ident, w13, offsets, 10.0)
    assert normwise_rel_err(b, ref) < 4 * 2.0**-8, "gather"
    assert normwise_rel_err(a, ref) < 4 * 2.0**-8, "tma"
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("grid", [1, 3, 7, 50, 148, 149, 300])
@pytest.mark.parametrize("counts,hidden,inter,block_m", [([16, 64, 1, 0, 33], 1024, 384, 64), ([130], 512, 256, 128)])
def test_stream_k_cut_for_any_number_of_ctas(grid, counts, hidden, inter, block_m):
    """Stream-K with fewer CTAs than units, more CTAs than K steps, and shares that start or end exactly on
    a unit boundary: same result (within tolerance of fp32 PyTorch) for every grid size."""
    from moeflow_b200.ops.grouped_gemm import down_proj, gate_up_swiglu, plan_from_offsets

    w13, w2, x, row_index, offsets, scale = _problem(counts, hidden, inter, seed=77)
    n = offsets[-1]
    tp = plan_from_offsets(offsets, block_m, x.device)
    status = torch.zeros(1, dtype=torch.int64, device=x.device)
    act = gate_up_swiglu(x, w13, tp, row_index=row_index[:n], split=0, status=status, wait_ns=50_000_000, grid=grid)
    y = down_proj(act, w2, tp, row_scale=scale[:n], split=0, status=status, wait_ns=50_000_000, grid=grid)
    torch.cuda.synchronize()
    _status_ok(status)
    assert normwise_rel_err(act, _ref_gate_up(x, row_index[:n], w13, offsets, 10.0)) < 4 * 2.0**-8
    assert normwise_rel_err(y, _ref_down(act, w2, offsets, scale[:n])) < 4 * 2.0**-8


def test_a_plan_that_does_not_fit_the_scratch_is_refused_on_the_device():
    """The plan words live in device memory; the kernel compares them with the capacities in its arguments and
    reports 'bad argument' without storing anything when they do not fit."""
    from moeflow_b200.ops._lib import decode_status
    from moeflow_b200.ops.grouped_gemm import down_proj, plan_from_offsets

    _, w2, _, _, offsets, scale = _problem([40, 9], 512, 256, seed=3)
    n = offsets[-1]
    act = torch.randn(n, 256).bfloat16().cuda()
    tp = plan_from_offsets(offsets, 64, act.device)
    status = torch.zeros(1, dtype=torch.int64, device=act.device)
    tp.plan[0] = 1000  # claims far more tiles than the tile arrays and counters hold
    y = down_proj(act, w2, tp, row_scale=scale[:n], split=2, status=status, wait_ns=50_000_000)
    torch.cuda.synchronize()
    st = decode_status(int(status.item()))
    assert st["code"] == 7, st
    assert float(y.float().abs().sum()) == 0.0


@pytest.mark.parametrize("counts,hidden,inter,block_m,split", [([3, 0, 17, 5], 512, 256, 64, 1), ([70, 2, 130], 512, 128, 64, 2),
                                                          ([128], 256, 128, 128, 1), ([256, 700, 1], 512, 256, 256, 1),
                                                          ([300, 5, 600], 1024, 384, 256, 0)])
def test_down_proj_over_two_weight_blocks_per_unit_equals_one_block_bitwise(counts, hidden, inter, block_m, split):
    """``two_blocks``: a unit covers two adjacent 128-row weight blocks (two accumulators, the token tile fetched
    once); every output element is the same dot product, so the bits equal the one-block kernel's."""
    from moeflow_b200.ops.grouped_gemm import down_proj, plan_from_offsets

    _, w2, _, _, offsets, scale = _problem(counts, hidden, inter, seed=41)
    n = offsets[-1]
    act = torch.randn(n, inter, generator=torch.Generator().manual_seed(4)).bfloat16().cuda()
    tp = plan_from_offsets(offsets, block_m, act.device)
    status = torch.zeros(1, dtype=torch.int64, device=act.device)
    one = down_proj(act, w2, tp, row_scale=scale[:n], split=split, status=status, wait_ns=50_000_000).clone()
    two = down_proj(act, w2, tp, row_scale=scale[:n], split=split, status=status, wait_ns=50_000_000, two_blocks=True).clone()
    torch.cuda.synchronize()
    _status_ok(status)
    assert normwise_rel_err(two, _ref_down(act, w2, offsets, scale[:n])) < 4 * 2.0**-8
    if split != 0:  # stream-K cuts units at different K positions in the two forms: equal values, other rounding
        assert torch.equal(one.view(torch.int16), two.view(torch.int16))
