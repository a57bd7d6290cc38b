"""Host-side planning rules: tile rows, metadata CTAs, and the K-split rule shared with the metadata kernels."""

import shutil

import pytest

from moeflow_b200.fixed import choose_block_m, choose_meta_ctas


def test_tile_rows_follow_the_expected_rows_per_expert_not_the_worst_case():
    assert choose_block_m(128, 8, 288) == 64     # EP=1 decode: 3.5 rows per expert
    assert choose_block_m(128, 8, 36) == 64      # EP=8, T=128: 28 rows per expert (worst case would be 227)
    assert choose_block_m(256, 8, 36) == 128     # 57 rows per expert: one tile per expert instead of two for some
    assert choose_block_m(512, 8, 72) == 128     # 57 rows
    assert choose_block_m(512, 8, 144) == 64     # 28 rows
    assert choose_block_m(2048, 8, 144) == 256   # EP=2 prefill: 114 rows per expert
    assert choose_block_m(8192, 8, 36) == 256    # EP=8 long prefill: 1820 rows per expert
    assert choose_block_m(1, 8, 1) == 64


def test_tile_rows_for_layers_that_will_hold_e4m3_experts():
    assert choose_block_m(256, 8, 36, fp8=True) == 64      # 57 rows
    assert choose_block_m(2048, 8, 144, fp8=True) == 128   # 114 rows: the e4m3 kernels, no expansion
    assert choose_block_m(8192, 8, 144, fp8=True) == 128   # 455 rows
    assert choose_block_m(8192, 8, 36, fp8=True) == 256    # 1820 rows: expanded to bf16 per forward


def test_metadata_ctas_by_size():
    assert choose_meta_ctas(8, 148) == 1
    assert choose_meta_ctas(2048, 148) == 1
    assert choose_meta_ctas(8192, 148) == 1       # EP=8, 128 tokens per rank, top-8: still the one-pass single CTA
    assert choose_meta_ctas(8193, 148) == 65
    assert choose_meta_ctas(16384, 148) == 128
    assert choose_meta_ctas(1 << 20, 148) == 148
    assert choose_meta_ctas(16384, 8) == 8


@pytest.fixture(scope="module")
def plan_split():
    from moeflow_b200.ops import _lib

    if not _lib.LIB_PATH.exists() and shutil.which("nvcc") is None:
        pytest.skip("native library not built and no nvcc")
    return _lib.lib().mf_plan_split


def test_wide_tiles_are_not_split_for_an_uneven_last_round(plan_split):
    # EP=8, T=128: 40 token tiles x 12 blocks = 480 units of 64-column tiles, just over three rounds of 148 CTAs;
    # splitting K in two there doubled the gate/up GEMM's time
    assert plan_split(480, 64, 148, 1024, 4, 64) == 1
    assert plan_split(432, 64, 148, 1024, 4, 64) == 1
    assert plan_split(40 * 32, 24, 148, 2048, 8, 64) == 1


def test_decode_sizes_split_k_to_fill_the_sms(plan_split):
    assert plan_split(8 * 12, 64, 148, 4096, 4, 16) >= 2      # T=1: 8 experts x 12 blocks on 148 SMs
    assert plan_split(1 * 12, 64, 148, 4096, 4, 16) == 8
    assert plan_split(0, 64, 148, 4096, 4, 16) == 1
    assert plan_split(8 * 12, 64, 148, 100, 4, 16) == 1        # not enough partial-sum slots for any split


@pytest.mark.parametrize("units", [1, 7, 96, 148, 149, 480, 2640])
@pytest.mark.parametrize("k_blocks", [24, 64, 6])
@pytest.mark.parametrize("cols", [16, 64, 128])
def test_split_always_divides_k_and_fits_the_slots(plan_split, units, k_blocks, cols):
    s = plan_split(units, k_blocks, 148, 1024, 4, cols)
    assert s in (1, 2, 4, 8) and k_blocks % s == 0 and (s == 1 or (k_blocks // s >= 2 and units * s <= 1024))
