"""Byte-level comparison and the GEMM acceptance threshold."""

import pytest
import torch

from moeflow_b200.tolerances import BF16_U, bitwise_equal, calc_diff, gemm_tolerance, normwise_rel_err


def test_signed_zero_is_a_difference():
    assert not bitwise_equal(torch.tensor([0.0]), torch.tensor([-0.0]))
    assert bitwise_equal(torch.tensor([-0.0]), torch.tensor([-0.0]))


def test_nan_payloads_compare_as_bytes():
    a = torch.tensor([float("nan")])
    assert bitwise_equal(a, a.clone())


def test_dtype_shape_mismatch():
    assert not bitwise_equal(torch.ones(2), torch.ones(2, dtype=torch.bfloat16))
    assert not bitwise_equal(torch.ones(2), torch.ones(1, 2))


@pytest.mark.parametrize("value", [torch.tensor(1.0), torch.empty(0, 2), torch.arange(6).reshape(2, 3).t()])
def test_scalars_empty_and_strided(value):
    assert bitwise_equal(value, value.contiguous().clone())


def test_thresholds():
    assert gemm_tolerance() == 4 * BF16_U
    assert gemm_tolerance(0.1) == 0.2
    assert gemm_tolerance(1e-5) == 4 * BF16_U
    ref = torch.tensor([3.0, 4.0])
    assert normwise_rel_err(ref, ref) == 0.0
    assert abs(normwise_rel_err(torch.tensor([3.0, 4.5]), ref) - 0.1) < 1e-12
    assert normwise_rel_err(torch.tensor([1.0]), torch.tensor([0.0])) == 1.0
    assert calc_diff(ref, ref) == 0.0


def test_first_difference_points_at_the_first_differing_element():
    from moeflow_b200.tolerances import first_difference

    a = torch.tensor([1.0, 0.0, 3.0, 4.0])
    assert first_difference(a, a.clone()) is None
    b = a.clone()
    b[1], b[3] = -0.0, 5.0
    where = first_difference(a, b)
    assert where["index"] == 1 and where["count"] == 2 and where["b"] == 0.0
    assert "reason" in first_difference(a, a.to(torch.bfloat16))
    assert first_difference(torch.empty(0), torch.empty(0)) is None
