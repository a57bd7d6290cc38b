"""Simulated row exchange: ordering contract."""

import torch

from moeflow_b200.comm import simulated_exchange


def test_rows_arrive_grouped_by_source_in_send_order():
    sends = [torch.tensor([[0.0], [1.0], [2.0]]), torch.tensor([[10.0], [11.0]])]
    counts = [torch.tensor([1, 2]), torch.tensor([2, 0])]
    recvs, recv_counts = simulated_exchange(sends, counts)
    assert recvs[0].flatten().tolist() == [0.0, 10.0, 11.0]
    assert recvs[1].flatten().tolist() == [1.0, 2.0]
    assert [c.tolist() for c in recv_counts] == [[1, 2], [2, 0]]


def test_empty_ranks():
    sends = [torch.empty(0, 3), torch.ones(2, 3)]
    counts = [torch.tensor([0, 0]), torch.tensor([1, 1])]
    recvs, _ = simulated_exchange(sends, counts)
    assert recvs[0].shape == (1, 3) and recvs[1].shape == (1, 3)
