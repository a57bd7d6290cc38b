"""The pencil-and-paper example: each stage's result against numbers derived by hand, and the end result
against the closed form computed from the scenario table alone."""

import pytest
import torch

from moeflow_b200 import hand_example as hx

# Derivation.  Experts 0, 1 live on rank 0 and 2, 3 on rank 1; expert g multiplies by g + 1.
# rank 0 sends a and b to itself and b, c to rank 1; rank 1 sends d to both ranks.
WORKED = {
    # rows per destination, and which local token each row carries
    "send_counts": [[2, 2], [1, 1]],
    "send_token": [[0, 1, 1, 2], [0, 0]],
    # local expert ids per slot as seen by the destination (-1: slot lives elsewhere)
    "send_slots": [[[0, 1], [1, -1], [-1, 1], [0, 1]], [[-1, 0], [1, -1]]],
    "recv_counts": [[2, 1], [2, 1]],
    "recv_slots": [[[0, 1], [1, -1], [-1, 0]], [[-1, 1], [0, 1], [1, -1]]],
    "recv_weights": [[[1.5, 1.0], [2.0, 0.0], [0.0, 0.5]], [[0.0, 0.5], [1.25, 1.25], [2.0, 0.0]]],
    # expert-major layout: offsets, then (row, slot) of every entry in stable order
    "expert_offsets": [[0, 2, 4], [0, 1, 4]],
    "expert_entries": [[(0, 0), (2, 1), (0, 1), (1, 0)], [(1, 0), (0, 1), (1, 1), (2, 0)]],
    # rank 0: a -> (1.5*1 + 1.0*2) a = 3.5 a;  b -> 2.0*2 b = 4 b;  d -> 0.5*1 d
    # rank 1: b -> 0.5*4 b = 2 b;  c -> (1.25*3 + 1.25*4) c = 8.75 c;  d -> 2.0*4 d = 8 d
    "partials": [[[3.5, 7.0], [12.0, -4.0], [0.25, 2.0]], [[6.0, -2.0], [17.5, 4.375], [4.0, 32.0]]],
    "returned": [[[3.5, 7.0], [12.0, -4.0], [6.0, -2.0], [17.5, 4.375]], [[0.25, 2.0], [4.0, 32.0]]],
    # a = 3.5 a;  b = 4 b + 2 b;  c = 8.75 c;  d = 0.5 d + 8 d
    "out": [[[3.5, 7.0], [18.0, -6.0], [17.5, 4.375]], [[4.25, 34.0]]],
}


@pytest.fixture(scope="module")
def record():
    return hx.run()


@pytest.mark.parametrize("stage", sorted(WORKED))
def test_stage_matches_the_hand_derivation(record, stage):
    got = record[stage]
    if stage == "expert_entries":
        got = [[tuple(e) for e in rank] for rank in got]
    assert got == WORKED[stage]


def test_received_rows_are_the_senders_tokens(record):
    # rank 0 receives a, b (from itself) and d; rank 1 receives b, c and d
    assert record["recv_x"] == [[[1.0, 2.0], [3.0, -1.0], [0.5, 4.0]], [[3.0, -1.0], [2.0, 0.5], [0.5, 4.0]]]


def test_closed_form_agrees_with_the_pipeline(record):
    assert hx.expected_outputs() == WORKED["out"] == record["out"]


def test_scenario_views_keep_their_shapes():
    assert [tuple(x.shape) for x in hx.X] == [(3, 2), (1, 2)]
    assert all(i.dtype == torch.int32 and i.shape[1] == hx.CFG.top_k for i in hx.TOPK_IDS)
    assert torch.equal(hx.TOPK_W[1], torch.tensor([[2.0, 0.5]]))


def test_fp32_run_gives_the_same_numbers():
    assert hx.run(torch.float32)["out"] == WORKED["out"]
