"""Row transports of the variable-size pipeline.

Contract of one exchange (the same for every transport): the sender's rows are grouped by destination rank
in ascending order, ``send_counts[d]`` of them are for rank d; the receiver gets the rows grouped by source
rank in ascending order, every source's rows in the order it sent them, ``recv_counts[s]`` rows from rank s.

``CollectiveRowExchange``  over ``torch.distributed``: one all-to-all where the backend has it (NCCL), pairwise
                           sends and receives where it does not (gloo).  The split sizes have to be known on the
                           host, so every exchange copies the counts back: this path cannot be captured in a
                           CUDA graph, which is why it is the baseline and not the product path.
``simulated_exchange``     all ranks of a single-process simulation at once (tests, hand example).
``pack_meta``              the per-slot metadata (local expert ids, routing weights) as one int32 block, so
                           that it travels in a single exchange next to the hidden rows.

Behavioural counterpart of ``moeflow/comm.py:17-65`` of the reference; ``NcclRowExchange`` is its name for the
collective transport.
"""

from __future__ import annotations

from typing import Protocol, Sequence

import torch
import torch.distributed as dist


class RowExchange(Protocol):
    rank: int
    world: int

    def exchange_counts(self, send_counts: torch.Tensor) -> torch.Tensor: ...

    def exchange(self, send: torch.Tensor, send_counts: torch.Tensor, recv_counts: torch.Tensor) -> torch.Tensor: ...


def _host_sizes(counts: torch.Tensor) -> list[int]:
    return [int(c) for c in counts.tolist()]  # device-to-host copy: inherent in a variable-size exchange


class CollectiveRowExchange:
    def __init__(self, group: dist.ProcessGroup | None = None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        # None: not known yet; decided by the first exchange and remembered
        self._has_all_to_all: bool | None = None

    # ---- the two ways to move the pieces --------------------------------------------------------------
    def _pairwise(self, outgoing: Sequence[torch.Tensor], incoming: Sequence[torch.Tensor]) -> None:
        """Every rank posts all its sends and receives, then waits; the own piece is a local copy."""
        incoming[self.rank].copy_(outgoing[self.rank])
        absolute = (lambda r: dist.get_global_rank(self.group, r)) if self.group is not None else (lambda r: r)
        posted = []
        for peer in range(self.world):
            if peer != self.rank:
                posted.append(dist.isend(outgoing[peer].contiguous(), absolute(peer), group=self.group))
                posted.append(dist.irecv(incoming[peer], absolute(peer), group=self.group))
        for request in posted:
            request.wait()

    def _move(self, src: torch.Tensor, dst: torch.Tensor, src_sizes: list[int] | None, dst_sizes: list[int] | None) -> None:
        if self._has_all_to_all is not False:
            try:
                dist.all_to_all_single(dst, src, dst_sizes, src_sizes, group=self.group)
                self._has_all_to_all = True
                return
            except RuntimeError as problem:
                if self._has_all_to_all or "does not support" not in str(problem):
                    raise
                self._has_all_to_all = False
        even = lambda t: list(t.chunk(self.world))  # noqa: E731 - counts are exchanged as world equal pieces
        self._pairwise(even(src) if src_sizes is None else list(src.split(src_sizes)),
                       even(dst) if dst_sizes is None else list(dst.split(dst_sizes)))

    # ---- RowExchange -----------------------------------------------------------------------------------
    def exchange_counts(self, send_counts: torch.Tensor) -> torch.Tensor:
        arriving = torch.empty_like(send_counts)
        self._move(send_counts.contiguous(), arriving, None, None)
        return arriving

    def exchange(self, send: torch.Tensor, send_counts: torch.Tensor, recv_counts: torch.Tensor) -> torch.Tensor:
        leaving, arriving = _host_sizes(send_counts), _host_sizes(recv_counts)
        received = send.new_empty((sum(arriving), *send.shape[1:]))
        self._move(send.contiguous(), received, leaving, arriving)
        return received


NcclRowExchange = CollectiveRowExchange


def simulated_exchange(sends: list[torch.Tensor], send_counts: list[torch.Tensor]) -> tuple[list[torch.Tensor], list[torch.Tensor]]:
    """One exchange for all ranks held in this process: ``(received rows per rank, recv_counts per rank)``."""
    world = len(sends)
    counts = torch.stack([c.reshape(world) for c in send_counts])  # [src, dst]
    starts = counts.cumsum(dim=1) - counts                          # first row of each destination's piece
    received = []
    for dst in range(world):
        pieces = [sends[src].narrow(0, int(starts[src, dst]), int(counts[src, dst])) for src in range(world)]
        received.append(torch.cat(pieces, dim=0))
    return received, [counts[:, dst].clone() for dst in range(world)]


def pack_meta(local_id: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``[S, K]`` local expert ids and ``[S, K]`` fp32 weights -> ``[S, 2K]`` int32 (weight bits unchanged)."""
    rows, top_k = local_id.shape
    block = torch.empty(rows, 2 * top_k, dtype=torch.int32, device=local_id.device)
    block[:, :top_k] = local_id
    block[:, top_k:] = weight.to(torch.float32).contiguous().view(torch.int32)
    return block


def unpack_meta(meta: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    ids, weight_bits = meta.tensor_split(2, dim=1)
    return ids.contiguous(), weight_bits.contiguous().view(torch.float32)
