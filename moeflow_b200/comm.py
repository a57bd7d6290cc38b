"""Row-exchange transports of the variable-size pipeline.

``exchange(send, send_counts, recv_counts)``: ``send`` rows are grouped by destination rank in
ascending order, ``send_counts[d]`` rows go to rank d; the receiver gets the rows grouped by source
rank in ascending order, each source's rows in the order they were sent.

``CollectiveRowExchange`` runs over any ``torch.distributed`` backend (NCCL on GPUs, gloo on CPU) and
copies the counts to the host to size the variable split, which is why this path cannot be captured
in a CUDA graph.  ``simulated_exchange`` does the same exchange for all ranks inside one process.
Behavioural counterpart of the reference's ``moeflow/comm.py:17-65``.
"""

from __future__ import annotations

from typing import Protocol

import torch
import torch.distributed as dist


class RowExchange(Protocol):
    rank: int
    world: int

    def exchange_counts(self, send_counts: torch.Tensor) -> torch.Tensor: ...

    def exchange(self, send: torch.Tensor, send_counts: torch.Tensor, recv_counts: torch.Tensor) -> torch.Tensor: ...


class CollectiveRowExchange:
    """Variable-split all-to-all through ``torch.distributed`` (host round trip for the counts)."""

    def __init__(self, group: dist.ProcessGroup | None = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def _a2a(self, out, inp, out_splits=None, in_splits=None):
        try:
            dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)
            return
        except RuntimeError as exc:
            if "does not support" not in str(exc):
                raise
        # Backend without an all-to-all: pairwise sends and receives.
        ins = list(inp.split(in_splits)) if in_splits is not None else list(inp.chunk(self.world))
        outs = list(out.split(out_splits)) if out_splits is not None else list(out.chunk(self.world))
        outs[self.rank].copy_(ins[self.rank])
        peers = [p for p in range(self.world) if p != self.rank]
        to_global = (lambda p: dist.get_global_rank(self.group, p)) if self.group is not None else (lambda p: p)
        pending = [dist.isend(ins[p].contiguous(), to_global(p), group=self.group) for p in peers]
        pending += [dist.irecv(outs[p], to_global(p), group=self.group) for p in peers]
        for req in pending:
            req.wait()

    def exchange_counts(self, send_counts: torch.Tensor) -> torch.Tensor:
        recv_counts = torch.empty_like(send_counts)
        self._a2a(recv_counts, send_counts.contiguous())
        return recv_counts

    def exchange(self, send, send_counts, recv_counts):
        in_splits = [int(v) for v in send_counts.tolist()]  # device-to-host sync, by design
        out_splits = [int(v) for v in recv_counts.tolist()]
        recv = send.new_empty((sum(out_splits), *send.shape[1:]))
        self._a2a(recv, send.contiguous(), out_splits, in_splits)
        return recv


# Name used by the reference for the NCCL-backed transport.
NcclRowExchange = CollectiveRowExchange


def simulated_exchange(
    sends: list[torch.Tensor], send_counts: list[torch.Tensor]
) -> tuple[list[torch.Tensor], list[torch.Tensor]]:
    """One collective for all ranks of a single-process simulation."""
    world = len(sends)
    pieces = [list(s.split([int(v) for v in c.tolist()], dim=0)) for s, c in zip(sends, send_counts)]
    recvs, recv_counts = [], []
    for dst in range(world):
        recvs.append(torch.cat([pieces[src][dst] for src in range(world)], dim=0))
        recv_counts.append(torch.stack([send_counts[src][dst] for src in range(world)]))
    return recvs, recv_counts


def pack_meta(local_id: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``[S, K] int32`` ids and ``[S, K] fp32`` weights -> ``[S, 2K] int32`` (weights bit-cast)."""
    return torch.cat([local_id.to(torch.int32), weight.to(torch.float32).contiguous().view(torch.int32)], dim=1)


def unpack_meta(meta: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    top_k = meta.shape[1] // 2
    return meta[:, :top_k].contiguous(), meta[:, top_k:].contiguous().view(torch.float32)
