"""Serving-side wrapper of one routed MoE layer: static buffers + one CUDA graph.

``GraphedMoELayer`` is the call a user makes on the hot path.  It owns device-side input buffers of
the layer's capacity, captures ``FixedEPLayer.forward`` once, and then every call is: copy this step's
hidden states and router logits in (host pinned memory or device tensors), replay the graph, and
hand back the output rows.  Nothing is allocated and nothing is read back to the host by the layer
itself, so the call can sit inside a larger captured decode step as well.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..fixed import FixedEPLayer


class GraphedMoELayer:
    def __init__(self, layer: FixedEPLayer, bias: torch.Tensor | None, warmup: int = 2):
        self.layer, self.bias = layer, bias
        cfg, dev = layer.cfg, layer.device
        self.x = torch.zeros(layer.C, cfg.hidden_size, dtype=layer.dtype, device=dev)
        self.logits = torch.zeros(layer.C, cfg.n_routed_experts, dtype=torch.float32, device=dev)
        self.num_valid = torch.full((), layer.C, dtype=torch.int32, device=dev)
        self.graph: torch.cuda.CUDAGraph | None = None
        self._warmup = warmup
        # route+dispatch, meta (two launches in its multi-CTA form), gate/up, down(+reduce+push), combine
        self.kernels_per_step = (5 if getattr(layer, "fuse_return", False) else 6) + (
            1 if getattr(layer, "meta_ctas", 1) > 1 else 0) + (1 if getattr(layer, "permute_rows", False) else 0)

    def _forward(self) -> torch.Tensor:
        return self.layer.forward(self.x, self.logits, self.bias, self.num_valid)

    def capture(self) -> "GraphedMoELayer":
        """Warm up on a side stream, then capture one forward.  Every rank must call this together."""
        side = torch.cuda.Stream(device=self.layer.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self._warmup):
                self._forward()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if dist.is_available() and dist.is_initialized():
            dist.barrier(group=self.layer.group)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.out = self._forward()
        self.graph = graph
        torch.cuda.synchronize()
        return self

    def load(self, x: torch.Tensor, logits: torch.Tensor) -> int:
        """Copy one step's inputs (``[T, H]``, ``[T, E]``; host-pinned or device) into the static buffers."""
        t = x.shape[0]
        if t > self.layer.C:
            raise ValueError(f"{t} tokens exceed capacity {self.layer.C}")
        self.x[:t].copy_(x, non_blocking=True)
        self.logits[:t].copy_(logits, non_blocking=True)
        self.num_valid.fill_(t)
        return t

    def replay(self) -> torch.Tensor:
        if self.graph is None:
            self.capture()
        self.graph.replay()
        return self.out

    def __call__(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """One step.  With ``out`` (e.g. a pinned host tensor ``[T, H]``) the rows are copied there."""
        t = self.load(x, logits)
        res = self.replay()[:t]
        if out is not None:
            out.copy_(res, non_blocking=True)
            return out
        return res

    def close(self) -> None:
        """Drop the graph (do this before destroying the process group)."""
        self.graph = None
