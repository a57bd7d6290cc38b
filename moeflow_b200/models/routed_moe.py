"""Serving-side wrapper of one routed MoE layer: static buffers + one CUDA graph.

``GraphedMoELayer`` is the call a user makes on the hot path.  It owns device-side input buffers of
the layer's capacity, captures ``FixedEPLayer.forward`` once, and then every call is: copy this step's
hidden states and router logits in (host pinned memory or device tensors), replay the graph, and
hand back the output rows.  Nothing is allocated and nothing is read back to the host by the layer
itself, so the call can sit inside a larger captured decode step as well.

Two ways to feed it:

* ``layer(x, logits, out)``: two tensors (pinned host or device), two copies and a fill of the row count.
* ``layer.step(block, out)``: ``block = layer.new_pinned_inputs()`` is one pinned host block laid out exactly
  like the device-side input block — hidden rows, logits, row count — which the caller fills in place
  (``block.x``, ``block.logits``, ``block.set_rows(t)``).  A step is then a single host-to-device copy, the
  replay, and one device-to-host copy of the output rows: three stream operations instead of five.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..fixed import FixedEPLayer


class PinnedInputs:
    """One step's inputs in pinned host memory, in the layout of the layer's device input block."""

    def __init__(self, raw: torch.Tensor, x: torch.Tensor, logits: torch.Tensor, rows: torch.Tensor):
        self.raw, self.x, self.logits, self._rows = raw, x, logits, rows
        self.rows = 0

    def set_rows(self, t: int) -> None:
        self.rows = int(t)
        self._rows.fill_(int(t))


class GraphedMoELayer:
    def __init__(self, layer: FixedEPLayer, bias: torch.Tensor | None, warmup: int = 2):
        self.layer, self.bias = layer, bias
        cfg, dev = layer.cfg, layer.device
        # one block: [C, H] activations | [C, E] fp32 logits | int32 row count (16-byte aligned sections)
        itemsize = torch.empty((), dtype=layer.dtype).element_size()
        self._x_bytes = layer.C * cfg.hidden_size * itemsize
        self._lg_off = (self._x_bytes + 15) // 16 * 16
        self._lg_bytes = layer.C * cfg.n_routed_experts * 4
        self._nv_off = (self._lg_off + self._lg_bytes + 15) // 16 * 16
        self.packed_bytes = self._nv_off + 16
        self._block = torch.zeros(self.packed_bytes, dtype=torch.uint8, device=dev)
        self.x, self.logits, self.num_valid = self._views(self._block)
        self.num_valid.fill_(layer.C)
        self.graph: torch.cuda.CUDAGraph | None = None
        self._warmup = warmup
        # route+dispatch, meta (two launches in its multi-CTA form), gate/up, down(+reduce+push), combine
        self.kernels_per_step = (5 if getattr(layer, "fuse_return", False) else 6) + (
            1 if getattr(layer, "meta_ctas", 1) > 1 else 0) + (1 if getattr(layer, "permute_rows", False) else 0)

    def _views(self, block: torch.Tensor):
        cfg, C = self.layer.cfg, self.layer.C
        x = block[: self._x_bytes].view(self.layer.dtype).view(C, cfg.hidden_size)
        logits = block[self._lg_off : self._lg_off + self._lg_bytes].view(torch.float32).view(C, cfg.n_routed_experts)
        rows = block[self._nv_off : self._nv_off + 4].view(torch.int32).view(())
        return x, logits, rows

    def new_pinned_inputs(self) -> PinnedInputs:
        """A pinned host block for one step's inputs (fill ``.x[:t]``, ``.logits[:t]``, then ``set_rows(t)``)."""
        raw = torch.zeros(self.packed_bytes, dtype=torch.uint8).pin_memory()
        x, logits, rows = self._views(raw)
        return PinnedInputs(raw, x, logits, rows)

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

    def step(self, inputs: PinnedInputs, out: torch.Tensor | None = None) -> torch.Tensor:
        """One step from a pinned input block: one host-to-device copy, the replay, one copy of the rows out."""
        if inputs.rows > self.layer.C:
            raise ValueError(f"{inputs.rows} tokens exceed capacity {self.layer.C}")
        self._block.copy_(inputs.raw, non_blocking=True)
        res = self.replay()[: inputs.rows]
        if out is not None:
            out[: inputs.rows].copy_(res, non_blocking=True)
            return out
        return res

    def close(self) -> None:
        """Drop the graph (do this before destroying the process group)."""
        self.graph = None
