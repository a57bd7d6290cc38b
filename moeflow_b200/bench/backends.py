"""Benchmark backends: every class exposes ``run(x, logits) -> out [T, H]`` for one EP rank.

``init_dist`` sets up ``torch.distributed`` with NCCL for device tensors and gloo for Python objects.
``FusedFixedBackend`` is the product path (cuda backend, peer-memory transport); ``TorchFixedBackend`` is
its PyTorch/NCCL twin; ``NaiveBackend`` is the variable-size pipeline with a host round trip.
``ReferenceFixedBackend`` drives the reference's own ``FixedEPLayer`` when it is installed under
``baseline/_ref``.  Counterpart of ``scripts/bench/backends.py:33-325`` (the vLLM-backed arms of that file
need vLLM's modular-kernel objects and live in ``moeflow_b200.integrations``).
"""

from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.distributed as dist

from ..comm import CollectiveRowExchange
from ..config import MoEConfig
from ..ep_moe import EPMoELayer
from ..fixed import FixedEPLayer

BACKENDS = ("fused", "torch_fixed", "naive", "naive_tcgen05", "fixed_vllm_experts", "vllm_agrs", "reference_fixed")


@dataclass
class DistInfo:
    rank: int
    world: int
    local_rank: int
    device: torch.device


def init_dist(timeout_s: int = 600) -> DistInfo:
    """One process per GPU; rendezvous on 127.0.0.1 unless the launcher says otherwise."""
    from datetime import timedelta

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        kw = {"device_id": device} if cuda else {}
        dist.init_process_group("cpu:gloo,cuda:nccl" if cuda else "gloo", rank=rank, world_size=world,
                                timeout=timedelta(seconds=timeout_s), **kw)
    return DistInfo(rank, world, local, device)


class FusedFixedBackend:
    name = "fused"

    def __init__(self, cfg: MoEConfig, info: DistInfo, w13_local, w2_local, bias, capacity: int, **layer_kw):
        self.layer = FixedEPLayer(cfg, info.rank, info.world, w13_local, w2_local, capacity=capacity, backend="cuda",
                                  **layer_kw)
        self.bias = bias

    def run(self, x, logits):
        return self.layer.forward(x, logits, self.bias)[: x.shape[0]]


class TorchFixedBackend:
    name = "torch_fixed"

    def __init__(self, cfg, info, w13_local, w2_local, bias, capacity, **layer_kw):
        self.layer = FixedEPLayer(cfg, info.rank, info.world, w13_local, w2_local, capacity=capacity, backend="torch",
                                  **layer_kw)
        self.bias = bias

    def run(self, x, logits):
        return self.layer.forward(x, logits, self.bias)[: x.shape[0]]


class NaiveBackend:
    name = "naive"

    def __init__(self, cfg, info, w13_local, w2_local, bias, capacity=None, **_):
        self.layer = EPMoELayer(cfg, info.rank, info.world, w13_local, w2_local)
        self.comm = CollectiveRowExchange()
        self.bias = bias

    def run(self, x, logits):
        return self.layer.forward(x, logits, self.bias, self.comm)


class NaiveTcgen05Backend(NaiveBackend):
    """Variable-size pipeline over the collective transport, experts on the tcgen05 grouped GEMMs."""

    name = "naive_tcgen05"

    def __init__(self, cfg, info, w13_local, w2_local, bias, capacity=None, **_):
        from ..experts import Tcgen05GroupedExperts

        self.layer = EPMoELayer(cfg, info.rank, info.world, w13_local, w2_local, experts=Tcgen05GroupedExperts())
        self.comm = CollectiveRowExchange()
        self.bias = bias


class FixedVllmExpertsBackend:
    """Fused peer-memory transport around the serving engine's own bf16 fused-experts kernel.

    Same router and transport as ``fused``; only the expert GEMMs differ (vLLM's ``fused_experts``), so an
    A/B against ``fused`` isolates the expert kernels and one against the engine's native all-gather /
    reduce-scatter isolates the transport.  Needs an importable vLLM; library code, comparison arm only.
    """

    name = "fixed_vllm_experts"

    def __init__(self, cfg, info, w13_local, w2_local, bias, capacity, **layer_kw):
        from vllm.model_executor.layers.fused_moe import fused_experts  # noqa: F401 - fails early without vLLM

        self._fused_experts = fused_experts
        self.cfg, self.bias, self.w13, self.w2 = cfg, bias, w13_local, w2_local
        self.layer = FixedEPLayer(cfg, info.rank, info.world, None, None, capacity=capacity, backend="cuda",
                                  device=w13_local.device, dtype=w13_local.dtype, **layer_kw)

    def _experts(self, hidden, local_ids, weights):
        # absent slots: expert 0 with weight 0; rows without any hit may hold stale payload, so zero them
        live = local_ids >= 0
        x = torch.where(live.any(dim=-1, keepdim=True), hidden, torch.zeros_like(hidden))
        ids = torch.where(live, local_ids, torch.zeros_like(local_ids)).to(torch.int32)
        w = torch.where(live, weights, torch.zeros_like(weights))
        # the engine's SiLU-and-mul has no clamp; with a finite swiglu_limit the two arms differ where it bites
        return self._fused_experts(x.contiguous(), self.w13, self.w2, w, ids)

    def run(self, x, logits):
        w, ids = self.layer.stage_route(logits, self.bias)
        return self.layer.forward_routed(x, w, ids, expert_fn=self._experts)[: x.shape[0]]


class VllmNativeAgRsBackend:
    """The serving engine's native expert-parallel data path, ``allgather_reducescatter``: every rank all-gathers
    the hidden rows and routing of all ranks (NCCL), runs the engine's own fused experts on the gathered batch
    with an expert map that keeps only its local experts, and a reduce-scatter (NCCL, bf16) returns to every rank
    the sum of the ranks' partial outputs for its own tokens.

    Assembled from vLLM's kernel object (``fused_experts`` with ``expert_map``) and ``torch.distributed``
    collectives rather than through the engine's ``get_ep_group().dispatch``, which needs a fully initialised
    engine (parallel state, forward context, workspace manager).  The steps and their order are those of the
    engine's ``MoEPrepareAndFinalizeNaiveDPEPModular`` with the all-gather / reduce-scatter manager.  Same
    router as the ``fused`` arm (the sm_100a router kernel), static buffers, CUDA-graph capturable.  Library
    code on purpose: this is the comparison arm the routed layer has to beat.
    Counterpart of ``VllmModularBackend("allgather_reducescatter")`` (``scripts/bench/backends.py:114-241``).
    """

    name = "vllm_agrs"

    def __init__(self, cfg, info, w13_local, w2_local, bias, capacity, **_):
        from vllm.model_executor.layers.fused_moe import fused_experts  # noqa: F401 - fails early without vLLM

        self._fused_experts = fused_experts
        self.cfg, self.bias, self.w13, self.w2, self.info = cfg, bias, w13_local, w2_local, info
        dev, R, C, H, K, E = w13_local.device, info.world, capacity, cfg.hidden_size, cfg.top_k, cfg.n_routed_experts
        L = cfg.experts_per_rank(R)
        self.C = C
        self.expert_map = torch.full((E,), -1, dtype=torch.int32, device=dev)
        self.expert_map[info.rank * L:(info.rank + 1) * L] = torch.arange(L, dtype=torch.int32, device=dev)
        self.x = torch.zeros(C, H, dtype=torch.bfloat16, device=dev)
        self.w = torch.zeros(C, K, dtype=torch.float32, device=dev)
        self.ids = torch.zeros(C, K, dtype=torch.int32, device=dev)
        self.gx = torch.zeros(R * C, H, dtype=torch.bfloat16, device=dev)
        self.gw = torch.zeros(R * C, K, dtype=torch.float32, device=dev)
        self.gids = torch.zeros(R * C, K, dtype=torch.int32, device=dev)
        self.out = torch.zeros(C, H, dtype=torch.bfloat16, device=dev)

    def run(self, x, logits):
        from ..ops.kernels import router_topk

        T = x.shape[0]
        self.x[:T].copy_(x)
        router_topk(logits, self.bias, self.cfg, self.w[:T], self.ids[:T])
        if T < self.C:  # padding rows: weight 0 on a valid expert
            self.w[T:].zero_()
            self.ids[T:].zero_()
        if self.info.world > 1:
            dist.all_gather_into_tensor(self.gx, self.x)
            dist.all_gather_into_tensor(self.gw, self.w)
            dist.all_gather_into_tensor(self.gids, self.ids)
        else:
            self.gx.copy_(self.x)
            self.gw.copy_(self.w)
            self.gids.copy_(self.ids)
        # the engine's SiLU-and-mul has no clamp; with a finite swiglu_limit the two arms differ where it bites
        partial = self._fused_experts(self.gx, self.w13, self.w2, self.gw, self.gids,
                                      global_num_experts=self.cfg.n_routed_experts, expert_map=self.expert_map)
        if self.info.world > 1:
            dist.reduce_scatter_tensor(self.out, partial.contiguous())
        else:
            self.out.copy_(partial)
        return self.out[:T]


class ReferenceFixedBackend:
    """The reference's own fixed layer with all four of its fusion switches (Triton + NCCL)."""

    name = "reference_fixed"

    def __init__(self, cfg, info, w13_local, w2_local, bias, capacity, **_):
        root = Path(__file__).resolve().parents[2] / "baseline" / "_ref"
        if not (root / "moeflow" / "fixed.py").exists():
            raise RuntimeError("the reference is not installed under baseline/_ref")
        if str(root) not in sys.path:
            sys.path.insert(0, str(root))
        loaded = sys.modules.get("moeflow")
        if loaded is not None and not str(getattr(loaded, "__file__", "")).startswith(str(root)):
            raise RuntimeError("the name 'moeflow' is already bound to this framework's import alias in this process; "
                               "run the reference arm in a process that has not imported it")
        from moeflow.config import MoEConfig as RefConfig  # type: ignore
        from moeflow.fixed import FixedEPLayer as RefLayer  # type: ignore

        ref_cfg = RefConfig(**cfg.to_dict())
        self.layer = RefLayer(ref_cfg, info.rank, info.world, w13_local, w2_local, capacity=capacity,
                              metadata_kernel=True, fused_reduce=True, fused_combine=True, fused_dispatch=True)
        self.bias = bias

    def run(self, x, logits):
        return self.layer.forward(x, logits, self.bias)[: x.shape[0]]


def make_backend(name: str, *args, **kw):
    table = {"fused": FusedFixedBackend, "torch_fixed": TorchFixedBackend, "naive": NaiveBackend,
             "naive_tcgen05": NaiveTcgen05Backend, "fixed_vllm_experts": FixedVllmExpertsBackend,
             "vllm_agrs": VllmNativeAgRsBackend,
             "reference_fixed": ReferenceFixedBackend}
    if name not in table:
        raise ValueError(f"unknown backend {name!r}; choose from {BACKENDS}")
    return table[name](*args, **kw)
