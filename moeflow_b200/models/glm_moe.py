"""GLM-5.3-Flash-shaped decoder built on the fused expert-parallel MoE layer.

Components (all inference-only, bf16, one process per GPU, attention TP=1 with data-parallel tokens,
DP = EP = world):

``SharedExpert``   the always-on SwiGLU MLP, run through the same tcgen05 grouped GEMM kernels as the
                   routed experts with a static one-expert plan;
``MoEBlock``       RMSNorm (sm_100a kernel) -> router logits (``RouterLogits``: the tcgen05 grouped kernel, fp32 output) ->
                   routed experts (``FixedEPLayer``: fused route+dispatch, expert GEMMs, return push,
                   combine) + shared expert -> residual;
``Attention``      grouped-query attention over a static KV cache for single-token decode steps, with
                   PyTorch's scaled-dot-product attention (library code: attention is outside the scope of
                   the MoE backend and is served by the host engine in production);
``DecodeModel``    ``n_layers`` x (attention + MoE block), random-initialised, with one CUDA graph per
                   decode step.

In production the host engine (vLLM) owns model loading and attention and reaches the MoE layer
through ``moeflow_b200.integrations``; this module exists so that a whole decode step of the named
shape can be measured and tested without that engine.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..config import MoEConfig
from ..experts import swiglu_clamp
from ..fixed import FixedEPLayer


@dataclass(frozen=True)
class AttentionConfig:
    n_heads: int = 32
    n_kv_heads: int = 4
    head_dim: int = 128
    max_seq: int = 2304
    rope_theta: float = 10000.0


def _rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16:
        from ..ops.kernels import rmsnorm

        return rmsnorm(x, gamma, eps)
    xf = x.to(torch.float32)
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.to(torch.float32)).to(x.dtype)


class SharedExpert:
    """Dense SwiGLU MLP ``w2 . swiglu(w13 . x)`` for up to ``capacity`` rows per call."""

    def __init__(self, w13: torch.Tensor, w2: torch.Tensor, capacity: int, limit: float | None, block_m: int = 64):
        self.w13, self.w2, self.C, self.limit, self.block_m = w13.contiguous(), w2.contiguous(), capacity, limit, block_m
        self.inter, self.hidden = w2.shape[-1], w2.shape[-2]
        self.cuda = w13.is_cuda and w13.dtype == torch.bfloat16 and self.hidden % 128 == 0 and self.inter % 128 == 0
        if not self.cuda:
            return
        from ..ops import _lib
        from ..ops.grouped_gemm import plan_from_offsets
        from ..ops.kernels import make_weight_tmap, sm_count

        dev = w13.device
        self._lib = _lib
        self.n_sms = sm_count(dev.index or 0)
        n_tiles = (capacity + block_m - 1) // block_m

        # One expert has few weight blocks (12 and 32 at the GLM shape): the stream-K cut (plan word 0) lays the
        # K steps of all units end to end and gives every SM the same share of the weight stream.
        self.tp = plan_from_offsets([0, capacity], block_m, dev, split1=0, split2=0)
        self.act = torch.zeros(capacity, self.inter, dtype=torch.bfloat16, device=dev)
        self.out = torch.zeros(capacity, self.hidden, dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(1, dtype=torch.int64, device=dev)
        self._x = torch.zeros(capacity, self.hidden, dtype=torch.bfloat16, device=dev)
        self._tm13 = make_weight_tmap(self.w13.view(1, 2 * self.inter, self.hidden))
        self._tm2 = make_weight_tmap(self.w2.view(1, self.hidden, self.inter))
        slots = 2 * self.n_sms  # stream-K: two partial tiles per CTA
        self._scratch = torch.zeros(slots * 2 * block_m * 128, dtype=torch.float32, device=dev)
        self._counters = torch.zeros(self.tp.n_tiles * max(self.inter, self.hidden) // 128 * 4, dtype=torch.int32, device=dev)
        common = dict(tile_e=self.tp.tile_e.data_ptr(), tile_s=self.tp.tile_s.data_ptr(), tile_n=self.tp.tile_n.data_ptr(),
                      plan=self.tp.plan.data_ptr(), partial=self._scratch.data_ptr(), counters=self._counters.data_ptr(),
                      max_split_slots=slots, status=self.status.data_ptr(), wait_ns=2_000_000_000,
                      partial_floats=self._scratch.numel(), n_counters=self._counters.numel(),
                      max_tiles=self.tp.tile_e.numel())
        self._a1 = _lib.GemmArgs(b_base=self._x.data_ptr(), b_pitch=self.hidden * 2, b_index=None, split_word=_lib.PLAN_SPLIT1,
                                 m_blocks=self.inter // 128, k_blocks=self.hidden // 64, rows_per_expert=2 * self.inter,
                                 up_row_offset=self.inter, out=self.act.data_ptr(), out_pitch=self.inter, row_scale=None,
                                 limit=float(limit) if limit is not None else 0.0, round_h=0, **common)
        self._a2 = _lib.GemmArgs(b_base=self.act.data_ptr(), b_pitch=self.inter * 2, b_index=None, split_word=_lib.PLAN_SPLIT2,
                                 m_blocks=self.hidden // 128, k_blocks=self.inter // 64, rows_per_expert=self.hidden,
                                 up_row_offset=0, out=self.out.data_ptr(), out_pitch=self.hidden, row_scale=None, limit=0.0,
                                 round_h=0, **common)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        t = x.shape[0]
        if not self.cuda:
            h = swiglu_clamp(x @ self.w13.transpose(0, 1), self.limit)
            return h @ self.w2.transpose(0, 1)
        self._x[:t].copy_(x)
        lib, s = self._lib.lib(), self._lib.stream_ptr()
        self._lib.check(lib.mf_gemm_gate_up(self._tm13, C.byref(self._a1), self.block_m, self.n_sms, s), "shared gate/up")
        self._lib.check(lib.mf_gemm_down(self._tm2, C.byref(self._a2), self.block_m, self.n_sms, s), "shared down")
        return self.out[:t]


class RouterLogits:
    """Router logits ``h . gate_w^T`` as fp32 ``[T, E]`` on the grouped down-projection kernel (tcgen05, bf16
    operands, fp32 accumulation and fp32 output): the gate matrix is one "expert" whose rows are padded to a
    multiple of 128, K is split so that the few weight blocks spread over several SMs, and only the E real
    columns are stored.  With it the MoE block issues no library GEMM."""

    def __init__(self, gate_w: torch.Tensor, capacity: int, block_m: int = 64):
        from ..ops import _lib
        from ..ops.grouped_gemm import plan_from_offsets
        from ..ops.kernels import make_weight_tmap, sm_count

        E, H = gate_w.shape
        dev = gate_w.device
        if H % 64:
            raise ValueError("hidden size must be a multiple of 64")
        self._lib, self.E, self.H, self.C, self.block_m = _lib, E, H, capacity, block_m
        rows = (E + 127) // 128 * 128
        self.w = torch.zeros(1, rows, H, dtype=torch.bfloat16, device=dev)
        self.w[0, :E] = gate_w.to(torch.bfloat16)
        self.n_sms = sm_count(dev.index or 0)
        k_blocks = H // 64
        split = max(s for s in (1, 2, 4, 8) if k_blocks % s == 0 and k_blocks // s >= 2 or s == 1)
        self.tp = plan_from_offsets([0, capacity], block_m, dev, split2=split)
        m_blocks = rows // 128
        slots = self.tp.n_tiles * m_blocks * split
        self._x = torch.zeros(max(capacity, block_m), H, dtype=torch.bfloat16, device=dev)
        self.logits = torch.zeros(capacity, E, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int64, device=dev)
        self._scratch = torch.zeros(max(1, slots) * block_m * 128, dtype=torch.float32, device=dev)
        self._counters = torch.zeros(self.tp.n_tiles * m_blocks * 8, dtype=torch.int32, device=dev)
        self._tmap = make_weight_tmap(self.w)
        self._args = _lib.GemmArgs(
            b_base=self._x.data_ptr(), b_pitch=H * 2, b_index=None, tile_e=self.tp.tile_e.data_ptr(),
            tile_s=self.tp.tile_s.data_ptr(), tile_n=self.tp.tile_n.data_ptr(), plan=self.tp.plan.data_ptr(),
            split_word=_lib.PLAN_SPLIT2, m_blocks=m_blocks, k_blocks=k_blocks, rows_per_expert=rows, up_row_offset=0,
            out=self.logits.data_ptr(), out_pitch=E, row_scale=None, partial=self._scratch.data_ptr(),
            counters=self._counters.data_ptr(), max_split_slots=slots, limit=0.0, round_h=0, status=self.status.data_ptr(),
            wait_ns=2_000_000_000, partial_floats=self._scratch.numel(), n_counters=self._counters.numel(),
            max_tiles=self.tp.tile_e.numel(), out_fp32=1, out_cols=E,
        )

    def __call__(self, h: torch.Tensor) -> torch.Tensor:
        t = h.shape[0]
        self._x[:t].copy_(h)
        self._lib.check(self._lib.lib().mf_gemm_down(self._tmap, C.byref(self._args), self.block_m, self.n_sms,
                                                     self._lib.stream_ptr()), "router logits")
        return self.logits[:t]


class MoEBlock:
    """Pre-norm MoE block: ``x + routed(norm(x)) + shared(norm(x))``."""

    def __init__(self, cfg: MoEConfig, routed: FixedEPLayer, gate_w: torch.Tensor, bias: torch.Tensor | None,
                 norm_w: torch.Tensor, shared: SharedExpert | None, eps: float = 1e-6, router: RouterLogits | None = None):
        self.cfg, self.routed, self.gate_w, self.bias, self.norm_w, self.shared, self.eps = cfg, routed, gate_w, bias, norm_w, shared, eps
        self.router = router

    def __call__(self, x: torch.Tensor, num_valid: torch.Tensor | None = None) -> torch.Tensor:
        h = _rmsnorm(x, self.norm_w, self.eps)
        if self.router is not None:
            logits = self.router(h)
        else:
            logits = torch.matmul(h.to(self.gate_w.dtype), self.gate_w.transpose(0, 1)).to(torch.float32)
        routed = self.routed.forward(h, logits, self.bias, num_valid)[: x.shape[0]]
        out = x + routed
        if self.shared is not None:
            out = out + self.shared(h)
        return out


class Attention:
    """Single-token GQA decode step over a static KV cache ``[B, n_kv, max_seq, d]`` (library SDPA)."""

    def __init__(self, hidden: int, acfg: AttentionConfig, batch: int, device, seed: int):
        self.acfg, self.hidden, self.batch = acfg, hidden, batch
        g = torch.Generator(device=device).manual_seed(seed)
        q_out, kv_out = acfg.n_heads * acfg.head_dim, acfg.n_kv_heads * acfg.head_dim

        def w(rows, cols):
            return (torch.randn(rows, cols, generator=g, device=device) / math.sqrt(cols)).to(torch.bfloat16)

        self.wqkv, self.wo = w(q_out + 2 * kv_out, hidden), w(hidden, q_out)
        self.norm_w = torch.ones(hidden, dtype=torch.bfloat16, device=device)
        self.k_cache = torch.zeros(batch, acfg.n_kv_heads, acfg.max_seq, acfg.head_dim, dtype=torch.bfloat16, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)

    def fill_cache(self, length: int, seed: int) -> None:
        """Stand-in for a prefill: random keys/values for the first ``length`` positions."""
        g = torch.Generator(device=self.k_cache.device).manual_seed(seed)
        self.k_cache[:, :, :length].copy_(torch.randn(self.k_cache[:, :, :length].shape, generator=g, device=self.k_cache.device) * 0.5)
        self.v_cache[:, :, :length].copy_(torch.randn(self.v_cache[:, :, :length].shape, generator=g, device=self.k_cache.device) * 0.5)

    def __call__(self, x: torch.Tensor, pos: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """``x [B, H]``; ``pos`` device int64 scalar (position being written); ``mask [1,1,1,max_seq]`` additive."""
        a = self.acfg
        h = _rmsnorm(x, self.norm_w, 1e-6)
        qkv = h @ self.wqkv.transpose(0, 1)
        q_out, kv_out = a.n_heads * a.head_dim, a.n_kv_heads * a.head_dim
        q = qkv[:, :q_out].view(self.batch, a.n_heads, 1, a.head_dim)
        k = qkv[:, q_out : q_out + kv_out].view(self.batch, a.n_kv_heads, 1, a.head_dim)
        v = qkv[:, q_out + kv_out :].view(self.batch, a.n_kv_heads, 1, a.head_dim)
        idx = pos.view(1, 1, 1, 1).expand(self.batch, a.n_kv_heads, 1, a.head_dim)
        self.k_cache.scatter_(2, idx, k)
        self.v_cache.scatter_(2, idx, v)
        o = F.scaled_dot_product_attention(q, self.k_cache, self.v_cache, attn_mask=mask, enable_gqa=True)
        return x + o.reshape(self.batch, q_out) @ self.wo.transpose(0, 1)


class DecodeModel:
    """``n_layers`` decoder layers for a fixed per-rank batch; ``step()`` runs one decode step from a graph."""

    def __init__(self, cfg: MoEConfig, rank: int, world: int, batch: int, n_layers: int, device, acfg: AttentionConfig | None = None,
                 group=None, seed: int = 0, attention: bool = True, weights_factory=None, fp8: bool = False,
                 own_router_gemm: bool = True):
        """``fp8``: the routed experts are kept as block-scaled e4m3 (one fp32 scale per 128x128 block, quantised
        from the random bf16 weights) and run on the ``kind::f8f6f4`` grouped GEMMs.  ``own_router_gemm``: router
        logits on the tcgen05 grouped kernel instead of a library matmul."""
        self.cfg, self.rank, self.world, self.batch, self.device = cfg, rank, world, batch, torch.device(device)
        self.acfg = acfg or AttentionConfig()
        dev, H, I, L = self.device, cfg.hidden_size, cfg.moe_intermediate_size, cfg.experts_per_rank(world)
        g = torch.Generator(device=dev).manual_seed(seed * 7919 + rank)

        def randn(*shape, scale):
            return (torch.randn(*shape, generator=g, device=dev) * scale).to(torch.bfloat16)

        capacity = 1
        while capacity < batch:
            capacity *= 2
        # one set of communication buffers for all layers (they run one at a time)
        self.routed = FixedEPLayer(cfg, rank, world, None, None, capacity=capacity, group=group, device=dev, backend="cuda")
        self.layers = []
        for layer in range(n_layers):
            given = weights_factory(layer) if weights_factory is not None else None
            prequantised = given is not None and len(given) == 4  # (w13_q, w13_s, w2_q, w2_s): e4m3 + block scales
            if prequantised:
                w13 = w2 = None
            elif given is not None:
                w13, w2 = given
            else:
                w13 = torch.empty(L, 2 * I, H, dtype=torch.bfloat16, device=dev)
                w2 = torch.empty(L, H, I, dtype=torch.bfloat16, device=dev)
                for e in range(L):
                    w13[e] = randn(2 * I, H, scale=2.0 / math.sqrt(H))
                    w2[e] = randn(H, I, scale=1.0 / math.sqrt(I))
            pack = None
            if prequantised:
                pack = self.routed.make_fp8_pack(*given)
                maps = (None, None)
            elif fp8:
                from ..weights import quant_block_fp8

                def quantise(w):
                    qs, ss = zip(*(quant_block_fp8(w[e]) for e in range(w.shape[0])))
                    return torch.stack([q.view(torch.uint8) for q in qs]).view(torch.float8_e4m3fn), torch.stack(ss)

                q13, s13 = quantise(w13)
                q2, s2 = quantise(w2)
                pack = self.routed.make_fp8_pack(q13, s13, q2, s2)
                w13 = w2 = None  # only the e4m3 copies are kept
                maps = (None, None)
            else:
                maps = self.routed.make_weight_maps(w13, w2)
            gate_w = randn(cfg.n_routed_experts, H, scale=1.0 / math.sqrt(H)).to(torch.float32)
            router = RouterLogits(gate_w, capacity) if own_router_gemm else None
            bias = 0.05 * torch.randn(cfg.n_routed_experts, generator=g, device=dev)
            shared = None
            if cfg.n_shared_experts:
                Is = I * cfg.n_shared_experts
                shared = SharedExpert(randn(2 * Is, H, scale=2.0 / math.sqrt(H)), randn(H, Is, scale=1.0 / math.sqrt(Is)),
                                      capacity, cfg.swiglu_limit)
            norm_w = torch.ones(H, dtype=torch.bfloat16, device=dev)
            attn = Attention(H, self.acfg, batch, dev, seed * 31 + layer) if attention else None
            self.layers.append({"w13": w13, "w2": w2, "maps": maps, "fp8": pack, "gate_w": gate_w, "bias": bias,
                                "shared": shared, "norm_w": norm_w, "attn": attn, "router": router})
        self.x = torch.zeros(batch, H, dtype=torch.bfloat16, device=dev)
        self.out = torch.zeros_like(self.x)
        self.pos = torch.zeros((), dtype=torch.int64, device=dev)
        self.mask = torch.full((1, 1, 1, self.acfg.max_seq), float("-inf"), dtype=torch.bfloat16, device=dev)
        self.graph: torch.cuda.CUDAGraph | None = None

    def prefill_standin(self, length: int) -> None:
        for i, layer in enumerate(self.layers):
            if layer["attn"] is not None:
                layer["attn"].fill_cache(length, 1000 + i)
        self.pos.fill_(length)
        self.mask.fill_(float("-inf"))
        self.mask[..., : length + 1] = 0

    def _forward(self) -> None:
        x = self.x
        for layer in self.layers:
            if layer["attn"] is not None:
                x = layer["attn"](x, self.pos, self.mask)
            if layer["fp8"] is not None:
                self.routed.bind_weights_fp8(layer["fp8"])
            else:
                self.routed.bind_weights(layer["w13"], layer["w2"], *layer["maps"])
            block = MoEBlock(self.cfg, self.routed, layer["gate_w"], layer["bias"], layer["norm_w"], layer["shared"],
                             router=layer["router"])
            x = block(x)
        self.out.copy_(x)

    def capture(self) -> "DecodeModel":
        import torch.distributed as dist

        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._forward()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._forward()
        torch.cuda.synchronize()
        return self

    def step(self) -> torch.Tensor:
        """One decode step for the whole batch; advances the position (mask and KV write index)."""
        if self.graph is None:
            self._forward()
        else:
            self.graph.replay()
        self.pos.add_(1)
        self.mask.view(-1).index_fill_(0, self.pos.view(1), 0.0)
        return self.out

    def close(self) -> None:
        self.graph = None
