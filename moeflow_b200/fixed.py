"""Fixed-capacity, CUDA-graph-capturable expert-parallel MoE layer.

Same contract as the variable-size pipeline (``ep_moe``) — one copy per (token, rank), slot-ordered
fp32 owner reduce, ascending-rank fp32 combine — with static shapes and no device-to-host traffic:

* Positions are fixed: token t of rank s bound for rank d always occupies ``send[d, t]`` which lands
  in ``recv[s, t]`` on d; a valid flag says whether t really hits d.  No count exchange.
* A row is ``[H hidden lanes | K int32 local ids | K fp32 weights | int32 valid]`` bit-packed into
  lanes of the activation dtype; the row pitch is padded to a multiple of 16 bytes so that rows can be
  moved with 16-byte vector stores and read by TMA.

Two backends share this surface:

``backend="cuda"`` (B200): five kernels per forward (six when the return push is not fused) and no library collective.  ``dispatch_push``
packs rows and stores them straight into the owners' ``recv`` buffers over peer memory, then publishes
an epoch flag; ``expert_meta`` waits for the flags and builds expert offsets, the tile map and the
K-split plan on the device; two tcgen05 grouped GEMMs (gate/up + SwiGLU, down + routing weight)
stream the expert weights by TMA; ``owner_reduce_push`` sums each row's slots in order and stores the
partial row straight into the source rank's ``ret_recv``; ``combine`` waits for the return flags and
merges by ascending rank in fp32.

``backend="torch"``: the same stages in plain PyTorch for any device and dtype, exchanging the static
buffers with ``all_to_all_single`` (NCCL or gloo).  It is the CPU path and the twin the CUDA kernels are
compared against.

Public surface follows the reference's ``moeflow/fixed.py:35-279``.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .config import MoEConfig
from .experts import BatchedTorchExperts, TorchLoopExperts
from .router import route

STAGES = ("ROUTER", "DISPATCH", "A2A_FORWARD", "EXPERT", "A2A_RETURN", "COMBINE")
#: Finer prefixes of the EXPERT stage that only the cuda backend can stop after (one per kernel).
CUDA_SUBSTAGES = ("META", "GEMM1", "GEMM2")

_DEFAULT_WAIT_NS = 2_000_000_000


def meta_lanes(top_k: int, itemsize: int = 2) -> int:
    """Lanes of ``itemsize`` bytes needed for K int32 ids + K fp32 weights + one int32 valid flag."""
    nbytes = 4 * (2 * top_k + 1)
    return (nbytes + itemsize - 1) // itemsize


def row_pitch_lanes(hidden: int, top_k: int, itemsize: int = 2) -> int:
    """Row pitch in lanes: hidden + metadata lanes, rounded up so that the pitch is a multiple of 16 B."""
    per16 = max(1, 16 // itemsize)
    lanes = hidden + meta_lanes(top_k, itemsize)
    return (lanes + per16 - 1) // per16 * per16


def _ordered_masked_sum(values: torch.Tensor, present: torch.Tensor) -> torch.Tensor:
    """fp32 sum over dim 1 in index order from +0.0, skipping absent terms. ``values [N,S,H]``."""
    acc = torch.zeros(values.shape[0], values.shape[2], dtype=torch.float32, device=values.device)
    for i in range(values.shape[1]):
        acc = torch.where(present[:, i, None], acc + values[:, i].to(torch.float32), acc)
    return acc


class FixedEPLayer:
    def __init__(
        self,
        cfg: MoEConfig,
        rank: int,
        world: int,
        w13_local: torch.Tensor | None,
        w2_local: torch.Tensor | None,
        capacity: int,
        group: dist.ProcessGroup | None = None,
        gemm_kwargs: dict | None = None,
        metadata_kernel: bool = False,
        fused_reduce: bool = False,
        fused_combine: bool = False,
        device: torch.device | None = None,
        fused_dispatch: bool = False,
        *,
        backend: str | None = None,
        dtype: torch.dtype | None = None,
        peer_region=None,
        wait_ns: int = _DEFAULT_WAIT_NS,
        combine_mode: str = "fp32",
    ):
        """``capacity`` C is the static per-rank token budget of this layer instance.

        The four boolean switches keep the reference's names.  On the torch backend they are accepted
        and select nothing (every stage is PyTorch).  On the cuda backend every stage is a fused
        kernel regardless; they exist so that call sites written for the reference keep working.

        ``peer_region`` (cuda backend) is a ``SymmetricRegion`` of ``peer_bytes(...)`` bytes; when it is
        None the layer allocates one through ``PeerGroup.from_dist(group)``.
        """
        if fused_reduce and not metadata_kernel:
            raise ValueError("fused_reduce consumes the inverse map produced by metadata_kernel")
        if combine_mode not in ("fp32", "bf16_ring"):
            raise ValueError(f"unknown combine mode {combine_mode!r}")
        self.cfg, self.rank, self.world, self.C = cfg, rank, world, capacity
        self.L = cfg.experts_per_rank(world)
        self.K, self.H, self.I = cfg.top_k, cfg.hidden_size, cfg.moe_intermediate_size
        self.w13, self.w2 = w13_local, w2_local
        self.group = group
        self.gemm_kwargs = dict(gemm_kwargs or {})
        self.metadata_kernel, self.fused_reduce = metadata_kernel, fused_reduce
        self.fused_combine, self.fused_dispatch = fused_combine, fused_dispatch
        self.combine_mode = combine_mode
        self.wait_ns = int(wait_ns)
        if device is None:
            if w13_local is None:
                raise ValueError("device is required when no weights are given")
            device = w13_local.device
        self.device = torch.device(device)
        if dtype is None:
            dtype = w13_local.dtype if w13_local is not None else torch.bfloat16
        self.dtype = dtype
        if backend is None:
            backend = "cuda" if (self.device.type == "cuda" and dtype == torch.bfloat16 and _cuda_ok(cfg)) else "torch"
        if backend not in ("cuda", "torch"):
            raise ValueError(f"unknown backend {backend!r}")
        self.backend = backend

        R, Cc, K, H = world, capacity, self.K, self.H
        itemsize = torch.empty((), dtype=dtype).element_size()
        self.row_width = H + meta_lanes(K, itemsize)
        self.pitch = row_pitch_lanes(H, K, itemsize)
        self.n_entries = R * Cc * K
        dev = self.device

        if backend == "cuda":
            self._init_cuda(peer_region)
        else:
            self._recv_store = torch.zeros(R, Cc, self.pitch, dtype=dtype, device=dev)
            self.ret_recv = torch.zeros(R, Cc, H, dtype=dtype, device=dev)
            self.out = torch.zeros(Cc, H, dtype=dtype, device=dev)
        # Send-side staging exists only on the torch backend (the cuda backend stores into peers).
        if backend == "torch":
            self._send_store = torch.zeros(R, Cc, self.pitch, dtype=dtype, device=dev)
            self.ret_send = torch.zeros(R, Cc, H, dtype=dtype, device=dev)
            self.send = self._send_store[:, :, : self.row_width]
        self.recv = self._recv_store[:, :, : self.row_width]
        self._rank_ids = torch.arange(R, device=dev)
        self._tok_ids = torch.arange(Cc, device=dev)
        self.torch_experts = self.gemm_kwargs.get("torch_experts") or (
            TorchLoopExperts() if dev.type == "cpu" else BatchedTorchExperts()
        )

    # ------------------------------------------------------------------------------------------
    # views
    # ------------------------------------------------------------------------------------------
    def _meta_view(self, store: torch.Tensor) -> torch.Tensor:
        """int32 view ``[R, C, 2K+1]`` of the metadata lanes of a row store."""
        lanes = meta_lanes(self.K, store.element_size())
        return store[:, :, self.H : self.H + lanes].view(torch.int32)[:, :, : 2 * self.K + 1]

    @staticmethod
    def peer_bytes(cfg: MoEConfig, world: int, capacity: int) -> int:
        """Bytes of the symmetric region one cuda-backend layer needs."""
        return _CudaLayout(cfg, world, capacity).total

    # ------------------------------------------------------------------------------------------
    # stage 1 (source): route and pack
    # ------------------------------------------------------------------------------------------
    def stage_route(self, logits: torch.Tensor, bias: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
        """ROUTER: ``logits [T, E]`` -> ``(weights [T, K] fp32, ids [T, K])``."""
        if self.backend == "cuda":
            from .ops.kernels import router_topk

            T = logits.shape[0]
            return router_topk(logits, bias, self.cfg, self._route_w[:T], self._route_ids[:T])
        weights, ids = route(logits, bias, self.cfg)
        return weights, ids.to(torch.int64)

    def stage_dispatch_pack(
        self, x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, num_valid: torch.Tensor | None = None
    ) -> torch.Tensor:
        """DISPATCH: fill the rows this rank sends.  Rows ``t >= num_valid`` (device scalar) are padding.

        Returns ``hit [C, R]``: token t has at least one expert on rank r.  On the cuda backend the rows
        are stored directly into the owners' ``recv`` buffers (this stage *is* the forward all-to-all).
        """
        T = x.shape[0]
        if T > self.C:
            raise ValueError(f"{T} tokens exceed capacity {self.C}")
        if self.backend == "cuda":
            return self._cuda_dispatch(x, weights, ids, num_valid)
        R, K, H, L = self.world, self.K, self.H, self.L
        ids = ids.to(torch.int64)
        owner = torch.div(ids, L, rounding_mode="floor")  # [T, K]
        on = owner[:, None, :] == self._rank_ids[None, :, None]  # [T, R, K]
        hit = on.any(dim=-1)
        if num_valid is not None:
            hit = hit & (self._tok_ids[:T] < num_valid)[:, None]
        on = on & hit[:, :, None]
        local = torch.where(on, ids[:, None, :] - self._rank_ids[None, :, None] * L, -1).to(torch.int32)
        w = torch.where(on, weights.to(torch.float32)[:, None, :], 0.0)

        self._send_store[:, :T, :H] = x.to(self.dtype)[None]
        meta = self._meta_view(self._send_store)
        meta[:, :T, :K] = local.permute(1, 0, 2)
        meta[:, :T, K : 2 * K] = w.permute(1, 0, 2).contiguous().view(torch.int32)
        meta[:, :T, 2 * K] = hit.transpose(0, 1).to(torch.int32)
        if T < self.C:
            meta[:, T:, :K] = -1
            meta[:, T:, K:] = 0
            hit = torch.cat([hit, hit.new_zeros(self.C - T, R)], dim=0)
        return hit

    def stage_pack(self, x, logits, bias, num_valid=None) -> torch.Tensor:
        """ROUTER + DISPATCH. Returns ``hit [C, R]``.  One kernel on the cuda backend."""
        if self.backend == "cuda":
            if x.shape[0] > self.C:
                raise ValueError(f"{x.shape[0]} tokens exceed capacity {self.C}")
            return self._cuda_dispatch(x, None, None, num_valid, logits=logits, bias=bias)
        weights, ids = self.stage_route(logits, bias)
        return self.stage_dispatch_pack(x, weights, ids, num_valid)

    # ------------------------------------------------------------------------------------------
    # stage 2 (owner): experts + slot-ordered reduce
    # ------------------------------------------------------------------------------------------
    def received_routing(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Unpack ``recv``: ``(hidden [RC, H], local ids [RC, K] (-1 = none), weights [RC, K] fp32)``."""
        R, Cc, K, H = self.world, self.C, self.K, self.H
        rows = self._recv_store.view(R * Cc, self.pitch)
        meta = self._meta_view(self._recv_store).reshape(R * Cc, 2 * K + 1)
        valid = meta[:, 2 * K] != 0
        local = torch.where(valid[:, None], meta[:, :K].to(torch.int64), -1)
        wts = meta[:, K : 2 * K].contiguous().view(torch.float32)
        return rows[:, :H], local, wts

    def stage_experts(self, expert_fn=None, prepare_fn=None, *, direct_output: bool = False) -> torch.Tensor | None:
        """Consume ``recv [R(src), C, row]`` and produce one partial row per received row.

        ``expert_fn(x_rows [RC, H], local_ids [RC, K] (-1 = no hit), weights [RC, K] fp32) -> [RC, H]``
        replaces the built-in experts and owner reduce.  ``prepare_fn(rows [RC, row_width])`` may own
        the received-row format and returns the argument tuple for ``expert_fn``.  With
        ``direct_output`` the tensor ``expert_fn`` returns is itself used as the return buffer (no
        copy) after a strict shape/dtype/device/contiguity check, and is returned as ``[R, C, H]``.
        """
        R, Cc, H = self.world, self.C, self.H
        if direct_output and prepare_fn is None:
            raise ValueError("Direct expert output requires custom input preparation")
        if prepare_fn is not None:
            if expert_fn is None:
                raise ValueError("Custom input preparation requires an external expert function")
            if self.backend == "cuda":
                self._cuda_meta()  # waits for the dispatch flags of every source rank
            rows = self._recv_store.view(R * Cc, self.pitch)[:, : self.row_width]
            output = expert_fn(*prepare_fn(rows))
            if direct_output:
                if (
                    tuple(output.shape) != (R * Cc, H)
                    or output.dtype != self.dtype
                    or output.device != self._recv_store.device
                    or not output.is_contiguous()
                ):
                    raise ValueError("Direct expert output must be contiguous and match return shape, dtype and device")
                return output.view(R, Cc, H)
            self._store_partials(output)
            return None
        if expert_fn is not None:
            if self.backend == "cuda":
                self._cuda_meta()  # waits for the dispatch flags of every source rank
            x_rows, local, wts = self.received_routing()
            self._store_partials(expert_fn(x_rows, local, wts))
            return None
        if self.backend == "cuda":
            self._cuda_experts()
            return None
        self._torch_experts()
        return None

    def _store_partials(self, partials: torch.Tensor) -> None:
        """Partial rows ``[RC, H]`` -> the return path (staging buffer, or peers on the cuda backend)."""
        if self.backend == "cuda":
            self._cuda_push_partials(partials)
        else:
            self.ret_send.view(self.world * self.C, self.H).copy_(partials)

    def _torch_layout(self, local: torch.Tensor):
        """Stable expert-major order of the (row, slot) entries; sentinel L collects empty slots."""
        L, K = self.L, self.K
        keys = torch.where(local >= 0, local, L).reshape(-1)
        order = torch.sort(keys, stable=True).indices
        # scatter_add instead of bincount: no host round trip, so the twin can be captured in a graph too
        counts = torch.zeros(L + 1, dtype=torch.int64, device=keys.device).scatter_add_(0, keys, torch.ones_like(keys))
        offsets = torch.zeros(L + 1, dtype=torch.int64, device=keys.device)
        torch.cumsum(counts[:L], dim=0, out=offsets[1:])
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device)
        inv = torch.where(keys < L, inv, -1)
        return order, offsets, inv, torch.div(order, K, rounding_mode="floor"), order % K

    def _torch_experts(self) -> None:
        R, Cc, K, H = self.world, self.C, self.K, self.H
        x_rows, local, wts = self.received_routing()
        order, offsets, inv, entry_row, entry_slot = self._torch_layout(local)
        n_live = offsets[-1]
        if isinstance(self.torch_experts, TorchLoopExperts):
            n = int(n_live)  # host read: the torch backend is not the graph-captured product path
            rows = x_rows[entry_row[:n]]
            y = self.torch_experts(rows, offsets, self.w13, self.w2, self.cfg.swiglu_limit, wts[entry_row[:n], entry_slot[:n]])
            y = torch.cat([y, y.new_zeros(order.numel() - n + 1, H)], dim=0)
        else:
            rows = x_rows[entry_row]
            y = self.torch_experts(rows, offsets, self.w13, self.w2, self.cfg.swiglu_limit, wts[entry_row, entry_slot])
            y = torch.cat([y, y.new_zeros(1, H)], dim=0)
        gathered = y[inv.view(R * Cc, K)]  # -1 picks the trailing zero row and is masked anyway
        partial = _ordered_masked_sum(gathered, local >= 0)
        self.ret_send.view(R * Cc, H).copy_(partial.to(self.dtype))

    # ------------------------------------------------------------------------------------------
    # stage 3 (source): combine
    # ------------------------------------------------------------------------------------------
    def stage_combine(self, hit: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        if self.backend == "cuda" and out_dtype == torch.bfloat16:
            return self._cuda_combine(hit)
        return combine_partials(self.ret_recv, hit, out_dtype, self.rank, self.combine_mode)

    # ------------------------------------------------------------------------------------------
    # exchanges (torch backend) and SPMD entry points
    # ------------------------------------------------------------------------------------------
    def _exchange(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        if self.world == 1 and (self.group is None or not dist.is_initialized()):
            out.copy_(inp)
            return
        dist.all_to_all_single(out, inp, group=self.group)

    def forward_routed(
        self,
        x,
        weights,
        ids,
        num_valid: torch.Tensor | None = None,
        expert_fn=None,
        combine_fn=None,
        prepare_fn=None,
        direct_expert_output: bool = False,
    ):
        """Pre-routed forward; ``combine_fn(ret_recv, hit)`` may replace the built-in combine."""
        T = x.shape[0]
        hit = self.stage_dispatch_pack(x, weights, ids, num_valid)
        if self.backend == "torch":
            self._exchange(self._recv_store, self._send_store)
        partials = self.stage_experts(expert_fn, prepare_fn=prepare_fn, direct_output=direct_expert_output)
        if self.backend == "torch":
            self._exchange(self.ret_recv, self.ret_send if partials is None else partials)
        elif partials is not None:
            self._cuda_push_partials(partials.view(self.world * self.C, self.H))
        if combine_fn is not None:
            if self.backend == "cuda":
                self._cuda_wait_return()
            out = combine_fn(self.ret_recv, hit)
        else:
            out = self.stage_combine(hit, x.dtype)
        return out[:T]

    def forward(self, x, logits, bias, num_valid: torch.Tensor | None = None, stop_after: str | None = None):
        """Whole layer; ``stop_after`` (one of ``STAGES``) truncates it for prefix-graph stage timing."""
        if stop_after is not None and stop_after not in STAGES:
            if not (self.backend == "cuda" and stop_after in CUDA_SUBSTAGES):
                raise ValueError(f"stop_after must be one of {STAGES}")
        if self.backend == "cuda" and stop_after != "ROUTER":
            hit = self.stage_pack(x, logits, bias, num_valid)  # routing fused into the dispatch kernel
        else:
            weights, ids = self.stage_route(logits, bias)
            if stop_after == "ROUTER":
                return weights
            hit = self.stage_dispatch_pack(x, weights, ids, num_valid)
        if stop_after == "DISPATCH":
            return hit
        if self.backend == "torch":
            self._exchange(self._recv_store, self._send_store)
        if stop_after == "A2A_FORWARD":
            return self.recv
        if stop_after in CUDA_SUBSTAGES:
            self._cuda_experts(stop_after)
            return self.plan
        self.stage_experts()
        if stop_after == "EXPERT":
            return self.ret_recv if self.backend == "cuda" else self.ret_send
        if self.backend == "torch":
            self._exchange(self.ret_recv, self.ret_send)
        if stop_after == "A2A_RETURN":
            return self.ret_recv
        return self.stage_combine(hit, x.dtype)

    # ------------------------------------------------------------------------------------------
    # cuda backend
    # ------------------------------------------------------------------------------------------
    def _init_cuda(self, peer_region) -> None:
        from .ops import _lib
        from .ops.kernels import make_weight_tmap, sm_count
        from .parallel.peer import PeerGroup

        cfg, R, Cc, K, H, I, L = self.cfg, self.world, self.C, self.K, self.H, self.I, self.L
        dev = self.device
        if not _cuda_ok(cfg):
            raise ValueError("cuda backend needs hidden and intermediate sizes that are multiples of 128")
        lay = _CudaLayout(cfg, R, Cc)
        self._layout = lay
        if peer_region is None:
            peer_region = PeerGroup(self.rank, R, self.group, dev).allocate(lay.total)
        if peer_region.world != R or peer_region.local.nbytes < lay.total:
            raise ValueError("peer region does not fit this layer")
        self.peer_region = peer_region
        self._recv_store = peer_region.view(lay.recv_off, (R, Cc, self.pitch), torch.bfloat16)
        self.ret_recv = peer_region.view(lay.ret_off, (R, Cc, H), torch.bfloat16)
        self._disp_flags = peer_region.view(lay.dflag_off, (R,), torch.int32)
        self._ret_flags = peer_region.view(lay.rflag_off, (R,), torch.int32)
        self._peer_recv = peer_region.table(lay.recv_off)
        self._peer_ret = peer_region.table(lay.ret_off)
        self._peer_dflag = peer_region.table(lay.dflag_off)
        self._peer_rflag = peer_region.table(lay.rflag_off)

        i32 = dict(dtype=torch.int32, device=dev)
        N = self.n_entries
        # token rows per tile: 64 for decode; 128 when experts see many rows (prefill), which halves the
        # number of times an expert's weights are streamed.  The estimate is the expectation under even
        # routing (R*C*K entries over R*L experts), not the worst case: wide tiles cost pipeline stages, and
        # with few rows per expert the narrower tile keeps more weight bytes in flight.
        # A buffer set built without weights may be bound to e4m3 experts later: plan its tiles for them unless told
        # otherwise (gemm_kwargs fp8_weights=False / True).
        fp8_hint = bool(self.gemm_kwargs.get("fp8_weights", self.w13 is None))
        self.block_m = int(self.gemm_kwargs.get("block_m", choose_block_m(Cc, K, L, fp8=fp8_hint)))
        if self.block_m not in (32, 64, 128, 256):
            raise ValueError("block_m must be 32, 64, 128 or 256")
        self.n_sms = int(self.gemm_kwargs.get("n_sms", sm_count(dev.index if dev.index is not None else 0)))
        self.max_tiles = (N + self.block_m - 1) // self.block_m + L
        self.out = torch.zeros(Cc, H, dtype=torch.bfloat16, device=dev)
        self.hit = torch.zeros(Cc, R, dtype=torch.uint8, device=dev)
        self._route_w = torch.zeros(Cc, K, dtype=torch.float32, device=dev)
        self._route_ids = torch.zeros(Cc, K, **i32)
        self._epoch = torch.zeros(1, **i32)
        self._done = torch.zeros(4, **i32)
        self._push_epoch = torch.zeros(1, **i32)  # return pushes so far (the combine expects this many x C arrivals)
        self.status = torch.zeros(1, dtype=torch.int64, device=dev)
        self.offsets = torch.zeros(L + 1, **i32)
        self.entry_row = torch.zeros(N, **i32)
        self.entry_slot = torch.zeros(N, **i32)
        self.entry_w = torch.zeros(N, dtype=torch.float32, device=dev)
        self.inv = torch.zeros(N, **i32)
        self.tile_e = torch.zeros(self.max_tiles, **i32)
        self.tile_s = torch.zeros(self.max_tiles, **i32)
        self.tile_n = torch.zeros(self.max_tiles, **i32)
        self.plan = torch.zeros(_lib.PLAN_WORDS, **i32)
        self.act = torch.zeros(max(N, self.block_m), I, dtype=torch.bfloat16, device=dev)  # >= one TMA box of rows
        self.y = torch.zeros(N, H, dtype=torch.bfloat16, device=dev)
        mb1, mb2 = I // 128, H // 128
        # arrival counters of cut units: one per (unit, 32-row quarter) and, in the fp8 kernels with 128-column
        # tiles, per column group (two)
        n_cnt1 = self.max_tiles * mb1 * 8
        # the tail of the first counter array (cleared with it by the metadata kernel) counts, per token tile, the
        # gate/up quarters whose activations are final: the down GEMM starts a tile as soon as it is complete
        self._counters1 = torch.zeros(n_cnt1 + self.max_tiles, **i32)
        self._tile_done = self._counters1[n_cnt1:]
        self._counters2 = torch.zeros(self.max_tiles * mb2 * 8, **i32)
        # split-K scratch: a byte budget; the metadata kernel sizes the partial slots for the widest token tile
        # (each GEMM gets its own half: the down GEMM may run while gate/up units are still being fixed up)
        partial_floats = int(self.gemm_kwargs.get("split_scratch_mb", 64)) * (1 << 20) // 4 // 2
        self.max_split_slots = partial_floats // (2 * self.block_m * 128)
        self._partial = torch.zeros(2 * partial_floats, dtype=torch.float32, device=dev)
        self._keep: list = []  # ctypes objects and temporaries that must outlive launches

        S = _lib
        self._a_dispatch = S.DispatchArgs(
            peer_recv=self._peer_recv.data_ptr(), peer_flag=self._peer_dflag.data_ptr(), hit=self.hit.data_ptr(),
            epoch=self._epoch.data_ptr(), done_counter=self._done[0:].data_ptr(), T=0, C=Cc, H=H, K=K, R=R, L=L,
            rank=self.rank, pitch=self.pitch * 2, skip_payload=int(self.gemm_kwargs.get("skip_payload", 1)),
            route_w=self._route_w.data_ptr(), route_ids=self._route_ids.data_ptr(), E=cfg.n_routed_experts,
            n_group=cfg.n_group, topk_group=cfg.topk_group, sigmoid=int(cfg.scoring_func == "sigmoid"),
            renorm=int(cfg.norm_topk_prob), scale=float(cfg.routed_scaling_factor),
        )
        if cfg.scoring_func not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown scoring function {cfg.scoring_func!r}")
        self._a_meta = S.MetaArgs(
            recv=self._recv_store.data_ptr(), pitch=self.pitch * 2, H=H, K=K, L=L, rows=R * Cc, R=R,
            flags=self._disp_flags.data_ptr(), epoch=self._epoch.data_ptr(), offsets=self.offsets.data_ptr(),
            entry_row=self.entry_row.data_ptr(), entry_slot=self.entry_slot.data_ptr(), entry_w=self.entry_w.data_ptr(),
            inv=self.inv.data_ptr(), tile_e=self.tile_e.data_ptr(), tile_s=self.tile_s.data_ptr(),
            tile_n=self.tile_n.data_ptr(), plan=self.plan.data_ptr(), counters1=self._counters1.data_ptr(),
            n_counters1=self._counters1.numel(), counters2=self._counters2.data_ptr(),
            n_counters2=self._counters2.numel(), block_m=self.block_m, max_tiles=self.max_tiles, m_blocks1=mb1,
            k_blocks1=H // 64, m_blocks2=mb2, k_blocks2=I // 64, n_sms=self.n_sms,
            max_split_slots=self.max_split_slots, status=self.status.data_ptr(), wait_ns=self.wait_ns,
            partial_floats=partial_floats, stream_k=int(self.gemm_kwargs.get("stream_k", 0)),
            # The metadata kernel is launched without programmatic serialization: started early, in the shadow of the
            # dispatch kernel, its phases after the wait ran three times slower (measured on B200: 18 us against
            # 8 us from dispatch end to plan), which cost more than the microsecond of launch latency it hid.  The
            # GEMMs behind it still start early and overlap their prologues with it.
            late_launch=int(self.gemm_kwargs.get("meta_late_launch", 0)), plain_launch=int(self.gemm_kwargs.get("meta_plain_launch", 1)),
        )
        # Metadata: one CTA for decode sizes; for prefill sizes (many received rows) the counting sort is
        # split over several CTAs in two chained launches.  Same result either way.
        n_words = R * Cc * K
        # up to 8192 slot words one CTA keeps them all in registers (one pass); above that the two chained
        # multi-CTA launches take 11-18 us where a sweeping single CTA would take 134 us at 32768 words
        self.meta_ctas = int(self.gemm_kwargs.get("meta_ctas", choose_meta_ctas(n_words, self.n_sms)))
        if not 1 <= self.meta_ctas <= 1024:
            raise ValueError("meta_ctas must be between 1 and 1024")
        if self.meta_ctas > 1:
            self._cta_hist = torch.zeros(self.meta_ctas * L, **i32)
            self._meta_acc = torch.zeros(2, **i32)
            self._a_meta.n_ctas = self.meta_ctas
            self._a_meta.cta_hist = self._cta_hist.data_ptr()
            self._a_meta.acc = self._meta_acc.data_ptr()
        limit = cfg.swiglu_limit if cfg.swiglu_limit is not None else 0.0
        common = dict(
            tile_e=self.tile_e.data_ptr(), tile_s=self.tile_s.data_ptr(), tile_n=self.tile_n.data_ptr(),
            plan=self.plan.data_ptr(), partial=self._partial.data_ptr(), max_split_slots=self.max_split_slots,
            limit=float(limit), round_h=int(self.gemm_kwargs.get("round_h", 0)), status=self.status.data_ptr(),
            wait_ns=self.wait_ns, partial_floats=partial_floats, max_tiles=self.max_tiles,
        )
        self._a_gemm1 = S.GemmArgs(
            b_base=self._recv_store.data_ptr(), b_pitch=self.pitch * 2, b_index=self.entry_row.data_ptr(),
            split_word=S.PLAN_SPLIT1, m_blocks=mb1, k_blocks=H // 64, rows_per_expert=2 * I, up_row_offset=I,
            out=self.act.data_ptr(), out_pitch=I, row_scale=None, counters=self._counters1.data_ptr(),
            n_counters=n_cnt1, **common,
        )
        self._a_gemm2 = S.GemmArgs(
            b_base=self.act.data_ptr(), b_pitch=I * 2, b_index=None, split_word=S.PLAN_SPLIT2, m_blocks=mb2,
            k_blocks=I // 64, rows_per_expert=H, up_row_offset=0, out=self.y.data_ptr(), out_pitch=H,
            row_scale=self.entry_w.data_ptr(), counters=self._counters2.data_ptr(),
            n_counters=self._counters2.numel(), **common,
        )
        self._a_gemm2.partial = self._partial[partial_floats:].data_ptr()
        # Long prefill (256-row tiles): a down-projection unit covers two adjacent weight blocks, so a token tile is
        # fetched from L2 once per 256 output columns (gemm_kwargs down_two_blocks overrides).
        self.down_two_blocks = bool(self.gemm_kwargs.get("down_two_blocks", self.block_m >= 256)) and H % 256 == 0
        if self.down_two_blocks:
            g2 = self._a_gemm2
            g2.two_blocks, g2.m_blocks, g2.up_row_offset = 1, H // 256, 128
            self._a_meta.m_blocks2 = H // 256
        # Tile-level hand-over of the activations (gemm_kwargs tile_handover=False: the down GEMM waits for the
        # whole gate/up grid instead).
        self.tile_handover = bool(self.gemm_kwargs.get("tile_handover", True))
        if self.tile_handover:
            self._a_gemm1.tile_done = self._tile_done.data_ptr()
            self._a_gemm2.tile_wait = self._tile_done.data_ptr()
            # one count per epilogue warp of the gate/up GEMM and weight block: two groups of four at 256-row tiles
            self._a_gemm2.tile_wait_target = (8 if self.block_m >= 256 else 4) * mb1
        # The down GEMM reads its token operand (act, contiguous in expert-major order) by TMA, one bulk copy
        # per pipeline stage; gemm_kwargs b_tma=False falls back to the 16-byte gather the gate/up GEMM uses.
        self._tmap_act = None
        if bool(self.gemm_kwargs.get("b_tma", True)):
            from .ops.kernels import make_tile_tmap

            self._tmap_act = make_tile_tmap(self.act, self.block_m)
            self._a_gemm2.b_tmap = C.addressof(self._tmap_act)
        # Opt-in (gemm_kwargs permute_rows=True): copy the received hidden rows into expert-major order first,
        # so that the gate/up GEMM reads token tiles by TMA too instead of gathering them by entry index.
        # Default: on with 256-row tiles, where 64 gather threads would have to place 32 chunks each per stage.
        self.permute_rows = bool(self.gemm_kwargs.get("permute_rows", self.block_m >= 256))
        if self.permute_rows:
            from .ops.kernels import make_tile_tmap

            self._xg = torch.zeros(max(N, self.block_m), H, dtype=torch.bfloat16, device=dev)
            self._tmap_xg = make_tile_tmap(self._xg, self.block_m)
            g1 = self._a_gemm1
            g1.b_base, g1.b_pitch, g1.b_index = self._xg.data_ptr(), H * 2, None
            g1.b_tmap = C.addressof(self._tmap_xg)
        # Owner reduce + return push can run inside the down GEMM (gemm_kwargs fuse_return=True: four extra
        # warps reduce a row as soon as its last slot is written and store it into the source rank's
        # buffer) or as the separate owner_reduce_push kernel chained by programmatic launch.  Measured on
        # B200 the separate kernel is 3-24 us faster per layer at T = 1..128, so it is the default.
        self.fuse_return = bool(self.gemm_kwargs.get("fuse_return", False))
        self.row_hits = torch.zeros(R * Cc, **i32)
        self._a_meta.row_hits = self.row_hits.data_ptr()
        if self.fuse_return:
            self._row_cnt = torch.zeros(R * Cc * mb2 * 4, **i32)
            g2 = self._a_gemm2
            g2.ret_peer, g2.ret_flag = self._peer_ret.data_ptr(), self._peer_rflag.data_ptr()
            g2.ret_epoch, g2.ret_done = self._push_epoch.data_ptr(), self._done[3:].data_ptr()
            g2.row_cnt, g2.row_hits = self._row_cnt.data_ptr(), self.row_hits.data_ptr()
            g2.entry_row, g2.inv = self.entry_row.data_ptr(), self.inv.data_ptr()
            g2.ret_rank, g2.ret_R, g2.ret_C, g2.ret_K = self.rank, R, Cc, K
        self._a_reduce = S.ReducePushArgs(
            y=self.y.data_ptr(), inv=self.inv.data_ptr(), recv=self._recv_store.data_ptr(), pitch=self.pitch * 2,
            peer_ret=self._peer_ret.data_ptr(), peer_flag=self._peer_rflag.data_ptr(), epoch=self._epoch.data_ptr(),
            done_counter=self._done[1:].data_ptr(), R=R, C=Cc, H=H, K=K, rank=self.rank, valid_word=2 * K,
            push_epoch=self._push_epoch.data_ptr(),
        )
        self._row_ids = torch.arange(R * Cc, **i32)
        self._a_push = S.ReducePushArgs(
            y=None, inv=self._row_ids.data_ptr(), recv=self._recv_store.data_ptr(), pitch=self.pitch * 2,
            peer_ret=self._peer_ret.data_ptr(), peer_flag=self._peer_rflag.data_ptr(), epoch=self._epoch.data_ptr(),
            done_counter=self._done[2:].data_ptr(), R=R, C=Cc, H=H, K=1, rank=self.rank, valid_word=2 * K,
            push_epoch=self._push_epoch.data_ptr(),
        )
        self._scratch_out = None
        self._a_combine = S.CombineArgs(
            ret=self.ret_recv.data_ptr(), hit=self.hit.data_ptr(), out=self.out.data_ptr(),
            flags=self._ret_flags.data_ptr(), epoch=self._push_epoch.data_ptr(), R=R, C=Cc, H=H, rank=self.rank,
            ring=int(self.combine_mode == "bf16_ring"), status=self.status.data_ptr(), wait_ns=self.wait_ns,
        )
        self._tmap13 = self._tmap2 = None
        self._fp8 = None  # set by set_weights_fp8
        self._expand = None  # e4m3 pack expanded to bf16 per forward (256-row token tiles)
        self._lib = _lib.lib()
        if self.w13 is not None:
            self.set_weights(self.w13, self.w2)

    def set_weights(self, w13_local: torch.Tensor, w2_local: torch.Tensor) -> None:
        """(Re)bind the local expert shard: ``w13 [L, 2I, H]``, ``w2 [L, H, I]`` bf16, contiguous."""
        from .ops.kernels import make_weight_tmap

        L, H, I = self.L, self.H, self.I
        if tuple(w13_local.shape) != (L, 2 * I, H) or tuple(w2_local.shape) != (L, H, I):
            raise ValueError("weight shard has the wrong shape")
        if w13_local.dtype != torch.bfloat16 or w2_local.dtype != torch.bfloat16:
            raise ValueError("cuda backend takes bf16 weights")
        self.w13, self.w2 = w13_local.contiguous(), w2_local.contiguous()
        self._fp8 = self._expand = None
        self._tmap13 = make_weight_tmap(self.w13)
        self._tmap2 = make_weight_tmap(self.w2)

    def set_weights_fp8(self, w13_q, w13_s, w2_q, w2_s) -> None:
        """Bind block-scaled e4m3 expert weights (kept un-dequantised).

        ``w13_q [L, 2I, H]`` / ``w2_q [L, H, I]`` float8_e4m3fn with fp32 scales per 128x128 block
        (``w13_s [L, 2I/128, H/128]``, ``w2_s [L, H/128, I/128]``).  The forward then quantises the
        received rows and the SwiGLU activations per 1x128 group on the device and runs the
        ``kind::f8f6f4`` grouped GEMMs; inputs and outputs of the layer stay bf16.
        """
        self.bind_weights_fp8(self.make_fp8_pack(w13_q, w13_s, w2_q, w2_s))

    def make_fp8_pack(self, w13_q, w13_s, w2_q, w2_s) -> dict:
        """Validate one MoE layer's e4m3 weights and build what binding them needs (TMA descriptors, fp32 scale
        tensors).  Build once per MoE layer, then ``bind_weights_fp8(pack)`` before its forward: a decoder
        shares one buffer set between all its MoE layers."""
        from .ops.kernels import make_weight_tmap

        if self.backend != "cuda":
            raise ValueError("fp8 weights need the cuda backend")
        L, H, I = self.L, self.H, self.I
        if tuple(w13_q.shape) != (L, 2 * I, H) or tuple(w2_q.shape) != (L, H, I):
            raise ValueError("weight shard has the wrong shape")
        if w13_q.dtype != torch.float8_e4m3fn or w2_q.dtype != torch.float8_e4m3fn:
            raise ValueError("e4m3 weights expected")
        if tuple(w13_s.shape) != (L, 2 * I // 128, H // 128) or tuple(w2_s.shape) != (L, H // 128, I // 128):
            raise ValueError("scales must be one fp32 per 128x128 block")
        if H > 4096 or I > 4096:
            raise ValueError("fp8 path supports K <= 4096")
        pack = {"w13": w13_q.contiguous(), "w2": w2_q.contiguous(), "s13": w13_s.to(torch.float32).contiguous(),
                "s2": w2_s.to(torch.float32).contiguous()}
        if self.block_m > 128:
            # Long-prefill layers (256-row token tiles): the block-scaled kernels take tiles of up to 128 rows and are
            # bound by their per-K-block promotion there, so every forward expands the bound experts into a bf16
            # scratch (shared by all layers of this shape on the device) and runs the bf16 kernels on it.
            pack["expand"] = True
            return pack
        pack["tm13"] = make_weight_tmap(pack["w13"].view(torch.uint8))
        pack["tm2"] = make_weight_tmap(pack["w2"].view(torch.uint8))
        return pack

    # (device index, L, I, H) -> bf16 weight scratch + tensor maps.  Shared by every layer of that shape on the device:
    # each forward rewrites it before its GEMMs, so forwards that use it must be ordered on one stream (they are: a
    # decoder runs its layers one after the other).  `release_expand_scratch()` frees it.
    _expand_scratch: dict = {}

    @classmethod
    def release_expand_scratch(cls) -> None:
        """Drop the bf16 expansion scratch of all shapes (layers bound to e4m3 packs rebuild it on their next bind)."""
        cls._expand_scratch.clear()

    def _expanded_weights(self) -> dict:
        from .ops.kernels import make_weight_tmap

        key = (self.device.index, self.L, self.I, self.H)
        e = FixedEPLayer._expand_scratch.get(key)
        if e is None:
            w13 = torch.empty(self.L, 2 * self.I, self.H, dtype=torch.bfloat16, device=self.device)
            w2 = torch.empty(self.L, self.H, self.I, dtype=torch.bfloat16, device=self.device)
            e = {"w13": w13, "w2": w2, "tm13": make_weight_tmap(w13), "tm2": make_weight_tmap(w2)}
            FixedEPLayer._expand_scratch[key] = e
        return e

    def _fp8_buffers(self) -> dict:
        """Quantised activations and the fp8 GEMM argument blocks of this buffer set (allocated on first use)."""
        if getattr(self, "_fp8_shared", None) is not None:
            return self._fp8_shared
        from .ops import _lib

        H, I, N, dev = self.H, self.I, self.n_entries, self.device
        rows = self.world * self.C
        f = {}
        f["xq"] = torch.zeros(rows, H, dtype=torch.uint8, device=dev)
        f["xs"] = torch.zeros(rows, H // 128, dtype=torch.float32, device=dev)
        f["aq"] = torch.zeros(max(N, self.block_m), I, dtype=torch.uint8, device=dev)  # >= one TMA box of rows
        f["as"] = torch.zeros(max(N, self.block_m), I // 128, dtype=torch.float32, device=dev)
        g1, g2 = self._a_gemm1, self._a_gemm2
        common = dict(tile_e=g1.tile_e, tile_s=g1.tile_s, tile_n=g1.tile_n, plan=g1.plan, partial=g1.partial,
                      max_split_slots=g1.max_split_slots, limit=g1.limit, round_h=0, status=g1.status, wait_ns=g1.wait_ns,
                      partial_floats=g1.partial_floats, max_tiles=g1.max_tiles)
        f["a1"] = _lib.GemmArgs(b_base=f["xq"].data_ptr(), b_pitch=H, b_index=self.entry_row.data_ptr(),
                                split_word=_lib.PLAN_SPLIT1, m_blocks=I // 128, k_blocks=H // 128, rows_per_expert=2 * I,
                                up_row_offset=I, out=self.act.data_ptr(), out_pitch=I, row_scale=None, counters=g1.counters,
                                n_counters=g1.n_counters, w_scale=None, b_scale=f["xs"].data_ptr(), b_scale_pitch=H // 128,
                                **common)
        f["a2"] = _lib.GemmArgs(b_base=f["aq"].data_ptr(), b_pitch=I, b_index=None, split_word=_lib.PLAN_SPLIT2,
                                m_blocks=H // 128, k_blocks=I // 128, rows_per_expert=H, up_row_offset=0,
                                out=self.y.data_ptr(), out_pitch=H, row_scale=self.entry_w.data_ptr(), counters=g2.counters,
                                n_counters=g2.n_counters, w_scale=None, b_scale=f["as"].data_ptr(), b_scale_pitch=I // 128,
                                **common)
        if bool(self.gemm_kwargs.get("b_tma", True)):
            from .ops.kernels import make_tile_tmap

            f["tm_aq"] = make_tile_tmap(f["aq"], self.block_m)  # the down GEMM reads its e4m3 token tiles by TMA
            f["a2"].b_tmap = C.addressof(f["tm_aq"])
        self._fp8_shared = f
        return f

    def bind_weights_fp8(self, pack: dict) -> None:
        """Point this (possibly shared) buffer set at one MoE layer's e4m3 weights; no copies."""
        if pack.get("expand"):
            e = self._expanded_weights()
            self._fp8, self._expand = None, pack
            self.w13, self.w2, self._tmap13, self._tmap2 = e["w13"], e["w2"], e["tm13"], e["tm2"]
            return
        self._expand = None
        f = self._fp8_buffers()
        f["a1"].w_scale, f["a2"].w_scale = pack["s13"].data_ptr(), pack["s2"].data_ptr()
        f["tm13"], f["tm2"], f["pack"] = pack["tm13"], pack["tm2"], pack
        self._fp8 = f
        self.w13, self.w2 = pack["w13"], pack["w2"]
        self._tmap13, self._tmap2 = pack["tm13"], pack["tm2"]

    def make_weight_maps(self, w13_local: torch.Tensor, w2_local: torch.Tensor):
        """TMA descriptors for a weight pair (build once per MoE layer, then pass to ``bind_weights``)."""
        if self.backend != "cuda":
            return None, None
        from .ops.kernels import make_weight_tmap

        return make_weight_tmap(w13_local), make_weight_tmap(w2_local)

    def bind_weights(self, w13_local: torch.Tensor, w2_local: torch.Tensor, tmap13=None, tmap2=None) -> None:
        """Point this (possibly shared) buffer set at one MoE layer's expert weights; no copies."""
        if self.backend != "cuda":
            self.w13, self.w2 = w13_local, w2_local
            return
        if tmap13 is None or tmap2 is None:
            self.set_weights(w13_local, w2_local)
            return
        self._fp8 = self._expand = None
        self.w13, self.w2, self._tmap13, self._tmap2 = w13_local, w2_local, tmap13, tmap2

    def _cuda_dispatch(self, x, weights, ids, num_valid, logits=None, bias=None) -> torch.Tensor:
        from .ops import _lib

        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("x must be contiguous bf16")
        a = self._a_dispatch
        if logits is not None:
            if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.shape[1] != self.cfg.n_routed_experts:
                raise ValueError("logits must be contiguous fp32 [T, E]")
            if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous()):
                raise ValueError("bias must be contiguous fp32 [E]")
            a.logits, a.bias = logits.data_ptr(), None if bias is None else bias.data_ptr()
            a.weights = a.ids = None
        else:
            if ids.dtype != torch.int32:
                ids = ids.to(torch.int32)
            weights = weights.to(torch.float32).contiguous()
            ids = ids.contiguous()
            a.logits = a.bias = None
            a.weights, a.ids = weights.data_ptr(), ids.data_ptr()
        a.x = x.data_ptr()
        a.num_valid = None if num_valid is None else num_valid.data_ptr()
        a.T = x.shape[0]
        self._keep = [x, weights, ids, num_valid, logits, bias]
        _lib.check(self._lib.mf_dispatch_push(C.byref(a), _lib.stream_ptr()), "dispatch_push")
        return self.hit

    def _cuda_meta(self) -> None:
        from .ops import _lib

        _lib.check(self._lib.mf_expert_meta(C.byref(self._a_meta), _lib.stream_ptr()), "expert_meta")

    def _cuda_experts(self, stop_after: str | None = None) -> None:
        from .ops import _lib

        if self._tmap13 is None:
            raise RuntimeError("no expert weights bound (set_weights)")
        s = _lib.stream_ptr()
        if self._expand is not None:
            # before the metadata kernel: the expansion depends on nothing of this forward
            p, lib = self._expand, self._lib
            _lib.check(lib.mf_dequant_block_fp8(p["w13"].data_ptr(), p["s13"].data_ptr(), self.w13.data_ptr(),
                                                self.L * 2 * self.I, self.H, s), "expand e4m3 gate/up weights")
            _lib.check(lib.mf_dequant_block_fp8(p["w2"].data_ptr(), p["s2"].data_ptr(), self.w2.data_ptr(),
                                                self.L * self.H, self.I, s), "expand e4m3 down weights")
        self._cuda_meta()
        if stop_after == "META":
            return
        if self._fp8 is not None:
            f, lib = self._fp8, self._lib
            valid_off = self.H * 2 + 2 * self.K * 4  # byte offset of a received row's valid flag
            _lib.check(lib.mf_quant_rows_1x128(self._recv_store.data_ptr(), self.pitch * 2, None, self.world * self.C, self.H,
                                               f["xq"].data_ptr(), f["xs"].data_ptr(), valid_off, None, s), "quantise rows")
            _lib.check(lib.mf_gemm_gate_up_fp8(f["tm13"], C.byref(f["a1"]), self.block_m, self.n_sms, s), "fp8 gate/up gemm")
            if stop_after == "GEMM1":
                return
            entries = self.plan[_lib.PLAN_N_ENTRIES :]
            _lib.check(lib.mf_quant_rows_1x128(self.act.data_ptr(), self.I * 2, None, self.n_entries, self.I, f["aq"].data_ptr(),
                                               f["as"].data_ptr(), -1, entries.data_ptr(), s), "quantise activations")
            _lib.check(lib.mf_gemm_down_fp8(f["tm2"], C.byref(f["a2"]), self.block_m, self.n_sms, s), "fp8 down gemm")
            if stop_after == "GEMM2":
                return
            _lib.check(lib.mf_owner_reduce_push(C.byref(self._a_reduce), s), "owner_reduce_push")
            return
        if self.permute_rows:
            _lib.check(self._lib.mf_permute_rows(self._recv_store.data_ptr(), self.pitch * 2, self.entry_row.data_ptr(),
                                                 self.plan.data_ptr(), self._xg.data_ptr(), self.H, self.world * self.C,
                                                 min(self.n_entries, 8 * self.n_sms), s), "permute rows")
        _lib.check(self._lib.mf_gemm_gate_up(self._tmap13, C.byref(self._a_gemm1), self.block_m, self.n_sms, s), "gate/up gemm")
        if stop_after == "GEMM1":
            return
        _lib.check(self._lib.mf_gemm_down(self._tmap2, C.byref(self._a_gemm2), self.block_m, self.n_sms, s), "down gemm")
        if stop_after == "GEMM2" or self.fuse_return:
            return
        _lib.check(self._lib.mf_owner_reduce_push(C.byref(self._a_reduce), s), "owner_reduce_push")

    def _cuda_push_partials(self, partials: torch.Tensor) -> None:
        """Return path for externally computed partial rows ``[RC, H]``: peer stores + return flags."""
        from .ops import _lib

        if tuple(partials.shape) != (self.world * self.C, self.H) or partials.dtype != torch.bfloat16:
            raise ValueError("partial rows must be bf16 [R*C, H]")
        partials = partials.contiguous()
        self._a_push.y = partials.data_ptr()
        self._keep.append(partials)
        _lib.check(self._lib.mf_owner_reduce_push(C.byref(self._a_push), _lib.stream_ptr()), "return push")

    def _cuda_wait_return(self) -> None:
        """Block the stream until every owner's return flag of this forward has arrived."""
        self._cuda_combine(self.hit)

    def _cuda_combine(self, hit: torch.Tensor) -> torch.Tensor:
        from .ops import _lib

        _lib.check(self._lib.mf_combine(C.byref(self._a_combine), _lib.stream_ptr()), "combine")
        return self.out

    def check_status(self) -> dict:
        """Read the layer's status word (device-to-host; call it outside captured regions)."""
        from .ops import _lib

        if self.backend != "cuda":
            return _lib.decode_status(0)
        return _lib.decode_status(int(self.status.item()))


class _CudaLayout:
    """Offsets inside the symmetric region of one cuda-backend layer."""

    def __init__(self, cfg: MoEConfig, world: int, capacity: int):
        pitch_bytes = row_pitch_lanes(cfg.hidden_size, cfg.top_k, 2) * 2

        def up(n: int, a: int = 1024) -> int:
            return (n + a - 1) // a * a

        self.recv_off = 0
        self.ret_off = up(world * capacity * pitch_bytes)
        self.dflag_off = self.ret_off + up(world * capacity * cfg.hidden_size * 2)
        self.rflag_off = self.dflag_off + up(world * 4, 256)
        self.total = self.rflag_off + up(world * 4, 256)


def choose_block_m(capacity: int, top_k: int, local_experts: int, fp8: bool = False) -> int:
    """Token rows per GEMM tile from the expected rows per expert under even routing (``R * C * K`` entries over
    ``R * L`` experts): 64 for decode, 128 from 36 expected rows, 256 from 80.

    Measured on 72 local experts (whole layer, us, narrower / wider tile): 28 rows 468 / 480, 43 rows 514 / 495,
    57 rows 557 / 505, 85 rows 705 / 583 (64 / 128); 85 rows 588 / 568, 114 rows 663 / 591, 171 rows 854 / 700,
    341 rows 1393 / 1155 (128 / 256).  A wider tile keeps an expert's rows in one tile (one pass over its weights)
    and, at 256 rows, halves the operand bytes per flop that a CTA pulls from L2.

    ``fp8``: the layer will hold block-scaled e4m3 experts.  Their kernels take tiles of up to 128 rows (128 from 96
    expected rows), and 256-row tiles mean expanding the experts to bf16 in every forward, which pays from about
    512 expected rows per expert on.
    """
    expected = (capacity * top_k) / max(local_experts, 1)
    if fp8:
        return 256 if expected >= 512 else 128 if expected >= 96 else 64
    return 256 if expected >= 80 else 128 if expected >= 36 else 64


def choose_meta_ctas(slot_words: int, n_sms: int) -> int:
    """CTAs of the metadata pass for ``rows * K`` received slot words: one up to 8192 (the single CTA then keeps
    every slot word in registers and needs one pass), else one per 128 words up to one per SM."""
    return 1 if slot_words <= 8192 else max(2, min(n_sms, (slot_words + 127) // 128))


def _cuda_ok(cfg: MoEConfig) -> bool:
    from .ops import _lib

    return (
        cfg.hidden_size % 128 == 0 and cfg.moe_intermediate_size % 128 == 0 and cfg.top_k <= 32 and _lib.available()
    )


def combine_partials(ret_recv: torch.Tensor, hit: torch.Tensor, out_dtype, rank: int = 0, mode: str = "fp32"):
    """Source-side merge of ``ret_recv [R, C, H]`` under ``hit [C, R]`` in PyTorch.

    ``fp32``: ascending rank, fp32 accumulator from +0.0, one cast.  ``bf16_ring``: start at the rank
    after ``rank`` and round to bf16 after every add (the arithmetic of a bf16 ring reduce-scatter).
    """
    R = ret_recv.shape[0]
    present = hit.to(torch.bool)
    if mode == "fp32":
        return _ordered_masked_sum(ret_recv.permute(1, 0, 2), present).to(out_dtype)
    acc = torch.zeros(ret_recv.shape[1], ret_recv.shape[2], dtype=torch.float32, device=ret_recv.device)
    for step in range(1, R + 1):
        d = (rank + step) % R
        term = torch.where(present[:, d, None], ret_recv[d].to(torch.float32), 0.0)
        acc = (acc + term).to(torch.bfloat16).to(torch.float32)
    return acc.to(out_dtype)


def simulate_fixed(layers: list[FixedEPLayer], xs, logits, bias, num_valid=None) -> list[torch.Tensor]:
    """All ranks in lock-step inside one process.

    Torch-backend layers exchange by copying ``recv[d][s] = send[s][d]``; cuda-backend layers built on
    ``PeerGroup.local`` regions store into each other directly, so running the stages rank after rank
    is the exchange (every flag is already published when its waiter runs).
    """
    R = len(layers)
    hits = [
        ly.stage_pack(x, lg, bias, None if num_valid is None else num_valid[i])
        for i, (ly, x, lg) in enumerate(zip(layers, xs, logits))
    ]
    if layers[0].backend == "torch":
        for d in range(R):
            for s in range(R):
                layers[d]._recv_store[s].copy_(layers[s]._send_store[d])
    for ly in layers:
        ly.stage_experts()
    if layers[0].backend == "torch":
        for d in range(R):
            for s in range(R):
                layers[d].ret_recv[s].copy_(layers[s].ret_send[d])
    return [ly.stage_combine(h, x.dtype) for ly, h, x in zip(layers, hits, xs)]
