"""Tensor helpers of the vLLM runner.  No vLLM imports: everything here is unit-testable on CPU.

Counterpart of ``moeflow/integrations/vllm_runner_ops.py:10-65`` and of the received-row unpacking in
``moeflow/kernels/expert_prepare.py:10-75``.
"""

from __future__ import annotations

from functools import partial

import torch


def filler_expert(rank_offset: int, num_experts: int) -> int:
    """An expert id this rank does not own: the last expert for the first rank, expert 0 otherwise."""
    return num_experts - 1 if rank_offset == 0 else 0


def local_to_global_ids(local_ids: torch.Tensor, weights: torch.Tensor, rank_offset: int, num_experts: int):
    """Per-rank local expert ids (-1 = no hit) -> global ids for a local fused-experts call.

    Empty slots are pointed at an expert that lives on another rank, so that the expert map of the
    local kernel turns them into "skip"; their weight is forced to zero.
    """
    empty = local_ids < 0
    gids = torch.where(empty, filler_expert(rank_offset, num_experts), local_ids + rank_offset)
    return gids, torch.where(empty, 0.0, weights).to(weights.dtype)


def prepare_expert_inputs(rows: torch.Tensor, hidden_size: int, top_k: int, rank_offset: int, num_experts: int,
                          ids_dtype: torch.dtype = torch.int32):
    """Unpack received rows ``[N, >= H + meta]`` into ``(hidden [N, H], global ids [N, K], weights [N, K])``.

    Slots that are empty, and all slots of rows whose valid flag is 0, get the filler expert and weight
    0, so garbage (NaN) in the hidden lanes or weights of such rows never reaches an output.
    """
    n = rows.shape[0]
    if rows.is_cuda and rows.dtype == torch.bfloat16 and rows.stride(1) == 1 and ids_dtype in (torch.int32, torch.int64):
        from ..ops import _lib

        if _lib.available() and (rows.stride(0) * 2) % 16 == 0 and rows.data_ptr() % 16 == 0:
            # one sm_100a kernel instead of a chain of PyTorch ops
            hidden = torch.empty(n, hidden_size, dtype=torch.bfloat16, device=rows.device)
            gids = torch.empty(n, top_k, dtype=ids_dtype, device=rows.device)
            weights = torch.empty(n, top_k, dtype=torch.float32, device=rows.device)
            is32 = ids_dtype == torch.int32
            _lib.check(
                _lib.lib().mf_expert_prepare(rows.data_ptr(), rows.stride(0) * 2, n, hidden_size, top_k, rank_offset,
                                             filler_expert(rank_offset, num_experts), hidden.data_ptr(),
                                             gids.data_ptr() if is32 else None, None if is32 else gids.data_ptr(),
                                             weights.data_ptr(), _lib.stream_ptr()),
                "expert_prepare",
            )
            return hidden, gids, weights
    lanes = (4 * (2 * top_k + 1) + rows.element_size() - 1) // rows.element_size()
    meta = rows[:, hidden_size : hidden_size + lanes].contiguous().view(torch.int32)[:, : 2 * top_k + 1]
    valid = meta[:, 2 * top_k] != 0
    local = meta[:, :top_k]
    live = valid[:, None] & (local >= 0)
    gids = torch.where(live, local + rank_offset, filler_expert(rank_offset, num_experts)).to(ids_dtype)
    weights = torch.where(live, meta[:, top_k : 2 * top_k].contiguous().view(torch.float32), 0.0)
    del n
    return rows[:, :hidden_size].contiguous(), gids, weights


def combine_bf16_ring(partials: torch.Tensor, hit: torch.Tensor, rank: int) -> torch.Tensor:
    """Sum ``partials [R, T, H]`` in the order ``rank+1, rank+2, ...`` (mod R), rounding to bf16 after
    every add: the arithmetic of a bf16 ring reduce-scatter that ends on ``rank``.  Opt-in: other
    collective algorithms round in other orders."""
    if partials.dtype != torch.bfloat16:
        raise ValueError("BF16 Ring combine requires BF16 partials")
    world = partials.shape[0]
    if not 0 <= rank < world:
        raise ValueError("Source rank is outside the partials")
    present = hit.to(torch.bool)
    acc = torch.zeros_like(partials[0])
    for step in range(1, world + 1):
        owner = (rank + step) % world
        term = torch.where(present[:, owner, None], partials[owner], torch.zeros_like(partials[owner]))
        acc = (acc.to(torch.float32) + term.to(torch.float32)).to(torch.bfloat16)
    return acc


def combine_bf16_ring_fused(partials: torch.Tensor, hit: torch.Tensor, rank: int, out: torch.Tensor | None = None):
    """Same arithmetic in one sm_100a kernel launch (``mf_combine`` with the ring order)."""
    import ctypes as C

    from ..ops import _lib

    if partials.dtype != torch.bfloat16 or not partials.is_cuda or not partials.is_contiguous():
        raise ValueError("BF16 Ring combine requires contiguous CUDA BF16 partials")
    world, tokens, hidden = partials.shape
    if not 0 <= rank < world:
        raise ValueError("Source rank is outside the partials")
    out = out if out is not None else torch.empty(tokens, hidden, dtype=torch.bfloat16, device=partials.device)
    hit_u8 = hit if hit.dtype == torch.uint8 else hit.to(torch.uint8)
    hit_u8 = hit_u8.contiguous()
    if tokens:
        args = _lib.CombineArgs(ret=partials.data_ptr(), hit=hit_u8.data_ptr(), out=out.data_ptr(), flags=None, epoch=None,
                                R=world, C=tokens, H=hidden, rank=rank, ring=1, status=None, wait_ns=0)
        _lib.check(_lib.lib().mf_combine(C.byref(args), _lib.stream_ptr()), "ring combine")
        out._keep = hit_u8
    return out


def make_combine_fn(mode: str, rank: int):
    """Adapter combine for the bf16 ring modes; ``None`` keeps the layer's own fp32 combine."""
    if mode == "fp32":
        return None
    if mode == "bf16_ring":
        return partial(combine_bf16_ring, rank=rank)
    if mode == "bf16_ring_fused":
        return partial(combine_bf16_ring_fused, rank=rank)
    raise ValueError("combine mode must be fp32, bf16_ring or bf16_ring_fused")


def make_prepare_fn(cfg, rank_offset: int, num_experts: int, ids_dtype: torch.dtype):
    """Received-row unpacking bound to this rank's expert range."""
    return partial(prepare_expert_inputs, hidden_size=cfg.hidden_size, top_k=cfg.top_k, rank_offset=rank_offset,
                   num_experts=num_experts, ids_dtype=ids_dtype)


def fixed_capacity(local_tokens: int, tokens_across_dp, max_tokens: int) -> int | None:
    """Capacity of the fixed path for this step, or ``None`` when the step must use the native path.

    ``tokens_across_dp`` is the host-side list/tensor of token counts of all DP ranks (identical on
    every rank, so every rank takes the same branch).  The capacity is the next power of two that
    holds the largest count.
    """
    largest = local_tokens if tokens_across_dp is None else int(max(int(v) for v in tokens_across_dp))
    if largest > max_tokens:
        return None
    need = max(largest, local_tokens, 1)
    cap = 1
    while cap < need:
        cap *= 2
    return cap


def compare_routing(ids, w, other_ids, other_w) -> dict:
    """Two routers may order slots differently: compare per token as {expert: weight} maps."""
    n = ids.shape[0]
    if n == 0:
        return {"intercepted": True, "tokens": 0}
    a_sorted, a_order = ids.to(torch.int64).sort(dim=-1)
    b_sorted, b_order = other_ids.to(torch.int64).sort(dim=-1)
    same = (a_sorted == b_sorted).all(dim=-1)
    diff = (w.float().gather(1, a_order) - other_w.float().gather(1, b_order)).abs()[same]
    return {
        "intercepted": True,
        "tokens": n,
        "token_expert_set_match": same.float().mean().item(),
        "max_abs_weight_diff_on_match": diff.max().item() if diff.numel() else None,
    }
