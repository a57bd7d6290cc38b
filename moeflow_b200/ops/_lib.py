"""ctypes binding of libmoeflow_b200.so (the sm_100a kernels and the peer-memory runtime).

The library is built in-tree by ``moeflow_b200.build``.  On a machine with a GPU a missing or
unloadable library is an error (never a silent PyTorch fallback); on a CPU-only machine the CUDA ops
are simply unavailable and ``available()`` is False.
"""

from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libmoeflow_b200.so"

PLAN_N_TILES, PLAN_SPLIT1, PLAN_SPLIT2, PLAN_N_ENTRIES, PLAN_SLOT_COLS, PLAN_VALID_ROWS, PLAN_WORDS = 0, 1, 2, 3, 4, 5, 8

STATUS_NAMES = {
    0: "ok",
    1: "dispatch flag wait ran out",
    2: "return flag wait ran out",
    3: "gemm: operand tiles never arrived",
    4: "gemm: no free pipeline stage",
    5: "gemm: accumulator hand-off ran out",
    6: "gemm: tensor memory",
    7: "bad argument",
    8: "peer ping wait ran out",
}


class GemmArgs(C.Structure):
    _fields_ = [
        ("b_base", C.c_void_p),
        ("b_pitch", C.c_longlong),
        ("b_index", C.c_void_p),
        ("tile_e", C.c_void_p),
        ("tile_s", C.c_void_p),
        ("tile_n", C.c_void_p),
        ("plan", C.c_void_p),
        ("split_word", C.c_int),
        ("m_blocks", C.c_int),
        ("k_blocks", C.c_int),
        ("rows_per_expert", C.c_int),
        ("up_row_offset", C.c_int),
        ("out", C.c_void_p),
        ("out_pitch", C.c_longlong),
        ("row_scale", C.c_void_p),
        ("partial", C.c_void_p),
        ("counters", C.c_void_p),
        ("max_split_slots", C.c_int),
        ("limit", C.c_float),
        ("round_h", C.c_int),
        ("status", C.c_void_p),
        ("wait_ns", C.c_ulonglong),
        ("w_scale", C.c_void_p),
        ("b_scale", C.c_void_p),
        ("b_scale_pitch", C.c_longlong),
        ("out_scale", C.c_void_p),
        ("trace", C.c_void_p),
        ("ret_peer", C.c_void_p),
        ("ret_flag", C.c_void_p),
        ("ret_epoch", C.c_void_p),
        ("ret_done", C.c_void_p),
        ("row_cnt", C.c_void_p),
        ("row_hits", C.c_void_p),
        ("entry_row", C.c_void_p),
        ("inv", C.c_void_p),
        ("ret_rank", C.c_int),
        ("ret_R", C.c_int),
        ("ret_C", C.c_int),
        ("ret_K", C.c_int),
        ("b_tmap", C.c_void_p),
        ("partial_floats", C.c_longlong),
        ("n_counters", C.c_int),
        ("max_tiles", C.c_int),
        ("out_fp32", C.c_int),
        ("out_cols", C.c_int),
        ("tile_done", C.c_void_p),
        ("tile_wait", C.c_void_p),
        ("tile_wait_target", C.c_int),
        ("two_blocks", C.c_int),
    ]


class DispatchArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p),
        ("weights", C.c_void_p),
        ("ids", C.c_void_p),
        ("num_valid", C.c_void_p),
        ("peer_recv", C.c_void_p),
        ("peer_flag", C.c_void_p),
        ("hit", C.c_void_p),
        ("epoch", C.c_void_p),
        ("done_counter", C.c_void_p),
        ("T", C.c_int),
        ("C", C.c_int),
        ("H", C.c_int),
        ("K", C.c_int),
        ("R", C.c_int),
        ("L", C.c_int),
        ("rank", C.c_int),
        ("pitch", C.c_longlong),
        ("skip_payload", C.c_int),
        ("logits", C.c_void_p),
        ("bias", C.c_void_p),
        ("route_w", C.c_void_p),
        ("route_ids", C.c_void_p),
        ("E", C.c_int),
        ("n_group", C.c_int),
        ("topk_group", C.c_int),
        ("sigmoid", C.c_int),
        ("renorm", C.c_int),
        ("scale", C.c_float),
        ("trace", C.c_void_p),
    ]


class MetaArgs(C.Structure):
    _fields_ = [
        ("recv", C.c_void_p),
        ("pitch", C.c_longlong),
        ("H", C.c_int),
        ("K", C.c_int),
        ("L", C.c_int),
        ("rows", C.c_int),
        ("R", C.c_int),
        ("flags", C.c_void_p),
        ("epoch", C.c_void_p),
        ("offsets", C.c_void_p),
        ("entry_row", C.c_void_p),
        ("entry_slot", C.c_void_p),
        ("entry_w", C.c_void_p),
        ("inv", C.c_void_p),
        ("tile_e", C.c_void_p),
        ("tile_s", C.c_void_p),
        ("tile_n", C.c_void_p),
        ("plan", C.c_void_p),
        ("counters1", C.c_void_p),
        ("n_counters1", C.c_int),
        ("counters2", C.c_void_p),
        ("n_counters2", C.c_int),
        ("block_m", C.c_int),
        ("max_tiles", C.c_int),
        ("m_blocks1", C.c_int),
        ("k_blocks1", C.c_int),
        ("m_blocks2", C.c_int),
        ("k_blocks2", C.c_int),
        ("n_sms", C.c_int),
        ("max_split_slots", C.c_int),
        ("status", C.c_void_p),
        ("wait_ns", C.c_ulonglong),
        ("partial_floats", C.c_longlong),
        ("row_hits", C.c_void_p),
        ("n_ctas", C.c_int),
        ("cta_hist", C.c_void_p),
        ("acc", C.c_void_p),
        ("stream_k", C.c_int),
        ("trace", C.c_void_p),
        ("late_launch", C.c_int),
        ("plain_launch", C.c_int),
    ]


class ReducePushArgs(C.Structure):
    _fields_ = [
        ("y", C.c_void_p),
        ("inv", C.c_void_p),
        ("recv", C.c_void_p),
        ("pitch", C.c_longlong),
        ("peer_ret", C.c_void_p),
        ("peer_flag", C.c_void_p),
        ("epoch", C.c_void_p),
        ("done_counter", C.c_void_p),
        ("R", C.c_int),
        ("C", C.c_int),
        ("H", C.c_int),
        ("K", C.c_int),
        ("rank", C.c_int),
        ("valid_word", C.c_int),
        ("push_epoch", C.c_void_p),
        ("trace", C.c_void_p),
    ]


class CombineArgs(C.Structure):
    _fields_ = [
        ("ret", C.c_void_p),
        ("hit", C.c_void_p),
        ("out", C.c_void_p),
        ("flags", C.c_void_p),
        ("epoch", C.c_void_p),
        ("R", C.c_int),
        ("C", C.c_int),
        ("H", C.c_int),
        ("rank", C.c_int),
        ("ring", C.c_int),
        ("status", C.c_void_p),
        ("wait_ns", C.c_ulonglong),
        ("trace", C.c_void_p),
    ]


class NativeLibraryError(RuntimeError):
    pass


def available() -> bool:
    """True when the native library can be used (built and a CUDA device is present)."""
    import torch

    return LIB_PATH.exists() and torch.cuda.is_available()


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    """Load the library, building it first when the sources changed and nvcc is present."""
    if not LIB_PATH.exists():
        from ..build import build

        build()
    try:
        handle = C.CDLL(str(LIB_PATH))
    except OSError as exc:  # pragma: no cover - depends on the machine
        raise NativeLibraryError(f"cannot load {LIB_PATH}: {exc}") from exc
    P, I, LL, ULL, F = C.c_void_p, C.c_int, C.c_longlong, C.c_ulonglong, C.c_float
    sigs = {
        "mf_make_weight_tmap": [P, P, LL, LL, I],
        "mf_make_tile_tmap": [P, P, LL, LL, I, I],
        "mf_gemm_gate_up": [P, C.POINTER(GemmArgs), I, I, P],
        "mf_gemm_down": [P, C.POINTER(GemmArgs), I, I, P],
        "mf_gemm_smem_bytes": [I, I],
        "mf_gemm_gate_up_fp8": [P, C.POINTER(GemmArgs), I, I, P],
        "mf_gemm_down_fp8": [P, C.POINTER(GemmArgs), I, I, P],
        "mf_quant_rows_1x128": [P, LL, P, I, I, P, P, LL, P, P],
        "mf_dequant_block_fp8": [P, P, P, LL, I, P],
        "mf_router_topk": [P, P, P, P, I, I, I, I, I, I, I, F, P],
        "mf_rmsnorm": [P, P, P, I, I, F, P],
        "mf_dispatch_push": [C.POINTER(DispatchArgs), P],
        "mf_expert_meta": [C.POINTER(MetaArgs), P],
        "mf_plan_split": [I, I, I, I, I, I],
        "mf_permute_rows": [P, LL, P, P, P, I, I, I, P],
        "mf_owner_reduce_push": [C.POINTER(ReducePushArgs), P],
        "mf_combine": [C.POINTER(CombineArgs), P],
        "mf_expert_prepare": [P, LL, I, I, I, I, I, P, P, P, P, P],
        "mf_peer_alloc": [C.POINTER(P), ULL],
        "mf_peer_free": [P],
        "mf_peer_export": [P, P],
        "mf_peer_open": [P, C.POINTER(P)],
        "mf_peer_close": [P],
        "mf_peer_can_access": [I, I, C.POINTER(I)],
        "mf_peer_ping": [P, P, I, I, C.c_uint, I, P, ULL, P],
        "mf_device_sm_count": [C.POINTER(I)],
    }
    for name, argtypes in sigs.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = I
    handle.mf_set_pdl.argtypes = [I]
    handle.mf_set_pdl.restype = None
    handle.mf_pdl_enabled.argtypes = []
    handle.mf_pdl_enabled.restype = I
    handle.mf_error_string.argtypes = [I]
    handle.mf_error_string.restype = C.c_char_p
    return handle


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().mf_error_string(code).decode() if code > 0 else f"bad argument ({code})"
        raise NativeLibraryError(f"{what} failed: {msg}")


def ptr(t) -> int | None:
    """Device address of a tensor (None stays None)."""
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def decode_status(word: int) -> dict:
    code = word & 0xFF
    return {
        "code": code,
        "name": STATUS_NAMES.get(code, "unknown"),
        "who": (word >> 8) & 0xFF,
        "detail": (word >> 16) & 0xFFFF,
        "epoch": (word >> 32) & 0xFFFFFFFF,
    }
