"""ctypes binding of ``libkeepvq.so`` (declarations in ``include/keepvq.h``).

The library is the only compute path: if it is missing or fails to load, every operator raises.
There is no CPU or eager fallback.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

import torch

LIBRARY_PATH = Path(__file__).resolve().parent / "libkeepvq.so"

F32, F16, BF16 = 0, 1, 2
TABLE_PACKED, TABLE_PAIR_PACKED, TABLE_HALF2_PAIRS = 0, 1, 2
NO_RESIDUAL = 0xFFFFFFFF

_DTYPE_TAG = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


class KeepVQError(RuntimeError):
    """A non-zero status from the native library."""


class DecodeArgs(Structure):
    _fields_ = [
        ("codes", c_void_p), ("code_bits", c_int32),
        ("scales", c_void_p), ("scales_dtype", c_int32),
        ("codebook", c_void_p),
        ("rows", c_int64), ("codewords", c_int64), ("groups", c_int64),
        ("out", c_void_p), ("out_dtype", c_int32),
    ]


class MatvecArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("x_dtype", c_int32), ("x_rows", c_int64),
        ("codes", c_void_p), ("code_bits", c_int32),
        ("scales", c_void_p), ("scales_dtype", c_int32),
        ("experts", c_int64), ("out_dim", c_int64), ("in_dim", c_int64), ("groups", c_int64),
        ("codebook", c_void_p), ("codebook_layout", c_int32),
        ("rhs", c_void_p), ("lhs", c_void_p), ("x_div", c_int32), ("routes", c_int64),
        ("res_codes", c_void_p), ("res_scales", c_void_p), ("res_scales_dtype", c_int32),
        ("res_rows", c_int64), ("res_groups", c_int64),
        ("res_table", c_void_p), ("hot_of_slot", c_void_p),
        ("out", c_void_p), ("out_dtype", c_int32),
    ]


class RouterLogitsArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("x_dtype", c_int32), ("router_w", c_void_p), ("router_dtype", c_int32),
        ("tokens", c_int64), ("pool", c_int64), ("hidden", c_int64), ("gate_temp", c_float), ("logits", c_void_p),
    ]


class RoutedTopkArgs(Structure):
    _fields_ = [
        ("logits", c_void_p), ("tokens", c_int64), ("pool", c_int64), ("top_k", c_int32), ("score_func", c_int32),
        ("norm_topk_prob", c_int32), ("route_scale", c_float), ("tau", c_float),
        ("served_bias", c_void_p), ("pool_bias", c_void_p), ("slot_of", c_void_p), ("scores", c_void_p),
        ("served_expert", c_void_p), ("served_slot", c_void_p), ("served_weight", c_void_p),
        ("want", c_void_p), ("want_score", c_void_p), ("admit", c_void_p),
    ]


class ExpertWeights(Structure):
    _fields_ = [
        ("codes", c_void_p), ("scales", c_void_p), ("groups", c_int64),
        ("res_codes", c_void_p), ("res_scales", c_void_p), ("res_groups", c_int64),
    ]


class MoELayerArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("x_dtype", c_int32), ("tokens", c_int64), ("hidden", c_int64), ("inter", c_int64),
        ("router_w", c_void_p), ("router_dtype", c_int32), ("pool", c_int64), ("top_k", c_int32),
        ("score_func", c_int32), ("norm_topk_prob", c_int32), ("gate_temp", c_float), ("route_scale", c_float),
        ("tau", c_float), ("served_bias", c_void_p), ("pool_bias", c_void_p), ("slot_of", c_void_p),
        ("slots", c_int64), ("w1", ExpertWeights), ("w3", ExpertWeights), ("w2", ExpertWeights),
        ("scales_dtype", c_int32), ("codebook", c_void_p), ("res_rows", c_int64), ("res_table", c_void_p),
        ("hot_of_slot", c_void_p), ("swiglu_limit", c_float), ("codebook_all_odd", c_int32),
        ("out", c_void_p), ("served_expert", c_void_p), ("served_slot", c_void_p), ("served_weight", c_void_p),
        ("want", c_void_p), ("want_score", c_void_p), ("admit", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_int64), ("expected_routes", c_int64), ("shared", c_void_p),
    ]


class ResidencyArgs(Structure):
    _fields_ = [
        ("slot_expert", c_void_p), ("slot_of", c_void_p), ("served_bias", c_void_p), ("pool_bias", c_void_p),
        ("last_use", c_void_p), ("free_list", c_void_p), ("cooling", c_void_p), ("reading", c_void_p),
        ("counts", c_void_p), ("stats", c_void_p), ("pool", c_int64), ("slots", c_int64),
        ("want", c_void_p), ("want_score", c_void_p), ("tokens", c_int64), ("top_k", c_int32),
        ("landed", c_void_p), ("call", c_int64), ("step", c_int64), ("tau", c_float), ("route_scale", c_float),
        ("spare", c_int32), ("first_layer", c_int32),
        ("actions", c_void_p), ("action_count", c_void_p), ("max_actions", c_int32),
    ]


class GroupedProjectionArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("x_dtype", c_int32), ("routes", c_int64), ("rhs", c_void_p), ("codes", c_void_p), ("scales", c_void_p),
        ("scales_dtype", c_int32), ("slots", c_int64), ("out_dim", c_int64), ("in_dim", c_int64), ("groups", c_int64),
        ("codebook", c_void_p), ("codebook_all_odd", c_int32), ("out", c_void_p), ("out_dtype", c_int32),
        ("workspace", c_void_p), ("workspace_bytes", c_int64), ("x_div", c_int32),
        ("res_codes", c_void_p), ("res_scales", c_void_p), ("res_rows", c_int64), ("res_groups", c_int64),
        ("res_table", c_void_p), ("hot_of_slot", c_void_p),
    ]


class EpPackArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("row_bytes", c_int64), ("served_expert", c_void_p), ("served_weight", c_void_p),
        ("tokens", c_int64), ("top_k", c_int32), ("world", c_int32), ("experts_per_rank", c_int32), ("capacity", c_int64),
        ("send_x", c_void_p), ("send_meta", c_void_p), ("position", c_void_p),
    ]


class EpPeerArgs(Structure):
    _fields_ = [
        ("world", c_int32), ("rank", c_int32), ("capacity", c_int64), ("row_bytes", c_int64),
        ("recv_x", c_void_p), ("recv_meta", c_void_p), ("back", c_void_p), ("flags", c_void_p), ("epoch", c_void_p), ("status", c_void_p),
        ("wait_spins", ctypes.c_uint32), ("arrivals", c_void_p),
    ]


class EpCombineArgs(Structure):
    _fields_ = [
        ("back", c_void_p), ("dtype", c_int32), ("rows", c_int64), ("hidden", c_int64), ("position", c_void_p),
        ("tokens", c_int64), ("top_k", c_int32), ("out", c_void_p),
    ]


SCORE_FUNCS = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}
STATIC_SCRATCH_BYTES = 8 << 20  # KEEPVQ_STATIC_SCRATCH_BYTES
STAGE_ROUTER, STAGE_PREPARE, STAGE_GATE_UP, STAGE_DOWN, STAGE_COMBINE, STAGE_ALL = 1, 2, 4, 8, 16, 31

#: ctypes mirror of every argument struct in the header, by its C name (the layout test walks this).
EXTRA_STRUCTS = {
    "keepvq_router_logits_args": RouterLogitsArgs, "keepvq_routed_topk_args": RoutedTopkArgs,
    "keepvq_expert_weights": ExpertWeights, "keepvq_moe_layer_args": MoELayerArgs,
    "keepvq_residency_args": ResidencyArgs, "keepvq_grouped_projection_args": GroupedProjectionArgs, "keepvq_ep_pack_args": EpPackArgs, "keepvq_ep_peer_args": EpPeerArgs, "keepvq_ep_combine_args": EpCombineArgs,
}

_SIGNATURES = {
    "keepvq_abi_version": (c_int, []),
    "keepvq_status_string": (c_char_p, [c_int]),
    "keepvq_last_cuda_error": (c_char_p, []),
    "keepvq_decode_weights": (c_int, [POINTER(DecodeArgs), c_void_p]),
    "keepvq_routed_matvec": (c_int, [POINTER(MatvecArgs), c_void_p]),
    "keepvq_router_logits": (c_int, [POINTER(RouterLogitsArgs), c_void_p]),
    "keepvq_routed_topk": (c_int, [POINTER(RoutedTopkArgs), c_void_p]),
    "keepvq_moe_layer_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int64, c_int32]),
    "keepvq_moe_layer_status_offset": (c_int64, [c_int64, c_int64, c_int64, c_int64, c_int32]),
    "keepvq_moe_layer_route_output_offset": (c_int64, [c_int64, c_int64, c_int64, c_int64, c_int32]),
    "keepvq_moe_layer_route_hidden_offset": (c_int64, [c_int64, c_int64, c_int64, c_int64, c_int32]),
    "keepvq_moe_decode_layer": (c_int, [POINTER(MoELayerArgs), c_void_p]),
    "keepvq_moe_decode_stages": (c_int, [POINTER(MoELayerArgs), c_int32, c_void_p]),
    "keepvq_moe_decode_layer_static": (c_int, [POINTER(MoELayerArgs), c_void_p]),
    "keepvq_residency_tick": (c_int, [POINTER(ResidencyArgs), c_void_p]),
    "keepvq_grouped_projection_workspace_bytes": (c_int64, [c_int64, c_int64]),
    "keepvq_grouped_projection_status_offset": (c_int64, [c_int64, c_int64]),
    "keepvq_grouped_projection": (c_int, [POINTER(GroupedProjectionArgs), c_void_p]),
    "keepvq_wait_selftest_workspace_bytes": (c_int64, []),
    "keepvq_wait_selftest": (c_int, [c_void_p, c_int64, c_int64, c_void_p]),
    "keepvq_ep_pack": (c_int, [POINTER(EpPackArgs), c_void_p]),
    "keepvq_ep_combine": (c_int, [POINTER(EpCombineArgs), c_void_p]),
    "keepvq_ep_dispatch_peer": (c_int, [POINTER(EpPackArgs), POINTER(EpPeerArgs), c_void_p]),
    "keepvq_ep_return_peer": (c_int, [c_void_p, POINTER(EpPeerArgs), c_void_p]),
}

_lock = threading.Lock()
_lib = None


def load() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built (``python -m keep_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not LIBRARY_PATH.exists():
                raise KeepVQError(
                    f"{LIBRARY_PATH} is missing: build it with `python -m keep_b200.build` "
                    "(needs nvcc; there is no CPU fallback)"
                )
            lib = ctypes.CDLL(str(LIBRARY_PATH))
            for name, (restype, argtypes) in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = restype, argtypes
            _lib = lib
    return _lib


def exported_names() -> list[str]:
    return sorted(_SIGNATURES)


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        text = lib.keepvq_status_string(status).decode()
        detail = lib.keepvq_last_cuda_error().decode() if status == -6 else ""
        raise KeepVQError(f"{what}: {text} ({status}){': ' + detail if detail else ''}")


def dtype_tag(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_TAG[dtype]
    except KeyError:
        raise ValueError(f"unsupported floating dtype {dtype}") from None


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(None if t is None else t.data_ptr())


def stream_handle(device: torch.device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    """All tensors on one CUDA device; that device is returned.  CPU tensors are refused: the
    operators never compute on the host."""
    device = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KeepVQError("keep_b200 operators need CUDA tensors; there is no CPU path")
        if device is None:
            device = t.device
        elif t.device != device:
            raise ValueError(f"tensors on different devices: {device} and {t.device}")
    if device is None:
        raise KeepVQError("no CUDA tensor given")
    return device
