"""ctypes binding of the C ABI declared in include/b200moe.h.

The shared library is built in-tree by `shark_platform_b200.build`.  There is
no fallback: if the library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
import re
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
# B200MOE_LIB points at another build of the same library (e.g. a diagnostic build)
LIB_PATH = os.environ.get("B200MOE_LIB") or os.path.join(HERE, "lib", "libb200moe.so")
HEADER_PATH = os.path.join(os.path.dirname(HERE), "include", "b200moe.h")

LAYOUT_Q8_0, LAYOUT_Q4_K, LAYOUT_F16 = 0, 1, 2
ACT_SILU, ACT_GELU = 0, 1
DT_F32, DT_F16, DT_BF16 = 0, 1, 2
REGIME_AUTO, REGIME_STREAM, REGIME_TENSOR, REGIME_TENSOR_PAIR = 0, 1, 2, 3


class B200MoeError(RuntimeError):
    pass


class WeightDesc(ctypes.Structure):
    _fields_ = [
        ("layout", c_int32),
        ("experts", c_int32),
        ("rows", c_int32),
        ("cols", c_int32),
        ("qs", c_void_p),
        ("d", c_void_p),
        ("sub", c_void_p),
    ]


class LayerDesc(ctypes.Structure):
    _fields_ = [
        ("hidden", c_int32),
        ("ffn", c_int32),
        ("experts", c_int32),
        ("top_k", c_int32),
        ("activation", c_int32),
        ("rms_epsilon", c_float),
        ("ffn_norm_weight", c_void_p),
        ("router_weight", c_void_p),
        ("router_bias", c_void_p),
        ("layer_output_norm_weight", c_void_p),
        ("gate", WeightDesc),
        ("up", WeightDesc),
        ("down", WeightDesc),
        ("expert_begin", c_int32),
    ]


class KvCacheDesc(ctypes.Structure):
    _fields_ = [
        ("blocks", c_int32),
        ("stride", c_int32),
        ("kv_heads", c_int32),
        ("head_dim", c_int32),
        ("page_count", c_int32),
    ]


class EpDesc(ctypes.Structure):
    _fields_ = [
        ("world", c_int32),
        ("rank", c_int32),
        ("experts_local", c_int32),
        ("counts_all", c_void_p * 16),
        ("flags", c_void_p * 16),
        ("recv_x", c_void_p * 16),
        ("ret_y", c_void_p * 16),
    ]


def declared_symbols() -> list[str]:
    """Names of every function the public header declares."""
    with open(HEADER_PATH) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


if not os.path.exists(LIB_PATH):
    raise B200MoeError(
        f"{LIB_PATH} is missing: build it with `python -m shark_platform_b200.build` "
        "(there is no CPU or eager fallback)"
    )

lib = ctypes.CDLL(LIB_PATH)

_W = POINTER(WeightDesc)
_L = POINTER(LayerDesc)
_P = c_void_p

_PROTOS = {
    "b200moe_version": (c_char_p, []),
    "b200moe_last_error": (c_char_p, []),
    "b200moe_device_status": (c_int, [_P, POINTER(c_int32)]),
    "b200moe_set_wait_limit": (c_int, [c_int64]),
    "b200moe_dequant": (c_int, [_W, c_int, _P, _P]),
    "b200moe_q4k_prepare": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, _P, _P]),
    "b200moe_q8_prepare": (c_int, [_P, c_int64, c_int32, _P, _P]),
    "b200moe_gguf_unpack_q8_0": (c_int, [_P, c_int64, _P, _P, _P]),
    "b200moe_gguf_unpack_q4_k": (c_int, [_P, c_int64, _P, _P, _P, _P, _P, _P, _P, _P]),
    "b200moe_router": (c_int, [_P, c_int, c_int32, _L, _P, _P, _P, _P]),
    "b200moe_front_supported": (c_int, [c_int32, _L]),
    "b200moe_front": (c_int, [_P, c_int, c_int32, _L, c_int, _P, _P, _P, _P, _P, _P, _P, _P]),
    "b200moe_route_plan": (c_int, [_P, c_int32, c_int32, c_int32, _P, _P, _P, _P, _P]),
    "b200moe_permute_rows": (c_int, [_P, _P, _P, c_int32, c_int32, c_int32, c_int32, c_int32, _P, _P]),
    "b200moe_kperm": (c_int, [c_int, c_int, c_int32]),
    "b200moe_gate_up": (c_int, [_P, _P, c_int32, c_int32, _W, _W, c_int, c_int, c_int32, _P, _P]),
    "b200moe_down_ksplit": (c_int, [_W, c_int32, c_int32, c_int]),
    "b200moe_down": (c_int, [_P, _P, c_int32, c_int32, _W, c_int, c_int32, _P, _P]),
    "b200moe_down_noalloc": (c_int, [_P, _P, c_int32, c_int32, _W, _P, _P]),
    "b200moe_combine": (c_int, [_P, c_int, c_int32, c_int32, _P, _P, _P, c_int, c_int32, _L, c_int, _P, c_int, _P]),
    "b200moe_exchange_plan": (c_int, [_P, c_int32, c_int32, _P, _P, _P, _P]),
    "b200moe_gather_rows": (c_int, [_P, _P, c_int32, c_int32, c_int32, _P, _P]),
    "b200moe_ep_publish_counts": (c_int, [POINTER(EpDesc), _P, _P]),
    "b200moe_ep_barrier": (c_int, [POINTER(EpDesc), c_int32, _P, _P]),
    "b200moe_ep_dispatch": (c_int, [POINTER(EpDesc), _P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, c_int32, _P]),
    "b200moe_ep_return": (c_int, [POINTER(EpDesc), _P, c_int32, c_int32, _P, c_int32, c_int32, _P]),
    "b200moe_ep_workspace_bytes": (c_size_t, [_L, c_int32, c_int32, c_int32]),
    "b200moe_ep_layer_forward": (c_int, [_L, POINTER(EpDesc), _P, _P, c_int, c_int32, c_int, c_int32, c_int32,
                                         c_int32, c_int32, c_int32, _P, c_size_t, _P]),
    "b200moe_workspace_bytes": (c_size_t, [_L, c_int32]),
    "b200moe_layer_forward": (c_int, [_L, _P, _P, c_int, c_int32, c_int, _P, c_size_t, _P, _P, _P]),
    "b200moe_layer_forward_host": (c_int, [_L, _P, _P, c_int, c_int32, c_int, _P, _P, c_size_t, _P]),
    "b200moe_rms_norm": (c_int, [_P, c_int, _P, c_int64, c_int32, c_float, _P, c_int, _P]),
    "b200moe_attn_rope_kv_write": (c_int, [_P, _P, _P, _P, _P, c_int, _P, c_int, POINTER(KvCacheDesc), c_int32, _P, _P,
                                           _P, c_int32, c_int32, c_int32, c_int32, _P]),
    "b200moe_attn_decode_scratch_bytes": (c_size_t, [POINTER(KvCacheDesc), c_int32, c_int32, c_int32]),
    "b200moe_attn_decode": (c_int, [_P, c_int, _P, c_int, POINTER(KvCacheDesc), c_int32, _P, _P, c_int32, c_int32,
                                    c_int32, c_int32, c_float, c_float, _P, c_int, _P, c_size_t, _P]),
    "b200moe_pipeline_bytes": (c_size_t, [_L, c_int, c_int32, c_int32]),
    "b200moe_pipeline_create": (c_int, [_L, c_int, c_int32, c_int, c_int32, _P, c_size_t, POINTER(c_void_p)]),
    "b200moe_pipeline_submit": (c_int, [_P, _P, _P, c_int32, _P]),
    "b200moe_pipeline_drain": (c_int, [_P]),
    "b200moe_pipeline_destroy": (c_int, [_P]),
    "b200moe_set_token_tile": (c_int, [c_int32]),
    "b200moe_set_stream_wide": (c_int, [c_int32]),
    "b200moe_trace_enable": (c_int, [c_int]),
    "b200moe_trace_read": (c_int, [POINTER(c_int64), c_size_t]),
    "b200moe_profile_enable": (c_int, [c_int]),
    "b200moe_profile_read": (c_int, [POINTER(c_float), POINTER(c_int32)]),
}

for _name, (_res, _args) in _PROTOS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.b200moe_last_error().decode()


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        raise B200MoeError(f"{what or 'b200moe call'} failed ({rc}): {last_error()}")
