"""ctypes view of include/pmoe.h."""
from __future__ import annotations

import ctypes as C
import os

F32, F16, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 8, 10, 11, 12, 13, 14, 30
TRACE_PHASES = 8

STATUS_NAMES = {
    0: "PMOE_OK", -1: "PMOE_ERR_INVALID_ARG", -2: "PMOE_ERR_UNSUPPORTED_DTYPE",
    -3: "PMOE_ERR_UNSUPPORTED_SHAPE", -4: "PMOE_ERR_CUDA", -5: "PMOE_ERR_TOO_MANY_TOKENS",
    -6: "PMOE_ERR_TRAINING_MODE", -7: "PMOE_ERR_TIMEOUT", -8: "PMOE_ERR_BAD_INDEX", -9: "PMOE_ERR_NO_DEVICE",
}


class PmoeError(RuntimeError):
    """A libpmoe call returned a negative status (the analogue of candle::Error::Msg)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


class LayerDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("device", C.c_int32),
        ("H", C.c_int32), ("F", C.c_int32), ("E", C.c_int32), ("k", C.c_int32),
        ("max_tokens", C.c_int32),
        ("expert_base", C.c_int32), ("E_local", C.c_int32),
        ("gate_dtype", C.c_int32), ("up_dtype", C.c_int32), ("down_dtype", C.c_int32),
        ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
        ("has_shared", C.c_int32),
        ("sh_gate_dtype", C.c_int32), ("sh_up_dtype", C.c_int32), ("sh_down_dtype", C.c_int32),
        ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p),
        ("sh_gate_inp", C.c_void_p),
        ("router_dtype", C.c_int32), ("router_w", C.c_void_p), ("router_bias", C.c_void_p),
        ("weights_location", C.c_int32), ("training_mode", C.c_int32),
        ("ep_placement", C.c_int32), ("ep_rank", C.c_int32), ("ep_size", C.c_int32),
    ]


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "libpmoe.so")


_lib = None

# every symbol include/pmoe.h declares: (name, restype, argtypes)
_V, _I, _Z = C.c_void_p, C.c_int, C.c_size_t
SYMBOLS = [
    ("pmoe_layer_create", _I, [C.POINTER(LayerDesc), C.POINTER(_V)]),
    ("pmoe_layer_destroy", _I, [_V]),
    ("pmoe_forward", _I, [_V, _V, _I, _I, _V, _I, _V, _V, _V, _V]),
    ("pmoe_forward_host", _I, [_V, _V, _I, _I, _V, _I, _V, _V, _V, _V]),
    ("pmoe_route", _I, [_V, _V, _I, _I, _V, _V, _V, _V]),
    ("pmoe_router_stats", _I, [_V, _V, _V, _I, _I, _V, _V, _V]),
    ("pmoe_experts_forward", _I, [_V, _V, _I, _V, _V, _I, _I, _V, _I, _V]),
    ("pmoe_experts_forward_ep", _I, [_V, _V, _I, _V, _V, _I, _I, _I, _I, _V, _I, _V]),
    ("pmoe_layer_set_block_multipliers", _I, [_V, _V, _V, _V, _V]),
    ("pmoe_layer_set_shared_scales", _I, [_V, _V, _V, _V, _V]),
    ("pmoe_modify_block_scales", _I, [_I, _I, _V, _Z, _V, _V, _V]),
    ("pmoe_ep_unique_id", _I, [_V, _Z]),
    ("pmoe_ep_comm_create", _I, [_V, _Z, _I, _I, _I, C.POINTER(_V)]),
    ("pmoe_ep_comm_adopt", _I, [_V, _I, _I, _I, C.POINTER(_V)]),
    ("pmoe_ep_comm_destroy", _I, [_V]),
    ("pmoe_ep_forward", _I, [_V, _V, _V, _I, _I, _V, _I, _V, _V, _V, _I, _V]),
    ("pmoe_ep_profile", _I, [_V, _I, _V, _V]),
    ("pmoe_shared_forward", _I, [_V, _V, _I, _I, _V, _I, _V]),
    ("pmoe_qmatmul", _I, [_I, _I, _V, _Z, _Z, _V, _Z, _V, _V]),
    ("pmoe_qmatmul_noalloc", _I, [_I, _I, _V, _Z, _Z, _V, _Z, _V, _V]),
    ("pmoe_dequantize", _I, [_I, _I, _V, _Z, _V, _V]),
    ("pmoe_reduce_rows", _I, [_I, _V, _I, _V, _I, _I, _I, _V, _I, _V]),
    ("pmoe_add_rms_norm", _I, [_I, _V, _V, _V, _I, _I, C.c_float, _V, _V, _V]),
    ("pmoe_layer_status", _I, [_V, _V]),
    ("pmoe_layer_trace", _I, [_V, _I]),
    ("pmoe_layer_trace_read", _I, [_V, _V]),
    ("pmoe_trace_phase_name", C.c_char_p, [_I]),
    ("pmoe_launch_count", C.c_uint64, []),
    ("pmoe_block_size", _Z, [_I]),
    ("pmoe_type_size", _Z, [_I]),
    ("pmoe_last_error", C.c_char_p, []),
    ("pmoe_version", _I, []),
]


def lib():
    """Loads libpmoe.so; raises ImportError when the CUDA library has not been built."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `make -C paramecia_b200/csrc` "
                "(or __graft_entry__.build()); there is no CPU fallback")
        L = C.CDLL(path)
        for name, res, args in SYMBOLS:
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int):
    if rc != 0:
        raise PmoeError(rc, lib().pmoe_last_error().decode())


def launch_count() -> int:
    return int(lib().pmoe_launch_count())


def block_size(dtype: int) -> int:
    return int(lib().pmoe_block_size(dtype))


def type_size(dtype: int) -> int:
    return int(lib().pmoe_type_size(dtype))


def row_bytes(dtype: int, cols: int) -> int:
    return cols // block_size(dtype) * type_size(dtype)
