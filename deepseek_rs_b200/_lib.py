"""Loads libdsmoe.so and declares its C ABI (include/dsmoe.h) for ctypes.

There is no CPU fallback: if the library is missing or does not load, importing the kernels fails with the reason.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdsmoe.so")

OK = 0
ERR_ARG, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_BOUNDS, ERR_NOMEM, ERR_STATE = -1, -2, -3, -4, -5, -6, -7
LAYOUT_NATIVE, LAYOUT_ROWSOA = 0, 1
DEBUG_WAIT_LIMIT_KCLOCKS, DEBUG_DROP_ONE_COPY, DEBUG_CLEAR_STATUS = 1, 2, 3


class Config(C.Structure):
    _fields_ = [("n_embd", C.c_uint32), ("n_ff", C.c_uint32), ("n_expert", C.c_uint32),
                ("n_expert_used", C.c_uint32), ("swiglu_clamp", C.c_float), ("route_scale", C.c_float),
                ("f16_ieee", C.c_uint32), ("max_tokens", C.c_uint32), ("max_layers", C.c_uint32)]


_vp, _u32, _u64, _i32, _f32, _int = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_int

# name -> (restype, argtypes); every symbol include/dsmoe.h declares
SIGNATURES = {
    "dsmoe_version": (C.c_char_p, []),
    "dsmoe_default_config": (None, [C.POINTER(Config)]),
    "dsmoe_create": (_int, [C.POINTER(Config), _int, C.POINTER(_vp)]),
    "dsmoe_destroy": (_int, [_vp]),
    "dsmoe_last_error": (C.c_char_p, [_vp]),
    "dsmoe_launch_count": (_u64, [_vp]),
    "dsmoe_set_phase_events": (_int, [_vp, C.POINTER(_vp), _int]),
    "dsmoe_device_status": (_int, [_vp, _vp, C.POINTER(C.c_int)]),
    "dsmoe_q8k_quantize": (_int, [_vp, _vp, _vp, _vp, _u32, _u32]),
    "dsmoe_router_select": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _u32, _u32, _u32, _u32]),
    "dsmoe_gate_up_mid": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64, _u32, _u32, _u32, _u32,
                                 _f32, _int]),
    "dsmoe_down": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64, _u32, _u32, _u32, _u32, _int]),
    "dsmoe_down_sum": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64, _u32, _u32, _u32, _u32, _int]),
    "dsmoe_moe_sum": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32]),
    "dsmoe_moe_sum_indexed": (_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32]),
    "dsmoe_quantize_q8_0": (_int, [_vp, _vp, _vp, _vp, _vp, _u64, _u64]),
    "dsmoe_matmul_q8_0": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64, _u64]),
    "dsmoe_swiglu": (_int, [_vp, _vp, _vp, _vp, _vp, _u64, _f32, _f32]),
    "dsmoe_matmul_f16": (_int, [_vp, _vp, _vp, _vp, _vp, _u64, _u64, _u64]),
    "dsmoe_shared_expert": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _vp]),
    "dsmoe_dequant_iq2xxs": (_int, [_vp, _vp, _vp, _u64, _vp]),
    "dsmoe_dequant_q2k": (_int, [_vp, _vp, _vp, _u64, _vp]),
    "dsmoe_relayout_iq2xxs": (_int, [_vp, _vp, _vp, _vp, _u64, _u32, _int]),
    "dsmoe_relayout_q2k": (_int, [_vp, _vp, _vp, _vp, _u64, _u32, _int]),
    "dsmoe_fp8_quantize": (_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _int]),
    "dsmoe_fp8_linear": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32]),
    "dsmoe_layer_register": (_int, [_vp, _u32, _vp, _vp, _vp, _int]),
    "dsmoe_moe_forward": (_int, [_vp, _vp, _u32, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_expert_ffn": (_int, [_vp, _vp, _u32, _vp, _vp, _vp, _u32, _vp]),
    "dsmoe_moe_forward_host": (_int, [_vp, _u32, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_moe_forward_host_async": (_int, [_vp, _u32, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_host_synchronize": (_int, [_vp]),
    "dsmoe_moe_forward_noalloc": (_int, [_vp, _vp, _vp, _vp, _int, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_noalloc_device_status": (_int, [_vp, _vp]),
    "dsmoe_debug_set": (_int, [_vp, _int, _int]),
}

_lib = None


def load() -> C.CDLL:
    """Returns the loaded library; raises if it has not been built (python -m deepseek_rs_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m deepseek_rs_b200.build`; "
                              "there is no fallback path")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means the library is stale
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
