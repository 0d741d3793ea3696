"""Loads libdsmoe.so and declares its C ABI (include/dsmoe.h) for ctypes.

There is no CPU fallback: if the library is missing or does not load, importing the kernels fails with the reason.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# DSMOE_CHECKED_BUILD=1 loads the checked variant (python -m deepseek_rs_b200.build --bounds) instead
LIB_PATH = os.path.join(HERE, "libdsmoe_bounds.so" if os.environ.get("DSMOE_CHECKED_BUILD") == "1" else "libdsmoe.so")

OK = 0
ERR_ARG, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_BOUNDS, ERR_NOMEM, ERR_STATE = -1, -2, -3, -4, -5, -6, -7
LAYOUT_NATIVE, LAYOUT_ROWSOA = 0, 1
DEBUG_WAIT_LIMIT_KCLOCKS, DEBUG_DROP_ONE_COPY, DEBUG_CLEAR_STATUS = 1, 2, 3


class Config(C.Structure):
    _fields_ = [("n_embd", C.c_uint32), ("n_ff", C.c_uint32), ("n_expert", C.c_uint32),
                ("n_expert_used", C.c_uint32), ("swiglu_clamp", C.c_float), ("route_scale", C.c_float),
                ("f16_ieee", C.c_uint32), ("max_tokens", C.c_uint32), ("max_layers", C.c_uint32)]


class FfnArgs(C.Structure):
    """dsmoe_ffn_args of include/dsmoe.h."""
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int32), ("n_tokens", C.c_uint32), ("logits", C.c_void_p),
                ("tokens", C.c_void_p), ("token_scalar", C.c_int32), ("hash_mode", C.c_uint32),
                ("routed_out", C.c_void_p), ("shared_out", C.c_void_p), ("residual_hc", C.c_void_p),
                ("hc_split", C.c_void_p), ("out_hc", C.c_void_p), ("n_hc", C.c_uint32), ("mix_hc", C.c_uint32),
                ("selected_out", C.c_void_p), ("weights_out", C.c_void_p)]


DTYPE_F32, DTYPE_BF16 = 0, 1
GGUF_F32, GGUF_F16, GGUF_Q8_0, GGUF_Q2_K, GGUF_Q4_K, GGUF_IQ2_XXS, GGUF_I32 = 0, 1, 8, 10, 12, 16, 26


class GgufTensor(C.Structure):
    """dsmoe_gguf_tensor of include/dsmoe.h."""
    _fields_ = [("name", C.c_char_p), ("type", C.c_uint32), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4),
                ("offset", C.c_uint64), ("bytes", C.c_uint64), ("host_data", C.c_void_p)]


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
    "dsmoe_layer_register_extras": (_int, [_vp, _u32, _vp, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_ffn_forward": (_int, [_vp, _vp, _u32, C.POINTER(FfnArgs)]),
    "dsmoe_hc_split_weighted_sum_norm": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _f32,
                                                _f32]),
    "dsmoe_hc_expand": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32]),
    "dsmoe_moe_forward": (_int, [_vp, _vp, _u32, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_expert_ffn": (_int, [_vp, _vp, _u32, _vp, _vp, _vp, _u32, _vp]),
    "dsmoe_moe_forward_host": (_int, [_vp, _u32, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_moe_forward_host_async": (_int, [_vp, _u32, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_host_synchronize": (_int, [_vp]),
    "dsmoe_moe_forward_noalloc": (_int, [_vp, _vp, _vp, _vp, _int, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_noalloc_device_status": (_int, [_vp, _vp]),
    "dsmoe_ep_get_unique_id": (_int, [_vp]),
    "dsmoe_ep_init": (_int, [_vp, _vp, _int, _int, _u32, _u32]),
    "dsmoe_ep_init_comm": (_int, [_vp, _vp, _int, _int, _u32, _u32]),
    "dsmoe_ep_layer_register": (_int, [_vp, _u32, _vp, _vp, _vp, _int]),
    "dsmoe_ep_set_replicas": (_int, [_vp, _vp, _u32]),
    "dsmoe_ep_expert_counts": (_int, [_vp, _vp, _vp, _int]),
    "dsmoe_ep_last_recv_rows": (_int, [_vp, _vp]),
    "dsmoe_ep_set_phase_events": (_int, [_vp, C.POINTER(_vp), _int]),
    "dsmoe_ep_combine_is_fused": (_int, [_vp]),
    "dsmoe_moe_forward_ep": (_int, [_vp, _vp, _u32, _vp, _vp, _u32, _vp, _vp, _vp]),
    "dsmoe_gguf_open": (_int, [C.c_char_p, C.POINTER(_vp)]),
    "dsmoe_gguf_open_memory": (_int, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "dsmoe_gguf_close": (_int, [_vp]),
    "dsmoe_gguf_last_error": (C.c_char_p, [_vp]),
    "dsmoe_gguf_tensor_count": (_u64, [_vp]),
    "dsmoe_gguf_data_offset": (_u64, [_vp]),
    "dsmoe_gguf_tensor_at": (_int, [_vp, _u64, C.POINTER(GgufTensor)]),
    "dsmoe_gguf_find_tensor": (_int, [_vp, C.c_char_p, C.POINTER(GgufTensor)]),
    "dsmoe_gguf_expert_shard_bytes": (_int, [C.POINTER(Config), _u32, C.POINTER(_u64), C.POINTER(_u64)]),
    "dsmoe_gguf_upload_experts": (_int, [_vp, C.POINTER(Config), _vp, _u32, _u32, _u32, _int, _vp, _vp, _vp, _vp]),
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
