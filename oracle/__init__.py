"""ctypes front end of the CPU oracle (``dsmoe_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the benchmark's CPU-baseline leg, never
by the shipped package. It restates the reference's arithmetic for the routed-expert path in plain C; the reference
itself (Rust through cuda-oxide) cannot be built here, so this is a port, pinned against the known answers of the
reference's own CPU tests (engine/tests/quant_cpu.rs). See the header of ``dsmoe_oracle.c`` for what is pinned and
what is not.

All arrays are numpy, C-contiguous. Packed blocks travel as ``uint8`` arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libdsmoe_oracle.so")

IQ2XXS_BYTES = 66
Q2K_BYTES = 84
Q8K_BYTES = 292
QK_K = 256


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it; returns the library path."""
    src = os.path.join(_HERE, "dsmoe_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_i8p = C.POINTER(C.c_int8)
_u16p = C.POINTER(C.c_uint16)


def _declare(L: C.CDLL) -> None:
    L.orc_f16_to_f32.restype = C.c_float
    L.orc_f16_to_f32.argtypes = [C.c_uint16, C.c_int]
    for name in ("orc_expf", "orc_logf", "orc_softplus", "orc_router_score"):
        getattr(L, name).restype = C.c_float
        getattr(L, name).argtypes = [C.c_float]
    L.orc_iq2xxs_codes.argtypes = [_u8p, _i32p]
    L.orc_dequant_iq2xxs.argtypes = [_u8p, C.c_int64, _f32p, C.c_int]
    L.orc_dequant_q2k.argtypes = [_u8p, C.c_int64, _f32p, C.c_int]
    L.orc_q8k_quantize.argtypes = [_f32p, _u8p, C.c_int64, C.c_int64]
    L.orc_dot_iq2xxs_q8k.restype = C.c_float
    L.orc_dot_iq2xxs_q8k.argtypes = [_u8p, _u8p, C.c_int]
    L.orc_dot_q2k_q8k.restype = C.c_float
    L.orc_dot_q2k_q8k.argtypes = [_u8p, _u8p, C.c_int]
    L.orc_router_select.argtypes = [_f32p, _f32p, _i32p, _i32p, _f32p, _i32p, _f32p, C.c_int32, C.c_uint32,
                                    C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int]
    L.orc_matmul_f16.argtypes = [_u16p, _f32p, _f32p, C.c_int64, C.c_int64, C.c_int64]
    L.orc_matvec_iq2xxs.argtypes = [_u8p, _u8p, _f32p, C.c_int64, C.c_uint32, C.c_int64, C.c_int]
    L.orc_matvec_q2k.argtypes = [_u8p, _u8p, _f32p, C.c_int64, C.c_uint32, C.c_int64, C.c_int]
    L.orc_gate_up_mid.argtypes = [_u8p, _u8p, _u8p, _i32p, _f32p, _f32p, _f32p, _f32p, C.c_uint64, C.c_uint64,
                                  C.c_uint32, C.c_uint32, C.c_uint32, C.c_int64, C.c_float, C.c_int]
    L.orc_down.argtypes = [_u8p, _u8p, _i32p, _f32p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32,
                           C.c_int64, C.c_int]
    L.orc_down_sum.argtypes = L.orc_down.argtypes
    L.orc_swiglu.argtypes = [_f32p, _f32p, _f32p, C.c_int64, C.c_float, C.c_float]
    L.orc_moe_layer.restype = C.c_int
    L.orc_moe_layer.argtypes = [_f32p, _f32p, _u8p, _u8p, _u8p, _f32p, _i32p, _f32p, _f32p, C.c_int64, C.c_uint32,
                                C.c_uint32, C.c_int, C.c_int, C.c_float, C.c_int]
    L.orc_quantize_q8_0.argtypes = [_f32p, _i8p, _f32p, C.c_int64, C.c_int64]
    L.orc_matmul_q8_0.argtypes = [_u8p, _i8p, _f32p, _f32p, C.c_int64, C.c_int64, C.c_int64]
    L.orc_check_div_rn.argtypes = [C.c_int64, C.c_uint64, C.POINTER(C.c_int64)]
    L.orc_check_div_rn.restype = C.c_int64
    L.orc_e4m3_value.restype = C.c_float
    L.orc_e4m3_value.argtypes = [C.c_int]
    L.orc_e4m3_encode.restype = C.c_uint8
    L.orc_e4m3_encode.argtypes = [C.c_float]
    L.orc_e4m3_decode.restype = C.c_float
    L.orc_e4m3_decode.argtypes = [C.c_uint8]
    L.orc_fp8_quantize.argtypes = [_f32p, _u8p, _f32p, C.c_int64, C.c_int64, C.c_int]
    L.orc_fp8_gemm.argtypes = [_u8p, _f32p, _u8p, _f32p, _f32p, C.c_int64, C.c_int64, C.c_int64]
    L.orc_hc_expand.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int]
    L.orc_hc_split_weighted_sum_norm.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, C.c_int64,
                                                 C.c_int64, C.c_int, C.c_float, C.c_float]
    L.orc_num_threads.restype = C.c_int
    L.orc_set_num_threads.argtypes = [C.c_int]


def _p(a, ty):
    return None if a is None else a.ctypes.data_as(ty)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


# ---------------------------------------------------------------------------------------------------------------
# scalar helpers
# ---------------------------------------------------------------------------------------------------------------

def f16_to_f32(bits: int, ieee: bool = False) -> float:
    return float(lib().orc_f16_to_f32(int(bits) & 0xFFFF, int(ieee)))


def softplus(x: float) -> float:
    return float(lib().orc_softplus(np.float32(x)))


def router_score(x: float) -> float:
    return float(lib().orc_router_score(np.float32(x)))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


# ---------------------------------------------------------------------------------------------------------------
# array functions
# ---------------------------------------------------------------------------------------------------------------

def dequant_iq2xxs(blocks: np.ndarray, ieee: bool = False) -> np.ndarray:
    blocks = _c(blocks, np.uint8).reshape(-1)
    n = blocks.size // IQ2XXS_BYTES
    out = np.empty(n * QK_K, np.float32)
    lib().orc_dequant_iq2xxs(_p(blocks, _u8p), n, _p(out, _f32p), int(ieee))
    return out


def dequant_q2k(blocks: np.ndarray, ieee: bool = False) -> np.ndarray:
    blocks = _c(blocks, np.uint8).reshape(-1)
    n = blocks.size // Q2K_BYTES
    out = np.empty(n * QK_K, np.float32)
    lib().orc_dequant_q2k(_p(blocks, _u8p), n, _p(out, _f32p), int(ieee))
    return out


def q8k_quantize(x: np.ndarray) -> np.ndarray:
    """x: f32 [rows, in_dim] -> uint8 [rows, in_dim/256, 292]"""
    x = _c(x, np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    rows, in_dim = x2.shape
    out = np.zeros((rows, in_dim // QK_K, Q8K_BYTES), np.uint8)
    if rows and in_dim:
        lib().orc_q8k_quantize(_p(x2, _f32p), _p(out, _u8p), in_dim, rows)
    return out


def dot_iq2xxs_q8k(iq2_blk: np.ndarray, q8k_blk: np.ndarray, ieee: bool = False) -> float:
    a, b = _c(iq2_blk, np.uint8), _c(q8k_blk, np.uint8)
    assert a.size == IQ2XXS_BYTES and b.size == Q8K_BYTES
    return float(lib().orc_dot_iq2xxs_q8k(_p(a, _u8p), _p(b, _u8p), int(ieee)))


def dot_q2k_q8k(q2k_blk: np.ndarray, q8k_blk: np.ndarray, ieee: bool = False) -> float:
    a, b = _c(q2k_blk, np.uint8), _c(q8k_blk, np.uint8)
    assert a.size == Q2K_BYTES and b.size == Q8K_BYTES
    return float(lib().orc_dot_q2k_q8k(_p(a, _u8p), _p(b, _u8p), int(ieee)))


def router_select(logits: np.ndarray, k: int = 6, bias=None, hash_table=None, tokens=None, token_scalar: int = 0):
    """Returns (probs [T,E], selected [T,k] int32, weights [T,k])."""
    logits = _c(logits, np.float32)
    T, E = logits.shape
    probs = np.empty((T, E), np.float32)
    sel = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    bias_a = None if bias is None else _c(bias, np.float32)
    hash_a = None if hash_table is None else _c(hash_table, np.int32)
    tok_a = None if tokens is None else _c(tokens, np.int32)
    hash_rows = 0 if hash_a is None else hash_a.size // k
    if T:
        lib().orc_router_select(_p(logits, _f32p), _p(bias_a, _f32p), _p(hash_a, _i32p), _p(tok_a, _i32p),
                                _p(probs, _f32p), _p(sel, _i32p), _p(w, _f32p), int(token_scalar), hash_rows, T,
                                int(bias_a is not None), int(hash_a is not None), k, E)
    return probs, sel, w


def matmul_f16(w_bits: np.ndarray, x: np.ndarray) -> np.ndarray:
    w_bits = _c(w_bits, np.uint16)
    x = _c(x, np.float32)
    out_dim, in_dim = w_bits.shape
    n_tok = x.shape[0]
    out = np.empty((n_tok, out_dim), np.float32)
    lib().orc_matmul_f16(_p(w_bits, _u16p), _p(x, _f32p), _p(out, _f32p), in_dim, out_dim, n_tok)
    return out


def matvec_iq2xxs(w: np.ndarray, xq: np.ndarray, n_rows: int, blocks: int, ieee: bool = False) -> np.ndarray:
    w, xq = _c(w, np.uint8), _c(xq, np.uint8)
    n_tok = xq.size // (blocks * Q8K_BYTES)
    out = np.empty((n_tok, n_rows), np.float32)
    lib().orc_matvec_iq2xxs(_p(w, _u8p), _p(xq, _u8p), _p(out, _f32p), n_rows, blocks, n_tok, int(ieee))
    return out


def matvec_q2k(w: np.ndarray, xq: np.ndarray, n_rows: int, blocks: int, ieee: bool = False) -> np.ndarray:
    w, xq = _c(w, np.uint8), _c(xq, np.uint8)
    n_tok = xq.size // (blocks * Q8K_BYTES)
    out = np.empty((n_tok, n_rows), np.float32)
    lib().orc_matvec_q2k(_p(w, _u8p), _p(xq, _u8p), _p(out, _f32p), n_rows, blocks, n_tok, int(ieee))
    return out


def gate_up_mid(gate: np.ndarray, up: np.ndarray, xq: np.ndarray, selected: np.ndarray, weights: np.ndarray,
                n_ff: int, xq_blocks: int, clamp: float = 10.0, ieee: bool = False):
    """Returns (gate_out, up_out, mid_out), each f32 [T*k, n_ff]."""
    gate, up, xq = _c(gate, np.uint8), _c(up, np.uint8), _c(xq, np.uint8)
    sel, w = _c(selected, np.int32), _c(weights, np.float32)
    T, k = sel.shape
    row_b = xq_blocks * IQ2XXS_BYTES
    g = np.empty((T * k, n_ff), np.float32)
    u = np.empty_like(g)
    m = np.empty_like(g)
    if T:
        lib().orc_gate_up_mid(_p(gate, _u8p), _p(up, _u8p), _p(xq, _u8p), _p(sel, _i32p), _p(w, _f32p), _p(g, _f32p),
                              _p(u, _f32p), _p(m, _f32p), n_ff * row_b, row_b, xq_blocks, n_ff, k, T, clamp, int(ieee))
    return g, u, m


def down(down_w: np.ndarray, midq: np.ndarray, selected: np.ndarray, out_dim: int, midq_blocks: int,
         ieee: bool = False) -> np.ndarray:
    down_w, midq, sel = _c(down_w, np.uint8), _c(midq, np.uint8), _c(selected, np.int32)
    T, k = sel.shape
    row_b = midq_blocks * Q2K_BYTES
    out = np.empty((T * k, out_dim), np.float32)
    if T:
        lib().orc_down(_p(down_w, _u8p), _p(midq, _u8p), _p(sel, _i32p), _p(out, _f32p), out_dim * row_b, row_b,
                       midq_blocks, out_dim, k, T, int(ieee))
    return out


def down_sum(down_w: np.ndarray, midq: np.ndarray, selected: np.ndarray, out_dim: int, midq_blocks: int,
             ieee: bool = False) -> np.ndarray:
    down_w, midq, sel = _c(down_w, np.uint8), _c(midq, np.uint8), _c(selected, np.int32)
    T, k = sel.shape
    row_b = midq_blocks * Q2K_BYTES
    out = np.empty((T, out_dim), np.float32)
    if T:
        lib().orc_down_sum(_p(down_w, _u8p), _p(midq, _u8p), _p(sel, _i32p), _p(out, _f32p), out_dim * row_b, row_b,
                           midq_blocks, out_dim, k, T, int(ieee))
    return out


def swiglu(gate: np.ndarray, up: np.ndarray, clamp: float, weight: float) -> np.ndarray:
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(gate)
    lib().orc_swiglu(_p(gate, _f32p), _p(up, _f32p), _p(out, _f32p), gate.size, clamp, weight)
    return out


def moe_layer(x: np.ndarray, logits: np.ndarray, gate: np.ndarray, up: np.ndarray, down_w: np.ndarray, k: int = 6,
              clamp: float = 10.0, n_ff: int = 2048, ieee: bool = False, return_mid: bool = False):
    """Router -> Q8_K -> gate/up/SwiGLU -> Q8_K -> down -> slot sum. Returns (out [T,n_embd], selected, weights[, mid])."""
    x, logits = _c(x, np.float32), _c(logits, np.float32)
    gate, up, down_w = _c(gate, np.uint8), _c(up, np.uint8), _c(down_w, np.uint8)
    T, n_embd = x.shape
    out = np.empty((T, n_embd), np.float32)
    sel = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    mid = np.empty((T * k, n_ff), np.float32) if return_mid else None
    if T:
        rc = lib().orc_moe_layer(_p(x, _f32p), _p(logits, _f32p), _p(gate, _u8p), _p(up, _u8p), _p(down_w, _u8p),
                                 _p(out, _f32p), _p(sel, _i32p), _p(w, _f32p), _p(mid, _f32p), T, n_embd, n_ff,
                                 logits.shape[1], k, clamp, int(ieee))
        if rc != 0:
            raise MemoryError("oracle scratch allocation failed")
    return (out, sel, w, mid) if return_mid else (out, sel, w)


def quantize_q8_0(x: np.ndarray):
    x = _c(x, np.float32)
    n_tok, in_dim = x.shape
    blocks = (in_dim + 31) // 32
    xq = np.empty((n_tok, blocks * 32), np.int8)
    xs = np.empty((n_tok, blocks), np.float32)
    lib().orc_quantize_q8_0(_p(x, _f32p), _p(xq, _i8p), _p(xs, _f32p), in_dim, n_tok)
    return xq, xs


def matmul_q8_0(w: np.ndarray, xq: np.ndarray, xscale: np.ndarray, in_dim: int, out_dim: int) -> np.ndarray:
    w, xq, xscale = _c(w, np.uint8), _c(xq, np.int8), _c(xscale, np.float32)
    n_tok = xq.shape[0]
    out = np.empty((n_tok, out_dim), np.float32)
    lib().orc_matmul_q8_0(_p(w, _u8p), _p(xq, _i8p), _p(xscale, _f32p), _p(out, _f32p), in_dim, out_dim, n_tok)
    return out


def e4m3_encode(x: float) -> int:
    return int(lib().orc_e4m3_encode(np.float32(x)))


def e4m3_decode(c: int) -> float:
    return float(lib().orc_e4m3_decode(int(c) & 0xFF))


def fp8_quantize(x: np.ndarray, rows_per_block: int):
    x = _c(x, np.float32)
    rows, cols = x.shape
    codes = np.empty((rows, cols), np.uint8)
    scales = np.empty(((rows + rows_per_block - 1) // rows_per_block, cols // 128), np.float32)
    lib().orc_fp8_quantize(_p(x, _f32p), _p(codes, _u8p), _p(scales, _f32p), rows, cols, rows_per_block)
    return codes, scales


def fp8_gemm(a: np.ndarray, a_scale: np.ndarray, w: np.ndarray, w_scale: np.ndarray) -> np.ndarray:
    a, w = _c(a, np.uint8), _c(w, np.uint8)
    a_scale, w_scale = _c(a_scale, np.float32), _c(w_scale, np.float32)
    M, K = a.shape
    N = w.shape[0]
    out = np.empty((M, N), np.float32)
    lib().orc_fp8_gemm(_p(a, _u8p), _p(a_scale, _f32p), _p(w, _u8p), _p(w_scale, _f32p), _p(out, _f32p), M, N, K)
    return out


def hc_expand(block_out: np.ndarray, block_add, residual_hc: np.ndarray, split: np.ndarray) -> np.ndarray:
    """hc_expand of engine/src/kernels/hc.rs:212-251. block_out / block_add [T, n_embd] (block_add may be None),
    residual_hc [T, n_hc, n_embd], split [T, mix_hc]. Returns out_hc [T, n_hc, n_embd]."""
    bo, res, sp = _c(block_out, np.float32), _c(residual_hc, np.float32), _c(split, np.float32)
    ba = None if block_add is None else _c(block_add, np.float32)
    T, n_hc, n_embd = res.shape
    out = np.empty_like(res)
    if T:
        lib().orc_hc_expand(_p(bo, _f32p), _p(ba, _f32p), _p(res, _f32p), _p(sp, _f32p), _p(out, _f32p), n_embd, n_hc, T,
                            sp.shape[1], int(ba is not None))
    return out


def hc_split_weighted_sum_norm(mix, scale, base, residual_hc, norm_w, iters: int = 20, epsv: float = 1e-6,
                               norm_eps: float = 1e-6):
    """hc_split_weighted_sum_norm_fused of engine/src/kernels/hc.rs:313-394. mix [T, 24], scale [3], base [24], residual_hc
    [T, 4, n_embd], norm_w [n_embd]. Returns (split [T, 24], out [T, n_embd], norm_out [T, n_embd])."""
    mix, scale, base = _c(mix, np.float32), _c(scale, np.float32), _c(base, np.float32)
    res, nw = _c(residual_hc, np.float32), _c(norm_w, np.float32)
    T, _, n_embd = res.shape
    split = np.empty((T, 24), np.float32)
    out = np.empty((T, n_embd), np.float32)
    norm_out = np.empty_like(out)
    if T:
        lib().orc_hc_split_weighted_sum_norm(_p(mix, _f32p), _p(scale, _f32p), _p(base, _f32p), _p(res, _f32p), _p(nw, _f32p),
                                             _p(split, _f32p), _p(out, _f32p), _p(norm_out, _f32p), n_embd, T, iters, epsv,
                                             norm_eps)
    return split, out, norm_out


def check_div_rn(n: int, seed: int = 1):
    """(mismatches, skipped) of the SwiGLU division sequence against IEEE division over n pseudo-random pairs."""
    skipped = C.c_int64(0)
    bad = lib().orc_check_div_rn(int(n), int(seed), C.byref(skipped))
    return int(bad), int(skipped.value)
