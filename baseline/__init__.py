"""GPU baseline beside the product: a CUDA restatement of the reference kernels' thread mapping (ref_mapping.cu).

Bench and test infrastructure only; the product never imports this package. ``RefMapping`` wraps the library's entry
points over torch CUDA tensors. Build: ``python -m baseline`` (nvcc, sm_100a, cross-compiles without a GPU).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "ref_mapping.cu")
LIB = os.path.join(HERE, "libref_mapping.so")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false", "-prec-div=true",
         "-prec-sqrt=true", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-cudart", "static", "--shared"]


def build(force: bool = False) -> str:
    deps = [SRC, os.path.join(HERE, "..", "include", "dsmoe_iq2_tables.h")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(d) <= os.path.getmtime(LIB) for d in deps):
        return LIB
    nvcc = os.environ.get("NVCC") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "nvcc")
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    r = subprocess.run([nvcc] + FLAGS + ["-o", LIB, SRC], capture_output=True, text=True, env=env)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed building libref_mapping.so")
    return LIB


_u32, _u64, _vp, _f = C.c_uint32, C.c_uint64, C.c_void_p, C.c_float
_SIGS = {
    "refmap_init": [_vp],
    "refmap_q8k_quantize": [_vp, _vp, _vp, _u32, _u32],
    "refmap_gate_up_mid": [_vp] * 9 + [_u64, _u64, _u32, _u32, _u32, _u32, _f],
    "refmap_down_sum6": [_vp] * 5 + [_u64, _u64, _u32, _u32],
    "refmap_tokens": [_vp] * 11 + [_u32, _u32, _u32, _f],
    "refmap_batched": [_vp] * 13 + [_u32, _u32, _u32, _f],
}


class RefMapping:
    """The restated reference kernels on the current CUDA device and torch stream."""

    def __init__(self):
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("the reference-mapping baseline needs a CUDA device")
        self.torch = torch
        self.lib = C.CDLL(build())
        for name, args in _SIGS.items():
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = args, C.c_int
        self._check(self.lib.refmap_init(self._stream()))

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    @staticmethod
    def _p(t):
        return C.c_void_p(0 if t is None else t.data_ptr())

    @staticmethod
    def _check(rc):
        if rc != 0:
            raise RuntimeError(f"reference-mapping baseline: CUDA error {rc}")

    def q8k_quantize(self, x, out, in_dim: int, n_rows: int):
        self._check(self.lib.refmap_q8k_quantize(self._stream(), self._p(x), self._p(out), in_dim, n_rows))

    def gate_up_mid(self, gate, up, xq, selected, weights, gate_out, up_out, mid_out, expert_bytes: int, row_bytes: int,
                    xq_blocks: int, mid_dim: int, k: int, n_tokens: int, clamp: float):
        self._check(self.lib.refmap_gate_up_mid(self._stream(), self._p(gate), self._p(up), self._p(xq), self._p(selected),
                                                self._p(weights), self._p(gate_out), self._p(up_out), self._p(mid_out),
                                                expert_bytes, row_bytes, xq_blocks, mid_dim, k, n_tokens, clamp))

    def down_sum6(self, down, midq, selected, out, expert_bytes: int, row_bytes: int, midq_blocks: int, out_dim: int):
        self._check(self.lib.refmap_down_sum6(self._stream(), self._p(down), self._p(midq), self._p(selected), self._p(out),
                                              expert_bytes, row_bytes, midq_blocks, out_dim))

    def tokens(self, gate, up, down, x, selected, weights, xq, mid, midq, out, n_embd: int, n_ff: int, n_tokens: int,
               clamp: float):
        """n_tokens tokens one after the other, four launches each, as the reference's prefill loop does."""
        self._check(self.lib.refmap_tokens(self._stream(), self._p(gate), self._p(up), self._p(down), self._p(x),
                                           self._p(selected), self._p(weights), self._p(xq), self._p(mid), self._p(midq),
                                           self._p(out), n_embd, n_ff, n_tokens, clamp))


    def batched(self, gate, up, down, x, selected, weights, out, n_embd: int, n_ff: int, n_tokens: int, clamp: float):
        """One chunk through the reference's sorted-pair kernels (the batched form it contains but never calls); scratch
        is allocated here, outside any timed region of the caller if it passes the returned tuple back in."""
        torch = self.torch
        dev, P = x.device, n_tokens * 6
        scratch = (torch.empty(n_tokens * (n_embd // 256) * 292, dtype=torch.uint8, device=dev),
                   torch.empty((P, n_ff), device=dev),
                   torch.empty(P * (n_ff // 256) * 292, dtype=torch.uint8, device=dev),
                   torch.empty((P, n_embd), device=dev),
                   torch.empty(770 + P, dtype=torch.int32, device=dev))
        self.batched_with(scratch, gate, up, down, x, selected, weights, out, n_embd, n_ff, n_tokens, clamp)
        return scratch

    def batched_with(self, scratch, gate, up, down, x, selected, weights, out, n_embd: int, n_ff: int, n_tokens: int,
                     clamp: float):
        xq, mid, midq, rows, idx = scratch
        self._check(self.lib.refmap_batched(self._stream(), self._p(gate), self._p(up), self._p(down), self._p(x),
                                            self._p(selected), self._p(weights), self._p(xq), self._p(mid), self._p(midq),
                                            self._p(rows), self._p(idx), self._p(out), n_embd, n_ff, n_tokens, clamp))
