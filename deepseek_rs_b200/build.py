"""Builds libdsmoe.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Usage: ``python -m deepseek_rs_b200.build [--force] [--verbose]``. Cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libdsmoe.so")
LIB_BOUNDS = os.path.join(HERE, "libdsmoe_bounds.so")  # the checked build (-DDSMOE_BOUNDS)
SOURCES = ["api.cu", "quant_router.cu", "experts.cu", "experts_tma.cu", "noalloc.cu", "prefill.cu", "fp8.cu", "shared.cu", "gguf.cu", "ep.cu"]
HEADERS = ["common.cuh", "launch.h", "async.cuh", "tc05.cuh", "ep.h", os.path.join("..", "..", "include", "dsmoe.h"),
           os.path.join("..", "..", "include", "dsmoe_iq2_tables.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # no fused multiply-add contraction: the f32 epilogues must round each operation like the reference's
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-cudart", "static", "--shared", "-ldl",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> str:
    """bounds=True builds the checked variant: expert indices handed to the tier-2 calls are copied, range-checked and
    replaced by 0 when outside the layer, with the violation recorded in the status word (no trap, no fault)."""
    lib = LIB_BOUNDS if bounds else LIB
    if not force and not needs_build(lib):
        return lib
    cmd = [_nvcc()] + NVCC_FLAGS + (["-DDSMOE_BOUNDS"] if bounds else []) + (["-Xptxas", "-v"] if verbose else []) + \
          ["-o", lib] + [os.path.join(CSRC, s) for s in SOURCES]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed building {os.path.basename(lib)}")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, bounds="--bounds" in sys.argv))
