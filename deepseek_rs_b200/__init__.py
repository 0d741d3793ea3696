"""dsmoe: B200-native kernels for the quantized routed-expert path of the deepseek-rs engine.

The product is ``libdsmoe.so`` (hand-written CUDA for sm_100a behind the C ABI of ``include/dsmoe.h``). This package
is the thin host-side mirror used by the tests and the benchmark: ``kernels.MoeKernels`` exposes the reference's
kernel call surface (same names and operands as engine/src/kernels/moe.rs and quantize.rs) over torch tensors, and
``kernels.MoeLayer`` the fused per-layer call. ``formats`` holds the packed block formats and synthetic generators.
"""
from . import formats  # noqa: F401

__all__ = ["formats"]
