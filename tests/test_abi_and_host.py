"""CPU-side checks of the boundary: the library builds, loads and exports every symbol the header declares, and the
host-side mirror refuses to run without a GPU instead of falling back."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    from deepseek_rs_b200 import build

    return build.build()


def _declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            names |= set(re.findall(r"DSMOE_API[^;(]*?\b(dsmoe_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    declared = _declared_symbols()
    assert len(declared) >= 19
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_ctypes_signatures_cover_the_header(built_lib):
    from deepseek_rs_b200 import _lib

    assert set(_lib.SIGNATURES) == _declared_symbols()
    lib = _lib.load()
    assert lib.dsmoe_version().startswith(b"dsmoe")


def test_default_config_matches_reference_constants(built_lib):
    from deepseek_rs_b200 import _lib

    cfg = _lib.Config()
    _lib.load().dsmoe_default_config(ctypes.byref(cfg))
    # engine/src/model.rs:4, 15-18; engine/src/session.rs:21; engine/src/kernels/moe.rs:284
    assert (cfg.n_embd, cfg.n_ff, cfg.n_expert, cfg.n_expert_used) == (4096, 2048, 256, 6)
    assert cfg.swiglu_clamp == 10.0 and cfg.route_scale == 1.5 and cfg.f16_ieee == 0


def test_no_cpu_fallback(built_lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from deepseek_rs_b200.kernels import MoeKernels

    with pytest.raises(RuntimeError):
        MoeKernels(device=0)


def test_create_rejects_bad_config_without_touching_a_device(built_lib):
    from deepseek_rs_b200 import _lib

    lib = _lib.load()
    h = ctypes.c_void_p()
    cfg = _lib.Config(4000, 2048, 256, 6, 10.0, 1.5, 0, 1, 1)  # n_embd not a multiple of 256
    assert lib.dsmoe_create(ctypes.byref(cfg), 0, ctypes.byref(h)) == _lib.ERR_ARG
    cfg = _lib.Config(4096, 2048, 256, 9, 10.0, 1.5, 0, 1, 1)  # k > 8
    assert lib.dsmoe_create(ctypes.byref(cfg), 0, ctypes.byref(h)) == _lib.ERR_ARG
    assert lib.dsmoe_destroy(None) == 0


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "deepseek_rs_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "import oracle" not in text and "from oracle" not in text and "dsmoe_oracle" not in text, fn
                # nor the GPU baseline (the restated reference mapping), which is bench and test infrastructure too
                assert "import baseline" not in text and "from baseline" not in text and "ref_mapping" not in text, fn
