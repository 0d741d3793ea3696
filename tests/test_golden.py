"""Golden fixtures (tests/golden/*.npz, made by tests/golden/make_golden.py): seeded inputs of the benchmark
configurations with the oracle's outputs stored as exact bit patterns. The CPU tests pin the input generators and the
oracle; the GPU tests compare the kernels, through the C ABI, with the stored outputs."""
import importlib.util
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)

CASES = ["iq2xxs_matvec", "q2k_matvec", "moe_layer", "fp8"]


@pytest.fixture(scope="module")
def cases():
    return make_golden.inputs()


def load(name):
    return np.load(os.path.join(HERE, "golden", name + ".npz"))


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and a.dtype == b.dtype and a.tobytes() == b.tobytes()


@pytest.mark.parametrize("name", CASES)
def test_inputs_regenerate_identically(cases, name):
    g = load(name)
    for k, v in cases[name].items():
        assert bytes(g["sha256_in_" + k]).hex() == make_golden.sha(v), f"{name}.{k}: the seeded generator drifted"


def test_oracle_reproduces_the_fixtures(cases, oracle):
    o = make_golden.outputs(cases, oracle)
    for name in CASES:
        g = load(name)
        for k, v in o[name].items():
            assert same_bits(g[k], v), f"{name}.{k}"


# ---- GPU --------------------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.gpu
def test_gpu_iq2xxs_matvec_fixture(torch_cuda, cases):
    """Configuration 1 through q8k_quantize and the gate/up kernel with one expert and one slot: gate_out is W x."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import MoeKernels

    c, g = cases["iq2xxs_matvec"], load("iq2xxs_matvec")
    K = MoeKernels(device=0, n_expert=32, n_expert_used=1, max_tokens=1)
    xq = torch.empty((1, 16, 292), dtype=torch.uint8, device="cuda")
    K.q8k_quantize(dev(torch, c["x"]), xq, 4096, 1)
    w = dev(torch, c["w"])
    gate_out, up_out, mid = (torch.empty((1, 2048), device="cuda") for _ in range(3))
    sel = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    wt = torch.ones((1, 1), device="cuda")
    # clamp 0 switches the clamp off: gate_out / up_out are then the plain projections
    K.moe_gate_up_mid_qwarp32(w, w, xq, sel, wt, gate_out, up_out, mid, 2048 * 16 * 66, 16 * 66, 16, 2048, 1, 0.0)
    torch.cuda.synchronize()
    assert same_bits(xq.cpu().numpy(), g["xq"])
    assert same_bits(gate_out.cpu().numpy(), g["y"]) and same_bits(up_out.cpu().numpy(), g["y"])
    K.close()


@pytest.mark.gpu
@pytest.mark.parametrize("T", [1, 4, 16])
def test_gpu_q2k_matvec_fixture(torch_cuda, cases, T):
    """Configuration 2 through the down kernel with one expert and one slot per token."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import MoeKernels

    c, g = cases["q2k_matvec"], load("q2k_matvec")
    K = MoeKernels(device=0, n_expert=32, n_expert_used=1, max_tokens=16)
    xq = torch.empty((T, 16, 292), dtype=torch.uint8, device="cuda")
    K.q8k_quantize(dev(torch, c["x"][:T]), xq, 4096, T)
    out = torch.empty((T, 2048), device="cuda")
    sel = torch.zeros((T, 1), dtype=torch.int32, device="cuda")
    K.moe_down_qwarp32(dev(torch, c["w"]), xq, sel, out, 2048 * 16 * 84, 16 * 84, 16, 2048, 1, T)
    torch.cuda.synchronize()
    assert same_bits(out.cpu().numpy(), g["y16"][:T])
    K.close()


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["native", "rowsoa"])
def test_gpu_moe_layer_fixture(torch_cuda, cases, layout):
    """Configuration 3 (32 experts) through the tier-2 call on the decode kernels: bit-identical to the fixture."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA, MoeKernels, MoeLayer

    c, g = cases["moe_layer"], load("moe_layer")
    K = MoeKernels(device=0, n_expert=32, max_tokens=8)
    layer = MoeLayer(K, c["gate"], c["up"], c["down"], layout=LAYOUT_ROWSOA if layout == "rowsoa" else LAYOUT_NATIVE)
    sel = torch.zeros((8, 6), dtype=torch.int32, device="cuda")
    wts = torch.zeros((8, 6), device="cuda")
    out = layer.forward(dev(torch, c["x"]), dev(torch, c["logits"]), selected_out=sel, weights_out=wts)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    assert same_bits(sel.cpu().numpy(), g["selected"])
    assert same_bits(wts.cpu().numpy(), g["weights"])
    assert same_bits(out.cpu().numpy(), g["out"])
    K.close()


@pytest.mark.gpu
def test_gpu_fp8_fixture(torch_cuda, cases):
    """Configuration 5 at a small shape: codes and scales bit-exact, the product within rel 2e-2 of the f64 oracle."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import MoeKernels

    c, g = cases["fp8"], load("fp8")
    K = MoeKernels(device=0, n_expert=32, max_tokens=8)
    ac = torch.empty((8, 512), dtype=torch.uint8, device="cuda")
    asc = torch.empty((8, 4), device="cuda")
    wc = torch.empty((256, 512), dtype=torch.uint8, device="cuda")
    wsc = torch.empty((2, 4), device="cuda")
    K.fp8_quantize(dev(torch, c["a"]), ac, asc, 8, 512, 1)
    K.fp8_quantize(dev(torch, c["w"]), wc, wsc, 256, 512, 128)
    out = torch.empty((8, 256), dtype=torch.bfloat16, device="cuda")
    K.fp8_linear(ac, asc, wc, wsc, out, 8, 256, 512)
    torch.cuda.synchronize()
    assert same_bits(ac.cpu().numpy(), g["a_codes"]) and same_bits(asc.cpu().numpy(), g["a_scales"])
    assert make_golden.sha(wc.cpu().numpy()) == bytes(g["w_codes_sha"]).hex() and same_bits(wsc.cpu().numpy(), g["w_scales"])
    y = out.float().cpu().numpy()
    assert np.all(np.abs(y - g["y"]) <= 2e-2 * np.abs(g["y"]) + 2e-2 * np.abs(g["y"]).max() * 2.0 ** -7)
    K.close()
