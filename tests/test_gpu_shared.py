"""Router logits (f16 matmul) and the shared expert (Q8_0) on the GPU against the oracle: the kernels keep the
reference's partial sums and their order, so everything here is compared bit for bit."""
import numpy as np
import pytest

from deepseek_rs_b200 import formats as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return torch


@pytest.fixture(scope="module")
def K(torch_cuda):
    from deepseek_rs_b200.kernels import MoeKernels

    k = MoeKernels(device=0, n_expert=32, max_tokens=1500)
    yield k
    k.close()


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("T,in_dim", [(1, 4096), (5, 2048), (3, 100)])
def test_quantize_q8_0_bit_exact(torch_cuda, oracle, K, T, in_dim):
    torch = torch_cuda
    rng = np.random.default_rng(in_dim + T)
    x = rng.standard_normal((T, in_dim)).astype(np.float32)
    x[0, :32] = 0.0  # a zero block: d = 0, id = 0
    want_q, want_s = oracle.quantize_q8_0(x)
    blocks = (in_dim + 31) // 32
    xq = torch.full((T, blocks * 32), 77, dtype=torch.int8, device="cuda")
    xs = torch.empty((T, blocks), device="cuda")
    K.quantize_q8_0(dev(torch, x), xq, xs, in_dim, T)
    torch.cuda.synchronize()
    assert np.array_equal(xq.cpu().numpy(), want_q)
    assert np.array_equal(xs.cpu().numpy().view(np.uint32), want_s.view(np.uint32))


@pytest.mark.parametrize("T,in_dim,out_dim", [(1, 4096, 2048), (1, 2048, 4096), (6, 4096, 264), (9, 96, 40)])
def test_matmul_q8_0_bit_exact(torch_cuda, oracle, K, T, in_dim, out_dim):
    """Even and odd block counts per row (the 34-byte blocks then start on both 2-byte phases), one and many tokens."""
    torch = torch_cuda
    rng = np.random.default_rng(T * 7 + out_dim)
    blocks = in_dim // 32
    w = F.random_q8_0(rng, out_dim * blocks)
    x = rng.standard_normal((T, in_dim)).astype(np.float32)
    xq, xs = oracle.quantize_q8_0(x)
    want = oracle.matmul_q8_0(w, xq, xs, in_dim, out_dim)
    out = torch.empty((T, out_dim), device="cuda")
    K.matmul_q8_0_preq_warp8(dev(torch, w), dev(torch, xq), dev(torch, xs), out, in_dim, out_dim, T)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_swiglu_bit_exact(torch_cuda, oracle, K):
    torch = torch_cuda
    rng = np.random.default_rng(3)
    g = (rng.standard_normal(5000) * 6).astype(np.float32)
    u = (rng.standard_normal(5000) * 6).astype(np.float32)
    g[:4] = [0.0, -0.0, 30.0, -90.0]
    for clamp, weight in ((10.0, 1.0), (0.0, 0.37)):
        out = torch.empty(5000, device="cuda")
        K.swiglu(dev(torch, g), dev(torch, u), out, 5000, clamp, weight)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint32), oracle.swiglu(g, u, clamp, weight).view(np.uint32))


@pytest.mark.parametrize("T,in_dim,out_dim", [(1, 4096, 256), (7, 4096, 32), (2, 1000, 10), (3, 2048, 6), (2, 4352, 9)])
def test_matmul_f16_router_logits_bit_exact(torch_cuda, oracle, K, T, in_dim, out_dim):
    torch = torch_cuda
    rng = np.random.default_rng(out_dim)
    w = (rng.standard_normal((out_dim, in_dim)) * 0.05).astype(np.float16)
    x = F.bf16_round(rng.standard_normal((T, in_dim)).astype(np.float32))
    want = oracle.matmul_f16(w.view(np.uint16), x)
    out = torch.empty((T, out_dim), device="cuda")
    K.matmul_f16(dev(torch, w), dev(torch, x), out, in_dim, out_dim, T)  # the f16 tensor's bits are the weights
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("T,shift", [(1, 0), (2, 0), (3, 0), (5, 0), (8, 0), (1, 4), (3, 4), (9, 0), (64, 0), (9, 4), (1300, 0)])
def test_shared_expert_whole(torch_cuda, oracle, K, T, shift):
    """The one-call shared expert against the oracle's four steps. Up to 8 tokens take the two-launch kernels: with
    16-byte aligned tensors the form that stages whole weight rows in shared memory by bulk copies, with tensors that
    start 4 bytes off such a boundary (shift) the form that loads words; 9 and 1300 tokens take the six-launch path, the
    latter across the library's 1024-token chunks."""
    torch = torch_cuda
    rng = np.random.default_rng(T)
    n_embd, n_ff = 4096, 2048
    gw = F.random_q8_0(rng, n_ff * (n_embd // 32))
    uw = F.random_q8_0(rng, n_ff * (n_embd // 32))
    dw = F.random_q8_0(rng, n_embd * (n_ff // 32))
    x = F.bf16_round(rng.standard_normal((T, n_embd)).astype(np.float32))
    xq, xs = oracle.quantize_q8_0(x)
    g = oracle.matmul_q8_0(gw, xq, xs, n_embd, n_ff)
    u = oracle.matmul_q8_0(uw, xq, xs, n_embd, n_ff)
    mid = oracle.swiglu(g, u, 10.0, 1.0).reshape(T, n_ff)
    mq, ms = oracle.quantize_q8_0(mid)
    want = oracle.matmul_q8_0(dw, mq, ms, n_ff, n_embd)
    out = torch.empty((T, n_embd), device="cuda")
    def place(w):  # the tensor's bytes at `shift` bytes past a 256-byte aligned allocation
        buf = torch.empty(w.size + 16, dtype=torch.uint8, device="cuda")
        view = buf[shift:shift + w.size]
        view.copy_(torch.from_numpy(w.reshape(-1)))
        assert view.data_ptr() % 16 == shift
        return view

    K.shared_expert(place(gw), place(uw), place(dw), dev(torch, x), T, out)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
