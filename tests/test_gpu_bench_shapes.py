"""Parity at the shapes the benchmark times: 256 full-size experts, top-6, hidden 4096, width 2048.

The CPU oracle needs the packed bytes of the experts it evaluates on the host. A 256-expert layer is 1.8 GB, so the
layer is drawn on the device, the product runs on all of it, and only the experts that a seeded sample of tokens is
routed to are copied back: the oracle then evaluates that sample with the expert ids renumbered into the compact copy.
Routing is compared on every token."""
import numpy as np
import pytest

from deepseek_rs_b200 import formats as F

pytestmark = pytest.mark.gpu

REL, ABS = 1e-3, 1e-4  # tolerance for expert outputs (f32 accumulate)
N_E, K_USED, N_EMBD, N_FF = 256, 6, 4096, 2048


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="module")
def device_layer(torch_cuda):
    """(gate, up, down) of one 256-expert layer in NATIVE order on the device."""
    torch = torch_cuda
    return F.random_layer_device(torch, torch.device("cuda", 0), seed=4242)


def _oracle_sample(oracle, torch, layer_native, x, sel, wts, sample):
    """Expert outputs of tokens ``sample`` from the oracle, given the routing (already checked against the oracle's)."""
    gate, up, down = layer_native
    ge, de = N_FF * (N_EMBD // 256) * F.IQ2XXS_BYTES, N_EMBD * (N_FF // 256) * F.Q2K_BYTES
    s_sel = np.maximum(sel[sample], 0)
    used = np.unique(s_sel)
    idx = torch.from_numpy(used.astype(np.int64)).cuda()
    g = gate.view(N_E, ge)[idx].cpu().numpy().reshape(-1)
    u = up.view(N_E, ge)[idx].cpu().numpy().reshape(-1)
    d = down.view(N_E, de)[idx].cpu().numpy().reshape(-1)
    compact = np.searchsorted(used, s_sel).astype(np.int32)
    xq = oracle.q8k_quantize(x[sample])
    _, _, mid = oracle.gate_up_mid(g, u, xq, compact, wts[sample], N_FF, N_EMBD // 256)
    midq = oracle.q8k_quantize(mid)
    return oracle.down_sum(d, midq, compact, N_EMBD, N_FF // 256), mid


@pytest.mark.parametrize("layout", ["rowsoa", "native"])
def test_prefill_chunk_4096_tokens_256_experts_zipf(torch_cuda, oracle, device_layer, layout):
    """The prefill workload as benchmarked: 4096 tokens, Zipf s = 1.1 expert popularity, grouped GEMM path. Routing
    bit-exact on all 4096 tokens; outputs of a seeded 64-token sample within tolerance of the oracle."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA, MoeKernels, MoeLayer

    T = 4096
    rng = np.random.default_rng(77)
    x = F.bf16_round(rng.standard_normal((T, N_EMBD)).astype(np.float32))
    logits = F.zipf_logits(rng, T, N_E, s=1.1)
    K = MoeKernels(device=0, max_tokens=T)
    layer = MoeLayer(K, *device_layer, layout=LAYOUT_ROWSOA if layout == "rowsoa" else LAYOUT_NATIVE)
    sel = torch.zeros((T, K_USED), dtype=torch.int32, device="cuda")
    wts = torch.zeros((T, K_USED), dtype=torch.float32, device="cuda")
    out = layer.forward(torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda(), selected_out=sel, weights_out=wts)
    assert K.device_status() == 0
    sel_h, wts_h = sel.cpu().numpy(), wts.cpu().numpy()
    _, ref_sel, ref_w = oracle.router_select(logits, k=K_USED)
    assert np.array_equal(sel_h, ref_sel), "routing differs from the oracle"
    assert np.array_equal(wts_h, ref_w)
    counts = np.bincount(sel_h.reshape(-1), minlength=N_E)
    assert counts.max() > 20 * 128, "the workload should make one expert span dozens of token tiles"
    sample = np.sort(rng.choice(T, size=64, replace=False))
    ref, _ = _oracle_sample(oracle, torch, device_layer, x, sel_h, wts_h, sample)
    got = out.cpu().numpy()[sample]
    err = np.abs(got - ref)
    bad = err > ABS + REL * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside tolerance, max abs err {err.max()}"
    assert err.max() <= 1e-5 * np.abs(ref).max()  # only the down projection's summation order differs
    assert bool(torch.isfinite(out).all())
    K.close()


@pytest.mark.parametrize("T", [1, 8, 64])
def test_decode_layer_256_experts(torch_cuda, oracle, device_layer, T):
    """The decode workloads as benchmarked (batch 1, 8, 64; N(0,1) logits; decode kernels): bit-identical to the oracle."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import LAYOUT_ROWSOA, MoeKernels, MoeLayer

    rng = np.random.default_rng(500 + T)
    x = F.bf16_round(rng.standard_normal((T, N_EMBD)).astype(np.float32))
    logits = rng.standard_normal((T, N_E)).astype(np.float32)
    K = MoeKernels(device=0, max_tokens=64)
    layer = MoeLayer(K, *device_layer, layout=LAYOUT_ROWSOA)
    sel = torch.zeros((T, K_USED), dtype=torch.int32, device="cuda")
    wts = torch.zeros((T, K_USED), dtype=torch.float32, device="cuda")
    out = layer.forward(torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda(), selected_out=sel, weights_out=wts)
    assert K.device_status() == 0
    sel_h, wts_h = sel.cpu().numpy(), wts.cpu().numpy()
    _, ref_sel, ref_w = oracle.router_select(logits, k=K_USED)
    assert np.array_equal(sel_h, ref_sel) and np.array_equal(wts_h, ref_w)
    ref, _ = _oracle_sample(oracle, torch, device_layer, x, sel_h, wts_h, np.arange(T))
    got = out.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), f"max abs err {np.abs(got - ref).max()}"
    K.close()


@pytest.mark.parametrize("T,layout", [(16, "rowsoa"), (40, "native"), (100, "rowsoa")])
def test_decode_layer_skewed_routing_twice(torch_cuda, oracle, device_layer, T, layout):
    """Decode kernels with many tokens on the same few experts (Zipf s = 1.1 popularity): from 16 tokens on the pairs are
    sorted by expert and walked in aligned runs, and the gate/up kernel quantises mid block by block as the blocks fill
    up. Bit-identical to the oracle, and the same again from a second call on the same handle (the block counters must
    come back to zero)."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA, MoeKernels, MoeLayer

    rng = np.random.default_rng(900 + T)
    x = F.bf16_round(rng.standard_normal((T, N_EMBD)).astype(np.float32))
    logits = F.zipf_logits(rng, T, N_E, s=1.1)
    K = MoeKernels(device=0, max_tokens=128)
    layer = MoeLayer(K, *device_layer, layout=LAYOUT_ROWSOA if layout == "rowsoa" else LAYOUT_NATIVE)
    sel = torch.zeros((T, K_USED), dtype=torch.int32, device="cuda")
    wts = torch.zeros((T, K_USED), dtype=torch.float32, device="cuda")
    xd, ld = torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda()
    out1 = layer.forward(xd, ld, selected_out=sel, weights_out=wts).clone()
    out2 = layer.forward(xd, ld, selected_out=sel, weights_out=wts).clone()
    assert K.device_status() == 0
    sel_h, wts_h = sel.cpu().numpy(), wts.cpu().numpy()
    _, ref_sel, ref_w = oracle.router_select(logits, k=K_USED)
    assert np.array_equal(sel_h, ref_sel) and np.array_equal(wts_h, ref_w)
    assert np.bincount(sel_h.reshape(-1), minlength=N_E).max() >= T // 3, "the routing should pile tokens on one expert"
    ref, _ = _oracle_sample(oracle, torch, device_layer, x, sel_h, wts_h, np.arange(T))
    got1, got2 = out1.cpu().numpy(), out2.cpu().numpy()
    assert np.array_equal(got1.view(np.uint32), ref.view(np.uint32)), f"max abs err {np.abs(got1 - ref).max()}"
    assert np.array_equal(got2.view(np.uint32), got1.view(np.uint32))
    K.close()
