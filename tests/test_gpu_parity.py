"""GPU parity: every kernel of the routed-expert path, called through the C ABI, against the CPU oracle on the same
seeded inputs.

Bars: dequantised weights, Q8_K blocks and router indices bit-exact; expert outputs within rel 1e-3 / abs 1e-4
(they are in fact bit-identical to the oracle, which the tests also record, because the kernels keep the reference's
f32 summation order)."""
import numpy as np
import pytest

from deepseek_rs_b200 import formats as F

pytestmark = pytest.mark.gpu

REL, ABS = 1e-3, 1e-4  # tolerance for expert outputs (f32 accumulate)


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return torch


def _make_kernels(tma: bool, **kw):
    """A handle with the bulk-copy (TMA) staging kernels on or off; the switch is read at handle creation."""
    import os

    from deepseek_rs_b200.kernels import MoeKernels

    old = os.environ.get("DSMOE_DISABLE_TMA")
    os.environ["DSMOE_DISABLE_TMA"] = "0" if tma else "1"
    try:
        return MoeKernels(device=0, **kw)
    finally:
        if old is None:
            del os.environ["DSMOE_DISABLE_TMA"]
        else:
            os.environ["DSMOE_DISABLE_TMA"] = old


@pytest.fixture(scope="module")
def K(torch_cuda):
    return _make_kernels(True, max_tokens=64)


@pytest.fixture(scope="module")
def K_plain(torch_cuda):
    return _make_kernels(False, max_tokens=64)


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def assert_close(got, ref):
    err = np.abs(got - ref)
    assert np.all(err <= ABS + REL * np.abs(ref)), f"max abs err {err.max()}"


# ---------------------------------------------------------------------------------------------------------------
# dequantised weights: bit-exact
# ---------------------------------------------------------------------------------------------------------------

def test_dequant_iq2xxs_bit_exact(torch_cuda, K, oracle):
    torch = torch_cuda
    rng = np.random.default_rng(1)
    blocks = F.random_iq2xxs(rng, 4096)
    blocks[:64, 0:2] = np.frombuffer(np.arange(1, 65, dtype=np.uint16).tobytes(), np.uint8).reshape(64, 2)  # subnormal d
    out = torch.empty(4096 * 256, dtype=torch.float32, device="cuda")
    K.dequant_iq2xxs(dev(torch, blocks.reshape(-1)), 4096, out)
    ref = oracle.dequant_iq2xxs(blocks)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    assert np.all(ref[:64 * 256] == 0.0)  # subnormal scales are flushed


def test_dequant_q2k_bit_exact(torch_cuda, K, oracle):
    torch = torch_cuda
    rng = np.random.default_rng(2)
    blocks = F.random_q2k(rng, 4096)
    blocks[:32, 80:82] = np.frombuffer(np.arange(1, 33, dtype=np.uint16).tobytes(), np.uint8).reshape(32, 2)
    out = torch.empty(4096 * 256, dtype=torch.float32, device="cuda")
    K.dequant_q2k(dev(torch, blocks.reshape(-1)), 4096, out)
    ref = oracle.dequant_q2k(blocks)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


def test_ieee_f16_switch(torch_cuda, oracle):
    torch = torch_cuda
    from deepseek_rs_b200.kernels import MoeKernels

    Ki = MoeKernels(device=0, f16_ieee=True, max_tokens=1)
    rng = np.random.default_rng(3)
    blocks = F.random_iq2xxs(rng, 256)
    blocks[:, 0:2] = np.frombuffer(rng.integers(1, 0x400, 256, dtype=np.uint16).tobytes(), np.uint8).reshape(256, 2)
    out = torch.empty(256 * 256, dtype=torch.float32, device="cuda")
    Ki.dequant_iq2xxs(dev(torch, blocks.reshape(-1)), 256, out)
    ref = oracle.dequant_iq2xxs(blocks, ieee=True)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    assert np.any(ref != 0.0)
    Ki.close()


@pytest.mark.parametrize("xb", [1, 3, 16])
def test_relayout_iq2xxs_is_a_row_permutation(torch_cuda, K, xb):
    torch = torch_cuda
    rng = np.random.default_rng(4)
    rows = 37
    src = rng.integers(0, 256, rows * xb * 66, dtype=np.uint8)
    s = dev(torch, src)
    d = torch.zeros_like(s)
    back = torch.zeros_like(s)
    K.relayout_iq2xxs(s, d, rows, xb)
    K.relayout_iq2xxs(d, back, rows, xb, inverse=True)
    assert torch.equal(back, s)
    dn = d.cpu().numpy().reshape(rows, xb * 66)
    sn = src.reshape(rows, xb, 66)
    assert np.array_equal(dn[:, :2 * xb].reshape(rows, xb, 2), sn[:, :, :2])
    assert np.array_equal(dn[:, 2 * xb:].reshape(rows, xb, 64), sn[:, :, 2:])


@pytest.mark.parametrize("mb", [1, 5, 8])
def test_relayout_q2k_is_a_row_permutation(torch_cuda, K, mb):
    torch = torch_cuda
    rng = np.random.default_rng(5)
    rows = 29
    src = rng.integers(0, 256, rows * mb * 84, dtype=np.uint8)
    s = dev(torch, src)
    d = torch.zeros_like(s)
    back = torch.zeros_like(s)
    K.relayout_q2k(s, d, rows, mb)
    K.relayout_q2k(d, back, rows, mb, inverse=True)
    assert torch.equal(back, s)
    dn = d.cpu().numpy().reshape(rows, mb * 84)
    sn = src.reshape(rows, mb, 84)
    assert np.array_equal(dn[:, :16 * mb].reshape(rows, mb, 16), sn[:, :, :16])
    assert np.array_equal(dn[:, 16 * mb:80 * mb].reshape(rows, mb, 64), sn[:, :, 16:80])
    assert np.array_equal(dn[:, 80 * mb:].reshape(rows, mb, 4), sn[:, :, 80:])


# ---------------------------------------------------------------------------------------------------------------
# Q8_K quantiser: bit-exact
# ---------------------------------------------------------------------------------------------------------------

def _q8k_gpu(torch, K, x):
    rows, in_dim = x.shape
    out = torch.zeros((rows, in_dim // 256, 292), dtype=torch.uint8, device="cuda")
    K.q8k_quantize(dev(torch, x), out, in_dim, rows)
    return out.cpu().numpy()


def test_q8k_quantize_bit_exact_random(torch_cuda, K, oracle):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((48, 4096)).astype(np.float32)
    x[3] *= 1e-30
    x[4] *= 1e30
    x[5, 256:512] = 0.0  # an all-zero block
    x[6] = 0.0
    assert np.array_equal(_q8k_gpu(torch_cuda, K, x), oracle.q8k_quantize(x))


def test_q8k_quantize_ties_and_signs(torch_cuda, K, oracle):
    rng = np.random.default_rng(7)
    # many equal magnitudes with both signs: the winner of the reference's tree decides the sign of d
    x = rng.choice(np.array([-2.0, 2.0, -1.0, 1.0, 0.5], np.float32), size=(64, 512)).astype(np.float32)
    x[0, :256] = -3.0
    x[1, :256] = 3.0
    x[2, 255] = -7.0
    x[3, 0] = 7.0
    got, ref = _q8k_gpu(torch_cuda, K, x), oracle.q8k_quantize(x)
    assert np.array_equal(got, ref)
    # rounding is half away from zero: 0.5 * iscale lands on .5 boundaries often in this set
    vals = np.linspace(-1.0, 1.0, 256, dtype=np.float32)[None, :].repeat(4, 0)
    assert np.array_equal(_q8k_gpu(torch_cuda, K, vals), oracle.q8k_quantize(vals))


def test_q8k_quantize_empty(torch_cuda, K):
    torch = torch_cuda
    K.q8k_quantize(torch.empty((0, 256), device="cuda"), torch.empty((0,), dtype=torch.uint8, device="cuda"), 256, 0)


# ---------------------------------------------------------------------------------------------------------------
# router: indices and weights bit-exact
# ---------------------------------------------------------------------------------------------------------------

def _router_gpu(torch, K, logits, bias=None, hash_table=None, tokens=None, token_scalar=0):
    T, E = logits.shape
    k = K.cfg.n_expert_used
    probs = torch.zeros((T, E), dtype=torch.float32, device="cuda")
    sel = torch.zeros((T, k), dtype=torch.int32, device="cuda")
    w = torch.zeros((T, k), dtype=torch.float32, device="cuda")
    K.router_select_parallel(dev(torch, logits), None if bias is None else dev(torch, bias),
                             None if hash_table is None else dev(torch, hash_table),
                             None if tokens is None else dev(torch, tokens), probs, sel, w, token_scalar,
                             0 if hash_table is None else hash_table.shape[0], T, int(bias is not None),
                             int(hash_table is not None))
    return probs.cpu().numpy(), sel.cpu().numpy(), w.cpu().numpy()


def _assert_router_equal(got, ref):
    assert np.array_equal(got[1], ref[1]), "selected experts differ"
    nan = np.isnan(ref[0])
    assert np.array_equal(np.isnan(got[0]), nan), "probs differ in NaN positions"
    assert np.array_equal(got[0][~nan].view(np.uint32), ref[0][~nan].view(np.uint32)), "probs differ"
    wnan = np.isnan(ref[2])  # only reachable through hash routing onto an expert whose logit is NaN
    assert np.array_equal(np.isnan(got[2]), wnan), "weights differ in NaN positions"
    assert np.array_equal(got[2][~wnan].view(np.uint32), ref[2][~wnan].view(np.uint32)), "weights differ"


def test_router_random_and_zipf(torch_cuda, K, oracle):
    rng = np.random.default_rng(8)
    logits = rng.standard_normal((64, 256)).astype(np.float32)
    _assert_router_equal(_router_gpu(torch_cuda, K, logits), oracle.router_select(logits, k=6))
    z = F.zipf_logits(rng, 4096)
    got, ref = _router_gpu(torch_cuda, K, z), oracle.router_select(z, k=6)
    _assert_router_equal(got, ref)
    assert np.allclose(got[2].sum(axis=1), 1.5, atol=1e-5)


def test_router_ties_extremes_bias_hash(torch_cuda, K, oracle):
    rng = np.random.default_rng(9)
    logits = rng.standard_normal((16, 256)).astype(np.float32)
    logits[0] = 0.25                      # all equal: lowest indices win
    logits[1, ::2] = 1.0                  # half equal
    logits[2] = -40.0                     # softplus underflow branch
    logits[3, 5] = 30.0                   # identity branch
    logits[4, 10:20] = np.nan             # never selected
    logits[5] = np.nan                    # nothing selectable -> -1, weights 0
    _assert_router_equal(_router_gpu(torch_cuda, K, logits), oracle.router_select(logits, k=6))
    bias = rng.standard_normal(256).astype(np.float32)
    bias[7] = -np.inf
    _assert_router_equal(_router_gpu(torch_cuda, K, logits, bias=bias), oracle.router_select(logits, k=6, bias=bias))
    table = rng.integers(0, 256, (50, 6)).astype(np.int32)
    table[3, 2] = -1
    tokens = rng.integers(-2, 60, 16).astype(np.int32)  # out-of-range ids fall back to row 0
    _assert_router_equal(_router_gpu(torch_cuda, K, logits, hash_table=table, tokens=tokens),
                         oracle.router_select(logits, k=6, hash_table=table, tokens=tokens))
    _assert_router_equal(_router_gpu(torch_cuda, K, logits[:1], hash_table=table, token_scalar=7),
                         oracle.router_select(logits[:1], k=6, hash_table=table, token_scalar=7))


def test_router_top8_variant(torch_cuda, oracle):
    from deepseek_rs_b200.kernels import MoeKernels

    K8 = MoeKernels(device=0, n_expert_used=8, max_tokens=1)
    logits = np.random.default_rng(10).standard_normal((33, 256)).astype(np.float32)
    _assert_router_equal(_router_gpu(torch_cuda, K8, logits), oracle.router_select(logits, k=8))
    K8.close()


# ---------------------------------------------------------------------------------------------------------------
# gate / up / mid and down
# ---------------------------------------------------------------------------------------------------------------

def _relaid(torch, K, w_np, n_rows, blocks, kind):
    s = dev(torch, w_np)
    d = torch.empty_like(s)
    (K.relayout_iq2xxs if kind == "iq2" else K.relayout_q2k)(s, d, n_rows, blocks)
    return d


@pytest.mark.parametrize("path", ["tma", "plain"])
@pytest.mark.parametrize("layout", ["native", "rowsoa"])
@pytest.mark.parametrize("xb,n_ff,T,n_e", [(16, 2048, 3, 4), (16, 200, 2, 3), (1, 40, 2, 3), (3, 17, 1, 2), (8, 64, 4, 5),
                                           (20, 24, 2, 2)])
def test_gate_up_mid(torch_cuda, K, K_plain, oracle, path, layout, xb, n_ff, T, n_e):
    torch = torch_cuda
    if path == "plain":
        K = K_plain
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA

    rng = np.random.default_rng(100 + xb + n_ff)
    k = 6
    gate = F.random_iq2xxs(rng, n_e * n_ff * xb).reshape(-1)
    up = F.random_iq2xxs(rng, n_e * n_ff * xb).reshape(-1)
    x = rng.standard_normal((T, xb * 256)).astype(np.float32) * 30.0  # large enough that the clamp at 10 bites
    xq = oracle.q8k_quantize(x)
    sel = rng.integers(0, n_e, (T, k)).astype(np.int32)
    sel[0, 1] = -1  # clamped to expert 0 as in the reference
    w = rng.random((T, k)).astype(np.float32)
    rg, ru, rm = oracle.gate_up_mid(gate, up, xq, sel, w, n_ff, xb, clamp=10.0)
    if layout == "rowsoa":
        dg, du = _relaid(torch, K, gate, n_e * n_ff, xb, "iq2"), _relaid(torch, K, up, n_e * n_ff, xb, "iq2")
        lay = LAYOUT_ROWSOA
    else:
        dg, du, lay = dev(torch, gate), dev(torch, up), LAYOUT_NATIVE
    outs = [torch.zeros((T * k, n_ff), dtype=torch.float32, device="cuda") for _ in range(3)]
    K.moe_gate_up_mid_qwarp32(dg, du, dev(torch, xq), dev(torch, sel), dev(torch, w), outs[0], outs[1], outs[2],
                              n_ff * xb * 66, xb * 66, xb, n_ff, k, 10.0, n_tokens=T, layout=lay)
    g, u, m = (o.cpu().numpy() for o in outs)
    for got, ref in ((g, rg), (u, ru), (m, rm)):
        assert_close(got, ref)
    assert rg.max() <= 10.0 and np.abs(ru).max() <= 10.0
    bit_exact = all(np.array_equal(a.view(np.uint32), b.view(np.uint32)) for a, b in ((g, rg), (u, ru), (m, rm)))
    assert bit_exact, "within tolerance but not bit-identical to the oracle's summation order"
    # gate_out / up_out are optional
    m2 = torch.zeros_like(outs[2])
    K.moe_gate_up_mid_qwarp32(dg, du, dev(torch, xq), dev(torch, sel), dev(torch, w), None, None, m2, n_ff * xb * 66,
                              xb * 66, xb, n_ff, k, 10.0, n_tokens=T, layout=lay)
    assert torch.equal(m2, outs[2])


@pytest.mark.parametrize("path", ["tma", "plain"])
@pytest.mark.parametrize("layout", ["native", "rowsoa"])
@pytest.mark.parametrize("mb,out_dim,T,n_e,k", [(8, 4096, 2, 4, 6), (8, 100, 3, 3, 6), (1, 33, 2, 2, 6), (5, 20, 1, 3, 4),
                                                (16, 64, 4, 2, 1), (9, 31, 2, 2, 8), (8, 4096, 20, 3, 8)])
def test_down_and_down_sum(torch_cuda, K, K_plain, oracle, path, layout, mb, out_dim, T, n_e, k):
    torch = torch_cuda
    if path == "plain":
        K = K_plain
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA

    rng = np.random.default_rng(200 + mb + out_dim)
    down = F.random_q2k(rng, n_e * out_dim * mb).reshape(-1)
    mid = rng.standard_normal((T * k, mb * 256)).astype(np.float32)
    midq = oracle.q8k_quantize(mid)
    sel = rng.integers(0, n_e, (T, k)).astype(np.int32)
    ref_pair = oracle.down(down, midq, sel, out_dim, mb)
    ref_sum = oracle.down_sum(down, midq, sel, out_dim, mb)
    if layout == "rowsoa":
        dd, lay = _relaid(torch, K, down, n_e * out_dim, mb, "q2k"), LAYOUT_ROWSOA
    else:
        dd, lay = dev(torch, down), LAYOUT_NATIVE
    o_pair = torch.zeros((T * k, out_dim), dtype=torch.float32, device="cuda")
    o_sum = torch.zeros((T, out_dim), dtype=torch.float32, device="cuda")
    K.moe_down_qwarp32(dd, dev(torch, midq), dev(torch, sel), o_pair, out_dim * mb * 84, mb * 84, mb, out_dim, k,
                       n_tokens=T, layout=lay)
    K.moe_down_sum6_qwarp32(dd, dev(torch, midq), dev(torch, sel), o_sum, out_dim * mb * 84, mb * 84, mb, out_dim,
                            n_expert=k, n_tokens=T, layout=lay)
    assert_close(o_pair.cpu().numpy(), ref_pair)
    assert_close(o_sum.cpu().numpy(), ref_sum)
    assert np.array_equal(o_pair.cpu().numpy().view(np.uint32), ref_pair.view(np.uint32))
    assert np.array_equal(o_sum.cpu().numpy().view(np.uint32), ref_sum.view(np.uint32))
    # moe_sum over the per-pair rows gives the same numbers as the fused sum
    o2 = torch.zeros_like(o_sum)
    K.moe_sum(o_pair, o2, out_dim, k, T)
    assert torch.equal(o2, o_sum)


# ---------------------------------------------------------------------------------------------------------------
# the benchmark's single-matrix configurations
# ---------------------------------------------------------------------------------------------------------------

def test_config_iq2xxs_matvec_2048x4096_seed0(torch_cuda, K, oracle):
    """Single IQ2_XXS matvec, W 2048 x 4096, x ~ N(0,1), one token, seed 0."""
    torch = torch_cuda
    rng = np.random.default_rng(0)
    W = F.random_iq2xxs(rng, 2048 * 16).reshape(-1)
    x = rng.standard_normal((1, 4096)).astype(np.float32)
    xq = oracle.q8k_quantize(x)
    ref = oracle.matvec_iq2xxs(W, xq, 2048, 16)
    dW = dev(torch, W)
    sel = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    w1 = torch.ones((1, 1), dtype=torch.float32, device="cuda")
    y, u, m = (torch.zeros((1, 2048), dtype=torch.float32, device="cuda") for _ in range(3))
    K.moe_gate_up_mid_qwarp32(dW, dW, dev(torch, xq), sel, w1, y, u, m, 2048 * 16 * 66, 16 * 66, 16, 2048, 1, 0.0,
                              n_tokens=1)
    assert_close(y.cpu().numpy(), ref)
    assert np.array_equal(y.cpu().numpy(), ref)
    # and the device-side quantiser feeds it the same blocks
    xq_gpu = torch.zeros((1, 16, 292), dtype=torch.uint8, device="cuda")
    K.q8k_quantize(dev(torch, x), xq_gpu, 4096, 1)
    assert np.array_equal(xq_gpu.cpu().numpy(), xq)


@pytest.mark.parametrize("batch", [1, 4, 16])
def test_config_q2k_matvec_2048x4096(torch_cuda, K, oracle, batch):
    """Q2_K matvec, W 2048 x 4096, batch 1 / 4 / 16 tokens, seed 0."""
    torch = torch_cuda
    rng = np.random.default_rng(0)
    W = F.random_q2k(rng, 2048 * 16).reshape(-1)
    x = rng.standard_normal((batch, 4096)).astype(np.float32)
    xq = oracle.q8k_quantize(x)
    ref = oracle.matvec_q2k(W, xq, 2048, 16)
    sel = torch.zeros((batch, 1), dtype=torch.int32, device="cuda")
    y = torch.zeros((batch, 2048), dtype=torch.float32, device="cuda")
    K.moe_down_qwarp32(dev(torch, W), dev(torch, xq), sel, y, 2048 * 16 * 84, 16 * 84, 16, 2048, 1, n_tokens=batch)
    assert_close(y.cpu().numpy(), ref)
    assert np.array_equal(y.cpu().numpy(), ref)


# ---------------------------------------------------------------------------------------------------------------
# the whole routed-expert step (tier 2)
# ---------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("layout", ["native", "rowsoa"])
@pytest.mark.parametrize("T", [1, 8])
def test_moe_forward_layer(torch_cuda, oracle, layout, T):
    """hidden 4096, width 2048, top-6, 32 experts (full-size experts, fewer of them so the CPU oracle stays quick)."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA, MoeKernels, MoeLayer

    n_e = 32
    Kl = MoeKernels(device=0, n_expert=n_e, max_tokens=8)
    layer_w = F.ExpertLayer(seed=11, n_expert=n_e)
    rng = np.random.default_rng(12)
    x = F.bf16_round(rng.standard_normal((T, 4096)).astype(np.float32))
    logits = rng.standard_normal((T, n_e)).astype(np.float32)
    ref_out, ref_sel, ref_w = oracle.moe_layer(x, logits, layer_w.gate, layer_w.up, layer_w.down, k=6)
    layer = MoeLayer(Kl, layer_w.gate, layer_w.up, layer_w.down,
                     layout=LAYOUT_ROWSOA if layout == "rowsoa" else LAYOUT_NATIVE)
    sel = torch.zeros((T, 6), dtype=torch.int32, device="cuda")
    w = torch.zeros((T, 6), dtype=torch.float32, device="cuda")
    out = layer.forward(dev(torch, x), dev(torch, logits), selected_out=sel, weights_out=w)
    assert np.array_equal(sel.cpu().numpy(), ref_sel)
    assert np.array_equal(w.cpu().numpy(), ref_w)
    assert_close(out.cpu().numpy(), ref_out)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref_out.view(np.uint32))
    assert Kl.device_status() == 0  # no bounded wait expired
    # host-buffer entry point gives the same result
    xh, lh = torch.from_numpy(x).pin_memory(), torch.from_numpy(logits).pin_memory()
    oh = torch.zeros((T, 4096), dtype=torch.float32).pin_memory()
    Kl.moe_forward_host(0, xh, lh, T, oh)
    assert np.array_equal(oh.numpy(), out.cpu().numpy())
    # the queued form on two handles in turn (copies of one overlap kernels of the other): same results
    K2 = MoeKernels(device=0, n_expert=n_e, max_tokens=8)
    K2.layer_register(0, layer.gate, layer.up, layer.down, layer.layout)
    outs = [torch.zeros((T, 4096), dtype=torch.float32).pin_memory() for _ in range(4)]
    for i, o in enumerate(outs):
        hnd = (Kl, K2)[i % 2]
        hnd.host_synchronize()
        hnd.moe_forward_host_async(0, xh, lh, T, o)
    Kl.host_synchronize()
    K2.host_synchronize()
    for o in outs:
        assert np.array_equal(o.numpy(), out.cpu().numpy())
    K2.close()
    # bounds and state errors come back as statuses, not crashes
    from deepseek_rs_b200.kernels import DsmoeError
    with pytest.raises(DsmoeError):
        Kl.moe_forward(0, dev(torch, np.zeros((9, 4096), np.float32)), dev(torch, np.zeros((9, n_e), np.float32)), 9,
                       torch.zeros((9, 4096), device="cuda"))
    Kl.close()


# ---------------------------------------------------------------------------------------------------------------
# batched path (tcgen05 grouped GEMM)
# ---------------------------------------------------------------------------------------------------------------

def _batched_kernels(n_e, max_tokens):
    """A handle whose tier-2 call takes the batched path from one token upwards."""
    import os

    from deepseek_rs_b200.kernels import MoeKernels

    old = os.environ.get("DSMOE_PREFILL_MIN_TOKENS")
    os.environ["DSMOE_PREFILL_MIN_TOKENS"] = "1"
    try:
        return MoeKernels(device=0, n_expert=n_e, max_tokens=max_tokens)
    finally:
        if old is None:
            del os.environ["DSMOE_PREFILL_MIN_TOKENS"]
        else:
            os.environ["DSMOE_PREFILL_MIN_TOKENS"] = old


@pytest.mark.parametrize("layout", ["rowsoa", "native"])
@pytest.mark.parametrize("T,n_e,zipf", [(5, 32, False), (70, 32, False), (200, 32, True)])
def test_moe_forward_batched_tcgen05(torch_cuda, oracle, layout, T, n_e, zipf):
    """The grouped-GEMM path against the oracle: routing bit-exact, outputs within rel 1e-3 / abs 1e-4. The gate/up
    kernel folds its per-superblock partial sums in the reference's order, so mid (and with it the Q8_K codes of mid)
    is bit-identical; the down projection sums superblocks in ascending order, which differs from the reference's
    tree in the last bits only. Zipf routing makes one expert span more than one 128-row tile and leaves others
    empty."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA, MoeLayer

    Kb = _batched_kernels(n_e, T)
    lw = F.ExpertLayer(seed=31, n_expert=n_e)
    rng = np.random.default_rng(32 + T)
    x = F.bf16_round(rng.standard_normal((T, 4096)).astype(np.float32))
    logits = F.zipf_logits(rng, T, n_e, s=2.0) if zipf else rng.standard_normal((T, n_e)).astype(np.float32)
    ref_out, ref_sel, ref_w = oracle.moe_layer(x, logits, lw.gate, lw.up, lw.down, k=6)
    layer = MoeLayer(Kb, lw.gate, lw.up, lw.down, layout=LAYOUT_ROWSOA if layout == "rowsoa" else LAYOUT_NATIVE)
    sel = torch.zeros((T, 6), dtype=torch.int32, device="cuda")
    out = layer.forward(dev(torch, x), dev(torch, logits), selected_out=sel)
    assert Kb.device_status() == 0
    assert np.array_equal(sel.cpu().numpy(), ref_sel)
    got = out.cpu().numpy()
    err = np.abs(got - ref_out)
    bad = err > ABS + REL * np.abs(ref_out)
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside tolerance, max abs err {err.max()}, ref scale {np.abs(ref_out).max()}"
    assert err.max() <= 1e-5 * np.abs(ref_out).max()  # only summation-order noise is left
    Kb.close()


def test_expert_parallel_world1_matches_forward(torch_cuda, oracle):
    """The expert-parallel host path on one rank (NCCL group of one): dispatch, owner compute through dsmoe_expert_ffn
    with an n_expert_used = 1 handle, combine. With both sides on the decode kernels it must equal the tier-2 call bit
    for bit; when the owner's 54 rows go through the grouped GEMM instead, only the down projection's summation
    order differs (last bits)."""
    torch = torch_cuda
    import os

    import torch.distributed as dist

    from deepseek_rs_b200.ep import ExpertParallelMoe, gpu_functions, gpu_sum_function
    from deepseek_rs_b200.kernels import LAYOUT_ROWSOA, MoeKernels, MoeLayer

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        n_e, T = 32, 9
        lw = F.ExpertLayer(seed=51, n_expert=n_e)
        rng = np.random.default_rng(52)
        x = dev(torch, F.bf16_round(rng.standard_normal((T, 4096)).astype(np.float32)))
        logits = dev(torch, rng.standard_normal((T, n_e)).astype(np.float32))
        K_full = MoeKernels(device=0, n_expert=n_e, max_tokens=T)
        layer = MoeLayer(K_full, lw.gate, lw.up, lw.down, layout=LAYOUT_ROWSOA)
        want = layer.forward(x, logits)
        for min_tokens, exact in (("1000000", True), ("1", False)):
            os.environ["DSMOE_PREFILL_MIN_TOKENS"] = min_tokens
            try:
                K_owner = MoeKernels(device=0, n_expert=n_e, n_expert_used=1, max_tokens=T * 6)
            finally:
                del os.environ["DSMOE_PREFILL_MIN_TOKENS"]
            MoeLayer(K_owner, lw.gate, lw.up, lw.down, layout=LAYOUT_ROWSOA)
            rf, ef = gpu_functions(K_full, K_owner)
            out, sel = ExpertParallelMoe(rf, ef, n_e, 6, 4096, sum_fn=gpu_sum_function(K_full)).forward(x, logits)
            assert K_owner.device_status() == 0
            if exact:
                assert torch.equal(out, want)
            else:
                assert float((out - want).abs().max()) <= 1e-5 * float(want.abs().max())
            K_owner.close()
        K_full.close()
    finally:
        if created:
            dist.destroy_process_group()


def test_expert_parallel_c_abi_world1_and_replicas(torch_cuda, oracle):
    """dsmoe_moe_forward_ep on a one-rank NCCL communicator: counting, placement, gather, self send/recv, owner compute
    and the indexed slot sum must reproduce dsmoe_moe_forward bit for bit when both sides run the decode kernels, with
    and without replicated experts (replicas change where a pair is computed, never the result)."""
    torch = torch_cuda
    import os

    from deepseek_rs_b200.ep import ExpertParallelHandle
    from deepseek_rs_b200.kernels import LAYOUT_ROWSOA, MoeKernels, MoeLayer

    n_e, T = 32, 9
    lw = F.ExpertLayer(seed=51, n_expert=n_e)
    rng = np.random.default_rng(52)
    x = dev(torch, F.bf16_round(rng.standard_normal((T, 4096)).astype(np.float32)))
    logits = dev(torch, rng.standard_normal((T, n_e)).astype(np.float32))
    K_full = MoeKernels(device=0, n_expert=n_e, max_tokens=T)
    layer = MoeLayer(K_full, lw.gate, lw.up, lw.down, layout=LAYOUT_ROWSOA)
    sel_want = torch.zeros((T, 6), dtype=torch.int32, device="cuda")
    want = layer.forward(x, logits, selected_out=sel_want)
    ge, de = lw.gate_expert_bytes, lw.down_expert_bytes
    for replicas in ([], [3, 17, 4]):
        os.environ["DSMOE_PREFILL_MIN_TOKENS"] = "1000000"  # owner side on the decode kernels as well
        try:
            K = MoeKernels(device=0, n_expert=n_e, max_tokens=T)
            ep = ExpertParallelHandle(K, 0, 1, max_replicas=32)
        finally:
            del os.environ["DSMOE_PREFILL_MIN_TOKENS"]
        # shard = all 32 experts, then the replica slots (unused slots stay zero)
        def shard(t, per):
            buf = torch.zeros((n_e + 32) * per, dtype=torch.uint8, device="cuda")
            buf[: n_e * per] = t
            for i, e in enumerate(replicas):
                buf[(n_e + i) * per:(n_e + i + 1) * per] = t[e * per:(e + 1) * per]
            return buf
        g, u, d = shard(layer.gate, ge), shard(layer.up, ge), shard(layer.down, de)
        ep.layer_register(0, g, u, d, LAYOUT_ROWSOA)
        ep.set_replicas(replicas)
        sel = torch.zeros((T, 6), dtype=torch.int32, device="cuda")
        out = ep.forward(0, x, logits, selected_out=sel)
        torch.cuda.synchronize()
        assert K.device_status() == 0
        assert torch.equal(sel, sel_want)
        assert torch.equal(out, want)
        assert sum(ep.last_recv_rows()) == T * 6
        counts = ep.expert_counts()
        assert int(counts.sum()) == T * 6 and torch.equal(counts, torch.bincount(sel_want.flatten().cpu().long(), minlength=n_e))
        K.close()
    K_full.close()
