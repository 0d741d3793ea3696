"""dsmoe_ffn_forward: shared expert, router logits, routing (score / bias / hash), routed experts, slot sum and the
hyper-connection merge in one call, against the oracle's restatement of each step (engine/src/session.rs:1894-2180)."""
import numpy as np
import pytest

from deepseek_rs_b200 import formats as F

pytestmark = pytest.mark.gpu

N_EMBD, N_FF, N_E, K_USED, N_HC = 4096, 2048, 32, 6, 4
MIX_HC = 2 * N_HC + N_HC * N_HC


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _shared_oracle(oracle, x, sg, su, sd):
    xq, xs = oracle.quantize_q8_0(x)
    g = oracle.matmul_q8_0(sg, xq, xs, N_EMBD, N_FF)
    u = oracle.matmul_q8_0(su, xq, xs, N_EMBD, N_FF)
    mid = oracle.swiglu(g, u, 10.0, 1.0)
    mq, ms = oracle.quantize_q8_0(mid)
    return oracle.matmul_q8_0(sd, mq, ms, N_FF, N_EMBD)


def _routed_oracle(oracle, x, lw, sel, w):
    xq = oracle.q8k_quantize(x)
    _, _, mid = oracle.gate_up_mid(lw.gate, lw.up, xq, sel, w, N_FF, N_EMBD // 256)
    return oracle.down_sum(lw.down, oracle.q8k_quantize(mid), sel, N_EMBD, N_FF // 256)


@pytest.mark.parametrize("T,batched,mode,bf16", [(1, False, "score", False), (5, False, "bias", True), (3, False, "hash", False),
                                                 (40, True, "score", True), (33, True, "hash", False)])
def test_ffn_forward_matches_the_oracle(torch_cuda, oracle, T, batched, mode, bf16):
    torch = torch_cuda
    import os

    from deepseek_rs_b200.kernels import LAYOUT_ROWSOA, MoeKernels, MoeLayer

    rng = np.random.default_rng(1000 + T)
    lw = F.ExpertLayer(seed=71, n_expert=N_E)
    router = (rng.standard_normal((N_E, N_EMBD)) * 0.05).astype(np.float16)
    bias = (rng.standard_normal(N_E) * 0.3).astype(np.float32) if mode == "bias" else None
    hash_rows = 50
    table = np.stack([rng.permutation(N_E)[:K_USED] for _ in range(hash_rows)]).astype(np.int32) if mode == "hash" else None
    sg = F.random_q8_0(rng, N_FF * (N_EMBD // 32))
    su = F.random_q8_0(rng, N_FF * (N_EMBD // 32))
    sd = F.random_q8_0(rng, N_EMBD * (N_FF // 32))
    x = F.bf16_round(rng.standard_normal((T, N_EMBD)).astype(np.float32))
    tokens = rng.integers(-2, hash_rows + 3, size=T).astype(np.int32)  # out-of-range ids fall back to row 0
    residual = rng.standard_normal((T, N_HC, N_EMBD)).astype(np.float32)
    split = rng.standard_normal((T, MIX_HC)).astype(np.float32)

    # oracle, step by step
    logits = oracle.matmul_f16(router.view(np.uint16), x)
    _, sel, w = oracle.router_select(logits, k=K_USED, bias=bias, hash_table=table, tokens=tokens if mode == "hash" else None)
    routed = _routed_oracle(oracle, x, lw, sel, w)
    shared = _shared_oracle(oracle, x, sg, su, sd)
    out_hc = oracle.hc_expand(shared, routed, residual, split)

    if batched:
        os.environ["DSMOE_PREFILL_MIN_TOKENS"] = "1"
    try:
        K = MoeKernels(device=0, n_expert=N_E, max_tokens=T)
    finally:
        os.environ.pop("DSMOE_PREFILL_MIN_TOKENS", None)
    layer = MoeLayer(K, lw.gate, lw.up, lw.down, layout=LAYOUT_ROWSOA)
    keep = [dev(torch, router.view(np.uint16)), None if bias is None else dev(torch, bias),
            None if table is None else dev(torch, table), dev(torch, sg.reshape(-1)), dev(torch, su.reshape(-1)),
            dev(torch, sd.reshape(-1))]
    K.layer_register_extras(0, *keep)
    xd = dev(torch, x)
    if bf16:
        xd = xd.to(torch.bfloat16)  # exact: x holds bf16 values
    r_out = torch.zeros((T, N_EMBD), device="cuda")
    s_out = torch.zeros((T, N_EMBD), device="cuda")
    h_out = torch.zeros((T, N_HC, N_EMBD), device="cuda")
    sel_d = torch.zeros((T, K_USED), dtype=torch.int32, device="cuda")
    w_d = torch.zeros((T, K_USED), device="cuda")
    K.ffn_forward(0, xd, r_out, tokens=dev(torch, tokens) if mode == "hash" else None, hash_mode=int(mode == "hash"),
                  shared_out=s_out, residual_hc=dev(torch, residual), hc_split=dev(torch, split), out_hc=h_out,
                  selected_out=sel_d, weights_out=w_d)
    assert K.device_status() == 0
    assert np.array_equal(sel_d.cpu().numpy(), sel)
    assert np.array_equal(w_d.cpu().numpy().view(np.uint32), w.view(np.uint32))
    assert np.array_equal(s_out.cpu().numpy().view(np.uint32), shared.view(np.uint32)), "shared expert differs"
    got_r, got_h = r_out.cpu().numpy(), h_out.cpu().numpy()
    if not batched:  # decode kernels: bit-identical
        assert np.array_equal(got_r.view(np.uint32), routed.view(np.uint32))
        assert np.array_equal(got_h.view(np.uint32), out_hc.view(np.uint32))
    else:            # grouped GEMM: the down projection sums its superblocks in ascending order
        assert np.all(np.abs(got_r - routed) <= 1e-4 + 1e-3 * np.abs(routed))
        assert np.abs(got_r - routed).max() <= 1e-5 * np.abs(routed).max()
        # the merge itself is exact on the routed values the kernel produced
        assert np.array_equal(got_h.view(np.uint32), oracle.hc_expand(shared, got_r, residual, split).view(np.uint32))

    # a second call that only wants the routed output and brings its own logits gives the same routed rows
    r2 = torch.zeros((T, N_EMBD), device="cuda")
    if mode == "score":
        K.ffn_forward(0, xd, r2, logits=dev(torch, logits))
        torch.cuda.synchronize()
        assert torch.equal(r2, r_out)
    K.close()


def test_hc_expand_kernel_bit_exact(torch_cuda, oracle):
    torch = torch_cuda
    from deepseek_rs_b200.kernels import MoeKernels

    K = MoeKernels(device=0, n_expert=32, max_tokens=1)
    rng = np.random.default_rng(9)
    for T, n_embd, n_hc, has_add in ((1, 4096, 4, 1), (3, 100, 4, 0), (2, 64, 2, 1)):
        mix = 2 * n_hc + n_hc * n_hc + 3  # a row stride longer than the data, as MIX_HC may be
        bo = rng.standard_normal((T, n_embd)).astype(np.float32)
        ba = rng.standard_normal((T, n_embd)).astype(np.float32)
        res = rng.standard_normal((T, n_hc, n_embd)).astype(np.float32)
        sp = rng.standard_normal((T, mix)).astype(np.float32)
        want = oracle.hc_expand(bo, ba if has_add else None, res, sp)
        out = torch.zeros((T, n_hc, n_embd), device="cuda")
        K.hc_expand(dev(torch, bo), dev(torch, ba), dev(torch, res), dev(torch, sp), out, n_embd, n_hc, T, mix, has_add)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    K.close()


def test_ffn_pre_norm_producer_bit_exact(torch_cuda, oracle):
    """hc_split_weighted_sum_norm_fused (the kernel that produces ffn_norm and hc_split) against the oracle, then the
    whole neighbourhood of the path in sequence: producer -> dsmoe_ffn_forward -> merged residual streams."""
    torch = torch_cuda
    from deepseek_rs_b200.kernels import MoeKernels

    K = MoeKernels(device=0, n_expert=32, max_tokens=4)
    rng = np.random.default_rng(77)
    for T, n_embd in ((1, 4096), (3, 1000)):
        mix = rng.standard_normal((T, 24)).astype(np.float32) * 2
        scale = np.array([0.7, 1.3, 0.9], np.float32)
        base = (rng.standard_normal(24) * 0.5).astype(np.float32)
        res = rng.standard_normal((T, 4, n_embd)).astype(np.float32)
        nw = (1.0 + 0.1 * rng.standard_normal(n_embd)).astype(np.float32)
        want_split, want_out, want_norm = oracle.hc_split_weighted_sum_norm(mix, scale, base, res, nw, 20, 1e-6, 1e-6)
        split = torch.zeros((T, 24), device="cuda")
        out = torch.zeros((T, n_embd), device="cuda")
        norm = torch.zeros((T, n_embd), device="cuda")
        K.hc_split_weighted_sum_norm_fused(dev(torch, mix), dev(torch, scale), dev(torch, base), dev(torch, res), dev(torch, nw),
                                           split, out, norm, n_embd, 4, T, 20, 1e-6, 1e-6)
        torch.cuda.synchronize()
        assert np.array_equal(split.cpu().numpy().view(np.uint32), want_split.view(np.uint32))
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want_out.view(np.uint32))
        assert np.array_equal(norm.cpu().numpy().view(np.uint32), want_norm.view(np.uint32))
        # the comb matrix is doubly stochastic up to the eps terms
        comb = want_split[:, 8:].reshape(T, 4, 4)
        assert np.allclose(comb.sum(axis=1), 1.0, atol=1e-4) and np.allclose(comb.sum(axis=2), 1.0, atol=1e-3)
    K.close()
