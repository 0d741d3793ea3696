"""The GPU baseline (baseline/ref_mapping.cu, a restatement of the reference kernels' thread mapping) against the CPU
oracle. The baseline keeps the reference's arithmetic order, so it has to agree with the oracle bit for bit; that is
what makes its timing a fair stand-in for the reference's kernels in bench.py."""
import numpy as np
import pytest

from deepseek_rs_b200 import formats as F

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return torch


@pytest.fixture(scope="module")
def refmap(torch_cuda):
    from baseline import RefMapping

    return RefMapping()


def test_q8k_quantize_matches_oracle(torch_cuda, oracle, refmap):
    torch = torch_cuda
    rng = np.random.default_rng(5)
    x = rng.standard_normal((7, 4096)).astype(np.float32)
    x[2, 256:512] = 0.0                      # a zero block
    x[3, 0] = x[3, 1] = 3.5                  # equal maxima: the tree's tie rule decides
    x[4, 10], x[4, 200] = -2.25, 2.25
    out = torch.zeros((7, 16, 292), dtype=torch.uint8, device="cuda")
    refmap.q8k_quantize(dev(torch, x), out, 4096, 7)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.q8k_quantize(x))


def test_gate_up_and_down_match_oracle(torch_cuda, oracle, refmap):
    torch = torch_cuda
    n_e, T, k = 8, 3, 6
    lw = F.ExpertLayer(seed=11, n_expert=n_e)
    rng = np.random.default_rng(12)
    x = F.bf16_round(rng.standard_normal((T, 4096)).astype(np.float32))
    sel = np.stack([rng.permutation(n_e)[:k] for _ in range(T)]).astype(np.int32)
    w = rng.uniform(0.1, 0.4, size=(T, k)).astype(np.float32)
    xq = oracle.q8k_quantize(x)
    g_ref, u_ref, m_ref = oracle.gate_up_mid(lw.gate, lw.up, xq, sel, w, 2048, 16)
    g = torch.empty((T * k, 2048), device="cuda")
    u, m = torch.empty_like(g), torch.empty_like(g)
    refmap.gate_up_mid(dev(torch, lw.gate), dev(torch, lw.up), dev(torch, xq), dev(torch, sel), dev(torch, w), g, u, m,
                       2048 * 16 * 66, 16 * 66, 16, 2048, k, T, 10.0)
    torch.cuda.synchronize()
    assert np.array_equal(g.cpu().numpy(), g_ref) and np.array_equal(u.cpu().numpy(), u_ref)
    assert np.array_equal(m.cpu().numpy(), m_ref)
    midq = oracle.q8k_quantize(m_ref)
    want = oracle.down_sum(lw.down, midq, sel, 4096, 8)
    down_d, midq_d = dev(torch, lw.down), dev(torch, midq)
    for t in range(T):  # the reference's kernel sums the six slots of ONE token
        out = torch.empty(4096, device="cuda")
        refmap.down_sum6(down_d, midq_d[t * k:(t + 1) * k], dev(torch, sel[t]), out, 4096 * 8 * 84, 8 * 84, 8, 4096)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want[t])


def test_per_token_loop_matches_oracle_layer(torch_cuda, oracle, refmap):
    torch = torch_cuda
    n_e, T = 16, 4
    lw = F.ExpertLayer(seed=21, n_expert=n_e)
    rng = np.random.default_rng(22)
    x = F.bf16_round(rng.standard_normal((T, 4096)).astype(np.float32))
    logits = rng.standard_normal((T, n_e)).astype(np.float32)
    want, sel, w = oracle.moe_layer(x, logits, lw.gate, lw.up, lw.down, k=6)
    out = torch.empty((T, 4096), device="cuda")
    xq = torch.empty(16 * 292, dtype=torch.uint8, device="cuda")
    mid = torch.empty((6, 2048), device="cuda")
    midq = torch.empty(6 * 8 * 292, dtype=torch.uint8, device="cuda")
    refmap.tokens(dev(torch, lw.gate), dev(torch, lw.up), dev(torch, lw.down), dev(torch, x), dev(torch, sel), dev(torch, w),
                  xq, mid, midq, out, 4096, 2048, T, 10.0)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)


def test_batched_sorted_form_matches_oracle_layer(torch_cuda, oracle, refmap):
    """The reference's unused batched formulation (count / prefix / scatter of pairs into expert order, sorted gate/up
    and down kernels, slot sum; engine/src/kernels/moe.rs:299-362, 721-916, 983-1005): the atomic scatter makes the
    order inside an expert arbitrary, the result does not depend on it and equals the oracle bit for bit."""
    torch = torch_cuda
    n_e, T = 16, 9
    lw = F.ExpertLayer(seed=23, n_expert=n_e)
    rng = np.random.default_rng(24)
    x = F.bf16_round(rng.standard_normal((T, 4096)).astype(np.float32))
    logits = rng.standard_normal((T, n_e)).astype(np.float32)
    want, sel, w = oracle.moe_layer(x, logits, lw.gate, lw.up, lw.down, k=6)
    out = torch.empty((T, 4096), device="cuda")
    scratch = refmap.batched(dev(torch, lw.gate), dev(torch, lw.up), dev(torch, lw.down), dev(torch, x), dev(torch, sel),
                             dev(torch, w), out, 4096, 2048, T, 10.0)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)
    sorted_pairs = scratch[4][770:770 + T * 6].cpu().numpy()
    assert sorted(sorted_pairs.tolist()) == list(range(T * 6))
    assert np.all(np.diff(sel.reshape(-1)[sorted_pairs]) >= 0)  # grouped by expert
