"""FP8 E4M3 block-scaled projection against the oracle's definition (the reference has no FP8 GEMM: parity unpinned).

Codes and scales are bit-exact against the oracle's quantiser. GEMM outputs (bf16) are held to rel 2e-2 against the
oracle's f64 evaluation, with an absolute floor of 1e-3 x rms(reference) for outputs that cancel to almost zero."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from deepseek_rs_b200.kernels import MoeKernels

    return torch, MoeKernels(device=0, max_tokens=1)


def _quant_gpu(torch, K, x, rpb):
    rows, cols = x.shape
    xd = torch.from_numpy(x).cuda()
    codes = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(((rows + rpb - 1) // rpb, cols // 128), dtype=torch.float32, device="cuda")
    K.fp8_quantize(xd, codes, scales, rows, cols, rpb)
    return codes, scales


def test_fp8_quantize_bit_exact(env, oracle):
    torch, K = env
    rng = np.random.default_rng(0)
    x = rng.standard_normal((200, 512)).astype(np.float32)
    x[3] *= 1e-6      # below the 1e-4 floor
    x[4] *= 1e4
    x[5, :128] = 0.0
    for rpb in (1, 128):
        codes, scales = _quant_gpu(torch, K, x, rpb)
        rc, rs = oracle.fp8_quantize(x, rpb)
        assert np.array_equal(scales.cpu().numpy(), rs)
        assert np.array_equal(codes.cpu().numpy(), rc)
    # every code decodes to the value the oracle's table gives; ties go to the even code
    ties = np.array([[(oracle.e4m3_decode(c) + oracle.e4m3_decode(c + 1)) / 2 for c in range(8, 120)] + [0.0] * 16],
                    np.float32)
    ties[0, -1] = 448.0  # pins the scale to exactly 1
    codes, scales = _quant_gpu(torch, K, ties, 1)
    assert scales.cpu().numpy()[0, 0] == 1.0
    assert np.array_equal(codes.cpu().numpy(), oracle.fp8_quantize(ties, 1)[0])


def _check(got, ref):
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    err = np.abs(got.astype(np.float64) - ref)
    bad = err > 2e-2 * np.abs(ref) + 1e-3 * rms
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside rel 2e-2, max err {err.max()}, rms {rms}"


@pytest.mark.parametrize("N,K", [(4096, 4096), (1536, 4096), (256, 384)])
@pytest.mark.parametrize("M", [1, 5, 128, 200, 4096])
def test_fp8_linear(env, oracle, M, N, K):
    torch, Kh = env
    if M == 4096 and N == 256:
        pytest.skip("covered by the larger shapes")
    rng = np.random.default_rng(M + N)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    ac, asc = _quant_gpu(torch, Kh, a, 1)
    wc, wsc = _quant_gpu(torch, Kh, w, 128)
    out = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    Kh.fp8_linear(ac, asc, wc, wsc, out, M, N, K)
    assert Kh.device_status() == 0
    got = out.float().cpu().numpy()
    rows = np.arange(M) if M <= 200 else np.sort(rng.choice(M, 48, replace=False))  # sampled rows at full size
    ref = oracle.fp8_gemm(ac.cpu().numpy()[rows], asc.cpu().numpy()[rows], wc.cpu().numpy(), wsc.cpu().numpy())
    _check(got[rows], ref)
    # the quantised product also tracks the unquantised one (sanity of the whole chain, loose)
    exact = a[rows].astype(np.float64) @ w.T.astype(np.float64)
    assert np.corrcoef(exact.ravel(), got[rows].ravel())[0, 1] > 0.995


def test_fp8_linear_ragged_rows_on_the_persistent_kernel(env, oracle):
    """M = 1000 is not a multiple of the 128-row tile and 80 tiles select the persistent warp-specialised kernel: the
    last tile's missing rows are zero-filled on load and never stored; every row is checked."""
    torch, Kh = env
    M, N, K = 1000, 2560, 512
    rng = np.random.default_rng(77)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    ac, asc = _quant_gpu(torch, Kh, a, 1)
    wc, wsc = _quant_gpu(torch, Kh, w, 128)
    out = torch.full((M + 8, N), 7.0, dtype=torch.bfloat16, device="cuda")  # guard rows after the result
    Kh.fp8_linear(ac, asc, wc, wsc, out, M, N, K)
    assert Kh.device_status() == 0
    got = out.float().cpu().numpy()
    assert np.all(got[M:] == 7.0), "rows past M were written"
    ref = oracle.fp8_gemm(ac.cpu().numpy(), asc.cpu().numpy(), wc.cpu().numpy(), wsc.cpu().numpy())
    _check(got[:M], ref)
