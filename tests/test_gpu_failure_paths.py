"""Failure paths that can be shown without hanging or faulting a GPU.

Every device-side wait in the library is bounded. Here one wait is made to run out on purpose, through the test hook
``dsmoe_debug_set``: the wait limit is shortened to a fraction of a millisecond and the TMA-staged down kernel is
told to leave one of its bulk copies out, so the mbarrier it would complete never flips. The kernel must return, the
status word must report the timeout, and the device must stay usable."""
import numpy as np
import pytest

from deepseek_rs_b200 import formats as F

pytestmark = pytest.mark.gpu


def _down_case(torch, K, oracle, n_e=3, T=2, k=6, seed=5):
    rng = np.random.default_rng(seed)
    mb, out_dim = 8, 4096
    w = F.random_q2k(rng, n_e * out_dim * mb).reshape(-1)
    mid = rng.standard_normal((T * k, mb * 256)).astype(np.float32)
    midq = oracle.q8k_quantize(mid)
    sel = rng.integers(0, n_e, size=(T, k)).astype(np.int32)
    ref = oracle.down_sum(w, midq, sel, out_dim, mb)
    wd = torch.from_numpy(w).cuda()
    mqd = torch.from_numpy(midq.reshape(-1)).cuda()
    sd = torch.from_numpy(sel).cuda()
    out = torch.zeros((T, out_dim), device="cuda")

    def run():
        K.moe_down_sum6_qwarp32(wd, mqd, sd, out, out_dim * mb * 84, mb * 84, mb, out_dim, n_expert=k, n_tokens=T)
        return out

    return run, ref


def test_expired_wait_is_reported_and_the_device_stays_usable(oracle):
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from deepseek_rs_b200 import _lib
    from deepseek_rs_b200.kernels import DsmoeError, MoeKernels

    K = MoeKernels(device=0, n_expert=32, max_tokens=2)
    run, ref = _down_case(torch, K, oracle)
    got = run()
    assert K.device_status() == 0
    assert np.array_equal(got.cpu().numpy(), ref)

    K.debug_set(_lib.DEBUG_WAIT_LIMIT_KCLOCKS, 200)  # about 0.1 ms of SM clocks
    K.debug_set(_lib.DEBUG_DROP_ONE_COPY, 1)
    run()  # returns: the wait for the missing copy gives up
    with pytest.raises(DsmoeError) as ei:
        K.device_status()
    assert ei.value.code == _lib.ERR_TIMEOUT
    torch.cuda.synchronize()  # the context is healthy: no sticky CUDA error

    # the same handle recovers once the hook is cleared ...
    K.debug_set(_lib.DEBUG_DROP_ONE_COPY, 0)
    K.debug_set(_lib.DEBUG_WAIT_LIMIT_KCLOCKS, 0)
    K.debug_set(_lib.DEBUG_CLEAR_STATUS, 0)
    got = run()
    assert K.device_status() == 0
    assert np.array_equal(got.cpu().numpy(), ref)
    # ... and a fresh handle is unaffected
    K2 = MoeKernels(device=0, n_expert=32, max_tokens=2)
    run2, ref2 = _down_case(torch, K2, oracle, seed=6)
    assert np.array_equal(run2().cpu().numpy(), ref2)
    assert K2.device_status() == 0
    K.close()
    K2.close()


def test_calls_on_the_wrong_current_device_are_refused():
    """A handle's pointers belong to its device; with two devices visible a call made while the other one is current
    returns DSMOE_ERR_STATE instead of launching there."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible devices")
    from deepseek_rs_b200 import _lib
    from deepseek_rs_b200.kernels import DsmoeError, MoeKernels

    K0 = MoeKernels(device=0, n_expert=32, max_tokens=1)
    K1 = MoeKernels(device=1, n_expert=32, max_tokens=1)  # second device in one process: per-device kernel attributes
    assert torch.cuda.current_device() == 1
    with pytest.raises(DsmoeError) as ei:
        K0.device_status()
    assert ei.value.code == _lib.ERR_STATE
    K1.close()
    torch.cuda.set_device(0)
    K0.close()


def test_zero_max_tokens_handle_serves_tier1_calls():
    import torch

    from deepseek_rs_b200.kernels import MoeKernels

    K = MoeKernels(device=0, n_expert=32, max_tokens=0)
    x = torch.randn((2, 256), device="cuda")
    out = torch.zeros((2, 292), dtype=torch.uint8, device="cuda")
    K.q8k_quantize(x, out, 256, 2)
    torch.cuda.synchronize()
    K.close()


def test_checked_build_catches_an_out_of_range_expert_index(oracle):
    """The checked build (-DDSMOE_BOUNDS) in a child process: an expert index beyond the layer handed to dsmoe_expert_ffn is
    replaced by 0 before any kernel sees it, the output equals the run with index 0, and the status word reports
    DSMOE_ERR_BOUNDS. Output buffers carry canary rows on both sides, which must come back untouched."""
    import os
    import subprocess
    import sys
    import textwrap

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = textwrap.dedent("""
        import numpy as np, torch
        from deepseek_rs_b200 import _lib, formats as F
        from deepseek_rs_b200.kernels import DsmoeError, LAYOUT_ROWSOA, MoeKernels, MoeLayer
        assert b"checked" in _lib.load().dsmoe_version()
        n_e, T = 32, 4
        K = MoeKernels(device=0, n_expert=n_e, n_expert_used=1, max_tokens=T)
        lw = F.ExpertLayer(seed=3, n_expert=n_e)
        layer = MoeLayer(K, lw.gate, lw.up, lw.down, layout=LAYOUT_ROWSOA)
        rng = np.random.default_rng(4)
        x = torch.from_numpy(rng.standard_normal((T, 4096)).astype(np.float32)).cuda()
        xq = torch.empty((T, 16, 292), dtype=torch.uint8, device="cuda")
        K.q8k_quantize(x, xq, 4096, T)
        w = torch.ones((T, 1), device="cuda")
        def run(sel):
            guard = torch.full((T + 2, 4096), 7.25, device="cuda")  # canary rows before and after the output
            K.expert_ffn(0, xq, torch.tensor(sel, dtype=torch.int32, device="cuda").reshape(T, 1), w, T, guard[1:T + 1])
            torch.cuda.synchronize()
            assert bool((guard[0] == 7.25).all()) and bool((guard[T + 1] == 7.25).all()), "canary overwritten"
            return guard[1:T + 1].clone()
        good = run([3, 0, 9, 31])
        assert K.device_status() == 0
        bad = run([3, n_e + 5, 9, 31])  # would address memory behind the layer's tensors
        try:
            K.device_status()
            raise SystemExit("the out-of-range index was not reported")
        except DsmoeError as e:
            assert e.code == _lib.ERR_BOUNDS, e
        assert torch.equal(bad, good)
        print("checked build ok")
    """)
    env = dict(os.environ, DSMOE_CHECKED_BUILD="1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=root, timeout=600)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout + r.stderr
