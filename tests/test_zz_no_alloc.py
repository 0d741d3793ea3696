"""dsmoe_moe_forward_noalloc — the entry point for hosts that cannot call cudaMalloc (their allocator owns the whole
device, or they sit on a thread that must not take the driver's allocation lock) — must give the same output as the
handle-based dsmoe_moe_forward, whose scratch is cudaMalloc'd. Two calls in a row share the library's static scratch
array, so the second call also shows that leftovers of the first do not leak into it.

Collected last on purpose: a run that stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest

from deepseek_rs_b200 import formats as F

pytestmark = pytest.mark.gpu

REL, ABS = 1e-3, 1e-4  # the tolerance of the other expert-output tests; the results are in fact identical


def test_noalloc_matches_handle_path_twice_in_a_row():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from deepseek_rs_b200 import _lib
    from deepseek_rs_b200.kernels import LAYOUT_ROWSOA, MoeKernels, MoeLayer

    lib = _lib.load()
    torch.cuda.set_device(0)
    n_e = 256  # the entry point is fixed to the reference's 256 experts; only the routed ones need real weights
    rng = np.random.default_rng(21)
    used = 12
    lw = F.ExpertLayer(seed=22, n_expert=used)
    K = MoeKernels(device=0, n_expert=n_e, max_tokens=8)
    # 256-expert tensors whose first `used` experts are real; logits keep the routing inside them
    def full(t, per):
        buf = np.zeros(n_e * per, np.uint8)
        buf[: t.size] = t
        return buf
    gate = full(lw.gate, lw.gate_expert_bytes)
    up = full(lw.up, lw.gate_expert_bytes)
    down = full(lw.down, lw.down_expert_bytes)
    layer = MoeLayer(K, gate, up, down, layout=LAYOUT_ROWSOA)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())

    for T, seed in ((8, 1), (3, 2)):  # the second, smaller call runs over the first call's leftovers
        r = np.random.default_rng(seed)
        x = F.bf16_round(r.standard_normal((T, 4096)).astype(np.float32))
        logits = np.full((T, n_e), -30.0, np.float32)
        logits[:, :used] = r.standard_normal((T, used))
        xd, ld = torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda()
        ref = layer.forward(xd, ld)
        out = torch.full((T, 4096), float("nan"), device="cuda")
        sel = torch.zeros((T, 6), dtype=torch.int32, device="cuda")
        rc = lib.dsmoe_moe_forward_noalloc(stream, p(layer.gate), p(layer.up), p(layer.down), LAYOUT_ROWSOA, p(xd),
                                           p(ld), T, p(out), p(sel), None)
        assert rc == 0
        torch.cuda.synchronize()
        got, want = out.cpu().numpy(), ref.cpu().numpy()
        assert int(sel.max()) < used
        err = np.abs(got - want)
        assert np.all(err <= ABS + REL * np.abs(want)), f"max abs err {err.max()}"
        assert np.array_equal(got, want)

    # NATIVE byte order, the weights output, and a call that asks for neither routing output
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE

    native = MoeLayer(K, gate, up, down, layout=LAYOUT_NATIVE)
    r = np.random.default_rng(3)
    T = 5
    x = F.bf16_round(r.standard_normal((T, 4096)).astype(np.float32))
    logits = np.full((T, n_e), -30.0, np.float32)
    logits[:, :used] = r.standard_normal((T, used))
    xd, ld = torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda()
    w_ref = torch.zeros((T, 6), device="cuda")
    ref = native.forward(xd, ld, weights_out=w_ref)
    for want_outputs in (True, False):
        out = torch.full((T, 4096), float("nan"), device="cuda")
        wts = torch.zeros((T, 6), device="cuda")
        rc = lib.dsmoe_moe_forward_noalloc(stream, p(native.gate), p(native.up), p(native.down), LAYOUT_NATIVE, p(xd),
                                           p(ld), T, p(out), None, p(wts) if want_outputs else None)
        assert rc == 0
        code = C.c_int(-1)
        assert lib.dsmoe_noalloc_device_status(stream, C.byref(code)) == 0 and code.value == 0  # no wait expired
        assert torch.equal(out, ref)
        if want_outputs:
            assert torch.equal(wts, w_ref)

    # sizes beyond the static scratch are refused, not truncated
    big = torch.zeros((9, 4096), device="cuda")
    rc = lib.dsmoe_moe_forward_noalloc(stream, p(layer.gate), p(layer.up), p(layer.down), LAYOUT_ROWSOA, p(big),
                                       p(torch.zeros((9, n_e), device="cuda")), 9, p(big.clone()), None, None)
    assert rc == _lib.ERR_BOUNDS
    K.close()
