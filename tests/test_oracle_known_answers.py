"""The oracle replays every known answer the reference's own CPU tests hold for the routed-expert path
(engine/tests/quant_cpu.rs) plus the swiglu pins of engine/tests/kernels_smoke.rs. Same inputs, same expected
numbers, same tolerances."""
import math

import numpy as np

from deepseek_rs_b200.formats import F16_ONE, make_iq2_blk, make_q2k_blk, make_q8k_blk

ONES = np.ones(256, np.int8)


# --- IQ2_XXS (quant_cpu.rs:304-364) ------------------------------------------------------------------------------

def test_iq2_xxs_zero_q8k_scale_gives_zero(oracle):
    assert oracle.dot_iq2xxs_q8k(make_iq2_blk(F16_ONE, 0, 0, 1), make_q8k_blk(0.0, ONES)) == 0.0


def test_iq2_xxs_zero_iq2_scale_gives_zero(oracle):
    assert oracle.dot_iq2xxs_q8k(make_iq2_blk(0x0000, 0, 0, 1), make_q8k_blk(1.0, ONES)) == 0.0


def test_iq2_xxs_grid0_sign0_ls1_all_ones_q8k(oracle):
    r = oracle.dot_iq2xxs_q8k(make_iq2_blk(F16_ONE, 0, 0, 1), make_q8k_blk(1.0, ONES))
    assert abs(r - 256.0) < 0.01


def test_iq2_xxs_ls_scales_result(oracle):
    q8k = make_q8k_blk(1.0, ONES)
    r1 = oracle.dot_iq2xxs_q8k(make_iq2_blk(F16_ONE, 0, 0, 1), q8k)
    r3 = oracle.dot_iq2xxs_q8k(make_iq2_blk(F16_ONE, 0, 0, 3), q8k)
    assert abs(r3 - 3.0 * r1) < 0.01


def test_iq2_xxs_scale_linearity(oracle):
    iq2 = make_iq2_blk(F16_ONE, 0, 0, 1)
    r1 = oracle.dot_iq2xxs_q8k(iq2, make_q8k_blk(1.0, ONES))
    r2 = oracle.dot_iq2xxs_q8k(iq2, make_q8k_blk(2.0, ONES))
    assert abs(r2 - 2.0 * r1) < 0.01


# --- Q2_K (quant_cpu.rs:391-429) ---------------------------------------------------------------------------------

def test_q2k_zero_qs_gives_minus_dmin_term(oracle):
    r = oracle.dot_q2k_q8k(make_q2k_blk(1.0, 0.0, 1, 1, 0x00), make_q8k_blk(1.0, ONES))
    assert abs(r) < 0.01


def test_q2k_all_ones_q2_all_ones_q8k(oracle):
    r = oracle.dot_q2k_q8k(make_q2k_blk(1.0, 0.0, 1, 1, 0x55), make_q8k_blk(1.0, ONES))
    assert abs(r - 256.0) < 0.5


def test_q2k_dmin_term_subtracts(oracle):
    q8k = make_q8k_blk(1.0, ONES)
    r0 = oracle.dot_q2k_q8k(make_q2k_blk(1.0, 0.0, 1, 0, 0x55), q8k)
    r1 = oracle.dot_q2k_q8k(make_q2k_blk(1.0, 1.0, 1, 0, 0x55), q8k)
    assert abs(r0 - r1) < 0.01


def test_q2k_dmin_term_value(oracle):
    # beyond the reference: hi nibble 2, dmin 0.5, bsums 16 each -> 0.5 * 16*16*2 = 256 subtracted from 256
    r = oracle.dot_q2k_q8k(make_q2k_blk(1.0, 0.5, 1, 2, 0x55), make_q8k_blk(1.0, ONES))
    assert r == 0.0


# --- router math (quant_cpu.rs:453-501) --------------------------------------------------------------------------

def test_softplus_limits(oracle):
    assert abs(oracle.softplus(100.0) - 100.0) < 0.01
    assert oracle.softplus(-100.0) < 1e-30
    assert abs(oracle.softplus(0.0) - math.log(2.0)) < 1e-5


def test_router_score_at_zero_is_sqrt_ln2(oracle):
    assert abs(oracle.router_score(0.0) - math.sqrt(math.log(2.0))) < 1e-5


def _weights_for_scores(oracle, scores):
    """Run the oracle router on logits whose six best probabilities are the given scores."""
    # invert p = sqrt(softplus(x)) -> x = ln(exp(p^2) - 1); everything else is far below
    logits = np.full((1, 256), -30.0, np.float32)
    for i, s in enumerate(scores):
        logits[0, 10 * i + 3] = math.log(math.expm1(s * s))
    probs, sel, w = oracle.router_select(logits, k=len(scores))
    return probs, sel, w


def test_router_normalize_sums_to_1_5(oracle):
    scores = [1.0, 2.0, 0.5, 1.5, 0.8, 1.2]
    _, sel, w = _weights_for_scores(oracle, scores)
    assert abs(float(w.sum()) - 1.5) < 1e-5
    # selection is by descending score
    assert [int(e) for e in sel[0]] == [13, 33, 53, 3, 43, 23]


def test_router_normalize_preserves_ratios(oracle):
    _, _, w = _weights_for_scores(oracle, [2.0, 1.0])
    assert abs(float(w[0, 0] / w[0, 1]) - 2.0) < 1e-4


def test_router_score_matches_ds4_bos_top_expert(oracle):
    assert abs(oracle.router_score(3.8282) - 1.9621) < 0.002


# --- swiglu (kernels_smoke.rs:398-514) ---------------------------------------------------------------------------

def test_swiglu_pins(oracle):
    g = np.array([10.0, 0.0, 10.0], np.float32)
    u = np.array([2.0, 5.0, 2.0], np.float32)
    out = oracle.swiglu(g, u, 10.0, 1.0)
    assert abs(out[0] - 20.0) < 0.01 and out[1] == 0.0
    out2 = oracle.swiglu(g, u, 10.0, 2.0)
    assert abs(out2[0] - 2.0 * out[0]) < 1e-5
    # clamp: gate above 10 is cut to 10, up beyond +-10 is cut
    out3 = oracle.swiglu(np.array([50.0], np.float32), np.array([-30.0], np.float32), 10.0, 1.0)
    assert abs(out3[0] - (-10.0 * 10.0 / (1.0 + math.exp(-10.0)))) < 1e-3


# --- f16 conversion (utils.rs:16-29) -----------------------------------------------------------------------------

def test_f16_device_conversion_flushes_subnormals(oracle):
    assert oracle.f16_to_f32(0x3C00) == 1.0
    assert oracle.f16_to_f32(0xC000) == -2.0
    assert oracle.f16_to_f32(0x03FF) == 0.0  # largest subnormal -> +0
    assert math.copysign(1.0, oracle.f16_to_f32(0x8001)) == -1.0 and oracle.f16_to_f32(0x8001) == 0.0
    assert oracle.f16_to_f32(0x0400) == 2.0 ** -14
    assert oracle.f16_to_f32(0x7C00) == math.inf
    assert math.isnan(oracle.f16_to_f32(0x7E00))
    assert oracle.f16_to_f32(0x03FF, ieee=True) == 1023 * 2.0 ** -24
    # all normals agree with numpy
    bits = np.arange(0x0400, 0x7C00, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in bits[::37]], np.float32)
    assert np.array_equal(got, ref[::37])
