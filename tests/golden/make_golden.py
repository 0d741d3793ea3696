"""Generates the golden fixtures in this folder from seeded inputs and the CPU oracle.

Run from the repository root: ``python tests/golden/make_golden.py``. The inputs are NOT stored: they are regenerated
from the seeds below through ``deepseek_rs_b200.formats`` (numpy's PCG64 streams are stable across versions), and a
SHA-256 of every input array is stored beside the outputs so that a drifting generator is noticed instead of being
mistaken for a kernel bug. Outputs are stored as exact f32 / int bit patterns.

Cases (the configurations the benchmark specification names, at sizes that stay small in the repository):
  iq2xxs_matvec   W 2048 x 4096 IQ2_XXS, x ~ N(0,1), 1 token, seed 0            (configuration 1)
  q2k_matvec      W 2048 x 4096 Q2_K, batches of 1, 4 and 16 tokens, seed 1      (configuration 2)
  moe_layer       32 experts, top-6, 8 tokens: routing, mid, layer output, seed 2 (configuration 3, fewer experts)
  fp8             E4M3 block quantisation of a 8 x 512 activation and 256 x 512 weight, and their product, seed 4
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
HERE = os.path.dirname(os.path.abspath(__file__))


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def inputs():
    """Every case's inputs from its seed (shared with tests/test_golden.py)."""
    from deepseek_rs_b200 import formats as F

    c = {}
    rng = np.random.default_rng(0)
    c["iq2xxs_matvec"] = dict(w=F.random_iq2xxs(rng, 2048 * 16), x=rng.standard_normal((1, 4096)).astype(np.float32))
    rng = np.random.default_rng(1)
    c["q2k_matvec"] = dict(w=F.random_q2k(rng, 2048 * 16), x=rng.standard_normal((16, 4096)).astype(np.float32))
    lw = F.ExpertLayer(seed=2, n_expert=32)
    rng = np.random.default_rng(3)
    c["moe_layer"] = dict(gate=lw.gate, up=lw.up, down=lw.down,
                          x=F.bf16_round(rng.standard_normal((8, 4096)).astype(np.float32)),
                          logits=rng.standard_normal((8, 32)).astype(np.float32))
    rng = np.random.default_rng(4)
    c["fp8"] = dict(a=rng.standard_normal((8, 512)).astype(np.float32), w=rng.standard_normal((256, 512)).astype(np.float32))
    return c


def outputs(c, oracle):
    o = {}
    xq = oracle.q8k_quantize(c["iq2xxs_matvec"]["x"])
    o["iq2xxs_matvec"] = dict(xq=xq, y=oracle.matvec_iq2xxs(c["iq2xxs_matvec"]["w"], xq, 2048, 16))
    xq = oracle.q8k_quantize(c["q2k_matvec"]["x"])
    y = oracle.matvec_q2k(c["q2k_matvec"]["w"], xq, 2048, 16)
    o["q2k_matvec"] = dict(y16=y)  # batches of 1 and 4 are its first rows
    m = c["moe_layer"]
    out, sel, w, mid = oracle.moe_layer(m["x"], m["logits"], m["gate"], m["up"], m["down"], k=6, return_mid=True)
    o["moe_layer"] = dict(out=out, selected=sel, weights=w, mid_sha=np.frombuffer(bytes.fromhex(sha(mid)), np.uint8))
    ac, asc = oracle.fp8_quantize(c["fp8"]["a"], 1)
    wc, wsc = oracle.fp8_quantize(c["fp8"]["w"], 128)
    o["fp8"] = dict(a_codes=ac, a_scales=asc, w_codes_sha=np.frombuffer(bytes.fromhex(sha(wc)), np.uint8), w_scales=wsc,
                    y=oracle.fp8_gemm(ac, asc, wc, wsc))
    return o


def main():
    import oracle

    oracle.build()
    c = inputs()
    o = outputs(c, oracle)
    for name in c:
        arrays = dict(o[name])
        for k, v in c[name].items():
            arrays["sha256_in_" + k] = np.frombuffer(bytes.fromhex(sha(v)), np.uint8)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
        print(name, {k: v.shape for k, v in arrays.items()})


if __name__ == "__main__":
    main()
