"""Packed block formats of the routed-expert path and seeded synthetic tensors in those formats.

Formats (all little-endian; sizes from engine/src/model.rs:57-67 and engine/src/kernels/moe.rs:601-611 of the
reference):

* IQ2_XXS superblock, 66 B / 256 weights: ``u16 d`` (f16) then 8 groups of 8 B. Group ``ib32`` holds ``aux0`` (four
  8-bit codebook indices) and ``aux1`` (four 7-bit sign indices at shifts 0/7/14/21, 4-bit scale in the top nibble).
* Q2_K superblock, 84 B / 256 weights: ``u8 scales[16]`` (low nibble scale, high nibble min), ``u8 qs[64]``,
  ``u16 d``, ``u16 dmin`` (f16).
* Q8_K activation block, 292 B / 256 values: ``f32 d``, ``i8 qs[256]``, ``i16 bsums[16]``.

The generators draw the distributions the benchmark configurations name: f16 scales ``|N(0,1)| * 1e-3``, uniform
codebook / sign / scale / quant fields. They are plain numpy so that the CPU oracle and the GPU harness consume the
same bytes.
"""
from __future__ import annotations

import numpy as np

QK_K = 256
IQ2XXS_BYTES = 66
Q2K_BYTES = 84
Q8K_BYTES = 292
Q8_0_BYTES = 34

# reference model constants (engine/src/model.rs:4, 15-18)
N_EMBD = 4096
N_FF_EXP = 2048
N_EXPERT = 256
N_EXPERT_USED = 6
SWIGLU_CLAMP = 10.0  # engine/src/session.rs:21

F16_ONE = 0x3C00


# ---------------------------------------------------------------------------------------------------------------
# single-block builders: same inputs as the reference's test helpers, so its known answers can be replayed
# ---------------------------------------------------------------------------------------------------------------

def make_iq2_blk(d_bits: int, grid_idx: int, sign_idx: int, ls_val: int) -> np.ndarray:
    """One IQ2_XXS block whose 32 sub-groups all use ``grid_idx`` / ``sign_idx`` and group scale ``ls_val`` (odd,
    1..31). Same construction as make_iq2_blk in engine/tests/quant_cpu.rs:251-284."""
    aux1 = ((((ls_val - 1) // 2) & 0xF) << 28) | sign_idx | (sign_idx << 7) | (sign_idx << 14) | (sign_idx << 21)
    aux0 = grid_idx * 0x01010101
    blk = np.zeros(IQ2XXS_BYTES, np.uint8)
    blk[0:2] = np.frombuffer(np.uint16(d_bits).tobytes(), np.uint8)
    grp = np.frombuffer(np.array([aux0, aux1], np.uint32).tobytes(), np.uint8)
    for ib32 in range(8):
        blk[2 + 8 * ib32:10 + 8 * ib32] = grp
    return blk


def make_q8k_blk(d: float, qs) -> np.ndarray:
    """One Q8_K block from a scale and 256 int8 values (engine/tests/quant_cpu.rs:287-301)."""
    qs = np.asarray(qs, np.int8).reshape(QK_K)
    blk = np.zeros(Q8K_BYTES, np.uint8)
    blk[0:4] = np.frombuffer(np.float32(d).tobytes(), np.uint8)
    blk[4:260] = qs.view(np.uint8)
    bsums = qs.astype(np.int32).reshape(16, 16).sum(axis=1).astype(np.int16)
    blk[260:292] = np.frombuffer(bsums.tobytes(), np.uint8)
    return blk


def make_q2k_blk(d: float, dmin: float, scale_lo: int, scale_hi: int, qs_byte: int) -> np.ndarray:
    """One Q2_K block with uniform fields (engine/tests/quant_cpu.rs:369-388)."""
    blk = np.zeros(Q2K_BYTES, np.uint8)
    blk[0:16] = ((scale_hi & 0xF) << 4) | (scale_lo & 0xF)
    blk[16:80] = qs_byte
    blk[80:82] = np.frombuffer(np.float16(d).tobytes(), np.uint8)
    blk[82:84] = np.frombuffer(np.float16(dmin).tobytes(), np.uint8)
    return blk


# ---------------------------------------------------------------------------------------------------------------
# seeded synthetic tensors
# ---------------------------------------------------------------------------------------------------------------

def _f16_scale_bits(rng: np.random.Generator, n: int) -> np.ndarray:
    return (np.abs(rng.standard_normal(n)) * 1e-3).astype(np.float16).view(np.uint16)


def random_iq2xxs(rng: np.random.Generator, n_blocks: int) -> np.ndarray:
    """uint8 [n_blocks, 66]: f16 d ~ |N(0,1)|*1e-3, codebook indices U{0..255}, sign indices U{0..127}, scales
    U{0..15}."""
    out = np.empty((n_blocks, IQ2XXS_BYTES), np.uint8)
    out[:, 0:2] = _f16_scale_bits(rng, n_blocks).reshape(-1, 1).view(np.uint8)
    aux0 = rng.integers(0, 1 << 32, size=(n_blocks, 8), dtype=np.uint64).astype(np.uint32)
    s = rng.integers(0, 128, size=(n_blocks, 8, 4), dtype=np.uint32)
    sc = rng.integers(0, 16, size=(n_blocks, 8), dtype=np.uint32)
    aux1 = s[..., 0] | (s[..., 1] << 7) | (s[..., 2] << 14) | (s[..., 3] << 21) | (sc << 28)
    grp = np.stack([aux0, aux1], axis=-1).astype("<u4")  # [n, 8, 2]
    out[:, 2:] = grp.view(np.uint8).reshape(n_blocks, 64)
    return out


def random_q2k(rng: np.random.Generator, n_blocks: int) -> np.ndarray:
    """uint8 [n_blocks, 84]: scale bytes and quant bytes uniform, f16 d and dmin ~ |N(0,1)|*1e-3."""
    out = np.empty((n_blocks, Q2K_BYTES), np.uint8)
    out[:, 0:80] = rng.integers(0, 256, size=(n_blocks, 80), dtype=np.uint8)
    out[:, 80:82] = _f16_scale_bits(rng, n_blocks).reshape(-1, 1).view(np.uint8)
    out[:, 82:84] = _f16_scale_bits(rng, n_blocks).reshape(-1, 1).view(np.uint8)
    return out


def random_q8_0(rng: np.random.Generator, n_blocks: int) -> np.ndarray:
    """uint8 [n_blocks, 34]: f16 scale ~ |N(0,1)|*1e-3, int8 quants U{-127..127} (shared-expert weights)."""
    out = np.empty((n_blocks, Q8_0_BYTES), np.uint8)
    out[:, 0:2] = _f16_scale_bits(rng, n_blocks).reshape(-1, 1).view(np.uint8)
    out[:, 2:] = rng.integers(-127, 128, size=(n_blocks, 32), dtype=np.int8).view(np.uint8)
    return out


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round f32 to the nearest bf16 (ties to even) and widen back: the hidden states enter the path as bf16 values
    held in f32."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def zipf_logits(rng: np.random.Generator, n_tokens: int, n_expert: int = N_EXPERT, s: float = 1.1) -> np.ndarray:
    """Router logits with a Zipf(s) expert popularity: N(0,1) - s*ln(rank_e), rank a seeded permutation of 1..E."""
    rank = rng.permutation(n_expert) + 1
    return (rng.standard_normal((n_tokens, n_expert)) - s * np.log(rank)[None, :]).astype(np.float32)


class ExpertLayer:
    """One layer's routed-expert tensors in the reference's byte layout: gate/up ``[E][n_ff][n_embd/256]`` IQ2_XXS
    blocks, down ``[E][n_embd][n_ff/256]`` Q2_K blocks (engine/src/session.rs:2076-2080, 2129-2131)."""

    def __init__(self, seed: int, n_expert: int = N_EXPERT, n_embd: int = N_EMBD, n_ff: int = N_FF_EXP):
        rng = np.random.default_rng(seed)
        self.n_expert, self.n_embd, self.n_ff = n_expert, n_embd, n_ff
        self.xq_blocks, self.mid_blocks = n_embd // QK_K, n_ff // QK_K
        self.gate = random_iq2xxs(rng, n_expert * n_ff * self.xq_blocks).reshape(-1)
        self.up = random_iq2xxs(rng, n_expert * n_ff * self.xq_blocks).reshape(-1)
        self.down = random_q2k(rng, n_expert * n_embd * self.mid_blocks).reshape(-1)

    @property
    def gate_row_bytes(self) -> int:
        return self.xq_blocks * IQ2XXS_BYTES

    @property
    def gate_expert_bytes(self) -> int:
        return self.n_ff * self.gate_row_bytes

    @property
    def down_row_bytes(self) -> int:
        return self.mid_blocks * Q2K_BYTES

    @property
    def down_expert_bytes(self) -> int:
        return self.n_embd * self.down_row_bytes

    @property
    def packed_bytes_per_expert(self) -> int:
        return 2 * self.gate_expert_bytes + self.down_expert_bytes


def random_layer_device(torch, device, seed: int, n_expert: int = N_EXPERT, n_embd: int = N_EMBD, n_ff: int = N_FF_EXP):
    """One layer's expert tensors (gate, up, down; NATIVE byte order, flat uint8) generated on a CUDA device with the
    distributions of ``ExpertLayer``: uniform bytes give uniform codebook / sign / scale / quant fields, the f16 scales
    are |N(0,1)| * 1e-3. A full 256-expert layer is 1.8 GB, which numpy takes minutes to draw; the device takes
    milliseconds. The bytes differ from ``ExpertLayer(seed)``: a consumer that needs them on the host copies them back."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def scales(n):
        return (torch.randn(n, device=device, generator=g).abs() * 1e-3).to(torch.float16).view(torch.uint8).view(n, 2)

    def iq2(n):
        t = torch.randint(0, 256, (n, IQ2XXS_BYTES), dtype=torch.uint8, device=device, generator=g)
        t[:, 0:2] = scales(n)
        return t.view(-1)

    def q2k(n):
        t = torch.randint(0, 256, (n, Q2K_BYTES), dtype=torch.uint8, device=device, generator=g)
        t[:, 80:82] = scales(n)
        t[:, 82:84] = scales(n)
        return t.view(-1)

    nb_gate, nb_down = n_expert * n_ff * (n_embd // QK_K), n_expert * n_embd * (n_ff // QK_K)
    return iq2(nb_gate), iq2(nb_gate), q2k(nb_down)
