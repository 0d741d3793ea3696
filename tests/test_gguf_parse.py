"""GGUF reader: the reference's parser tests replayed (engine/tests/gguf_parse.rs:82-219: type ids, dims, offsets,
data slices, lookup by name) over the C ABI, plus the failure cases a loader meets (truncated file, bad magic, unknown
type id, tensor running past the end), which must come back as statuses. No GPU is needed for parsing."""
import numpy as np
import pytest

from deepseek_rs_b200 import _lib
from deepseek_rs_b200.gguf import GgufBuilder, GgufError, GgufFile


def test_single_f16_tensor():
    b = GgufBuilder()
    b.add_tensor("blk.0.ffn_gate_inp.weight", _lib.GGUF_F16, [4096, 256], bytes(4096 * 256 * 2))
    g = GgufFile(data=b.build())
    (t,) = g.tensors
    assert (t.name, t.type, t.dims, t.offset, t.bytes) == ("blk.0.ffn_gate_inp.weight", 1, [4096, 256], 0, 4096 * 256 * 2)


def test_block_type_byte_sizes():
    b = GgufBuilder()
    b.add_tensor("blk.0.attn_kv.weight", _lib.GGUF_Q8_0, [4096, 512], None, 0)
    b.add_tensor("blk.0.ffn_gate_exps.weight", _lib.GGUF_IQ2_XXS, [4096, 2048], None, 0)
    b.add_tensor("blk.0.ffn_down_exps.weight", _lib.GGUF_Q2_K, [2048, 4096], None, 0)
    g = GgufFile(data=b.build(extra_data_bytes=4096 * 2048 // 256 * 84))
    q8, iq2, q2k = g.tensors
    assert q8.type == 8 and q8.bytes == 4096 * 512 // 32 * 34
    assert iq2.type == 16 and iq2.bytes == 4096 * 2048 // 256 * 66
    assert q2k.type == 10 and q2k.bytes == 4096 * 2048 // 256 * 84


def test_type_id_1_is_f16_not_q8_0():
    b = GgufBuilder()
    b.add_tensor("router", 1, [4096, 256], bytes(4096 * 256 * 2))
    t = GgufFile(data=b.build()).tensors[0]
    assert t.type == _lib.GGUF_F16 and t.type != _lib.GGUF_Q8_0


def test_multiple_tensors_offsets_and_data_slices():
    b = GgufBuilder()
    b.add_kv_u32("general.alignment", 32)
    b.add_kv_string_array("tokenizer.ggml.tokens", ["a", "bc", ""])  # metadata of any type is skipped
    first = np.arange(64, dtype=np.uint8)
    second = (np.arange(128) % 251).astype(np.uint8)
    b.add_tensor("tensor0", _lib.GGUF_F16, [4, 8], first)
    b.add_tensor("tensor1", _lib.GGUF_F16, [8, 8], second)
    image = b.build()
    g = GgufFile(data=image)
    t0, t1 = g.tensors
    assert (t0.offset, t1.offset, t0.bytes, t1.bytes) == (0, 64, 64, 128)
    assert g.data_offset % 32 == 0
    assert np.array_equal(g.tensor_data(t0), first) and np.array_equal(g.tensor_data(t1), second)
    assert image[g.data_offset + 64:g.data_offset + 64 + 128] == second.tobytes()


def test_f16_pattern_comes_back():
    b = GgufBuilder()
    b.add_tensor("w", _lib.GGUF_F16, [1, 4], bytes([0x00, 0x3C] * 4))
    g = GgufFile(data=b.build())
    assert g.tensor_data(g.tensors[0]).tolist() == [0x00, 0x3C] * 4


def test_find_by_name():
    b = GgufBuilder()
    b.add_tensor("alpha", _lib.GGUF_F32, [4], bytes(16))
    b.add_tensor("beta", _lib.GGUF_F32, [4], bytes(16))
    g = GgufFile(data=b.build())
    assert g.find("alpha") is not None and g.find("gamma") is None
    assert g.find("beta").offset == 32  # payloads are placed on 32-byte boundaries by the builder


def test_failures_are_statuses():
    b = GgufBuilder()
    b.add_tensor("w", _lib.GGUF_F16, [8, 8], bytes(128))
    image = b.build()
    with pytest.raises(GgufError) as e:
        GgufFile(data=b"GGUX" + image[4:])
    assert e.value.code == _lib.ERR_ARG
    with pytest.raises(GgufError) as e:
        GgufFile(data=image[:-1])  # the tensor's last byte is missing
    assert e.value.code == _lib.ERR_BOUNDS
    with pytest.raises(GgufError) as e:
        GgufFile(data=image[:30])  # ends inside the tensor table
    assert e.value.code == _lib.ERR_BOUNDS
    bad = GgufBuilder()
    bad.add_tensor("w", 99, [8], bytes(32))
    with pytest.raises(GgufError) as e:
        GgufFile(data=bad.build())
    assert e.value.code == _lib.ERR_ARG
    old = GgufBuilder(version=1)
    old.add_tensor("w", 0, [8], bytes(32))
    with pytest.raises(GgufError):
        GgufFile(data=old.build())
    with pytest.raises(GgufError):
        GgufFile.open("/nonexistent/model.gguf")


def test_open_from_a_file(tmp_path):
    b = GgufBuilder()
    payload = np.arange(256, dtype=np.uint8)
    b.add_tensor("blk.3.ffn_gate_tid2eid.weight", _lib.GGUF_I32, [6, 10], payload[:240])
    path = tmp_path / "tiny.gguf"
    path.write_bytes(b.build())
    g = GgufFile.open(str(path))
    t = g.find("blk.3.ffn_gate_tid2eid.weight")
    assert t.type == _lib.GGUF_I32 and t.bytes == 240
    assert np.array_equal(g.tensor_data(t), payload[:240])
    g.close()


@pytest.mark.gpu
def test_upload_experts_shards_and_layouts(oracle):
    """A small layer written as GGUF, uploaded whole and as two expert-parallel shards, NATIVE and ROWSOA: the bytes on
    the device equal the direct upload's, wrong types / dims are refused before anything is copied, and the uploaded
    layer computes what the oracle computes."""
    import torch

    from deepseek_rs_b200 import formats as F
    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA, MoeKernels, MoeLayer

    assert torch.cuda.is_available()
    n_e = 32
    lw = F.ExpertLayer(seed=5, n_expert=n_e)
    b = GgufBuilder()
    b.add_tensor("blk.7.ffn_gate_exps.weight", _lib.GGUF_IQ2_XXS, [4096, 2048, n_e], lw.gate)
    b.add_tensor("blk.7.ffn_up_exps.weight", _lib.GGUF_IQ2_XXS, [4096, 2048, n_e], lw.up)
    b.add_tensor("blk.7.ffn_down_exps.weight", _lib.GGUF_Q2_K, [2048, 4096, n_e], lw.down)
    b.add_tensor("blk.8.ffn_gate_exps.weight", _lib.GGUF_Q2_K, [4096, 2048, n_e], None, 0)  # mislabelled layer
    g = GgufFile(data=b.build())
    K = MoeKernels(device=0, n_expert=n_e, max_tokens=4)
    direct = MoeLayer(K, lw.gate, lw.up, lw.down, layout=LAYOUT_ROWSOA)
    for layout in (LAYOUT_NATIVE, LAYOUT_ROWSOA):
        gate, up, down = g.upload_experts(K, 7, layout=layout)
        if layout == LAYOUT_ROWSOA:
            assert torch.equal(gate, direct.gate) and torch.equal(up, direct.up) and torch.equal(down, direct.down)
        else:
            assert np.array_equal(gate.cpu().numpy(), lw.gate) and np.array_equal(down.cpu().numpy(), lw.down)
        lo = g.upload_experts(K, 7, 0, 16, layout)
        hi = g.upload_experts(K, 7, 16, 16, layout)
        for whole, a, c in zip((gate, up, down), lo, hi):
            assert torch.equal(whole, torch.cat([a, c]))
    with pytest.raises(GgufError) as e:
        g.upload_experts(K, 8)  # wrong type id for gate, and no up / down at all
    assert e.value.code in (_lib.ERR_ARG, _lib.ERR_STATE)
    with pytest.raises(GgufError):
        g.upload_experts(K, 7, 20, 16)  # shard runs past the last expert
    gate, up, down = g.upload_experts(K, 7, layout=LAYOUT_ROWSOA)
    K.layer_register(0, gate, up, down, LAYOUT_ROWSOA)
    rng = np.random.default_rng(6)
    x = F.bf16_round(rng.standard_normal((3, 4096)).astype(np.float32))
    logits = rng.standard_normal((3, n_e)).astype(np.float32)
    out = torch.empty((3, 4096), device="cuda")
    K.moe_forward(0, torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda(), 3, out)
    ref, _, _ = oracle.moe_layer(x, logits, lw.gate, lw.up, lw.down, k=6)
    assert np.array_equal(out.cpu().numpy(), ref)
    K.close()
