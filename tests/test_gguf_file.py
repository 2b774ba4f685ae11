"""GGUF container: a synthetic model written as a file parses back to the same metadata and the same raw tensor
bytes (CPU), and a model loaded from the file decodes exactly like the model loaded from memory (GPU)."""
import os
import struct

import numpy as np
import pytest

from alice_llm_b200 import synth
from alice_llm_b200.gguf_file import GgufError, GgufFile, write_gguf

CFG = dict(num_layers=2, hidden_dim=512, intermediate_dim=1024, num_heads=4, num_kv_heads=2, head_dim=128,
           vocab_size=1000, max_seq_len=64, rope_theta=500000.0, eps=1e-5)


def test_write_parse_round_trip(tmp_path):
    rng = np.random.default_rng(21)
    model = synth.make_llama(rng, CFG, {"v": synth.Q6_K, "down": synth.Q5_K})
    path = os.path.join(tmp_path, "tiny.gguf")
    write_gguf(path, model)
    gf = GgufFile.open(path)
    assert gf.metadata["general.architecture"] == "llama" and gf.tensor_data_start % 32 == 0
    cfg = gf.model_config()
    for k, v in CFG.items():
        assert cfg[k] == pytest.approx(v), k
    back = gf.load_model()
    for i, L in enumerate(model["layers"]):
        for role in ("q", "k", "v", "o", "gate", "up", "down"):
            assert back["layers"][i][role][0] == L[role][0]
            assert np.array_equal(back["layers"][i][role][1], L[role][1]), (i, role)
        assert np.array_equal(back["layers"][i]["attn_norm"], L["attn_norm"])
    assert np.array_equal(back["embedding"][1], model["embedding"][1]) and back["embedding"][0] == synth.Q8_0
    assert np.array_equal(back["output"][1], model["output"][1])
    info = gf.tensors["blk.1.ffn_down.weight"]
    assert (info.rows, info.cols, info.qtype) == (512, 1024, synth.Q5_K) and info.dims == [1024, 512]


def test_rejects_malformed(tmp_path):
    with pytest.raises(GgufError):
        GgufFile.parse(b"NOPE" + b"\0" * 32)
    with pytest.raises(GgufError):
        GgufFile.parse(struct.pack("<II", 0x46554747, 9) + b"\0" * 32)       # version outside 2..3
    with pytest.raises(GgufError):
        GgufFile.parse(struct.pack("<IIQQ", 0x46554747, 3, 5, 0))            # tensor infos cut off
    rng = np.random.default_rng(22)
    model = synth.make_llama(rng, dict(CFG, num_layers=1))
    path = os.path.join(tmp_path, "t.gguf")
    write_gguf(path, model)
    gf = GgufFile.open(path)
    del gf.tensors["blk.0.attn_k.weight"]
    with pytest.raises(GgufError):
        gf.load_model()


@pytest.mark.gpu
def test_model_from_file_equals_model_from_memory(tmp_path):
    from alice_llm_b200.gpu import GpuEngine, GpuModel
    rng = np.random.default_rng(23)
    model = synth.make_llama(rng, CFG)
    path = os.path.join(tmp_path, "m.gguf")
    write_gguf(path, model)
    eng = GpuEngine(0)
    a, b = GpuModel.load(eng, model), GpuModel.load_gguf(eng, path)
    for tok in (3, 77, 999):
        la, lb = a.forward_and_read(tok), b.forward_and_read(tok)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    assert np.array_equal(a.decode_greedy(5, 6), b.decode_greedy(5, 6))
    eng.close()


# ---- the reference's own in-memory fixtures, rebuilt byte for byte ------------------------------------------------------
# The reference tests its GGUF parser on files assembled by hand (src/llama3.rs:23178-23208 `tiny_gguf_with`,
# :23238-23270 the 2 x 3 tensor `w`, :780-940 the synthetic kimi-k3 header). The same byte sequences are assembled here
# and must parse to what those tests assert.
def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _kv_u32(key, v):
    return _s(key) + struct.pack("<II", 4, v)


def _kv_f32(key, v):
    return _s(key) + struct.pack("<If", 6, v)


def _kv_bool(key, v):
    return _s(key) + struct.pack("<IB", 7, 1 if v else 0)


def _kv_str(key, v):
    return _s(key) + struct.pack("<I", 8) + _s(v)


def _kv_u32_array(key, vs):
    return _s(key) + struct.pack("<IIQ", 9, 4, len(vs)) + b"".join(struct.pack("<I", v) for v in vs)


def _pad32(buf):
    return buf + b"\0" * (-len(buf) % 32)


def _tiny_gguf_with(tensor_name):
    buf = b"GGUF" + struct.pack("<IQQ", 3, 1, 1) + _kv_u32("general.alignment", 32)
    buf += _s(tensor_name) + struct.pack("<IQIQ", 1, 4, 0, 0)          # 1 dim of 4, F32, offset 0
    return _pad32(buf) + struct.pack("<4f", 1.0, 2.0, 3.0, 4.0)


def test_reference_fixture_single_f32_tensor():
    for name in ("blk.0.ffn_norm.weight", "blk.0.post_attention_norm.weight"):
        gf = GgufFile.parse(_tiny_gguf_with(name))
        assert gf.metadata == {"general.alignment": 32} and list(gf.tensors) == [name]
        assert gf.tensor_f32(name).tolist() == [1.0, 2.0, 3.0, 4.0]
    gf = GgufFile.parse(_tiny_gguf_with("blk.0.something_else.weight"))
    with pytest.raises(GgufError):
        gf.tensor_f32("blk.0.ffn_norm.weight")


def test_reference_fixture_rows_come_from_dims():
    buf = b"GGUF" + struct.pack("<IQQ", 3, 1, 1) + _kv_u32("general.alignment", 32)
    buf += _s("w") + struct.pack("<IQQIQ", 2, 2, 3, 0, 0)              # dims [2, 3]: cols 2, rows 3
    buf = _pad32(buf) + struct.pack("<6f", *range(6))
    gf = GgufFile.parse(buf)
    w = gf.tensors["w"]
    assert (w.rows, w.cols) == (3, 2)
    assert gf.tensor_f32("w").tolist() == [0.0, 1.0, 2.0, 3.0, 4.0, 5.0]
    assert "not_present" not in gf.tensors


def test_reference_fixture_metadata_of_every_value_type():
    kv = [_kv_str("general.architecture", "kimi-k3"), _kv_u32("general.alignment", 32), _kv_u32("kimi-k3.block_count", 8),
          _kv_u32("kimi-k3.embedding_length", 64), _kv_u32("kimi-k3.feed_forward_length", 128),
          _kv_u32("kimi-k3.context_length", 4096), _kv_u32("kimi-k3.vocab_size", 256),
          _kv_u32("kimi-k3.attention.head_count", 8), _kv_f32("kimi-k3.attention.layer_norm_rms_epsilon", 1e-5),
          _kv_bool("kimi-k3.mla_use_nope", True), _kv_f32("kimi-k3.gate_lower_bound", -5.0),
          _kv_str("kimi-k3.activation", "situ"), _kv_u32_array("kimi-k3.full_attn_layers", [3, 7]),
          _kv_u32_array("kimi-k3.kda_layers", [0, 1, 2, 4, 5, 6])]
    buf = b"GGUF" + struct.pack("<IQQ", 3, 1, len(kv)) + b"".join(kv)
    buf += _s("token_embd.weight") + struct.pack("<IQIQ", 1, 1, 0, 0)
    buf = _pad32(buf) + struct.pack("<f", 42.0)
    gf = GgufFile.parse(buf)
    m = gf.metadata
    assert m["general.architecture"] == "kimi-k3" and m["kimi-k3.block_count"] == 8 and m["kimi-k3.mla_use_nope"] is True
    assert m["kimi-k3.attention.layer_norm_rms_epsilon"] == pytest.approx(1e-5) and m["kimi-k3.gate_lower_bound"] == -5.0
    assert m["kimi-k3.activation"] == "situ"
    assert m["kimi-k3.full_attn_layers"] == [3, 7] and m["kimi-k3.kda_layers"] == [0, 1, 2, 4, 5, 6]
    assert gf.tensor_f32("token_embd.weight").tolist() == [42.0]
    # only the Llama branch of the decode graph exists here: another architecture is refused, not mis-decoded
    with pytest.raises(GgufError, match="architecture"):
        gf.model_config()


def test_rejects_hostile_headers():
    head = b"GGUF" + struct.pack("<I", 3)
    with pytest.raises(GgufError, match="claims"):
        GgufFile.parse(head + struct.pack("<QQ", 1 << 60, 0))                       # tensor count no file could hold
    with pytest.raises(GgufError, match="claims"):
        GgufFile.parse(head + struct.pack("<QQ", 0, 1 << 60))
    with pytest.raises(GgufError, match="array"):
        GgufFile.parse(head + struct.pack("<QQ", 0, 1) + _s("a") + struct.pack("<IIQ", 9, 4, 1 << 50))
    with pytest.raises(GgufError, match="nested"):
        GgufFile.parse(head + struct.pack("<QQ", 0, 1) + _s("a") + struct.pack("<IIQ", 9, 9, 1) + b"\0" * 64)
    for bad in (0, 3, 48):
        with pytest.raises(GgufError, match="alignment"):
            GgufFile.parse(head + struct.pack("<QQ", 0, 1) + _kv_u32("general.alignment", bad) + b"\0" * 64)
    with pytest.raises(GgufError, match="alignment"):
        GgufFile.parse(head + struct.pack("<QQ", 0, 1) + _kv_str("general.alignment", "32") + b"\0" * 64)
    with pytest.raises(GgufError, match="dimensions"):
        GgufFile.parse(head + struct.pack("<QQ", 1, 0) + _s("t") + struct.pack("<I", 200) + b"\0" * 64)
