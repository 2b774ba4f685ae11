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
