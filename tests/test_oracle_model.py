"""CPU checks of the oracle's model glue (rms_norm, RoPE, attention, Llama forward) against plain numpy
statements of src/llama3.rs:5244-5256, 5323-5333, 5431-5690, and threaded == single-thread forward."""
import ctypes as C

import numpy as np

from alice_llm_b200 import synth

CFG = dict(num_layers=2, hidden_dim=256, intermediate_dim=512, num_heads=4, num_kv_heads=2, head_dim=128,
           vocab_size=300, max_seq_len=32, rope_theta=500000.0, eps=1e-5)


def test_rms_norm_matches_numpy(oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal(512).astype(np.float32)
    w = (1 + 0.02 * rng.standard_normal(512)).astype(np.float32)
    got = oracle.rms_norm(x, w, 1e-5)
    mean = np.float32((x.astype(np.float64) ** 2).sum() / 512)
    scale = np.float32(1.0) / np.sqrt(np.float32(mean + np.float32(1e-5)))
    want = (x * scale) * w
    assert np.allclose(got, want, rtol=1e-6, atol=0)


def test_rope_and_attention_match_numpy(oracle):
    rng = np.random.default_rng(2)
    lib = oracle.lib()
    v = rng.standard_normal(128).astype(np.float32)
    for neox in (0, 1):
        got = v.copy()
        lib.orc_apply_rope(got.ctypes.data_as(C.POINTER(C.c_float)), C.c_size_t(77), C.c_size_t(128), C.c_float(500000.0), neox)
        want = v.astype(np.float64).copy()
        for j in range(64):
            ang = 77.0 / (500000.0 ** (2 * j / 128))
            i0, i1 = (j, j + 64) if neox else (2 * j, 2 * j + 1)
            want[i0] = v[i0] * np.cos(ang) - v[i1] * np.sin(ang)
            want[i1] = v[i0] * np.sin(ang) + v[i1] * np.cos(ang)
        assert np.allclose(got, want, rtol=1e-4, atol=1e-5)
    H, KV, D, T = 4, 2, 128, 9
    q = rng.standard_normal(H * D).astype(np.float32)
    kc = rng.standard_normal((T, KV * D)).astype(np.float32)
    vc = rng.standard_normal((T, KV * D)).astype(np.float32)
    out = np.empty(H * D, np.float32)
    fp = C.POINTER(C.c_float)
    lib.orc_gqa_attention(q.ctypes.data_as(fp), kc.ctypes.data_as(fp), vc.ctypes.data_as(fp), C.c_size_t(T - 1),
                          C.c_size_t(H), C.c_size_t(KV), C.c_size_t(D), out.ctypes.data_as(fp))
    for h in range(H):
        k = kc[:, (h // 2) * D:(h // 2 + 1) * D].astype(np.float64)
        s = k @ q[h * D:(h + 1) * D].astype(np.float64) / np.sqrt(D)
        p = np.exp(s - s.max())
        p /= p.sum()
        want = p @ vc[:, (h // 2) * D:(h // 2 + 1) * D].astype(np.float64)
        assert np.allclose(out[h * D:(h + 1) * D], want, rtol=1e-4, atol=1e-5)


def test_forward_is_deterministic_and_threaded_equals_serial(oracle):
    rng = np.random.default_rng(3)
    model = synth.make_llama(rng, CFG)
    a, b = oracle.LlamaOracle(model), oracle.LlamaOracle(model, threads=4)
    for tok in (1, 5, 299):
        la, lb = a.forward(tok), b.forward(tok)
        assert np.isfinite(la).all()
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    assert np.array_equal(a.kcache, b.kcache) and a.pos == 3
    # the first layer's appended K row is the RoPE'd K projection of the normalised embedding
    assert a.kcache[0, :3].any() and not a.kcache[0, 3:].any()


def test_ternary_forward_is_the_same_skeleton_with_f32_ternary_matvec(oracle):
    """forward_ternary (src/llama3.rs:16960-17062): every projection and the head through ternary_matvec on f32
    activations. A one-layer model is recomputed here from the oracle's own pinned pieces (ternary_matvec,
    rms_norm, RoPE, attention) and must equal the fused forward bit for bit."""
    cfg = dict(CFG, num_layers=1)
    rng = np.random.default_rng(4)
    roles = ("q", "k", "v", "o", "gate", "up", "down", "output")
    model = synth.make_llama(rng, cfg, {n: synth.TERNARY for n in roles})
    H, F, D = cfg["hidden_dim"], cfg["intermediate_dim"], cfg["head_dim"]
    nh, nkv = cfg["num_heads"], cfg["num_kv_heads"]
    o = oracle.LlamaOracle(model)
    got = o.forward(7)
    lib, fp = oracle.lib(), C.POINTER(C.c_float)
    L = model["layers"][0]

    def tmv(entry, rows, cols, x):
        pos, neg, sc = entry[1]
        return oracle.ternary_matvec(pos, neg, sc, rows, cols, x)

    hidden = oracle.dequantize(synth.Q8_0, model["embedding"][1][7 * (H // 32) * 34:8 * (H // 32) * 34])
    norm = oracle.rms_norm(hidden, L["attn_norm"], cfg["eps"])
    q, k, v = tmv(L["q"], nh * D, H, norm), tmv(L["k"], nkv * D, H, norm), tmv(L["v"], nkv * D, H, norm)
    for vec, n in ((q, nh), (k, nkv)):
        for h in range(n):
            head = np.ascontiguousarray(vec[h * D:(h + 1) * D])
            lib.orc_apply_rope(head.ctypes.data_as(fp), C.c_size_t(0), C.c_size_t(D), C.c_float(cfg["rope_theta"]), 0)
            vec[h * D:(h + 1) * D] = head
    assert np.array_equal(o.kcache[0, 0], k) and np.array_equal(o.vcache[0, 0], v)
    attn = np.empty(nh * D, np.float32)
    kc, vc = np.ascontiguousarray(k[None, :]), np.ascontiguousarray(v[None, :])
    lib.orc_gqa_attention(q.ctypes.data_as(fp), kc.ctypes.data_as(fp), vc.ctypes.data_as(fp), C.c_size_t(0), C.c_size_t(nh),
                          C.c_size_t(nkv), C.c_size_t(D), attn.ctypes.data_as(fp))
    hidden = hidden + tmv(L["o"], H, nh * D, attn)
    norm = oracle.rms_norm(hidden, L["ffn_norm"], cfg["eps"])
    g, u = tmv(L["gate"], F, H, norm), tmv(L["up"], F, H, norm)
    act = np.array([lib.orc_silu(C.c_float(float(x))) for x in g], np.float32) * u
    hidden = hidden + tmv(L["down"], H, F, act)
    want = tmv(model["output"], cfg["vocab_size"], H, oracle.rms_norm(hidden, model["output_norm"], cfg["eps"]))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
