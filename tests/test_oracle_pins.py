"""Pins the CPU oracle to every known-answer case the reference's own unit tests hold for this
path (ALICE-LLM src/gguf.rs, #[cfg(test)] module), and to an independent numpy statement of the
block formats. Runs on CPU."""
import numpy as np
import pytest

from alice_llm_b200 import synth
from tests import npref, refblocks

Q8_0, Q4_K, Q5_K, Q6_K, Q1_0, Q2_0 = synth.Q8_0, synth.Q4_K, synth.Q5_K, synth.Q6_K, synth.Q1_0, synth.Q2_0


def bits(v):
    return np.asarray(v, dtype=np.float32).view(np.uint32)


# src/gguf.rs:6627-6650
def test_f16_known_values(oracle):
    assert oracle.f16_to_f32(0x0000) == 0.0
    assert oracle.f16_to_f32(0x3C00) == 1.0
    assert oracle.f16_to_f32(0xBC00) == -1.0
    assert oracle.f16_to_f32(0x4000) == 2.0
    assert oracle.f16_to_f32(0x3800) == 0.5
    assert oracle.f16_to_f32(0x7C00) == np.inf
    assert oracle.f16_to_f32(0xFC00) == -np.inf
    assert np.isnan(oracle.f16_to_f32(0x7C01))


def test_f16_all_patterns_match_ieee(oracle):
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(v)) for v in h], dtype=np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(bits(got)[~nan], bits(want)[~nan])


# src/gguf.rs:7163-7178
def test_block_size_table(oracle):
    assert oracle.block_bytes(Q8_0) == 34 and oracle.elements_per_block(Q8_0) == 32
    assert oracle.block_bytes(Q4_K) == 144 and oracle.elements_per_block(Q4_K) == 256
    assert oracle.block_bytes(Q5_K) == 176 and oracle.block_bytes(Q6_K) == 210
    assert oracle.block_bytes(Q1_0) == 18 and oracle.elements_per_block(Q1_0) == 128
    assert oracle.block_bytes(Q2_0) == 34 and oracle.elements_per_block(Q2_0) == 128


# src/gguf.rs:7181-7224
def test_q1_0_dequantize_known_answer(oracle):
    data = np.zeros(36, dtype=np.uint8)
    data[0:2] = [0x00, 0x3C]
    data[2:18] = 0xAA
    data[18:20] = [0x00, 0x38]
    data[20:36] = 0xFF
    out = oracle.dequantize(Q1_0, data)
    assert np.array_equal(out[0:128:2], np.full(64, -1.0, np.float32))
    assert np.array_equal(out[1:128:2], np.full(64, 1.0, np.float32))
    assert np.array_equal(out[128:], np.full(128, 0.5, np.float32))


# src/gguf.rs:7227-7254
def test_q2_0_dequantize_known_answer(oracle):
    data = np.zeros(34, dtype=np.uint8)
    data[0:2] = [0x00, 0x40]
    data[2:] = 0xE4
    out = oracle.dequantize(Q2_0, data)
    assert np.array_equal(out, np.tile(np.array([-2.0, 0.0, 2.0, 4.0], np.float32), 32))


# src/gguf.rs:7257-7283
def test_q2_0_matvec_known_answer(oracle):
    data = np.zeros(34, dtype=np.uint8)
    data[0:2] = [0x00, 0x3C]
    data[2:] = 0x46
    x = np.arange(1, 129, dtype=np.float32)
    y = oracle.matvec(Q2_0, x, data, 1, 128)
    assert abs(y[0] - -64.0) < 1e-3


def _g128_case(bb, mul, badd, xor):
    rows, cols = 4, 256
    bpr = cols // 128
    data = np.zeros(rows * bpr * bb, dtype=np.uint8)
    for r in range(rows):
        for b in range(bpr):
            base = (r * bpr + b) * bb
            sc = (0x3800 + r * 0x0080) & 0xFFFF
            data[base:base + 2] = [sc & 0xFF, sc >> 8]
            for k in range(bb - 2):
                data[base + 2 + k] = (((r * mul) & 0xFF) + ((b * badd + k) & 0xFF) & 0xFF) ^ xor
    return rows, cols, data


# src/gguf.rs:7294-7340 and 7346-7390
@pytest.mark.parametrize("qtype,bb,mul,badd,xor,fn,w", [(Q1_0, 18, 37, 11, 0xA5, np.sin, 0.037),
                                                       (Q2_0, 34, 53, 7, 0x3C, np.cos, 0.041)])
def test_g128_matvec_matches_dequant_dot(oracle, qtype, bb, mul, badd, xor, fn, w):
    rows, cols, data = _g128_case(bb, mul, badd, xor)
    x = fn(np.arange(cols, dtype=np.float32) * np.float32(w)).astype(np.float32)
    y = oracle.matvec(qtype, x, data, rows, cols)
    wd = oracle.dequantize(qtype, data).reshape(rows, cols)
    for r in range(rows):
        acc = np.float32(0)
        for i in range(cols):
            acc = np.float32(acc + np.float32(wd[r, i] * x[i]))
        assert abs(y[r] - acc) / max(abs(acc), 1e-6) < 1e-4
        assert bits(y[r]) == bits(acc)  # the x86 arm is exactly this loop


# src/gguf.rs:7393-7416
def test_q8_0_dequantize_known_answer(oracle):
    blk = np.zeros(34, dtype=np.uint8)
    blk[0:2] = [0x66, 0x2E]
    blk[2:] = np.arange(32)
    out = oracle.dequantize(Q8_0, blk)
    s = np.float32(oracle.f16_to_f32(0x2E66))
    assert np.allclose(out, s * np.arange(32, dtype=np.float32), atol=1e-4)


# src/gguf.rs:7419-7445
def test_q8_0_fused_matvec_known_answer(oracle):
    data = np.zeros(68, dtype=np.uint8)
    data[0:2] = [0x00, 0x3C]
    data[2] = 1
    data[34:36] = [0x00, 0x3C]
    data[37] = 1
    x = np.zeros(32, dtype=np.float32)
    x[0], x[1] = 3.0, 7.0
    y = oracle.matvec(Q8_0, x, data, 2, 32)
    assert abs(y[0] - 3.0) < 1e-4 and abs(y[1] - 7.0) < 1e-4


# src/gguf.rs:7448-7459 (and the j >= 4 arm, which the reference test leaves out)
def test_get_scale_min_k4(oracle):
    s = np.array([10, 20, 30, 40, 50, 60, 70, 80, 0xAB, 0xCD, 0xEF, 0x12], dtype=np.uint8)
    assert oracle.get_scale_min_k4(0, s) == (10 & 63, 50 & 63)
    assert oracle.get_scale_min_k4(3, s) == (40 & 63, 80 & 63)
    sc, mn = npref.k4_scales(s)
    for j in range(8):
        assert oracle.get_scale_min_k4(j, s) == (sc[j], mn[j])
    rng = np.random.default_rng(3)
    scs = rng.integers(0, 64, size=(50, 8))
    mns = rng.integers(0, 64, size=(50, 8))
    packed = synth.pack_scales_k4(scs, mns)
    for i in range(50):
        for j in range(8):
            assert oracle.get_scale_min_k4(j, packed[i]) == (scs[i, j], mns[i, j])


# Seeded blocks of src/gguf.rs:7810-7970: the reference pins its SIMD kernels bit-exactly to the
# scalar fallbacks on these; here the oracle's restatement of the fallbacks is pinned to an
# independent numpy statement on the same blocks.
@pytest.mark.parametrize("seed", refblocks.SEEDS)
def test_kquant_block_dots_on_reference_seeds(oracle, seed):
    for qtype, mk, mul, ref in [(Q4_K, refblocks.make_q4k_block, 13, npref.q4k_dot),
                                (Q6_K, refblocks.make_q6k_block, 11, npref.q6k_dot),
                                (Q5_K, refblocks.make_q5k_block, 17, npref.q5k_dot)]:
        blk = mk(seed)
        d8, q8, bs = refblocks.make_q8k_block((seed * mul) & 0xFF)
        got = oracle.kquant_block_dot(qtype, blk, d8, q8, bs)
        want = ref(blk, d8, q8, bs)
        assert bits(got) == bits(want), (qtype, seed, got, want)


def test_kquant_block_dots_random_blocks(oracle):
    rng = np.random.default_rng(11)
    for qtype, ref in [(Q4_K, npref.q4k_dot), (Q5_K, npref.q5k_dot), (Q6_K, npref.q6k_dot)]:
        data = synth.make_weights(qtype, rng, 8, 256).reshape(8, -1)
        x = synth.make_x(rng, 256)
        d8, q8, bs = oracle.quantize_row_q8_k(x)
        for r in range(8):
            got = oracle.kquant_block_dot(qtype, data[r], d8[0], q8[0], bs[0])
            assert bits(got) == bits(ref(data[r], d8[0], q8[0], bs[0]))


def test_dequant_matches_numpy_statement(oracle):
    rng = np.random.default_rng(5)
    blk = synth.make_q4k(rng, 1, 256)
    d, dmin = npref.f16(blk[0], blk[1]), npref.f16(blk[2], blk[3])
    sc, mn = npref.k4_scales(blk[4:16])
    q = npref.q4k_quants(blk)
    want = np.concatenate([(d * np.float32(sc[i])) * q[32 * i:32 * i + 32].astype(np.float32)
                           - dmin * np.float32(mn[i]) for i in range(8)]).astype(np.float32)
    assert np.array_equal(bits(oracle.dequantize(Q4_K, blk)), bits(want))
    blk = synth.make_q5k(rng, 1, 256)
    d, dmin = npref.f16(blk[0], blk[1]), npref.f16(blk[2], blk[3])
    sc, mn = npref.k4_scales(blk[4:16])
    q = npref.q5k_quants(blk)
    want = np.concatenate([(d * np.float32(sc[i])) * q[32 * i:32 * i + 32].astype(np.float32)
                           - dmin * np.float32(mn[i]) for i in range(8)]).astype(np.float32)
    assert np.array_equal(bits(oracle.dequantize(Q5_K, blk)), bits(want))
    blk = synth.make_q6k(rng, 1, 256)
    d = npref.f16(blk[208], blk[209])
    q = npref.q6k_quants(blk)
    s = blk[192:208].view(np.int8).astype(np.float32)
    order = np.concatenate([np.repeat(s[8 * n:8 * n + 8], 16) for n in range(2)])
    want = ((d * order).astype(np.float32) * q.astype(np.float32)).astype(np.float32)
    assert np.array_equal(bits(oracle.dequantize(Q6_K, blk)), bits(want))


def test_row_dequantizers_agree_with_block_dequantizers(oracle):
    """src/gguf.rs spells Q4_K/Q6_K/Q8_0 dequantization twice (:903/:6211, :1205/:6264, :990/:6308)."""
    rng = np.random.default_rng(6)
    for qtype in (Q4_K, Q5_K, Q6_K, Q8_0):
        data = synth.make_weights(qtype, rng, 3, 512)
        a = oracle.dequantize(qtype, data)
        b = oracle.dequantize_weight_row(qtype, data, a.size)
        assert np.array_equal(bits(a), bits(b))
    # types the public dispatcher does not list give zeros (src/gguf.rs:6193)
    assert not oracle.dequantize_weight_row(Q1_0, synth.make_q1_0(rng, 1, 256), 256).any()


def test_q8k_quantizer(oracle):
    rng = np.random.default_rng(2)
    x = synth.make_x(rng, 4096)
    x[256:512] = 0.0                      # all-zero block -> d = 0, qs = 0
    x[512] = -9.0                         # negative element of largest magnitude
    x[768 + 5], x[768 + 9] = 7.5, -7.5    # tie: the first one wins
    d, qs, bs = oracle.quantize_row_q8_k(x)
    d2, qs2, bs2 = npref.q8k_quantize(x)
    assert np.array_equal(bits(d), bits(d2)) and np.array_equal(qs, qs2) and np.array_equal(bs, bs2)
    assert d[1] == 0 and not qs[1].any()
    assert qs[2, 0] == 127 and d[2] < 0   # iscale = 128/max_val keeps the sign; +128 clamps to 127
    assert qs[3, 5] == 127 and qs[3, 9] == -128 and d[3] > 0


# src/gguf.rs:8083-8153: scalar ternary dot on the reference's seeded rows, incl. the 100-col tail.
@pytest.mark.parametrize("cols,seeds,mul,scale", [(128, refblocks.SEEDS, 7, 0.125), (100, [1, 42, 200], 11, 0.5)])
def test_ternary_scalar_on_reference_seeds(oracle, cols, seeds, mul, scale):
    for seed in seeds:
        pos, neg = refblocks.make_ternary_row(seed, cols)
        x = refblocks.make_ternary_input((seed * mul) & 0xFF, cols)
        y = oracle.ternary_matvec(pos, neg, np.array([scale], np.float32), 1, cols, x)
        p = np.unpackbits(pos, bitorder="little")[:cols].astype(bool)
        n = np.unpackbits(neg, bitorder="little")[:cols].astype(bool)
        want = scale * (x[p].astype(np.float64).sum() - x[n].astype(np.float64).sum())
        assert abs(y[0] - want) / max(abs(want), 1e-6) < 1e-4


# src/gguf.rs:7520-7530, 7533-7576, 7597-7626
def test_sparse_ternary_reference_cases(oracle):
    w = np.array([1.0, -2.0, 0.5, -0.1, 3.0, -0.3, 0.8, -0.05, 0.02, -1.5, 0.7, -0.9, 0.01, -0.4, 2.5, -0.6],
                 dtype=np.float32)
    pos, neg, sc = oracle.ternarize_row(w, 0.1)
    active, sign, _ = oracle.sparsify_row(pos, neg, sc, w, 4)
    assert bin(int(active[0])).count("1") == 4
    assert int(active[0]) == (1 << 4) | (1 << 14) | (1 << 1) | (1 << 9)  # the 4 largest magnitudes

    w2 = np.concatenate([w, -w])
    x = np.array([1.0, 0.5, -1.0, 2.0, 0.3, -0.7, 1.5, -0.2, 0.8, -1.2, 0.4, 0.6, -0.9, 1.1, -0.3, 0.7], np.float32)
    dense, sparse = [], []
    for r in range(2):
        p, n, s = oracle.ternarize_row(w2[16 * r:16 * r + 16], 0.05)
        dense.append(oracle.ternary_matvec(p, n, np.array([s]), 1, 16, x)[0])
        a, sg, s2 = oracle.sparsify_row(p, n, s, w2[16 * r:16 * r + 16], 16)
        sparse.append(oracle.sparse_ternary_matvec(a, sg, np.array([s2]), 1, 16, x)[0])
    for d_, s_ in zip(dense, sparse):
        assert abs(d_ - s_) < max(abs(d_), 0.01) * 0.05

    w3 = np.zeros(16, dtype=np.float32)
    w3[3], w3[10] = 5.0, -3.0
    p, n, s = oracle.ternarize_row(w3, 0.01)
    a, sg, s2 = oracle.sparsify_row(p, n, s, w3, 2)
    assert int(a[0]) == (1 << 3) | (1 << 10) and int(sg[0]) == (1 << 10)
    xin = np.zeros(16, dtype=np.float32)
    xin[3], xin[10] = 10.0, 7.0
    y = oracle.sparse_ternary_matvec(a, sg, np.array([s2]), 1, 16, xin)
    assert abs(y[0] - s2 * 3.0) < abs(s2 * 3.0) * 0.05
    # 2-bit packing: 00 = 0, 01 = +1, 11 = -1 (src/gguf.rs:5560-5583)
    pk = oracle.sparse_pack_2bit(a, sg, 1, 16)
    assert list(pk) == [0b01000000, 0, 0b00110000, 0]


def test_sparse_and_dense_ternary_agree_on_synthetic(oracle):
    rng = np.random.default_rng(9)
    rows, cols = 6, 512
    pos, neg, sc = synth.make_ternary(rng, rows, cols)
    x = synth.make_x(rng, cols)
    active, sign = synth.ternary_to_sparse(pos, neg, cols)
    yd = oracle.ternary_matvec(pos, neg, sc, rows, cols, x)
    ys = oracle.sparse_ternary_matvec(active, sign, sc, rows, cols, x)
    assert np.allclose(yd, ys, rtol=1e-4, atol=1e-5)


def test_synthetic_sparse_packing_equals_oracle_packer(oracle):
    """synth.pack_2bit (what GpuModel.load uploads for sparse-ternary tensors) against the oracle's restatement of
    SparseTernaryMatrix's packer (src/gguf.rs:5432-5450), ragged column counts included."""
    import numpy as np
    from alice_llm_b200 import synth
    rng = np.random.default_rng(8)
    for rows, cols in [(5, 70), (3, 16), (9, 1000), (2, 8192)]:
        pos, neg, _ = synth.make_ternary(rng, rows, cols)
        active, sign = synth.ternary_to_sparse(pos, neg, cols)
        assert np.array_equal(synth.pack_2bit(pos, neg, cols).reshape(-1), oracle.sparse_pack_2bit(active, sign, rows, cols))
