"""GPU parity: every CUDA entry point against the CPU oracle on the same seeded inputs.

Gates (the reference's own convention, src/gpu.rs:7133, src/gguf.rs:8038):
  dequantized weights  bit-exact
  Q8_K activations     bit-exact
  matvec / SwiGLU      max_i |y_i - ref_i| / max(|ref_i|, 1) <= 1e-3  and  rel-L2 <= 1e-3
"""
import numpy as np
import pytest

from alice_llm_b200 import synth

pytestmark = pytest.mark.gpu

Q8_0, Q4_K, Q5_K, Q6_K, Q1_0, Q2_0 = synth.Q8_0, synth.Q4_K, synth.Q5_K, synth.Q6_K, synth.Q1_0, synth.Q2_0
TOL = 1e-3


@pytest.fixture(scope="module")
def eng():
    from alice_llm_b200.gpu import GpuEngine
    e = GpuEngine(0)
    yield e
    e.close()


def bits(a):
    return np.asarray(a, np.float32).view(np.uint32)


def assert_close(got, ref, what=""):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    err = np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)
    l2 = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
    assert np.isfinite(got).all(), what
    assert err.max() <= TOL and l2 <= TOL, f"{what}: max err {err.max():.3e} at {err.argmax()}, rel-L2 {l2:.3e}"


def quant(qtype):
    from alice_llm_b200.gpu import GpuQuantType
    return GpuQuantType(qtype)


SHAPES = {
    Q4_K: [(1, 256), (3, 512), (70, 4096), (129, 1024), (33, 14336), (64, 16384)],
    Q5_K: [(1, 256), (5, 768), (70, 4096), (16, 14336)],
    Q6_K: [(1, 256), (3, 512), (7, 768), (70, 4096), (40, 14336)],
    Q8_0: [(2, 32), (3, 96), (70, 4096), (50, 5120), (9, 14336)],
    # (1000, 5120): many 16-row tiles and stages per CTA; (40, 61440): rows too wide for shared memory, run as column chunks
    Q1_0: [(4, 256), (3, 128), (70, 5120), (20, 25600), (1000, 5120), (40, 61440)],
    Q2_0: [(4, 256), (70, 5120), (10, 16384)],
}


@pytest.mark.parametrize("qtype", [Q4_K, Q5_K, Q6_K, Q8_0, Q1_0, Q2_0])
def test_dequantize_bit_exact(eng, oracle, qtype):
    rng = np.random.default_rng(100 + qtype)
    for rows, cols in SHAPES[qtype][:4]:
        data = synth.make_weights(qtype, rng, rows, cols)
        w = eng.upload_weights_typed(data, rows, cols, quant(qtype))
        got = eng.dequantize(w)
        ref = oracle.dequantize(qtype, data)
        assert np.array_equal(bits(got), bits(ref)), (synth.TYPE_NAMES[qtype], rows, cols)


def test_q8k_quantizer_bit_exact(eng, oracle):
    rng = np.random.default_rng(7)
    for cols, batch in [(256, 1), (4096, 1), (14336, 1), (4096, 4), (5120, 8)]:
        x = synth.make_x(rng, cols, batch)
        x[:256] = 0.0
        if cols > 512:
            x[300], x[301] = 5.5, -5.5
            x[700] = -9.25
        q = eng.alloc_q8k(cols, batch)
        eng.quantize_q8k(eng.upload_f32(x), q)
        d, qs, bs = q.read()
        eng.sync()
        for k in range(batch):
            rd, rqs, rbs = oracle.quantize_row_q8_k(x[k * cols:(k + 1) * cols])
            assert np.array_equal(bits(d[k]), bits(rd))
            assert np.array_equal(qs[k], rqs) and np.array_equal(bs[k], rbs)


@pytest.mark.parametrize("qtype", [Q4_K, Q5_K, Q6_K, Q8_0, Q1_0, Q2_0])
def test_matvec_matches_oracle(eng, oracle, qtype):
    rng = np.random.default_rng(200 + qtype)
    for rows, cols in SHAPES[qtype]:
        data = synth.make_weights(qtype, rng, rows, cols)
        x = synth.make_x(rng, cols)
        w = eng.upload_weights_typed(data, rows, cols, quant(qtype))
        got = eng.matvec(w, x)
        ref = oracle.matvec(qtype, x, data, rows, cols)
        assert_close(got, ref, f"{synth.TYPE_NAMES[qtype]} {rows}x{cols}")


@pytest.mark.parametrize("qtype", [Q4_K, Q6_K, Q1_0])
def test_matvec_preq_matches_oracle(eng, oracle, qtype):
    rng = np.random.default_rng(300 + qtype)
    rows, cols = 37, 5120 if qtype == Q1_0 else 4096
    cols = cols // 256 * 256
    data = synth.make_weights(qtype, rng, rows, cols)
    x = synth.make_x(rng, cols)
    q8 = oracle.quantize_row_q8_k(x)
    w = eng.upload_weights_typed(data, rows, cols, quant(qtype))
    q = eng.upload_q8k(*q8, cols, 1)
    y = eng.alloc_f32(rows)
    eng.matvec_preq_dev(w, q, y)
    got = eng.read_f32(y)
    eng.sync()
    assert_close(got, oracle.matvec_preq(qtype, data, rows, cols, q8), synth.TYPE_NAMES[qtype])


@pytest.mark.parametrize("qtype", [Q4_K, Q5_K, Q6_K])
def test_fused_quantization_equals_prequantized_path(eng, oracle, qtype):
    """alice_matvec quantizes x to Q8_K inside the kernel; the result must be bit-identical to
    alice_matvec_preq fed with the oracle's Q8_K blocks of the same x (same kernel arithmetic)."""
    rng = np.random.default_rng(900 + qtype)
    for rows, cols in [(50, 4096), (9, 14336), (4, 256)]:
        data = synth.make_weights(qtype, rng, rows, cols)
        x = synth.make_x(rng, cols)
        x[:256] = 0.0
        if cols > 512:
            x[300], x[301], x[700] = 5.5, -5.5, -9.25
        w = eng.upload_weights_typed(data, rows, cols, quant(qtype))
        fused = eng.matvec(w, x)
        q = eng.upload_q8k(*oracle.quantize_row_q8_k(x), cols, 1)
        y = eng.alloc_f32(rows)
        eng.matvec_preq_dev(w, q, y)
        pre = eng.read_f32(y)
        eng.sync()
        assert np.array_equal(bits(fused), bits(pre)), (synth.TYPE_NAMES[qtype], rows, cols)


@pytest.mark.parametrize("qtype,rows,cols", [(Q4_K, 300, 4096), (Q4_K, 17, 512), (Q1_0, 200, 5120), (Q6_K, 33, 1024),
                                             (Q8_0, 40, 1024)])
def test_swiglu_matches_oracle(eng, oracle, qtype, rows, cols):
    rng = np.random.default_rng(400 + qtype)
    gate = synth.make_weights(qtype, rng, rows, cols)
    up = synth.make_weights(qtype, rng, rows, cols)
    x = synth.make_x(rng, cols)
    g = eng.upload_weights_typed(gate, rows, cols, quant(qtype))
    u = eng.upload_weights_typed(up, rows, cols, quant(qtype))
    y = eng.alloc_f32(rows)
    eng.swiglu_dev(g, u, eng.upload_f32(x), y, 1)
    got = eng.read_f32(y)
    eng.sync()
    assert_close(got, oracle.swiglu(qtype, x, gate, up, rows, cols), synth.TYPE_NAMES[qtype])


@pytest.mark.parametrize("qtype,batch,rows,cols", [(Q4_K, 4, 130, 4096), (Q6_K, 4, 130, 4096), (Q1_0, 8, 130, 5120), (Q8_0, 2, 130, 5120),
                                                   (Q4_K, 8, 1000, 4096), (Q5_K, 3, 77, 2048), (Q6_K, 8, 300, 14336), (Q4_K, 2, 33, 256),
                                                   (Q4_K, 5, 4096, 14336), (Q6_K, 7, 16, 1024)])
def test_batched_matvec_matches_oracle(eng, oracle, qtype, batch, rows, cols):
    rng = np.random.default_rng(500 + qtype)
    data = synth.make_weights(qtype, rng, rows, cols)
    x = synth.make_x(rng, cols, batch)
    w = eng.upload_weights_typed(data, rows, cols, quant(qtype))
    y = eng.alloc_f32(rows * batch)
    eng.matvec_dev(w, eng.upload_f32(x), y, batch)
    got = eng.read_f32(y).reshape(batch, rows)
    eng.sync()
    for k in range(batch):   # layout x[k*cols + c] -> y[k*rows + r] (src/gpu.rs:1141-1143)
        assert_close(got[k], oracle.matvec(qtype, x[k * cols:(k + 1) * cols], data, rows, cols), f"batch {k}")
    launches, passes = eng.batch_plan(w, batch)
    if qtype in (Q4_K, Q5_K, Q6_K) and synth.row_bytes(qtype, cols) % 16 == 0:
        # the weights stream once for the whole batch; one launch unless 16 rows do not fit a shared-memory stage
        # (rows that are not a multiple of 16 bytes cannot be staged row by row and fall back to one pass per vector)
        assert passes == 1 and launches == (1 if cols <= 4096 else launches), (launches, passes)
        assert launches <= 8


@pytest.mark.parametrize("batch", [4, 8])
def test_batched_swiglu_one_pass_over_the_weights(eng, oracle, batch):
    rng = np.random.default_rng(77)
    rows, cols = 600, 4096
    gate, up = synth.make_q4k(rng, rows, cols), synth.make_q4k(rng, rows, cols)
    x = synth.make_x(rng, cols, batch)
    g, u = eng.upload_weights(gate, rows, cols), eng.upload_weights(up, rows, cols)
    y = eng.alloc_f32(rows * batch)
    eng.swiglu_dev(g, u, eng.upload_f32(x), y, batch)
    got = eng.read_f32(y).reshape(batch, rows)
    eng.sync()
    for k in range(batch):
        assert_close(got[k], oracle.swiglu(Q4_K, x[k * cols:(k + 1) * cols], gate, up, rows, cols), f"swiglu batch {k}")
    assert eng.batch_plan(g, batch, swiglu=True) == (1, 1)


@pytest.mark.parametrize("rows,cols", [(5, 128), (3, 100), (70, 8192), (12, 28672), (9, 1000), (600, 8192), (33, 14336 + 128)])
def test_ternary_matvec_matches_oracle(eng, oracle, rows, cols):
    rng = np.random.default_rng(600 + cols)
    pos, neg, sc = synth.make_ternary(rng, rows, cols)
    x = synth.make_x(rng, cols)
    w = eng.upload_ternary(pos, neg, sc, rows, cols)
    assert_close(eng.matvec(w, x), oracle.ternary_matvec(pos, neg, sc, rows, cols, x), f"ternary {rows}x{cols}")
    # bit-exact dequantization: scale * {-1, 0, +1}
    p = np.unpackbits(pos, axis=1, bitorder="little")[:, :cols].astype(np.float32)
    n = np.unpackbits(neg, axis=1, bitorder="little")[:, :cols].astype(np.float32)
    assert np.array_equal(bits(eng.dequantize(w)), bits((sc[:, None] * (p - n)).reshape(-1)))


@pytest.mark.parametrize("rows,cols", [(5, 128), (4, 48), (70, 8192), (12, 28672)])
def test_sparse_ternary_matvec_matches_oracle(eng, oracle, rows, cols):
    rng = np.random.default_rng(700 + cols)
    pos, neg, sc = synth.make_ternary(rng, rows, cols)
    active, sign = synth.ternary_to_sparse(pos, neg, cols)
    packed = oracle.sparse_pack_2bit(active, sign, rows, cols)
    x = synth.make_x(rng, cols)
    w = eng.upload_sparse_ternary(packed, sc, rows, cols)
    assert_close(eng.matvec(w, x), oracle.sparse_ternary_matvec(active, sign, sc, rows, cols, x), f"sparse {rows}x{cols}")


def test_ternary_swiglu_matches_oracle(eng, oracle):
    rng = np.random.default_rng(8)
    rows, cols = 150, 8192
    g = synth.make_ternary(rng, rows, cols)
    u = synth.make_ternary(rng, rows, cols)
    x = synth.make_x(rng, cols)
    y = eng.alloc_f32(rows)
    eng.swiglu_dev(eng.upload_ternary(*g, rows, cols), eng.upload_ternary(*u, rows, cols), eng.upload_f32(x), y, 1)
    got = eng.read_f32(y)
    eng.sync()
    assert_close(got, oracle.ternary_swiglu(g, u, rows, cols, x), "ternary swiglu")


def test_reference_known_answers_on_gpu(eng):
    """The reference's own known-answer cases (src/gguf.rs:7257-7283, 7419-7445) through the C ABI."""
    from alice_llm_b200 import gguf
    data = np.zeros(68, dtype=np.uint8)
    data[0:2] = [0x00, 0x3C]; data[2] = 1
    data[34:36] = [0x00, 0x3C]; data[37] = 1
    x = np.zeros(32, np.float32); x[0], x[1] = 3.0, 7.0
    y = gguf.q8_0_matvec(x, data, 2, 32)
    assert abs(y[0] - 3.0) < 1e-4 and abs(y[1] - 7.0) < 1e-4
    d2 = np.zeros(34, dtype=np.uint8); d2[0:2] = [0x00, 0x3C]; d2[2:] = 0x46
    y = gguf.quantized_matvec(np.arange(1, 129, dtype=np.float32), d2, gguf.GgmlType.Q2_0, 1, 128)
    assert abs(y[0] + 64.0) < 1e-3


def test_errors_instead_of_panics(eng):
    from alice_llm_b200.gpu import AliceError, GpuQuantType
    with pytest.raises(AliceError):   # cols not a whole number of blocks
        eng.upload_weights_typed(np.zeros(144, np.uint8), 1, 200, GpuQuantType.Q4K)
    with pytest.raises(AliceError):   # byte count does not match
        eng.upload_weights_typed(np.zeros(100, np.uint8), 1, 256, GpuQuantType.Q4K)
    w = eng.upload_weights_typed(np.zeros(144, np.uint8), 1, 256, GpuQuantType.Q4K)
    with pytest.raises(AliceError):   # input too short
        eng.matvec_dev(w, eng.alloc_f32(100), eng.alloc_f32(1), 1)
    with pytest.raises(AliceError):   # batch outside 1..8
        eng.matvec_dev(w, eng.alloc_f32(256 * 9), eng.alloc_f32(9), 9)


def test_handles_may_outlive_their_engine():
    """A binding whose drop order frees the engine first must not crash: handles keep what they need alive."""
    from alice_llm_b200 import _lib
    from alice_llm_b200.gpu import GpuEngine, GpuQuantType
    e = GpuEngine(0)
    rng = np.random.default_rng(3)
    w = e.upload_weights_typed(synth.make_q4k(rng, 8, 256), 8, 256, GpuQuantType.Q4K)
    b = e.alloc_f32(256)
    q = e.alloc_q8k(256, 1)
    lib = _lib.load()
    h, e._h = e._h, None          # destroy the engine behind the wrappers' back, children still alive
    assert lib.alice_engine_destroy(h) == 0
    w.free(); b.free(); q.free()


def test_host_pointer_entry_points_match_oracle(oracle):
    """alice_matvec_host / alice_dequantize_host are what a gguf.rs-level binding of quantized_matvec and
    dequantize_weight_row calls (host slices in, host slices out)."""
    import ctypes as C
    from alice_llm_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(12)
    for qtype, rows, cols in [(Q4_K, 300, 4096), (Q6_K, 64, 1024), (Q8_0, 33, 512), (Q1_0, 17, 1024)]:
        data = synth.make_weights(qtype, rng, rows, cols)
        x = synth.make_x(rng, cols)
        y = np.empty(rows, np.float32)
        rc = lib.alice_matvec_host(qtype, C.c_void_p(data.ctypes.data), data.size, rows, cols, C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data))
        assert rc == 0, lib.alice_last_error()
        assert_close(y, oracle.matvec(qtype, x, data, rows, cols), f"host matvec {synth.TYPE_NAMES[qtype]}")
        rb = synth.row_bytes(qtype, cols)
        out = np.empty(cols, np.float32)
        rc = lib.alice_dequantize_host(qtype, C.c_void_p(data.ctypes.data), rb, C.c_void_p(out.ctypes.data), cols)
        assert rc == 0, lib.alice_last_error()
        # (dequantize_weight_row itself returns zeros for Q1_0 / Q2_0, src/gguf.rs:6168-6195; the library dequantizes them)
        assert np.array_equal(bits(out), bits(oracle.dequantize(qtype, data[:rb])))
    assert lib.alice_matvec_host(2, C.c_void_p(data.ctypes.data), data.size, rows, cols, C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data)) != 0


def test_engines_on_two_devices_in_one_process(oracle):
    """Per-device state (the opt-in shared-memory attribute of every kernel instance, the fixed no-allocation scratch) must
    be set up on each device an engine is created on: the same matvecs on device 0, then device 1, then device 0 again."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from alice_llm_b200.gpu import GpuEngine
    rng = np.random.default_rng(77)
    cases = [(Q4_K, 70, 4096), (Q6_K, 40, 14336), (Q1_0, 70, 5120), (Q8_0, 50, 5120)]
    data = {(qt, r, c): (synth.make_weights(qt, rng, r, c), synth.make_x(rng, c)) for qt, r, c in cases}
    engines = [GpuEngine(0), GpuEngine(1)]
    for eng in (engines[0], engines[1], engines[0]):
        for (qt, r, c), (w, x) in data.items():
            got = eng.matvec(eng.upload_weights_typed(w, r, c, quant(qt)), x)
            assert_close(got, oracle.matvec(qt, x, w, r, c), f"device {eng.device} type {qt}")
        # the no-allocation entry point keeps one fixed array per device
        w, x = data[(Q1_0, 70, 5120)]
        wd = eng.upload_weights_typed(w, 70, 5120, quant(Q1_0))
        q = eng.alloc_q8k(5120, 1)
        eng.quantize_q8k(eng.upload_f32(x), q)
        y1, y2 = eng.alloc_f32(70), eng.alloc_f32(70)
        eng.matvec_preq_dev(wd, q, y1)
        eng.matvec_preq_noalloc_dev(wd, q, y2)
        assert np.array_equal(eng.read_f32(y1).view(np.uint32), eng.read_f32(y2).view(np.uint32))
    for eng in engines:
        eng.close()


@pytest.mark.parametrize("rows,cols", [(70, 200), (33, 8192), (5, 16), (130, 1000)])
def test_device_ternarizers_bit_exact(eng, oracle, rows, cols):
    """alice_ternarize / alice_sparsify against the oracle's TernaryRow::from_f32 and SparseTernaryRow::from_ternary_row:
    masks, packed codes and scales equal bit for bit (weights rounded to a coarse grid, so magnitudes tie often and the
    stable-sort rule decides which weights of a block stay)."""
    rng = np.random.default_rng(rows * 7 + cols)
    w = np.round(rng.standard_normal((rows, cols)).astype(np.float32) * 4) / 4
    w[0] = 0.0                                       # a row that keeps nothing
    wd = eng.upload_f32(w)
    src_pb, pb = (cols + 7) // 8, (cols + 31) // 32 * 4
    for ratio in (0.7, 0.0):
        t = eng.ternarize(wd, rows, cols, ratio)
        got_rows, got_scales = eng.download_weights(t)
        want = [oracle.ternarize_row(w[r], ratio) for r in range(rows)]
        for r, (pos, neg, scale) in enumerate(want):
            assert np.array_equal(got_rows[r, :src_pb], pos) and np.array_equal(got_rows[r, pb:pb + src_pb], neg), (ratio, r)
            assert not got_rows[r, src_pb:pb].any() and not got_rows[r, pb + src_pb:].any()
            assert bits(got_scales[r]) == bits(scale), (ratio, r, got_scales[r], scale)
        # the device matrix is usable as it is
        x = synth.make_x(rng, cols)
        pos = np.stack([p for p, _, _ in want]); neg = np.stack([n for _, n, _ in want])
        sc = np.array([s for _, _, s in want], np.float32)
        y = eng.alloc_f32(rows)
        eng.matvec_dev(t, eng.upload_f32(x), y, 1)
        assert_close(eng.read_f32(y), oracle.ternary_matvec(pos, neg, sc, rows, cols, x), "matvec over the device-made planes")
        for n_keep in (3, 16):
            s = eng.sparsify(t, wd, n_keep)
            got_packed, got_sscales = eng.download_weights(s)
            for r, (p, n, scale) in enumerate(want):
                active, sign, sscale = oracle.sparsify_row(p, n, scale, w[r], n_keep)
                packed = oracle.sparse_pack_2bit(active, sign, 1, cols)
                assert np.array_equal(got_packed[r], packed), (ratio, n_keep, r)
                assert bits(got_sscales[r]) == bits(sscale), (ratio, n_keep, r)
            s.free()
        t.free()


def test_bounded_wait_runs_out_and_engine_stays_usable(oracle):
    """A wait inside a kernel that nothing will ever satisfy (a hand-over flag nobody raises) returns after the engine's
    cycle budget with a status the host reads: ALICE_E_KERNEL from alice_sync, naming the wait, and work queued after it
    is correct. Nothing here faults or hangs the GPU: the kernel gives up by itself after a few milliseconds."""
    import time
    from alice_llm_b200 import _lib
    from alice_llm_b200.gpu import AliceError, GpuEngine
    eng = GpuEngine(0)
    rng = np.random.default_rng(5)
    data, x = synth.make_q4k(rng, 70, 4096), synth.make_x(rng, 4096)
    w = eng.upload_weights(data, 70, 4096)
    ref = oracle.matvec(Q4_K, x, data, 70, 4096)
    assert_close(eng.matvec(w, x), ref, "before")
    eng.set_wait_limit(4_000_000)            # about 2 ms of SM cycles
    t0 = time.perf_counter()
    eng.debug_expire_wait()
    with pytest.raises(AliceError) as ei:
        eng.sync()
    assert time.perf_counter() - t0 < 1.0
    assert ei.value.code == _lib.E_KERNEL and "status 6" in str(ei.value) and "peer" in str(ei.value)
    eng.sync()                               # the status word was cleared by the report
    eng.set_wait_limit(0)
    assert_close(eng.matvec(w, x), ref, "after")
    eng.close()
