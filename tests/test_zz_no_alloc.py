"""alice_matvec_preq_noalloc: the pre-quantized Q1_0 / Q2_0 matvec for callers that cannot allocate
device memory (all HBM owned by their own pool, or a decode thread that must not pay the device-wide
synchronisation of cudaMalloc / cudaFree). Its f32 scratch is a fixed array inside the library, so the
test checks, through the C ABI, that it returns what alice_matvec_preq returns - twice in a row, since
the array is shared and keeps the previous call's contents - and that it refuses what does not fit.
Collected last on purpose: a failure here cannot hide one elsewhere in a run that stops at the first."""
import numpy as np
import pytest

from alice_llm_b200 import synth

pytestmark = pytest.mark.gpu
NOALLOC_MAX_FLOATS = 65536


def test_noalloc_preq_equals_preq_twice_in_a_row(oracle):
    from alice_llm_b200.gpu import AliceError, GpuEngine, GpuQuantType
    eng = GpuEngine(0)
    rng = np.random.default_rng(42)
    cases = [(synth.Q1_0, 96, 5120, 1), (synth.Q2_0, 40, 2048, 3)]
    for round_ in range(2):                      # second round runs on top of the first round's scratch contents
        for qtype, rows, cols, batch in cases:
            data = synth.make_weights(qtype, rng, rows, cols)
            x = synth.make_x(rng, cols, batch)
            w = eng.upload_weights_typed(data, rows, cols, GpuQuantType(qtype))
            q = eng.alloc_q8k(cols, batch)
            eng.quantize_q8k(eng.upload_f32(x), q)
            y_ref, y_new = eng.alloc_f32(rows * batch), eng.alloc_f32(rows * batch)
            eng.matvec_preq_dev(w, q, y_ref)
            eng.matvec_preq_noalloc_dev(w, q, y_new)
            ref, new = eng.read_f32(y_ref), eng.read_f32(y_new)
            eng.sync()
            # same kernels, same inputs: equal within the suite's matvec tolerance (in fact bit for bit)
            err = np.abs(new.astype(np.float64) - ref) / np.maximum(np.abs(ref), 1.0)
            assert err.max() <= 1e-3, (round_, qtype, err.max())
            assert np.array_equal(new.view(np.uint32), ref.view(np.uint32))
            # and both agree with the CPU oracle's quantized_matvec_preq
            for k in range(batch):
                q8 = oracle.quantize_row_q8_k(x[k * cols:(k + 1) * cols])
                want = oracle.matvec_preq(qtype, data, rows, cols, q8)
                e2 = np.abs(new[k * rows:(k + 1) * rows].astype(np.float64) - want) / np.maximum(np.abs(want), 1.0)
                assert e2.max() <= 1e-3

    # sizes beyond the fixed array are refused, as are formats that need no scratch
    cols = 25600
    w_big = eng.upload_weights_typed(synth.make_q1_0(rng, 2, cols), 2, cols, GpuQuantType.Q1_0)
    q_big = eng.alloc_q8k(cols, 3)               # 3 * 25600 = 76800 > 65536
    assert 3 * cols > NOALLOC_MAX_FLOATS
    with pytest.raises(AliceError) as ei:
        eng.matvec_preq_noalloc_dev(w_big, q_big, eng.alloc_f32(6))
    assert "exceeds the fixed scratch" in str(ei.value)
    w_q4 = eng.upload_weights_typed(synth.make_q4k(rng, 2, 256), 2, 256, GpuQuantType.Q4K)
    with pytest.raises(AliceError):
        eng.matvec_preq_noalloc_dev(w_q4, eng.alloc_q8k(256, 1), eng.alloc_f32(2))
    eng.close()


def test_noalloc_calls_leave_free_memory_unchanged():
    """After one warm-up call per shape (module loading, the address look-up of the fixed array) further calls must not
    change the device's free memory: no cudaMalloc, no growth of a scratch buffer."""
    import torch
    from alice_llm_b200.gpu import GpuEngine, GpuQuantType
    eng = GpuEngine(0)
    rng = np.random.default_rng(43)
    cases = []
    for qtype, rows, cols, batch in [(synth.Q1_0, 96, 5120, 1), (synth.Q2_0, 40, 2048, 3), (synth.Q1_0, 64, 25600, 2)]:
        w = eng.upload_weights_typed(synth.make_weights(qtype, rng, rows, cols), rows, cols, GpuQuantType(qtype))
        q = eng.alloc_q8k(cols, batch)
        eng.quantize_q8k(eng.upload_f32(synth.make_x(rng, cols, batch)), q)
        cases.append((w, q, eng.alloc_f32(rows * batch)))
    for w, q, y in cases:                        # warm-up
        eng.matvec_preq_noalloc_dev(w, q, y)
    eng.sync()
    free0, _ = torch.cuda.mem_get_info(0)
    for _ in range(20):
        for w, q, y in cases:
            eng.matvec_preq_noalloc_dev(w, q, y)
    eng.sync()
    free1, _ = torch.cuda.mem_get_info(0)
    assert free1 == free0, (free0, free1)
    eng.close()
