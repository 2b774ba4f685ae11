"""GPU parity of the decode attention and of the whole step at model shapes, against the CPU oracle's forward
(gqa_attention, src/llama3.rs:5431-5690, is the contract for the attention; forward_with_layer_hook for the step).

synth.make_llama draws weights whose q.k scores are so large that the softmax is one-hot on the row the model itself
appended, so a kernel that mis-read the pre-filled context would pass.  Here the q / k / v projections are scaled down
until the pre-filled rows carry the attention, and every case first proves that on the oracle: zeroing a band of
pre-filled V rows must move the oracle's logits by far more than the parity tolerance."""
import numpy as np
import pytest

from alice_llm_b200 import synth

pytestmark = pytest.mark.gpu

from softmodel import SMOOTH_MIX, scale_blocks, soft_model, steps_pass  # noqa: F401


@pytest.fixture(scope="module")
def eng():
    from alice_llm_b200.gpu import GpuEngine
    e = GpuEngine(0)
    yield e
    e.close()


def rel_err(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)).max())


def rel_l2(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


def fill(rng, cfg, npos, gm, oracles):
    kv_dim = cfg["num_kv_heads"] * cfg["head_dim"]
    for l in range(cfg["num_layers"]):
        k = rng.standard_normal((npos, kv_dim), dtype=np.float32)
        v = rng.standard_normal((npos, kv_dim), dtype=np.float32)
        if gm is not None:
            gm.kv_write(l, 0, k, v)
        for o in oracles:
            o.kcache[l, :npos] = k
            o.vcache[l, :npos] = v
    if gm is not None:
        gm.set_position(npos)
    for o in oracles:
        o.pos = npos


@pytest.mark.parametrize("heads", [(2, 2), (4, 2), (8, 2), (10, 2), (16, 2)])   # 1, 2, 4, 5, 8 query heads per KV head
@pytest.mark.parametrize("ctx,mix", [(37, SMOOTH_MIX), (2048, SMOOTH_MIX), (4096, SMOOTH_MIX), (2048, None)])
def test_attention_over_prefilled_context(eng, oracle, heads, ctx, mix):
    from alice_llm_b200.gpu import GpuModel
    cfg = dict(num_layers=2, hidden_dim=512, intermediate_dim=1024, num_heads=heads[0], num_kv_heads=heads[1], head_dim=128,
               vocab_size=1000, max_seq_len=ctx + 16, rope_theta=500000.0, eps=1e-5)
    toks = [3, 700, 41, 999, 5, 12]
    lo, hi = ctx // 3, ctx // 3 + max(4, ctx // 4)
    for attempt in range(8):
        # the pre-filled rows must matter: without a band of them the oracle's own logits have to move by >> 1e-3;
        # a draw whose softmax is (nearly) one-hot is discarded
        rng = np.random.default_rng(1234 + ctx + heads[0] + 100000 * attempt)
        model = soft_model(rng, cfg, mix)
        ref, probe = oracle.LlamaOracle(model), oracle.LlamaOracle(model)
        fill(rng, cfg, ctx, None, [ref, probe])
        kv = [(ref.kcache[l, :ctx].copy(), ref.vcache[l, :ctx].copy()) for l in range(cfg["num_layers"])]
        probe.vcache[:, lo:hi] = 0.0
        first = ref.forward(toks[0])
        moved = rel_err(probe.forward(toks[0]), first)
        if moved > 2e-2:
            break
    assert moved > 2e-2, f"attention of this model ignores its context (probe moved logits by {moved:.2e})"
    want = [first] + [ref.forward(t) for t in toks[1:]]
    gm = GpuModel.load(eng, model)
    for l, (k, v) in enumerate(kv):
        gm.kv_write(l, 0, k, v)
    gm.set_position(ctx)
    errs, l2s = [], []
    for step, t in enumerate(toks):
        got = gm.forward_and_read(t)
        errs.append(rel_err(got, want[step]))
        l2s.append(rel_l2(got, want[step]))
    if mix is SMOOTH_MIX:      # f32 activations throughout: every step within the gate
        assert max(errs) <= 1e-3 and max(l2s) <= 1e-3, (heads, ctx, errs, l2s)
    else:                      # Q8_K activations (the Q4_K_M mix): see softmodel.steps_pass
        assert steps_pass(errs, l2s), (heads, ctx, errs, l2s)
    k, v = gm.kv_read(1, ctx, len(toks))
    assert rel_err(k, ref.kcache[1, ctx:ctx + len(toks)]) <= 1e-3 and rel_err(v, ref.vcache[1, ctx:ctx + len(toks)]) <= 1e-3
    gm.free()


def test_8b_shapes_two_layers_context_2048(eng, oracle):
    """Llama-3-8B shapes (hidden 4096, ffn 14336, 32 / 8 heads, vocab 128256, Q4_K_M mix), two layers, context 2048
    pre-filled: logits of the first steps and 16 greedy ids against the oracle."""
    from alice_llm_b200.gpu import GpuModel
    cfg = dict(num_layers=2, hidden_dim=4096, intermediate_dim=14336, num_heads=32, num_kv_heads=8, head_dim=128,
               vocab_size=128256, max_seq_len=2048 + 32, rope_theta=500000.0, eps=1e-5)
    rng = np.random.default_rng(8)
    model = soft_model(rng, cfg)
    gm = GpuModel.load(eng, model)
    ref = oracle.LlamaOracle(model, threads=oracle.hw_threads())
    fill(rng, cfg, 2048, gm, [ref])
    errs, l2s = [], []
    for t in (1, 90000, 12345):
        got, want_l = gm.forward_and_read(t), ref.forward(t)
        errs.append(rel_err(got, want_l))
        l2s.append(rel_l2(got, want_l))
    assert steps_pass(errs, l2s), (errs, l2s)
    n = 16
    got = gm.decode_greedy(7, n)
    tok, gaps, want = 7, [], []
    for _ in range(n):
        logits = ref.forward(tok)
        top = np.sort(logits)[-2:]
        gaps.append(float(top[1] - top[0]))
        tok = int(np.argmax(logits))
        want.append(tok)
    diff = [i for i in range(n) if int(got[i]) != want[i]]
    # identical ids unless the oracle's own top-2 gap at the first difference is within rounding noise
    assert not diff or gaps[diff[0]] < 1e-3 * max(1.0, float(np.abs(logits).max())), (list(got), want, gaps)
    if not diff:   # 19 steps of self-appended K / V rows later: drift, not a per-step gate
        assert rel_l2(gm.read_logits(), logits) <= 5e-3
    assert len(set(want)) > 1, "degenerate greedy sequence"
    gm.free()
