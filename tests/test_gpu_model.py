"""GPU parity of the decode model (alice_model_*) against the CPU oracle's Llama forward on small
synthetic models: logits per step, greedy token ids, KV cache contents, rollback / reset."""
import numpy as np
import pytest

from alice_llm_b200 import synth

pytestmark = pytest.mark.gpu

CFG = dict(num_layers=2, hidden_dim=512, intermediate_dim=1024, num_heads=4, num_kv_heads=2, head_dim=128,
           vocab_size=1000, max_seq_len=160, rope_theta=500000.0, eps=1e-5)


def close(got, ref, tol=1e-3):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    err = np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)
    l2 = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
    return err.max(), l2


@pytest.fixture(scope="module")
def eng():
    from alice_llm_b200.gpu import GpuEngine
    e = GpuEngine(0)
    yield e
    e.close()


def prefill(rng, cfg, gm, orc, npos):
    kv_dim = cfg["num_kv_heads"] * cfg["head_dim"]
    for l in range(cfg["num_layers"]):
        k = rng.standard_normal((npos, kv_dim), dtype=np.float32)
        v = rng.standard_normal((npos, kv_dim), dtype=np.float32)
        gm.kv_write(l, 0, k, v)
        orc.kcache[l, :npos] = k
        orc.vcache[l, :npos] = v
    gm.set_position(npos)
    orc.pos = npos


Q1_MIX = {n: synth.Q1_0 for n in ("q", "k", "v", "o", "gate", "up", "down")}
Q1_MIX["output"] = synth.Q8_0   # the 27B binary-weight configuration: Q1_0 projections, Q8_0 head, 5 query heads per KV head


@pytest.mark.parametrize("mix,heads", [(None, (4, 2)), ({"v": synth.Q6_K, "down": synth.Q4_K, "output": synth.Q8_0}, (8, 2)),
                                       ({n: synth.TERNARY for n in ("q", "k", "v", "o", "gate", "up", "down", "output")}, (8, 2)),
                                       (Q1_MIX, (10, 2)), ({**Q1_MIX, "k": synth.Q2_0, "gate": synth.Q2_0, "up": synth.Q2_0}, (4, 4))])
def test_forward_logits_match_oracle(eng, oracle, mix, heads):
    from alice_llm_b200.gpu import GpuModel
    cfg = dict(CFG, num_heads=heads[0], num_kv_heads=heads[1])
    rng = np.random.default_rng(5)
    model = synth.make_llama(rng, cfg, mix)
    gm = GpuModel.load(eng, model)
    orc = oracle.LlamaOracle(model)
    prefill(rng, cfg, gm, orc, 37)
    for step, tok in enumerate([1, 17, 999, 3, 500]):
        got = gm.forward_and_read(tok)
        ref = orc.forward(tok)
        e, l2 = close(got, ref)
        assert e <= 1e-3 and l2 <= 1e-3, (step, e, l2)
        assert gm.position() == orc.pos
    # the K/V rows appended on the device equal the oracle's
    for l in range(cfg["num_layers"]):
        k, v = gm.kv_read(l, 37, 5)
        assert close(k, orc.kcache[l, 37:42])[0] <= 1e-3 and close(v, orc.vcache[l, 37:42])[0] <= 1e-3
    gm.free()


def test_greedy_decode_matches_oracle_and_graph_replay(eng, oracle):
    from alice_llm_b200.gpu import GpuModel
    rng = np.random.default_rng(6)
    model = synth.make_llama(rng, CFG)
    gm = GpuModel.load(eng, model)
    orc = oracle.LlamaOracle(model)
    prefill(rng, CFG, gm, orc, 20)
    n = 12
    got = gm.decode_greedy(1, n)
    tok, want, gaps = 1, [], []
    for _ in range(n):
        logits = orc.forward(tok)
        top = np.sort(logits)[-2:]
        gaps.append(float(top[1] - top[0]))
        tok = int(np.argmax(logits))
        want.append(tok)
    # identical ids unless the oracle's own top-2 gap at the first difference is within rounding noise
    diff = [i for i in range(n) if got[i] != want[i]]
    assert not diff or gaps[diff[0]] < 1e-4, (list(got), want, gaps)
    assert gm.position() == 20 + n
    # a second call continues from the device-side state and replays the captured graph
    got2 = gm.decode_greedy(int(got[-1]), 4)
    if not diff:
        for i in range(4):
            logits = orc.forward(tok)
            tok = int(np.argmax(logits))
            assert got2[i] == tok or np.sort(logits)[-1] - np.sort(logits)[-2] < 1e-4
    gm.free()


def test_rollback_reset_and_limits(eng, oracle):
    from alice_llm_b200.gpu import AliceError, GpuModel
    rng = np.random.default_rng(7)
    model = synth.make_llama(rng, CFG)
    gm = GpuModel.load(eng, model)
    a = gm.forward_and_read(5)
    gm.forward(6)
    gm.forward(7)
    assert gm.position() == 3
    gm.rollback_to(1)                    # only lowers the counter (src/gpu.rs:5645)
    assert gm.position() == 1
    gm.rollback_to(9)
    assert gm.position() == 1
    gm.reset()                           # zeroes the cache too (src/gpu.rs:5618)
    assert gm.position() == 0
    k, v = gm.kv_read(0, 0, 3)
    assert not k.any() and not v.any()
    b = gm.forward_and_read(5)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))   # deterministic run to run
    gm.set_position(CFG["max_seq_len"])
    with pytest.raises(AliceError):
        gm.forward(1)
    with pytest.raises(AliceError):
        gm.forward_and_read(CFG["vocab_size"])
    gm.free()


@pytest.mark.parametrize("mix,heads", [(None, (4, 2)), ("smooth", (8, 2)), (Q1_MIX, (10, 2)),
                                       ({n: synth.TERNARY for n in ("q", "k", "v", "o", "gate", "up", "down", "output")}, (8, 2))])
@pytest.mark.parametrize("nbatch", [4, 8])
def test_forward_batch_matches_token_by_token_oracle(eng, oracle, mix, heads, nbatch):
    """forward_batch_and_read (src/gpu.rs:6057): token k of the batch sits at position + k and attends position + k + 1
    rows, so its logits equal those of feeding the tokens one by one; then rollback_to and a second, different batch
    (the accept / reject loop of examples/speculative_dual_gpu.rs:230-322)."""
    from alice_llm_b200.gpu import GpuModel
    from softmodel import SMOOTH_MIX, soft_model, steps_pass
    cfg = dict(CFG, num_heads=heads[0], num_kv_heads=heads[1])
    rng = np.random.default_rng(21)
    smooth = mix == "smooth"
    mix = SMOOTH_MIX if smooth else mix
    model = soft_model(rng, cfg, mix) if (mix is None or smooth) else synth.make_llama(rng, cfg, mix)
    gm = GpuModel.load(eng, model)
    orc = oracle.LlamaOracle(model)
    prefill(rng, cfg, gm, orc, 29)
    toks = [int(t) for t in rng.integers(0, cfg["vocab_size"], nbatch)]
    got = gm.forward_batch_and_read(toks).reshape(nbatch, -1)
    assert gm.position() == 29 + nbatch
    res = [close(got[k], orc.forward(t)) for k, t in enumerate(toks)]
    errs, l2s = [r[0] for r in res], [r[1] for r in res]
    assert (max(errs) <= 1e-3 and max(l2s) <= 1e-3) if smooth else steps_pass(errs, l2s), (errs, l2s)
    k_dev, v_dev = gm.kv_read(1, 29, nbatch)
    assert close(k_dev, orc.kcache[1, 29:29 + nbatch])[0] <= 1e-3 and close(v_dev, orc.vcache[1, 29:29 + nbatch])[0] <= 1e-3
    # reject everything after the second token, verify another continuation from there
    gm.rollback_to(31)
    orc.pos = 31
    toks2 = [int(t) for t in rng.integers(0, cfg["vocab_size"], 4)]
    got2 = gm.forward_batch_and_read(toks2).reshape(4, -1)
    res = [close(got2[k], orc.forward(t)) for k, t in enumerate(toks2)]
    errs, l2s = [r[0] for r in res], [r[1] for r in res]
    assert (max(errs) <= 1e-3 and max(l2s) <= 1e-3) if smooth else steps_pass(errs, l2s), ("after rollback", errs, l2s)
    gm.free()


def test_forward_sparse_ternary_matches_oracle(eng, oracle):
    """Every projection and the head as SparseTernaryMatrix (packed 2-bit codes) through GpuModel.load: the weights are
    those of the ternary bit-plane model, so the oracle's forward of that model is the reference
    (Llama3Model::forward_sparse_ternary, src/llama3.rs:17216-17330, sums the same +x / -x terms)."""
    from alice_llm_b200.gpu import GpuModel
    cfg = dict(CFG, num_heads=8, num_kv_heads=2)
    rng = np.random.default_rng(15)
    tern = synth.make_llama(rng, cfg, {n: synth.TERNARY for n in ("q", "k", "v", "o", "gate", "up", "down", "output")})
    model = synth.to_sparse_ternary(tern)
    # the packing agrees with the oracle's restatement of the reference packer
    pos, neg, _ = tern["layers"][0]["down"][1]
    active, sign = synth.ternary_to_sparse(pos, neg, cfg["intermediate_dim"])
    want = oracle.sparse_pack_2bit(active, sign, cfg["hidden_dim"], cfg["intermediate_dim"])
    assert np.array_equal(model["layers"][0]["down"][1][0].reshape(-1), want)
    gm = GpuModel.load(eng, model)
    orc = oracle.LlamaOracle(tern)
    prefill(rng, cfg, gm, orc, 29)
    for step, tok in enumerate([2, 640, 77]):
        e, l2 = close(gm.forward_and_read(tok), orc.forward(tok))
        assert e <= 1e-3 and l2 <= 1e-3, (step, e, l2)
    got = gm.decode_greedy(9, 6)
    ref, tok = [], 9
    for _ in range(6):
        tok = int(np.argmax(orc.forward(tok)))
        ref.append(tok)
    assert [int(t) for t in got] == ref
    gm.free()


def test_two_models_share_one_engine(eng, oracle):
    """GpuModel::load_shared: a draft and a target model on one engine, steps interleaved (the speculative-decoding loop
    of examples/speculative_dual_gpu.rs: the draft proposes, the target verifies a batch, both roll back on a mismatch);
    each must decode exactly as it does alone."""
    from alice_llm_b200.gpu import GpuModel
    rng = np.random.default_rng(31)
    big_cfg = dict(CFG, num_heads=8, num_kv_heads=2)
    small_cfg = dict(CFG, num_layers=1, intermediate_dim=512)
    target, draft = synth.make_llama(rng, big_cfg), synth.make_llama(rng, small_cfg)
    gt, gd = GpuModel.load_shared(eng, target), GpuModel.load_shared(eng, draft)
    alone_t, alone_d = oracle.LlamaOracle(target), oracle.LlamaOracle(draft)
    tok_t, tok_d = 7, 7
    for step in range(4):
        lt, ld = gt.forward_and_read(tok_t), gd.forward_and_read(tok_d)     # interleaved on the shared stream
        rt, rd = alone_t.forward(tok_t), alone_d.forward(tok_d)
        for got, ref in ((lt, rt), (ld, rd)):
            e, l2 = close(got, ref)
            assert e <= 1e-3 and l2 <= 1e-3, (step, e, l2)
        tok_t, tok_d = int(np.argmax(rt)), int(np.argmax(rd))
    # the draft runs ahead, the target verifies the proposals as one batch, then both return to the accepted prefix
    proposals = [int(t) for t in gd.decode_greedy(tok_d, 3)]
    pos = gt.position()
    logits = gt.forward_batch_and_read([tok_t] + proposals[:2])
    assert logits.size == 3 * big_cfg["vocab_size"] and gt.position() == pos + 3
    gt.rollback_to(pos + 1)
    gd.rollback_to(pos + 1)
    assert gt.position() == pos + 1 and gd.position() == pos + 1
    gt.free(); gd.free()
