"""One rank of the tensor-parallel decode check (started by tests/test_gpu_tp.py, one process per GPU).

Every rank builds the same seeded synthetic model, uploads its row shards, joins the group and decodes
greedily; rank 0 compares logits and token ids with the CPU oracle's forward of the whole model, and all
ranks must agree on the tokens. The group id travels through a gloo process group (host side only).
usage: tp_worker.py RANK WORLD PORT [MIX]   (MIX: kquant (default) | q1_0 | q8_0 | ternary - the weight formats of the model)"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    mix_name = sys.argv[4] if len(sys.argv) > 4 else "kquant"
    import torch.distributed as dist
    from alice_llm_b200 import synth
    from alice_llm_b200.gpu import GpuEngine, GpuModel

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    cfg = dict(num_layers=2, hidden_dim=512, intermediate_dim=1024, num_heads=8, num_kv_heads=4, head_dim=128,
               vocab_size=1000, max_seq_len=96, rope_theta=500000.0, eps=1e-5)
    rng = np.random.default_rng(11)
    roles = ("q", "k", "v", "o", "gate", "up", "down")
    if mix_name == "q1_0":       # the binary-weight configuration: Q1_0 projections, Q8_0 head, 5 query heads per KV head
        cfg.update(num_heads=10, num_kv_heads=2)
        mix = {**{n: synth.Q1_0 for n in roles}, "output": synth.Q8_0}
    elif mix_name == "q8_0":     # f32-activation per-lane kernels on the exchanged vectors: o reads the gathered attention
        mix = {"o": synth.Q8_0, "down": synth.Q8_0, "output": synth.Q8_0}   # output, down the gathered SwiGLU output (the
        # other projections stay K-quant: the reference reaches them through matvec_preq, which has no Q8_0 form)
    elif mix_name == "ternary":  # every projection and the head as ternary bit planes
        mix = {n: synth.TERNARY for n in roles + ("output",)}
    else:
        mix = None
    model = synth.make_llama(rng, cfg, mix)
    # q / k / v scaled down so that the softmax spreads over the pre-filled rows (a dropped or misplaced part of
    # the sharded KV cache then shows up in the logits)
    from softmodel import scale_blocks
    for L in model["layers"]:
        for n in ("q", "k", "v"):
            L[n] = scale_blocks(L[n], 0.3 / float(np.sqrt(cfg["hidden_dim"])))
    kv_dim = cfg["num_kv_heads"] * cfg["head_dim"]
    npos = 21
    pre = [(rng.standard_normal((npos, kv_dim), dtype=np.float32), rng.standard_normal((npos, kv_dim), dtype=np.float32))
           for _ in range(cfg["num_layers"])]

    eng = GpuEngine(rank)
    ids = [eng.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    eng.tp_init(rank, world, ids[0])
    assert eng.tp_info() == (rank, world)
    lkv = kv_dim // world
    from oracle import oracle as orc
    result = {"rank": rank}
    # the same model twice: NCCL all-gathers, then rows pushed into the peers' memory by the kernels
    for mode in ("nccl", "peer"):
        gm = GpuModel.load(eng, model)
        if mode == "peer":
            handles = [None] * world
            dist.all_gather_object(handles, gm.tp_export())
            gm.tp_connect(handles)
        for l, (k, v) in enumerate(pre):   # this rank keeps the cache of its own KV heads
            gm.kv_write(l, 0, np.ascontiguousarray(k[:, rank * lkv:(rank + 1) * lkv]),
                        np.ascontiguousarray(v[:, rank * lkv:(rank + 1) * lkv]))
        gm.set_position(npos)
        logits = [gm.forward_and_read(t) for t in (1, 17, 999)]
        toks = gm.decode_greedy(5, 12)
        last = gm.read_logits()
        result[mode + "_tokens"] = [int(t) for t in toks]
        if rank == 0:
            orc.build()
            o = orc.LlamaOracle(model)
            for l, (k, v) in enumerate(pre):
                o.kcache[l, :npos] = k
                o.vcache[l, :npos] = v
            o.pos = npos
            errs = []
            for t, got in zip((1, 17, 999), logits):
                ref = o.forward(t)
                errs.append(float((np.abs(got.astype(np.float64) - ref) / np.maximum(np.abs(ref), 1.0)).max()))
            ref_toks, tok = [], 5
            for _ in range(12):
                ref = o.forward(tok)
                tok = int(np.argmax(ref))
                ref_toks.append(tok)
            errs.append(float((np.abs(last.astype(np.float64) - ref) / np.maximum(np.abs(ref), 1.0)).max()))
            result[mode + "_max_rel_err"] = max(errs)
            result["oracle_tokens"] = ref_toks
        dist.barrier()      # no rank frees memory its peers may still be writing into
        gm.free()
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    eng.close()
    if rank == 0:
        print(json.dumps(gathered), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
