"""Host-side logic of the row-sharded tensor-parallel path, run as 2 gloo ranks on CPU: the row shards are
contiguous byte ranges that reassemble into the tensor, and a matvec over a shard equals the matching slice
of the matvec over the whole matrix (rows are independent - the property the sharding relies on)."""
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from alice_llm_b200 import synth
    from alice_llm_b200.gpu import shard_rows
    from oracle import oracle as orc
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(3)
        rows, cols = 48, 512
        ok = True
        for qt in (synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q1_0):
            w = synth.make_weights(qt, rng, rows, cols)
            x = synth.make_x(rng, cols)
            shard, n = shard_rows(w, rows, rank, world)
            assert n == rows // world and shard.size == w.size // world
            parts = [torch.empty(shard.size, dtype=torch.uint8) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(shard)))
            ok &= bool(np.array_equal(torch.cat(parts).numpy(), w))
            y_full = orc.matvec(qt, x, w, rows, cols)
            y_shard = orc.matvec(qt, x, shard, n, cols)
            ok &= bool(np.array_equal(y_shard.view(np.uint32), y_full[rank * n:(rank + 1) * n].view(np.uint32)))
            ys = [torch.empty(n) for _ in range(world)]
            dist.all_gather(ys, torch.from_numpy(y_shard.copy()))
            ok &= bool(np.array_equal(torch.cat(ys).numpy().view(np.uint32), y_full.view(np.uint32)))
        q.put((rank, ok))
    except Exception as exc:   # report instead of leaving the parent waiting
        q.put((rank, repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


def test_row_shards_reassemble_and_match_full_matvec(oracle):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True), (1, True)]


def test_shard_rows_rejects_ragged_split():
    sys.path.insert(0, ROOT)
    import pytest
    from alice_llm_b200.gpu import shard_rows
    from alice_llm_b200._lib import AliceError
    with pytest.raises(AliceError):
        shard_rows(np.zeros(10 * 4, np.uint8), 10, 0, 4)
