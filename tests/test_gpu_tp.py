"""Row-sharded tensor-parallel decode on 2 GPUs (one process per GPU) against the CPU oracle's forward of the whole
model, once with NCCL all-gathers inside the library and once with the kernels pushing their rows into the peer's
memory. Skipped on a box with a single GPU."""
import json
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mix", ["kquant", "q1_0", "q8_0", "ternary"])
@pytest.mark.parametrize("world", [2])
def test_tp_decode_matches_oracle(world, mix):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), str(world), str(port), mix],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env) for r in range(world)]
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=120))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, (p, (so, se)) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{se[-3000:]}"
    res = json.loads(outs[0][0].strip().splitlines()[-1])
    for mode in ("nccl", "peer"):
        assert res[0][mode + "_max_rel_err"] <= 1e-3, (mode, res[0])
        for r in res:
            assert r[mode + "_tokens"] == res[0]["oracle_tokens"], (mode, r)
