"""Synthetic decode models generated directly in device memory (torch CUDA RNG), for timing runs.

The numpy generators of ``synth.py`` feed the parity tests, which need host copies of every tensor;
a timing run of a 5-17 GB model only needs bytes of the right layout and value ranges on the device, so the
tensors are drawn there and handed to the library as borrowed device pointers (no host round trip).
Scale fields get the distributions of the benchmark configurations so activations stay finite.
A rank of a tensor-parallel group builds only its own row shards."""
from __future__ import annotations

import numpy as np
import torch

from . import synth
from .gpu import GpuEngine, GpuModel, GpuModelConfig, GpuQuantType

# the three decode configurations of the benchmark definition
CONFIGS = {
    # Llama-3-8B shapes, Q4_K_M mix: q/k/v/o/gate/up Q4_K, down and head Q6_K, embedding Q8_0; context 2048
    "c3_8b_q4km": dict(num_layers=32, hidden_dim=4096, intermediate_dim=14336, num_heads=32, num_kv_heads=8, head_dim=128,
                       vocab_size=128256, rope_theta=500000.0, eps=1e-5, context=2048,
                       mix=dict(q=synth.Q4_K, k=synth.Q4_K, v=synth.Q4_K, o=synth.Q4_K, gate=synth.Q4_K, up=synth.Q4_K,
                                down=synth.Q6_K, output=synth.Q6_K)),
    # 27B-class dense model in Q1_0 binary weights, Q8_0 head; context 4096
    "c4_27b_q1_0": dict(num_layers=64, hidden_dim=5120, intermediate_dim=25600, num_heads=40, num_kv_heads=8, head_dim=128,
                        vocab_size=151936, rope_theta=1000000.0, eps=1e-6, context=4096,
                        mix=dict(q=synth.Q1_0, k=synth.Q1_0, v=synth.Q1_0, o=synth.Q1_0, gate=synth.Q1_0, up=synth.Q1_0,
                                 down=synth.Q1_0, output=synth.Q8_0)),
    # Llama-2-70B shapes in ternary bit planes; context 2048
    "c5_70b_ternary": dict(num_layers=80, hidden_dim=8192, intermediate_dim=28672, num_heads=64, num_kv_heads=8, head_dim=128,
                           vocab_size=32000, rope_theta=10000.0, eps=1e-5, context=2048,
                           mix={n: synth.TERNARY for n in ("q", "k", "v", "o", "gate", "up", "down", "output")}),
}

# byte offset of the f16 scale fields inside a block, and their sigma (|N(0,1)| * sigma)
_SCALES = {synth.Q4_K: ((0, 0.01), (2, 0.005)), synth.Q5_K: ((0, 0.01), (2, 0.005)), synth.Q6_K: ((208, 0.01),),
           synth.Q8_0: ((0, 0.01),), synth.Q1_0: ((0, 0.02),), synth.Q2_0: ((0, 0.02),)}


def _ggml_tensor(gen, dev, qtype, rows, cols):
    bb, be = synth.BLOCK_BYTES[qtype], synth.BLOCK_ELEMS[qtype]
    nblk = rows * (cols // be)
    t = torch.randint(0, 256, (nblk, bb), dtype=torch.uint8, device=dev, generator=gen)
    for off, sigma in _SCALES[qtype]:
        d = (torch.randn(nblk, device=dev, generator=gen).abs() * sigma).to(torch.float16)
        t[:, off:off + 2] = d.view(torch.uint8).reshape(nblk, 2)
    if qtype == synth.Q6_K:   # int8 sub-block scales uniform -32..31
        t[:, 192:208] = torch.randint(-32, 32, (nblk, 16), dtype=torch.int8, device=dev, generator=gen).view(torch.uint8)
    if qtype == synth.Q2_0:   # 2-bit slots over the three codes the encoder emits
        s = torch.randint(0, 3, (nblk, 32, 4), dtype=torch.uint8, device=dev, generator=gen)
        t[:, 2:] = s[..., 0] | (s[..., 1] << 2) | (s[..., 2] << 4) | (s[..., 3] << 6)
    return t.reshape(-1)


def _ternary_tensor(gen, dev, rows, cols):
    """Device layout of the library: row = [pos plane | neg plane]; P(+1) = P(-1) = 0.25, P(0) = 0.5."""
    pb = (cols + 31) // 32 * 4
    a = torch.randint(0, 256, (rows, pb), dtype=torch.uint8, device=dev, generator=gen)
    b = torch.randint(0, 256, (rows, pb), dtype=torch.uint8, device=dev, generator=gen)
    planes = torch.stack([a & b, ~a & b], dim=1).reshape(-1)     # disjoint, each bit set with probability 1/4
    scales = (torch.randn(rows, device=dev, generator=gen).abs() * 0.01).float()
    return planes, scales


def build_model(engine: GpuEngine, name: str, seed: int = 0, extra_positions: int = 160):
    """Builds configuration `name` on the engine's device (this rank's shards when the engine belongs to a
    tensor-parallel group). Returns (GpuModel, info) with info = config dict plus weight_bytes_per_token of the
    WHOLE model (all ranks) and the tensors that must stay alive."""
    c = CONFIGS[name]
    rank, world = engine.tp_info()
    dev = torch.device("cuda", engine.device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed * 1000 + rank)
    H, F, V = c["hidden_dim"], c["intermediate_dim"], c["vocab_size"]
    q_dim, kv_dim = c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"]
    shapes = {"q": (q_dim, H), "k": (kv_dim, H), "v": (kv_dim, H), "o": (H, q_dim), "gate": (F, H), "up": (F, H), "down": (H, F)}
    keep, total_bytes = [], 0

    def tensor(role, rows, cols):
        nonlocal total_bytes
        qt = c["mix"][role]
        lrows = rows // world
        if qt == synth.TERNARY:
            planes, scales = _ternary_tensor(gen, dev, lrows, cols)
            keep.extend([planes, scales])
            total_bytes += rows * ((cols + 7) // 8 * 2 + 4)
            return engine.ternary_from_device(planes.data_ptr(), scales.data_ptr(), lrows, cols)
        t = _ggml_tensor(gen, dev, qt, lrows, cols)
        keep.append(t)
        total_bytes += synth.row_bytes(qt, cols) * rows
        return engine.weights_from_device(t.data_ptr(), t.numel(), lrows, cols, GpuQuantType(qt))

    def norm():
        return (1.0 + 0.02 * np.random.default_rng(seed).standard_normal(H)).astype(np.float32)

    layers = [dict({r: tensor(r, *shapes[r]) for r in shapes}, attn_norm=norm(), ffn_norm=norm()) for _ in range(c["num_layers"])]
    shared = torch.Generator(device=dev)
    shared.manual_seed(seed)                                # the same table on every rank
    emb = _ggml_tensor(shared, dev, synth.Q8_0, V, H)       # whole table on every rank; a decode step reads one row
    keep.append(emb)
    model = {"layers": layers, "embedding": engine.weights_from_device(emb.data_ptr(), emb.numel(), V, H, GpuQuantType.Q8_0),
             "output_norm": norm(), "output": tensor("output", V, H)}
    cfg = GpuModelConfig(c["num_layers"], H, F, c["num_heads"], c["num_kv_heads"], c["head_dim"], c["rope_theta"], c["eps"],
                         c["context"] + extra_positions, V)
    gm = GpuModel.load(engine, model, cfg)
    gm._keep.append(keep)
    # KV cache prefilled with N(0,1) to the context length: one [context, kv_dim/world] block reused for every layer
    rng = np.random.default_rng(seed + 1)
    k = rng.standard_normal((c["context"], kv_dim // world), dtype=np.float32)
    v = rng.standard_normal((c["context"], kv_dim // world), dtype=np.float32)
    for l in range(c["num_layers"]):
        gm.kv_write(l, 0, k, v)
    gm.set_position(c["context"])
    info = dict(name=name, weight_bytes_per_token=total_bytes + (H // 32) * 34, context=c["context"],
                kv_bytes_per_token=2 * c["context"] * kv_dim * 4 * c["num_layers"])
    return gm, info
