#!/usr/bin/env python
"""Benchmark of the quantized-matvec decode path on B200.

Headline workload ("ffn_q4k_q6k_b1"): the mixed-quant SwiGLU FFN block at Llama-3-8B shapes, batch 1:
gate/up 14336x4096 Q4_K, down 4096x14336 Q6_K, x f32[4096] ~ N(0,1); out = down(silu(gate x) * (up x)).
One step = one pass of the block = the library's SwiGLU call followed by its matvec call = 4 kernels (Q8_K quantizer of x,
fused SwiGLU gate/up matvec, Q8_K quantizer of its output, down matvec; each is the programmatic dependent of the one
before, so the matvec CTAs are resident and streaming weights while the small quantizer runs) over 114,229,248 weight bytes. Weights are synthetic (seed 0, the
distributions of alice_llm_b200/synth.py); 8 distinct copies of the block (914 MB, far above the 126 MB L2) are cycled
so every step streams its weights from HBM. The result of the first step is compared with the CPU oracle before
anything is timed (`parity`).

  metric     weight_stream_gbs = algorithmic weight bytes per step / step time (whole job)
  e2e        same metric through the C ABI with host buffers: x copied from pinned host memory and y read back to the
             host inside every timed step
  roofline   the slower of the step's two matvec kernels (each with the small quantizer kernel in front of it, timed alone
             with CUDA events) against the measured HBM copy bandwidth
  cpu_baseline  the C++ restatement of the reference CPU path on the host cores (the reference is Rust; no toolchain here)
  formats    every weight format on a matrix of >= 64 MB (several copies cycled): GB/s and fraction of the measured peak
  configs    the other single-GPU configurations of the benchmark definition: the Q4_K 4096x4096 GEMV alone, the FFN block
             at batch 4 (weights streamed once for the four inputs), the 70B shapes in the packed 2-bit ternary form
  decode     greedy decode of the synthetic whole-model configurations (128 tokens after a prefilled context): the 8B
             Q4_K_M mix, the 27B Q1_0 model and the 70B ternary model on one GPU; with --gpus N > 1 the 27B and 70B
             models row-sharded over the N GPUs, both exchange mechanisms, with the same seeded weights at every N,
             plus a small seed-shared model checked against the CPU oracle on rank 0 (tp_parity).

`--impl reference` times the CPU path alone, with all host threads, on the same block.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, FFN = 4096, 14336
Q4_K, Q6_K = 12, 14
GU_BYTES = FFN * (HIDDEN // 256) * 144        # 33,030,144 per matrix
DOWN_BYTES = HIDDEN * (FFN // 256) * 210      # 48,168,960
STEP_BYTES = 2 * GU_BYTES + DOWN_BYTES        # 114,229,248
NCOPIES = 8
KERNELS_PER_STEP = 4   # Q8_K quantizer of x, fused SwiGLU matvec, Q8_K quantizer of its output, down matvec
CONFIG = {"workload": "ffn_q4k_q6k_b1", "hidden": HIDDEN, "ffn": FFN, "gate_up": "Q4_K", "down": "Q6_K", "batch": 1,
          "weight_bytes_per_step": STEP_BYTES}


def make_block(seed=0):
    from alice_llm_b200 import synth
    rng = np.random.default_rng(seed)
    gate = synth.make_q4k(rng, FFN, HIDDEN)
    up = synth.make_q4k(rng, FFN, HIDDEN)
    down = synth.make_q6k(rng, HIDDEN, FFN)
    x = synth.make_x(rng, HIDDEN)
    return gate, up, down, x


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


CPU_SAMPLE = ("full FFN-block passes; C++ restatement of the reference CPU path (scalar block kernels of src/gguf.rs, "
              "auto-vectorised with -O3 -march=native, rows split over a persistent thread pool standing in for rayon); "
              "the reference itself is Rust and cannot be built on the box")


def cpu_ffn_rate(block, threads, min_seconds, max_passes):
    """FFN passes on the host cores until min_seconds have elapsed -> (GB/s, passes, seconds)."""
    from oracle import oracle as orc
    gate, up, down, x = block
    orc.base_ffn(Q4_K, gate, up, Q6_K, down, HIDDEN, FFN, x, threads)  # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        orc.base_ffn(Q4_K, gate, up, Q6_K, down, HIDDEN, FFN, x, threads)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or n >= max_passes:
            return STEP_BYTES * n / dt / 1e9, n, dt


def run_reference(args, rank, world):
    """The reference arm: the CPU path alone on the host cores of the box (rank 0 only)."""
    if rank != 0:
        return
    from oracle import oracle as orc
    orc.build()
    threads = orc.hw_threads()
    block = make_block(0)
    gate, up, down, x = block
    for _ in range(args.warmup):
        orc.base_ffn(Q4_K, gate, up, Q6_K, down, HIDDEN, FFN, x, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.base_ffn(Q4_K, gate, up, Q6_K, down, HIDDEN, FFN, x, threads)
    dt = time.perf_counter() - t0
    value = STEP_BYTES * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": "weight_stream_gbs", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
        "config": dict(CONFIG),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": f"{args.steps} {CPU_SAMPLE}"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# synthetic tensors drawn on the device (timing runs of 5-17 GB models need bytes of the right layout and value ranges,
# not host copies); every tensor has its own seed, the same on every rank, and a rank keeps only its row shard
# ---------------------------------------------------------------------------------------------------------------------
DECODE_CONFIGS = {
    # Llama-3-8B shapes, Q4_K_M mix: q/k/v/o/gate/up Q4_K, down and head Q6_K, embedding Q8_0; context 2048
    "c3_8b_q4km": dict(num_layers=32, hidden_dim=4096, intermediate_dim=14336, num_heads=32, num_kv_heads=8, head_dim=128,
                       vocab_size=128256, rope_theta=500000.0, eps=1e-5, context=2048,
                       mix=dict(q=12, k=12, v=12, o=12, gate=12, up=12, down=14, output=14)),
    # 27B-class dense model in Q1_0 binary weights, Q8_0 head; context 4096
    "c4_27b_q1_0": dict(num_layers=64, hidden_dim=5120, intermediate_dim=25600, num_heads=40, num_kv_heads=8, head_dim=128,
                        vocab_size=151936, rope_theta=1000000.0, eps=1e-6, context=4096,
                        mix=dict(q=41, k=41, v=41, o=41, gate=41, up=41, down=41, output=8)),
    # Llama-2-70B shapes in ternary bit planes; context 2048
    "c5_70b_ternary": dict(num_layers=80, hidden_dim=8192, intermediate_dim=28672, num_heads=64, num_kv_heads=8, head_dim=128,
                           vocab_size=32000, rope_theta=10000.0, eps=1e-5, context=2048,
                           mix={n: 1000 for n in ("q", "k", "v", "o", "gate", "up", "down", "output")}),
}
# byte offset of the f16 scale fields inside a block, and their sigma (|N(0,1)| * sigma)
_SCALES = {12: ((0, 0.01), (2, 0.005)), 13: ((0, 0.01), (2, 0.005)), 14: ((208, 0.01),), 8: ((0, 0.01),), 41: ((0, 0.02),), 42: ((0, 0.02),)}


def dev_ggml_tensor(gen, dev, qtype, rows, cols):
    import torch
    from alice_llm_b200 import synth
    bb, be = synth.BLOCK_BYTES[qtype], synth.BLOCK_ELEMS[qtype]
    nblk = rows * (cols // be)
    t = torch.randint(0, 256, (nblk, bb), dtype=torch.uint8, device=dev, generator=gen)
    for off, sigma in _SCALES[qtype]:
        d = (torch.randn(nblk, device=dev, generator=gen).abs() * sigma).to(torch.float16)
        t[:, off:off + 2] = d.view(torch.uint8).reshape(nblk, 2)
    if qtype == 14:   # int8 sub-block scales uniform -32..31
        t[:, 192:208] = torch.randint(-32, 32, (nblk, 16), dtype=torch.int8, device=dev, generator=gen).view(torch.uint8)
    if qtype == 42:   # 2-bit slots over the three codes the encoder emits
        s = torch.randint(0, 3, (nblk, 32, 4), dtype=torch.uint8, device=dev, generator=gen)
        t[:, 2:] = s[..., 0] | (s[..., 1] << 2) | (s[..., 2] << 4) | (s[..., 3] << 6)
    return t.reshape(-1)


def dev_ternary_tensor(gen, dev, rows, cols):
    """Device layout of the library: row = [pos plane | neg plane]; P(+1) = P(-1) = 0.25, P(0) = 0.5."""
    import torch
    pb = (cols + 31) // 32 * 4
    a = torch.randint(0, 256, (rows, pb), dtype=torch.uint8, device=dev, generator=gen)
    b = torch.randint(0, 256, (rows, pb), dtype=torch.uint8, device=dev, generator=gen)
    planes = torch.stack([a & b, ~a & b], dim=1).reshape(rows, 2 * pb)   # disjoint, each bit set with probability 1/4
    scales = (torch.randn(rows, device=dev, generator=gen).abs() * 0.01).float()
    return planes, scales


def build_model(engine, name, seed=0, extra_positions=160, force_world=None):
    """Configuration `name` on the engine's device: this rank's row shards when the engine belongs to a tensor-parallel
    group. The WHOLE tensor is drawn from its own seed on every rank and the rank keeps its rows, so the model is the
    same at every group size. Returns (GpuModel, info)."""
    import torch
    from alice_llm_b200 import synth
    from alice_llm_b200.gpu import GpuModel, GpuModelConfig, GpuQuantType
    c = DECODE_CONFIGS[name]
    rank, world = engine.tp_info()
    dev = torch.device("cuda", engine.device)
    H, F, V = c["hidden_dim"], c["intermediate_dim"], c["vocab_size"]
    q_dim, kv_dim = c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"]
    shapes = {"q": (q_dim, H), "k": (kv_dim, H), "v": (kv_dim, H), "o": (H, q_dim), "gate": (F, H), "up": (F, H), "down": (H, F)}
    keep, total_bytes, counter = [], 0, [0]
    probe = {}      # layer 0's q projection (this rank's rows), kept for the parity check of the decode entry

    def tensor(role, rows, cols, shard=True):
        nonlocal total_bytes
        counter[0] += 1
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed * 100003 + counter[0])
        qt = c["mix"][role] if role != "embedding" else synth.Q8_0
        lo, n = (rank * (rows // world), rows // world) if shard else (0, rows)
        if qt == synth.TERNARY:
            planes, scales = dev_ternary_tensor(gen, dev, rows, cols)
            planes, scales = planes[lo:lo + n].contiguous().reshape(-1), scales[lo:lo + n].contiguous()
            keep.extend([planes, scales])
            total_bytes += rows * ((cols + 7) // 8 * 2 + 4)
            h = engine.ternary_from_device(planes.data_ptr(), scales.data_ptr(), n, cols)
            if role == "q" and not probe:
                probe.update(handle=h, qtype=qt, rows=n, cols=cols, planes=planes.reshape(n, -1), scales=scales)
            return h
        rb = synth.row_bytes(qt, cols)
        t = dev_ggml_tensor(gen, dev, qt, rows, cols)
        if n != rows:
            t = t[lo * rb:(lo + n) * rb].clone()
        keep.append(t)
        if role != "embedding":
            total_bytes += rb * rows
        h = engine.weights_from_device(t.data_ptr(), t.numel(), n, cols, GpuQuantType(qt))
        if role == "q" and not probe:
            probe.update(handle=h, qtype=qt, rows=n, cols=cols, blocks=t)
        return h

    def norm():
        return (1.0 + 0.02 * np.random.default_rng(seed).standard_normal(H)).astype(np.float32)

    layers = [dict({r: tensor(r, *shapes[r]) for r in shapes}, attn_norm=norm(), ffn_norm=norm()) for _ in range(c["num_layers"])]
    model = {"layers": layers, "embedding": tensor("embedding", V, H, shard=False), "output_norm": norm(), "output": tensor("output", V, H)}
    cfg = GpuModelConfig(c["num_layers"], H, F, c["num_heads"], c["num_kv_heads"], c["head_dim"], c["rope_theta"], c["eps"],
                         c["context"] + extra_positions, V)
    gm = GpuModel.load(engine, model, cfg)
    gm._keep.append(keep)
    # KV cache prefilled with N(0,1) to the context length: one [context, kv_dim] block reused for every layer
    rng = np.random.default_rng(seed + 1)
    k = rng.standard_normal((c["context"], kv_dim), dtype=np.float32)
    v = rng.standard_normal((c["context"], kv_dim), dtype=np.float32)
    lkv = kv_dim // world
    k, v = np.ascontiguousarray(k[:, rank * lkv:(rank + 1) * lkv]), np.ascontiguousarray(v[:, rank * lkv:(rank + 1) * lkv])
    for l in range(c["num_layers"]):
        gm.kv_write(l, 0, k, v)
    gm.set_position(c["context"])
    info = dict(name=name, weight_bytes_per_token=total_bytes + (H // 32) * 34, context=c["context"],
                kv_bytes_per_token=2 * c["context"] * kv_dim * 4 * c["num_layers"], probe=probe)
    return gm, info


def projection_check(eng, probe):
    """Layer 0's q projection of a device-drawn model (the rows this rank holds): the tensor is copied back to the host and
    the matvec of a seeded N(0,1) vector compared with the CPU oracle. Returns max |err| / max(|ref|, 1)."""
    from oracle import oracle as orc
    orc.build()
    rows, cols, qt = probe["rows"], probe["cols"], probe["qtype"]
    x = np.random.default_rng(99).standard_normal(cols).astype(np.float32)
    got = eng.matvec(probe["handle"], x).astype(np.float64)
    if "planes" in probe:
        planes = probe["planes"].cpu().numpy()
        pb, nb = planes.shape[1] // 2, (cols + 7) // 8
        ref = orc.ternary_matvec(np.ascontiguousarray(planes[:, :nb]), np.ascontiguousarray(planes[:, pb:pb + nb]),
                                 probe["scales"].cpu().numpy(), rows, cols, x)
    else:
        ref = orc.matvec(qt, x, probe["blocks"].cpu().numpy(), rows, cols)
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)).max())


def timed_decode(gm, ctx, tokens, stream, world, dist, dev):
    import torch
    gm.decode_greedy(1, 8)          # warm-up; also captures the step graph
    gm.set_position(ctx)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record(stream)
    toks = gm.decode_greedy(1, tokens)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, toks


def run_decode(eng, name, tokens, stream, world, dist, dev, peak, n1):
    """Greedy decode of one whole-model configuration; returns its report entry (device-timed, max over ranks).
    n1: {config: ms per token of the single-GPU model}, measured by the caller on rank 0's GPU when world > 1."""
    import torch
    gm, info = build_model(eng, name)
    ctx = info["context"]
    nccl_ms = None
    check = None
    if world == 1 or dist.get_rank() == 0:
        try:
            check = projection_check(eng, info["probe"])
        except Exception as exc:
            check = f"{type(exc).__name__}: {exc}"[:200]
    if world > 1:
        # first with NCCL all-gathers (the baseline), then with the kernels pushing their rows into the peers' memory
        nccl_ms, nccl_toks = timed_decode(gm, ctx, tokens, stream, world, dist, dev)
        handles = [None] * world
        dist.all_gather_object(handles, gm.tp_export())
        gm.tp_connect(handles)
        gm.set_position(ctx)
    ms, toks = timed_decode(gm, ctx, tokens, stream, world, dist, dev)
    verify = None
    if world == 1:
        # speculative verify: 8 consecutive tokens per step (GpuModel::forward_batch), logits of all of them kept on the device
        try:
            batch_tokens = [int(t) for t in toks[:8]]
            gm.set_position(ctx)
            gm.forward_batch(batch_tokens)          # warm-up
            eng.sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            nsteps = 8
            gm.set_position(ctx)
            e0.record(stream)
            for _ in range(nsteps):
                gm.forward_batch(batch_tokens)
            e1.record(stream)
            eng.sync()
            vms = e0.elapsed_time(e1) / nsteps
            verify = {"tokens_per_step": 8, "ms_per_step": vms, "ms_per_token": vms / 8, "tok_s": 8 / (vms * 1e-3)}
        except Exception as exc:
            verify = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    if world > 1:
        dist.barrier()              # no rank frees memory its peers may still be writing into
    gm.free()
    del gm
    torch.cuda.empty_cache()
    wb = info["weight_bytes_per_token"]
    bound_ms = wb / world / (peak * 1e9) * 1e3
    entry = {"config": name, "tokens": tokens, "context": ctx, "weight_bytes_per_token": wb,
             "kv_bytes_per_token_at_context": info["kv_bytes_per_token"], "stream_bound_ms_per_token": bound_ms,
             "first_tokens": [int(t) for t in toks[:8]],
             "layer0_q_projection_max_rel_err_vs_oracle": check, "verify_batch8": verify}
    if world == 1:
        entry["parallelism"] = "single GPU"
    else:
        entry["parallelism"] = f"tp{world}: rows of every projection sharded"
        entry["pushed_rows_ms_per_token"] = ms / tokens
        entry["nccl_all_gather_ms_per_token"] = nccl_ms / tokens
        entry["nccl_first_tokens"] = [int(t) for t in nccl_toks[:8]]
        entry["exchange"] = "rows pushed into the peers' vectors by the producing kernels (NVLink stores, one flag per vector)" \
            if ms <= nccl_ms else "NCCL all-gather issued by the library"
        ms = min(ms, nccl_ms)
        if n1 and name in n1:
            entry["ms_per_token_n1"] = n1[name]["ms_per_token"]
            entry["first_tokens_n1"] = n1[name]["first_tokens"]
            entry["tp_speedup"] = n1[name]["ms_per_token"] / (ms / tokens)
    entry.update({"tok_s": tokens / (ms * 1e-3), "ms_per_token": ms / tokens, "weight_gbs": wb * tokens / (ms * 1e-3) / 1e9,
                  "x_of_stream_bound": (ms / tokens) / bound_ms})
    return entry


def tp_parity(eng, world, rank, dist):
    """A small seed-shared model (same weights on every rank, shards cut from it), 8 greedy tokens in both exchange
    modes; rank 0 compares token ids and the last logits with the CPU oracle of the whole model."""
    from alice_llm_b200 import synth
    from alice_llm_b200.gpu import GpuModel
    cfg = dict(num_layers=2, hidden_dim=1024, intermediate_dim=2048, num_heads=16, num_kv_heads=8, head_dim=128,
               vocab_size=2048, max_seq_len=96, rope_theta=500000.0, eps=1e-5)
    rng = np.random.default_rng(11)
    model = synth.soften_attention(synth.make_llama(rng, cfg))
    kv_dim = cfg["num_kv_heads"] * cfg["head_dim"]
    npos = 33
    pre = [(rng.standard_normal((npos, kv_dim), dtype=np.float32), rng.standard_normal((npos, kv_dim), dtype=np.float32))
           for _ in range(cfg["num_layers"])]
    lkv = kv_dim // world
    out = {}
    ref_toks = ref_logits = None
    if rank == 0:
        from oracle import oracle as orc
        orc.build()
        o = orc.LlamaOracle(model, threads=orc.hw_threads())
        for l, (k, v) in enumerate(pre):
            o.kcache[l, :npos] = k
            o.vcache[l, :npos] = v
        o.pos = npos
        ref_toks, tok = [], 5
        for _ in range(8):
            ref_logits = o.forward(tok)
            tok = int(np.argmax(ref_logits))
            ref_toks.append(tok)
    for mode in ("nccl", "pushed_rows"):
        gm = GpuModel.load(eng, model)
        if mode == "pushed_rows":
            handles = [None] * world
            dist.all_gather_object(handles, gm.tp_export())
            gm.tp_connect(handles)
        for l, (k, v) in enumerate(pre):
            gm.kv_write(l, 0, np.ascontiguousarray(k[:, rank * lkv:(rank + 1) * lkv]), np.ascontiguousarray(v[:, rank * lkv:(rank + 1) * lkv]))
        gm.set_position(npos)
        toks = [int(t) for t in gm.decode_greedy(5, 8)]
        logits = gm.read_logits()
        if rank == 0:
            err = float((np.abs(logits.astype(np.float64) - ref_logits) / np.maximum(np.abs(ref_logits), 1.0)).max())
            out[mode] = {"tokens_match_oracle": toks == ref_toks, "last_logits_max_rel_err": err}
        dist.barrier()
        gm.free()
    return out


def extras(eng, dev, stream, peak, steps, block_handles, xd4, hd4, yd4, only, use_graph=True):
    """formats / configs keys (single GPU, rank 0): CUDA events around `n` launches that cycle distinct weight copies."""
    import torch
    from alice_llm_b200 import synth
    from alice_llm_b200.gpu import GpuQuantType
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)

    def timed(fn, n):
        """us per call; the calls are captured once into a CUDA graph and replayed, so that launch overhead of the host
        (several us per call from Python) does not hide the device time."""
        for i in range(5):
            fn(i)
        torch.cuda.synchronize()
        if not use_graph:        # plain launches (for a profiler): the figure then includes the host's launch overhead
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(n):
                fn(i)
            e1.record(stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n * 1e3
        chunk = 48
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
            for i in range(chunk):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        reps = max(1, n // chunk)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (reps * chunk) * 1e3

    n = max(20, min(steps, 100))
    out_formats, out_configs = {}, {}
    cases = [("Q4_K", 12, 32768, 4096), ("Q5_K", 13, 32768, 4096), ("Q6_K", 14, 32768, 4096), ("Q8_0", 8, 32768, 4096),
             ("Q1_0", 41, 102400, 5120), ("Q2_0", 42, 51200, 5120), ("ternary", 1000, 28672, 8192), ("sparse_ternary_packed_2bit", 1001, 28672, 8192)]
    for name, qt, rows, cols in cases:
        if only and name not in only:
            continue
        try:
            if qt == 1000:
                per = rows * ((cols + 31) // 32 * 8)
            elif qt == 1001:
                per = rows * ((cols + 15) // 16 * 4)
            else:
                per = rows * synth.row_bytes(qt, cols)
            ncopy = max(2, int(300e6 // per) + 1)
            keep, ws = [], []
            for _ in range(ncopy):
                if qt == 1000:
                    planes, sc = dev_ternary_tensor(gen, dev, rows, cols)
                    keep += [planes, sc]
                    ws.append(eng.ternary_from_device(planes.data_ptr(), sc.data_ptr(), rows, cols))
                elif qt == 1001:
                    # packed 2-bit codes 00 / 01 / 11 with P(0) = 0.5, P(+1) = P(-1) = 0.25; uploaded through the host API
                    a = torch.randint(0, 256, (per,), dtype=torch.uint8, device=dev, generator=gen) & 0x55
                    b = torch.randint(0, 256, (per,), dtype=torch.uint8, device=dev, generator=gen) & 0x55
                    packed = (a | ((a & b) << 1)).cpu().numpy()
                    sc = (np.abs(np.random.default_rng(3).standard_normal(rows)) * 0.01).astype(np.float32)
                    ws.append(eng.upload_sparse_ternary(packed, sc, rows, cols))
                else:
                    t = dev_ggml_tensor(gen, dev, qt, rows, cols)
                    keep.append(t)
                    ws.append(eng.weights_from_device(t.data_ptr(), t.numel(), rows, cols, GpuQuantType(qt)))
            x = eng.upload_f32(np.random.default_rng(1).standard_normal(cols).astype(np.float32))
            y = eng.alloc_f32(rows)
            us = timed(lambda i: eng.matvec_dev(ws[i % ncopy], x, y, 1), n)
            gbs = per / us / 1e3
            out_formats[name] = {"rows": rows, "cols": cols, "bytes_per_launch": per, "us_per_launch": us, "gbs": gbs, "frac_of_peak": gbs / peak}
            for w in ws:
                w.free()
            x.free(); y.free()
            del keep, ws
            torch.cuda.empty_cache()
        except Exception as exc:
            out_formats[name] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    # configuration 1 alone: Q4_K 4096 x 4096, 32 copies (302 MB) cycled
    try:
        per = 4096 * 16 * 144
        ts = [dev_ggml_tensor(gen, dev, 12, 4096, 4096) for _ in range(32)]
        ws = [eng.weights_from_device(t.data_ptr(), t.numel(), 4096, 4096, GpuQuantType.Q4K) for t in ts]
        x = eng.upload_f32(np.random.default_rng(0).standard_normal(4096).astype(np.float32))
        y = eng.alloc_f32(4096)
        us = timed(lambda i: eng.matvec_dev(ws[i % 32], x, y, 1), n)
        out_configs["c1_q4k_4096x4096_b1"] = {"bytes_per_launch": per, "us_per_launch": us, "gbs": per / us / 1e3, "frac_of_peak": per / us / 1e3 / peak}
        del ts, ws
    except Exception as exc:
        out_configs["c1_q4k_4096x4096_b1"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    # configuration 2 at batch 4: the weights stream once for the four inputs
    try:
        def step4(i):
            g, u, d = block_handles[i % NCOPIES]
            eng.swiglu_dev(g, u, xd4, hd4, 4)
            eng.matvec_dev(d, hd4, yd4, 4)
        us = timed(step4, n)
        g, u, d = block_handles[0]
        plan = [eng.batch_plan(g, 4, swiglu=True), eng.batch_plan(d, 4)]
        out_configs["c2_ffn_q4k_q6k_b4"] = {"weight_bytes_per_step": STEP_BYTES, "us_per_step": us, "gbs": STEP_BYTES / us / 1e3,
                                            "frac_of_peak": STEP_BYTES / us / 1e3 / peak, "tokens_per_step": 4,
                                            "launches_and_weight_passes": {"swiglu": plan[0], "down": plan[1]}}
    except Exception as exc:
        out_configs["c2_ffn_q4k_q6k_b4"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    return out_formats, out_configs


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from alice_llm_b200.gpu import GpuEngine, GpuQuantType

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    t_start = time.time()
    # stdout carries the one JSON line and nothing else: libraries that print there (NCCL's version banner) are sent to
    # stderr for the duration of the run
    sys.stdout.flush()
    line_fd = os.dup(1)
    os.dup2(2, 1)

    def log(msg):
        print(f"[bench rank {rank} +{time.time() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=240))

    block = make_block(0)
    gate, up, down, x = block
    eng = GpuEngine(local_rank)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    eng.set_stream(stream.cuda_stream)

    def dev_bytes(a):
        return torch.from_numpy(a).to(dev)

    base = [dev_bytes(gate), dev_bytes(up), dev_bytes(down)]
    copies, keep = [], []
    for c in range(NCOPIES):
        t = base if c == 0 else [b.clone() for b in base]
        keep.append(t)
        copies.append((eng.weights_from_device(t[0].data_ptr(), GU_BYTES, FFN, HIDDEN, GpuQuantType.Q4K),
                       eng.weights_from_device(t[1].data_ptr(), GU_BYTES, FFN, HIDDEN, GpuQuantType.Q4K),
                       eng.weights_from_device(t[2].data_ptr(), DOWN_BYTES, HIDDEN, FFN, GpuQuantType.Q6K)))
    xd = eng.upload_f32(x)
    hd = eng.alloc_f32(FFN)
    yd = eng.alloc_f32(HIDDEN)
    x4 = np.concatenate([x, np.random.default_rng(5).standard_normal(3 * HIDDEN).astype(np.float32)])
    xd4, hd4, yd4 = eng.upload_f32(x4), eng.alloc_f32(4 * FFN), eng.alloc_f32(4 * HIDDEN)
    x_pin = torch.from_numpy(x).pin_memory()
    y_pin = torch.empty(HIDDEN, dtype=torch.float32).pin_memory()

    def step(i):
        g, u, d = copies[i % NCOPIES]
        eng.swiglu_dev(g, u, xd, hd, 1)
        eng.matvec_dev(d, hd, yd, 1)

    def step_e2e(i):
        g, u, d = copies[i % NCOPIES]
        # x from pinned host memory, the block, y back to pinned host memory, one wait: y is read on the host every step
        eng.write_f32_async(xd, x_pin.data_ptr(), HIDDEN)
        eng.swiglu_dev(g, u, xd, hd, 1)
        eng.matvec_dev(d, hd, yd, 1)
        eng.read_f32_async(yd, y_pin.data_ptr(), HIDDEN)
        eng.sync()

    # parity of the timed code path, untimed: one step against the CPU oracle (rank 0)
    parity = None
    if rank == 0 and not args.no_cpu:
        from oracle import oracle as orc
        orc.build()
        step(0)
        got = eng.read_f32(yd).astype(np.float64)
        eng.sync()
        ref = orc.base_ffn(Q4_K, gate, up, Q6_K, down, HIDDEN, FFN, x, orc.hw_threads()).astype(np.float64)
        parity = {"ffn_block_rel_l2": float(np.linalg.norm(got - ref) / np.linalg.norm(ref)),
                  "ffn_block_max_abs_err_over_rms": float(np.abs(got - ref).max() / np.sqrt(np.mean(ref * ref))),
                  "tolerance": 1e-3,
                  "against": "CPU oracle (oracle/), same seeded inputs"}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    GRAPH_STEPS = 40    # a multiple of the number of weight copies

    def timed(fn, n, graph=True):
        """Milliseconds for exactly n calls of fn (max over ranks). graph: the calls are queued as replays of a CUDA
        graph holding GRAPH_STEPS consecutive calls (plus single calls for the remainder): four kernel launches per
        step from Python would otherwise bound the loop by the host, not the device."""
        g = None
        if graph and n >= GRAPH_STEPS:
            try:
                g = torch.cuda.CUDAGraph()
                # thread-local capture: the process group's watchdog thread may query events meanwhile
                with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                    for i in range(GRAPH_STEPS):
                        fn(i)
                g.replay()
            except Exception as exc:       # fall back to queueing every step from the host
                log(f"graph capture failed ({exc}); steps are queued one by one")
                g = None
                torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        done = 0
        while g is not None and n - done >= GRAPH_STEPS:
            g.replay()
            done += GRAPH_STEPS
        for i in range(done, n):
            fn(i)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    warm = max(args.warmup, 3)
    for i in range(warm):
        step(i)
        step_e2e(i)
    eng.sync()
    if parity is not None:    # the host-buffer step returns the same vector (all weight copies are equal)
        parity["e2e_equals_device_path"] = bool(np.array_equal(y_pin.numpy().view(np.uint32), eng.read_f32(yd).view(np.uint32))
                                                and np.array_equal(y_pin.numpy(), got.astype(np.float32)))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    use_graph = not args.no_graph
    ms = timed(step, args.steps, graph=use_graph)
    ms_e2e = timed(step_e2e, args.steps, graph=False)   # host buffers, a blocking read per step: not capturable
    # each half of the step alone (quantizer + matvec), over the weight copies
    ms_sw = timed(lambda i: eng.swiglu_dev(copies[i % NCOPIES][0], copies[i % NCOPIES][1], xd, hd, 1), args.steps, graph=use_graph)
    ms_down = timed(lambda i: eng.matvec_dev(copies[i % NCOPIES][2], hd, yd, 1), args.steps, graph=use_graph)
    clocks = sampler.stop() if rank == 0 else None
    eng.sync()

    peak, peak_src = measured_peak()
    log("FFN block timed")
    formats, configs = {}, {}
    if rank == 0 and not args.no_extras:
        formats, configs = extras(eng, dev, stream, peak, args.steps, copies, xd4, hd4, yd4,
                                  set(args.formats.split(",")) if args.formats else None, use_graph=not args.no_graph)
        log("format and configuration tables done")

    # ---- the line, complete except for the whole-model entries ------------------------------------------------------
    line = None
    if rank == 0:
        value = STEP_BYTES * world * args.steps / (ms * 1e-3) / 1e9
        e2e = STEP_BYTES * world * args.steps / (ms_e2e * 1e-3) / 1e9
        sw_gbs = 2 * GU_BYTES / (ms_sw / args.steps * 1e-3) / 1e9
        down_gbs = DOWN_BYTES / (ms_down / args.steps * 1e-3) / 1e9
        traffic = {}
        try:
            with open(os.path.join(ROOT, "profiles", "roofline_traffic.json")) as f:
                traffic = json.load(f)
        except Exception:
            pass
        kernels = {
            "swiglu_q4k": {"kernel": "quantize_q8k_kernel + stream_gemv_kernel<FmtQ4K, fused SwiGLU>", "achieved": sw_gbs, "frac": sw_gbs / peak,
                           "bytes_per_launch": 2 * GU_BYTES, "us_per_launch": ms_sw / args.steps * 1e3,
                           "traffic": traffic.get("swiglu_q4k_bytes_per_launch")},
            "down_q6k": {"kernel": "quantize_q8k_kernel + stream_gemv_kernel<FmtQ6K>", "achieved": down_gbs, "frac": down_gbs / peak,
                         "bytes_per_launch": DOWN_BYTES, "us_per_launch": ms_down / args.steps * 1e3,
                         "traffic": traffic.get("down_q6k_bytes_per_launch")},
        }
        slow = min(kernels.values(), key=lambda k: k["frac"])      # the roofline names the slower kernel of the step
        line = {
            "metric": "weight_stream_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
            "config": dict(CONFIG),
            "l2": f"{NCOPIES} distinct weight copies cycled ({NCOPIES * STEP_BYTES >> 20} MiB > 126 MB L2)",
            "parallelism": f"replicas x{world} (the FFN block does not shard; sharded work is under `decode`)" if world > 1 else "single",
            "roofline": {"bound": "hbm", "kernel": slow["kernel"], "achieved": slow["achieved"], "peak": peak, "unit": "GB/s",
                         "frac": slow["frac"], "peak_source": f"{peak_src} (of {peak_src})", "bytes_per_launch": slow["bytes_per_launch"],
                         "us_per_launch": slow["us_per_launch"], "traffic": slow["traffic"],
                         "frac_of_8000_nominal": slow["achieved"] / 8000.0, "whole_step_frac": value / world / peak,
                         "kernels": kernels},
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": HIDDEN * 4, "d2h_bytes_per_step": HIDDEN * 4,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": KERNELS_PER_STEP * args.steps,
            "launch": (f"steps queued as replays of a CUDA graph of {GRAPH_STEPS} steps" if use_graph else "one API call sequence per step from the host")
                      + "; e2e: one API call sequence per step from the host",
            "clocks": clocks,
            "parity": parity,
            "formats": formats,
            "configs": configs,
            "decode": [],
        }
        if world == 1 and not args.no_cpu:
            from oracle import oracle as orc
            orc.build()
            threads = orc.hw_threads()
            v, n, dt = cpu_ffn_rate(block, threads, args.cpu_seconds, 2000)
            line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": f"{n} {CPU_SAMPLE}; {dt:.1f} s"}
            log("CPU baseline timed")

    # ---- whole-model decode entries; a time limit guards the line: when it runs out, rank 0 prints what it has and
    # every rank leaves (a rank stuck in a collective would otherwise keep the launcher waiting) ------------------------
    decode, n1, tp_par = [], {}, None
    printed = threading.Lock()

    def finish(note=None):
        if not printed.acquire(blocking=False):
            return
        if rank == 0:
            line["decode"] = decode + ([{"error": note}] if note else [])
            if tp_par is not None:
                line["tp_parity"] = tp_par
            os.write(line_fd, (json.dumps(line) + "\n").encode())

    def out_of_time():
        log(f"whole-model section exceeded {args.decode_seconds:.0f} s: leaving")
        finish(f"time limit of {args.decode_seconds:.0f} s for the whole-model section reached")
        os._exit(0)

    if args.decode != "none":
        guard = threading.Timer(args.decode_seconds, out_of_time)
        guard.daemon = True
        guard.start()
        import faulthandler
        faulthandler.dump_traceback_later(max(1.0, args.decode_seconds - 3.0), file=sys.stderr)   # where it was stuck
        names = (["c3_8b_q4km", "c4_27b_q1_0", "c5_70b_ternary"] if world == 1 else ["c4_27b_q1_0", "c5_70b_ternary"]) \
            if args.decode == "auto" else args.decode.split(",")
        for t in keep:      # the FFN weight copies are no longer needed
            t.clear()
        del copies, base
        torch.cuda.empty_cache()
        if world > 1:
            # the single-GPU figure of every sharded model, on rank 0's GPU, before the group is formed
            if rank == 0:
                for name in names:
                    try:
                        gm1, info1 = build_model(eng, name)
                        ms1, toks1 = timed_decode(gm1, info1["context"], args.decode_tokens, stream, 1, None, dev)
                        n1[name] = {"ms_per_token": ms1 / args.decode_tokens, "first_tokens": [int(t) for t in toks1[:8]]}
                        gm1.free()
                        del gm1
                        torch.cuda.empty_cache()
                        log(f"{name} on one GPU: {ms1 / args.decode_tokens:.3f} ms per token")
                    except Exception as exc:
                        log(f"{name} on one GPU failed: {exc}")
            log("waiting for the other ranks")
            dist.barrier()
            ids = [eng.tp_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            eng.tp_init(rank, world, ids[0])
            log("tensor-parallel group formed")
            try:
                tp_par = tp_parity(eng, world, rank, dist)
            except Exception as exc:
                tp_par = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            log(f"tensor-parallel parity check done: {tp_par}")
        for name in names:
            try:
                decode.append(run_decode(eng, name, args.decode_tokens, stream, world, dist, dev, peak, n1))
                log(f"{name}: {decode[-1].get('ms_per_token')} ms per token")
            except Exception as exc:   # the line must still be printed; every wait in the library is bounded
                decode.append({"config": name, "error": f"{type(exc).__name__}: {exc}"[:300]})
                log(f"{name} failed: {exc}")
                break
        guard.cancel()
        faulthandler.cancel_dump_traceback_later()
    finish()
    if world > 1:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-format and per-configuration tables")
    ap.add_argument("--no-graph", action="store_true", help="queue every step from the host instead of replaying CUDA graphs (for profilers)")
    ap.add_argument("--formats", default="", help="comma list restricting the per-format table (default: all eight)")
    ap.add_argument("--decode", default="auto", help="auto | none | comma list of c3_8b_q4km,c4_27b_q1_0,c5_70b_ternary")
    ap.add_argument("--decode-tokens", type=int, default=128)
    ap.add_argument("--decode-seconds", type=float, default=300.0, help="time limit of the whole-model section")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.steps > 200:
            args.steps = 200  # ~20-60 ms per pass on the host cores: keep the arm within minutes
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
