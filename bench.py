#!/usr/bin/env python
"""Benchmark of the quantized-matvec decode path on B200.

Workload ("ffn_q4k_q6k_b1"): the mixed-quant SwiGLU FFN block at Llama-3-8B shapes, batch 1:
gate/up 14336x4096 Q4_K, down 4096x14336 Q6_K, x f32[4096] ~ N(0,1); out = down(silu(gate x) * (up x)).
One step = one pass of the block = 2 kernels (fused SwiGLU gate/up matvec, down matvec; each quantizes
its f32 input to Q8_K in its prologue, bit-exactly as the reference does) over 114,229,248 weight bytes.  Weights are synthetic (seed 0, the distributions of
alice_llm_b200/synth.py); 8 distinct copies of the block (914 MB, far above the 126 MB L2) are
cycled so every step streams its weights from HBM.

  metric  weight_stream_gbs = algorithmic weight bytes per step / step time (whole job)
  e2e     same metric through the C ABI with host buffers: x copied from pinned host memory and
          y read back to the host inside every timed step
  roofline  the fused SwiGLU Q4_K kernel alone (66,060,288 bytes per launch) against the measured
          HBM copy bandwidth of MEASURED_PEAKS.json
  cpu_baseline  the C++ restatement of the reference CPU path on the host cores (the reference
          itself is Rust and cannot be built here)

  decode  greedy decode of the synthetic whole-model configurations (128 tokens after a prefilled context):
          the 8B Q4_K_M mix, the 27B Q1_0 model and the 70B ternary model on one GPU; with --gpus N > 1 the
          27B and 70B models row-sharded over the N GPUs (one process per GPU, NCCL all-gather of every
          projection output inside the library). tok/s, ms/token and the ratio to the pure weight-streaming
          time at the measured HBM bandwidth. `--decode none` skips it.

`--impl reference` times that CPU path alone, with all host threads, on the same block.
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
KERNELS_PER_STEP = 2


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
        "config": {"workload": "ffn_q4k_q6k_b1", "hidden": HIDDEN, "ffn": FFN, "gate_up": "Q4_K", "down": "Q6_K",
                   "batch": 1, "weight_bytes_per_step": STEP_BYTES},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{args.steps} full FFN-block passes; C++ restatement of the reference CPU path "
                                   "(reference is Rust, no toolchain on the box)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_decode(eng, name, tokens, stream, world, dist, dev, peak):
    """Greedy decode of one whole-model configuration; returns its report entry (device-timed, max over ranks)."""
    import torch
    from alice_llm_b200.synth_device import build_model
    gm, info = build_model(eng, name)
    ctx = info["context"]
    def timed_decode():
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

    nccl_ms = None
    if world > 1:
        # first with NCCL all-gathers (the baseline), then with the kernels pushing their rows into the peers' memory
        nccl_ms, _ = timed_decode()
        handles = [None] * world
        dist.all_gather_object(handles, gm.tp_export())
        gm.tp_connect(handles)
        gm.set_position(ctx)
    ms, toks = timed_decode()
    if world > 1:
        dist.barrier()              # no rank frees memory its peers may still be writing into
    gm.free()
    del gm
    torch.cuda.empty_cache()
    wb = info["weight_bytes_per_token"]
    bound_ms = wb / world / (peak * 1e9) * 1e3
    entry = {"config": name, "tokens": tokens, "context": ctx, "weight_bytes_per_token": wb,
             "kv_bytes_per_token_at_context": info["kv_bytes_per_token"], "stream_bound_ms_per_token": bound_ms,
             "first_tokens": [int(t) for t in toks[:4]]}
    if world == 1:
        entry["parallelism"] = "single GPU"
    else:
        # both exchange mechanisms were timed; the entry's headline is the faster one, both are listed
        entry["parallelism"] = f"tp{world}: rows of every projection sharded"
        entry["pushed_rows_ms_per_token"] = ms / tokens
        entry["nccl_all_gather_ms_per_token"] = nccl_ms / tokens
        entry["exchange"] = "rows pushed into the peers' vectors by the producing kernels (NVLink stores, tagged elements)" \
            if ms <= nccl_ms else "NCCL all-gather issued by the library"
        ms = min(ms, nccl_ms)
    entry.update({"tok_s": tokens / (ms * 1e-3), "ms_per_token": ms / tokens, "weight_gbs": wb * tokens / (ms * 1e-3) / 1e9,
                  "x_of_stream_bound": (ms / tokens) / bound_ms})
    return entry


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from alice_llm_b200.gpu import GpuEngine, GpuQuantType

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

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
    x_pin = torch.from_numpy(x).pin_memory()
    y_pin = torch.empty(HIDDEN, dtype=torch.float32).pin_memory()
    import ctypes as C
    lib = eng._lib

    def step(i):
        g, u, d = copies[i % NCOPIES]
        eng.swiglu_dev(g, u, xd, hd, 1)
        eng.matvec_dev(d, hd, yd, 1)

    def step_e2e(i):
        g, u, d = copies[i % NCOPIES]
        lib.alice_buf_write_f32(eng._h, xd._h, C.c_void_p(x_pin.data_ptr()), HIDDEN)
        eng.swiglu_dev(g, u, xd, hd, 1)
        eng.matvec_dev(d, hd, yd, 1)
        lib.alice_buf_read_f32(eng._h, yd._h, C.c_void_p(y_pin.data_ptr()), HIDDEN)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for i in range(n):
            fn(i)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for i in range(max(args.warmup, 3)):
        step(i)
        step_e2e(i)
    eng.sync()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(step, args.steps)
    ms_e2e = timed(step_e2e, args.steps)
    # dominant kernel alone: the fused SwiGLU Q4_K matvec, one launch per weight copy
    ms_k = timed(lambda i: eng.swiglu_dev(copies[i % NCOPIES][0], copies[i % NCOPIES][1], xd, hd, 1), args.steps)
    ms_down = timed(lambda i: eng.matvec_dev(copies[i % NCOPIES][2], hd, yd, 1), args.steps)
    clocks = sampler.stop() if rank == 0 else None
    eng.sync()

    peak, peak_src = measured_peak()
    decode = []
    if args.decode != "none":
        names = (["c3_8b_q4km", "c4_27b_q1_0", "c5_70b_ternary"] if world == 1 else ["c4_27b_q1_0", "c5_70b_ternary"]) \
            if args.decode == "auto" else args.decode.split(",")
        for t in keep:      # the FFN weight copies are no longer needed
            t.clear()
        del copies, base
        torch.cuda.empty_cache()
        if world > 1:
            ids = [eng.tp_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            eng.tp_init(rank, world, ids[0])
        for name in names:
            try:
                decode.append(run_decode(eng, name, args.decode_tokens, stream, world, dist, dev, peak))
            except Exception as exc:   # the headline line must still be printed; every wait in the library is bounded
                decode.append({"config": name, "error": f"{type(exc).__name__}: {exc}"[:300]})
                break

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    value = STEP_BYTES * world * args.steps / (ms * 1e-3) / 1e9
    e2e = STEP_BYTES * world * args.steps / (ms_e2e * 1e-3) / 1e9
    k_gbs = 2 * GU_BYTES / (ms_k / args.steps * 1e-3) / 1e9
    traffic = None
    try:
        with open(os.path.join(ROOT, "profiles", "roofline_traffic.json")) as f:
            traffic = json.load(f).get("swiglu_q4k_bytes_per_launch")
    except Exception:
        pass
    line = {
        "metric": "weight_stream_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
        "config": {"workload": "ffn_q4k_q6k_b1", "hidden": HIDDEN, "ffn": FFN, "gate_up": "Q4_K", "down": "Q6_K",
                   "batch": 1, "weight_bytes_per_step": STEP_BYTES,
                   "l2": f"{NCOPIES} distinct weight copies cycled ({NCOPIES * STEP_BYTES >> 20} MiB > 126 MB L2)",
                   "parallelism": f"replicas x{world}" if world > 1 else "single"},
        "roofline": {"bound": "hbm", "kernel": "stream_gemv_kernel<FmtQ4K, swiglu>", "achieved": k_gbs, "peak": peak,
                     "unit": "GB/s", "frac": k_gbs / peak, "peak_source": f"{peak_src} (of {peak_src})",
                     "bytes_per_launch": 2 * GU_BYTES, "us_per_launch": ms_k / args.steps * 1e3, "traffic": traffic,
                     "frac_of_8000_nominal": k_gbs / 8000.0,
                     "down_q6k": {"achieved": DOWN_BYTES / (ms_down / args.steps * 1e-3) / 1e9,
                                  "us_per_launch": ms_down / args.steps * 1e3, "bytes_per_launch": DOWN_BYTES}},
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": HIDDEN * 4, "d2h_bytes_per_step": HIDDEN * 4,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": KERNELS_PER_STEP * args.steps,
        "clocks": clocks,
        "decode": decode,
    }
    if world == 1 and not args.no_cpu:
        from oracle import oracle as orc
        orc.build()
        threads = orc.hw_threads()
        v, n, dt = cpu_ffn_rate(block, threads, args.cpu_seconds, 2000)
        line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"{n} full FFN-block passes in {dt:.1f} s; C++ restatement of the "
                                          "reference CPU path, row-parallel threads"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--decode", default="auto", help="auto | none | comma list of c3_8b_q4km,c4_27b_q1_0,c5_70b_ternary")
    ap.add_argument("--decode-tokens", type=int, default=128)
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
