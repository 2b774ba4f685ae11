"""Weight-streaming rate of the matvec kernel of every format on large synthetic matrices.

    python -m alice_llm_b200.format_rates [NAME ...]

For each case several distinct copies of the matrix (together > 300 MB, far above the 126 MB L2) are cycled, so
every launch streams its weights from HBM; CUDA events on the launching stream bracket 60 launches that follow 10 warm-up
launches. Prints rows x cols, bytes per launch, microseconds per launch, GB/s and the fraction of the measured copy
bandwidth (MEASURED_PEAKS.json next to the repository root when present, else 6650 GB/s)."""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

from . import synth
from .gpu import GpuEngine, GpuQuantType
from .synth_device import _ggml_tensor, _ternary_tensor

CASES = [("Q4_K", synth.Q4_K, 32768, 4096), ("Q5_K", synth.Q5_K, 32768, 4096), ("Q6_K", synth.Q6_K, 32768, 4096),
         ("Q8_0", synth.Q8_0, 32768, 4096), ("Q1_0", synth.Q1_0, 102400, 5120), ("Q2_0", synth.Q2_0, 51200, 5120),
         ("Q1_0_gate", synth.Q1_0, 25600, 5120), ("Q1_0_down", synth.Q1_0, 5120, 25600),
         ("TERNARY", synth.TERNARY, 28672, 8192), ("TERNARY_down", synth.TERNARY, 8192, 28672),
         ("SPARSE_TERNARY", "sparse", 28672, 8192)]


def peak_gbs():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0


def main(argv):
    only = set(argv)
    eng = GpuEngine(0)
    dev = torch.device("cuda", 0)
    st = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(st)
    eng.set_stream(st.cuda_stream)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    peak = peak_gbs()
    for name, qt, rows, cols in CASES:
        if only and name not in only:
            continue
        if qt == "sparse":
            per = rows * ((cols + 15) // 16 * 4)
        else:
            per = rows * ((cols + 31) // 32 * 8) if qt == synth.TERNARY else rows * synth.row_bytes(qt, cols)
        ncopy = max(2, int(300e6 // per) + 1)
        keep, ws = [], []
        for _ in range(ncopy):
            if qt == "sparse":
                # packed 2-bit codes 00 / 01 / 11 with P(0) = 0.5, P(+1) = P(-1) = 0.25; uploaded through the host API
                r1 = torch.randint(0, 256, (per,), dtype=torch.uint8, device=dev, generator=gen) & 0x55
                r2 = torch.randint(0, 256, (per,), dtype=torch.uint8, device=dev, generator=gen) & r1
                sc = (torch.randn(rows, device=dev, generator=gen).abs() * 0.01).float()
                ws.append(eng.upload_sparse_ternary((r1 | (r2 << 1)).cpu().numpy(), sc.cpu().numpy(), rows, cols))
            elif qt == synth.TERNARY:
                planes, scales = _ternary_tensor(gen, dev, rows, cols)
                keep += [planes, scales]
                ws.append(eng.ternary_from_device(planes.data_ptr(), scales.data_ptr(), rows, cols))
            else:
                t = _ggml_tensor(gen, dev, qt, rows, cols)
                keep.append(t)
                ws.append(eng.weights_from_device(t.data_ptr(), t.numel(), rows, cols, GpuQuantType(qt)))
        x = eng.upload_f32(np.random.default_rng(0).standard_normal(cols).astype(np.float32))
        y = eng.alloc_f32(rows)
        for i in range(10):
            eng.matvec_dev(ws[i % ncopy], x, y, 1)
        n = 60
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(st)
        for i in range(n):
            eng.matvec_dev(ws[i % ncopy], x, y, 1)
        e1.record(st)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / n * 1e3
        print(f"{name:13s} {rows}x{cols}  copies {ncopy}  bytes/launch {per}  {us:7.1f} us  {per / us / 1e3:6.0f} GB/s  "
              f"{per / us / 1e3 / peak:.2f} of measured", flush=True)
        for w in ws:
            w.free()
        x.free()
        y.free()
        del ws, keep
        torch.cuda.empty_cache()
    eng.close()


if __name__ == "__main__":
    main(sys.argv[1:])
