"""Builds libalice_cuda.so (the C-ABI library of include/alice_cuda.h) for sm_100a with nvcc.

The same command line is what a Rust `build.rs` of the reference crate would run; it needs no
GPU (nvcc cross-compiles). Output: alice_llm_b200/libalice_cuda.so, kept in-tree.
"""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libalice_cuda.so")
SOURCES = ["abi.cu", "gemv_launch.cu", "q8k.cu", "dequant.cu", "ternarize.cu", "glue.cu", "model.cu", "tp.cu"]
# never --use_fast_math: dequantization and the Q8_K quantizer must round like the reference
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fno-strict-aliasing"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "alice_cuda.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    def compile_one(src):
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        subprocess.check_call(cmd)
        return obj

    # the translation units are independent: compile them side by side
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    subprocess.check_call([_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart", "-ldl"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
