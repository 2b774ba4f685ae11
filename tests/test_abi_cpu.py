"""CPU checks of the boundary: the C-ABI library builds for sm_100a, loads, exports every symbol
include/alice_cuda.h declares, and refuses to compute without a CUDA device (no CPU fallback)."""
import os
import re

import numpy as np
import pytest

from alice_llm_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "alice_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(alice_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    assert os.path.exists(path)
    lib = _lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in alice_cuda.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == declared


def test_block_geometry_matches_reference_table():
    lib = _lib.load()
    # GgmlType::block_bytes / elements_per_block, src/gguf.rs:126-176
    for t, bb, be in [(8, 34, 32), (12, 144, 256), (13, 176, 256), (14, 210, 256), (41, 18, 128), (42, 34, 128)]:
        assert lib.alice_type_block_bytes(t) == bb and lib.alice_type_block_elems(t) == be
    assert lib.alice_type_block_bytes(2) == 0  # Q4_0 is not on this path


def test_no_cpu_fallback_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from alice_llm_b200 import gguf, gpu
    with pytest.raises(gpu.AliceError) as ei:
        gpu.GpuEngine(0)
    assert "no CPU path" in str(ei.value)
    with pytest.raises(gpu.AliceError):
        gguf.quantized_matvec(np.zeros(256, np.float32), np.zeros(144, np.uint8), gguf.GgmlType.Q4_K, 1, 256)


def test_product_code_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "alice_llm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                src = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"
