"""Host-slice entry points with the signatures of ALICE-LLM src/gguf.rs, executed on the GPU.

``quantized_matvec`` (src/gguf.rs:4214), ``quantized_matvec_preq`` (:4574), ``q4k_matvec`` /
``q5k_matvec`` / ``q6k_matvec`` / ``q8_0_matvec`` (:3600, :3502, :4077, :3811), their ``_preq``
forms (:3607, :3509, :4084), ``quantize_row_q8_k`` (:1323), ``ternary_matvec`` (:5303),
``sparse_ternary_matvec`` (:5808) and ``dequantize_weight_row`` (:6168).  Inputs are numpy arrays
standing in for the Rust slices; each call uploads, runs the CUDA kernels and reads back.  An
unsupported type raises, as the reference panics (src/gguf.rs:4243, :4606).
"""
from __future__ import annotations

from enum import IntEnum

import numpy as np

from .gpu import AliceError, GpuEngine, GpuQuantType

QK_K = 256


class GgmlType(IntEnum):
    """The subset of src/gguf.rs:57-98 on the decode path, with the GGML ids of :101-122."""
    Q8_0 = 8
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    Q1_0 = 41
    Q2_0 = 42

    def block_bytes(self) -> int:      # src/gguf.rs:126
        return {8: 34, 12: 144, 13: 176, 14: 210, 41: 18, 42: 34}[int(self)]

    def elements_per_block(self) -> int:  # src/gguf.rs:161
        return {8: 32, 12: 256, 13: 256, 14: 256, 41: 128, 42: 128}[int(self)]


class BlockQ8K:
    """Structure-of-arrays form of Vec<BlockQ8K> (src/gguf.rs:1306): d[nb], qs[nb,256], bsums[nb,16]."""

    def __init__(self, d, qs, bsums):
        self.d, self.qs, self.bsums = d, qs, bsums


class TernaryMatrix:
    """src/gguf.rs:5198 with the per-row Vecs flattened: pos/neg [rows, ceil(cols/8)], scales [rows]."""

    def __init__(self, pos_mask, neg_mask, scales, num_rows, num_cols):
        self.pos_mask, self.neg_mask, self.scales = pos_mask, neg_mask, scales
        self.num_rows, self.num_cols = num_rows, num_cols


class SparseTernaryMatrix:
    """src/gguf.rs:5425: packed_2bit [rows, ceil(cols/16)*4] and scales [rows]."""

    def __init__(self, packed_2bit, scales, num_rows, num_cols):
        self.packed_2bit, self.scales, self.num_rows, self.num_cols = packed_2bit, scales, num_rows, num_cols


_engine = None


def engine() -> GpuEngine:
    """Process-wide engine on device 0 used by the host-slice calls."""
    global _engine
    if _engine is None:
        _engine = GpuEngine(0)
    return _engine


def _quant(qtype) -> GpuQuantType:
    try:
        return GpuQuantType(int(qtype))
    except ValueError:
        raise AliceError(-2, f"unsupported quantization type: {qtype!r}") from None


def quantized_matvec(input_, data, qtype, rows: int, cols: int, output=None) -> np.ndarray:
    e = engine()
    w = e.upload_weights_typed(data, rows, cols, _quant(qtype))
    x = np.ascontiguousarray(input_, np.float32)
    if x.size < cols:
        raise AliceError(-3, f"input length {x.size} < cols {cols}")
    y = e.matvec(w, x[:cols])
    w.free()
    if output is not None:
        output[:rows] = y
        return output
    return y


def q4k_matvec(input_, data, rows, cols, output=None):
    return quantized_matvec(input_, data, GgmlType.Q4_K, rows, cols, output)


def q5k_matvec(input_, data, rows, cols, output=None):
    return quantized_matvec(input_, data, GgmlType.Q5_K, rows, cols, output)


def q6k_matvec(input_, data, rows, cols, output=None):
    return quantized_matvec(input_, data, GgmlType.Q6_K, rows, cols, output)


def q8_0_matvec(input_, data, rows, cols, output=None):
    return quantized_matvec(input_, data, GgmlType.Q8_0, rows, cols, output)


def quantize_row_q8_k(input_) -> BlockQ8K:
    e = engine()
    x = np.ascontiguousarray(input_, np.float32)
    n = x.size // QK_K * QK_K   # input.len() / QK_K whole blocks (src/gguf.rs:1324)
    if n == 0:
        return BlockQ8K(np.zeros(0, np.float32), np.zeros((0, 256), np.int8), np.zeros((0, 16), np.int16))
    bx = e.upload_f32(x[:n])
    q = e.alloc_q8k(n, 1)
    e.quantize_q8k(bx, q)
    d, qs, bs = q.read()
    e.sync()
    return BlockQ8K(d[0], qs[0], bs[0])


def quantized_matvec_preq(data, qtype, rows: int, cols: int, q8_blocks: BlockQ8K, output=None) -> np.ndarray:
    e = engine()
    w = e.upload_weights_typed(data, rows, cols, _quant(qtype))
    q = e.upload_q8k(q8_blocks.d, q8_blocks.qs, q8_blocks.bsums, cols, 1)
    y = e.alloc_f32(rows)
    e.matvec_preq_dev(w, q, y)
    out = e.read_f32(y)
    e.sync()
    if output is not None:
        output[:rows] = out
        return output
    return out


def q4k_matvec_preq(data, rows, cols, q8_blocks, output=None):
    return quantized_matvec_preq(data, GgmlType.Q4_K, rows, cols, q8_blocks, output)


def q5k_matvec_preq(data, rows, cols, q8_blocks, output=None):
    return quantized_matvec_preq(data, GgmlType.Q5_K, rows, cols, q8_blocks, output)


def q6k_matvec_preq(data, rows, cols, q8_blocks, output=None):
    return quantized_matvec_preq(data, GgmlType.Q6_K, rows, cols, q8_blocks, output)


def ternary_matvec(matrix: TernaryMatrix, input_, output=None) -> np.ndarray:
    e = engine()
    w = e.upload_ternary(matrix.pos_mask, matrix.neg_mask, matrix.scales, matrix.num_rows, matrix.num_cols)
    y = e.matvec(w, np.ascontiguousarray(input_, np.float32)[: matrix.num_cols])
    if output is not None:
        output[: matrix.num_rows] = y
        return output
    return y


def sparse_ternary_matvec(matrix: SparseTernaryMatrix, input_, output=None) -> np.ndarray:
    e = engine()
    w = e.upload_sparse_ternary(matrix.packed_2bit, matrix.scales, matrix.num_rows, matrix.num_cols)
    y = e.matvec(w, np.ascontiguousarray(input_, np.float32)[: matrix.num_cols])
    if output is not None:
        output[: matrix.num_rows] = y
        return output
    return y


def dequantize_weight_row(data, qtype, out_len: int) -> np.ndarray:
    """src/gguf.rs:6168. Types its dispatcher does not list (Q1_0, Q2_0) give zeros there; here
    they are dequantized (src/gguf.rs:1264-1300), which the model loader needs for Q1_0 weights."""
    e = engine()
    w = e.upload_weights_typed(data, 1, out_len, _quant(qtype))
    return e.dequantize(w)
