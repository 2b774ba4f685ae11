"""Host-side mirror of ALICE-LLM's device API (src/gpu.rs) over the CUDA C ABI.

Names, argument meaning and error behaviour follow the reference so that tests read like its
own: ``GpuEngine`` (src/gpu.rs:320, methods :434-964), ``GpuWeightBuffer`` (:302), ``GpuBuffer``
(:277), ``GpuPass`` (:418, :1016-2105).  Shape or format violations raise (the reference panics).
Nothing here computes on the CPU; every method is a call into libalice_cuda.so.
"""
from __future__ import annotations

import ctypes as C
import weakref
from enum import Enum

import numpy as np

from . import _lib
from ._lib import AliceError, check  # noqa: F401


class GpuQuantType(Enum):
    """src/gpu.rs:285 plus the two in-memory ternary packings of src/gguf.rs."""
    Q4K = 12
    Q5K = 13
    Q6K = 14
    Q8_0 = 8
    Q1_0 = 41
    Q2_0 = 42
    Ternary = 1000
    SparseTernary = 1001


def _np(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def _ptr(a):
    return C.c_void_p(a.ctypes.data)


class GpuBuffer:
    """f32 storage on the device (src/gpu.rs:277)."""

    def __init__(self, engine, handle, length):
        self.engine, self._h, self.len = engine, handle, length
        engine._children.add(self)

    def free(self):
        if self._h:
            _lib.load().alice_buf_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class GpuWeightBuffer:
    """Raw quantized blocks on the device (src/gpu.rs:302)."""

    def __init__(self, engine, handle, rows, cols, quant):
        self.engine, self._h, self.rows, self.cols, self.quant = engine, handle, rows, cols, quant
        engine._children.add(self)

    def free(self):
        if self._h:
            _lib.load().alice_weights_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Q8KBuffer:
    """Vec<BlockQ8K> on the device (src/gguf.rs:1306)."""

    def __init__(self, engine, handle, cols, batch):
        self.engine, self._h, self.cols, self.batch = engine, handle, cols, batch
        engine._children.add(self)

    def read(self):
        """-> (d[batch, nb], qs[batch, nb, 256], bsums[batch, nb, 16])"""
        nb = self.cols // 256
        d = np.empty((self.batch, nb), np.float32)
        qs = np.empty((self.batch, nb, 256), np.int8)
        bs = np.empty((self.batch, nb, 16), np.int16)
        check(_lib.load().alice_q8k_read(self.engine._h, self._h, _ptr(d), _ptr(qs), _ptr(bs)))
        return d, qs, bs

    def free(self):
        if self._h:
            _lib.load().alice_q8k_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class GpuEngine:
    """GpuEngine (src/gpu.rs:320). ``GpuEngine()`` = ``GpuEngine::new`` (:434)."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        self._children = weakref.WeakSet()
        h = C.c_void_p()
        check(self._lib.alice_engine_create(device, C.byref(h)))
        self._h = h
        self.device = device

    def close(self):
        """Frees every buffer still alive on this engine (their C handles point at it), then the engine."""
        if getattr(self, "_h", None):
            children = list(self._children)
            for child in [c for c in children if isinstance(c, GpuModel)] + [c for c in children if not isinstance(c, GpuModel)]:
                child.free()
            self._lib.alice_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- configuration (no reference counterpart) --
    def set_stream(self, cuda_stream: int):
        check(self._lib.alice_engine_set_stream(self._h, C.c_void_p(cuda_stream)))

    def set_pdl(self, enabled: bool):
        check(self._lib.alice_engine_set_pdl(self._h, int(enabled)))

    def set_tuning(self, rows_per_set: int = 0, stages: int = 0):
        check(self._lib.alice_engine_set_tuning(self._h, rows_per_set, stages))

    def set_wait_limit(self, sm_cycles: int = 0):
        """Cycle budget of every bounded wait inside the kernels (0 = about one second)."""
        check(self._lib.alice_engine_set_wait_limit(self._h, sm_cycles))

    def debug_expire_wait(self):
        """Queues a hand-over whose flag nobody raises: its bounded wait runs out (self-test of that path)."""
        check(self._lib.alice_debug_expire_wait(self._h))

    # -- tensor parallel: one engine (one process) per GPU, rows of every projection sharded over the group --
    TP_ID_BYTES = 128

    def tp_unique_id(self) -> bytes:
        """Group id made by rank 0; hand it to the other ranks (e.g. torch.distributed.broadcast_object_list)."""
        buf = C.create_string_buffer(self.TP_ID_BYTES)
        check(self._lib.alice_tp_unique_id(buf, self.TP_ID_BYTES))
        return bytes(buf.raw)

    def tp_init(self, rank: int, world: int, unique_id: bytes):
        """Joins the group (collective: every rank calls it with the same id)."""
        buf = C.create_string_buffer(bytes(unique_id), self.TP_ID_BYTES)
        check(self._lib.alice_engine_tp_init(self._h, rank, world, buf, self.TP_ID_BYTES))

    def tp_info(self):
        r, w = C.c_uint32(), C.c_uint32()
        check(self._lib.alice_engine_tp_info(self._h, C.byref(r), C.byref(w)))
        return r.value, w.value

    # -- weights: upload_weights* (src/gpu.rs:698-798) --
    def upload_weights_typed(self, data, rows: int, cols: int, quant: GpuQuantType) -> GpuWeightBuffer:
        d = _np(data, np.uint8)
        h = C.c_void_p()
        check(self._lib.alice_upload_weights(self._h, _ptr(d), d.size, quant.value, rows, cols, C.byref(h)))
        return GpuWeightBuffer(self, h, rows, cols, quant)

    def upload_weights(self, data, rows, cols):
        return self.upload_weights_typed(data, rows, cols, GpuQuantType.Q4K)

    def upload_weights_q5k(self, data, rows, cols):
        return self.upload_weights_typed(data, rows, cols, GpuQuantType.Q5K)

    def upload_weights_q6k(self, data, rows, cols):
        return self.upload_weights_typed(data, rows, cols, GpuQuantType.Q6K)

    def upload_weights_q8_0(self, data, rows, cols):
        return self.upload_weights_typed(data, rows, cols, GpuQuantType.Q8_0)

    def upload_weights_q1_0(self, data, rows, cols):
        return self.upload_weights_typed(data, rows, cols, GpuQuantType.Q1_0)

    def upload_weights_q2_0(self, data, rows, cols):
        return self.upload_weights_typed(data, rows, cols, GpuQuantType.Q2_0)

    def weights_from_device(self, device_ptr: int, nbytes: int, rows, cols, quant: GpuQuantType) -> GpuWeightBuffer:
        h = C.c_void_p()
        check(self._lib.alice_weights_from_device(self._h, C.c_void_p(device_ptr), nbytes, quant.value, rows, cols,
                                                  C.byref(h)))
        return GpuWeightBuffer(self, h, rows, cols, quant)

    def upload_ternary(self, pos, neg, scales, rows, cols) -> GpuWeightBuffer:
        """TernaryMatrix (src/gguf.rs:5198): bit planes [rows][ceil(cols/8)] + per-row scale."""
        p, n, s = _np(pos, np.uint8), _np(neg, np.uint8), _np(scales, np.float32)
        if p.size != rows * ((cols + 7) // 8) or n.size != p.size or s.size != rows:
            raise AliceError(_lib.E_SHAPE, "upload_ternary: plane or scale size does not match rows x cols")
        h = C.c_void_p()
        check(self._lib.alice_upload_ternary(self._h, _ptr(p), _ptr(n), _ptr(s), rows, cols, C.byref(h)))
        return GpuWeightBuffer(self, h, rows, cols, GpuQuantType.Ternary)

    def ternary_from_device(self, rows_ptr: int, scales_ptr: int, rows, cols) -> GpuWeightBuffer:
        """Borrowed device-resident ternary matrix: row = [pos plane | neg plane], planes of ceil(cols/32)*4 bytes."""
        h = C.c_void_p()
        check(self._lib.alice_ternary_from_device(self._h, C.c_void_p(rows_ptr), C.c_void_p(scales_ptr), rows, cols,
                                                  C.byref(h)))
        return GpuWeightBuffer(self, h, rows, cols, GpuQuantType.Ternary)

    def upload_sparse_ternary(self, packed_2bit, scales, rows, cols) -> GpuWeightBuffer:
        """SparseTernaryMatrix.packed_2bit (src/gguf.rs:5432) + per-row scale."""
        p, s = _np(packed_2bit, np.uint8), _np(scales, np.float32)
        if p.size < rows * ((cols + 15) // 16) * 4 or s.size != rows:
            raise AliceError(_lib.E_SHAPE, "upload_sparse_ternary: packed or scale size does not match rows x cols")
        h = C.c_void_p()
        check(self._lib.alice_upload_sparse_ternary(self._h, _ptr(p), _ptr(s), rows, cols, C.byref(h)))
        return GpuWeightBuffer(self, h, rows, cols, GpuQuantType.SparseTernary)

    def ternarize(self, w: GpuBuffer, rows: int, cols: int, threshold_ratio: float) -> GpuWeightBuffer:
        """TernaryRow::from_f32 of every row of the f32 matrix ``w`` (src/gguf.rs:5207-5245), on the device."""
        h = C.c_void_p()
        check(self._lib.alice_ternarize(self._h, w._h, rows, cols, threshold_ratio, C.byref(h)))
        return GpuWeightBuffer(self, h, rows, cols, GpuQuantType.Ternary)

    def sparsify(self, ternary: GpuWeightBuffer, w: GpuBuffer, n_keep: int) -> GpuWeightBuffer:
        """SparseTernaryRow::from_ternary_row of every row (src/gguf.rs:5451-5507), on the device."""
        h = C.c_void_p()
        check(self._lib.alice_sparsify(self._h, ternary._h, w._h, n_keep, C.byref(h)))
        return GpuWeightBuffer(self, h, ternary.rows, ternary.cols, GpuQuantType.SparseTernary)

    def download_weights(self, w: GpuWeightBuffer):
        """(device rows as uint8 [rows][row bytes], per-row scales or None) of a ternary / sparse-ternary matrix."""
        if w.quant is GpuQuantType.Ternary:
            rb = (w.cols + 31) // 32 * 8
        elif w.quant is GpuQuantType.SparseTernary:
            rb = (w.cols + 15) // 16 * 4
        else:
            raise AliceError(_lib.E_UNSUPPORTED, "download_weights: ternary forms only")
        rows = np.empty((w.rows, rb), np.uint8)
        scales = np.empty(w.rows, np.float32)
        check(self._lib.alice_weights_download(self._h, w._h, _ptr(rows), rows.size, _ptr(scales)))
        return rows, scales

    # -- f32 buffers (src/gpu.rs:667-695, 801-824) --
    def alloc_f32(self, length: int) -> GpuBuffer:
        h = C.c_void_p()
        check(self._lib.alice_buf_alloc_f32(self._h, length, C.byref(h)))
        return GpuBuffer(self, h, length)

    def upload_f32(self, data) -> GpuBuffer:
        d = _np(data, np.float32).reshape(-1)
        h = C.c_void_p()
        check(self._lib.alice_buf_upload_f32(self._h, _ptr(d), d.size, C.byref(h)))
        return GpuBuffer(self, h, d.size)

    def write_f32(self, buf: GpuBuffer, data):
        d = _np(data, np.float32).reshape(-1)
        check(self._lib.alice_buf_write_f32(self._h, buf._h, _ptr(d), d.size))

    def read_f32(self, buf: GpuBuffer, length: int | None = None) -> np.ndarray:
        n = buf.len if length is None else length
        out = np.empty(n, np.float32)
        check(self._lib.alice_buf_read_f32(self._h, buf._h, _ptr(out), n))
        return out

    def write_f32_async(self, buf: GpuBuffer, host_ptr: int, length: int):
        """Queues the copy of `length` floats at the (pinned) host address into `buf`; the memory must stay valid until the
        next sync(). GpuEngine::write_f32 (queue.write_buffer) does not block either."""
        check(self._lib.alice_buf_write_f32_async(self._h, buf._h, C.c_void_p(host_ptr), length))

    def read_f32_async(self, buf: GpuBuffer, host_ptr: int, length: int):
        """Queues the copy of `buf` to the (pinned) host address; the values are there after the next sync()."""
        check(self._lib.alice_buf_read_f32_async(self._h, buf._h, C.c_void_p(host_ptr), length))

    def buf_from_device(self, device_ptr: int, length: int) -> GpuBuffer:
        h = C.c_void_p()
        check(self._lib.alice_buf_from_device(self._h, C.c_void_p(device_ptr), length, C.byref(h)))
        return GpuBuffer(self, h, length)

    # -- Q8_K (src/gguf.rs:1323) --
    def alloc_q8k(self, cols: int, batch: int = 1) -> Q8KBuffer:
        h = C.c_void_p()
        check(self._lib.alice_q8k_alloc(self._h, cols, batch, C.byref(h)))
        return Q8KBuffer(self, h, cols, batch)

    def quantize_q8k(self, x: GpuBuffer, q: Q8KBuffer):
        check(self._lib.alice_quantize_q8k(self._h, x._h, q._h))

    def upload_q8k(self, d, qs, bsums, cols: int, batch: int = 1) -> Q8KBuffer:
        d, qs, bs = _np(d, np.float32), _np(qs, np.int8), _np(bsums, np.int16)
        nb = cols // 256
        if d.size != batch * nb or qs.size != batch * nb * 256 or bs.size != batch * nb * 16:
            raise AliceError(_lib.E_SHAPE, "upload_q8k: array sizes do not match cols x batch")
        h = C.c_void_p()
        check(self._lib.alice_q8k_upload(self._h, _ptr(d), _ptr(qs), _ptr(bs), cols, batch, C.byref(h)))
        return Q8KBuffer(self, h, cols, batch)

    # -- device-side ops --
    def matvec_dev(self, w: GpuWeightBuffer, x: GpuBuffer, y: GpuBuffer, batch: int = 1):
        check(self._lib.alice_matvec(self._h, w._h, x._h, y._h, batch))

    def matvec_preq_dev(self, w: GpuWeightBuffer, q: Q8KBuffer, y: GpuBuffer):
        check(self._lib.alice_matvec_preq(self._h, w._h, q._h, y._h))

    def matvec_preq_noalloc_dev(self, w: GpuWeightBuffer, q: Q8KBuffer, y: GpuBuffer):
        """alice_matvec_preq_noalloc: the Q1_0 / Q2_0 pre-quantized matvec for callers that cannot
        allocate device memory; its f32 scratch is a fixed 65536-float array inside the library."""
        check(self._lib.alice_matvec_preq_noalloc(self._h, w._h, q._h, y._h))

    def swiglu_dev(self, gate: GpuWeightBuffer, up: GpuWeightBuffer, x: GpuBuffer, y: GpuBuffer, batch: int = 1):
        check(self._lib.alice_swiglu(self._h, gate._h, up._h, x._h, y._h, batch))

    def swiglu_preq_dev(self, gate, up, q: Q8KBuffer, y: GpuBuffer):
        check(self._lib.alice_swiglu_preq(self._h, gate._h, up._h, q._h, y._h))

    def dequantize_dev(self, w: GpuWeightBuffer, out: GpuBuffer):
        check(self._lib.alice_dequantize(self._h, w._h, out._h))

    def plan_query(self, w: GpuWeightBuffer, swiglu: bool = False, preq: bool = False) -> dict:
        """Launch geometry the planner picks for a matvec over `w` (diagnostic; no reference counterpart)."""
        out = (C.c_uint32 * 10)()
        check(self._lib.alice_plan_query(self._h, w._h, int(swiglu), int(preq), out, 10))
        keys = ("grid", "warps_per_row", "row_sets", "rows_per_set", "groups", "stages", "units_per_lane", "mma", "col_chunks",
                "ctas_per_sm")
        return dict(zip(keys, (int(v) for v in out)))

    def batch_plan(self, w: GpuWeightBuffer, batch: int, swiglu: bool = False):
        """-> (kernel launches, passes over the weight bytes) of a batch of `batch` vectors (diagnostic)."""
        a, b = C.c_uint32(), C.c_uint32()
        check(self._lib.alice_batch_plan(self._h, w._h, int(swiglu), batch, C.byref(a), C.byref(b)))
        return a.value, b.value

    # -- one-shot helpers (src/gpu.rs:838, 962) --
    def matvec(self, weights: GpuWeightBuffer, input_) -> np.ndarray:
        """GpuEngine::matvec (src/gpu.rs:838): upload input, run, read back."""
        x = self.upload_f32(input_)
        y = self.alloc_f32(weights.rows)
        self.matvec_dev(weights, x, y, 1)
        out = self.read_f32(y)
        self.sync()
        return out

    # -- pre-bound matvec helpers of the reference's benchmarks (src/gpu.rs:311-318, 848-964) --
    def create_matvec_context(self, weights: GpuWeightBuffer) -> "MatvecContext":
        """GpuEngine::create_matvec_context: input and output buffers bound to one weight matrix, made once."""
        return MatvecContext(self, weights, self.alloc_f32(weights.cols), self.alloc_f32(weights.rows))

    def matvec_fast(self, ctx: "MatvecContext", input_) -> np.ndarray:
        """GpuEngine::matvec_fast: write the input, one dispatch, read the result back."""
        self.dispatch_matvec_only(ctx, input_)
        return self.read_f32(ctx.output)

    def dispatch_matvec_only(self, ctx: "MatvecContext", input_):
        """GpuEngine::dispatch_matvec_only: write the input and queue one dispatch; no read-back, no wait."""
        self.write_f32(ctx.input, input_)
        self.matvec_dev(ctx.weights, ctx.input, ctx.output, 1)

    def bench_dispatch_batch(self, ctx: "MatvecContext", input_, n: int):
        """GpuEngine::bench_dispatch_batch: the input once, then n dispatches queued back to back (the reference encodes
        them into one command buffer and polls once); returns after the last has completed."""
        self.write_f32(ctx.input, input_)
        for _ in range(n):
            self.matvec_dev(ctx.weights, ctx.input, ctx.output, 1)
        self.sync()

    def dequantize(self, weights: GpuWeightBuffer) -> np.ndarray:
        out = self.alloc_f32(weights.rows * weights.cols)
        self.dequantize_dev(weights, out)
        r = self.read_f32(out)
        self.sync()
        return r

    def begin_pass(self) -> "GpuPass":
        return GpuPass(self)

    def sync(self):
        check(self._lib.alice_sync(self._h))


class MatvecContext:
    """MatvecContext (src/gpu.rs:311): one weight matrix with its input and output buffers."""

    def __init__(self, engine: "GpuEngine", weights: GpuWeightBuffer, input_: GpuBuffer, output: GpuBuffer):
        self.engine, self.weights, self.input, self.output, self.rows = engine, weights, input_, output, weights.rows


class GpuPass:
    """GpuPass (src/gpu.rs:418): ops are queued in order and run by ``execute``. On CUDA the
    engine's stream is already an in-order queue, so encoding an op launches it and ``execute``
    is the blocking wait (src/gpu.rs:2087)."""

    def __init__(self, engine: GpuEngine):
        self.engine = engine

    def _mv(self, weights, input_, output, quant, batch=1):
        if quant is not None and weights.quant != quant:
            raise AliceError(_lib.E_INVALID, f"weights are {weights.quant.name}, op wants {quant.name}")
        self.engine.matvec_dev(weights, input_, output, batch)

    def matvec_q4k(self, weights, input_, output):
        self._mv(weights, input_, output, GpuQuantType.Q4K)

    def matvec_q5k(self, weights, input_, output):
        self._mv(weights, input_, output, GpuQuantType.Q5K)

    def matvec_q6k(self, weights, input_, output):
        self._mv(weights, input_, output, GpuQuantType.Q6K)

    def matvec_q8_0(self, weights, input_, output):
        self._mv(weights, input_, output, GpuQuantType.Q8_0)

    def matvec_q1_0(self, weights, input_, output):
        self._mv(weights, input_, output, GpuQuantType.Q1_0)

    # the row4 / row8 shader variants differ only in tiling (src/gpu.rs:1161-1344); one kernel serves all
    matvec_q1_0_row4 = matvec_q1_0

    def matvec_q1_0_batch4(self, weights, input_, output):
        self._mv(weights, input_, output, GpuQuantType.Q1_0, 4)

    matvec_q1_0_row4_batch4 = matvec_q1_0_batch4
    matvec_q1_0_row8_batch4 = matvec_q1_0_batch4

    def matvec_auto(self, weights, input_, output, batch: int = 1):
        """src/gpu.rs:1947: dispatch on the weight buffer's own type."""
        self._mv(weights, input_, output, None, batch)

    def swiglu(self, gate, up, input_, output, batch: int = 1):
        self.engine.swiglu_dev(gate, up, input_, output, batch)

    def execute(self):
        self.engine.sync()

    def execute_and_read(self, buf: GpuBuffer) -> np.ndarray:
        out = self.engine.read_f32(buf)
        self.engine.sync()
        return out


class GpuModelConfig:
    """GpuModelConfig (src/gpu.rs:2111-2151), the fields the Llama-style layer stack uses."""

    def __init__(self, num_layers, hidden_dim, intermediate_dim, num_heads, num_kv_heads, head_dim, rope_theta, eps,
                 max_seq_len, vocab_size, neox_rope=False):
        self.num_layers, self.hidden_dim, self.intermediate_dim = num_layers, hidden_dim, intermediate_dim
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.rope_theta, self.eps, self.max_seq_len = rope_theta, eps, max_seq_len
        self.vocab_size, self.neox_rope = vocab_size, neox_rope

    @classmethod
    def from_dict(cls, d):
        return cls(d["num_layers"], d["hidden_dim"], d["intermediate_dim"], d["num_heads"], d["num_kv_heads"],
                   d["head_dim"], d["rope_theta"], d["eps"], d["max_seq_len"], d["vocab_size"], bool(d.get("neox_rope", 0)))


def shard_rows(data, rows: int, rank: int, world: int):
    """Rows [rank*rows/world, (rank+1)*rows/world) of a row-major tensor of raw blocks (or of any per-row
    array): a contiguous byte range, since a row is a whole number of blocks. Returns (shard, shard_rows)."""
    if rows % world:
        raise AliceError(_lib.E_SHAPE, f"shard_rows: {rows} rows do not divide over {world} ranks")
    a = np.ascontiguousarray(data).reshape(-1)
    if a.size % rows:
        raise AliceError(_lib.E_SHAPE, f"shard_rows: {a.size} elements are not {rows} equal rows")
    per = a.size // rows
    n = rows // world
    return a[rank * n * per:(rank + 1) * n * per], n


class GpuModel:
    """GpuModel (src/gpu.rs:2348): the pre-built decode graph of a Llama-style model on one device.

    ``GpuModel.load(engine, model, config)`` takes the raw quantized tensors (a dict as built by
    ``synth.make_llama``, standing in for the GgufFile of src/gpu.rs:2831) and uploads them verbatim.
    On an engine that belongs to a tensor-parallel group (``engine.tp_init``) it uploads this rank's row
    shard of every projection; a tensor entry may also be a ready ``GpuWeightBuffer`` (already the shard)."""

    def __init__(self, engine: GpuEngine, handle, config: GpuModelConfig, keep):
        self.engine, self._h, self._config, self._keep = engine, handle, config, keep
        engine._children.add(self)

    @classmethod
    def load(cls, engine: GpuEngine, model: dict, config: GpuModelConfig | None = None) -> "GpuModel":
        cfg = config or GpuModelConfig.from_dict(model["config"])
        q_dim, kv_dim = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
        H, F = cfg.hidden_dim, cfg.intermediate_dim
        shapes = {"q": (q_dim, H), "k": (kv_dim, H), "v": (kv_dim, H), "o": (H, q_dim), "gate": (F, H), "up": (F, H),
                  "down": (H, F)}
        keep = []

        rank, world = engine.tp_info()

        def up(entry, rows, cols, shard=True):
            if isinstance(entry, GpuWeightBuffer):
                keep.append(entry)
                return entry
            t, data = entry
            if GpuQuantType(t) is GpuQuantType.SparseTernary:   # (packed 2-bit codes, per-row scales), SparseTernaryMatrix
                packed, sc = data
                packed = _np(packed, np.uint8).reshape(rows, -1)
                if shard and world > 1:
                    (packed, n), (sc, _) = shard_rows(packed, rows, rank, world), shard_rows(sc, rows, rank, world)
                    rows = n
                w = engine.upload_sparse_ternary(packed, sc, rows, cols)
                keep.append(w)
                return w
            if GpuQuantType(t) is GpuQuantType.Ternary:   # (pos planes, neg planes, per-row scales)
                pos, neg, sc = data
                if shard and world > 1:
                    (pos, n), (neg, _), (sc, _) = (shard_rows(a, rows, rank, world) for a in (pos, neg, sc))
                    rows = n
                w = engine.upload_ternary(pos, neg, sc, rows, cols)
                keep.append(w)
                return w
            if shard and world > 1:
                data, rows = shard_rows(data, rows, rank, world)
            w = engine.upload_weights_typed(data, rows, cols, GpuQuantType(t))
            keep.append(w)
            return w

        layers = (_lib.LayerWeights * cfg.num_layers)()
        for i, L in enumerate(model["layers"]):
            for n, (r, c) in shapes.items():
                setattr(layers[i], n, up(L[n], r, c)._h)
            an, fn = _np(L["attn_norm"], np.float32), _np(L["ffn_norm"], np.float32)
            keep += [an, fn]
            layers[i].attn_norm, layers[i].ffn_norm = an.ctypes.data, fn.ctypes.data
        emb = up(model["embedding"], cfg.vocab_size, H, shard=False)
        out = up(model["output"], cfg.vocab_size, H)
        onorm = _np(model["output_norm"], np.float32)
        c = _lib.ModelConfig(cfg.num_layers, H, F, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.vocab_size,
                             cfg.max_seq_len, cfg.rope_theta, cfg.eps, int(cfg.neox_rope))
        h = C.c_void_p()
        check(engine._lib.alice_model_create(engine._h, C.byref(c), C.byref(layers), emb._h, _ptr(onorm), out._h,
                                             C.byref(h)))
        return cls(engine, h, cfg, keep)

    @classmethod
    def load_shared(cls, engine: GpuEngine, model: dict, config: GpuModelConfig | None = None) -> "GpuModel":
        """GpuModel::load_shared (src/gpu.rs:2837): a model on an engine other models already use (draft and target of
        speculative decoding share device, stream and scratch). Engines here are shared by reference, so this is
        ``load``; the models' steps run in the order they are queued on the engine's stream."""
        return cls.load(engine, model, config)

    @classmethod
    def load_gguf(cls, engine: GpuEngine, path, max_seq_len=None) -> "GpuModel":
        """GpuModel::load (src/gpu.rs:2831) from a GGUF file: the file is mapped, the raw blocks of every tensor of
        the name table go to the device as they are (this rank's row shards on a tensor-parallel engine)."""
        from .gguf_file import GgufFile
        gf = GgufFile.open(path)
        gm = cls.load(engine, gf.load_model(max_seq_len))
        gm._keep.append(gf)
        return gm

    def config(self) -> GpuModelConfig:
        return self._config

    def free(self):
        if self._h:
            self.engine._lib.alice_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    # -- src/gpu.rs:5010-5052 --
    def forward(self, token_id: int):
        check(self.engine._lib.alice_model_forward(self._h, token_id))

    def forward_and_read(self, token_id: int) -> np.ndarray:
        out = np.empty(self._config.vocab_size, np.float32)
        check(self.engine._lib.alice_model_forward_read(self._h, token_id, _ptr(out)))
        return out

    def read_logits(self) -> np.ndarray:
        out = np.empty(self._config.vocab_size, np.float32)
        check(self.engine._lib.alice_model_read_logits(self._h, _ptr(out)))
        return out

    TP_HANDLE_BYTES = 64

    def tp_export(self) -> bytes:
        """Handle to this rank's exchange region (CUDA IPC); gather the handles of all ranks, in rank order."""
        buf = C.create_string_buffer(self.TP_HANDLE_BYTES)
        check(self.engine._lib.alice_model_tp_export(self._h, buf, self.TP_HANDLE_BYTES))
        return bytes(buf.raw)

    def tp_connect(self, handles):
        """handles[r] = tp_export() of rank r. Switches the sharded vectors from NCCL all-gathers to rows pushed by
        the producing kernels into the peers' memory."""
        blob = b"".join(bytes(h).ljust(self.TP_HANDLE_BYTES, b"\0") for h in handles)
        buf = C.create_string_buffer(blob, len(blob))
        check(self.engine._lib.alice_model_tp_connect(self._h, buf, self.TP_HANDLE_BYTES))

    # -- src/gpu.rs:6020-6094 --
    def forward_batch(self, token_ids):
        t = _np(token_ids, np.uint32).reshape(-1)
        check(self.engine._lib.alice_model_forward_batch(self._h, _ptr(t), t.size))

    def forward_batch_and_read(self, token_ids) -> np.ndarray:
        """-> logits[k * vocab + v] of the len(token_ids) consecutive tokens (src/gpu.rs:6057)."""
        t = _np(token_ids, np.uint32).reshape(-1)
        out = np.empty(t.size * self._config.vocab_size, np.float32)
        check(self.engine._lib.alice_model_forward_batch_read(self._h, _ptr(t), t.size, _ptr(out)))
        return out

    def decode_greedy(self, first_token: int, n: int) -> np.ndarray:
        out = np.empty(n, np.uint32)
        check(self.engine._lib.alice_model_decode_greedy(self._h, first_token, n, _ptr(out)))
        return out

    # -- src/gpu.rs:5618-5662 --
    def position(self) -> int:
        p = C.c_uint32()
        check(self.engine._lib.alice_model_position(self._h, C.byref(p)))
        return p.value

    def vocab_size(self) -> int:
        return self._config.vocab_size

    def rollback_to(self, pos: int):
        check(self.engine._lib.alice_model_rollback_to(self._h, pos))

    def reset(self):
        check(self.engine._lib.alice_model_reset(self._h))

    # -- pre-filled context (no reference counterpart: the benchmark starts from a filled KV cache) --
    def _local_kv_dim(self) -> int:
        """Floats per cached position on this rank: the KV heads are sharded over a tensor-parallel group."""
        return self._config.num_kv_heads * self._config.head_dim // self.engine.tp_info()[1]

    def kv_write(self, layer: int, pos0: int, k, v):
        """k, v: [npos, kv_dim / world] rows of this rank's KV heads."""
        k, v = _np(k, np.float32), _np(v, np.float32)
        kv_dim = self._local_kv_dim()
        if k.size != v.size or k.size % kv_dim:
            raise AliceError(_lib.E_SHAPE, f"kv_write: {k.size} / {v.size} floats are not whole rows of {kv_dim}")
        check(self.engine._lib.alice_model_kv_write(self._h, layer, pos0, k.size // kv_dim, _ptr(k), _ptr(v)))

    def kv_read(self, layer: int, pos0: int, npos: int):
        kv_dim = self._local_kv_dim()
        k, v = np.empty((npos, kv_dim), np.float32), np.empty((npos, kv_dim), np.float32)
        check(self.engine._lib.alice_model_kv_read(self._h, layer, pos0, npos, _ptr(k), _ptr(v)))
        return k, v

    def set_position(self, pos: int):
        check(self.engine._lib.alice_model_set_position(self._h, pos))
