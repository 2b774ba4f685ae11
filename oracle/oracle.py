"""ctypes front end of the CPU oracle (oracle/alice_oracle.cpp).

TEST INFRASTRUCTURE ONLY. The oracle is the checker for the CUDA path: tests,
the smoke check and the benchmark's CPU-baseline leg load it; nothing in the
product package does.  ``build()`` compiles the C++ restatement with the flags
its header states.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "alice_oracle.cpp")
_LIB = os.path.join(_HERE, "liboracle.so")
_BASE_SRC = os.path.join(_HERE, "cpu_baseline.cpp")
_BASE_LIB = os.path.join(_HERE, "libcpu_baseline.so")

_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_i16p = C.POINTER(C.c_int16)
_u16p = C.POINTER(C.c_uint16)
_f32p = C.POINTER(C.c_float)


def _stale(lib, src):
    return not os.path.exists(lib) or (os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(lib))


def _cpu_tag() -> str:
    """Identifies the instruction set of this host: the baseline is built with -march=native, so a
    library built on another machine must not be reused."""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return hashlib.sha1(line.encode()).hexdigest()
    except OSError:
        pass
    return "unknown"


def build(force: bool = False) -> None:
    """Compile the oracle (and the threaded CPU baseline when its source is present)."""
    if force or _stale(_LIB, _SRC):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fno-fast-math",
                               "-fPIC", "-shared", "-o", _LIB, _SRC])
    tag_file = _BASE_LIB + ".host"
    try:
        with open(tag_file) as f:
            same_host = f.read().strip() == _cpu_tag()
    except OSError:
        same_host = False
    if os.path.exists(_BASE_SRC) and (force or not same_host or _stale(_BASE_LIB, _BASE_SRC) or _stale(_BASE_LIB, _SRC)):   # it includes _SRC
        subprocess.check_call(["g++", "-O3", "-std=c++17", "-march=native", "-ffp-contract=off",
                               "-fno-fast-math", "-fPIC", "-shared", "-pthread", "-o", _BASE_LIB, _BASE_SRC])
        with open(tag_file, "w") as f:
            f.write(_cpu_tag())


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB)
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_kquant_block_dot.restype = C.c_float
        _lib.orc_kquant_block_dot.argtypes = [C.c_uint32, _u8p, C.c_float, _i8p, _i16p]
        _lib.orc_ternarize_row.restype = C.c_float
        _lib.orc_sparsify_row.restype = C.c_float
        _lib.orc_silu.restype = C.c_float
        _lib.orc_silu.argtypes = [C.c_float]
    return _lib


def _p(a, t):
    return a.ctypes.data_as(t)


def _u8(a):
    a = np.ascontiguousarray(a, dtype=np.uint8)
    return a


def f16_to_f32(h: int) -> float:
    return float(lib().orc_f16_to_f32(C.c_uint16(h)))


def block_bytes(t: int) -> int:
    return int(lib().orc_block_bytes(C.c_uint32(t)))


def elements_per_block(t: int) -> int:
    return int(lib().orc_elements_per_block(C.c_uint32(t)))


def get_scale_min_k4(j: int, scales) -> tuple[int, int]:
    s = _u8(scales)
    sc, m = C.c_uint8(), C.c_uint8()
    lib().orc_get_scale_min_k4(C.c_int(j), _p(s, _u8p), C.byref(sc), C.byref(m))
    return sc.value, m.value


def dequantize(qtype: int, data) -> np.ndarray:
    d = _u8(data)
    n = d.size // block_bytes(qtype) * elements_per_block(qtype)
    out = np.empty(n, dtype=np.float32)
    rc = lib().orc_dequantize(C.c_uint32(qtype), _p(d, _u8p), C.c_size_t(d.size), _p(out, _f32p))
    if rc:
        raise ValueError(f"oracle: unsupported type {qtype}")
    return out


def dequantize_weight_row(qtype: int, data, n_out: int) -> np.ndarray:
    d = _u8(data)
    out = np.empty(n_out, dtype=np.float32)
    lib().orc_dequantize_weight_row(C.c_uint32(qtype), _p(d, _u8p), _p(out, _f32p), C.c_size_t(n_out))
    return out


def quantize_row_q8_k(x):
    """-> (d[nb] f32, qs[nb,256] i8, bsums[nb,16] i16)"""
    x = np.ascontiguousarray(x, dtype=np.float32)
    nb = x.size // 256
    d = np.empty(nb, dtype=np.float32)
    qs = np.empty((nb, 256), dtype=np.int8)
    bs = np.empty((nb, 16), dtype=np.int16)
    lib().orc_quantize_row_q8_k(_p(x, _f32p), C.c_size_t(x.size), _p(d, _f32p), _p(qs, _i8p), _p(bs, _i16p))
    return d, qs, bs


def kquant_block_dot(qtype: int, block, d8: float, q8, bsums) -> np.float32:
    b = _u8(block)
    q8 = np.ascontiguousarray(q8, dtype=np.int8)
    bsums = np.ascontiguousarray(bsums, dtype=np.int16)
    return np.float32(lib().orc_kquant_block_dot(C.c_uint32(qtype), _p(b, _u8p), C.c_float(d8),
                                                 _p(q8, _i8p), _p(bsums, _i16p)))


def matvec(qtype: int, x, data, rows: int, cols: int) -> np.ndarray:
    """quantized_matvec (src/gguf.rs:4214)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    d = _u8(data)
    y = np.empty(rows, dtype=np.float32)
    rc = lib().orc_matvec(C.c_uint32(qtype), _p(x, _f32p), _p(d, _u8p), C.c_size_t(d.size),
                          C.c_size_t(rows), C.c_size_t(cols), _p(y, _f32p))
    if rc:
        raise ValueError(f"oracle: unsupported type {qtype}")
    return y


def matvec_preq(qtype: int, data, rows: int, cols: int, q8k) -> np.ndarray:
    """quantized_matvec_preq (src/gguf.rs:4574); q8k = (d, qs, bsums) from quantize_row_q8_k."""
    d8, qs, bs = q8k
    d = _u8(data)
    y = np.empty(rows, dtype=np.float32)
    rc = lib().orc_matvec_preq(C.c_uint32(qtype), _p(d, _u8p), C.c_size_t(d.size), C.c_size_t(rows),
                               C.c_size_t(cols), _p(d8, _f32p), _p(qs, _i8p), _p(bs, _i16p), _p(y, _f32p))
    if rc:
        raise ValueError(f"oracle: unsupported type {qtype}")
    return y


def swiglu(qtype: int, x, gate, up, rows: int, cols: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    g, u = _u8(gate), _u8(up)
    y = np.empty(rows, dtype=np.float32)
    rc = lib().orc_swiglu(C.c_uint32(qtype), _p(x, _f32p), _p(g, _u8p), _p(u, _u8p), C.c_size_t(g.size),
                          C.c_size_t(rows), C.c_size_t(cols), _p(y, _f32p))
    if rc:
        raise ValueError(f"oracle: unsupported type {qtype}")
    return y


def ternary_matvec(pos, neg, scales, rows: int, cols: int, x) -> np.ndarray:
    pos, neg = _u8(pos), _u8(neg)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(rows, dtype=np.float32)
    lib().orc_ternary_matvec(_p(pos, _u8p), _p(neg, _u8p), _p(scales, _f32p), C.c_size_t(rows),
                             C.c_size_t(cols), _p(x, _f32p), _p(y, _f32p))
    return y


def ternary_swiglu(gate, up, rows: int, cols: int, x) -> np.ndarray:
    gp, gn, gs = (_u8(gate[0]), _u8(gate[1]), np.ascontiguousarray(gate[2], dtype=np.float32))
    up_, un, us = (_u8(up[0]), _u8(up[1]), np.ascontiguousarray(up[2], dtype=np.float32))
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(rows, dtype=np.float32)
    lib().orc_ternary_swiglu(_p(gp, _u8p), _p(gn, _u8p), _p(gs, _f32p), _p(up_, _u8p), _p(un, _u8p),
                             _p(us, _f32p), C.c_size_t(rows), C.c_size_t(cols), _p(x, _f32p), _p(y, _f32p))
    return y


def sparse_ternary_matvec(active, sign, scales, rows: int, cols: int, x) -> np.ndarray:
    active = np.ascontiguousarray(active, dtype=np.uint16)
    sign = np.ascontiguousarray(sign, dtype=np.uint16)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(rows, dtype=np.float32)
    lib().orc_sparse_ternary_matvec(_p(active, _u16p), _p(sign, _u16p), _p(scales, _f32p), C.c_size_t(rows),
                                    C.c_size_t(cols), _p(x, _f32p), _p(y, _f32p))
    return y


def sparse_pack_2bit(active, sign, rows: int, cols: int) -> np.ndarray:
    active = np.ascontiguousarray(active, dtype=np.uint16)
    sign = np.ascontiguousarray(sign, dtype=np.uint16)
    bpr = (cols + 15) // 16
    out = np.empty(rows * bpr * 4, dtype=np.uint8)
    lib().orc_sparse_pack_2bit(_p(active, _u16p), _p(sign, _u16p), C.c_size_t(rows), C.c_size_t(cols),
                               _p(out, _u8p))
    return out


def ternarize_row(w, threshold_ratio: float):
    w = np.ascontiguousarray(w, dtype=np.float32)
    nbytes = (w.size + 7) // 8
    pos = np.zeros(nbytes, dtype=np.uint8)
    neg = np.zeros(nbytes, dtype=np.uint8)
    scale = lib().orc_ternarize_row(_p(w, _f32p), C.c_size_t(w.size), C.c_float(threshold_ratio),
                                    _p(pos, _u8p), _p(neg, _u8p))
    return pos, neg, np.float32(scale)


def sparsify_row(pos, neg, dense_scale: float, w, n_keep: int):
    w = np.ascontiguousarray(w, dtype=np.float32)
    pos, neg = _u8(pos), _u8(neg)
    nblk = (w.size + 15) // 16
    active = np.zeros(nblk, dtype=np.uint16)
    sign = np.zeros(nblk, dtype=np.uint16)
    scale = lib().orc_sparsify_row(_p(pos, _u8p), _p(neg, _u8p), C.c_float(dense_scale), _p(w, _f32p),
                                   C.c_size_t(w.size), C.c_size_t(n_keep), _p(active, _u16p), _p(sign, _u16p))
    return active, sign, np.float32(scale)


def silu(x: float) -> np.float32:
    return np.float32(lib().orc_silu(C.c_float(x)))


# ── threaded CPU baseline (oracle/cpu_baseline.cpp) ─────────────────────────
_base = None


def baseline():
    global _base
    if _base is None:
        build()
        _base = C.CDLL(_BASE_LIB)
    return _base


def hw_threads() -> int:
    return int(baseline().base_hw_threads())


def base_matvec(qtype: int, x, data, rows: int, cols: int, nthreads: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    d = _u8(data)
    y = np.empty(rows, dtype=np.float32)
    baseline().base_matvec(C.c_uint32(qtype), _p(x, _f32p), _p(d, _u8p), C.c_size_t(d.size), C.c_size_t(rows),
                           C.c_size_t(cols), _p(y, _f32p), C.c_int(nthreads))
    return y


def base_ffn(gu_type: int, gate, up, down_type: int, down, hidden: int, ffn: int, x, nthreads: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    g, u, dn = _u8(gate), _u8(up), _u8(down)
    y = np.empty(hidden, dtype=np.float32)
    baseline().base_ffn(C.c_uint32(gu_type), _p(g, _u8p), _p(u, _u8p), C.c_size_t(g.size), C.c_uint32(down_type),
                        _p(dn, _u8p), C.c_size_t(dn.size), C.c_size_t(hidden), C.c_size_t(ffn), _p(x, _f32p),
                        _p(y, _f32p), C.c_int(nthreads))
    return y


# ── Llama forward (orc_llama_forward / base_llama_forward) ──────────────────
class _OrcLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("q", "k", "v", "o", "gate", "up", "down")] + \
               [(n, C.c_uint32) for n in ("tq", "tk", "tv", "to", "tgate", "tup", "tdown")] + \
               [("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p)]


class _OrcModel(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("num_layers", "hidden", "ffn", "num_heads", "num_kv_heads", "head_dim",
                                          "vocab", "max_seq")] + \
               [("theta", C.c_float), ("eps", C.c_float), ("neox", C.c_uint32), ("layers", C.c_void_p),
                ("emb_q8_0", C.c_void_p), ("out_norm", C.c_void_p), ("out", C.c_void_p), ("tout", C.c_uint32),
                ("kcache", C.c_void_p), ("vcache", C.c_void_p)]


TERNARY = 1000   # model-tensor type id of the in-memory ternary bit planes (not a GGML id)


class LlamaOracle:
    """CPU forward of a synthetic model dict (alice_llm_b200.synth.make_llama): Llama branch of
    Llama3Model::forward_with_layer_hook (src/llama3.rs:13632-13687, 14167-14613)."""

    def __init__(self, model: dict, threads: int = 0):
        cfg = model["config"]
        self.cfg, self.model, self.threads = cfg, model, threads
        kv_dim = cfg["num_kv_heads"] * cfg["head_dim"]
        self.kcache = np.zeros((cfg["num_layers"], cfg["max_seq_len"], kv_dim), np.float32)
        self.vcache = np.zeros_like(self.kcache)
        self.pos = 0
        self._layers = (_OrcLayer * cfg["num_layers"])()
        self._keep = []
        for i, L in enumerate(model["layers"]):
            for n in ("q", "k", "v", "o", "gate", "up", "down"):
                t, data = self._blob(L[n])
                setattr(self._layers[i], n, data.ctypes.data)
                setattr(self._layers[i], "t" + n, t)
            self._layers[i].attn_norm = L["attn_norm"].ctypes.data
            self._layers[i].ffn_norm = L["ffn_norm"].ctypes.data
        m = _OrcModel()
        m.num_layers, m.hidden, m.ffn = cfg["num_layers"], cfg["hidden_dim"], cfg["intermediate_dim"]
        m.num_heads, m.num_kv_heads, m.head_dim = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
        m.vocab, m.max_seq = cfg["vocab_size"], cfg["max_seq_len"]
        m.theta, m.eps, m.neox = cfg["rope_theta"], cfg["eps"], int(cfg.get("neox_rope", 0))
        m.layers = C.addressof(self._layers)
        m.emb_q8_0 = model["embedding"][1].ctypes.data
        m.out_norm = model["output_norm"].ctypes.data
        m.tout, out = self._blob(model["output"])
        m.out = out.ctypes.data
        m.kcache, m.vcache = self.kcache.ctypes.data, self.vcache.ctypes.data
        self._m = m

    def _blob(self, entry):
        """(type, data) as the C side wants it; ternary (pos, neg, scales) -> one pos | neg | scales blob."""
        t, data = entry
        if t == TERNARY:
            pos, neg, scales = data
            data = np.concatenate([_u8(pos).reshape(-1), _u8(neg).reshape(-1),
                                   np.ascontiguousarray(scales, np.float32).view(np.uint8).reshape(-1)])
        self._keep.append(data)
        return t, data

    def forward(self, token: int) -> np.ndarray:
        logits = np.empty(self.cfg["vocab_size"], np.float32)
        if self.threads > 1:
            rc = baseline().base_llama_forward(C.byref(self._m), C.c_uint32(token), C.c_uint32(self.pos),
                                               _p(logits, _f32p), C.c_int(self.threads))
        else:
            rc = lib().orc_llama_forward(C.byref(self._m), C.c_uint32(token), C.c_uint32(self.pos), _p(logits, _f32p))
        if rc:
            raise ValueError(f"oracle forward failed: {rc}")
        self.pos += 1
        return logits


def rms_norm(x, w, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(x, _f32p), _p(w, _f32p), C.c_float(eps), _p(out, _f32p), C.c_size_t(x.size))
    return out
