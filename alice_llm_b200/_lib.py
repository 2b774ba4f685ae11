"""ctypes binding of libalice_cuda.so (the C ABI declared in include/alice_cuda.h).

Loading never falls back to anything: if the shared library is missing it is built with nvcc,
and if that fails, or a call returns a non-zero status, an exception is raised (the reference
panics in the same places, src/gguf.rs:4243, src/gpu.rs:721-734)."""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

OK, E_INVALID, E_UNSUPPORTED, E_SHAPE, E_CUDA, E_KERNEL, E_NOMEM = 0, -1, -2, -3, -4, -5, -6

_vp = C.c_void_p
_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_i8p = C.POINTER(C.c_int8)
_i16p = C.POINTER(C.c_int16)
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol include/alice_cuda.h declares
SIGNATURES = {
    "alice_last_error": (C.c_char_p, []),
    "alice_type_block_bytes": (C.c_uint32, [C.c_uint32]),
    "alice_type_block_elems": (C.c_uint32, [C.c_uint32]),
    "alice_engine_create": (C.c_int32, [C.c_int32, _pp]),
    "alice_engine_destroy": (C.c_int32, [_vp]),
    "alice_engine_set_stream": (C.c_int32, [_vp, _vp]),
    "alice_sync": (C.c_int32, [_vp]),
    "alice_engine_set_pdl": (C.c_int32, [_vp, C.c_int32]),
    "alice_engine_set_tuning": (C.c_int32, [_vp, C.c_int32, C.c_int32]),
    "alice_engine_set_wait_limit": (C.c_int32, [_vp, C.c_uint64]),
    "alice_upload_weights": (C.c_int32, [_vp, _vp, C.c_size_t, C.c_uint32, C.c_uint32, C.c_uint32, _pp]),
    "alice_weights_from_device": (C.c_int32, [_vp, _vp, C.c_size_t, C.c_uint32, C.c_uint32, C.c_uint32, _pp]),
    "alice_upload_ternary": (C.c_int32, [_vp, _vp, _vp, _vp, C.c_uint32, C.c_uint32, _pp]),
    "alice_upload_sparse_ternary": (C.c_int32, [_vp, _vp, _vp, C.c_uint32, C.c_uint32, _pp]),
    "alice_weights_free": (C.c_int32, [_vp]),
    "alice_buf_alloc_f32": (C.c_int32, [_vp, C.c_size_t, _pp]),
    "alice_buf_upload_f32": (C.c_int32, [_vp, _vp, C.c_size_t, _pp]),
    "alice_buf_write_f32": (C.c_int32, [_vp, _vp, _vp, C.c_size_t]),
    "alice_buf_read_f32": (C.c_int32, [_vp, _vp, _vp, C.c_size_t]),
    "alice_buf_from_device": (C.c_int32, [_vp, _vp, C.c_size_t, _pp]),
    "alice_buf_free": (C.c_int32, [_vp]),
    "alice_q8k_alloc": (C.c_int32, [_vp, C.c_uint32, C.c_uint32, _pp]),
    "alice_quantize_q8k": (C.c_int32, [_vp, _vp, _vp]),
    "alice_q8k_read": (C.c_int32, [_vp, _vp, _vp, _vp, _vp]),
    "alice_q8k_upload": (C.c_int32, [_vp, _vp, _vp, _vp, C.c_uint32, C.c_uint32, _pp]),
    "alice_q8k_free": (C.c_int32, [_vp]),
    "alice_debug_expire_wait": (C.c_int32, [_vp]),
    "alice_buf_write_f32_async": (C.c_int32, [_vp, _vp, _vp, C.c_size_t]),
    "alice_buf_read_f32_async": (C.c_int32, [_vp, _vp, _vp, C.c_size_t]),
    "alice_ternarize": (C.c_int32, [_vp, _vp, C.c_uint32, C.c_uint32, C.c_float, _pp]),
    "alice_sparsify": (C.c_int32, [_vp, _vp, _vp, C.c_uint32, _pp]),
    "alice_weights_download": (C.c_int32, [_vp, _vp, _vp, C.c_size_t, _vp]),
    "alice_matvec": (C.c_int32, [_vp, _vp, _vp, _vp, C.c_uint32]),
    "alice_matvec_preq": (C.c_int32, [_vp, _vp, _vp, _vp]),
    "alice_swiglu": (C.c_int32, [_vp, _vp, _vp, _vp, _vp, C.c_uint32]),
    "alice_swiglu_preq": (C.c_int32, [_vp, _vp, _vp, _vp, _vp]),
    "alice_dequantize": (C.c_int32, [_vp, _vp, _vp]),
    "alice_plan_query": (C.c_int32, [_vp, _vp, C.c_int32, C.c_int32, _vp, C.c_uint32]),
    "alice_batch_plan": (C.c_int32, [_vp, _vp, C.c_int32, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "alice_model_create": (C.c_int32, [_vp, _vp, _vp, _vp, _vp, _vp, _pp]),
    "alice_model_destroy": (C.c_int32, [_vp]),
    "alice_model_forward": (C.c_int32, [_vp, C.c_uint32]),
    "alice_model_forward_read": (C.c_int32, [_vp, C.c_uint32, _vp]),
    "alice_model_decode_greedy": (C.c_int32, [_vp, C.c_uint32, C.c_uint32, _vp]),
    "alice_ternary_from_device": (C.c_int32, [_vp, _vp, _vp, C.c_uint32, C.c_uint32, _pp]),
    "alice_tp_unique_id": (C.c_int32, [_vp, C.c_size_t]),
    "alice_engine_tp_init": (C.c_int32, [_vp, C.c_uint32, C.c_uint32, _vp, C.c_size_t]),
    "alice_engine_tp_info": (C.c_int32, [_vp, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "alice_model_tp_export": (C.c_int32, [_vp, _vp, C.c_size_t]),
    "alice_model_tp_connect": (C.c_int32, [_vp, _vp, C.c_size_t]),
    "alice_model_forward_batch": (C.c_int32, [_vp, _vp, C.c_uint32]),
    "alice_model_forward_batch_read": (C.c_int32, [_vp, _vp, C.c_uint32, _vp]),
    "alice_model_read_logits": (C.c_int32, [_vp, _vp]),
    "alice_model_position": (C.c_int32, [_vp, C.POINTER(C.c_uint32)]),
    "alice_model_vocab_size": (C.c_int32, [_vp, C.POINTER(C.c_uint32)]),
    "alice_model_rollback_to": (C.c_int32, [_vp, C.c_uint32]),
    "alice_model_reset": (C.c_int32, [_vp]),
    "alice_model_kv_write": (C.c_int32, [_vp, C.c_uint32, C.c_uint32, C.c_uint32, _vp, _vp]),
    "alice_model_kv_read": (C.c_int32, [_vp, C.c_uint32, C.c_uint32, C.c_uint32, _vp, _vp]),
    "alice_model_set_position": (C.c_int32, [_vp, C.c_uint32]),
    "alice_matvec_preq_noalloc": (C.c_int32, [_vp, _vp, _vp, _vp]),
    "alice_matvec_host": (C.c_int32, [C.c_uint32, _vp, C.c_size_t, C.c_uint32, C.c_uint32, _vp, _vp]),
    "alice_dequantize_host": (C.c_int32, [C.c_uint32, _vp, C.c_size_t, _vp, C.c_size_t]),
}


class ModelConfig(C.Structure):
    """alice_model_config"""
    _fields_ = [(n, C.c_uint32) for n in ("num_layers", "hidden_dim", "intermediate_dim", "num_heads", "num_kv_heads",
                                          "head_dim", "vocab_size", "max_seq_len")] + \
               [("rope_theta", C.c_float), ("eps", C.c_float), ("neox_rope", C.c_uint32)]


class LayerWeights(C.Structure):
    """alice_layer_weights"""
    _fields_ = [(n, C.c_void_p) for n in ("q", "k", "v", "o", "gate", "up", "down", "attn_norm", "ffn_norm")]


class AliceError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"alice_cuda error {code}: {msg}")
        self.code = code


_lib = None


def lib_path() -> str:
    return _build.LIB


def load():
    """Load (building first if the .so is absent or older than its sources)."""
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path) or os.environ.get("ALICE_REBUILD") == "1":
            path = _build.build()
        lib = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise AliceError(rc, load().alice_last_error().decode("utf-8", "replace"))
