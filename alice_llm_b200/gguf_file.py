"""GGUF container: parse a file (mmap, zero copy) and hand its raw tensor blocks to the device.

``GgufFile.parse`` follows ``GgufFile::parse`` of ALICE-LLM src/gguf.rs:439-505: magic ``GGUF``, version 2 or 3,
tensor count, metadata count, metadata key/values (src/gguf.rs:386-417), tensor infos (name, dims innermost first,
GGML type, offset), data section aligned to ``general.alignment`` (default 32); ``tensor_data`` =
``data[tensor_data_start + offset ..][..size]`` (src/gguf.rs:557-565). ``model_config`` mirrors
``Llama3Config::from_gguf`` (src/llama3.rs:4089-4140) for the Llama-style stack and ``load_model`` the tensor-name
table of ``load_layer_weights`` (src/llama3.rs:19392-19470): ``blk.{i}.attn_q.weight`` ... ``ffn_down.weight``,
``token_embd.weight``, ``output_norm.weight``, ``output.weight``.  ``write_gguf`` is the inverse of ``parse`` (the
reference builds its fixtures the same way, src/llama3.rs:836-1060) and lets a synthetic model travel as a file.
"""
from __future__ import annotations

import mmap
import struct

import numpy as np

from . import synth

GGUF_MAGIC = 0x46554747          # "GGUF", src/gguf.rs:11
DEFAULT_ALIGNMENT = 32
F32 = 0                          # GGML type id of plain f32 tensors (norm weights)

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class GgufError(ValueError):
    pass


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError("GGUF: truncated file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self):
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufError("GGUF: truncated string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s

    def value(self, vtype):
        if vtype in _SCALAR:
            return self.take(_SCALAR[vtype])
        if vtype == 8:
            return self.string()
        if vtype == 9:
            atype, n = self.take("<I"), self.take("<Q")
            # every element takes at least one byte of the file: a count beyond what is left is a corrupt header
            if n > len(self.buf) - self.pos:
                raise GgufError(f"GGUF: array of {n} elements in a file with {len(self.buf) - self.pos} bytes left")
            if atype == 9:
                raise GgufError("GGUF: nested arrays are not supported")
            return [self.value(atype) for _ in range(n)]
        raise GgufError(f"GGUF: unknown metadata value type {vtype}")


class TensorInfo:
    def __init__(self, name, dims, qtype, offset):
        self.name, self.dims, self.qtype, self.offset = name, dims, qtype, offset

    @property
    def cols(self):          # GGML stores the innermost dimension first
        return self.dims[0]

    @property
    def rows(self):
        n = 1
        for d in self.dims[1:]:
            n *= d
        return n

    def data_size(self):
        n = self.rows * self.cols
        if self.qtype == F32:
            return n * 4
        if self.qtype not in synth.BLOCK_BYTES:
            raise GgufError(f"GGUF: tensor {self.name} has GGML type {self.qtype}, outside the decode path")
        return n // synth.BLOCK_ELEMS[self.qtype] * synth.BLOCK_BYTES[self.qtype]


class GgufFile:
    def __init__(self, buf, metadata, tensors, data_start, keep=None):
        self.buf, self.metadata, self.tensors, self.tensor_data_start, self._keep = buf, metadata, tensors, data_start, keep

    @classmethod
    def parse(cls, data, keep=None) -> "GgufFile":
        """``data``: bytes-like (e.g. an mmap). Raises GgufError where the reference returns None."""
        r = _Reader(memoryview(data))
        if r.take("<I") != GGUF_MAGIC:
            raise GgufError("GGUF: bad magic")
        version = r.take("<I")
        if version not in (2, 3):
            raise GgufError(f"GGUF: unsupported version {version}")
        n_tensors, n_meta = r.take("<Q"), r.take("<Q")
        # a tensor info is at least 24 bytes, a metadata entry at least 12: counts the file cannot hold are rejected up front
        if n_tensors * 24 > len(r.buf) or n_meta * 12 > len(r.buf):
            raise GgufError(f"GGUF: header claims {n_tensors} tensors and {n_meta} metadata entries in a file of {len(r.buf)} bytes")
        metadata = {}
        for _ in range(n_meta):
            key = r.string()
            metadata[key] = r.value(r.take("<I"))
        tensors = {}
        for _ in range(n_tensors):
            name = r.string()
            n_dims = r.take("<I")
            if n_dims > 8:
                raise GgufError(f"GGUF: tensor {name} has {n_dims} dimensions")
            dims = [r.take("<Q") for _ in range(n_dims)]
            qtype, offset = r.take("<I"), r.take("<Q")
            tensors[name] = TensorInfo(name, dims, qtype, offset)
        align = metadata.get("general.alignment", DEFAULT_ALIGNMENT)
        if not isinstance(align, int) or isinstance(align, bool) or align < 1 or align & (align - 1) or align > (1 << 20):
            raise GgufError(f"GGUF: general.alignment = {align!r} (a power of two of at least 1 is expected)")
        start = (r.pos + align - 1) // align * align
        return cls(r.buf, metadata, tensors, start, keep)

    @classmethod
    def open(cls, path) -> "GgufFile":
        f = open(path, "rb")
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return cls.parse(mm, keep=(f, mm))

    def tensor_data(self, name) -> np.ndarray:
        """Raw bytes of a tensor as a zero-copy uint8 view of the file."""
        info = self.tensors.get(name)
        if info is None:
            raise GgufError(f"GGUF: tensor {name} missing")
        start, size = self.tensor_data_start + info.offset, info.data_size()
        if start + size > len(self.buf):
            raise GgufError(f"GGUF: tensor {name} reaches past the end of the file")
        return np.frombuffer(self.buf, dtype=np.uint8, count=size, offset=start)

    def tensor_f32(self, name) -> np.ndarray:
        info = self.tensors.get(name)
        if info is None or info.qtype != F32:
            raise GgufError(f"GGUF: f32 tensor {name} missing")
        return self.tensor_data(name).view(np.float32)

    # -- Llama3Config::from_gguf, the fields of the Llama-style stack --
    def model_config(self, max_seq_len=None) -> dict:
        arch = self.metadata.get("general.architecture", "llama")
        m = self.metadata
        # The decode graph built here is the Llama branch of the reference (interleaved RoPE pairs, no biases, RMSNorm,
        # SwiGLU). The reference dispatches on ModelArch (src/llama3.rs:74-236: NeoX RoPE for qwen2 / gemma / ...,
        # other defaults for mistral); until those branches exist a file of another architecture is refused rather
        # than decoded with the wrong semantics.
        if arch != "llama":
            raise GgufError(f"GGUF: architecture {arch!r} is not supported (only 'llama')")

        def need(key):
            if f"{arch}.{key}" not in m:
                raise GgufError(f"GGUF: metadata {arch}.{key} missing")
            return m[f"{arch}.{key}"]

        hidden, heads = int(need("embedding_length")), int(need("attention.head_count"))
        ffn = need("feed_forward_length")
        ffn = int(ffn[0] if isinstance(ffn, list) else ffn)
        vocab = m.get(f"{arch}.vocab_size")
        if vocab is None:
            vocab = len(m["tokenizer.ggml.tokens"]) if "tokenizer.ggml.tokens" in m else self.tensors["token_embd.weight"].rows
        ctx = min(int(m.get(f"{arch}.context_length", 8192)), 8192)
        return dict(num_layers=int(need("block_count")), hidden_dim=hidden, intermediate_dim=ffn, num_heads=heads,
                    num_kv_heads=int(m.get(f"{arch}.attention.head_count_kv", heads)),
                    head_dim=int(m.get(f"{arch}.attention.key_length", hidden // heads)), vocab_size=int(vocab),
                    max_seq_len=int(max_seq_len or ctx), rope_theta=float(m.get(f"{arch}.rope.freq_base", 500000.0)),
                    eps=float(m.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5)))

    # -- the tensor-name table of load_layer_weights --
    ROLES = {"q": "attn_q", "k": "attn_k", "v": "attn_v", "o": "attn_output", "gate": "ffn_gate", "up": "ffn_up", "down": "ffn_down"}

    def load_model(self, max_seq_len=None) -> dict:
        """The model as the dict ``GpuModel.load`` takes: raw blocks stay views of the file."""
        cfg = self.model_config(max_seq_len)
        q_dim, kv_dim = cfg["num_heads"] * cfg["head_dim"], cfg["num_kv_heads"] * cfg["head_dim"]
        H, F = cfg["hidden_dim"], cfg["intermediate_dim"]
        shapes = {"q": (q_dim, H), "k": (kv_dim, H), "v": (kv_dim, H), "o": (H, q_dim), "gate": (F, H), "up": (F, H), "down": (H, F)}

        def weight(name, rows, cols):
            info = self.tensors.get(name)
            if info is None:
                raise GgufError(f"GGUF: tensor {name} missing")
            if (info.rows, info.cols) != (rows, cols):
                raise GgufError(f"GGUF: tensor {name} is {info.rows}x{info.cols}, expected {rows}x{cols}")
            return info.qtype, self.tensor_data(name)

        layers = []
        for i in range(cfg["num_layers"]):
            L = {role: weight(f"blk.{i}.{stem}.weight", *shapes[role]) for role, stem in self.ROLES.items()}
            L["attn_norm"] = self.tensor_f32(f"blk.{i}.attn_norm.weight")
            L["ffn_norm"] = self.tensor_f32(f"blk.{i}.ffn_norm.weight")
            layers.append(L)
        emb = weight("token_embd.weight", cfg["vocab_size"], H)
        out_name = "output.weight" if "output.weight" in self.tensors else "token_embd.weight"   # tied embeddings
        return {"config": cfg, "layers": layers, "embedding": emb, "output_norm": self.tensor_f32("output_norm.weight"),
                "output": weight(out_name, cfg["vocab_size"], H)}


def _w_string(out, s):
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def write_gguf(path, model: dict, arch: str = "llama", alignment: int = DEFAULT_ALIGNMENT) -> None:
    """Writes a model dict (``synth.make_llama``) as a GGUF v3 file: the metadata ``model_config`` reads and the tensors
    ``load_model`` looks up, data section aligned, tensors in the order of the name table."""
    cfg = model["config"]
    meta = [("general.architecture", 8, arch), ("general.alignment", 4, alignment),
            (f"{arch}.block_count", 4, cfg["num_layers"]), (f"{arch}.embedding_length", 4, cfg["hidden_dim"]),
            (f"{arch}.feed_forward_length", 4, cfg["intermediate_dim"]), (f"{arch}.attention.head_count", 4, cfg["num_heads"]),
            (f"{arch}.attention.head_count_kv", 4, cfg["num_kv_heads"]), (f"{arch}.attention.key_length", 4, cfg["head_dim"]),
            (f"{arch}.context_length", 4, cfg["max_seq_len"]), (f"{arch}.vocab_size", 4, cfg["vocab_size"]),
            (f"{arch}.rope.freq_base", 6, cfg["rope_theta"]), (f"{arch}.attention.layer_norm_rms_epsilon", 6, cfg["eps"])]
    q_dim, kv_dim = cfg["num_heads"] * cfg["head_dim"], cfg["num_kv_heads"] * cfg["head_dim"]
    H, F = cfg["hidden_dim"], cfg["intermediate_dim"]
    shapes = {"q": (q_dim, H), "k": (kv_dim, H), "v": (kv_dim, H), "o": (H, q_dim), "gate": (F, H), "up": (F, H), "down": (H, F)}
    tensors = [("token_embd.weight", model["embedding"][0], (cfg["vocab_size"], H), model["embedding"][1]),
               ("output_norm.weight", F32, (H,), model["output_norm"]),
               ("output.weight", model["output"][0], (cfg["vocab_size"], H), model["output"][1])]
    for i, L in enumerate(model["layers"]):
        tensors.append((f"blk.{i}.attn_norm.weight", F32, (H,), L["attn_norm"]))
        tensors.append((f"blk.{i}.ffn_norm.weight", F32, (H,), L["ffn_norm"]))
        for role, stem in GgufFile.ROLES.items():
            tensors.append((f"blk.{i}.{stem}.weight", L[role][0], shapes[role], L[role][1]))
    head = bytearray(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(meta)))
    for key, vtype, value in meta:
        _w_string(head, key)
        head += struct.pack("<I", vtype)
        if vtype == 8:
            _w_string(head, value)
        else:
            head += struct.pack(_SCALAR[vtype], value)
    offset, blobs = 0, []
    for name, qtype, shape, data in tensors:
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        _w_string(head, name)
        dims = tuple(reversed(shape))                   # innermost first
        head += struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", qtype, offset)
        blobs.append((offset, raw))
        offset = (offset + raw.size + alignment - 1) // alignment * alignment
    start = (len(head) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (start - len(head)))
        for off, raw in blobs:
            f.seek(start + off)
            f.write(raw.tobytes())
        f.truncate(start + offset)
