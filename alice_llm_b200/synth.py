"""Seeded synthetic tensors in the GGUF block formats of the decode path.

No model file or dataset is involved anywhere in this repository: every weight
matrix used by the tests and by the benchmark is drawn here from
``numpy.random.default_rng(seed)`` with the value distributions the benchmark
configurations state (block scale ``|N(0,1)|*0.01`` as f16, uniform quants,
``x ~ N(0,1)``).  Block layouts follow ALICE-LLM ``src/gguf.rs`` (Q4_K :903-939,
Q5_K :949-988, Q6_K :1205-1246, Q8_0 :990-1004, Q1_0/Q2_0 :1248-1300, ternary
bit planes :5190-5195, sparse-ternary masks :5425-5445).
"""
from __future__ import annotations

import numpy as np

QK_K = 256

# GGML type ids (src/gguf.rs:101-122)
Q8_0, Q4_K, Q5_K, Q6_K, Q1_0, Q2_0 = 8, 12, 13, 14, 41, 42
TERNARY = 1000   # in-memory ternary bit planes (TernaryMatrix, src/gguf.rs:5198); not a GGML id
SPARSE_TERNARY = 1001   # SparseTernaryMatrix's packed 2-bit codes + per-row scales (src/gguf.rs:5432); not a GGML id
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210, Q1_0: 18, Q2_0: 34}
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256, Q1_0: 128, Q2_0: 128}
TYPE_NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", Q1_0: "Q1_0", Q2_0: "Q2_0"}


def row_bytes(qtype: int, cols: int) -> int:
    return cols // BLOCK_ELEMS[qtype] * BLOCK_BYTES[qtype]


def _f16_scale(rng, shape, sigma):
    """|N(0,1)|*sigma rounded to f16, returned as little-endian byte pairs."""
    v = (np.abs(rng.standard_normal(shape, dtype=np.float32)) * np.float32(sigma)).astype(np.float16)
    return v.view(np.uint8).reshape(*shape, 2)


def pack_scales_k4(sc, mn):
    """Inverse of get_scale_min_k4 (src/gguf.rs:794-802): eight 6-bit scales and
    eight 6-bit mins -> the 12-byte header. ``sc``/``mn`` have shape (..., 8)."""
    sc = np.asarray(sc, dtype=np.uint8)
    mn = np.asarray(mn, dtype=np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0xF) | ((mn[..., 4:8] & 0xF) << 4)
    return out


def make_q4k(rng, rows: int, cols: int) -> np.ndarray:
    """Q4_K matrix, [rows * cols/256 * 144] bytes: f16 d ~ |N|*0.01, f16 dmin ~ |N|*0.005,
    6-bit scales/mins uniform 0..63, nibbles uniform 0..15."""
    nb = cols // QK_K
    blk = rng.integers(0, 256, size=(rows, nb, 144), dtype=np.uint8)  # uniform bytes = uniform fields
    blk[:, :, 0:2] = _f16_scale(rng, (rows, nb), 0.01)
    blk[:, :, 2:4] = _f16_scale(rng, (rows, nb), 0.005)
    return blk.reshape(-1)


def make_q5k(rng, rows: int, cols: int) -> np.ndarray:
    nb = cols // QK_K
    blk = rng.integers(0, 256, size=(rows, nb, 176), dtype=np.uint8)
    blk[:, :, 0:2] = _f16_scale(rng, (rows, nb), 0.01)
    blk[:, :, 2:4] = _f16_scale(rng, (rows, nb), 0.005)
    return blk.reshape(-1)


def make_q6k(rng, rows: int, cols: int) -> np.ndarray:
    """Q6_K: ql/qh uniform bytes, 16 int8 scales uniform -32..31, f16 d ~ |N|*0.01."""
    nb = cols // QK_K
    blk = rng.integers(0, 256, size=(rows, nb, 210), dtype=np.uint8)
    blk[:, :, 192:208] = rng.integers(-32, 32, size=(rows, nb, 16), dtype=np.int8).view(np.uint8)
    blk[:, :, 208:210] = _f16_scale(rng, (rows, nb), 0.01)
    return blk.reshape(-1)


def make_q8_0(rng, rows: int, cols: int) -> np.ndarray:
    """Q8_0: f16 d ~ |N|*0.01, int8 uniform -127..127."""
    nb = cols // 32
    blk = np.empty((rows, nb, 34), dtype=np.uint8)
    blk[:, :, 0:2] = _f16_scale(rng, (rows, nb), 0.01)
    blk[:, :, 2:] = rng.integers(-127, 128, size=(rows, nb, 32), dtype=np.int8).view(np.uint8)
    return blk.reshape(-1)


def make_q1_0(rng, rows: int, cols: int) -> np.ndarray:
    """Q1_0: f16 d ~ |N|*0.02, 16 bytes of uniform sign bits per 128 weights."""
    nb = cols // 128
    blk = rng.integers(0, 256, size=(rows, nb, 18), dtype=np.uint8)
    blk[:, :, 0:2] = _f16_scale(rng, (rows, nb), 0.02)
    return blk.reshape(-1)


def make_q2_0(rng, rows: int, cols: int) -> np.ndarray:
    """Q2_0: f16 d ~ |N|*0.02, 2-bit slots uniform over the three codes the encoder emits."""
    nb = cols // 128
    slots = rng.integers(0, 3, size=(rows, nb, 32, 4), dtype=np.uint8)
    by = slots[..., 0] | (slots[..., 1] << 2) | (slots[..., 2] << 4) | (slots[..., 3] << 6)
    blk = np.empty((rows, nb, 34), dtype=np.uint8)
    blk[:, :, 0:2] = _f16_scale(rng, (rows, nb), 0.02)
    blk[:, :, 2:] = by
    return blk.reshape(-1)


MAKERS = {Q4_K: make_q4k, Q5_K: make_q5k, Q6_K: make_q6k, Q8_0: make_q8_0, Q1_0: make_q1_0, Q2_0: make_q2_0}


def make_weights(qtype: int, rng, rows: int, cols: int):
    """Raw blocks of a GGML type, or (pos, neg, scales) for TERNARY."""
    if qtype == TERNARY:
        return make_ternary(rng, rows, cols)
    return MAKERS[qtype](rng, rows, cols)


def make_ternary(rng, rows: int, cols: int):
    """Ternary bit planes: P(0)=0.5, P(+1)=P(-1)=0.25, per-row f32 scale ~ |N|*0.01.
    Returns (pos[rows, ceil(cols/8)], neg[...], scales[rows]); bit i%8 of byte i/8, LSB first."""
    code = rng.integers(0, 4, size=(rows, cols), dtype=np.uint8)  # 0,1 -> 0 ; 2 -> +1 ; 3 -> -1
    pos = np.packbits(code == 2, axis=1, bitorder="little")
    neg = np.packbits(code == 3, axis=1, bitorder="little")
    scales = (np.abs(rng.standard_normal(rows, dtype=np.float32)) * np.float32(0.01)).astype(np.float32)
    return np.ascontiguousarray(pos), np.ascontiguousarray(neg), scales


def ternary_to_sparse(pos: np.ndarray, neg: np.ndarray, cols: int):
    """Re-express bit planes as SparseTernaryMatrix masks (active u16, sign u16 per 16 columns;
    sign bit 1 = negative) without dropping any weight."""
    rows = pos.shape[0]
    bpr = (cols + 15) // 16
    padded = np.zeros((rows, bpr * 2), dtype=np.uint8)
    padded[:, : pos.shape[1]] = pos | neg
    active = padded.view("<u2").copy()
    padded[:] = 0
    padded[:, : neg.shape[1]] = neg
    sign = padded.view("<u2").copy()
    return active, sign


_F16_FIELDS = {Q4_K: (0, 2), Q5_K: (0, 2), Q6_K: (208,), Q8_0: (0,), Q1_0: (0,), Q2_0: (0,)}


def pack_2bit(pos: np.ndarray, neg: np.ndarray, cols: int) -> np.ndarray:
    """SparseTernaryMatrix.packed_2bit of bit planes (src/gguf.rs:5432-5450): per weight two bits, 00 = 0, 01 = +1,
    11 = -1, four weights per byte (lowest bits first), rows padded to whole blocks of 16 weights (4 bytes).
    Returns uint8 [rows][ceil(cols / 16) * 4]."""
    rows = pos.shape[0]
    bpr = (cols + 15) // 16
    bits_p = np.unpackbits(pos, axis=1, bitorder="little")[:, :cols]
    bits_n = np.unpackbits(neg, axis=1, bitorder="little")[:, :cols]
    codes = np.zeros((rows, bpr * 16), dtype=np.uint8)
    codes[:, :cols] = bits_p | bits_n | (bits_n << 1)          # +1 -> 01, -1 -> 11
    c = codes.reshape(rows, bpr * 4, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).astype(np.uint8)


def to_sparse_ternary(model: dict) -> dict:
    """A make_llama model whose TERNARY tensors become SPARSE_TERNARY ones holding the same weights (nothing dropped):
    the form Llama3Model::forward_sparse_ternary runs on (src/llama3.rs:17216-17330)."""
    def conv(entry, cols):
        t, data = entry
        if t != TERNARY:
            return entry
        pos, neg, sc = data
        return SPARSE_TERNARY, (pack_2bit(pos, neg, cols), sc)
    cfg = model["config"]
    H, F, q_dim = cfg["hidden_dim"], cfg["intermediate_dim"], cfg["num_heads"] * cfg["head_dim"]
    cols = {"q": H, "k": H, "v": H, "o": q_dim, "gate": H, "up": H, "down": F}
    out = dict(model)
    out["layers"] = [{**L, **{n: conv(L[n], c) for n, c in cols.items()}} for L in model["layers"]]
    out["output"] = conv(model["output"], H)
    return out


def scale_blocks(entry, factor):
    """(type, raw blocks) with every f16 block scale multiplied by `factor` (ternary planes: the per-row scales)."""
    t, data = entry
    if t == TERNARY:
        pos, neg, sc = data
        return t, (pos, neg, (sc * np.float32(factor)).astype(np.float32))
    blk = data.reshape(-1, BLOCK_BYTES[t]).copy()
    for off in _F16_FIELDS[t]:
        v = blk[:, off:off + 2].copy().view(np.float16).astype(np.float32) * np.float32(factor)
        blk[:, off:off + 2] = v.astype(np.float16).view(np.uint8).reshape(-1, 2)
    return t, blk.reshape(-1)


def soften_attention(model: dict, factor: float | None = None) -> dict:
    """Scales the q / k / v projections of a make_llama model (default 0.3 / sqrt(hidden)) so that the softmax spreads
    over the context instead of collapsing onto the newest row: the synthetic K-quant weights have a positive mean, so
    an unscaled q . k grows with hidden_dim. Returns the model (modified in place)."""
    if factor is None:
        factor = 0.3 / float(np.sqrt(model["config"]["hidden_dim"]))
    for L in model["layers"]:
        for n in ("q", "k", "v"):
            L[n] = scale_blocks(L[n], factor)
    return model


def make_x(rng, n: int, batch: int = 1) -> np.ndarray:
    """Activations ~ N(0,1), f32, layout x[k*n + c]."""
    return rng.standard_normal(batch * n, dtype=np.float32)


def make_llama(rng, cfg: dict, mix: dict | None = None) -> dict:
    """Random-init Llama-architecture model as raw quantized blocks.

    cfg keys: num_layers, hidden_dim, intermediate_dim, num_heads, num_kv_heads, head_dim, vocab_size,
    max_seq_len, rope_theta, eps. ``mix`` maps tensor role -> GGML type; the default is the Q4_K_M mix
    of the 8B benchmark configuration: q/k/v/o/gate/up Q4_K, down and output head Q6_K, embedding Q8_0.
    A role mapped to TERNARY carries (pos, neg, scales) bit planes instead of blocks (the 70B configuration:
    every projection and the output head ternary). RMSNorm weights are 1 + N(0, 0.02)."""
    mix = {"q": Q4_K, "k": Q4_K, "v": Q4_K, "o": Q4_K, "gate": Q4_K, "up": Q4_K, "down": Q6_K, "output": Q6_K,
           **(mix or {})}
    H, F = cfg["hidden_dim"], cfg["intermediate_dim"]
    q_dim, kv_dim = cfg["num_heads"] * cfg["head_dim"], cfg["num_kv_heads"] * cfg["head_dim"]
    shapes = {"q": (q_dim, H), "k": (kv_dim, H), "v": (kv_dim, H), "o": (H, q_dim), "gate": (F, H), "up": (F, H),
              "down": (H, F)}

    def norm():
        return (1.0 + 0.02 * rng.standard_normal(H, dtype=np.float32)).astype(np.float32)

    layers = []
    for _ in range(cfg["num_layers"]):
        L = {n: (mix[n], make_weights(mix[n], rng, *shapes[n])) for n in shapes}
        L["attn_norm"], L["ffn_norm"] = norm(), norm()
        layers.append(L)
    return {"config": dict(cfg), "layers": layers,
            "embedding": (Q8_0, make_q8_0(rng, cfg["vocab_size"], H)),
            "output_norm": norm(),
            "output": (mix["output"], make_weights(mix["output"], rng, cfg["vocab_size"], H))}
