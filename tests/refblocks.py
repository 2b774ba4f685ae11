"""Seeded block factories of the reference's own unit tests, rebuilt byte for byte
(ALICE-LLM src/gguf.rs:7747-7808 Q4_K/Q6_K/Q8_K, :7909-7928 Q5_K, :7978-8000 Q8_0,
:8054-8081 ternary). They fill every byte of a block from a u8 seed with wrapping
arithmetic, so the same seed gives the same block here and in the Rust tests."""
import numpy as np

SEEDS = [0, 1, 7, 128, 200, 255]


def _u8(v):
    return np.uint8(v & 0xFF)


def make_q4k_block(seed: int) -> np.ndarray:
    b = np.zeros(144, dtype=np.uint8)
    b[0:2] = [0x00, 0x38]  # f16 0.5
    b[2:4] = [0x00, 0x34]  # f16 0.25
    for i in range(12):
        b[4 + i] = (seed + i) & 0xFF
    for i in range(128):
        b[16 + i] = (seed * 3 + i) & 0xFF
    return b


def make_q5k_block(seed: int) -> np.ndarray:
    b = np.zeros(176, dtype=np.uint8)
    b[0:2] = [0x00, 0x38]
    b[2:4] = [0x00, 0x34]
    for i in range(12):
        b[4 + i] = (seed + i) & 0xFF
    for i in range(32):
        b[16 + i] = (seed * 7 + i) & 0xFF
    for i in range(128):
        b[48 + i] = (seed * 3 + i) & 0xFF
    return b


def make_q6k_block(seed: int) -> np.ndarray:
    b = np.zeros(210, dtype=np.uint8)
    for i in range(128):
        b[i] = (seed + i) & 0xFF
    for i in range(64):
        b[128 + i] = (seed * 5 + i) & 0xFF
    for i in range(16):
        b[192 + i] = (i - 4) & 0xFF
    b[208:210] = [0x00, 0x38]
    return b


def make_q8k_block(seed: int):
    """-> (d, qs[256] i8, bsums[16] i16)"""
    raw = (seed + np.arange(256)) & 0xFF
    qs = ((raw.astype(np.uint8).view(np.int8).astype(np.int32) - 64 + 128) % 256 - 128).astype(np.int8)
    bsums = qs.astype(np.int32).reshape(16, 16).sum(axis=1).astype(np.int16)
    return np.float32(0.125), qs, bsums


def make_q8_0_row_bytes(seed: int, cols: int) -> np.ndarray:
    out = []
    for bi in range(cols // 32):
        sb = (0x3800 + bi) & 0xFFFF
        out += [sb & 0xFF, sb >> 8]
        for l in range(32):
            raw = (seed + bi * 32 + l) & 0xFF
            s = raw - 256 if raw >= 128 else raw
            s = ((s - 32 + 128) % 256) - 128
            out.append(s & 0xFF)
    return np.array(out, dtype=np.uint8)


def make_q8_0_input(seed: int, cols: int) -> np.ndarray:
    raw = ((seed + np.arange(cols)) & 0xFF).astype(np.uint8).view(np.int8)
    return raw.astype(np.float32) * np.float32(0.01)


def make_ternary_row(seed: int, cols: int):
    nbytes = (cols + 7) // 8
    pos = np.zeros(nbytes, dtype=np.uint8)
    neg = np.zeros(nbytes, dtype=np.uint8)
    for i in range(cols):
        raw = (seed * 3 + i) & 0xFF
        s = raw - 256 if raw >= 128 else raw
        if s > 20:
            pos[i // 8] |= 1 << (i % 8)
        elif s < -20:
            neg[i // 8] |= 1 << (i % 8)
    return pos, neg


def make_ternary_input(seed: int, cols: int) -> np.ndarray:
    raw = ((seed + np.arange(cols)) & 0xFF).astype(np.uint8).view(np.int8)
    return raw.astype(np.float32) * np.float32(0.01)
