"""Independent numpy statement of the block formats (written from the layout tables, not from the
C++ oracle) used to cross-check the oracle on small cases. Integer parts are exact; the float
tail uses np.float32 scalars in the reference's order (ALICE-LLM src/gguf.rs:3250, 3318, 3393-3409)."""
import numpy as np

f32 = np.float32


def f16(b0, b1):
    return np.array([b0, b1], dtype=np.uint8).view(np.float16)[0].astype(np.float32)


def k4_scales(s12):
    s = [int(v) for v in s12]
    sc = [0] * 8
    mn = [0] * 8
    for j in range(4):
        sc[j] = s[j] & 63
        mn[j] = s[j + 4] & 63
        sc[j + 4] = (s[j + 8] & 0xF) | ((s[j] >> 6) << 4)
        mn[j + 4] = (s[j + 8] >> 4) | ((s[j + 4] >> 6) << 4)
    return sc, mn


def q4k_quants(blk):
    qs = blk[16:144].astype(np.int32).reshape(4, 32)
    return np.stack([qs & 0xF, qs >> 4], axis=1).reshape(256)


def q5k_quants(blk):
    qh = blk[16:48].astype(np.int32)
    qs = blk[48:176].astype(np.int32).reshape(4, 32)
    out = np.zeros((4, 2, 32), dtype=np.int32)
    for im in range(4):
        out[im, 0] = (qs[im] & 0xF) | (((qh >> (2 * im)) & 1) << 4)
        out[im, 1] = (qs[im] >> 4) | (((qh >> (2 * im + 1)) & 1) << 4)
    return out.reshape(256)


def q6k_quants(blk):
    ql = blk[0:128].astype(np.int32)
    qh = blk[128:192].astype(np.int32)
    e = np.zeros(256, dtype=np.int32)
    for n in range(2):
        for l in range(32):
            h = qh[32 * n + l]
            e[128 * n + l] = (ql[64 * n + l] & 0xF) | ((h & 3) << 4)
            e[128 * n + 32 + l] = (ql[64 * n + 32 + l] & 0xF) | (((h >> 2) & 3) << 4)
            e[128 * n + 64 + l] = (ql[64 * n + l] >> 4) | (((h >> 4) & 3) << 4)
            e[128 * n + 96 + l] = (ql[64 * n + 32 + l] >> 4) | (((h >> 6) & 3) << 4)
    return e - 32


def q4k_dot(blk, d8, q8, bsums):
    d, dmin = f16(blk[0], blk[1]), f16(blk[2], blk[3])
    sc, mn = k4_scales(blk[4:16])
    q = q4k_quants(blk)
    q8 = q8.astype(np.int32)
    total = sum(sc[i] * int((q[32 * i:32 * i + 32] * q8[32 * i:32 * i + 32]).sum()) for i in range(8))
    sumi = sum(int(bsums[j]) * mn[j // 2] for j in range(16))
    return f32(f32(f32(d * f32(d8)) * f32(total)) - f32(f32(dmin * f32(d8)) * f32(sumi)))


def q5k_dot(blk, d8, q8, bsums):
    d, dmin = f16(blk[0], blk[1]), f16(blk[2], blk[3])
    sc, mn = k4_scales(blk[4:16])
    q = q5k_quants(blk)
    q8 = q8.astype(np.int32)
    sumf = f32(0)
    for i in range(8):
        dot = int((q[32 * i:32 * i + 32] * q8[32 * i:32 * i + 32]).sum())
        s = int(q8[32 * i:32 * i + 32].sum())
        sumf = f32(sumf + f32(f32(f32(d * f32(sc[i])) * f32(dot)) - f32(f32(dmin * f32(mn[i])) * f32(s))))
    return f32(sumf * f32(d8))


def q6k_dot(blk, d8, q8, bsums):
    d = f16(blk[208], blk[209])
    q = q6k_quants(blk)
    sc = blk[192:208].view(np.int8).astype(np.int32)
    q8 = q8.astype(np.int32)
    total = sum(int(sc[i]) * int((q[16 * i:16 * i + 16] * q8[16 * i:16 * i + 16]).sum()) for i in range(16))
    return f32(f32(d * f32(d8)) * f32(total))


def q8k_quantize(x):
    """numpy restatement of quantize_row_q8_k (src/gguf.rs:1323-1374)."""
    x = np.asarray(x, dtype=np.float32).reshape(-1, 256)
    nb = x.shape[0]
    d = np.zeros(nb, dtype=np.float32)
    qs = np.zeros((nb, 256), dtype=np.int8)
    for i in range(nb):
        a = np.abs(x[i])
        j = int(np.argmax(a))  # first maximal element
        if a[j] == 0:
            continue
        iscale = f32(128.0) / x[i, j]
        v = (iscale * x[i]).astype(np.float32) + f32(12582912.0)
        q = (v.view(np.int32) & 0x007FFFFF) - 0x00400000
        qs[i] = np.clip(q, -128, 127).astype(np.int8)
        d[i] = f32(1.0) / iscale
    bsums = qs.astype(np.int32).reshape(nb, 16, 16).sum(axis=2).astype(np.int16)
    return d, qs, bsums
