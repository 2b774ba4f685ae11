// CPU oracle for the quantized-matvec decode path of ALICE-LLM.
//
// THIS FILE IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. It is a plain scalar C++
// restatement of the reference's CPU algorithm (src/gguf.rs, src/llama3.rs of
// ext-sakamoro/ALICE-LLM v1.6.0), written so that every floating-point operation
// happens in the same order and with the same rounding as the Rust original.
// Only tests/, the smoke check and the benchmark's CPU-baseline leg may load it.
// The CUDA library never links or calls it.
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fno-fast-math -fPIC -shared
// (Rust never contracts a*b+c into an FMA, so contraction is switched off.)
//
// Parity pins: the reference has no golden output vectors for the K-quants; its
// own tests pin the SIMD kernels bit-exactly to the scalar fallbacks restated
// here (src/gguf.rs:7810-7970) and hold known-answer cases for f16, Q1_0, Q2_0,
// Q8_0, get_scale_min_k4, ternary and sparse-ternary (src/gguf.rs:6627-6650,
// 7181-7459, 7507-7626, 8054-8153). tests/test_oracle_pins.py replays those.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>

namespace {

constexpr int QK_K = 256;    // src/gguf.rs:13
constexpr int QK8_0 = 32;    // src/gguf.rs:14
constexpr int QK_G128 = 128; // src/gguf.rs:180

// GGML type ids, src/gguf.rs:101-122.
enum : uint32_t { T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_Q1_0 = 41, T_Q2_0 = 42 };

inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

// src/gguf.rs:19-45
float f16_to_f32(uint16_t h) {
    uint32_t sign = (h >> 15) & 1u;
    uint32_t exponent = (h >> 10) & 0x1fu;
    uint32_t mantissa = h & 0x3ffu;
    if (exponent == 0) {
        if (mantissa == 0) return bits_f32(sign << 31);
        uint32_t e = 0, m = mantissa;
        while ((m & 0x400u) == 0) { m <<= 1; e += 1; }
        uint32_t exp = 127 - 15 - e + 1;
        uint32_t man = (m & 0x3ffu) << 13;
        return bits_f32((sign << 31) | (exp << 23) | man);
    } else if (exponent == 31) {
        return bits_f32((sign << 31) | (0xffu << 23) | (mantissa << 13));
    }
    uint32_t exp = exponent + 127 - 15;
    return bits_f32((sign << 31) | (exp << 23) | (mantissa << 13));
}

inline float rd_f16(const uint8_t* p) { return f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }

// src/gguf.rs:126-157
int block_bytes(uint32_t t) {
    switch (t) {
        case T_Q8_0: return 34; case T_Q4_K: return 144; case T_Q5_K: return 176;
        case T_Q6_K: return 210; case T_Q1_0: return 18; case T_Q2_0: return 34;
        default: return 0;
    }
}
// src/gguf.rs:161-176
int elements_per_block(uint32_t t) {
    switch (t) {
        case T_Q8_0: return QK8_0;
        case T_Q4_K: case T_Q5_K: case T_Q6_K: return QK_K;
        case T_Q1_0: case T_Q2_0: return QK_G128;
        default: return 1;
    }
}

// src/gguf.rs:794-802
void get_scale_min_k4(int j, const uint8_t* scales, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = scales[j] & 63; *m = scales[j + 4] & 63;
    } else {
        *sc = (uint8_t)((scales[j + 4] & 0xF) | ((scales[j - 4] >> 6) << 4));
        *m = (uint8_t)((scales[j + 4] >> 4) | ((scales[j] >> 6) << 4));
    }
}

// src/gguf.rs:903-939
void dequantize_q4_k(const uint8_t* data, size_t nbytes, float* out) {
    size_t nb = nbytes / 144, oi = 0;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 144;
        float d = rd_f16(b), dmin = rd_f16(b + 2);
        const uint8_t* scales = b + 4; const uint8_t* qs = b + 16;
        int is = 0; size_t qo = 0;
        for (int g = 0; g < 4; g++) {
            uint8_t sc1, m1, sc2, m2;
            get_scale_min_k4(is, scales, &sc1, &m1);
            get_scale_min_k4(is + 1, scales, &sc2, &m2);
            float d1 = d * (float)sc1, m1f = dmin * (float)m1;
            float d2 = d * (float)sc2, m2f = dmin * (float)m2;
            for (int l = 0; l < 32; l++) out[oi++] = d1 * (float)(qs[qo + l] & 0xF) - m1f;
            for (int l = 0; l < 32; l++) out[oi++] = d2 * (float)(qs[qo + l] >> 4) - m2f;
            qo += 32; is += 2;
        }
    }
}

// src/gguf.rs:949-988
void dequantize_q5_k(const uint8_t* data, size_t nbytes, float* out) {
    size_t nb = nbytes / 176, oi = 0;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 176;
        float d = rd_f16(b), dmin = rd_f16(b + 2);
        const uint8_t* scales = b + 4; const uint8_t* qh = b + 16; const uint8_t* qs = b + 48;
        int is = 0; size_t qo = 0;
        for (int im = 0; im < 4; im++) {
            uint8_t sc1, m1, sc2, m2;
            get_scale_min_k4(is, scales, &sc1, &m1);
            get_scale_min_k4(is + 1, scales, &sc2, &m2);
            float d1 = d * (float)sc1, m1f = dmin * (float)m1;
            float d2 = d * (float)sc2, m2f = dmin * (float)m2;
            for (int l = 0; l < 32; l++) {
                uint8_t hbit = (qh[l] >> (im * 2)) & 1;
                out[oi++] = d1 * (float)((qs[qo + l] & 0xF) | (hbit << 4)) - m1f;
            }
            for (int l = 0; l < 32; l++) {
                uint8_t hbit = (qh[l] >> (im * 2 + 1)) & 1;
                out[oi++] = d2 * (float)((qs[qo + l] >> 4) | (hbit << 4)) - m2f;
            }
            qo += 32; is += 2;
        }
    }
}

// src/gguf.rs:990-1004
void dequantize_q8_0(const uint8_t* data, size_t nbytes, float* out) {
    size_t nb = nbytes / 34, oi = 0;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 34;
        float d = rd_f16(b);
        for (int l = 0; l < QK8_0; l++) out[oi++] = d * (float)(int8_t)b[2 + l];
    }
}

// 6-bit unpack shared by src/gguf.rs:1222-1231, 3292-3305 and 6280-6293.
void q6k_unpack(const uint8_t* ql, const uint8_t* qh, int8_t* aux8) {
    int ao = 0, qlo = 0, qho = 0;
    for (int n = 0; n < 2; n++) {
        for (int l = 0; l < 32; l++) {
            aux8[ao + l] = (int8_t)((ql[qlo + l] & 0xF) | ((qh[qho + l] & 3) << 4)) - 32;
            aux8[ao + l + 32] = (int8_t)((ql[qlo + l + 32] & 0xF) | (((qh[qho + l] >> 2) & 3) << 4)) - 32;
            aux8[ao + l + 64] = (int8_t)((ql[qlo + l] >> 4) | (((qh[qho + l] >> 4) & 3) << 4)) - 32;
            aux8[ao + l + 96] = (int8_t)((ql[qlo + l + 32] >> 4) | (((qh[qho + l] >> 6) & 3) << 4)) - 32;
        }
        ao += 128; qlo += 64; qho += 32;
    }
}

// src/gguf.rs:1205-1246
void dequantize_q6_k(const uint8_t* data, size_t nbytes, float* out) {
    size_t nb = nbytes / 210, oi = 0;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 210;
        const uint8_t* ql = b; const uint8_t* qh = b + 128; const uint8_t* sc = b + 192;
        float d = rd_f16(b + 208);
        int qlo = 0, qho = 0, sco = 0;
        for (int n = 0; n < 2; n++) {
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int8_t q1 = (int8_t)((ql[qlo + l] & 0xF) | ((qh[qho + l] & 3) << 4)) - 32;
                int8_t q2 = (int8_t)((ql[qlo + l + 32] & 0xF) | (((qh[qho + l] >> 2) & 3) << 4)) - 32;
                int8_t q3 = (int8_t)((ql[qlo + l] >> 4) | (((qh[qho + l] >> 4) & 3) << 4)) - 32;
                int8_t q4 = (int8_t)((ql[qlo + l + 32] >> 4) | (((qh[qho + l] >> 6) & 3) << 4)) - 32;
                out[oi + l]      = d * (float)(int8_t)sc[sco + is]     * (float)q1;
                out[oi + l + 32] = d * (float)(int8_t)sc[sco + is + 2] * (float)q2;
                out[oi + l + 64] = d * (float)(int8_t)sc[sco + is + 4] * (float)q3;
                out[oi + l + 96] = d * (float)(int8_t)sc[sco + is + 6] * (float)q4;
            }
            oi += 128; qlo += 64; qho += 32; sco += 8;
        }
    }
}

// src/gguf.rs:1264-1281
void dequantize_q1_0(const uint8_t* data, size_t nbytes, float* out) {
    size_t nb = nbytes / 18, oi = 0;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 18;
        float d = rd_f16(b);
        for (int by = 0; by < 16; by++) {
            uint8_t byte = b[2 + by];
            for (int k = 0; k < 8; k++) out[oi++] = ((byte >> k) & 1) ? d : -d;
        }
    }
}

// src/gguf.rs:1283-1300
void dequantize_q2_0(const uint8_t* data, size_t nbytes, float* out) {
    size_t nb = nbytes / 34, oi = 0;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * 34;
        float d = rd_f16(b);
        for (int by = 0; by < 32; by++) {
            uint8_t byte = b[2 + by];
            for (int k = 0; k < 4; k++) {
                int8_t slot = (int8_t)((byte >> (k * 2)) & 3);
                out[oi++] = (float)(int8_t)(slot - 1) * d;
            }
        }
    }
}

// Row dequantizers that the reference spells a second time with a different
// loop structure (src/gguf.rs:6211-6261 Q4_K, 6264-6305 Q6_K, 6308-6319 Q8_0).
// Restated separately so a test can show both spellings give identical bits.
void dequantize_row_q4k(const uint8_t* data, float* out, size_t n_out) {
    size_t blocks = n_out / QK_K;
    for (size_t blk = 0; blk < blocks; blk++) {
        const uint8_t* b = data + blk * 144;
        float d = rd_f16(b), dmin = rd_f16(b + 2);
        const uint8_t* sr = b + 4; const uint8_t* qs = b + 16;
        uint8_t scales[8], mins[8];
        for (int i = 0; i < 4; i++) { scales[i] = sr[i] & 0x3F; mins[i] = sr[i + 4] & 0x3F; }
        for (int i = 0; i < 4; i++) {
            scales[4 + i] = (uint8_t)((sr[8 + i] & 0xF) | ((sr[i] >> 6) << 4));
            mins[4 + i] = (uint8_t)((sr[8 + i] >> 4) | ((sr[4 + i] >> 6) << 4));
        }
        for (int is = 0; is < 8; is++) {
            float sc = d * (float)scales[is], mn = dmin * (float)mins[is];
            for (int l = 0; l < 32; l++) {
                int byte_idx = (is / 2) * 32 + l;
                uint8_t qi = (is % 2 == 0) ? (qs[byte_idx] & 0xF) : (qs[byte_idx] >> 4);
                out[blk * QK_K + is * 32 + l] = sc * (float)qi - mn;
            }
        }
    }
}

void dequantize_row_q6k(const uint8_t* data, float* out, size_t n_out) {
    size_t blocks = n_out / QK_K;
    for (size_t blk = 0; blk < blocks; blk++) {
        const uint8_t* b = data + blk * 210;
        float d = rd_f16(b + 208);
        int8_t aux8[QK_K];
        q6k_unpack(b, b + 128, aux8);
        for (int is = 0; is < 16; is++) {
            float scale = d * (float)(int8_t)b[192 + is];
            for (int l = 0; l < 16; l++) out[blk * QK_K + is * 16 + l] = scale * (float)aux8[is * 16 + l];
        }
    }
}

// ── Q8_K activation quantizer ───────────────────────────────────────────────
// src/gguf.rs:1315-1319
inline int nearest_int(float fval) {
    float val = fval + 12582912.0f;
    int i = (int)f32_bits(val);
    return (i & 0x007fffff) - 0x00400000;
}

// src/gguf.rs:1323-1374. Output is structure-of-arrays: d[nb], qs[nb*256], bsums[nb*16].
void quantize_row_q8_k(const float* x, size_t n, float* d, int8_t* qs, int16_t* bsums) {
    size_t nb = n / QK_K;
    for (size_t i = 0; i < nb; i++) {
        const float* xb = x + i * QK_K;
        float amax = 0.0f, max_val = 0.0f;
        for (int j = 0; j < QK_K; j++) {
            float av = std::fabs(xb[j]);
            if (av > amax) { amax = av; max_val = xb[j]; }
        }
        int8_t* q = qs + i * QK_K; int16_t* bs = bsums + i * 16;
        if (amax == 0.0f) {
            d[i] = 0.0f; std::memset(q, 0, QK_K); std::memset(bs, 0, 32);
            continue;
        }
        float iscale = 128.0f / max_val;
        for (int j = 0; j < QK_K; j++) {
            int v = nearest_int(iscale * xb[j]);
            q[j] = (int8_t)std::min(std::max(v, -128), 127);
        }
        for (int j = 0; j < 16; j++) {
            int sum = 0;
            for (int ii = 0; ii < 16; ii++) sum += q[j * 16 + ii];
            bs[j] = (int16_t)sum;
        }
        d[i] = 1.0f / iscale;
    }
}

// ── per-block integer dot kernels (scalar fallbacks = ground truth) ─────────
// src/gguf.rs:3201-3251
float q4k_q8k_dot(const uint8_t* blk, float d8, const int8_t* q8, const int16_t* bsums) {
    const uint32_t KMASK1 = 0x3f3f3f3f, KMASK2 = 0x0f0f0f0f, KMASK3 = 0x03030303;
    float d = rd_f16(blk), dmin = rd_f16(blk + 2);
    const uint8_t* q4 = blk + 16;
    uint8_t aux8[QK_K];
    for (int g = 0; g < 4; g++)
        for (int l = 0; l < 32; l++) {
            aux8[g * 64 + l] = q4[g * 32 + l] & 0xF;
            aux8[g * 64 + 32 + l] = q4[g * 32 + l] >> 4;
        }
    uint32_t utmp[4];
    std::memcpy(utmp, blk + 4, 12);
    utmp[3] = ((utmp[2] >> 4) & KMASK2) | (((utmp[1] >> 6) & KMASK3) << 4);
    uint32_t uaux = utmp[1] & KMASK1;
    utmp[1] = (utmp[2] & KMASK2) | (((utmp[0] >> 6) & KMASK3) << 4);
    utmp[2] = uaux;
    utmp[0] &= KMASK1;
    uint8_t scales[8], mins[8];
    std::memcpy(scales, &utmp[0], 8);
    std::memcpy(mins, &utmp[2], 8);
    int32_t sumi = 0;
    for (int j = 0; j < 16; j++) sumi += (int32_t)bsums[j] * (int32_t)mins[j / 2];
    int32_t total = 0;
    for (int is = 0; is < 8; is++) {
        int32_t dot = 0;
        for (int l = 0; l < 32; l++) dot += (int32_t)aux8[is * 32 + l] * (int32_t)q8[is * 32 + l];
        total += (int32_t)scales[is] * dot;
    }
    return d * d8 * (float)total - dmin * d8 * (float)sumi;
}

// src/gguf.rs:3369-3410
float q5k_q8k_dot(const uint8_t* blk, float d8, const int8_t* q8, const int16_t* /*bsums*/) {
    float d = rd_f16(blk), dmin = rd_f16(blk + 2);
    const uint8_t* sr = blk + 4; const uint8_t* qh = blk + 16; const uint8_t* qs = blk + 48;
    float sumf = 0.0f;
    int is = 0, qo = 0, q8o = 0;
    for (int im = 0; im < 4; im++) {
        uint8_t sc1, m1, sc2, m2;
        get_scale_min_k4(is, sr, &sc1, &m1);
        get_scale_min_k4(is + 1, sr, &sc2, &m2);
        int32_t dot1 = 0, sum1 = 0;
        for (int l = 0; l < 32; l++) {
            int32_t hbit = (qh[l] >> (im * 2)) & 1;
            int32_t q = (int32_t)(qs[qo + l] & 0xF) | (hbit << 4);
            dot1 += q * (int32_t)q8[q8o + l];
            sum1 += (int32_t)q8[q8o + l];
        }
        sumf += d * (float)sc1 * (float)dot1 - dmin * (float)m1 * (float)sum1;
        int32_t dot2 = 0, sum2 = 0;
        for (int l = 0; l < 32; l++) {
            int32_t hbit = (qh[l] >> (im * 2 + 1)) & 1;
            int32_t q = (int32_t)(qs[qo + l] >> 4) | (hbit << 4);
            dot2 += q * (int32_t)q8[q8o + 32 + l];
            sum2 += (int32_t)q8[q8o + 32 + l];
        }
        sumf += d * (float)sc2 * (float)dot2 - dmin * (float)m2 * (float)sum2;
        qo += 32; q8o += 64; is += 2;
    }
    return sumf * d8;
}

// src/gguf.rs:3282-3319
float q6k_q8k_dot(const uint8_t* blk, float d8, const int8_t* q8, const int16_t* /*bsums*/) {
    float d = rd_f16(blk + 208);
    int8_t aux8[QK_K];
    q6k_unpack(blk, blk + 128, aux8);
    int32_t total = 0;
    for (int is = 0; is < 16; is++) {
        int32_t scale = (int32_t)(int8_t)blk[192 + is];
        int32_t dot = 0;
        for (int l = 0; l < 16; l++) dot += (int32_t)aux8[is * 16 + l] * (int32_t)q8[is * 16 + l];
        total += scale * dot;
    }
    return d * d8 * (float)total;
}

typedef float (*kdot_fn)(const uint8_t*, float, const int8_t*, const int16_t*);

// Row loop of src/gguf.rs:3677-3688 (Q4_K), 3537-3547 (Q5_K), 4077-4123 (Q6_K):
// sequential f32 sum of the per-block results.
void kquant_matvec_preq(kdot_fn dot, int bb, const uint8_t* data, size_t rows, size_t cols,
                        const float* d8, const int8_t* q8, const int16_t* bsums, float* y) {
    size_t nb = cols / QK_K, row_bytes = nb * bb;
    for (size_t r = 0; r < rows; r++) {
        const uint8_t* rd = data + r * row_bytes;
        float sumf = 0.0f;
        for (size_t bi = 0; bi < nb; bi++)
            sumf += dot(rd + bi * bb, d8[bi], q8 + bi * QK_K, bsums + bi * 16);
        y[r] = sumf;
    }
}

// src/gguf.rs:3855-3871 (scalar arm of q8_0_matvec; f32 activations)
void q8_0_matvec(const float* x, const uint8_t* data, size_t rows, size_t cols, float* y) {
    size_t nb = cols / QK8_0, row_bytes = nb * 34;
    for (size_t r = 0; r < rows; r++) {
        const uint8_t* rd = data + r * row_bytes;
        float acc = 0.0f;
        for (size_t bi = 0; bi < nb; bi++) {
            float d = rd_f16(rd + bi * 34);
            for (int l = 0; l < QK8_0; l++) {
                float w = d * (float)(int8_t)rd[bi * 34 + 2 + l];
                acc += w * x[bi * QK8_0 + l];
            }
        }
        y[r] = acc;
    }
}

// src/gguf.rs:4464-4475 (the branch taken on every non-aarch64 target) and :4495-4506.
void g128_matvec(uint32_t type, const float* x, const uint8_t* data, size_t nbytes, size_t rows,
                 size_t cols, float* y) {
    size_t row_bytes = nbytes / rows;
    std::vector<float> row(cols);
    for (size_t r = 0; r < rows; r++) {
        if (type == T_Q1_0) dequantize_q1_0(data + r * row_bytes, row_bytes, row.data());
        else dequantize_q2_0(data + r * row_bytes, row_bytes, row.data());
        float acc = 0.0f;
        for (size_t i = 0; i < cols; i++) acc += row[i] * x[i];
        y[r] = acc;
    }
}

// src/gguf.rs:5374-5399. Planes are flattened to [rows][ceil(cols/8)].
float ternary_dot_row_scalar(const uint8_t* pos, const uint8_t* neg, float scale, size_t cols,
                             const float* x) {
    float pos_sum = 0.0f, neg_sum = 0.0f;
    size_t nbytes = (cols + 7) / 8;
    for (size_t b = 0; b < nbytes; b++) {
        uint8_t pm = pos[b], nm = neg[b];
        if ((pm | nm) == 0) continue;
        for (int bit = 0; bit < 8; bit++) {
            size_t idx = b * 8 + bit;
            if (idx >= cols) break;
            float p = (float)((pm >> bit) & 1), n = (float)((nm >> bit) & 1);
            pos_sum += p * x[idx];
            neg_sum += n * x[idx];
        }
    }
    return scale * (pos_sum - neg_sum);
}

// src/gguf.rs:6130-6164. active/sign are [rows][blocks_per_row] u16 each.
float sparse_ternary_dot_scalar(const uint16_t* active, const uint16_t* sign, float scale,
                                size_t blocks_per_row, const float* x) {
    float sum = 0.0f;
    for (size_t blk = 0; blk < blocks_per_row; blk++) {
        uint16_t a = active[blk];
        if (a == 0) continue;
        uint16_t s = sign[blk];
        size_t base = blk * 16;
        uint16_t m = a & (uint16_t)~s;
        while (m) { int bit = __builtin_ctz(m); sum += x[base + bit]; m &= (uint16_t)(m - 1); }
        m = a & s;
        while (m) { int bit = __builtin_ctz(m); sum -= x[base + bit]; m &= (uint16_t)(m - 1); }
    }
    return scale * sum;
}

// src/llama3.rs:5767
inline float silu(float x) { return x / (1.0f + std::exp(-x)); }

// ── model glue (src/llama3.rs) ──────────────────────────────────────────────
// rms_norm, src/llama3.rs:5244-5256
void rms_norm(const float* x, const float* w, float eps, float* out, size_t n) {
    double ss = 0.0;
    for (size_t i = 0; i < n; i++) ss += (double)x[i] * (double)x[i];
    float mean = (float)(ss / (double)n);
    float scale = 1.0f / std::sqrt(mean + eps);
    for (size_t i = 0; i < n; i++) out[i] = x[i] * scale * w[i];
}

// apply_rope / apply_rope_neox, src/llama3.rs:5323-5333, 5367-5378
void apply_rope(float* v, size_t pos, size_t head_dim, float theta, bool neox) {
    if (!neox) {
        for (size_t i = 0; i < head_dim; i += 2) {
            float freq = 1.0f / std::pow(theta, (float)i / (float)head_dim);
            float angle = (float)pos * freq;
            float sn = std::sin(angle), cs = std::cos(angle);
            float x0 = v[i], x1 = v[i + 1];
            v[i] = x0 * cs - x1 * sn;
            v[i + 1] = x0 * sn + x1 * cs;
        }
    } else {
        size_t half = head_dim / 2;
        for (size_t i = 0; i < half; i++) {
            float freq = 1.0f / std::pow(theta, 2.0f * (float)i / (float)head_dim);
            float angle = (float)pos * freq;
            float sn = std::sin(angle), cs = std::cos(angle);
            float x0 = v[i], x1 = v[i + half];
            v[i] = x0 * cs - x1 * sn;
            v[i + half] = x0 * sn + x1 * cs;
        }
    }
}

// gqa_attention, default two-pass branch, src/llama3.rs:5560-5689 (no sliding window, no softcap).
// kc / vc: this layer's cache, [pos][kv_dim].
void gqa_attention(const float* q, const float* kc, const float* vc, size_t pos, size_t num_heads,
                   size_t num_kv_heads, size_t head_dim, float* out) {
    size_t seq_len = pos + 1, per_kv = num_heads / num_kv_heads, kv_dim = num_kv_heads * head_dim;
    float inv_sqrt_d = 1.0f / std::sqrt((float)head_dim);
    std::fill(out, out + num_heads * head_dim, 0.0f);
    std::vector<float> scores(seq_len);
    for (size_t h = 0; h < num_heads; h++) {
        size_t kvh = h / per_kv;
        const float* qh = q + h * head_dim;
        for (size_t t = 0; t < seq_len; t++) {
            const float* k = kc + t * kv_dim + kvh * head_dim;
            float acc = 0.0f;
            for (size_t d = 0; d < head_dim; d++) acc += qh[d] * k[d];
            scores[t] = acc * inv_sqrt_d;
        }
        float mx = -INFINITY;
        for (size_t t = 0; t < seq_len; t++) mx = std::max(mx, scores[t]);
        float sum = 0.0f;
        for (size_t t = 0; t < seq_len; t++) { scores[t] = std::exp(scores[t] - mx); sum += scores[t]; }
        if (sum > 0.0f) { float inv = 1.0f / sum; for (size_t t = 0; t < seq_len; t++) scores[t] *= inv; }
        for (size_t t = 0; t < seq_len; t++) {
            const float* v = vc + t * kv_dim + kvh * head_dim;
            float w = scores[t];
            for (size_t d = 0; d < head_dim; d++) out[h * head_dim + d] += w * v[d];
        }
    }
}

}  // namespace

// Plain-C description of a model for orc_llama_forward (shared with the CUDA tests through ctypes).
extern "C" {
struct OrcLayer {
    const uint8_t *q, *k, *v, *o, *gate, *up, *down;
    uint32_t tq, tk, tv, to, tgate, tup, tdown;   // GGML type ids
    const float *attn_norm, *ffn_norm;
};
struct OrcModel {
    uint32_t num_layers, hidden, ffn, num_heads, num_kv_heads, head_dim, vocab, max_seq;
    float theta, eps;
    uint32_t neox;
    const OrcLayer* layers;
    const uint8_t* emb_q8_0;      // [vocab][hidden] Q8_0
    const float* out_norm;
    const uint8_t* out;           // [vocab][hidden]
    uint32_t tout;
    float *kcache, *vcache;       // [layer][max_seq][kv_dim], written at `pos`
};
}

namespace {

// Model tensors in the in-memory ternary packing (TernaryMatrix, src/gguf.rs:5198) travel as one blob:
// pos planes [rows][ceil(cols/8)] | neg planes | f32 scale per row; type id T_TERNARY (not a GGML id).
constexpr uint32_t T_TERNARY = 1000;
size_t mat_bytes(uint32_t t, size_t rows, size_t cols) {
    if (t == T_TERNARY) return rows * (2 * ((cols + 7) / 8) + 4);
    return rows * (cols / elements_per_block(t)) * block_bytes(t);
}
int ternary_blob_matvec(const uint8_t* blob, size_t rows, size_t cols, const float* x, float* y) {
    const size_t pb = (cols + 7) / 8;
    const uint8_t* pos = blob;
    const uint8_t* neg = blob + rows * pb;
    std::vector<float> scales(rows);
    std::memcpy(scales.data(), blob + 2 * rows * pb, rows * 4);
    for (size_t r = 0; r < rows; r++) y[r] = ternary_dot_row_scalar(pos + r * pb, neg + r * pb, scales[r], cols, x);
    return 0;
}

// Llama branch of Llama3Model::forward_with_layer_hook (src/llama3.rs:13681-13687, 14167-14613).
// MV(type, x, data, nbytes, rows, cols, y) = WeightRef::matvec; MVP(..., d8, q8, bs, y) = matvec_preq.
// Tensors of type T_TERNARY take the forward_ternary skeleton instead (src/llama3.rs:16960-17062): the same
// layer sequence with ternary_matvec on f32 activations everywhere, no Q8_K step.
template <class MV, class MVP>
int llama_forward(const OrcModel& m, uint32_t token, uint32_t pos, float* logits, MV mv_g, MVP mvp_g) {
    auto mv = [&](uint32_t t, const float* x, const uint8_t* d, size_t nb, size_t r, size_t c, float* y) {
        return t == T_TERNARY ? ternary_blob_matvec(d, r, c, x, y) : mv_g(t, x, d, nb, r, c, y);
    };
    const float* cur_norm = nullptr;   // f32 vector behind the current Q8_K blocks
    auto mvp = [&](uint32_t t, const uint8_t* d, size_t nb, size_t r, size_t c, const float* d8, const int8_t* q8,
                   const int16_t* bs, float* y) {
        return t == T_TERNARY ? ternary_blob_matvec(d, r, c, cur_norm, y) : mvp_g(t, d, nb, r, c, d8, q8, bs, y);
    };
    const size_t H = m.hidden, F = m.ffn, hd = m.head_dim, q_dim = (size_t)m.num_heads * hd, kv_dim = (size_t)m.num_kv_heads * hd;
    if (token >= m.vocab || pos >= m.max_seq || H % QK_K) return -1;
    std::vector<float> hidden(H), norm(H), q(q_dim), k(kv_dim), v(kv_dim), attn(q_dim), o(H), gate(F), up(F), down(H);
    dequantize_q8_0(m.emb_q8_0 + (size_t)token * (H / 32) * 34, (H / 32) * 34, hidden.data());
    const size_t nb = H / QK_K;
    std::vector<float> d8(nb); std::vector<int8_t> q8(nb * QK_K); std::vector<int16_t> bs(nb * 16);
    for (uint32_t l = 0; l < m.num_layers; l++) {
        const OrcLayer& L = m.layers[l];
        float* kc = m.kcache + (size_t)l * m.max_seq * kv_dim;
        float* vc = m.vcache + (size_t)l * m.max_seq * kv_dim;
        rms_norm(hidden.data(), L.attn_norm, m.eps, norm.data(), H);
        cur_norm = norm.data();
        quantize_row_q8_k(norm.data(), H, d8.data(), q8.data(), bs.data());   // once for q, k, v (:14206)
        if (mvp(L.tq, L.q, mat_bytes(L.tq, q_dim, H), q_dim, H, d8.data(), q8.data(), bs.data(), q.data())) return -2;
        if (mvp(L.tk, L.k, mat_bytes(L.tk, kv_dim, H), kv_dim, H, d8.data(), q8.data(), bs.data(), k.data())) return -2;
        if (mvp(L.tv, L.v, mat_bytes(L.tv, kv_dim, H), kv_dim, H, d8.data(), q8.data(), bs.data(), v.data())) return -2;
        for (uint32_t h = 0; h < m.num_heads; h++) apply_rope(q.data() + h * hd, pos, hd, m.theta, m.neox != 0);
        for (uint32_t h = 0; h < m.num_kv_heads; h++) apply_rope(k.data() + h * hd, pos, hd, m.theta, m.neox != 0);
        std::memcpy(kc + (size_t)pos * kv_dim, k.data(), kv_dim * 4);
        std::memcpy(vc + (size_t)pos * kv_dim, v.data(), kv_dim * 4);
        gqa_attention(q.data(), kc, vc, pos, m.num_heads, m.num_kv_heads, hd, attn.data());
        if (mv(L.to, attn.data(), L.o, mat_bytes(L.to, H, q_dim), H, q_dim, o.data())) return -2;
        for (size_t i = 0; i < H; i++) hidden[i] += o[i];
        rms_norm(hidden.data(), L.ffn_norm, m.eps, norm.data(), H);
        quantize_row_q8_k(norm.data(), H, d8.data(), q8.data(), bs.data());   // once for gate, up (:14519)
        if (mvp(L.tgate, L.gate, mat_bytes(L.tgate, F, H), F, H, d8.data(), q8.data(), bs.data(), gate.data())) return -2;
        if (mvp(L.tup, L.up, mat_bytes(L.tup, F, H), F, H, d8.data(), q8.data(), bs.data(), up.data())) return -2;
        for (size_t i = 0; i < F; i++) gate[i] = silu(gate[i]) * up[i];
        if (mv(L.tdown, gate.data(), L.down, mat_bytes(L.tdown, H, F), H, F, down.data())) return -2;
        for (size_t i = 0; i < H; i++) hidden[i] += down[i];
    }
    rms_norm(hidden.data(), m.out_norm, m.eps, norm.data(), H);
    if (mv(m.tout, norm.data(), m.out, mat_bytes(m.tout, m.vocab, H), m.vocab, H, logits)) return -2;
    return 0;
}

}  // namespace

extern "C" {


float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
int orc_block_bytes(uint32_t t) { return block_bytes(t); }
int orc_elements_per_block(uint32_t t) { return elements_per_block(t); }
void orc_get_scale_min_k4(int j, const uint8_t* scales, uint8_t* sc, uint8_t* m) {
    get_scale_min_k4(j, scales, sc, m);
}

// Block dequantizers (src/gguf.rs:903-1300). Returns 0, or -1 for a type outside the path.
int orc_dequantize(uint32_t type, const uint8_t* data, size_t nbytes, float* out) {
    switch (type) {
        case T_Q4_K: dequantize_q4_k(data, nbytes, out); return 0;
        case T_Q5_K: dequantize_q5_k(data, nbytes, out); return 0;
        case T_Q6_K: dequantize_q6_k(data, nbytes, out); return 0;
        case T_Q8_0: dequantize_q8_0(data, nbytes, out); return 0;
        case T_Q1_0: dequantize_q1_0(data, nbytes, out); return 0;
        case T_Q2_0: dequantize_q2_0(data, nbytes, out); return 0;
        default: return -1;
    }
}

// dequantize_weight_row (src/gguf.rs:6168-6195): the public row dispatcher. Types it does
// not list (Q1_0, Q2_0 among them) produce zeros, as in the reference.
int orc_dequantize_weight_row(uint32_t type, const uint8_t* data, float* out, size_t n_out) {
    switch (type) {
        case T_Q4_K: dequantize_row_q4k(data, out, n_out); return 0;
        case T_Q5_K: dequantize_q5_k(data, n_out / QK_K * 176, out); return 0;
        case T_Q6_K: dequantize_row_q6k(data, out, n_out); return 0;
        case T_Q8_0: dequantize_q8_0(data, n_out / QK8_0 * 34, out); return 0;
        default: std::fill(out, out + n_out, 0.0f); return 0;
    }
}

void orc_quantize_row_q8_k(const float* x, size_t n, float* d, int8_t* qs, int16_t* bsums) {
    quantize_row_q8_k(x, n, d, qs, bsums);
}

float orc_kquant_block_dot(uint32_t type, const uint8_t* blk, float d8, const int8_t* q8,
                           const int16_t* bsums) {
    switch (type) {
        case T_Q4_K: return q4k_q8k_dot(blk, d8, q8, bsums);
        case T_Q5_K: return q5k_q8k_dot(blk, d8, q8, bsums);
        case T_Q6_K: return q6k_q8k_dot(blk, d8, q8, bsums);
        default: return NAN;
    }
}

// quantized_matvec_preq (src/gguf.rs:4574-4608).
int orc_matvec_preq(uint32_t type, const uint8_t* data, size_t nbytes, size_t rows, size_t cols,
                    const float* d8, const int8_t* q8, const int16_t* bsums, float* y) {
    switch (type) {
        case T_Q4_K: kquant_matvec_preq(q4k_q8k_dot, 144, data, rows, cols, d8, q8, bsums, y); return 0;
        case T_Q5_K: kquant_matvec_preq(q5k_q8k_dot, 176, data, rows, cols, d8, q8, bsums, y); return 0;
        case T_Q6_K: kquant_matvec_preq(q6k_q8k_dot, 210, data, rows, cols, d8, q8, bsums, y); return 0;
        case T_Q1_0: case T_Q2_0: {
            // src/gguf.rs:4593-4605: the Q8_K blocks are turned back into f32 first.
            std::vector<float> xf(cols, 0.0f);
            size_t nb = cols / QK_K + ((cols % QK_K) ? 1 : 0);
            for (size_t b = 0; b < nb; b++)
                for (int i = 0; i < QK_K; i++) {
                    if (b * QK_K + i >= cols) break;
                    xf[b * QK_K + i] = d8[b] * (float)q8[b * QK_K + i];
                }
            g128_matvec(type, xf.data(), data, nbytes, rows, cols, y);
            return 0;
        }
        default: return -1;
    }
}

// quantized_matvec (src/gguf.rs:4214-4245) for the formats on the path.
int orc_matvec(uint32_t type, const float* x, const uint8_t* data, size_t nbytes, size_t rows,
               size_t cols, float* y) {
    switch (type) {
        case T_Q4_K: case T_Q5_K: case T_Q6_K: {
            size_t nb = cols / QK_K;
            std::vector<float> d8(nb); std::vector<int8_t> q8(nb * QK_K); std::vector<int16_t> bs(nb * 16);
            quantize_row_q8_k(x, nb * QK_K, d8.data(), q8.data(), bs.data());
            return orc_matvec_preq(type, data, nbytes, rows, cols, d8.data(), q8.data(), bs.data(), y);
        }
        case T_Q8_0: q8_0_matvec(x, data, rows, cols, y); return 0;
        case T_Q1_0: case T_Q2_0: g128_matvec(type, x, data, nbytes, rows, cols, y); return 0;
        default: return -1;
    }
}

// ternary_matvec (src/gguf.rs:5303-5321) over flattened bit planes.
void orc_ternary_matvec(const uint8_t* pos, const uint8_t* neg, const float* scales, size_t rows,
                        size_t cols, const float* x, float* y) {
    size_t pb = (cols + 7) / 8;
    for (size_t r = 0; r < rows; r++)
        y[r] = ternary_dot_row_scalar(pos + r * pb, neg + r * pb, scales[r], cols, x);
}

// sparse_ternary_matvec, non-aarch64 arm (src/gguf.rs:5870-5885).
void orc_sparse_ternary_matvec(const uint16_t* active, const uint16_t* sign, const float* scales,
                               size_t rows, size_t cols, const float* x, float* y) {
    size_t bpr = (cols + 15) / 16;
    for (size_t r = 0; r < rows; r++)
        y[r] = sparse_ternary_dot_scalar(active + r * bpr, sign + r * bpr, scales[r], bpr, x);
}

// packed_2bit construction of SparseTernaryMatrix::from_rows (src/gguf.rs:5560-5583):
// 4 bytes per 16-column block, element j of a byte in bits 2j..2j+1, 00=0 01=+1 11=-1.
void orc_sparse_pack_2bit(const uint16_t* active, const uint16_t* sign, size_t rows, size_t cols,
                          uint8_t* packed) {
    size_t bpr = (cols + 15) / 16;
    for (size_t r = 0; r < rows; r++)
        for (size_t blk = 0; blk < bpr; blk++) {
            uint16_t a = active[r * bpr + blk], s = sign[r * bpr + blk];
            for (int byte = 0; byte < 4; byte++) {
                uint8_t pk = 0;
                for (int j = 0; j < 4; j++) {
                    int bit = byte * 4 + j;
                    uint8_t code = ((a >> bit) & 1) == 0 ? 0 : (((s >> bit) & 1) == 0 ? 1 : 3);
                    pk |= (uint8_t)(code << (j * 2));
                }
                packed[(r * bpr + blk) * 4 + byte] = pk;
            }
        }
}

// TernaryRow::from_f32 (src/gguf.rs:5207-5245) for one row; returns the scale.
float orc_ternarize_row(const float* w, size_t cols, float threshold_ratio, uint8_t* pos, uint8_t* neg) {
    size_t nbytes = (cols + 7) / 8;
    std::memset(pos, 0, nbytes); std::memset(neg, 0, nbytes);
    float s = 0.0f;
    for (size_t i = 0; i < cols; i++) s += std::fabs(w[i]);
    float mean_abs = s / (float)cols;
    float threshold = threshold_ratio * mean_abs;
    float abs_sum = 0.0f; size_t nz = 0;
    for (size_t i = 0; i < cols; i++) {
        if (std::fabs(w[i]) > threshold) {
            uint8_t bit = (uint8_t)(1u << (i % 8));
            if (w[i] > 0.0f) pos[i / 8] |= bit; else neg[i / 8] |= bit;
            abs_sum += std::fabs(w[i]); nz++;
        }
    }
    return nz > 0 ? abs_sum / (float)nz : 0.0f;
}

// SparseTernaryRow::from_ternary_row (src/gguf.rs:5451-5507) for one row; returns the scale.
float orc_sparsify_row(const uint8_t* pos, const uint8_t* neg, float dense_scale, const float* w,
                       size_t cols, size_t n_keep, uint16_t* active, uint16_t* sign) {
    size_t nblk = (cols + 15) / 16;
    double abs_sum = 0.0; size_t nz = 0;
    for (size_t blk = 0; blk < nblk; blk++) {
        active[blk] = 0; sign[blk] = 0;
        size_t base = blk * 16, end = std::min(base + 16, cols), len = end - base;
        std::vector<std::pair<size_t, float>> cand;
        for (size_t i = 0; i < len; i++) {
            size_t g = base + i; uint8_t bit = (uint8_t)(1u << (g % 8));
            if ((pos[g / 8] & bit) || (neg[g / 8] & bit)) cand.push_back({i, std::fabs(w[g])});
        }
        // Rust's sort_by is stable; descending by magnitude.
        std::stable_sort(cand.begin(), cand.end(),
                         [](const auto& a, const auto& b) { return a.second > b.second; });
        if (cand.size() > std::min(n_keep, len)) cand.resize(std::min(n_keep, len));
        for (auto& c : cand) {
            size_t g = base + c.first; uint8_t bit = (uint8_t)(1u << (g % 8));
            active[blk] |= (uint16_t)(1u << c.first);
            if (neg[g / 8] & bit) sign[blk] |= (uint16_t)(1u << c.first);
            abs_sum += (double)c.second; nz++;
        }
    }
    return nz > 0 ? (float)(abs_sum / (double)nz) : dense_scale;
}

// Fused SwiGLU as the CPU model computes it (src/llama3.rs:14519-14534): both projections
// from the same pre-quantized Q8_K input, then gate[i] = silu(gate[i]) * up[i].
int orc_swiglu(uint32_t type, const float* x, const uint8_t* gate, const uint8_t* up, size_t nbytes,
               size_t rows, size_t cols, float* y) {
    std::vector<float> g(rows), u(rows);
    int rc = orc_matvec(type, x, gate, nbytes, rows, cols, g.data());
    if (rc) return rc;
    rc = orc_matvec(type, x, up, nbytes, rows, cols, u.data());
    if (rc) return rc;
    for (size_t i = 0; i < rows; i++) y[i] = silu(g[i]) * u[i];
    return 0;
}

// forward_ternary's FFN (src/llama3.rs:17040-17048): separate gate / up, then silu * up.
void orc_ternary_swiglu(const uint8_t* gpos, const uint8_t* gneg, const float* gsc,
                        const uint8_t* upos, const uint8_t* uneg, const float* usc, size_t rows,
                        size_t cols, const float* x, float* y) {
    std::vector<float> g(rows), u(rows);
    orc_ternary_matvec(gpos, gneg, gsc, rows, cols, x, g.data());
    orc_ternary_matvec(upos, uneg, usc, rows, cols, x, u.data());
    for (size_t i = 0; i < rows; i++) y[i] = silu(g[i]) * u[i];
}

float orc_silu(float x) { return silu(x); }

void orc_rms_norm(const float* x, const float* w, float eps, float* out, size_t n) { rms_norm(x, w, eps, out, n); }
void orc_apply_rope(float* v, size_t pos, size_t head_dim, float theta, int neox) { apply_rope(v, pos, head_dim, theta, neox != 0); }
void orc_gqa_attention(const float* q, const float* kc, const float* vc, size_t pos, size_t num_heads, size_t num_kv_heads,
                       size_t head_dim, float* out) {
    gqa_attention(q, kc, vc, pos, num_heads, num_kv_heads, head_dim, out);
}

// One token through the Llama branch of the CPU forward; appends K/V at `pos` in m->kcache / vcache.
int orc_llama_forward(const OrcModel* m, uint32_t token, uint32_t pos, float* logits) {
    return llama_forward(*m, token, pos, logits,
                         [](uint32_t t, const float* x, const uint8_t* d, size_t nb, size_t r, size_t c, float* y) {
                             return orc_matvec(t, x, d, nb, r, c, y);
                         },
                         [](uint32_t t, const uint8_t* d, size_t nb, size_t r, size_t c, const float* d8, const int8_t* q8,
                            const int16_t* bs, float* y) { return orc_matvec_preq(t, d, nb, r, c, d8, q8, bs, y); });
}

}  // extern "C"
