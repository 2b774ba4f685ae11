// Per-format decode for the streaming matvec: how one lane turns one "unit" of a weight row
// (read from shared memory) and its register-resident activations into a partial dot product.
// Byte layouts and arithmetic follow ALICE-LLM src/gguf.rs (cited per format).
#pragma once
#include "gemv_stream.cuh"

namespace alice {

__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ldg64(const void* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }

// 6-bit scale/min pair of sub-blocks 2g, 2g+1 from the 12-byte K4 header words (s0,s1,s2);
// same bit surgery as get_scale_min_k4 (src/gguf.rs:794-802). Returns sc0 | sc1<<8 and m0 | m1<<8.
__device__ __forceinline__ void k4_scale_pair(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t g, uint32_t& sc01,
                                              uint32_t& m01) {
    const uint32_t sh = (g & 1u) * 16u;
    const uint32_t a = s0 >> sh, b = s1 >> sh, c = s2 >> sh;
    const uint32_t sc_lo = a & 0x3f3fu, m_lo = b & 0x3f3fu;
    const uint32_t sc_hi = (c & 0x0f0fu) | ((a >> 2) & 0x3030u);
    const uint32_t m_hi = ((c >> 4) & 0x0f0fu) | ((b >> 2) & 0x3030u);
    sc01 = g < 2 ? sc_lo : sc_hi;
    m01 = g < 2 ? m_lo : m_hi;
}

// Q8_K activations of one 64-element group (sub-blocks 2g and 2g+1 of a 256-block).
struct ActGroup64 {
    uint4 p0, p1, p2, p3;  // q8[0..16), [16..32), [32..48), [48..64) of the group
    int bs0, bs1;          // sum of q8 over [0..32) and [32..64)
    float d8;              // Q8_K block scale
};

// The Q8_K blocks sit in shared memory (fetched once per CTA) or, for shapes where that copy is not possible, in
// global memory written by an earlier kernel: generic loads serve both (a kernel boundary lies in between).
__device__ __forceinline__ void load_act_group64(ActGroup64& r, const Q8KView& v, uint32_t u, bool valid) {
    if (!valid) { r = ActGroup64{}; return; }
    const uint4* q = reinterpret_cast<const uint4*>(v.qs + (size_t)u * 64);
    r.p0 = q[0]; r.p1 = q[1]; r.p2 = q[2]; r.p3 = q[3];
    const uint2 b = *reinterpret_cast<const uint2*>(v.bsums + (size_t)u * 4);
    r.bs0 = (int)(short)(b.x & 0xffff) + (int)(short)(b.x >> 16);
    r.bs1 = (int)(short)(b.y & 0xffff) + (int)(short)(b.y >> 16);
    r.d8 = v.d[u >> 2];
}

// ── Q4_K: 144-byte block = d f16, dmin f16, 12 B scales, 128 B nibbles (src/gguf.rs:903-939).
// Unit = one 64-weight group g of a block: 32 nibble bytes; low nibbles are sub-block 2g,
// high nibbles sub-block 2g+1. Integer dot against Q8_K as in q4k_q8k_dot (src/gguf.rs:3201-3251).
struct FmtQ4K {
    static constexpr uint32_t BLOCK_BYTES = 144, UNITS_PER_BLOCK = 4;
    using Act = ActGroup64;
    static constexpr bool USES_Q8K = true;
    __device__ static void load_act(Act& r, const StreamArgs&, const Q8KView& q8, const float*, bool, uint32_t u, bool valid) { load_act_group64(r, q8, u, valid); }
    __device__ static float unit(uint32_t rb, uint32_t u, const Act& x, const StreamArgs& a) {
        const uint32_t g = u & 3u;
        const uint32_t blk = rb + (u >> 2) * BLOCK_BYTES;
        const uint4 h = lds128(blk);
        const uint4 q0 = lds128(blk + 16 + g * 32), q1 = lds128(blk + 32 + g * 32);
        uint32_t sc01, m01;
        k4_scale_pair(h.y, h.z, h.w, g, sc01, m01);
        constexpr uint32_t LO = 0x0f0f0f0fu, HI = 0xf0f0f0f0u;
        int dlo = 0, dhi = 0;  // dhi accumulates 16 * (high nibble dot)
        dlo = dp4a_us(q0.x & LO, x.p0.x, dlo); dhi = dp4a_us(q0.x & HI, x.p2.x, dhi);
        dlo = dp4a_us(q0.y & LO, x.p0.y, dlo); dhi = dp4a_us(q0.y & HI, x.p2.y, dhi);
        dlo = dp4a_us(q0.z & LO, x.p0.z, dlo); dhi = dp4a_us(q0.z & HI, x.p2.z, dhi);
        dlo = dp4a_us(q0.w & LO, x.p0.w, dlo); dhi = dp4a_us(q0.w & HI, x.p2.w, dhi);
        dlo = dp4a_us(q1.x & LO, x.p1.x, dlo); dhi = dp4a_us(q1.x & HI, x.p3.x, dhi);
        dlo = dp4a_us(q1.y & LO, x.p1.y, dlo); dhi = dp4a_us(q1.y & HI, x.p3.y, dhi);
        dlo = dp4a_us(q1.z & LO, x.p1.z, dlo); dhi = dp4a_us(q1.z & HI, x.p3.z, dhi);
        dlo = dp4a_us(q1.w & LO, x.p1.w, dlo); dhi = dp4a_us(q1.w & HI, x.p3.w, dhi);
        const int tot = (int)(sc01 & 0xff) * dlo + (int)(sc01 >> 8) * (dhi >> 4);
        const int smin = (int)(m01 & 0xff) * x.bs0 + (int)(m01 >> 8) * x.bs1;
        const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
        return (dm.x * x.d8) * (float)tot - (dm.y * x.d8) * (float)smin;
    }
    __device__ static float finish(float v, const StreamArgs&, const float*, uint32_t) { return v; }
};

// ── Q5_K: 176-byte block = d, dmin, 12 B scales, qh[32], qs[128] (src/gguf.rs:949-988);
// fifth bit of element 64g+l is bit 2g of qh[l], of 64g+32+l bit 2g+1. Dot as q5k_q8k_dot
// (src/gguf.rs:3369-3410): per 32-weight sub-block d*sc*dot - dmin*m*sum, times the Q8_K scale.
struct FmtQ5K {
    static constexpr uint32_t BLOCK_BYTES = 176, UNITS_PER_BLOCK = 4;
    using Act = ActGroup64;
    static constexpr bool USES_Q8K = true;
    __device__ static void load_act(Act& r, const StreamArgs&, const Q8KView& q8, const float*, bool, uint32_t u, bool valid) { load_act_group64(r, q8, u, valid); }
    __device__ static float unit(uint32_t rb, uint32_t u, const Act& x, const StreamArgs& a) {
        const uint32_t g = u & 3u;
        const uint32_t blk = rb + (u >> 2) * BLOCK_BYTES;
        const uint4 h = lds128(blk);
        const uint4 h0 = lds128(blk + 16), h1 = lds128(blk + 32);
        const uint4 q0 = lds128(blk + 48 + g * 32), q1 = lds128(blk + 64 + g * 32);
        uint32_t sc01, m01;
        k4_scale_pair(h.y, h.z, h.w, g, sc01, m01);
        constexpr uint32_t LO = 0x0f0f0f0fu, B0 = 0x01010101u;
        const uint32_t s = 2 * g;
        int dlo = 0, dhi = 0;
#define ALICE_Q5(qw, hw, pl, ph)                                                   \
        dlo = dp4a_us(((qw) & LO) | ((((hw) >> s) & B0) << 4), (pl), dlo);         \
        dhi = dp4a_us((((qw) >> 4) & LO) | ((((hw) >> (s + 1)) & B0) << 4), (ph), dhi);
        ALICE_Q5(q0.x, h0.x, x.p0.x, x.p2.x) ALICE_Q5(q0.y, h0.y, x.p0.y, x.p2.y)
        ALICE_Q5(q0.z, h0.z, x.p0.z, x.p2.z) ALICE_Q5(q0.w, h0.w, x.p0.w, x.p2.w)
        ALICE_Q5(q1.x, h1.x, x.p1.x, x.p3.x) ALICE_Q5(q1.y, h1.y, x.p1.y, x.p3.y)
        ALICE_Q5(q1.z, h1.z, x.p1.z, x.p3.z) ALICE_Q5(q1.w, h1.w, x.p1.w, x.p3.w)
#undef ALICE_Q5
        const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
        const float a0 = (dm.x * (float)(sc01 & 0xff)) * (float)dlo - (dm.y * (float)(m01 & 0xff)) * (float)x.bs0;
        const float a1 = (dm.x * (float)(sc01 >> 8)) * (float)dhi - (dm.y * (float)(m01 >> 8)) * (float)x.bs1;
        return (a0 + a1) * x.d8;
    }
    __device__ static float finish(float v, const StreamArgs&, const float*, uint32_t) { return v; }
};

// ── Q6_K: 210-byte block = ql[128], qh[64], 16 int8 scales, d f16 (src/gguf.rs:1205-1246);
// blocks are only 2-byte aligned. Unit = (half n, 8 columns l0..l0+7): 8 bytes of ql at 64n+l0,
// 8 at 64n+32+l0 and 8 of qh at 32n+l0 give the 32 weights at 128n + {0,32,64,96} + l0..l0+7.
// q8k dot as q6k_q8k_dot (src/gguf.rs:3282-3319); the -32 bias is folded in through the sum of
// the unit's q8 values.
struct FmtQ6K {
    static constexpr uint32_t BLOCK_BYTES = 210, UNITS_PER_BLOCK = 8;
    struct Act {
        uint2 p[4];  // q8 at 128n + 32j + l0 .. +8
        int s[4];    // their sums
        float d8;
    };
    static constexpr bool USES_Q8K = true;
    __device__ static void load_act(Act& r, const StreamArgs&, const Q8KView& v, const float*, bool, uint32_t u, bool valid) {
        if (!valid) { r = Act{}; return; }
        const uint32_t b = u >> 3, n = (u >> 2) & 1u, l0 = (u & 3u) * 8u;
        const int8_t* q = v.qs + (size_t)b * 256 + n * 128 + l0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            r.p[j] = *reinterpret_cast<const uint2*>(q + 32 * j);
            r.s[j] = dp4a_ss(0x01010101u, r.p[j].x, dp4a_ss(0x01010101u, r.p[j].y, 0));
        }
        r.d8 = v.d[b];
    }
    __device__ static float unit(uint32_t rb, uint32_t u, const Act& x, const StreamArgs& a) {
        const uint32_t n = (u >> 2) & 1u, l0 = (u & 3u) * 8u;
        const uint32_t blk = rb + (u >> 3) * BLOCK_BYTES;
        const uint32_t sh = (blk & 2u) * 8u;      // blocks start on 2-byte boundaries
        const uint32_t base = blk & ~3u;          // l0, 64n, 128+32n are multiples of 4
        uint32_t w0, w1, w2;
        const uint32_t oa = base + 64 * n + l0;
        w0 = lds32(oa); w1 = lds32(oa + 4); w2 = lds32(oa + 8);
        const uint32_t a0 = __funnelshift_r(w0, w1, sh), a1 = __funnelshift_r(w1, w2, sh);
        w0 = lds32(oa + 32); w1 = lds32(oa + 36); w2 = lds32(oa + 40);
        const uint32_t b0 = __funnelshift_r(w0, w1, sh), b1 = __funnelshift_r(w1, w2, sh);
        const uint32_t oh = base + 128 + 32 * n + l0;
        w0 = lds32(oh); w1 = lds32(oh + 4); w2 = lds32(oh + 8);
        const uint32_t h0 = __funnelshift_r(w0, w1, sh), h1 = __funnelshift_r(w1, w2, sh);
        // four int8 scales: index 8n + l0/16 + {0,2,4,6}
        const uint32_t os = base + 192 + 8 * n;
        w0 = lds32(os); w1 = lds32(os + 4); w2 = lds32(os + 8);
        const uint32_t sel = (l0 >> 4) * 8u;
        const uint32_t s01 = __funnelshift_r(w0, w1, sh) >> sel, s23 = __funnelshift_r(w1, w2, sh) >> sel;
        const int sc0 = (int)(int8_t)(s01 & 0xff), sc1 = (int)(int8_t)((s01 >> 16) & 0xff);
        const int sc2 = (int)(int8_t)(s23 & 0xff), sc3 = (int)(int8_t)((s23 >> 16) & 0xff);
        const uint32_t dw = lds16((blk + 208));
        constexpr uint32_t LO = 0x0f0f0f0fu, H2 = 0x30303030u;
        int d0 = 0, d1 = 0, d2 = 0, d3 = 0;
        d0 = dp4a_us((a0 & LO) | ((h0 << 4) & H2), x.p[0].x, d0);
        d0 = dp4a_us((a1 & LO) | ((h1 << 4) & H2), x.p[0].y, d0);
        d1 = dp4a_us((b0 & LO) | ((h0 << 2) & H2), x.p[1].x, d1);
        d1 = dp4a_us((b1 & LO) | ((h1 << 2) & H2), x.p[1].y, d1);
        d2 = dp4a_us(((a0 >> 4) & LO) | (h0 & H2), x.p[2].x, d2);
        d2 = dp4a_us(((a1 >> 4) & LO) | (h1 & H2), x.p[2].y, d2);
        d3 = dp4a_us(((b0 >> 4) & LO) | ((h0 >> 2) & H2), x.p[3].x, d3);
        d3 = dp4a_us(((b1 >> 4) & LO) | ((h1 >> 2) & H2), x.p[3].y, d3);
        const int tot = sc0 * (d0 - 32 * x.s[0]) + sc1 * (d1 - 32 * x.s[1]) + sc2 * (d2 - 32 * x.s[2]) +
                        sc3 * (d3 - 32 * x.s[3]);
        return (f16_bits_to_f32(dw) * x.d8) * (float)tot;
    }
    __device__ static float finish(float v, const StreamArgs&, const float*, uint32_t) { return v; }
};

// ── Q8_0: 34-byte block = d f16 + 32 int8, f32 activations (src/gguf.rs:3855-3871).
// Unit = half a block (16 weights); 16 activations stay in registers.
struct FmtQ8_0 {
    static constexpr uint32_t BLOCK_BYTES = 34, UNITS_PER_BLOCK = 2;
    struct Act { float x[16]; };
    static constexpr bool USES_Q8K = false;
    __device__ static void load_act(Act& r, const StreamArgs&, const Q8KView&, const float* x, bool cg, uint32_t u, bool valid) {
#pragma unroll
        for (int i = 0; i < 16; i++) r.x[i] = 0.0f;
        if (!valid) return;
        const float4* p = reinterpret_cast<const float4*>(x + (size_t)u * 16);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 v = cg ? __ldcg(p + i) : p[i];
            r.x[4 * i] = v.x; r.x[4 * i + 1] = v.y; r.x[4 * i + 2] = v.z; r.x[4 * i + 3] = v.w;
        }
    }
    __device__ static float unit(uint32_t rb, uint32_t u, const Act& x, const StreamArgs& a) {
        const uint32_t blk = rb + (u >> 1) * BLOCK_BYTES;
        const uint32_t qa = blk + 2 + (u & 1u) * 16;  // 2-byte aligned
        const uint32_t sh = (qa & 2u) * 8u, base = qa & ~3u;
        uint32_t w[5];
#pragma unroll
        for (int i = 0; i < 5; i++) w[i] = lds32(base + 4 * i);
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t q = __funnelshift_r(w[i], w[i + 1], sh) ^ 0x80808080u;  // bias to unsigned
            // 0x4B000000 | byte is the float 8388608 + byte; subtracting 8388736 leaves the int8 value
            acc = fmaf(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7650)) - 8388736.0f, x.x[4 * i], acc);
            acc = fmaf(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7651)) - 8388736.0f, x.x[4 * i + 1], acc);
            acc = fmaf(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7652)) - 8388736.0f, x.x[4 * i + 2], acc);
            acc = fmaf(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7653)) - 8388736.0f, x.x[4 * i + 3], acc);
        }
        return f16_bits_to_f32(lds16(blk)) * acc;
    }
    __device__ static float finish(float v, const StreamArgs&, const float*, uint32_t) { return v; }
};

// Adds x[i] for every set bit i of a 32-bit mask.
__device__ __forceinline__ float masked_sum32(uint32_t m, const float* x) {
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        if (m & (1u << i)) s0 += x[i];
        if (m & (2u << i)) s1 += x[i + 1];
    }
    return s0 + s1;
}

struct Act32 { float x[32]; float sum; };
__device__ __forceinline__ void load_act32(Act32& r, const float* x, bool cg, uint32_t u, uint32_t cols, bool valid) {
    r.sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const uint32_t c = u * 32 + i;
        r.x[i] = (valid && c < cols) ? (cg ? __ldcg(x + c) : x[c]) : 0.0f;
        r.sum += r.x[i];
    }
}

// ── Q1_0: 18-byte block = d f16 + 128 sign bits, LSB first, 1 -> +d, 0 -> -d (src/gguf.rs:1264-1281).
// Unit = 32 weights (4 bytes of a block): d * (2 * sum_{bit=1} x - sum x).
struct FmtQ1_0 {
    static constexpr uint32_t BLOCK_BYTES = 18, UNITS_PER_BLOCK = 4;
    using Act = Act32;
    static constexpr bool USES_Q8K = false;
    __device__ static void load_act(Act& r, const StreamArgs& a, const Q8KView&, const float* x, bool cg, uint32_t u, bool valid) { load_act32(r, x, cg, u, a.cols, valid); }
    __device__ static float unit(uint32_t rb, uint32_t u, const Act& x, const StreamArgs& a) {
        const uint32_t blk = rb + (u >> 2) * BLOCK_BYTES;
        const uint32_t bits = lds32_u2(blk + 2 + (u & 3u) * 4);
        return f16_bits_to_f32(lds16(blk)) * (2.0f * masked_sum32(bits, x.x) - x.sum);
    }
    __device__ static float finish(float v, const StreamArgs&, const float*, uint32_t) { return v; }
};

// ── Q2_0: 34-byte block = d f16 + 128 two-bit slots, value (slot - 1) * d (src/gguf.rs:1283-1300).
// Unit = 16 weights (one 32-bit word of slots).
struct FmtQ2_0 {
    static constexpr uint32_t BLOCK_BYTES = 34, UNITS_PER_BLOCK = 8;
    struct Act { float x[16]; float sum; };
    static constexpr bool USES_Q8K = false;
    __device__ static void load_act(Act& r, const StreamArgs&, const Q8KView&, const float* x, bool cg, uint32_t u, bool valid) {
        r.sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            r.x[i] = valid ? (cg ? __ldcg(x + (size_t)u * 16 + i) : x[(size_t)u * 16 + i]) : 0.0f;
            r.sum += r.x[i];
        }
    }
    __device__ static float unit(uint32_t rb, uint32_t u, const Act& x, const StreamArgs& a) {
        const uint32_t blk = rb + (u >> 3) * BLOCK_BYTES;
        const uint32_t w = lds32_u2(blk + 2 + (u & 7u) * 4);
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) acc = fmaf((float)((w >> (2 * i)) & 3u), x.x[i], acc);
        return f16_bits_to_f32(lds16(blk)) * (acc - x.sum);
    }
    __device__ static float finish(float v, const StreamArgs&, const float*, uint32_t) { return v; }
};

// ── Ternary bit planes (TernaryRow, src/gguf.rs:5190-5195; dot src/gguf.rs:5374-5399).
// Device row = [pos plane | neg plane], each plane 4*ceil(cols/32) bytes, bit i%8 of byte i/8.
// y = scale_row * (sum_{pos} x - sum_{neg} x). Unit = 32 columns.
struct FmtTernary {
    static constexpr uint32_t UNIT_COLS = 32;
    using Act = Act32;
    static constexpr bool USES_Q8K = false;
    __device__ static void load_act(Act& r, const StreamArgs& a, const Q8KView&, const float* x, bool cg, uint32_t u, bool valid) { load_act32(r, x, cg, u, a.cols, valid); }
    __device__ static float unit(uint32_t rb, uint32_t u, const Act& x, const StreamArgs& a) {
        const uint32_t pm = lds32(rb + 4 * u), nm = lds32(rb + (a.row_bytes >> 1) + 4 * u);
        return masked_sum32(pm, x.x) - masked_sum32(nm, x.x);
    }
    __device__ static float finish(float v, const StreamArgs&, const float* aux, uint32_t row) { return __ldg(aux + row) * v; }
};

// ── Sparse ternary, packed 2-bit codes (SparseTernaryMatrix::packed_2bit, src/gguf.rs:5560-5583):
// 4 bytes per 16 columns, element j in bits 2j..2j+1, 00 = 0, 01 = +1, 11 = -1.
// y = scale_row * sum(+-x) as in sparse_ternary_dot_scalar (src/gguf.rs:6130-6164). Unit = 32 columns.
struct FmtSparseTernary {
    static constexpr uint32_t UNIT_COLS = 32;
    using Act = Act32;
    static constexpr bool USES_Q8K = false;
    __device__ static void load_act(Act& r, const StreamArgs& a, const Q8KView&, const float* x, bool cg, uint32_t u, bool valid) { load_act32(r, x, cg, u, a.cols, valid); }
    __device__ static float half(uint32_t w, const float* x) {
        const uint32_t act = w & 0x55555555u, neg = (w >> 1) & act;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (act & (1u << (2 * i))) s += (neg & (1u << (2 * i))) ? -x[i] : x[i];
        }
        return s;
    }
    __device__ static float unit(uint32_t rb, uint32_t u, const Act& x, const StreamArgs& a) {
        const uint32_t w0 = lds32(rb + 8 * u);
        const uint32_t w1 = (8 * u + 4 < a.row_bytes) ? lds32(rb + 8 * u + 4) : 0u;
        return half(w0, x.x) + half(w1, x.x + 16);
    }
    __device__ static float finish(float v, const StreamArgs&, const float* aux, uint32_t row) { return __ldg(aux + row) * v; }
};

}  // namespace alice
