// Batched (2..8 input vectors) fused dequantize + matvec for the K-quant formats on the int8 tensor cores.
//
// The speculative-verify step feeds 4..8 tokens through every projection. The weights are streamed and unpacked ONCE:
// a warp owns a tile of 16 rows (mma M), the unpacked 4/5/6-bit quants of a 32-element sub-block are the A operand
// (u8, 16 rows x 32) of one mma.sync m16n8k32 and the Q8_K int8 activations of the up-to-8 input vectors are the B
// operand (32 x 8 columns = the batch), so one instruction yields the integer sub-block dot products of 16 rows x 8
// vectors. Per-sub-block scales are applied to the int32 results as in q4k_q8k_dot (src/gguf.rs:3201-3251); the
// min term sum_is m[is] * bsum[is] is one more pair of small MMAs (A = the 6-bit mins, B = the sub-block sums of the
// activations split into two signed base-64 digits). The reference does the same on the GPU with
// dequant_matvec_q4k_batch4.wgsl / swiglu_fused_q4k_batch4.wgsl (weights decoded once for 4 inputs, in f32).
//
// Same producer / ring / partial-sum machinery as the batch-1 kernels, with row-wise staging: the shared-memory row
// stride is padded to 32 mod 128 bytes so the 64-bit A loads of a half warp (4 rows x 4 column slices) hit 16 different
// bank pairs. The activations of all vectors sit in shared memory too (row stride cols + 32 for the same reason).
#pragma once
#include "gemv_mma.cuh"
#include "gemv_stream.cuh"

namespace alice {

struct KqActs {
    uint32_t qs;      // shared address of int8 [8][xs]
    uint32_t xs;      // bytes between vectors
    uint32_t d;       // shared address of f32 [8][nb]
    uint32_t bsd;     // shared address of s8 [8][nb][16]: base-64 digits of the 8 sub-block (32-element) sums, low digits in bytes 0..7, high in 8..15
    uint32_t bs16;    // shared address of s8 [8][nb][32]: base-64 digits of the 16 sub-block (16-element) sums, low 0..15, high 16..31 (Q6_K)
    uint32_t nb;
};
__host__ __device__ constexpr uint32_t kq_acts_bytes(uint32_t cols) {
    return ((8u * (cols + 32u) + 127u) & ~127u) + ((8u * (cols / 256u) * 4u + 127u) & ~127u) + ((8u * (cols / 256u) * 16u + 127u) & ~127u) +
           ((8u * (cols / 256u) * 32u + 127u) & ~127u);
}

__device__ __forceinline__ void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

// Brings the Q8_K blocks of the `batch` input vectors (global memory, prepared by an earlier kernel) into shared memory
// in the layout above; columns past `batch` are zero. Run by the NCW consumer warps.
static __device__ __noinline__ void kq_stage_acts(const StreamArgs& a, uint8_t* area, KqActs& x) {
    const uint32_t tid = threadIdx.x, nb = a.cols / QK_K, cols = a.cols, B = a.batch;
    const uint32_t vs = a.x_stride, vnb = a.x_stride / QK_K;   // strides between input vectors in global memory
    const uint32_t xs = cols + 32u;
    uint8_t* qs = area;
    float* d = reinterpret_cast<float*>(area + ((8u * xs + 127u) & ~127u));
    int8_t* bsd = reinterpret_cast<int8_t*>(reinterpret_cast<uint8_t*>(d) + ((8u * nb * 4u + 127u) & ~127u));
    int8_t* bs16 = bsd + ((8u * nb * 16u + 127u) & ~127u);
    for (uint32_t i = tid; i < 8u * (cols / 16u); i += NCW * 32) {
        const uint32_t c = i / (cols / 16u), j = i % (cols / 16u);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (c < B) v = *reinterpret_cast<const uint4*>(a.q8.qs + (size_t)c * vs + (size_t)j * 16);
        *reinterpret_cast<uint4*>(qs + (size_t)c * xs + (size_t)j * 16) = v;
    }
    for (uint32_t i = tid; i < 8u * nb; i += NCW * 32) {
        const uint32_t c = i / nb, b = i % nb;
        d[i] = c < B ? a.q8.d[(size_t)c * vnb + b] : 0.0f;
    }
    for (uint32_t i = tid; i < 8u * nb * 16u; i += NCW * 32) {
        const uint32_t c = i / (nb * 16u), r = i % (nb * 16u), b = r / 16u, is = r % 16u;
        int v16 = 0, v32 = 0;
        if (c < B) {
            const int16_t* bs = a.q8.bsums + ((size_t)c * vnb + b) * 16;
            v16 = bs[is];
            if (is < 8) v32 = (int)bs[2 * is] + (int)bs[2 * is + 1];
        }
        // signed base-64 digits: v = 64 * hi + lo, lo in [-32, 31]
        const int lo16 = ((v16 + 32) & 63) - 32, hi16 = (v16 - lo16) >> 6;
        bs16[((size_t)c * nb + b) * 32 + is] = (int8_t)lo16;
        bs16[((size_t)c * nb + b) * 32 + 16 + is] = (int8_t)hi16;
        if (is < 8) {
            const int lo = ((v32 + 32) & 63) - 32, hi = (v32 - lo) >> 6;
            bsd[((size_t)c * nb + b) * 16 + is] = (int8_t)lo;
            bsd[((size_t)c * nb + b) * 16 + 8 + is] = (int8_t)hi;
        }
    }
    x.qs = smem_u32(qs); x.xs = xs; x.d = smem_u32(d); x.bsd = smem_u32(bsd); x.bs16 = smem_u32(bs16); x.nb = nb;
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
}

// 6-bit scales (sc) and mins (m) of a K4 header as four words of four bytes each: sub-blocks 0..3 and 4..7
// (get_scale_min_k4, src/gguf.rs:794-802).
__device__ __forceinline__ void k4_unpack(const uint4& h, uint32_t& sc_lo, uint32_t& sc_hi, uint32_t& m_lo, uint32_t& m_hi) {
    sc_lo = h.y & 0x3f3f3f3fu;
    m_lo = h.z & 0x3f3f3f3fu;
    sc_hi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
    m_hi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
}

// Thread (g = lane / 4, t = lane % 4) of a tile holds outputs (row g, vectors 2t, 2t+1) and (row g + 8, vectors 2t, 2t+1).
// k slot mapping of one 32-element sub-block: slots 4t..4t+3 = elements 8t..8t+3, slots 16+4t..16+4t+3 = elements
// 8t+4..8t+7, so a thread's A bytes are 8 consecutive weight bytes and its B bytes 8 consecutive activations.

// ── Q4_K / Q5_K tile: blocks [b_lo, b_hi) of rows rowA (g) and rowB (g + 8).
template <bool Q5>
struct KqK4 {
    static constexpr uint32_t BLOCK_BYTES = Q5 ? 176 : 144;
    __device__ static void tile(uint32_t rowA, uint32_t rowB, uint32_t b_lo, uint32_t b_hi, const KqActs& x, uint32_t lane, float (&acc)[4]) {
        const uint32_t t = lane & 3u, g = lane >> 2;
        constexpr uint32_t LO = 0x0f0f0f0fu;
        constexpr uint32_t QS = Q5 ? 48u : 16u;
        for (uint32_t blk = b_lo; blk < b_hi; blk++) {
            const uint32_t pA = rowA + blk * BLOCK_BYTES, pB = rowB + blk * BLOCK_BYTES;
            const uint4 hA = lds128(pA), hB = lds128(pB);
            uint32_t scA_lo, scA_hi, mA_lo, mA_hi, scB_lo, scB_hi, mB_lo, mB_hi;
            k4_unpack(hA, scA_lo, scA_hi, mA_lo, mA_hi);
            k4_unpack(hB, scB_lo, scB_hi, mB_lo, mB_hi);
            uint2 qhA = make_uint2(0u, 0u), qhB = make_uint2(0u, 0u);
            if (Q5) { qhA = lds64(pA + 16 + 8 * t); qhB = lds64(pB + 16 + 8 * t); }
            const uint32_t xq = x.qs + g * x.xs + blk * 256 + 8 * t;
            int tot[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 wA = lds64(pA + QS + 32 * j + 8 * t), wB = lds64(pB + QS + 32 * j + 8 * t);
                const uint2 xl = lds64(xq + 64 * j), xh = lds64(xq + 64 * j + 32);
                uint32_t a0 = wA.x & LO, a1 = wB.x & LO, a2 = wA.y & LO, a3 = wB.y & LO;
                uint32_t e0 = (wA.x >> 4) & LO, e1 = (wB.x >> 4) & LO, e2 = (wA.y >> 4) & LO, e3 = (wB.y >> 4) & LO;
                if (Q5) {
                    constexpr uint32_t B0 = 0x01010101u;
                    a0 |= ((qhA.x >> (2 * j)) & B0) << 4; a1 |= ((qhB.x >> (2 * j)) & B0) << 4;
                    a2 |= ((qhA.y >> (2 * j)) & B0) << 4; a3 |= ((qhB.y >> (2 * j)) & B0) << 4;
                    e0 |= ((qhA.x >> (2 * j + 1)) & B0) << 4; e1 |= ((qhB.x >> (2 * j + 1)) & B0) << 4;
                    e2 |= ((qhA.y >> (2 * j + 1)) & B0) << 4; e3 |= ((qhB.y >> (2 * j + 1)) & B0) << 4;
                }
                int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
                mma_u8s8_k32(cl, a0, a1, a2, a3, xl.x, xl.y);
                mma_u8s8_k32(ch, e0, e1, e2, e3, xh.x, xh.y);
                // sub-blocks 2j (low nibbles) and 2j + 1 (high nibbles)
                const uint32_t wAs = j < 2 ? scA_lo : scA_hi, wBs = j < 2 ? scB_lo : scB_hi;
                const int sA0 = (int)((wAs >> (16 * (j & 1))) & 0xffu), sA1 = (int)((wAs >> (16 * (j & 1) + 8)) & 0xffu);
                const int sB0 = (int)((wBs >> (16 * (j & 1))) & 0xffu), sB1 = (int)((wBs >> (16 * (j & 1) + 8)) & 0xffu);
                tot[0] += sA0 * cl[0] + sA1 * ch[0]; tot[1] += sA0 * cl[1] + sA1 * ch[1];
                tot[2] += sB0 * cl[2] + sB1 * ch[2]; tot[3] += sB0 * cl[3] + sB1 * ch[3];
            }
            // min term: sum over the 8 sub-blocks of m[is] * (sum of the 32 activations), k slots 0..7 = sub-blocks
            const uint32_t aM0 = t == 0 ? mA_lo : (t == 1 ? mA_hi : 0u), aM1 = t == 0 ? mB_lo : (t == 1 ? mB_hi : 0u);
            const uint32_t dg = x.bsd + (g * x.nb + blk) * 16;
            const uint32_t bl = t < 2 ? lds32(dg + 4 * t) : 0u, bh = t < 2 ? lds32(dg + 8 + 4 * t) : 0u;
            int sm[4] = {0, 0, 0, 0};
            mma_u8s8_k16(sm, aM0, aM1, bh);
#pragma unroll
            for (int i = 0; i < 4; i++) sm[i] <<= 6;
            mma_u8s8_k16(sm, aM0, aM1, bl);
            const float2 dmA = __half22float2(*reinterpret_cast<const __half2*>(&hA.x));
            const float2 dmB = __half22float2(*reinterpret_cast<const __half2*>(&hB.x));
            const float d80 = ldsf(x.d + ((2 * t) * x.nb + blk) * 4), d81 = ldsf(x.d + ((2 * t + 1) * x.nb + blk) * 4);
            acc[0] += (dmA.x * d80) * (float)tot[0] - (dmA.y * d80) * (float)sm[0];
            acc[1] += (dmA.x * d81) * (float)tot[1] - (dmA.y * d81) * (float)sm[1];
            acc[2] += (dmB.x * d80) * (float)tot[2] - (dmB.y * d80) * (float)sm[2];
            acc[3] += (dmB.x * d81) * (float)tot[3] - (dmB.y * d81) * (float)sm[3];
        }
    }
};

// ── Q6_K tile: 210-byte blocks ql[128] qh[64] sc[16] d (src/gguf.rs:1205-1246); integer dot as q6k_q8k_dot
// (src/gguf.rs:3282-3319): sum over the 16 sub-blocks of 16 elements of sc[is] * dot(q - 32, q8). The -32 goes through
// the activation sums: sc * (dot(q, q8) - 32 * bsum[is]); the bias sum_is sc[is] * bsum[is] is a pair of s8 x s8 MMAs.
// Blocks are only 2-byte aligned in a row, so words are fetched as two aligned halves and funnel-shifted.
// A thread covers, for half n and 16-column group i, the columns l = 16 i + 4 t .. + 3 of all four quadrants: one ql
// word serves quadrants 0 / 2 (low / high nibbles), one serves 1 / 3, one qh word carries the two high bits of all four.
struct KqQ6K {
    static constexpr uint32_t BLOCK_BYTES = 210;
    __device__ static void tile(uint32_t rowA, uint32_t rowB, uint32_t b_lo, uint32_t b_hi, const KqActs& x, uint32_t lane, float (&acc)[4]) {
        const uint32_t t = lane & 3u, g = lane >> 2;
        constexpr uint32_t LO = 0x0f0f0f0fu, H2 = 0x30303030u;
        for (uint32_t blk = b_lo; blk < b_hi; blk++) {
            const uint32_t pA = rowA + blk * BLOCK_BYTES, pB = rowB + blk * BLOCK_BYTES;
            const uint32_t xq = x.qs + g * x.xs + blk * 256 + 4 * t;
            int tot[4] = {0, 0, 0, 0};
#pragma unroll
            for (int n = 0; n < 2; n++) {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint32_t o = 16 * i + 4 * t;
                    const uint32_t lA0 = lds32_u2(pA + 64 * n + o), lA1 = lds32_u2(pA + 64 * n + 32 + o), hA = lds32_u2(pA + 128 + 32 * n + o);
                    const uint32_t lB0 = lds32_u2(pB + 64 * n + o), lB1 = lds32_u2(pB + 64 * n + 32 + o), hB = lds32_u2(pB + 128 + 32 * n + o);
                    // the four int8 scales of this (n, i): index 8n + i + {0, 2, 4, 6}
                    const uint32_t sa = lds32_u2(pA + 192 + 8 * n) >> (8 * i), sa2 = lds32_u2(pA + 196 + 8 * n) >> (8 * i);
                    const uint32_t sb = lds32_u2(pB + 192 + 8 * n) >> (8 * i), sb2 = lds32_u2(pB + 196 + 8 * n) >> (8 * i);
                    const int scA[4] = {(int)(int8_t)(sa & 0xff), (int)(int8_t)((sa >> 16) & 0xff), (int)(int8_t)(sa2 & 0xff), (int)(int8_t)((sa2 >> 16) & 0xff)};
                    const int scB[4] = {(int)(int8_t)(sb & 0xff), (int)(int8_t)((sb >> 16) & 0xff), (int)(int8_t)(sb2 & 0xff), (int)(int8_t)((sb2 >> 16) & 0xff)};
                    const uint32_t qa[4] = {(lA0 & LO) | ((hA << 4) & H2), (lA1 & LO) | ((hA << 2) & H2), ((lA0 >> 4) & LO) | (hA & H2), ((lA1 >> 4) & LO) | ((hA >> 2) & H2)};
                    const uint32_t qb[4] = {(lB0 & LO) | ((hB << 4) & H2), (lB1 & LO) | ((hB << 2) & H2), ((lB0 >> 4) & LO) | (hB & H2), ((lB1 >> 4) & LO) | ((hB >> 2) & H2)};
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t bx = lds32(xq + 128 * n + 32 * q + 16 * i);
                        int c[4] = {0, 0, 0, 0};
                        mma_u8s8_k16(c, qa[q], qb[q], bx);
                        tot[0] += scA[q] * c[0]; tot[1] += scA[q] * c[1]; tot[2] += scB[q] * c[2]; tot[3] += scB[q] * c[3];
                    }
                }
            }
            // bias: 32 * sum over the 16 sub-blocks of sc[is] * bsum[is]; k slots = sub-blocks, 4t .. 4t+3 per thread
            const uint32_t aS0 = lds32_u2(pA + 192 + 4 * t), aS1 = lds32_u2(pB + 192 + 4 * t);
            const uint32_t dg = x.bs16 + (g * x.nb + blk) * 32;
            const uint32_t bl = lds32(dg + 4 * t), bh = lds32(dg + 16 + 4 * t);
            int bias[4] = {0, 0, 0, 0};
            mma_s8s8_k16(bias, aS0, aS1, bh);
#pragma unroll
            for (int i = 0; i < 4; i++) bias[i] <<= 6;
            mma_s8s8_k16(bias, aS0, aS1, bl);
            const float dA = f16_bits_to_f32(lds16(pA + 208)), dB = f16_bits_to_f32(lds16(pB + 208));
            const float d80 = ldsf(x.d + ((2 * t) * x.nb + blk) * 4), d81 = ldsf(x.d + ((2 * t + 1) * x.nb + blk) * 4);
            acc[0] += (dA * d80) * (float)(tot[0] - 32 * bias[0]);
            acc[1] += (dA * d81) * (float)(tot[1] - 32 * bias[1]);
            acc[2] += (dB * d80) * (float)(tot[2] - 32 * bias[2]);
            acc[3] += (dB * d81) * (float)(tot[3] - 32 * bias[3]);
        }
    }
};

// Shared-memory area for the partial sums of the P warps of a tile: [stage][warp][16 rows][8 vectors][gate | up]
struct KqPartials { float v[2][NCW][16][8][2]; };

// Consumer side (the NCW consumer warps). A stage holds slots * 16 rows; warp `part` of a tile covers blocks
// [nb * part / P, nb * (part + 1) / P) of every row of its tile. Returns false after an abort.
template <class T, bool SWIGLU>
__device__ __forceinline__ bool stream_consume_kq(const StreamArgs& a, StreamCtx& cx, KqPartials* pp, uint8_t* act_area) {
    StreamSmem* sm = cx.sm;
    volatile int* abort_flag = &sm->abort_flag;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t P = a.P, slots = a.slots, rps = a.rps;   // rps == 16
    const uint32_t rows_per_group = slots * rps;
    const uint32_t slot = warp / P, part = warp % P;
    KqActs x;
    kq_stage_acts(a, act_area, x);
    const uint32_t nb = a.cols / QK_K;                          // blocks of the (sub-)row this launch covers
    const uint32_t b_lo = nb * part / P, b_hi = nb * (part + 1) / P;
    const uint32_t t = lane & 3u, gid = lane >> 2;

    const uint32_t g0 = (uint32_t)(((uint64_t)a.groups * blockIdx.x) / gridDim.x);
    const uint32_t g1 = (uint32_t)(((uint64_t)a.groups * (blockIdx.x + 1)) / gridDim.x);
    for (uint32_t g = g0; g < g1; g++) {
        const uint32_t s = cx.cc % cx.nstages, ph = (cx.cc / cx.nstages) & 1;
        cx.cc++;
        uint32_t sg = 0;
        while (sg + 1 < a.nseg && g >= a.seg_g0[sg + 1]) sg++;
        const uint32_t seg_rows = a.seg_rows[sg];
        const uint32_t r0 = (g - a.seg_g0[sg]) * rows_per_group;
        const uint32_t set0 = slot * rps;
        const uint32_t nrow = r0 + set0 < seg_rows ? min(rps, seg_rows - r0 - set0) : 0;
        if (!wait_or_abort(smem_u32(&sm->full[s]), ph, abort_flag, a.status, KERR_WAIT_FULL, cx.limit)) return false;
        const uint32_t sb = cx.ring + s * cx.stage_stride + set0 * a.row_stride;
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
        if (nrow > 0) {
            // rows past nrow of a short last tile read whatever the stage holds; their results are never stored
            const uint32_t rowA = sb + gid * a.row_stride + a.row_pad, rowB = sb + (gid + 8) * a.row_stride + a.row_pad;
            T::tile(rowA, rowB, b_lo, b_hi, x, lane, acc);
            if (SWIGLU) T::tile(rowA + a.cap, rowB + a.cap, b_lo, b_hi, x, lane, up);
            if (P > 1) {
                float (*pv)[8][2] = pp->v[s & 1][warp];
                pv[gid][2 * t][0] = acc[0]; pv[gid][2 * t + 1][0] = acc[1]; pv[gid + 8][2 * t][0] = acc[2]; pv[gid + 8][2 * t + 1][0] = acc[3];
                if (SWIGLU) { pv[gid][2 * t][1] = up[0]; pv[gid][2 * t + 1][1] = up[1]; pv[gid + 8][2 * t][1] = up[2]; pv[gid + 8][2 * t + 1][1] = up[3]; }
            }
        }
        __syncwarp();
        {
            const uint32_t own0 = warp * rps;
            const bool used = P > 1 && warp < slots && r0 + own0 < seg_rows;
            if (!used && lane == 0) mbar_arrive_n(smem_u32(&sm->red[s][warp]), RED_COUNT);
        }
        if (nrow > 0) {
            if (part != 0) {
                if (lane == 0) mbar_arrive_n(smem_u32(&sm->red[s][slot]), RED_COUNT / (P - 1));
            } else {
                if (P > 1 && !wait_or_abort(smem_u32(&sm->red[s][slot]), ph, abort_flag, a.status, KERR_WAIT_PARTIALS, cx.limit)) return false;
                if (P > 1) {
#pragma unroll
                    for (int i = 0; i < 4; i++) { acc[i] = 0.f; up[i] = 0.f; }
                    for (uint32_t p = 0; p < P; p++) {
                        float (*pv)[8][2] = pp->v[s & 1][warp + p];
                        acc[0] += pv[gid][2 * t][0]; acc[1] += pv[gid][2 * t + 1][0]; acc[2] += pv[gid + 8][2 * t][0]; acc[3] += pv[gid + 8][2 * t + 1][0];
                        if (SWIGLU) { up[0] += pv[gid][2 * t][1]; up[1] += pv[gid][2 * t + 1][1]; up[2] += pv[gid + 8][2 * t][1]; up[3] += pv[gid + 8][2 * t + 1][1]; }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t rr = gid + 8 * (i >> 1), k = 2 * t + (i & 1);
                    if (rr < nrow && k < a.batch) {
                        float r = acc[i];
                        if (SWIGLU) r = silu_ref(r) * up[i];
                        const size_t yi = (size_t)k * a.y_stride + a.seg_y[sg] + r0 + set0 + rr;
                        if (a.resid != nullptr) r = __fadd_rn(__ldcg(a.resid + yi), r);
                        a.y[yi] = r;
                    }
                }
                continue;   // this warp has already released the stage
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
    }
    return true;
}

// The partial-sum area is double buffered by stage parity: a finalizer has read stage s before the producer may refill
// it (it arrives on `empty` after reading), and the helpers write their partials of the next use of the same parity only
// after that stage has landed again.
template <class T, bool SWIGLU, int CTAS>
__global__ void __launch_bounds__(STREAM_THREADS, CTAS) stream_gemv_kq_kernel(const __grid_constant__ StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    StreamSmem* sm = reinterpret_cast<StreamSmem*>(smem_raw);
    constexpr uint32_t HDR = (sizeof(StreamSmem) + 127) & ~127u;
    constexpr uint32_t PART = (sizeof(KqPartials) + 127) & ~127u;
    StreamCtx cx;
    cx.sm = sm; cx.smem_raw = smem_raw; cx.ring = smem_u32(smem_raw) + HDR + PART;
    cx.stage_stride = a.cap * (SWIGLU ? 2u : 1u); cx.nstages = a.nstages; cx.cc = 0;
    cx.limit = a.wait_limit > 0 ? a.wait_limit : WAIT_CYCLE_LIMIT;
    stream_init_ring(sm, a.nstages);
    __syncthreads();
    pdl_launch_dependents();
    if ((threadIdx.x >> 5) == NCW) {
        stream_produce_rows(a, cx);
        if ((threadIdx.x & 31) == 0 && sm->abort_flag) stream_drain(cx);
        return;
    }
    pdl_wait();
    stream_consume_kq<T, SWIGLU>(a, cx, reinterpret_cast<KqPartials*>(smem_raw + HDR), smem_raw + a.tab_off);
}

}  // namespace alice
