// Bit-plane tensor-core consumer for the 1- and 2-bit formats (Q1_0, Q2_0, ternary bit planes, sparse-ternary codes).
//
// At one or two bits per weight the CUDA-core path spends an instruction per weight per lane and is
// ALU-bound at a fraction of HBM speed. Here the raw weight bytes ARE the A operand of an int8
// mma.sync: for bit position j = 0..7 the fragment A_j = bytes & (0x01 << j) (one LOP per four
// weights, values 0 or 2^j) multiplies a B fragment that holds the activation of the element that
// bit j of each byte stands for, pre-divided by 2^j. The f32 activations are turned once per CTA into
// 26-bit fixed point (one power-of-two scale per vector) and split into four signed base-128 digits,
// which are the first four of the eight B columns; the integer accumulators of the four digit
// columns are recombined in f32. The fixed-point step costs at most 2^-20 of max|x| per element,
// far below f32 summation error at these row lengths.
//
//   S(row) = sum over set bits of x  =  kappa * sum_d 128^(3-d) * sum_{byte k, bit j} (byte_k & 2^j) * digit_d(x[8k+j] / 2^j)
//
// Q1_0 (src/gguf.rs:1264-1281, matvec :4441-4476):  y = sum_b d_b * (2 * S_b - T_b), T_b = sum of x over block b.
// Ternary planes (src/gguf.rs:5374-5399):            y = scale_row * (S_pos - S_neg).
//
// A warp owns a tile of 16 rows (mma M) and a contiguous range of 16-byte groups of the row; the P warps
// of a row set split the groups, their f32 partials meet in shared memory exactly as in the scalar path.
#pragma once
#include "gemv_stream.cuh"

namespace alice {

__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory activation table. A "group" is 16 consecutive weight bytes of a row (128 one-bit weights);
// entry (group G, digit d, quad lane t, bit j) is one 32-bit word whose byte i is digit d of
// x[8 * (16 G + 4 t + i) + j] / 2^j - exactly the B fragment register of thread (groupID d, quad lane t) for
// an m16n8k16 step over group G with mask bit j. Bits 0..3 and bits 4..7 live in two halves of the table, each
// a dense array of 16-byte records indexed (G * 4 + d) * 4 + t, so the eight lanes of a quarter warp read eight
// different records (no bank conflict) and a thread fetches its eight words with two 128-bit loads. A zero record
// follows the table for lanes whose B column must not take part in a step.
struct MmaTable {
    uint32_t words;      // shared address of the half that holds bits 0..3
    uint32_t half;       // byte distance to the half that holds bits 4..7
    uint32_t zero;       // shared address of 16 zero bytes
    uint32_t tsum;       // shared address of the per-128-element sums of x (f32), Q1_0 only
    float kappa;         // value of one fixed-point unit: S = kappa * integer sum
};
// bytes of the table for `groups` groups: two halves + zero record
__host__ __device__ constexpr uint32_t mma_table_bytes(uint32_t groups) { return groups * 512u + 16u; }

constexpr int MMA_FIX_BITS = 26;   // |x| / scale < 1 -> |fixed| < 2^26; digits of fixed >> j fit int8

// Builds the table from the f32 vector `x` (global or shared; cols a multiple of 4). All NCW consumer warps take
// part. Loads are float4 and issued TB_V at a time per thread, so a pass over x costs a few memory round trips
// instead of one per element. tsum_blocks > 0: also leave sum(x[128 b .. 128 b + 127]) for b < tsum_blocks
// (a warp's 32 float4 of one round are exactly one such block).
constexpr int TB_V = 8;

// CODE: how a weight byte maps to elements. 0: one bit per element (element 8*byte + j, bit j; Q1_0 signs, ternary
// planes). 1 / 2: two bits per element (element 4*byte + q, bits 2q and 2q+1) worth +1 and +2 (Q2_0 slots) or +1 and -2
// (sparse-ternary codes 00 = 0, 01 = +1, 11 = -1). A group is always 16 weight bytes, i.e. 128 or 64 elements.
template <int CODE>
__device__ __forceinline__ constexpr uint32_t mma_group_elems() { return CODE == 0 ? 128u : 64u; }

// four signed base-128 digits of f (|f| < 2^27) into digit records 64 bytes apart
__device__ __forceinline__ void mma_store_digits(uint8_t* w, int f) {
    const int d3 = ((f + 64) & 127) - 64; f = (f - d3) >> 7;
    const int d2 = ((f + 64) & 127) - 64; f = (f - d2) >> 7;
    const int d1 = ((f + 64) & 127) - 64; f = (f - d1) >> 7;
    w[0] = (uint8_t)f; w[64] = (uint8_t)d1; w[128] = (uint8_t)d2; w[192] = (uint8_t)d3;
}

// Bytes of the prepared activation blob of a vector of `groups` groups: digit table (two halves + zero record),
// per-128-element sums (one float per group at most), the fixed-point unit kappa. The same layout in shared memory
// (built per CTA) and in global memory (built once by mma_table_kernel and bulk-copied in). A multiple of 16.
__host__ __device__ constexpr uint32_t mma_blob_tsum_off(uint32_t groups) { return (mma_table_bytes(groups) + 15u) & ~15u; }
__host__ __device__ constexpr uint32_t mma_blob_kappa_off(uint32_t groups) { return mma_blob_tsum_off(groups) + ((groups * 4u + 15u) & ~15u); }
__host__ __device__ constexpr uint32_t mma_blob_bytes(uint32_t groups) { return mma_blob_kappa_off(groups) + 16u; }

// max |x| over the whole vector; all NCW*32 threads take part (red = NCW floats of shared memory).
static __device__ __forceinline__ float mma_vec_amax(float* red, const float* x, uint32_t nvec) {
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float amax = 0.0f;
#pragma unroll 1
    for (uint32_t base = 0; base < nvec; base += NCW * 32 * TB_V) {
        float4 v[TB_V];
#pragma unroll
        for (int k = 0; k < TB_V; k++) {
            const uint32_t i = base + k * NCW * 32 + tid;
            v[k] = i < nvec ? __ldcg(reinterpret_cast<const float4*>(x) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < TB_V; k++)
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v[k].x), fabsf(v[k].y))), fmaxf(fabsf(v[k].z), fabsf(v[k].w)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[warp] = amax;
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
    amax = 0.0f;
#pragma unroll
    for (int w = 0; w < NCW; w++) amax = fmaxf(amax, red[w]);
    return amax;
}

// Digits of the float4s [v_lo, v_hi) of x (v_lo a multiple of NCW*32, so that a warp's 32 float4 of one round are
// one 128-element block) into `table` (record of group G at G*256 in each half, the halves half_bytes apart; a caller
// that builds a slice passes a pointer moved back by the slice's first group) and their block sums into tsum[block].
template <int CODE>
static __device__ __forceinline__ void mma_build_digits(const float* x, uint32_t v_lo, uint32_t v_hi, uint8_t* table, uint32_t half_bytes,
                                                        float* tsum, uint32_t tsum_blocks, float to_fixed) {
    const uint32_t tid = threadIdx.x, lane = tid & 31;
#pragma unroll 1
    for (uint32_t base = v_lo; base < v_hi; base += NCW * 32 * TB_V) {
        float4 v[TB_V];
#pragma unroll
        for (int k = 0; k < TB_V; k++) {
            const uint32_t i = base + k * NCW * 32 + tid;
            v[k] = i < v_hi ? __ldcg(reinterpret_cast<const float4*>(x) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < TB_V; k++) {
            const uint32_t i = base + k * NCW * 32 + tid;
            if (base + k * NCW * 32 < v_hi) {     // warp-uniform: the whole warp takes part in the block sum
                float ts = (v[k].x + v[k].y) + (v[k].z + v[k].w);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
                if (lane == 0 && (i >> 5) < tsum_blocks) tsum[i >> 5] = ts;
            }
            if (i < v_hi) {
                const float xq[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
                if (CODE == 0) {
                    // this float4 is bits 4h .. 4h+3 (h = i & 1) of one weight byte
                    const uint32_t byte = i >> 1, G = byte >> 4, t = (byte >> 2) & 3u, bi = byte & 3u;
                    uint8_t* w = table + (size_t)(i & 1u) * half_bytes + ((size_t)(G * 4) * 4 + t) * 16 + bi;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int j = (int)(i & 1u) * 4 + q;
                        mma_store_digits(w + q * 4, (__float2int_rn(xq[q] * to_fixed) + ((1 << j) >> 1)) >> j);   // fixed / 2^j, to nearest
                    }
                } else {
                    // this float4 is the four elements of weight byte i: element q owns bits 2q (worth +1) and 2q+1
                    // (worth +2 or -2), so both want fixed / 2^(2q) (negated for -2); bits 0..3 live in half 0
                    const uint32_t byte = i, G = byte >> 4, t = (byte >> 2) & 3u, bi = byte & 3u;
                    uint8_t* rec = table + ((size_t)(G * 4) * 4 + t) * 16 + bi;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int sh = 2 * q;
                        const int f = (__float2int_rn(xq[q] * to_fixed) + ((1 << sh) >> 1)) >> sh;
                        uint8_t* w = rec + (size_t)(q >> 1) * half_bytes + ((2 * q) & 3) * 4;
                        mma_store_digits(w, f);
                        mma_store_digits(w + 4, CODE == 1 ? f : -f);
                    }
                }
            }
        }
    }
}

// Zeroes the part of the last group past `cols` (only a ragged ternary row has one; its weight bits there are zero,
// so the table content only has to be finite). Group indices as in mma_build_digits.
template <int CODE>
static __device__ __forceinline__ void mma_zero_tail(uint32_t cols, uint32_t groups, uint8_t* table, uint32_t half_bytes) {
    constexpr uint32_t GE = mma_group_elems<CODE>();
    for (uint32_t idx = cols + threadIdx.x; idx < groups * GE; idx += NCW * 32) {
        const uint32_t byte = CODE == 0 ? idx >> 3 : idx >> 2, G = byte >> 4, t = (byte >> 2) & 3u, bi = byte & 3u;
        uint8_t* rec = table + ((size_t)(G * 4) * 4 + t) * 16 + bi;
        if (CODE == 0) {
            const uint32_t j = idx & 7u;
            mma_store_digits(rec + (size_t)(j >> 2) * half_bytes + (j & 3u) * 4, 0);
        } else {
            const uint32_t q = idx & 3u;
            uint8_t* w = rec + (size_t)(q >> 1) * half_bytes + ((2 * q) & 3) * 4;
            mma_store_digits(w, 0);
            mma_store_digits(w + 4, 0);
        }
    }
}

// scale = 2^(exponent(amax) + 1) > amax; inf / nan inputs fall back to scale 1 (their products are garbage in the
// reference too). to_fixed turns x into 26-bit fixed point, kappa is the value of one unit.
__device__ __forceinline__ void mma_fixed_scale(float amax, float& to_fixed, float& kappa) {
    const uint32_t ebits = (__float_as_uint(amax) >> 23) & 0xffu;
    const int e = (ebits == 0u || ebits == 0xffu) ? 0 : (int)ebits - 126;
    to_fixed = ldexpf(1.0f, MMA_FIX_BITS - e);
    kappa = ldexpf(1.0f, e - MMA_FIX_BITS);
}

// The whole table, built by the NCW consumer warps of a matvec CTA in its own shared memory (the path for callers
// that give the matvec no room for a prepared copy).
template <int CODE>
static __device__ __noinline__ float mma_build_table(StreamSmem* sm, const float* x, uint32_t cols, uint8_t* table,
                                                     float* tsum, uint32_t tsum_blocks) {
    const uint32_t nvec = cols / 4;
    constexpr uint32_t GE = mma_group_elems<CODE>();
    const uint32_t groups = (cols + GE - 1) / GE;
    const uint32_t half_bytes = groups * 256;
    float to_fixed, kappa;
    mma_fixed_scale(mma_vec_amax(reinterpret_cast<float*>(sm->norm_part), x, nvec), to_fixed, kappa);
    mma_build_digits<CODE>(x, 0, nvec, table, half_bytes, tsum, tsum_blocks, to_fixed);
    mma_zero_tail<CODE>(cols, groups, table, half_bytes);
    if (threadIdx.x < 4) reinterpret_cast<uint32_t*>(table + 2 * (size_t)half_bytes)[threadIdx.x] = 0u;   // the zero record
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
    return kappa;
}

// The same table built ONCE per vector, ahead of the matvec, by a small grid: CTA b (NCW*32 threads) turns the
// elements [b * MMA_PREP_ELEMS, (b + 1) * MMA_PREP_ELEMS) into digits in shared memory and copies its slice of both
// halves (and of the block sums) to the blob in global memory with 16-byte stores; every CTA finds max |x| of the
// whole vector for itself (the vector is a few tens of KB in L2). The matvec's CTAs then fetch the blob with one bulk
// copy instead of each building the table (5120 columns: 20 KB of scattered byte stores per CTA, ~5 us on the critical
// path of every launch).
constexpr uint32_t MMA_PREP_ELEMS = 4096;   // a multiple of NCW*32*4 elements and of both group sizes
template <int CODE>
__global__ void __launch_bounds__(NCW * 32) mma_table_kernel(const float* x, uint32_t cols, uint8_t* blob, uint32_t tsum_blocks) {
    __shared__ float red[NCW];
    __shared__ __align__(16) uint8_t stage[2 * (MMA_PREP_ELEMS / mma_group_elems<CODE>()) * 256];
    __shared__ float ts[MMA_PREP_ELEMS / 128];
    pdl_launch_dependents();
    pdl_wait();   // x comes from the previous kernel; the blob may still be read by the matvec before it
    constexpr uint32_t GE = mma_group_elems<CODE>();
    const uint32_t nvec = cols / 4, groups = (cols + GE - 1) / GE, half_bytes = groups * 256;
    float to_fixed, kappa;
    mma_fixed_scale(mma_vec_amax(red, x, nvec), to_fixed, kappa);
    const uint32_t e_lo = blockIdx.x * MMA_PREP_ELEMS, e_hi = min(cols, e_lo + MMA_PREP_ELEMS);
    const uint32_t G_lo = e_lo / GE, G_hi = (e_hi + GE - 1) / GE, ng = G_hi - G_lo;   // this CTA's groups
    const uint32_t local_half = ng * 256;
    uint8_t* local = stage - (size_t)G_lo * 256;          // record of group G lands at stage + (G - G_lo) * 256
    float* local_ts = ts - e_lo / 128;
    mma_build_digits<CODE>(x, e_lo / 4, e_hi / 4, local, local_half, local_ts, tsum_blocks, to_fixed);
    if (e_hi == cols) mma_zero_tail<CODE>(cols, groups, local, local_half);
    __syncthreads();
    const uint32_t tid = threadIdx.x;
    for (uint32_t i = tid; i < ng * 16; i += NCW * 32) {   // 16-byte units of each half
        reinterpret_cast<uint4*>(blob + (size_t)G_lo * 256)[i] = reinterpret_cast<const uint4*>(stage)[i];
        reinterpret_cast<uint4*>(blob + half_bytes + (size_t)G_lo * 256)[i] = reinterpret_cast<const uint4*>(stage + local_half)[i];
    }
    float* tsum_g = reinterpret_cast<float*>(blob + mma_blob_tsum_off(groups));
    for (uint32_t b = e_lo / 128 + tid; b < min(tsum_blocks, (e_hi + 127) / 128); b += NCW * 32) tsum_g[b] = ts[b - e_lo / 128];
    if (blockIdx.x == 0 && tid < 4) reinterpret_cast<uint32_t*>(blob + 2 * (size_t)half_bytes)[tid] = 0u;   // the zero record
    if (blockIdx.x == 0 && tid == 4) *reinterpret_cast<float*>(blob + mma_blob_kappa_off(groups)) = kappa;
}

// f32 value of the four digit accumulators a thread holds for one row: quad lane 0 has digits 0, 1
// (weights 128^3, 128^2), quad lane 1 digits 2, 3 (128, 1); quad lanes 2, 3 hold the unused columns.
__device__ __forceinline__ float digits_to_f32(int c_lo, int c_hi, float w_lo, float w_hi) {
    return fmaf((float)c_lo, w_lo, (float)c_hi * w_hi);
}

// int -> float for |c| < 2^22 without the conversion unit: 0x4B400000 is 12582912.0f, whose ulp is 1
__device__ __forceinline__ float small_int_to_f32(int c) { return __int_as_float(c + 0x4B400000) - 12582912.0f; }

// ── Q1_0 tile: 16 rows x groups [g_lo, g_hi) of 18-byte blocks; returns this thread's partial of rows
// (groupID) and (groupID + 8); the caller adds the quad up.
// Two blocks share one k = 32 step: block G feeds k slots 0..15 and B columns 0..3, block G + 1 feeds k slots
// 16..31 and B columns 4..7 (each half of B is zero where the other block's bytes sit), so the eight columns of
// the accumulator hold the four digit sums of both blocks: quad lanes 0, 1 finish block G, quad lanes 2, 3 block G + 1.
struct MmaQ1_0 {
    static constexpr bool HAS_TSUM = true;
    static constexpr int CODE = 0;
    static constexpr uint32_t SPLIT_UNIT = 1;   // groups per unit the row may be split at between warps
    __device__ static void tile(uint32_t rowA, uint32_t rowB, uint32_t g_lo, uint32_t g_hi, const MmaTable& tb, uint32_t lane,
                                const StreamArgs&, float& y0, float& y1) {
        const uint32_t t = lane & 3u, d = lane >> 2;
        const uint32_t which = t >> 1;                  // the block of the pair this thread finishes
        const bool second = d >= 4;                     // this thread's B column belongs to block G + 1
        const float w_lo = (t & 1u) ? 128.0f : 2097152.0f, w_hi = (t & 1u) ? 1.0f : 16384.0f;
        const float k2 = 2.0f * tb.kappa;
        y0 = 0.0f; y1 = 0.0f;
        // The sign words of a block start 2 bytes after a 2-byte-aligned block; a pair of blocks is 36 bytes, so
        // every pair of this row starts with the same alignment: read aligned words and funnel-shift by a
        // loop-invariant amount (the second block of a pair has the opposite alignment).
        uint32_t pA = rowA + g_lo * 18 + 2 + t * 4, pB = rowB + g_lo * 18 + 2 + t * 4;
        const uint32_t shA = (pA & 2u) * 8u, shB = (pB & 2u) * 8u;
        pA &= ~3u; pB &= ~3u;
        // the second block's words: +18 bytes = 4 words and a flipped half-word
        const uint32_t oA2 = shA ? 20u : 16u, oB2 = shB ? 20u : 16u;
        // B records: a column of the first block takes part in k slots 0..15 only, a column of the second in 16..31
        uint32_t rec = tb.words + (((g_lo + (second ? 1u : 0u)) * 4 + (d & 3u)) * 4 + t) * 16;
        uint32_t dA = rowA + (g_lo + which) * 18, dB = rowB + (g_lo + which) * 18, ts = tb.tsum + (g_lo + which) * 4;
        for (uint32_t G = g_lo; G < g_hi; G += 2, pA += 36, pB += 36, rec += 512, dA += 36, dB += 36, ts += 8) {
            const bool pair = G + 1 < g_hi;             // an odd range ends with a single block
            const uint32_t a0 = __funnelshift_r(lds32(pA), lds32(pA + 4), shA);
            const uint32_t a1 = __funnelshift_r(lds32(pB), lds32(pB + 4), shB);
            uint32_t a2 = 0u, a3 = 0u;
            if (pair) {
                a2 = __funnelshift_r(lds32(pA + oA2), lds32(pA + oA2 + 4), shA ^ 16u);
                a3 = __funnelshift_r(lds32(pB + oB2), lds32(pB + oB2 + 4), shB ^ 16u);
            }
            const uint32_t live = (!second || pair) ? rec : tb.zero, liveh = (!second || pair) ? rec + tb.half : tb.zero;
            const uint4 lo03 = lds128(second ? tb.zero : live), lo47 = lds128(second ? tb.zero : liveh);    // k slots 0..15
            const uint4 hi03 = lds128(second ? live : tb.zero), hi47 = lds128(second ? liveh : tb.zero);    // k slots 16..31
            int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};   // two chains: even and odd bit positions
#define ALICE_Q1(m, bl, bh, c) mma_u8s8_k32(c, a0 & (m), a1 & (m), a2 & (m), a3 & (m), (bl), (bh));
            ALICE_Q1(0x01010101u, lo03.x, hi03.x, c0) ALICE_Q1(0x02020202u, lo03.y, hi03.y, c1)
            ALICE_Q1(0x04040404u, lo03.z, hi03.z, c0) ALICE_Q1(0x08080808u, lo03.w, hi03.w, c1)
            ALICE_Q1(0x10101010u, lo47.x, hi47.x, c0) ALICE_Q1(0x20202020u, lo47.y, hi47.y, c1)
            ALICE_Q1(0x40404040u, lo47.z, hi47.z, c0) ALICE_Q1(0x80808080u, lo47.w, hi47.w, c1)
#undef ALICE_Q1
            if (which == 0 || pair) {
                // per-block sums stay far below 2^22 (16 bytes x 8 bits x 2^j x |digit| <= 64)
                const float sA = fmaf(small_int_to_f32(c0[0] + c1[0]), w_lo, small_int_to_f32(c0[1] + c1[1]) * w_hi);
                const float sB = fmaf(small_int_to_f32(c0[2] + c1[2]), w_lo, small_int_to_f32(c0[3] + c1[3]) * w_hi);
                const float tsum = (t & 1u) ? 0.0f : ldsf(ts);
                y0 = fmaf(f16_bits_to_f32(lds16(dA)), fmaf(sA, k2, -tsum), y0);
                y1 = fmaf(f16_bits_to_f32(lds16(dB)), fmaf(sB, k2, -tsum), y1);
            }
        }
    }
    __device__ static float finish(float v, const StreamArgs&, const float*, uint32_t) { return v; }
};

// ── Ternary planes tile: row = [pos plane | neg plane], planes of row_bytes/2 bytes (multiples of 4).
// Groups are taken two at a time (k = 32); integer accumulation over the whole group range.
struct MmaTernary {
    static constexpr bool HAS_TSUM = false;
    static constexpr int CODE = 0;
    static constexpr uint32_t SPLIT_UNIT = 1;
    __device__ static void tile(uint32_t rowA, uint32_t rowB, uint32_t g_lo, uint32_t g_hi, const MmaTable& tb, uint32_t lane,
                                const StreamArgs& a, float& y0, float& y1) {
        const uint32_t t = lane & 3u, d = lane >> 2;
        const bool has_b = d < 4;
        const uint32_t plane = a.row_bytes >> 1;
        const float w_lo = t == 0 ? 2097152.0f : (t == 1 ? 128.0f : 0.0f), w_hi = t == 0 ? 16384.0f : (t == 1 ? 1.0f : 0.0f);
        int p0[4] = {0, 0, 0, 0}, p1[4] = {0, 0, 0, 0}, n0[4] = {0, 0, 0, 0}, n1[4] = {0, 0, 0, 0};
        const uint32_t plane_groups = plane / 16;   // whole 16-byte groups in a plane; a ragged tail is done with k = 16 steps
        uint32_t G = g_lo;
        for (; G + 2 <= g_hi && G + 2 <= plane_groups; G += 2) {
            const uint32_t off = G * 16 + t * 4;
            const uint32_t pa0 = lds32(rowA + off), pa1 = lds32(rowB + off), pa2 = lds32(rowA + off + 16), pa3 = lds32(rowB + off + 16);
            const uint32_t na0 = lds32(rowA + plane + off), na1 = lds32(rowB + plane + off), na2 = lds32(rowA + plane + off + 16),
                           na3 = lds32(rowB + plane + off + 16);
            // B of group G (k slots 0..15) and of group G + 1 (k slots 16..31); columns 4..7 are unused
            const uint32_t rec = has_b ? tb.words + ((G * 4 + d) * 4 + t) * 16 : tb.zero;
            const uint32_t rech = has_b ? rec + tb.half : tb.zero, nxt = has_b ? 256u : 0u;
            const uint4 x03 = lds128(rec), x47 = lds128(rech), z03 = lds128(rec + nxt), z47 = lds128(rech + nxt);
#define ALICE_TERN(m, bx, bz, cp, cn)                                                     \
            mma_u8s8_k32(cp, pa0 & (m), pa1 & (m), pa2 & (m), pa3 & (m), (bx), (bz));     \
            mma_u8s8_k32(cn, na0 & (m), na1 & (m), na2 & (m), na3 & (m), (bx), (bz));
            ALICE_TERN(0x01010101u, x03.x, z03.x, p0, n0) ALICE_TERN(0x02020202u, x03.y, z03.y, p1, n1)
            ALICE_TERN(0x04040404u, x03.z, z03.z, p0, n0) ALICE_TERN(0x08080808u, x03.w, z03.w, p1, n1)
            ALICE_TERN(0x10101010u, x47.x, z47.x, p0, n0) ALICE_TERN(0x20202020u, x47.y, z47.y, p1, n1)
            ALICE_TERN(0x40404040u, x47.z, z47.z, p0, n0) ALICE_TERN(0x80808080u, x47.w, z47.w, p1, n1)
#undef ALICE_TERN
        }
        for (; G < g_hi; G++) {   // odd group count, or the last partly filled group of a plane
            const uint32_t off = G * 16 + t * 4;
            const bool in = off + 4 <= plane;    // planes are multiples of 4 bytes: a word is inside or outside
            const uint32_t pa0 = in ? lds32(rowA + off) : 0u, pa1 = in ? lds32(rowB + off) : 0u;
            const uint32_t na0 = in ? lds32(rowA + plane + off) : 0u, na1 = in ? lds32(rowB + plane + off) : 0u;
            const uint32_t rec = has_b ? tb.words + ((G * 4 + d) * 4 + t) * 16 : tb.zero;
            const uint4 x03 = lds128(rec), x47 = lds128(has_b ? rec + tb.half : tb.zero);
#define ALICE_TERN16(m, bx, cp, cn)                              \
            mma_u8s8_k16(cp, pa0 & (m), pa1 & (m), (bx));        \
            mma_u8s8_k16(cn, na0 & (m), na1 & (m), (bx));
            ALICE_TERN16(0x01010101u, x03.x, p0, n0) ALICE_TERN16(0x02020202u, x03.y, p1, n1)
            ALICE_TERN16(0x04040404u, x03.z, p0, n0) ALICE_TERN16(0x08080808u, x03.w, p1, n1)
            ALICE_TERN16(0x10101010u, x47.x, p0, n0) ALICE_TERN16(0x20202020u, x47.y, p1, n1)
            ALICE_TERN16(0x40404040u, x47.z, p0, n0) ALICE_TERN16(0x80808080u, x47.w, p1, n1)
#undef ALICE_TERN16
        }
        y0 = tb.kappa * digits_to_f32(p0[0] + p1[0] - n0[0] - n1[0], p0[1] + p1[1] - n0[1] - n1[1], w_lo, w_hi);
        y1 = tb.kappa * digits_to_f32(p0[2] + p1[2] - n0[2] - n1[2], p0[3] + p1[3] - n0[3] - n1[3], w_lo, w_hi);
    }
    __device__ static float finish(float v, const StreamArgs&, const float* aux, uint32_t row) { return __ldg(aux + row) * v; }
};

// ── Q2_0 tile: 34-byte block = d f16 + 128 two-bit slots, value (slot - 1) * d (src/gguf.rs:1283-1300):
// y = sum_b d_b * (S_b - T_b), S_b = sum slot * x. A block is two groups = one k = 32 step with the four digit columns.
struct MmaQ2_0 {
    static constexpr bool HAS_TSUM = true;
    static constexpr int CODE = 1;
    static constexpr uint32_t SPLIT_UNIT = 2;
    __device__ static void tile(uint32_t rowA, uint32_t rowB, uint32_t g_lo, uint32_t g_hi, const MmaTable& tb, uint32_t lane,
                                const StreamArgs&, float& y0, float& y1) {
        const uint32_t t = lane & 3u, d = lane >> 2;
        const bool has_b = d < 4;
        const float w_lo = t == 0 ? 2097152.0f : (t == 1 ? 128.0f : 0.0f), w_hi = t == 0 ? 16384.0f : (t == 1 ? 1.0f : 0.0f);
        y0 = 0.0f; y1 = 0.0f;
        for (uint32_t b = g_lo / 2; b < g_hi / 2; b++) {
            const uint32_t blkA = rowA + b * 34, blkB = rowB + b * 34;
            const uint32_t a0 = lds32_u2(blkA + 2 + t * 4), a1 = lds32_u2(blkB + 2 + t * 4);
            const uint32_t a2 = lds32_u2(blkA + 18 + t * 4), a3 = lds32_u2(blkB + 18 + t * 4);
            const uint32_t rec = has_b ? tb.words + ((2 * b * 4 + d) * 4 + t) * 16 : tb.zero;
            const uint32_t rech = has_b ? rec + tb.half : tb.zero, nxt = has_b ? 256u : 0u;
            const uint4 x03 = lds128(rec), x47 = lds128(rech), z03 = lds128(rec + nxt), z47 = lds128(rech + nxt);
            int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
#define ALICE_Q2(m, bx, bz, c) mma_u8s8_k32(c, a0 & (m), a1 & (m), a2 & (m), a3 & (m), (bx), (bz));
            ALICE_Q2(0x01010101u, x03.x, z03.x, c0) ALICE_Q2(0x02020202u, x03.y, z03.y, c1)
            ALICE_Q2(0x04040404u, x03.z, z03.z, c0) ALICE_Q2(0x08080808u, x03.w, z03.w, c1)
            ALICE_Q2(0x10101010u, x47.x, z47.x, c0) ALICE_Q2(0x20202020u, x47.y, z47.y, c1)
            ALICE_Q2(0x40404040u, x47.z, z47.z, c0) ALICE_Q2(0x80808080u, x47.w, z47.w, c1)
#undef ALICE_Q2
            // per-block sums stay below 2^22 (32 bytes x 8 bits x 2^j x |digit| <= 64)
            const float sA = fmaf(small_int_to_f32(c0[0] + c1[0]), w_lo, small_int_to_f32(c0[1] + c1[1]) * w_hi);
            const float sB = fmaf(small_int_to_f32(c0[2] + c1[2]), w_lo, small_int_to_f32(c0[3] + c1[3]) * w_hi);
            const float tsum = t == 0 ? ldsf(tb.tsum + b * 4) : 0.0f;
            y0 = fmaf(f16_bits_to_f32(lds16(blkA)), fmaf(sA, tb.kappa, -tsum), y0);
            y1 = fmaf(f16_bits_to_f32(lds16(blkB)), fmaf(sB, tb.kappa, -tsum), y1);
        }
    }
    __device__ static float finish(float v, const StreamArgs&, const float*, uint32_t) { return v; }
};

// ── Sparse-ternary tile: packed 2-bit codes, 4 bytes per 16 columns (SparseTernaryMatrix::packed_2bit,
// src/gguf.rs:5560-5583), 00 = 0, 01 = +1, 11 = -1: the low bit of a code is worth +x, the high bit -2x.
// y = scale_row * S; integer accumulation over the whole group range.
struct MmaSparseTernary {
    static constexpr bool HAS_TSUM = false;
    static constexpr int CODE = 2;
    static constexpr uint32_t SPLIT_UNIT = 1;
    __device__ static void tile(uint32_t rowA, uint32_t rowB, uint32_t g_lo, uint32_t g_hi, const MmaTable& tb, uint32_t lane,
                                const StreamArgs& a, float& y0, float& y1) {
        const uint32_t t = lane & 3u, d = lane >> 2;
        const bool has_b = d < 4;
        const float w_lo = t == 0 ? 2097152.0f : (t == 1 ? 128.0f : 0.0f), w_hi = t == 0 ? 16384.0f : (t == 1 ? 1.0f : 0.0f);
        int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
        const uint32_t whole = a.row_bytes / 16;   // whole 16-byte groups in a row
        uint32_t G = g_lo;
        for (; G + 2 <= g_hi && G + 2 <= whole; G += 2) {
            const uint32_t off = G * 16 + t * 4;
            const uint32_t a0 = lds32(rowA + off), a1 = lds32(rowB + off), a2 = lds32(rowA + off + 16), a3 = lds32(rowB + off + 16);
            const uint32_t rec = has_b ? tb.words + ((G * 4 + d) * 4 + t) * 16 : tb.zero;
            const uint32_t rech = has_b ? rec + tb.half : tb.zero, nxt = has_b ? 256u : 0u;
            const uint4 x03 = lds128(rec), x47 = lds128(rech), z03 = lds128(rec + nxt), z47 = lds128(rech + nxt);
#define ALICE_SP(m, bx, bz, c) mma_u8s8_k32(c, a0 & (m), a1 & (m), a2 & (m), a3 & (m), (bx), (bz));
            ALICE_SP(0x01010101u, x03.x, z03.x, c0) ALICE_SP(0x02020202u, x03.y, z03.y, c1)
            ALICE_SP(0x04040404u, x03.z, z03.z, c0) ALICE_SP(0x08080808u, x03.w, z03.w, c1)
            ALICE_SP(0x10101010u, x47.x, z47.x, c0) ALICE_SP(0x20202020u, x47.y, z47.y, c1)
            ALICE_SP(0x40404040u, x47.z, z47.z, c0) ALICE_SP(0x80808080u, x47.w, z47.w, c1)
#undef ALICE_SP
        }
        for (; G < g_hi; G++) {   // odd group count, or the last partly filled group of a row
            const uint32_t off = G * 16 + t * 4;
            const bool in = off + 4 <= a.row_bytes;   // rows are multiples of 4 bytes
            const uint32_t a0 = in ? lds32(rowA + off) : 0u, a1 = in ? lds32(rowB + off) : 0u;
            const uint32_t rec = has_b ? tb.words + ((G * 4 + d) * 4 + t) * 16 : tb.zero;
            const uint4 x03 = lds128(rec), x47 = lds128(has_b ? rec + tb.half : tb.zero);
#define ALICE_SP16(m, bx, c) mma_u8s8_k16(c, a0 & (m), a1 & (m), (bx));
            ALICE_SP16(0x01010101u, x03.x, c0) ALICE_SP16(0x02020202u, x03.y, c1) ALICE_SP16(0x04040404u, x03.z, c0)
            ALICE_SP16(0x08080808u, x03.w, c1) ALICE_SP16(0x10101010u, x47.x, c0) ALICE_SP16(0x20202020u, x47.y, c1)
            ALICE_SP16(0x40404040u, x47.z, c0) ALICE_SP16(0x80808080u, x47.w, c1)
#undef ALICE_SP16
        }
        y0 = tb.kappa * digits_to_f32(c0[0] + c1[0], c0[1] + c1[1], w_lo, w_hi);
        y1 = tb.kappa * digits_to_f32(c0[2] + c1[2], c0[3] + c1[3], w_lo, w_hi);
    }
    __device__ static float finish(float v, const StreamArgs&, const float* aux, uint32_t row) { return __ldg(aux + row) * v; }
};

// Consumer side of one matvec in bit-plane tensor-core form (the NCW consumer warps). Same ring, barriers,
// partial-sum hand-over and epilogue as stream_consume; a stage holds slots * 16 rows and warp `part` of a
// row set covers groups [groups * part / P, groups * (part + 1) / P) of every row of its 16-row tile.
template <class M, bool SWIGLU, bool PEER>
__device__ __forceinline__ bool stream_consume_mma(const StreamArgs& a, StreamCtx& cx) {
    StreamSmem* sm = cx.sm;
    uint8_t* smem_raw = cx.smem_raw;
    volatile int* abort_flag = &sm->abort_flag;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t P = a.P, slots = a.slots, rps = a.rps;   // rps == 16
    const uint32_t rows_per_group = slots * rps;
    const uint32_t slot = warp / P, part = warp % P;

    constexpr uint32_t GE = mma_group_elems<M::CODE>();
    const uint32_t ngroups = (a.cols + GE - 1) / GE;
    MmaTable tb;
    uint8_t* table = smem_raw + a.tab_off;
    float* tsum = reinterpret_cast<float*>(table + ((mma_table_bytes(ngroups) + 15u) & ~15u));
    tb.words = smem_u32(table);
    tb.half = ngroups * 256u;
    tb.zero = tb.words + 2 * tb.half;
    tb.tsum = smem_u32(tsum);
    const uint32_t tsum_blocks = M::HAS_TSUM ? a.cols / 128 : 0u;
    if (a.tab_global != nullptr) {
        // prepared once by mma_table_kernel: one bulk copy per CTA, same layout as the table built in place
        const uint32_t bar = smem_u32(&sm->act_bar), bytes = mma_blob_bytes(ngroups);
        if (threadIdx.x == 0) {
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s(tb.words, a.tab_global, bytes, bar);
        }
        if (!wait_or_abort(bar, 0, abort_flag, a.status, KERR_WAIT_FULL, cx.limit)) return false;
        tb.kappa = *reinterpret_cast<const float*>(table + mma_blob_kappa_off(ngroups));
    } else {
        tb.kappa = mma_build_table<M::CODE>(sm, a.x, a.cols, table, tsum, tsum_blocks);
    }
    // the warps of a row set split the groups in whole SPLIT_UNITs (a Q2_0 block is two groups)
    const uint32_t nunits = (ngroups + M::SPLIT_UNIT - 1) / M::SPLIT_UNIT;
    const uint32_t g_lo = nunits * part / P * M::SPLIT_UNIT, g_hi = min(ngroups, nunits * (part + 1) / P * M::SPLIT_UNIT);
    const uint32_t rowsel_a = lane >> 2, rowsel_b = (lane >> 2) + 8;

    const uint32_t g0 = (uint32_t)(((uint64_t)a.groups * blockIdx.x) / gridDim.x);
    const uint32_t g1 = (uint32_t)(((uint64_t)a.groups * (blockIdx.x + 1)) / gridDim.x);
    for (uint32_t g = g0; g < g1; g++) {
        const uint32_t s = cx.cc % cx.nstages, ph = (cx.cc / cx.nstages) & 1;
        cx.cc++;
        uint32_t sg = 0;
        while (sg + 1 < a.nseg && g >= a.seg_g0[sg + 1]) sg++;
        const uint32_t seg_rows = a.seg_rows[sg];
        const uint32_t r0 = (g - a.seg_g0[sg]) * rows_per_group;
        const uint32_t pad = a.row_mode ? 0u : (uint32_t)(((uint64_t)r0 * a.row_bytes) & 15);
        const uint32_t set0 = slot * rps;
        const uint32_t nrow = r0 + set0 < seg_rows ? min(rps, seg_rows - r0 - set0) : 0;
        float res = 0.0f;
        if (a.resid != nullptr && part == 0 && lane < nrow) res = __ldcg(a.resid + a.seg_y[sg] + r0 + set0 + lane);
        if (!wait_or_abort(smem_u32(&sm->full[s]), ph, abort_flag, a.status, KERR_WAIT_FULL, cx.limit)) return false;
        const uint32_t sb = cx.ring + s * cx.stage_stride + pad + set0 * a.row_stride;
        if (nrow > 0) {
            // rows past nrow of a short last tile read whatever the stage holds; their results are never used
            const uint32_t rowA = sb + rowsel_a * a.row_stride, rowB = sb + rowsel_b * a.row_stride;
            float y0, y1, u0 = 0.0f, u1 = 0.0f;
            M::tile(rowA, rowB, g_lo, g_hi, tb, lane, a, y0, y1);
            if (SWIGLU) M::tile(rowA + a.cap, rowB + a.cap, g_lo, g_hi, tb, lane, a, u0, u1);
            // quad lanes 0 and 1 hold the two halves of the digit weights: add the quad up
            y0 += __shfl_xor_sync(0xffffffffu, y0, 1); y1 += __shfl_xor_sync(0xffffffffu, y1, 1);
            y0 += __shfl_xor_sync(0xffffffffu, y0, 2); y1 += __shfl_xor_sync(0xffffffffu, y1, 2);
            if (SWIGLU) {
                u0 += __shfl_xor_sync(0xffffffffu, u0, 1); u1 += __shfl_xor_sync(0xffffffffu, u1, 1);
                u0 += __shfl_xor_sync(0xffffffffu, u0, 2); u1 += __shfl_xor_sync(0xffffffffu, u1, 2);
            }
            if ((lane & 3u) == 0) {
                sm->partial[s][warp][rowsel_a][0] = y0; sm->partial[s][warp][rowsel_b][0] = y1;
                if (SWIGLU) { sm->partial[s][warp][rowsel_a][1] = u0; sm->partial[s][warp][rowsel_b][1] = u1; }
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
                unsigned long long key = 0ull;
                float v0 = 0.0f, v1 = 0.0f;
                if (lane < nrow) {
                    for (uint32_t p = 0; p < P; p++) {
                        v0 += sm->partial[s][warp + p][lane][0];
                        if (SWIGLU) v1 += sm->partial[s][warp + p][lane][1];
                    }
                }
                // everything this warp needed from the stage has been read: let the producer refill it while
                // the epilogue runs
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
                if (lane < nrow) {
                    const uint32_t row = r0 + set0 + lane;
                    float r = M::finish(v0, a, a.seg_aux[sg], row);
                    if (SWIGLU) r = silu_ref(r) * M::finish(v1, a, a.aux1, row);
                    key = stream_store_row<PEER>(a, r, res, a.resid != nullptr, a.seg_y[sg] + row);
                }
                if (a.argmax_key != nullptr) stream_argmax(a.argmax_key, key, lane);
                continue;   // this warp has already released the stage
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
    }
    return true;
}

// One matvec per launch, bit-plane tensor-core form. CTAS: resident CTAs per SM the launch is planned for.
template <class M, bool SWIGLU, int CTAS, bool PEER>
__global__ void __launch_bounds__(STREAM_THREADS, CTAS) stream_gemv_mma_kernel(const __grid_constant__ StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    StreamSmem* sm = reinterpret_cast<StreamSmem*>(smem_raw);
    constexpr uint32_t HDR = (sizeof(StreamSmem) + 127) & ~127u;
    StreamCtx cx;
    cx.sm = sm; cx.smem_raw = smem_raw; cx.ring = smem_u32(smem_raw) + HDR;
    cx.stage_stride = a.cap * (SWIGLU ? 2u : 1u); cx.nstages = a.nstages; cx.cc = 0;
    cx.limit = a.wait_limit > 0 ? a.wait_limit : WAIT_CYCLE_LIMIT;
    stream_init_ring(sm, a.nstages);
    __syncthreads();
    pdl_launch_dependents();
    if ((threadIdx.x >> 5) == NCW) {
        if (a.row_mode) {
            stream_produce_rows(a, cx);
            if ((threadIdx.x & 31) == 0 && sm->abort_flag) stream_drain(cx);
        } else if ((threadIdx.x & 31) == 0) {
            stream_produce(a, cx);
            if (sm->abort_flag) stream_drain(cx);
        }
        return;
    }
    pdl_wait();
    stream_consume_mma<M, SWIGLU, PEER>(a, cx);
}

}  // namespace alice
