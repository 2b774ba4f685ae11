// Preparing a vector ONCE for the op that consumes it.
//
// Every CTA of a matvec needs its whole input in the form its inner loop reads: Q8_K blocks for the K-quant
// formats, the RMS-normalised f32 vector for the others. That form is the same in every CTA, so it is computed
// once - by a small stand-alone kernel launched between producer and consumer (publish_vector_kernel, one CTA; the
// embedding kernel, itself one CTA, does it for its own output) - and left in global memory; the consumer's CTAs fetch
// it straight into registers. With a tensor-parallel group the same kernel first runs the hand-over of the rows the
// peers have pushed (publish_peer_gate). Arithmetic: rms_norm (src/llama3.rs:5244-5256:
// f64 sum of squares, f32 mean / sqrt / divide, (x * scale) * w) and quantize_row_q8_k (src/gguf.rs:1323-1374).
#pragma once
#include "common.cuh"
#include "q8k.cuh"

namespace alice {

constexpr uint32_t PUB_NONE = 0;
constexpr uint32_t PUB_VECTOR = 2;   // whole vector: optional rms_norm, then Q8_K and / or f32

constexpr uint32_t MAX_PEERS = 7;
constexpr int MAX_BATCH = 8;      // input vectors one pass over the weights can serve

// Destination of the prepared form; either part may be absent.
struct PublishDst {
    int8_t* qs;        // Q8_K, structure of arrays: qs[batch][n], d[batch][n/256], bsums[batch][n/16]
    float* d;
    int16_t* bsums;
    float* xn;         // f32 [batch][n]: the normalised vector, or (roundtrip) d * q of its Q8_K quantisation, which is
    uint32_t roundtrip;  // what quantized_matvec_preq hands a Q1_0 / Q2_0 matvec (src/gguf.rs:4593-4605)
};

struct Publish {
    uint32_t mode;
    uint32_t n;              // elements per vector
    uint32_t batch;          // vectors, src[k * n + i]
    const float* src;        // the f32 vector(s) this matvec writes rows of
    const float* norm_w;     // PUB_VECTOR: rms_norm weights, or null
    float eps;
    PublishDst dst;
    // Tensor parallel (PUB_VECTOR): other GPUs store rows of src straight into this GPU's copy. One thread tells every
    // peer that this GPU's rows have landed there (peer_flag[p] += 1, release) and waits, bounded, until all peers have
    // said the same here (*wait_flag >= (*epoch + 1) * npeers) before the vector is read.
    // key_src (optional): a 64-bit value of this GPU (the packed maximum of its logits rows) that goes to peer_key[p]
    // on every peer before the flag, so the same hand-over covers it.
    uint32_t npeers;
    unsigned int* peer_flag[MAX_PEERS];
    const unsigned int* wait_flag;
    const unsigned int* epoch;
    const unsigned long long* key_src;
    unsigned long long* peer_key[MAX_PEERS];
    long long wait_limit;    // SM cycles the wait may take; 0 = WAIT_CYCLE_LIMIT
};

// 8 consecutive elements starting at x[i0], zero past n; L2 loads (another SM, or another GPU, wrote them).
__device__ __forceinline__ Q8KLaneInput pub_load8(const float* x, uint32_t i0, uint32_t n) {
    Q8KLaneInput r;
    if (i0 + 8 <= n && ((reinterpret_cast<uintptr_t>(x + i0) & 15) == 0)) {
        r.a = __ldcg(reinterpret_cast<const float4*>(x + i0));
        r.b = __ldcg(reinterpret_cast<const float4*>(x + i0) + 1);
    } else {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = i0 + j < n ? __ldcg(x + i0 + j) : 0.0f;
        r.a = make_float4(v[0], v[1], v[2], v[3]);
        r.b = make_float4(v[4], v[5], v[6], v[7]);
    }
    return r;
}
__device__ __forceinline__ Q8KLaneInput pub_load8_w(const float* w, uint32_t i0, uint32_t n) {
    Q8KLaneInput r;
    if (i0 + 8 <= n && ((reinterpret_cast<uintptr_t>(w + i0) & 15) == 0)) {
        r.a = __ldg(reinterpret_cast<const float4*>(w + i0));
        r.b = __ldg(reinterpret_cast<const float4*>(w + i0) + 1);
    } else {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = i0 + j < n ? __ldg(w + i0 + j) : 0.0f;
        r.a = make_float4(v[0], v[1], v[2], v[3]);
        r.b = make_float4(v[4], v[5], v[6], v[7]);
    }
    return r;
}
__device__ __forceinline__ double pub_sumsq(const Q8KLaneInput& v) {
    return (double)v.a.x * (double)v.a.x + (double)v.a.y * (double)v.a.y + (double)v.a.z * (double)v.a.z + (double)v.a.w * (double)v.a.w +
           (double)v.b.x * (double)v.b.x + (double)v.b.y * (double)v.b.y + (double)v.b.z * (double)v.b.z + (double)v.b.w * (double)v.b.w;
}
__device__ __forceinline__ Q8KLaneInput pub_scale(const Q8KLaneInput& v, float s, const Q8KLaneInput& w) {
    Q8KLaneInput r;
    r.a = make_float4(__fmul_rn(__fmul_rn(v.a.x, s), w.a.x), __fmul_rn(__fmul_rn(v.a.y, s), w.a.y), __fmul_rn(__fmul_rn(v.a.z, s), w.a.z), __fmul_rn(__fmul_rn(v.a.w, s), w.a.w));
    r.b = make_float4(__fmul_rn(__fmul_rn(v.b.x, s), w.b.x), __fmul_rn(__fmul_rn(v.b.y, s), w.b.y), __fmul_rn(__fmul_rn(v.b.z, s), w.b.z), __fmul_rn(__fmul_rn(v.b.w, s), w.b.w));
    return r;
}

// One prepared 256-element block leaves the warp: Q8_K fields and / or f32.
__device__ __forceinline__ void pub_emit_block(const PublishDst& dst, const Q8KLaneInput& v, uint32_t lane, uint32_t vec, uint32_t blk, uint32_t n,
                                               bool store = true) {
    const uint32_t nb = n / QK_K;
    const size_t bi = (size_t)vec * nb + blk;
    if (dst.qs != nullptr) q8k_quantize_block_warp(v, lane, dst.qs + bi * QK_K, dst.d + bi, dst.bsums + bi * 16, nullptr, store);
    if (dst.xn != nullptr) {
        float* out = dst.xn + (size_t)vec * n + (size_t)blk * QK_K;
        if (dst.roundtrip) {
            q8k_quantize_block_warp<true>(v, lane, nullptr, nullptr, nullptr, out, store);
        } else if (store) {
            const uint32_t i0 = blk * QK_K + lane * 8;
            if (i0 + 8 <= n) {
                reinterpret_cast<float4*>(out + lane * 8)[0] = v.a;
                reinterpret_cast<float4*>(out + lane * 8)[1] = v.b;
            } else {
                const float e[8] = {v.a.x, v.a.y, v.a.z, v.a.w, v.b.x, v.b.y, v.b.z, v.b.w};
                for (uint32_t j = 0; j < 8 && i0 + j < n; j++) out[lane * 8 + j] = e[j];
            }
        }
    }
}

// Whole-vector form, run by NW warps (threads 0 .. NW*32-1 of the CTA) that meet on named barrier `BAR`.
// Warp w owns the 256-element blocks w, w + NW, ...; a lane owns 8 consecutive elements of each. Up to PUB_REG_BLOCKS
// blocks per warp stay in registers between the sum of squares and the second pass (one trip to L2 for vectors of up to
// NW * PUB_REG_BLOCKS * 256 elements), longer vectors are read twice. `red` = NW doubles of shared memory.
//
// Only ONE CTA of a launch runs this, once: its instructions are then in nobody's instruction cache, and a cold walk
// through a few hundred instructions costs on the order of 10 us (measured 14 us) - far more than the arithmetic.
// So every CTA of the launch first calls it with store == false while it waits for the previous kernel anyway: same
// instructions, results discarded, and the real call finds them in the SM's cache.
constexpr int PUB_REG_BLOCKS = 2;
template <int NW, int BAR>
static __device__ __noinline__ void publish_vector(const Publish& p, double* red, bool store) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n = p.n, nblk = (n + QK_K - 1) / QK_K;
    const bool in_regs = nblk <= (uint32_t)(NW * PUB_REG_BLOCKS);
    const uint32_t nvec = store ? p.batch : 1u;
    for (uint32_t k = 0; k < nvec; k++) {
        const float* x = p.src + (size_t)k * n;
        Q8KLaneInput xv[PUB_REG_BLOCKS], wv[PUB_REG_BLOCKS];
        float scale = 1.0f;
        if (in_regs) {
#pragma unroll
            for (int i = 0; i < PUB_REG_BLOCKS; i++) {
                const uint32_t b = warp + (uint32_t)i * NW;
                if (b < nblk) {
                    xv[i] = pub_load8(x, b * QK_K + lane * 8, n);
                    if (p.norm_w != nullptr) wv[i] = pub_load8_w(p.norm_w, b * QK_K + lane * 8, n);
                }
            }
        }
        if (p.norm_w != nullptr) {
            double ss = 0.0;
            if (in_regs) {
#pragma unroll
                for (int i = 0; i < PUB_REG_BLOCKS; i++)
                    if (warp + (uint32_t)i * NW < nblk) ss += pub_sumsq(xv[i]);
            } else {
                for (uint32_t b = warp; b < nblk; b += NW) ss += pub_sumsq(pub_load8(x, b * QK_K + lane * 8, n));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(NW * 32) : "memory");   // `red` free (previous vector read it)
            if (lane == 0) red[warp] = ss;
            asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(NW * 32) : "memory");
            double tot = 0.0;
#pragma unroll
            for (int w = 0; w < NW; w++) tot += red[w];
            const float mean = (float)(tot / (double)n);
            scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        }
        if (in_regs) {
#pragma unroll
            for (int i = 0; i < PUB_REG_BLOCKS; i++) {
                const uint32_t b = warp + (uint32_t)i * NW;
                if (b < nblk) pub_emit_block(p.dst, p.norm_w != nullptr ? pub_scale(xv[i], scale, wv[i]) : xv[i], lane, k, b, n, store);
            }
        } else {
            for (uint32_t b = warp; b < nblk; b += NW) {
                const Q8KLaneInput v = pub_load8(x, b * QK_K + lane * 8, n);
                if (p.norm_w != nullptr) pub_emit_block(p.dst, pub_scale(v, scale, pub_load8_w(p.norm_w, b * QK_K + lane * 8, n)), lane, k, b, n, store);
                else pub_emit_block(p.dst, v, lane, k, b, n, store);
            }
        }
    }
}

// Tensor-parallel gate in front of publish_vector: one thread. Returns false when the bounded wait ran out.
__device__ __forceinline__ bool publish_peer_gate(const Publish& p, int* status) {
    if (p.npeers == 0) return true;
    if (p.key_src != nullptr) {
        const unsigned long long key = __ldcg(p.key_src);
        for (uint32_t q = 0; q < p.npeers; q++) *p.peer_key[q] = key;
    }
    __threadfence_system();
    for (uint32_t q = 0; q < p.npeers; q++) red_release_sys_add_u32(p.peer_flag[q], 1u);
    const unsigned int expected = (ld_acquire_sys_u32(p.epoch) + 1u) * p.npeers;
    return peer_wait(p.wait_flag, expected, status, KERR_WAIT_PEER, p.wait_limit > 0 ? p.wait_limit : WAIT_CYCLE_LIMIT);
}

}  // namespace alice
