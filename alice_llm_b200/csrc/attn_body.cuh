// Device body of the fused decode attention (RoPE + KV append + split-KV GQA attention + split
// combine), shared by the stand-alone kernel (csrc/glue.cu) and the whole-step kernel
// (csrc/step_kernel.cu). Arithmetic: ALICE-LLM src/llama3.rs apply_rope :5323-5333, :5367-5378,
// KvCache::append :4773, gqa_attention :5431-5690, evaluated as an online softmax over KV splits.
#pragma once
#include "common.cuh"
#include "glue.cuh"
#include "q8k.cuh"

namespace alice {

struct RopeCoef { float sn[4], cs[4]; };
// Rotation table of one position: tab[2*j] = sin, tab[2*j + 1] = cos of pos * theta^(-2j / head_dim),
// j = 0 .. head_dim/2 - 1 (head_dim = 128). It depends on the position only, so it is computed once per
// decode step (by the embedding stage) and every layer's attention reads it.
__device__ __forceinline__ void rope_table_entry(float* tab, uint32_t j, uint32_t pos, float theta) {
    const float freq = __fdiv_rn(1.0f, powf(theta, __fdiv_rn((float)(2 * j), 128.0f)));
    float sn, cs;
    sincosf(__fmul_rn((float)pos, freq), &sn, &cs);
    tab[2 * j] = sn; tab[2 * j + 1] = cs;
}
// sin / cos of the rotation angles of the 4 dims a lane owns, fetched from the table (L2 reads: another
// SM wrote it). Pairs layout: dims 4*lane + i belong to pair 2*lane + i/2; NeoX: pair 4*(lane & 15) + i.
__device__ __forceinline__ RopeCoef rope_coef(const float* __restrict__ tab, uint32_t lane, int neox) {
    RopeCoef c;
    if (!neox) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(tab) + lane);   // pairs 2*lane, 2*lane + 1
        c.sn[0] = c.sn[1] = t.x; c.cs[0] = c.cs[1] = t.y;
        c.sn[2] = c.sn[3] = t.z; c.cs[2] = c.cs[3] = t.w;
    } else {
        const float4 t0 = __ldcg(reinterpret_cast<const float4*>(tab) + 2 * (lane & 15));
        const float4 t1 = __ldcg(reinterpret_cast<const float4*>(tab) + 2 * (lane & 15) + 1);
        c.sn[0] = t0.x; c.cs[0] = t0.y; c.sn[1] = t0.z; c.cs[1] = t0.w;
        c.sn[2] = t1.x; c.cs[2] = t1.y; c.sn[3] = t1.z; c.cs[3] = t1.w;
    }
    return c;
}
__device__ __forceinline__ float4 rope4(float4 v, uint32_t lane, const RopeCoef& c, int neox) {
    float r[4] = {v.x, v.y, v.z, v.w}, out[4];
    if (!neox) {
#pragma unroll
        for (int p = 0; p < 2; p++) {
            const float x0 = r[2 * p], x1 = r[2 * p + 1];
            out[2 * p] = __fsub_rn(__fmul_rn(x0, c.cs[2 * p]), __fmul_rn(x1, c.sn[2 * p]));
            out[2 * p + 1] = __fadd_rn(__fmul_rn(x0, c.sn[2 * p]), __fmul_rn(x1, c.cs[2 * p]));
        }
    } else {
        const bool upper = lane >= 16;   // dims 64..127 are the second element of their pair
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float other = __shfl_xor_sync(0xffffffffu, r[i], 16);
            const float x0 = upper ? other : r[i], x1 = upper ? r[i] : other;
            out[i] = upper ? __fadd_rn(__fmul_rn(x0, c.sn[i]), __fmul_rn(x1, c.cs[i]))
                           : __fsub_rn(__fmul_rn(x0, c.cs[i]), __fmul_rn(x1, c.sn[i]));
        }
    }
    return make_float4(out[0], out[1], out[2], out[3]);
}

// GQA decode attention with RoPE, KV append and the split combine fused in.
// One CTA = one KV head x one slice of positions; its GROUP = num_heads/num_kv_heads query heads share
// every K and V row it reads. Each warp walks positions t, t+NW, ...; a lane owns 4 of the 128 dims.
// qkv = [q | k | v] of the current token, un-rotated: q and k are rotated here, the new K/V row is
// used from registers and written to the cache at `pos` by the CTA whose slice contains it.
// Per (split, head) the CTA leaves (max, sum, accumulator); the last CTA of a KV head to finish
// (ticket counter) folds the splits into attn_out for its heads.
template <int GROUP>
struct AttnSmem {
    float m[8][GROUP], l[8][GROUP];
    float4 acc[8][GROUP][32];
    unsigned int last;
};

// CONSUMER_BAR: the 256 threads are the consumer warps of a larger CTA and meet on named barrier 1
// instead of __syncthreads().
template <bool CONSUMER_BAR>
__device__ __forceinline__ void attn_sync() {
    if (CONSUMER_BAR) asm volatile("bar.sync 1, 256;" ::: "memory");
    else __syncthreads();
}

template <int GROUP, bool CONSUMER_BAR>
__device__ __forceinline__ void attn_fused_body(const float* __restrict__ qkv, float* __restrict__ kcache,
                                                float* __restrict__ vcache, uint32_t pos, AttnShape s,
                                                const float* __restrict__ rope_tab, int neox, uint32_t nsplit, float* __restrict__ part,
                                                unsigned int* __restrict__ tickets, float* __restrict__ attn_out,
                                                uint32_t kvh, uint32_t split, AttnSmem<GROUP>* sh, long long* prof = nullptr,
                                                const AttnPeers* peers = nullptr, const AttnQ8Out* q8out = nullptr) {
    constexpr int NW = 8;
    const uint32_t seq = pos + 1;
    const uint32_t per = (seq + nsplit - 1) / nsplit;
    const uint32_t t0 = split * per, t1 = min(seq, t0 + per);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_dim = s.num_heads * s.head_dim, kv_dim = s.num_kv_heads * s.head_dim;
    const float inv_sqrt_d = __fdiv_rn(1.0f, sqrtf((float)s.head_dim));

    // KB positions per warp round: their 2*KB row loads are issued before the first is used, so a round costs one
    // memory round trip instead of KB (positions are still folded in ascending order). The first round is requested
    // before q and the rotation table are looked at: none of these loads depends on another.
    constexpr int KB = CONSUMER_BAR ? 2 : 4;   // inside the whole-step kernel registers are scarce
    float4 k[KB], v[KB];
    auto load_round = [&](uint32_t tb) {
#pragma unroll
        for (int j = 0; j < KB; j++) {
            const uint32_t t = tb + j * NW;
            k[j] = v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < t1 && t != pos) {
                k[j] = __ldcg(reinterpret_cast<const float4*>(kcache + (size_t)t * kv_dim + kvh * s.head_dim) + lane);
                v[j] = __ldcg(reinterpret_cast<const float4*>(vcache + (size_t)t * kv_dim + kvh * s.head_dim) + lane);
            }
        }
    };
    float4 q[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; g++) q[g] = __ldcg(reinterpret_cast<const float4*>(qkv + (size_t)(kvh * GROUP + g) * s.head_dim) + lane);
    if (t0 + warp < t1) load_round(t0 + warp);
    const RopeCoef rc = rope_coef(rope_tab, lane, neox);
#pragma unroll
    for (int g = 0; g < GROUP; g++) q[g] = rope4(q[g], lane, rc, neox);
    if (prof && threadIdx.x == 0) prof[1] = clock64();
    float m[GROUP], l[GROUP];
    float4 acc[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; g++) { m[g] = -INFINITY; l[g] = 0.0f; acc[g] = make_float4(0.f, 0.f, 0.f, 0.f); }

    for (uint32_t tb = t0 + warp; tb < t1; tb += NW * KB) {
        if (tb != t0 + warp) load_round(tb);
#pragma unroll
        for (int j = 0; j < KB; j++) {
            const uint32_t t = tb + j * NW;
            if (t < t1) {
                if (t == pos) {   // the token being decoded: rotate its K, append K and V (KvCache::append, src/llama3.rs:4773)
                    k[j] = rope4(__ldcg(reinterpret_cast<const float4*>(qkv + q_dim + (size_t)kvh * s.head_dim) + lane), lane, rc, neox);
                    v[j] = __ldcg(reinterpret_cast<const float4*>(qkv + q_dim + kv_dim + (size_t)kvh * s.head_dim) + lane);
                    reinterpret_cast<float4*>(kcache + (size_t)t * kv_dim + kvh * s.head_dim)[lane] = k[j];
                    reinterpret_cast<float4*>(vcache + (size_t)t * kv_dim + kvh * s.head_dim)[lane] = v[j];
                }
                float sc[GROUP];
#pragma unroll
                for (int g = 0; g < GROUP; g++) sc[g] = q[g].x * k[j].x + q[g].y * k[j].y + q[g].z * k[j].z + q[g].w * k[j].w;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                    for (int g = 0; g < GROUP; g++) sc[g] += __shfl_xor_sync(0xffffffffu, sc[g], o);
#pragma unroll
                for (int g = 0; g < GROUP; g++) {
                    const float x = sc[g] * inv_sqrt_d;
                    const float mn = fmaxf(m[g], x);
                    const float corr = expf(m[g] - mn), p = expf(x - mn);
                    l[g] = l[g] * corr + p;
                    acc[g].x = acc[g].x * corr + p * v[j].x; acc[g].y = acc[g].y * corr + p * v[j].y;
                    acc[g].z = acc[g].z * corr + p * v[j].z; acc[g].w = acc[g].w * corr + p * v[j].w;
                    m[g] = mn;
                }
            }
        }
    }
    if (prof && threadIdx.x == 0) prof[2] = clock64();
    // combine the NW warps of the CTA
#pragma unroll
    for (int g = 0; g < GROUP; g++) {
        if (lane == 0) { sh->m[warp][g] = m[g]; sh->l[warp][g] = l[g]; }
        sh->acc[warp][g][lane] = acc[g];
    }
    attn_sync<CONSUMER_BAR>();
    const uint32_t stride = s.head_dim + 4;   // (m, l, pad, pad, acc[128]): keeps acc 16-byte aligned
    if (warp < GROUP) {
        const int g = warp;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) M = fmaxf(M, sh->m[w][g]);
        float L = 0.0f;
        float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < NW; w++) {
                const float c = expf(sh->m[w][g] - M);   // exp(-inf) = 0 for warps that saw no position
                L += sh->l[w][g] * c;
                const float4 a = sh->acc[w][g][lane];
                A.x += a.x * c; A.y += a.y * c; A.z += a.z * c; A.w += a.w * c;
            }
        }
        float* out = part + ((size_t)split * s.num_heads + kvh * GROUP + g) * stride;
        if (lane == 0) { out[0] = M; out[1] = L; }
        reinterpret_cast<float4*>(out + 4)[lane] = A;
    }
    // last CTA of this KV head folds the splits
    if (prof && threadIdx.x == 0) prof[3] = clock64();
    __threadfence();
    attn_sync<CONSUMER_BAR>();
    if (threadIdx.x == 0) {
        const unsigned int ticket = atomicAdd(&tickets[kvh], 1u);
        sh->last = (ticket == nsplit - 1) ? 1u : 0u;
        if (sh->last) tickets[kvh] = 0;   // ready for the next launch
    }
    attn_sync<CONSUMER_BAR>();
    if (prof && threadIdx.x == 0) prof[6] = clock64();
    if (!sh->last) return;
    __threadfence();
    float4 o_keep = make_float4(0.f, 0.f, 0.f, 0.f);   // this warp's head, this lane's 4 dims
    if (warp < GROUP) {
        // one warp per head; lane <-> split for the (max, sum) pairs, so all loads are in flight at once
        const uint32_t head = kvh * GROUP + warp;
        float ms[2], ls[2];
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t sp = lane + 32 * i;
            ms[i] = -INFINITY; ls[i] = 0.0f;
            if (sp < nsplit) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(part + ((size_t)sp * s.num_heads + head) * stride));
                ms[i] = ml.x; ls[i] = ml.y;
            }
            M = fmaxf(M, ms[i]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float cs[2], L = 0.0f;
#pragma unroll
        for (int i = 0; i < 2; i++) { cs[i] = ms[i] == -INFINITY ? 0.0f : expf(ms[i] - M); L += ls[i] * cs[i]; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
        constexpr int SB = CONSUMER_BAR ? 8 : 16;   // split accumulators fetched per round trip
        for (uint32_t sp0 = 0; sp0 < nsplit; sp0 += SB) {
            float4 a[SB];
#pragma unroll
            for (int j = 0; j < SB; j++)
                if (sp0 + j < nsplit)
                    a[j] = __ldcg(reinterpret_cast<const float4*>(part + ((size_t)(sp0 + j) * s.num_heads + head) * stride + 4) + lane);
#pragma unroll
            for (int j = 0; j < SB; j++) {
                const uint32_t sp = sp0 + j;
                const float c = __shfl_sync(0xffffffffu, sp < 32 ? cs[0] : cs[1], sp & 31);
                if (sp < nsplit) { A.x += a[j].x * c; A.y += a[j].y * c; A.z += a[j].z * c; A.w += a[j].w * c; }
            }
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        const float4 o = make_float4(A.x * inv, A.y * inv, A.z * inv, A.w * inv);
        reinterpret_cast<float4*>(attn_out + (size_t)head * s.head_dim)[lane] = o;
        o_keep = o;
        if (peers && peers->out_ll) {   // tagged vector: this GPU's copy and the peers'
            const uint32_t tag = ld_acquire_sys_u32(peers->epoch) * peers->tag_n + peers->tag_seq + 1u;
            const size_t e0 = (size_t)head * s.head_dim + lane * 4;
            const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                ll_store(peers->out_ll + e0 + i, ov[i], tag);
                for (uint32_t p = 0; p < peers->npeers; p++) ll_store(peers->peer_ll[p] + e0 + i, ov[i], tag);
            }
        } else if (peers) {
            for (uint32_t p = 0; p < peers->npeers; p++) reinterpret_cast<float4*>(peers->out[p] + (size_t)head * s.head_dim)[lane] = o;
        }
    }
    if (q8out && q8out->qs && (GROUP % 2) == 0) {
        // Q8_K of this KV head's GROUP * 128 outputs = GROUP / 2 whole blocks (quantize_row_q8_k, src/gguf.rs:1323): the
        // outputs go through shared memory so that a warp sees the two heads of its block
        attn_sync<CONSUMER_BAR>();                      // the split accumulators in sh->acc are no longer needed
        if (warp < GROUP) sh->acc[0][warp][lane] = o_keep;
        attn_sync<CONSUMER_BAR>();
        if (warp < GROUP / 2) {
            const uint32_t blk = (kvh * GROUP) / 2 + warp;
            const int hsel = 2 * (int)warp + (int)(lane >> 4);
            Q8KLaneInput in;
            in.a = sh->acc[0][hsel][(lane & 15) * 2];
            in.b = sh->acc[0][hsel][(lane & 15) * 2 + 1];
            q8k_quantize_block_warp(in, lane, q8out->qs + (size_t)blk * 256, q8out->d + blk, q8out->bsums + (size_t)blk * 16);
        }
    }
    if (peers && peers->npeers && !peers->out_ll) {   // this KV head's output has been pushed: tell every peer
        __threadfence_system();
        attn_sync<CONSUMER_BAR>();
        if (threadIdx.x < peers->npeers) red_release_sys_add_u32(peers->flag[threadIdx.x], 1u);
    }
}

}  // namespace alice
