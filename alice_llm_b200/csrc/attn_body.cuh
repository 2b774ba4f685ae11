// Device body of the fused decode attention: RoPE + KV append + split-KV GQA attention + split combine, for one
// token or a batch of consecutive tokens (causal). Arithmetic: ALICE-LLM src/llama3.rs apply_rope :5323-5333,
// :5367-5378, KvCache::append :4773, gqa_attention :5431-5690, evaluated as an online softmax over KV splits; the
// batch form is the causal rule of src/shaders/attention.wgsl:45 (token k at position base + k attends base + k + 1 rows).
#pragma once
#include "common.cuh"
#include "glue.cuh"
#include "publish.cuh"
#include "q8k.cuh"

namespace alice {

struct RopeCoef { float sn[4], cs[4]; };
// Rotation table of one position: tab[2*j] = sin, tab[2*j + 1] = cos of pos * freq[j], j = 0 .. head_dim/2 - 1
// (head_dim = 128). freq[j] = 1 / theta^(2j / head_dim) is computed on the HOST at model creation with the same libm
// powf the CPU path uses: at a position of several thousand a one-ulp difference in freq already moves the angle by
// ~1e-3 rad, which the attention scores amplify. The table depends on the position only, so it is computed once per
// decode step (by the embedding stage) and every layer's attention reads it.
__device__ __forceinline__ void rope_table_entry(float* tab, uint32_t j, uint32_t pos, const float* __restrict__ freq) {
    float sn, cs;
    sincosf(__fmul_rn((float)pos, __ldg(freq + j)), &sn, &cs);
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
// One CTA = one KV head x one slice of positions x one token of the batch; its GROUP = num_heads/num_kv_heads query
// heads share every K and V row it reads. Each warp walks positions t, t+NW, ...; a lane owns 4 of the 128 dims.
// qkv[k] = [q | k | v] of batch token k, un-rotated: q and k are rotated here. Rows of the tokens of this very batch
// (positions >= pos0) are taken from qkv, not from the cache - their cache rows are being written by this launch -
// and token k's own row is written to the cache at pos0 + k by the CTA whose slice contains it.
// Per (token, split, head) the CTA leaves (max, sum, accumulator); the last CTA of a (token, KV head) to finish
// (ticket counter) folds the splits into attn_out for its heads.
template <int GROUP>
struct AttnSmem {
    float m[8][GROUP], l[8][GROUP];
    float4 acc[8][GROUP][32];
    double red[8];
    unsigned int last;
    int gate_ok;
};

template <int GROUP>
__device__ __forceinline__ void attn_fused_body(const AttnArgs& a, uint32_t pos0, uint32_t kvh, uint32_t split, uint32_t bk,
                                                AttnSmem<GROUP>* sh) {
    constexpr int NW = 8;
    const AttnShape s = a.shape;
    const uint32_t pos = pos0 + bk;            // position of this CTA's token
    const uint32_t seq = pos + 1;
    const uint32_t nsplit = a.nsplit;
    const uint32_t per = (seq + nsplit - 1) / nsplit;
    const uint32_t t0 = split * per, t1 = min(seq, t0 + per);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_dim = s.num_heads * s.head_dim, kv_dim = s.num_kv_heads * s.head_dim;
    const uint32_t qkv_stride = q_dim + 2 * kv_dim;
    const float* __restrict__ qkv = a.qkv + (size_t)bk * qkv_stride;
    float* __restrict__ kcache = a.kcache;
    float* __restrict__ vcache = a.vcache;
    const float inv_sqrt_d = __fdiv_rn(1.0f, sqrtf((float)s.head_dim));
    const int neox = a.neox;

    // KB positions per warp round: their 2*KB row loads are issued before the first is used, so a round costs one
    // memory round trip instead of KB (positions are still folded in ascending order). The first round is requested
    // before q and the rotation table are looked at: none of these loads depends on another.
    constexpr int KB = 4;
    float4 k[KB], v[KB];
    auto load_round = [&](uint32_t tb) {
#pragma unroll
        for (int j = 0; j < KB; j++) {
            const uint32_t t = tb + j * NW;
            k[j] = v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < t1 && t < pos0) {
                k[j] = __ldcg(reinterpret_cast<const float4*>(kcache + (size_t)t * kv_dim + kvh * s.head_dim) + lane);
                v[j] = __ldcg(reinterpret_cast<const float4*>(vcache + (size_t)t * kv_dim + kvh * s.head_dim) + lane);
            }
        }
    };
    float4 q[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; g++) q[g] = __ldcg(reinterpret_cast<const float4*>(qkv + (size_t)(kvh * GROUP + g) * s.head_dim) + lane);
    if (t0 + warp < t1) load_round(t0 + warp);
    const RopeCoef rc = rope_coef(a.rope_tab + (size_t)bk * 128, lane, neox);
#pragma unroll
    for (int g = 0; g < GROUP; g++) q[g] = rope4(q[g], lane, rc, neox);
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
                if (t >= pos0) {   // a token of this batch: rotate its K here; the token's own CTA appends K and V (KvCache::append, src/llama3.rs:4773)
                    const uint32_t bj = t - pos0;
                    const float* __restrict__ src = a.qkv + (size_t)bj * qkv_stride;
                    const RopeCoef rj = bj == bk ? rc : rope_coef(a.rope_tab + (size_t)bj * 128, lane, neox);
                    k[j] = rope4(__ldcg(reinterpret_cast<const float4*>(src + q_dim + (size_t)kvh * s.head_dim) + lane), lane, rj, neox);
                    v[j] = __ldcg(reinterpret_cast<const float4*>(src + q_dim + kv_dim + (size_t)kvh * s.head_dim) + lane);
                    if (bj == bk) {
                        reinterpret_cast<float4*>(kcache + (size_t)t * kv_dim + kvh * s.head_dim)[lane] = k[j];
                        reinterpret_cast<float4*>(vcache + (size_t)t * kv_dim + kvh * s.head_dim)[lane] = v[j];
                    }
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
    // combine the NW warps of the CTA
#pragma unroll
    for (int g = 0; g < GROUP; g++) {
        if (lane == 0) { sh->m[warp][g] = m[g]; sh->l[warp][g] = l[g]; }
        sh->acc[warp][g][lane] = acc[g];
    }
    __syncthreads();
    const uint32_t stride = s.head_dim + 4;   // (m, l, pad, pad, acc[128]): keeps acc 16-byte aligned
    float* __restrict__ part = a.part + (size_t)bk * nsplit * s.num_heads * stride;
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
                const float4 av = sh->acc[w][g][lane];
                A.x += av.x * c; A.y += av.y * c; A.z += av.z * c; A.w += av.w * c;
            }
        }
        float* out = part + ((size_t)split * s.num_heads + kvh * GROUP + g) * stride;
        if (lane == 0) { out[0] = M; out[1] = L; }
        reinterpret_cast<float4*>(out + 4)[lane] = A;
    }
    // last CTA of this (token, KV head) folds the splits
    __threadfence();
    __syncthreads();
    unsigned int* ticket_p = a.tickets + bk * s.num_kv_heads + kvh;
    if (threadIdx.x == 0) {
        const unsigned int ticket = atomicAdd(ticket_p, 1u);
        sh->last = (ticket == nsplit - 1) ? 1u : 0u;
        if (sh->last) *ticket_p = 0;   // ready for the next launch
    }
    __syncthreads();
    if (!sh->last) return;
    __threadfence();
    float* __restrict__ attn_out = a.attn_out + (size_t)bk * a.out_stride;
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
        constexpr int SB = 16;   // split accumulators fetched per round trip
        for (uint32_t sp0 = 0; sp0 < nsplit; sp0 += SB) {
            float4 av[SB];
#pragma unroll
            for (int j = 0; j < SB; j++)
                if (sp0 + j < nsplit)
                    av[j] = __ldcg(reinterpret_cast<const float4*>(part + ((size_t)(sp0 + j) * s.num_heads + head) * stride + 4) + lane);
#pragma unroll
            for (int j = 0; j < SB; j++) {
                const uint32_t sp = sp0 + j;
                const float c = __shfl_sync(0xffffffffu, sp < 32 ? cs[0] : cs[1], sp & 31);
                if (sp < nsplit) { A.x += av[j].x * c; A.y += av[j].y * c; A.z += av[j].z * c; A.w += av[j].w * c; }
            }
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        const float4 o = make_float4(A.x * inv, A.y * inv, A.z * inv, A.w * inv);
        reinterpret_cast<float4*>(attn_out + (size_t)head * s.head_dim)[lane] = o;
        for (uint32_t p = 0; p < a.npeers; p++)
            reinterpret_cast<float4*>(a.peer_out[p] + (size_t)bk * a.out_stride + (size_t)head * s.head_dim)[lane] = o;
        o_keep = o;
    }
    if (a.q8.qs != nullptr && (GROUP % 2) == 0) {
        // Q8_K of this KV head's GROUP * 128 outputs = GROUP / 2 whole blocks (quantize_row_q8_k, src/gguf.rs:1323): the
        // outputs go through shared memory so that a warp sees the two heads of its block
        __syncthreads();                      // the split accumulators in sh->acc are no longer needed
        if (warp < GROUP) sh->acc[0][warp][lane] = o_keep;
        __syncthreads();
        if (warp < GROUP / 2) {
            const uint32_t nb = q_dim / QK_K;
            const size_t blk = (size_t)bk * nb + (kvh * GROUP) / 2 + warp;
            const int hsel = 2 * (int)warp + (int)(lane >> 4);
            Q8KLaneInput in;
            in.a = sh->acc[0][hsel][(lane & 15) * 2];
            in.b = sh->acc[0][hsel][(lane & 15) * 2 + 1];
            q8k_quantize_block_warp(in, lane, a.q8.qs + blk * QK_K, a.q8.d + blk, a.q8.bsums + blk * 16);
        }
    }
}

}  // namespace alice
