// Per-token glue of the Llama decode step around the matvec kernels: embedding row, RoPE + KV
// append, split-KV GQA attention, greedy argmax. All read the position / token from device memory
// so one captured CUDA graph serves every step. Arithmetic follows ALICE-LLM src/llama3.rs:
// apply_rope :5323-5333, KvCache::append :4773, gqa_attention :5431-5690 (scores q.k/sqrt(d),
// softmax, weighted V sum; evaluated here as an online softmax over KV splits, which reorders
// the f32 sums but not the math).
#include "common.cuh"
#include "glue.cuh"

namespace alice {

// hidden[c] = d * q of row `token` of a Q8_0 table (dequantize_q8_0, src/gguf.rs:990-1004); the
// CPU model dequantizes the whole table at load (src/llama3.rs:12890) and copies a row per token.
__global__ void embed_q8_0_kernel(const uint8_t* __restrict__ table, const int* __restrict__ token, uint32_t cols,
                                  uint32_t vocab, float* __restrict__ hidden) {
    pdl_wait();
    pdl_launch_dependents();
    uint32_t t = (uint32_t)*token;
    if (t >= vocab) t = 0;
    const uint8_t* row = table + (size_t)t * (cols / 32) * 34;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        const uint8_t* b = row + (c >> 5) * 34;
        const float d = f16_bits_to_f32((uint32_t)b[0] | ((uint32_t)b[1] << 8));
        hidden[c] = __fmul_rn(d, (float)(int8_t)b[2 + (c & 31)]);
    }
}

// RoPE on the q and k heads of qkv = [q | k | v] in place (pairs (i, i+1), or (i, i+d/2) for the
// NeoX layout), then K and V of this position go into the cache at [pos][kv_dim].
__global__ void rope_kv_kernel(float* __restrict__ qkv, const int* __restrict__ pos_ptr, AttnShape s, float theta,
                               int neox, float* __restrict__ kcache, float* __restrict__ vcache) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t pos = (uint32_t)*pos_ptr;
    const uint32_t half = s.head_dim / 2;
    const uint32_t q_pairs = s.num_heads * half, k_pairs = s.num_kv_heads * half;
    const uint32_t q_dim = s.num_heads * s.head_dim, kv_dim = s.num_kv_heads * s.head_dim;
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (tid < q_pairs + k_pairs) {
        const bool is_k = tid >= q_pairs;
        const uint32_t p = is_k ? tid - q_pairs : tid;
        const uint32_t h = p / half, j = p % half;
        float* v = qkv + (is_k ? q_dim : 0) + h * s.head_dim;
        const uint32_t i0 = neox ? j : 2 * j, i1 = neox ? j + half : 2 * j + 1;
        // freq = 1 / theta^(i / head_dim) with i the even index 2j (both layouts)
        const float freq = __fdiv_rn(1.0f, powf(theta, __fdiv_rn((float)(2 * j), (float)s.head_dim)));
        const float angle = __fmul_rn((float)pos, freq);
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const float x0 = v[i0], x1 = v[i1];
        const float r0 = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        const float r1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
        v[i0] = r0; v[i1] = r1;
        if (is_k) {
            float* kc = kcache + (size_t)pos * kv_dim + h * s.head_dim;
            kc[i0] = r0; kc[i1] = r1;
        }
    } else if (tid < q_pairs + k_pairs + kv_dim) {
        const uint32_t i = tid - q_pairs - k_pairs;
        vcache[(size_t)pos * kv_dim + i] = qkv[q_dim + kv_dim + i];
    }
}

// One CTA = one KV head x one slice of positions; its GROUP = num_heads/num_kv_heads query heads share
// every K and V row it reads. Each warp walks positions t, t+NW, ...; a lane owns 4 of the 128 dims.
// Output per (split, head): running max m, sum l and the un-normalised accumulator acc[head_dim].
template <int GROUP>
__global__ void __launch_bounds__(256) attn_split_kernel(const float* __restrict__ qkv, const float* __restrict__ kcache,
                                                         const float* __restrict__ vcache,
                                                         const int* __restrict__ pos_ptr, AttnShape s, uint32_t nsplit,
                                                         float* __restrict__ part) {
    constexpr int NW = 8;
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t kvh = blockIdx.x, split = blockIdx.y;
    const uint32_t seq = (uint32_t)*pos_ptr + 1;
    const uint32_t per = (seq + nsplit - 1) / nsplit;
    const uint32_t t0 = split * per, t1 = min(seq, t0 + per);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t kv_dim = s.num_kv_heads * s.head_dim;
    const float inv_sqrt_d = __fdiv_rn(1.0f, sqrtf((float)s.head_dim));

    float4 q[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; g++)
        q[g] = reinterpret_cast<const float4*>(qkv + (size_t)(kvh * GROUP + g) * s.head_dim)[lane];
    float m[GROUP], l[GROUP];
    float4 acc[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; g++) { m[g] = -INFINITY; l[g] = 0.0f; acc[g] = make_float4(0.f, 0.f, 0.f, 0.f); }

    for (uint32_t t = t0 + warp; t < t1; t += NW) {
        const float4 k = reinterpret_cast<const float4*>(kcache + (size_t)t * kv_dim + kvh * s.head_dim)[lane];
        const float4 v = reinterpret_cast<const float4*>(vcache + (size_t)t * kv_dim + kvh * s.head_dim)[lane];
        float sc[GROUP];
#pragma unroll
        for (int g = 0; g < GROUP; g++) sc[g] = q[g].x * k.x + q[g].y * k.y + q[g].z * k.z + q[g].w * k.w;
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
            acc[g].x = acc[g].x * corr + p * v.x; acc[g].y = acc[g].y * corr + p * v.y;
            acc[g].z = acc[g].z * corr + p * v.z; acc[g].w = acc[g].w * corr + p * v.w;
            m[g] = mn;
        }
    }
    // combine the NW warps of the CTA
    __shared__ float sm_m[NW][GROUP], sm_l[NW][GROUP];
    __shared__ float4 sm_acc[NW][GROUP][32];
#pragma unroll
    for (int g = 0; g < GROUP; g++) {
        if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
        sm_acc[warp][g][lane] = acc[g];
    }
    __syncthreads();
    if (warp < GROUP) {
        const int g = warp;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) M = fmaxf(M, sm_m[w][g]);
        float L = 0.0f;
        float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < NW; w++) {
                const float c = expf(sm_m[w][g] - M);   // exp(-inf) = 0 for warps that saw no position
                L += sm_l[w][g] * c;
                const float4 a = sm_acc[w][g][lane];
                A.x += a.x * c; A.y += a.y * c; A.z += a.z * c; A.w += a.w * c;
            }
        }
        const uint32_t head = kvh * GROUP + g;
        float* out = part + ((size_t)split * s.num_heads + head) * (s.head_dim + 2);
        if (lane == 0) { out[0] = M; out[1] = L; }
        out[2 + 4 * lane] = A.x; out[3 + 4 * lane] = A.y; out[4 + 4 * lane] = A.z; out[5 + 4 * lane] = A.w;
    }
}

// attn_out[head][d] = sum_s exp(m_s - M) acc_s[d] / sum_s exp(m_s - M) l_s
__global__ void attn_combine_kernel(const float* __restrict__ part, AttnShape s, uint32_t nsplit,
                                    float* __restrict__ attn_out) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t head = blockIdx.x, d = threadIdx.x;
    if (d >= s.head_dim) return;
    const uint32_t stride = s.head_dim + 2;
    float M = -INFINITY;
    for (uint32_t sp = 0; sp < nsplit; sp++) M = fmaxf(M, part[((size_t)sp * s.num_heads + head) * stride]);
    float L = 0.0f, A = 0.0f;
    for (uint32_t sp = 0; sp < nsplit; sp++) {
        const float* p = part + ((size_t)sp * s.num_heads + head) * stride;
        if (p[0] == -INFINITY) continue;
        const float c = expf(p[0] - M);
        L += p[1] * c;
        A += p[2 + d] * c;
    }
    attn_out[(size_t)head * s.head_dim + d] = L > 0.0f ? A / L : 0.0f;
}

// Greedy next token: index of the largest logit (lowest index on ties); also advances the position.
__global__ void __launch_bounds__(1024) argmax_advance_kernel(const float* __restrict__ logits, uint32_t n,
                                                              int* __restrict__ token, int* __restrict__ pos,
                                                              int* __restrict__ trace, int write_token) {
    pdl_wait();
    pdl_launch_dependents();
    float best = -INFINITY;
    uint32_t bi = 0xFFFFFFFFu;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = logits[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < (blockDim.x >> 5); w++)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        const int p = *pos;
        if (write_token) { *token = (int)bi; if (trace) trace[p] = (int)bi; }
        *pos = p + 1;
    }
}

static void launch_cfg(cudaLaunchConfig_t& lc, cudaLaunchAttribute* at, dim3 grid, dim3 block, cudaStream_t st, bool pdl) {
    lc = {};
    lc.gridDim = grid; lc.blockDim = block; lc.dynamicSmemBytes = 0; lc.stream = st;
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = pdl ? 1 : 0;
}

cudaError_t launch_embed_q8_0(const uint8_t* table, const int* token, uint32_t cols, uint32_t vocab, float* hidden,
                              cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3((cols + 255) / 256), dim3(256), st, pdl);
    return cudaLaunchKernelEx(&lc, embed_q8_0_kernel, table, token, cols, vocab, hidden);
}

cudaError_t launch_rope_kv(float* qkv, const int* pos, AttnShape s, float theta, int neox, float* kc, float* vc,
                           cudaStream_t st, bool pdl) {
    const uint32_t n = (s.num_heads + s.num_kv_heads) * (s.head_dim / 2) + s.num_kv_heads * s.head_dim;
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3((n + 255) / 256), dim3(256), st, pdl);
    return cudaLaunchKernelEx(&lc, rope_kv_kernel, qkv, pos, s, theta, neox, kc, vc);
}

cudaError_t launch_attention(const float* qkv, const float* kc, const float* vc, const int* pos, AttnShape s,
                             uint32_t nsplit, float* part, float* attn_out, cudaStream_t st, bool pdl) {
    if (s.head_dim != 128 || s.num_heads % s.num_kv_heads) return cudaErrorInvalidValue;
    const uint32_t group = s.num_heads / s.num_kv_heads;
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3(s.num_kv_heads, nsplit), dim3(256), st, pdl);
    cudaError_t err;
    switch (group) {
        case 1: err = cudaLaunchKernelEx(&lc, attn_split_kernel<1>, qkv, kc, vc, pos, s, nsplit, part); break;
        case 2: err = cudaLaunchKernelEx(&lc, attn_split_kernel<2>, qkv, kc, vc, pos, s, nsplit, part); break;
        case 4: err = cudaLaunchKernelEx(&lc, attn_split_kernel<4>, qkv, kc, vc, pos, s, nsplit, part); break;
        case 5: err = cudaLaunchKernelEx(&lc, attn_split_kernel<5>, qkv, kc, vc, pos, s, nsplit, part); break;
        case 8: err = cudaLaunchKernelEx(&lc, attn_split_kernel<8>, qkv, kc, vc, pos, s, nsplit, part); break;
        default: return cudaErrorInvalidValue;
    }
    if (err != cudaSuccess) return err;
    launch_cfg(lc, at, dim3(s.num_heads), dim3(128), st, pdl);
    return cudaLaunchKernelEx(&lc, attn_combine_kernel, (const float*)part, s, nsplit, attn_out);
}

cudaError_t launch_argmax_advance(const float* logits, uint32_t n, int* token, int* pos, int* trace, int write_token,
                                  cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3(1), dim3(1024), st, pdl);
    return cudaLaunchKernelEx(&lc, argmax_advance_kernel, logits, n, token, pos, trace, write_token);
}

}  // namespace alice
