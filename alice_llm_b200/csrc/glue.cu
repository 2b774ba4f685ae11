// Per-token glue of the Llama decode step around the matvec kernels: embedding row, RoPE + KV
// append, split-KV GQA attention, greedy argmax. All read the position / token from device memory
// so one captured CUDA graph serves every step. Arithmetic follows ALICE-LLM src/llama3.rs:
// apply_rope :5323-5333, KvCache::append :4773, gqa_attention :5431-5690 (scores q.k/sqrt(d),
// softmax, weighted V sum; evaluated here as an online softmax over KV splits, which reorders
// the f32 sums but not the math).
#include "common.cuh"
#include "glue.cuh"
#include "attn_body.cuh"

namespace alice {

// hidden[c] = d * q of row `token` of a Q8_0 table (dequantize_q8_0, src/gguf.rs:990-1004); the
// CPU model dequantizes the whole table at load (src/llama3.rs:12890) and copies a row per token.
__global__ void __launch_bounds__(256) embed_q8_0_kernel(const __grid_constant__ EmbedArgs a) {
    __shared__ double red[8];
    pdl_launch_dependents();   // the next kernel may become resident (and prefetch its weights) while this one waits
    pdl_wait();
    const uint32_t pos0 = (uint32_t)*a.pos;
    for (uint32_t i = threadIdx.x; i < 64 * a.batch; i += blockDim.x) rope_table_entry(a.rope_tab + (size_t)(i >> 6) * 128, i & 63, pos0 + (i >> 6), a.rope_freq);
    // one thread per 34-byte block (f16 scale + 32 int8): 17 independent 16-bit loads, so the row costs one memory
    // round trip instead of one per element
    const uint32_t nblk = a.cols / 32;
    for (uint32_t i = threadIdx.x; i < nblk * a.batch; i += blockDim.x) {
        const uint32_t k = i / nblk, b = i % nblk;
        uint32_t t = (uint32_t)a.tokens[k];
        if (t >= a.vocab) t = 0;
        const unsigned short* src = reinterpret_cast<const unsigned short*>(a.table + (size_t)t * nblk * 34 + (size_t)b * 34);
        unsigned short h[17];
#pragma unroll
        for (int j = 0; j < 17; j++) h[j] = __ldg(src + j);
        const float d = f16_bits_to_f32(h[0]);
        float* out = a.hidden + (size_t)k * a.cols + (size_t)b * 32;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            out[2 * j] = __fmul_rn(d, (float)(int8_t)(h[1 + j] & 0xff));
            out[2 * j + 1] = __fmul_rn(d, (float)(int8_t)(h[1 + j] >> 8));
        }
    }
    if (a.pub.mode == PUB_VECTOR && (a.pub.dst.qs != nullptr || a.pub.dst.xn != nullptr)) {
        __threadfence();
        __syncthreads();
        publish_vector<8, 0>(a.pub, red, true);
    }
}

// RoPE (apply_rope / apply_rope_neox, src/llama3.rs:5323-5333, 5367-5378): pairs (i, i+1), or (i, i + d/2)
// for NeoX, freq = 1 / theta^(i_even / d), angle = pos * freq; a lane owns dims 4*lane .. 4*lane+3 of a
// head vector (head_dim = 128, so a NeoX partner sits in lane ^ 16).
template <int GROUP>
__global__ void __launch_bounds__(256, GROUP <= 5 ? 2 : 1) attn_fused_kernel(const __grid_constant__ AttnArgs a) {
    __shared__ AttnSmem<GROUP> sh;
    pdl_launch_dependents();   // the next kernel may become resident (and prefetch its weights) while this one waits
    pdl_wait();
    attn_fused_body<GROUP>(a, (uint32_t)*a.pos, blockIdx.x, blockIdx.y, blockIdx.z, &sh);
}

// Turns the packed (ordered logit, ~row) maxima the output-head kernels accumulated - one per rank of a
// tensor-parallel group, each over that rank's rows, all present on every rank by now - into the next token,
// records it, advances the position and clears the keys for the next step.
__global__ void finish_step_kernel(unsigned long long* __restrict__ keys, uint32_t nkeys, int* __restrict__ token,
                                   int* __restrict__ pos, int* __restrict__ trace, int write_token, uint32_t advance,
                                   unsigned int* __restrict__ epoch) {
    pdl_launch_dependents();   // the next kernel may become resident (and prefetch its weights) while this one waits
    pdl_wait();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        unsigned long long k = 0ull;
        for (uint32_t i = 0; i < nkeys; i++) {
            const unsigned long long ki = __ldcg(keys + i);
            k = ki > k ? ki : k;
            keys[i] = 0ull;
        }
        const int p = *pos;
        if (write_token) {
            const int t = (int)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
            *token = t;
            if (trace) trace[p] = t;
        }
        *pos = p + (int)advance;
        if (epoch) *epoch = *epoch + 1u;
    }
}

static void launch_cfg(cudaLaunchConfig_t& lc, cudaLaunchAttribute* at, dim3 grid, dim3 block, cudaStream_t st, bool pdl) {
    lc = {};
    lc.gridDim = grid; lc.blockDim = block; lc.dynamicSmemBytes = 0; lc.stream = st;
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = pdl ? 1 : 0;
}

cudaError_t launch_embed_q8_0(const EmbedArgs& a, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3(1), dim3(256), st, pdl);
    return cudaLaunchKernelEx(&lc, embed_q8_0_kernel, a);
}

cudaError_t launch_attention(const AttnArgs& a, uint32_t batch, cudaStream_t st, bool pdl) {
    const AttnShape& s = a.shape;
    if (s.head_dim != 128 || s.num_heads % s.num_kv_heads) return cudaErrorInvalidValue;
    const uint32_t group = s.num_heads / s.num_kv_heads;
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3(s.num_kv_heads, a.nsplit, batch), dim3(256), st, pdl);
    switch (group) {
        case 1: return cudaLaunchKernelEx(&lc, attn_fused_kernel<1>, a);
        case 2: return cudaLaunchKernelEx(&lc, attn_fused_kernel<2>, a);
        case 4: return cudaLaunchKernelEx(&lc, attn_fused_kernel<4>, a);
        case 5: return cudaLaunchKernelEx(&lc, attn_fused_kernel<5>, a);
        case 8: return cudaLaunchKernelEx(&lc, attn_fused_kernel<8>, a);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_finish_step(unsigned long long* keys, uint32_t nkeys, int* token, int* pos, int* trace, int write_token,
                               uint32_t advance, unsigned int* epoch, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3(1), dim3(32), st, pdl);
    return cudaLaunchKernelEx(&lc, finish_step_kernel, keys, nkeys, token, pos, trace, write_token, advance, epoch);
}

}  // namespace alice
