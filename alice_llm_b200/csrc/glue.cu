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
__global__ void embed_q8_0_kernel(const uint8_t* __restrict__ table, const int* __restrict__ token, uint32_t cols,
                                  uint32_t vocab, float* __restrict__ hidden, const int* __restrict__ pos, float theta,
                                  float* __restrict__ rope_tab, const EmbedTag tag) {
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x == 0 && threadIdx.x < 64) rope_table_entry(rope_tab, threadIdx.x, (uint32_t)*pos, theta);
    uint32_t t = (uint32_t)*token;
    if (t >= vocab) t = 0;
    const uint8_t* row = table + (size_t)t * (cols / 32) * 34;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        const uint8_t* b = row + (c >> 5) * 34;
        const float d = f16_bits_to_f32((uint32_t)b[0] | ((uint32_t)b[1] << 8));
        const float v = __fmul_rn(d, (float)(int8_t)b[2 + (c & 31)]);
        hidden[c] = v;
        if (tag.hidden_ll) ll_store(tag.hidden_ll + c, v, ld_acquire_sys_u32(tag.epoch) * tag.tag_n + 1u);
    }
}

// RoPE (apply_rope / apply_rope_neox, src/llama3.rs:5323-5333, 5367-5378): pairs (i, i+1), or (i, i + d/2)
// for NeoX, freq = 1 / theta^(i_even / d), angle = pos * freq; a lane owns dims 4*lane .. 4*lane+3 of a
// head vector (head_dim = 128, so a NeoX partner sits in lane ^ 16).
template <int GROUP>
__global__ void __launch_bounds__(256, GROUP <= 5 ? 2 : 1) attn_fused_kernel(const float* __restrict__ qkv, float* __restrict__ kcache,
                                                         float* __restrict__ vcache, const int* __restrict__ pos_ptr,
                                                         AttnShape s, const float* __restrict__ rope_tab, int neox, uint32_t nsplit,
                                                         float* __restrict__ part, unsigned int* __restrict__ tickets,
                                                         float* __restrict__ attn_out, const AttnPeers peers,
                                                         const AttnQ8Out q8out) {
    __shared__ AttnSmem<GROUP> sh;
    pdl_wait();
    pdl_launch_dependents();
    attn_fused_body<GROUP, false>(qkv, kcache, vcache, (uint32_t)*pos_ptr, s, rope_tab, neox, nsplit, part, tickets, attn_out,
                                  blockIdx.x, blockIdx.y, &sh, nullptr, &peers, &q8out);
}

// Turns the packed (ordered logit, ~row) maxima the output-head kernels accumulated - one per rank of a
// tensor-parallel group, each over that rank's rows, gathered to every rank - into the next token,
// records it, advances the position and clears the keys for the next step.
__global__ void finish_step_kernel(unsigned long long* __restrict__ keys, uint32_t nkeys, int* __restrict__ token,
                                   int* __restrict__ pos, int* __restrict__ trace, int write_token, const StepPeers peers) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        unsigned int e = 0;
        if (peers.npeers) {
            // publish this rank's maximum, then wait for the peers' maxima and for their rows of the logits vector
            const unsigned long long mine = keys[peers.rank];
            for (uint32_t p = 0; p < peers.npeers; p++) peers.keys[p][peers.rank] = mine;
            __threadfence_system();
            for (uint32_t p = 0; p < peers.npeers; p++) red_release_sys_add_u32(peers.key_flag[p], 1u);
            e = *peers.epoch;
            peer_wait(peers.my_key_flag, (e + 1u) * peers.npeers, peers.status, KERR_WAIT_PEER);
            peer_wait(peers.my_logits_flag, (e + 1u) * peers.logits_mult, peers.status, KERR_WAIT_PEER);
        }
        unsigned long long k = 0ull;
        for (uint32_t i = 0; i < nkeys; i++) {
            const unsigned long long ki = peers.npeers ? __ldcg(keys + i) : keys[i];
            k = ki > k ? ki : k;
            keys[i] = 0ull;
        }
        const int p = *pos;
        if (write_token) {
            const int t = (int)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
            *token = t;
            if (trace) trace[p] = t;
        }
        *pos = p + 1;
        if (peers.npeers) *peers.epoch = e + 1u;
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
                              const int* pos, float theta, float* rope_tab, const EmbedTag& tag, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3((cols + 255) / 256), dim3(256), st, pdl);
    return cudaLaunchKernelEx(&lc, embed_q8_0_kernel, table, token, cols, vocab, hidden, pos, theta, rope_tab, tag);
}

cudaError_t launch_attention(const float* qkv, float* kc, float* vc, const int* pos, AttnShape s, const float* rope_tab, int neox,
                             uint32_t nsplit, float* part, unsigned int* tickets, float* attn_out, const AttnPeers& peers,
                             const AttnQ8Out& q8out, cudaStream_t st, bool pdl) {
    if (s.head_dim != 128 || s.num_heads % s.num_kv_heads) return cudaErrorInvalidValue;
    const uint32_t group = s.num_heads / s.num_kv_heads;
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3(s.num_kv_heads, nsplit), dim3(256), st, pdl);
    switch (group) {
        case 1: return cudaLaunchKernelEx(&lc, attn_fused_kernel<1>, qkv, kc, vc, pos, s, rope_tab, neox, nsplit, part, tickets, attn_out, peers, q8out);
        case 2: return cudaLaunchKernelEx(&lc, attn_fused_kernel<2>, qkv, kc, vc, pos, s, rope_tab, neox, nsplit, part, tickets, attn_out, peers, q8out);
        case 4: return cudaLaunchKernelEx(&lc, attn_fused_kernel<4>, qkv, kc, vc, pos, s, rope_tab, neox, nsplit, part, tickets, attn_out, peers, q8out);
        case 5: return cudaLaunchKernelEx(&lc, attn_fused_kernel<5>, qkv, kc, vc, pos, s, rope_tab, neox, nsplit, part, tickets, attn_out, peers, q8out);
        case 8: return cudaLaunchKernelEx(&lc, attn_fused_kernel<8>, qkv, kc, vc, pos, s, rope_tab, neox, nsplit, part, tickets, attn_out, peers, q8out);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_finish_step(unsigned long long* keys, uint32_t nkeys, int* token, int* pos, int* trace, int write_token,
                               const StepPeers& peers, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t lc; cudaLaunchAttribute at[1];
    launch_cfg(lc, at, dim3(1), dim3(32), st, pdl);
    return cudaLaunchKernelEx(&lc, finish_step_kernel, keys, nkeys, token, pos, trace, write_token, peers);
}

}  // namespace alice
