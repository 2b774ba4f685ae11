// Launchers of the per-token glue kernels (csrc/glue.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "publish.cuh"

namespace alice {

struct AttnShape { uint32_t num_heads, num_kv_heads, head_dim; };   // this GPU's heads

// Optional Q8_K copy of the attention output for a K-quant output projection: the CTA that finishes a KV head holds
// whole 256-element blocks of it (when the heads of a KV head are an even number), so it quantizes them on the spot.
struct AttnQ8Out {
    int8_t* qs = nullptr;     // [batch][q_dim]
    float* d = nullptr;       // [batch][q_dim / 256]
    int16_t* bsums = nullptr; // [batch][q_dim / 16]
};

struct AttnArgs {
    const float* qkv;          // [batch][q | k | v] of the current tokens, un-rotated
    float* kcache;             // this layer's cache, [max_seq][kv_dim]
    float* vcache;
    const int* pos;            // position of batch token 0 (device)
    AttnShape shape;
    const float* rope_tab;     // [batch][128]: (sin, cos) per rotation pair at each token's position
    int neox;
    uint32_t nsplit;
    float* part;               // [batch][nsplit][num_heads][head_dim + 4]
    unsigned int* tickets;     // [batch][num_kv_heads], zero between launches
    float* attn_out;           // [batch][out_stride]; this GPU's heads start at attn_out (already offset by the caller)
    uint32_t out_stride;
    AttnQ8Out q8;
    // tensor parallel: the output of this GPU's heads also goes to the same place of every peer's vector (the hand-over
    // is a kernel of its own behind this one)
    uint32_t npeers;
    float* peer_out[MAX_PEERS];
    int* status;
};

struct EmbedArgs {
    const uint8_t* table;      // Q8_0 [vocab][cols]
    const int* tokens;         // [batch] (device)
    uint32_t cols, vocab, batch;
    float* hidden;             // [batch][cols]
    const int* pos;            // position of batch token 0
    const float* rope_freq;    // [64]
    float* rope_tab;           // [batch][128]
    Publish pub;               // hidden prepared for the first layer (PUB_VECTOR, or PUB_NONE)
    int* status;
};

// hidden[k] <- dequantized row tokens[k] of the Q8_0 table; rope_tab[k] <- (sin, cos) of (pos + k) * freq[j]; then the
// prepared form of hidden for the first projection. One CTA.
cudaError_t launch_embed_q8_0(const EmbedArgs& a, cudaStream_t st, bool pdl);
cudaError_t launch_attention(const AttnArgs& a, uint32_t batch, cudaStream_t st, bool pdl);
// token <- index held in the largest of keys[0 .. nkeys) (packed maxima written by the output-head kernels, one per
// tensor-parallel rank) when write_token; pos <- pos + advance; keys <- 0; *epoch += 1 (decode steps completed: the
// tensor-parallel hand-over counters are compared against it)
cudaError_t launch_finish_step(unsigned long long* keys, uint32_t nkeys, int* token, int* pos, int* trace, int write_token,
                               uint32_t advance, unsigned int* epoch, cudaStream_t st, bool pdl);
}  // namespace alice
