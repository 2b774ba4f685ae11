// Launchers of the per-token glue kernels (csrc/glue.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace alice {

struct AttnShape { uint32_t num_heads, num_kv_heads, head_dim; };
// Optional Q8_K copy of the attention output for a K-quant output projection: the CTA that finishes a KV head holds
// whole 256-element blocks of it (when the heads of a KV head are an even number), so it quantizes them on the spot and
// the projection starts from int8 activations instead of quantizing the whole vector in every CTA.
struct AttnQ8Out {
    int8_t* qs = nullptr;     // [q_dim]
    float* d = nullptr;       // [q_dim / 256]
    int16_t* bsums = nullptr; // [q_dim / 256][16]
};
// Tensor parallel: the attention output of this GPU's heads also goes to the same place of every peer's vector,
// and the CTA that finished a KV head adds 1 to the arrival counter on every peer.
struct AttnPeers {
    uint32_t npeers = 0;
    float* out[7] = {};
    unsigned int* flag[7] = {};
    // tagged form instead (see ll_store): this GPU's copy and the peers', both already offset to this GPU's heads;
    // tag = *epoch * tag_n + tag_seq + 1
    uint2* out_ll = nullptr;
    uint2* peer_ll[7] = {};
    const unsigned int* epoch = nullptr;
    uint32_t tag_seq = 0, tag_n = 0;
};
// Tagged copy of the embedding output (the first input of the layer stack), tag = *epoch * tag_n + 1.
struct EmbedTag {
    uint2* hidden_ll = nullptr;
    const unsigned int* epoch = nullptr;
    uint32_t tag_n = 0;
};
// Tensor parallel token hand-over: every rank publishes the packed maximum of its vocabulary rows to all peers.
struct StepPeers {
    uint32_t npeers = 0, rank = 0;
    unsigned long long* keys[7] = {};   // the key array of each peer
    unsigned int* key_flag[7] = {};     // its arrival counter on each peer
    const unsigned int* my_key_flag = nullptr;
    const unsigned int* my_logits_flag = nullptr;   // rows of the logits vector pushed by the peers' head kernels
    uint32_t logits_mult = 0;
    unsigned int* epoch = nullptr;      // decode steps completed, on this GPU
    int* status = nullptr;
};

// hidden <- dequantized row *token of the Q8_0 table; rope_tab (128 floats) <- (sin, cos) of *pos * theta^(-2j/128)
cudaError_t launch_embed_q8_0(const uint8_t* table, const int* token, uint32_t cols, uint32_t vocab, float* hidden,
                              const int* pos, float theta, float* rope_tab, const EmbedTag& tag, cudaStream_t st, bool pdl);
// qkv = [q (num_heads*head_dim) | k (kv_dim) | v (kv_dim)] of the current token, un-rotated; kc / vc = this
// layer's cache [max_seq][kv_dim] (row `pos` is written). part: nsplit * num_heads * (head_dim + 4) floats,
// tickets: num_kv_heads zero-initialised counters (left at zero). rope_tab: the table launch_embed_q8_0 wrote
// for this position.
cudaError_t launch_attention(const float* qkv, float* kc, float* vc, const int* pos, AttnShape s, const float* rope_tab, int neox,
                             uint32_t nsplit, float* part, unsigned int* tickets, float* attn_out, const AttnPeers& peers,
                             const AttnQ8Out& q8out, cudaStream_t st, bool pdl);
// token <- index held in the largest of keys[0 .. nkeys) (packed maxima written by the output-head kernels,
// one per tensor-parallel rank) when write_token; pos <- pos + 1; keys <- 0
cudaError_t launch_finish_step(unsigned long long* keys, uint32_t nkeys, int* token, int* pos, int* trace, int write_token,
                               const StepPeers& peers, cudaStream_t st, bool pdl);
}  // namespace alice
