// Launchers of the per-token glue kernels (csrc/glue.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace alice {

struct AttnShape { uint32_t num_heads, num_kv_heads, head_dim; };

// hidden <- dequantized row *token of the Q8_0 table; rope_tab (128 floats) <- (sin, cos) of *pos * theta^(-2j/128)
cudaError_t launch_embed_q8_0(const uint8_t* table, const int* token, uint32_t cols, uint32_t vocab, float* hidden,
                              const int* pos, float theta, float* rope_tab, cudaStream_t st, bool pdl);
// qkv = [q (num_heads*head_dim) | k (kv_dim) | v (kv_dim)] of the current token, un-rotated; kc / vc = this
// layer's cache [max_seq][kv_dim] (row `pos` is written). part: nsplit * num_heads * (head_dim + 4) floats,
// tickets: num_kv_heads zero-initialised counters (left at zero). rope_tab: the table launch_embed_q8_0 wrote
// for this position.
cudaError_t launch_attention(const float* qkv, float* kc, float* vc, const int* pos, AttnShape s, const float* rope_tab, int neox,
                             uint32_t nsplit, float* part, unsigned int* tickets, float* attn_out, cudaStream_t st, bool pdl);
// token <- index held in the largest of keys[0 .. nkeys) (packed maxima written by the output-head kernels,
// one per tensor-parallel rank) when write_token; pos <- pos + 1; keys <- 0
cudaError_t launch_finish_step(unsigned long long* keys, uint32_t nkeys, int* token, int* pos, int* trace, int write_token,
                               cudaStream_t st, bool pdl);
}  // namespace alice
