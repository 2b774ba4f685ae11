// Launchers of the per-token glue kernels (csrc/glue.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace alice {

struct AttnShape { uint32_t num_heads, num_kv_heads, head_dim; };

cudaError_t launch_embed_q8_0(const uint8_t* table, const int* token, uint32_t cols, uint32_t vocab, float* hidden,
                              cudaStream_t st, bool pdl);
// qkv = [q (num_heads*head_dim) | k (kv_dim) | v (kv_dim)]; kc / vc = this layer's cache [max_seq][kv_dim]
cudaError_t launch_rope_kv(float* qkv, const int* pos, AttnShape s, float theta, int neox, float* kc, float* vc,
                           cudaStream_t st, bool pdl);
// part: nsplit * num_heads * (head_dim + 2) floats of scratch
cudaError_t launch_attention(const float* qkv, const float* kc, const float* vc, const int* pos, AttnShape s,
                             uint32_t nsplit, float* part, float* attn_out, cudaStream_t st, bool pdl);
// token <- argmax(logits) when write_token (also recorded at trace[pos]); pos <- pos + 1
cudaError_t launch_argmax_advance(const float* logits, uint32_t n, int* token, int* pos, int* trace, int write_token,
                                  cudaStream_t st, bool pdl);

}  // namespace alice
