// Host-side description and launch of the streaming matvec.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "q8k.cuh"

namespace alice {

// Storage formats of a device-resident weight matrix.
enum WeightFormat : uint32_t {
    WF_Q8_0 = 8, WF_Q4_K = 12, WF_Q5_K = 13, WF_Q6_K = 14, WF_Q1_0 = 41, WF_Q2_0 = 42,  // GGML ids (src/gguf.rs:101-122)
    WF_TERNARY = 1000,         // interleaved bit planes, see FmtTernary
    WF_SPARSE_TERNARY = 1001,  // packed 2-bit codes, see FmtSparseTernary
};

struct WeightDesc {
    WeightFormat fmt;
    const uint8_t* data;   // device, 16-byte aligned
    const float* scales;   // device per-row scales (ternary formats) or null
    uint32_t rows, cols;
    uint32_t row_bytes;
};

bool format_uses_q8k(WeightFormat f);
// Bytes of one device row for a GGML block format; 0 if cols is not a whole number of blocks.
uint32_t ggml_row_bytes(WeightFormat f, uint32_t cols);
uint32_t ggml_block_bytes(WeightFormat f);
uint32_t ggml_block_elems(WeightFormat f);

struct LaunchCfg {
    cudaStream_t stream;
    int num_sms;
    int* status;      // device status word
    bool pdl;         // launch with programmatic stream serialization
    int force_rps;    // 0 = automatic
    int force_stages; // 0 = automatic
};

// One launch of the streaming matvec with its optional fused stages.
// Where a matvec's rows also go on the other GPUs of a tensor-parallel group (see StreamArgs::peer_y).
struct PeerPush {
    uint32_t npeers = 0;
    float* y[7] = {};             // the same vector as GemvOp::y in each peer's memory
    unsigned int* flag[7] = {};   // arrival counter of this matvec on each peer
    uint2* y_ll[7] = {};          // tagged form (GemvOp::y_ll) of the vector in each peer's memory
};

struct GemvOp {
    const WeightDesc* w[3] = {nullptr, nullptr, nullptr};  // 1..3 matrices of one format and width sharing the input
    uint32_t nw = 1;
    uint32_t y_off[3] = {0, 0, 0};                         // output offset (floats) of each matrix inside y
    const WeightDesc* up = nullptr;                        // fused SwiGLU: w[0] = gate, up = up (nw must be 1)
    const Q8KView* q8 = nullptr;                           // pre-quantized input (K-quants), else x
    const float* x = nullptr;                              // f32 input vector
    const float* norm_w = nullptr;                         // fused RMSNorm of x with these weights
    float norm_eps = 0.0f;
    bool q8k_roundtrip = false;                            // with norm_w, f32-activation formats: see StreamArgs
    const float* resid = nullptr;                          // y = resid + result
    unsigned long long* argmax_key = nullptr;              // atomicMax of packed (value, ~index), see StreamArgs
    float* y = nullptr;
    const PeerPush* push = nullptr;                        // tensor parallel: also store every row result on the peers
    const unsigned int* wait_flag = nullptr;               // tensor parallel: x is complete when *wait_flag >= (*epoch + 1) * wait_mult
    uint32_t wait_mult = 0;
    const unsigned int* epoch = nullptr;
    // tagged vectors (StreamArgs::x_ll ...): input, output (with push->y_ll on the peers) and residual
    const uint2* x_ll = nullptr;
    uint32_t x_seq = 0, x_n = 0;
    uint2* y_ll = nullptr;
    uint32_t y_seq = 0, y_n = 0;
    const uint2* resid_ll = nullptr;
};
int launch_stream_gemv_op(const GemvOp& op, const LaunchCfg& cfg);
// CTAs of the launch that stores the final rows of `op` (what a tensor-parallel peer counts as arrivals).
int stream_gemv_final_grid(const GemvOp& op, const LaunchCfg& cfg, uint32_t* grid);

// y[r] = W[r,:] . x  (or silu(W0 x) * (W1 x) when w1 != null). K-quant formats read `q8`,
// the others read the f32 vector `x`. Returns 0 or a negative ALICE_E_* code.
int launch_stream_gemv(const WeightDesc& w0, const WeightDesc* w1, const Q8KView* q8, const float* x, float* y,
                       const LaunchCfg& cfg);

// out[r*cols + c] = dequantized weight, bit-exact with the reference dequantizers.
int launch_dequantize(const WeightDesc& w, float* out, cudaStream_t stream);

// out[i] = d[i/256] * q[i] for i < total (the Q8_K -> f32 step of quantized_matvec_preq for
// Q1_0/Q2_0, src/gguf.rs:4593-4605); total = batch * cols.
void launch_q8k_to_f32(const Q8KView& q8, size_t total, float* out, cudaStream_t stream);

}  // namespace alice
