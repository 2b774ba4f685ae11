// Host-side description and launch of the streaming matvec.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "publish.cuh"
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

// One streaming matvec with its optional fused stages. The input is either already prepared (Q8_K blocks for the
// K-quant formats, the final f32 vector for the others; see csrc/publish.cuh) or the raw f32 vector, which every CTA
// then prepares for itself in shared memory (rms_norm, Q8_K quantization).
struct GemvOp {
    const WeightDesc* w[3] = {nullptr, nullptr, nullptr};  // 1..3 matrices of one format and width sharing the input
    uint32_t nw = 1;
    uint32_t y_off[3] = {0, 0, 0};                         // output offset (floats) of each matrix inside y
    const WeightDesc* up = nullptr;                        // fused SwiGLU: w[0] = gate, up = up (nw must be 1)
    const Q8KView* q8 = nullptr;                           // K-quants: input vector 0 as Q8_K; vector k follows at qs + k*cols, d + k*nb, bsums + k*nb*16
    const float* x = nullptr;                              // f32 input, x[k*cols + c]; K-quants without q8 quantize it per CTA
    const float* norm_w = nullptr;                         // rms_norm of x with these weights first, in every CTA (per-lane kernels only)
    float norm_eps = 0.0f;
    bool q8k_roundtrip = false;                            // with norm_w, f32-activation formats: round the vector to the Q8_K grid
    uint32_t batch = 1;                                    // input vectors
    uint32_t y_stride = 0;                                 // floats between the outputs of consecutive vectors (0: the rows of this op)
    const float* resid = nullptr;                          // y = resid + result (same layout as y)
    unsigned long long* argmax_key = nullptr;              // atomicMax of packed (value, ~index), see StreamArgs (batch 1 only)
    float* y = nullptr;
    uint32_t npeers = 0;                                   // tensor parallel: also store every row result on these GPUs
    float* peer_y[MAX_PEERS] = {};
    long long wait_limit = 0;                              // SM cycles a wait inside the kernel may take (0 = about a second)
    // Bit-plane tensor-core kernels: device scratch for the activation digit table, prepared once by a small kernel
    // ahead of the matvec; without it (or when it is too small) every CTA of the matvec builds the table itself.
    void* prep = nullptr;
    size_t prep_bytes = 0;
};
// Scratch bytes GemvOp::prep needs for a bit-plane matvec over `cols` columns (any such format, any column split).
size_t mma_prep_bytes(uint32_t cols);
int launch_stream_gemv_op(const GemvOp& op, const LaunchCfg& cfg);
// How a batch of op.batch vectors would run: kernel launches, and how many times the weight bytes stream from HBM.
int batch_plan(const GemvOp& op, const LaunchCfg& cfg, uint32_t* launches, uint32_t* weight_passes);


// out[r*cols + c] = dequantized weight, bit-exact with the reference dequantizers.
int launch_dequantize(const WeightDesc& w, float* out, cudaStream_t stream);

// The stand-alone form of csrc/publish.cuh: one CTA prepares `p.batch` vectors (optional rms_norm, then Q8_K and / or
// f32) - used where no producing kernel can do it (the embedding, NCCL-gathered vectors).
cudaError_t launch_publish_vector(const Publish& p, int* status, cudaStream_t stream, bool pdl);

// out[i] = d[i/256] * q[i] for i < total (the Q8_K -> f32 step of quantized_matvec_preq for
// Q1_0/Q2_0, src/gguf.rs:4593-4605); total = batch * cols.
void launch_q8k_to_f32(const Q8KView& q8, size_t total, float* out, cudaStream_t stream);

}  // namespace alice
