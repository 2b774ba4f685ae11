// Whole-decode-step kernel (csrc/step_kernel.cu): op list and launcher.
#pragma once
#include "gemv_plan.cuh"
#include "glue.cuh"

namespace alice {

enum StepOpType : uint32_t { SOP_EMBED = 0, SOP_GEMV = 1, SOP_ATTN = 2 };
// (format, activation positions per lane, fused SwiGLU) instances compiled into the step kernel
enum StepVariant : int { SV_Q4K_1 = 0, SV_Q4K_1_SW, SV_Q4K_2, SV_Q6K_1, SV_Q6K_2, SV_Q8_0_1, SV_Q8_0_2 };

struct alignas(16) StepOp {
    uint32_t type;
    int variant;            // SOP_GEMV
    StreamArgs g;           // SOP_GEMV (planned against the step kernel's ring)
    // SOP_ATTN
    const float* qkv; float* kc; float* vc; float* part; unsigned int* tickets; float* attn_out;
    AttnShape shape; int neox; uint32_t nsplit;
    float* rope_tab;        // SOP_EMBED writes it, SOP_ATTN reads it
    float theta;            // SOP_EMBED
    // SOP_EMBED
    const uint8_t* table; float* hidden; uint32_t cols, vocab;
};

struct StepArgs {
    const StepOp* ops;      // device array
    uint32_t nops, nsteps;
    int* pos; int* token; int* trace;
    unsigned long long* key;
    unsigned int* barrier;  // zero at launch
    int* status;
    int write_token;
    uint32_t nstages, stage_stride, aux_off;
    uint32_t ops_off;       // shared-memory offset of the consumers' two-entry StepOp buffer
    long long* prof;        // optional: 16 clock64 stamps per op, written by thread 0 of the middle CTA during the last step
};

constexpr uint32_t STEP_SMEM_BUDGET = 112 * 1024;   // two CTAs per SM

// -1 when the combination is not compiled into the step kernel (the caller then uses one launch per op).
int step_variant(WeightFormat f, uint32_t kl, bool swiglu);
cudaError_t launch_decode_steps(const StepArgs& sa, uint32_t grid, size_t smem, cudaStream_t st);
cudaError_t decode_step_max_ctas_per_sm(size_t smem, int* out);

}  // namespace alice
