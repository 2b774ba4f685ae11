// Planning of one streaming matvec separately from its launch, so that a kernel that runs many
// matvecs back to back (csrc/step_kernel.cu) can lay them out over one shared ring.
#pragma once
#include "gemv_launch.cuh"
#include "gemv_stream.cuh"

namespace alice {

struct PlanLimits {
    uint32_t nstages;       // ring depth fixed by the enclosing kernel
    uint32_t stage_stride;  // bytes a stage may use
    uint32_t ctas;          // CTAs that will share the rows
};

struct StreamPlan {
    StreamArgs args;
    uint32_t kl;        // activation positions per lane: 1, 2 or 4
    bool swiglu;
    uint32_t grid;      // CTAs for a stand-alone launch
    size_t smem;        // dynamic shared memory for a stand-alone launch
    uint32_t stage;     // bytes one stage really uses
    uint32_t q8_bytes, xn_bytes;
    bool mma = false;         // bit-plane tensor-core kernel (csrc/gemv_mma.cuh) instead of the per-lane one
    uint32_t ctas_per_sm = 2; // resident CTAs per SM the launch was planned for (mma kernels)
    uint32_t ksplit = 1;      // column chunks, one launch each, accumulating into y (mma kernels with rows too wide for shared memory)
};

// lim == nullptr: plan a stand-alone launch (ring sized from the CTA's own budget).
int plan_stream_gemv(const GemvOp& op, const LaunchCfg& cfg, const PlanLimits* lim, StreamPlan& pl);

constexpr uint32_t STREAM_HDR_BYTES = (sizeof(StreamSmem) + 127) & ~127u;

}  // namespace alice
