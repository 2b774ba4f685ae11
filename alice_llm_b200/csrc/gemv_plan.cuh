// Planning of one streaming matvec separately from its launch (the launch geometry is also what
// alice_plan_query reports).
#pragma once
#include "gemv_launch.cuh"
#include "gemv_stream.cuh"

namespace alice {

struct StreamPlan {
    StreamArgs args;
    uint32_t kl;        // activation positions per lane: 1, 2 or 4
    bool swiglu;
    uint32_t grid;      // CTAs for a stand-alone launch
    size_t smem;        // dynamic shared memory for a stand-alone launch
    uint32_t stage;     // bytes one stage really uses
    bool mma = false;         // bit-plane tensor-core kernel (csrc/gemv_mma.cuh) instead of the per-lane one
    uint32_t ctas_per_sm = 2; // resident CTAs per SM the launch was planned for (mma kernels)
    uint32_t ksplit = 1;      // column chunks, one launch each, accumulating into y (mma kernels with rows too wide for shared memory)
};

int plan_stream_gemv(const GemvOp& op, const LaunchCfg& cfg, StreamPlan& pl);

constexpr uint32_t STREAM_HDR_BYTES = (sizeof(StreamSmem) + 127) & ~127u;

}  // namespace alice
