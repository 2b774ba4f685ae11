// Stand-alone Q8_K activation quantizer (quantize_row_q8_k, ALICE-LLM src/gguf.rs:1323-1374):
// one warp per 256-element block; the per-block routine lives in q8k.cuh and is shared with the
// kernels that leave their output prepared for the next op (csrc/publish.cuh).
#include "common.cuh"
#include "q8k.cuh"

namespace alice {

__global__ void __launch_bounds__(128) quantize_q8k_kernel(const float* __restrict__ x, uint32_t nblocks,
                                                           int8_t* __restrict__ qs, float* __restrict__ d,
                                                           int16_t* __restrict__ bsums) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t blk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= nblocks) return;

    q8k_quantize_block_warp(q8k_load_lane(x + (size_t)blk * QK_K, lane, true), lane, qs + (size_t)blk * QK_K, d + blk, bsums + (size_t)blk * 16);
}

void launch_quantize_q8k(const float* x, uint32_t cols, uint32_t batch, void* base, cudaStream_t stream, bool pdl, uint32_t layout_batch) {
    const uint32_t nb = cols / QK_K;
    const Q8KLayout l = Q8KLayout::make(nb, layout_batch ? layout_batch : batch);
    const uint32_t nblocks = nb * batch;
    if (nblocks == 0) return;
    auto* p = static_cast<uint8_t*>(base);
    const uint32_t warps = 4;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((nblocks + warps - 1) / warps);
    lc.blockDim = dim3(warps * 32);
    lc.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = pdl ? 1 : 0;
    cudaLaunchKernelEx(&lc, quantize_q8k_kernel, x, nblocks, reinterpret_cast<int8_t*>(p + l.qs_off), reinterpret_cast<float*>(p + l.d_off),
                       reinterpret_cast<int16_t*>(p + l.bsums_off));
}

}  // namespace alice
