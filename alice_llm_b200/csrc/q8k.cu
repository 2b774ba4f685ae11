// Q8_K activation quantizer: one warp per 256-element block, 8 consecutive elements per lane.
// Follows quantize_row_q8_k (ALICE-LLM src/gguf.rs:1323-1374) bit for bit:
//   * the element of largest |x| wins, the FIRST one on ties, and its SIGNED value is used;
//   * iscale = 128 / max_val, q = clamp(nearest_int(iscale * x), -128, 127), d = 1 / iscale;
//   * nearest_int is the 12582912.0f magic-add (round half to even);
//   * bsums[j] = sum of 16 consecutive q; an all-zero block gives d = 0, q = 0.
#include "common.cuh"
#include "q8k.cuh"

namespace alice {

__global__ void __launch_bounds__(128) quantize_q8k_kernel(const float* __restrict__ x, uint32_t nblocks,
                                                           int8_t* __restrict__ qs, float* __restrict__ d,
                                                           int16_t* __restrict__ bsums) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t blk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= nblocks) return;

    const float4* src = reinterpret_cast<const float4*>(x + (size_t)blk * QK_K + lane * 8);
    float4 a = src[0], b = src[1];
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};

    // Local first-maximum, then a warp max over (|x| bits, reversed index) keys: the largest
    // magnitude wins and, among equal magnitudes, the lowest element index.
    float lmax = 0.0f, lval = 0.0f;
    uint32_t lidx = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float av = fabsf(v[i]);
        if (av > lmax) { lmax = av; lval = v[i]; lidx = i; }
    }
    unsigned long long key = ((unsigned long long)__float_as_uint(lmax) << 32) | (0xFFFFFFFFu - (lane * 8 + lidx));
    unsigned long long best = key;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    const float amax = __uint_as_float((uint32_t)(best >> 32));
    const uint32_t win_lane = (0xFFFFFFFFu - (uint32_t)best) >> 3;
    const float max_val = __shfl_sync(0xffffffffu, lval, win_lane);

    uint32_t w0 = 0, w1 = 0;
    int lsum = 0;
    float dval = 0.0f;
    if (amax != 0.0f) {
        const float iscale = __fdiv_rn(128.0f, max_val);
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float t = __fadd_rn(__fmul_rn(iscale, v[i]), 12582912.0f);
            int n = (int)(__float_as_uint(t) & 0x007fffffu) - 0x00400000;
            q[i] = max(-128, min(127, n));
            lsum += q[i];
        }
        w0 = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
        w1 = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
        dval = __fdiv_rn(1.0f, iscale);
    }
    reinterpret_cast<uint2*>(qs + (size_t)blk * QK_K)[lane] = make_uint2(w0, w1);
    int pair = lsum + __shfl_xor_sync(0xffffffffu, lsum, 1);
    if ((lane & 1) == 0) bsums[(size_t)blk * 16 + (lane >> 1)] = (int16_t)pair;
    if (lane == 0) d[blk] = dval;
}

void launch_quantize_q8k(const float* x, uint32_t cols, uint32_t batch, void* base, cudaStream_t stream) {
    const uint32_t nb = cols / QK_K;
    const Q8KLayout l = Q8KLayout::make(nb, batch);
    const uint32_t nblocks = nb * batch;
    if (nblocks == 0) return;
    auto* p = static_cast<uint8_t*>(base);
    const uint32_t warps = 4;
    quantize_q8k_kernel<<<(nblocks + warps - 1) / warps, warps * 32, 0, stream>>>(
        x, nblocks, reinterpret_cast<int8_t*>(p + l.qs_off), reinterpret_cast<float*>(p + l.d_off),
        reinterpret_cast<int16_t*>(p + l.bsums_off));
}

}  // namespace alice
