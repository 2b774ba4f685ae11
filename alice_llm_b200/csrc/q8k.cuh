// Device-side layout of Q8_K-quantized activations (BlockQ8K, ALICE-LLM src/gguf.rs:1306-1310)
// stored as structure-of-arrays so every field can be fetched with aligned vector loads:
//   qs    int8  [batch][nb][256]
//   d     f32   [batch][nb]
//   bsums int16 [batch][nb][16]
// nb = cols / 256. The three arrays live in one allocation, each section 16-byte aligned.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace alice {

struct Q8KView {
    const int8_t* qs;
    const float* d;
    const int16_t* bsums;
    uint32_t nb;  // blocks per vector
};

struct Q8KLayout {
    size_t qs_off, d_off, bsums_off, total;
    static Q8KLayout make(uint32_t nb, uint32_t batch) {
        Q8KLayout l;
        auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
        l.qs_off = 0;
        l.d_off = up((size_t)batch * nb * 256);
        l.bsums_off = l.d_off + up((size_t)batch * nb * 4);
        l.total = l.bsums_off + up((size_t)batch * nb * 32);
        return l;
    }
};

#ifdef __CUDACC__
// One warp quantizes one 256-element block (8 consecutive elements per lane), bit-exactly as
// quantize_row_q8_k (ALICE-LLM src/gguf.rs:1323-1374):
//   * the element of largest |x| wins, the FIRST one on ties, and its SIGNED value is used;
//   * iscale = 128 / max_val, q = clamp(nearest_int(iscale * x), -128, 127), d = 1 / iscale;
//   * nearest_int is the 12582912.0f magic add (round half to even);
//   * bsums[j] = sum of 16 consecutive q; an all-zero block gives d = 0, q = 0.
// qs / bsums / d may point to global or shared memory.
struct Q8KLaneInput { float4 a, b; };  // the 8 consecutive elements one lane owns
// `cg`: read through L2 only (ld.global.cg) - for a global vector that other SMs rewrite while this
// kernel runs; must be false for a shared-memory source.
__device__ __forceinline__ Q8KLaneInput q8k_load_lane(const float* xb, uint32_t lane, bool cg = false) {
    const float4* src = reinterpret_cast<const float4*>(xb + lane * 8);
    if (cg) return Q8KLaneInput{__ldcg(src), __ldcg(src + 1)};
    return Q8KLaneInput{src[0], src[1]};
}
// ROUNDTRIP: instead of storing the block, write d * q back as f32 to `rt` (256 floats) - the vector as a
// kernel sees it after quantized_matvec_preq turned the Q8_K blocks back into f32 (src/gguf.rs:4593-4605).
// store == false: everything is computed and nothing is written (used to pull the routine's instructions into the
// SM's instruction cache ahead of time).
template <bool ROUNDTRIP = false>
__device__ __forceinline__ void q8k_quantize_block_warp(const Q8KLaneInput in, uint32_t lane, int8_t* qs, float* d,
                                                        int16_t* bsums, float* rt = nullptr, bool store = true) {
    const float4 a = in.a, b = in.b;
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    // local first-maximum, then a warp max over (|x| bits, reversed index) keys
    float lmax = 0.0f, lval = 0.0f;
    uint32_t lidx = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float av = fabsf(v[i]);
        if (av > lmax) { lmax = av; lval = v[i]; lidx = i; }
    }
    unsigned long long best = ((unsigned long long)__float_as_uint(lmax) << 32) | (0xFFFFFFFFu - (lane * 8 + lidx));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    const float amax = __uint_as_float((uint32_t)(best >> 32));
    const uint32_t win_lane = (0xFFFFFFFFu - (uint32_t)best) >> 3;
    const float max_val = __shfl_sync(0xffffffffu, lval, win_lane);
    uint32_t w0 = 0, w1 = 0;
    int lsum = 0;
    float dval = 0.0f;
    int q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (amax != 0.0f) {
        const float iscale = __fdiv_rn(128.0f, max_val);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float t = __fadd_rn(__fmul_rn(iscale, v[i]), 12582912.0f);
            const int n = (int)(__float_as_uint(t) & 0x007fffffu) - 0x00400000;
            q[i] = max(-128, min(127, n));
            lsum += q[i];
        }
        w0 = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
        w1 = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
        dval = __fdiv_rn(1.0f, iscale);
    }
    if (ROUNDTRIP) {
        if (!store) return;
        float4* out = reinterpret_cast<float4*>(rt + lane * 8);
        out[0] = make_float4(__fmul_rn(dval, (float)q[0]), __fmul_rn(dval, (float)q[1]), __fmul_rn(dval, (float)q[2]), __fmul_rn(dval, (float)q[3]));
        out[1] = make_float4(__fmul_rn(dval, (float)q[4]), __fmul_rn(dval, (float)q[5]), __fmul_rn(dval, (float)q[6]), __fmul_rn(dval, (float)q[7]));
        return;
    }
    const int pair = lsum + __shfl_xor_sync(0xffffffffu, lsum, 1);
    if (!store) return;
    reinterpret_cast<uint2*>(qs)[lane] = make_uint2(w0, w1);
    if ((lane & 1) == 0) bsums[lane >> 1] = (int16_t)pair;
    if (lane == 0) *d = dval;
}
#endif

// Quantizes `batch` vectors of `cols` floats (x[k*cols + c]) into the layout above.
// Bit-exact with quantize_row_q8_k (src/gguf.rs:1323-1374).
void launch_quantize_q8k(const float* x, uint32_t cols, uint32_t batch, void* q8k_base, cudaStream_t stream, bool pdl = false, uint32_t layout_batch = 0);

}  // namespace alice
