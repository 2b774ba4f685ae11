// Bit-exact device dequantizers: one thread per output element, explicit _rn multiplies and
// subtracts so nothing is contracted into an FMA (the reference's f32 math is mul, mul, sub).
// Q4_K src/gguf.rs:903-939, Q5_K :949-988, Q6_K :1205-1246, Q8_0 :990-1004, Q1_0 :1264-1281,
// Q2_0 :1283-1300 of ALICE-LLM; ternary planes decode to scale * {-1, 0, +1}.
#include <algorithm>

#include "../../include/alice_cuda.h"
#include "common.cuh"
#include "gemv_launch.cuh"

namespace alice {
namespace {

__device__ __forceinline__ float rd_f16(const uint8_t* p) { return f16_bits_to_f32((uint32_t)p[0] | ((uint32_t)p[1] << 8)); }

__device__ __forceinline__ void k4_scale_min(const uint8_t* s, int j, uint32_t& sc, uint32_t& m) {
    if (j < 4) {
        sc = s[j] & 63; m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

__device__ float deq_elem(WeightFormat fmt, const uint8_t* row, uint32_t c, uint32_t row_bytes, const float* scales,
                          uint32_t r) {
    switch (fmt) {
        case WF_Q4_K: {
            const uint8_t* b = row + (c >> 8) * 144;
            const uint32_t e = c & 255, is = e >> 5, l = e & 31;
            uint32_t sc, m;
            k4_scale_min(b + 4, is, sc, m);
            const uint8_t qb = b[16 + (is >> 1) * 32 + l];
            const uint32_t q = (is & 1) ? (qb >> 4) : (qb & 0xF);
            return __fsub_rn(__fmul_rn(__fmul_rn(rd_f16(b), (float)sc), (float)q), __fmul_rn(rd_f16(b + 2), (float)m));
        }
        case WF_Q5_K: {
            const uint8_t* b = row + (c >> 8) * 176;
            const uint32_t e = c & 255, is = e >> 5, l = e & 31;
            uint32_t sc, m;
            k4_scale_min(b + 4, is, sc, m);
            const uint8_t qb = b[48 + (is >> 1) * 32 + l];
            const uint32_t hbit = (b[16 + l] >> is) & 1;
            const uint32_t q = ((is & 1) ? (qb >> 4) : (qb & 0xF)) | (hbit << 4);
            return __fsub_rn(__fmul_rn(__fmul_rn(rd_f16(b), (float)sc), (float)q), __fmul_rn(rd_f16(b + 2), (float)m));
        }
        case WF_Q6_K: {
            const uint8_t* b = row + (c >> 8) * 210;
            const uint32_t e = c & 255, n = e >> 7, j = (e >> 5) & 3, l = e & 31;
            const uint8_t qlb = b[64 * n + (j & 1) * 32 + l];
            const uint32_t lo = (j & 2) ? (qlb >> 4) : (qlb & 0xF);
            const uint32_t hi = (b[128 + 32 * n + l] >> (2 * j)) & 3;
            const int q = (int)(lo | (hi << 4)) - 32;
            const int sc = (int)(int8_t)b[192 + 8 * n + 2 * j + (l >> 4)];
            return __fmul_rn(__fmul_rn(rd_f16(b + 208), (float)sc), (float)q);
        }
        case WF_Q8_0: {
            const uint8_t* b = row + (c >> 5) * 34;
            return __fmul_rn(rd_f16(b), (float)(int8_t)b[2 + (c & 31)]);
        }
        case WF_Q1_0: {
            const uint8_t* b = row + (c >> 7) * 18;
            const uint32_t e = c & 127;
            const float d = rd_f16(b);
            return ((b[2 + (e >> 3)] >> (e & 7)) & 1) ? d : -d;
        }
        case WF_Q2_0: {
            const uint8_t* b = row + (c >> 7) * 34;
            const uint32_t e = c & 127;
            const int slot = (b[2 + (e >> 2)] >> ((e & 3) * 2)) & 3;
            return __fmul_rn((float)(slot - 1), rd_f16(b));
        }
        case WF_TERNARY: {
            const uint32_t pb = row_bytes >> 1;
            const int p = (row[c >> 3] >> (c & 7)) & 1, n = (row[pb + (c >> 3)] >> (c & 7)) & 1;
            return __fmul_rn(scales[r], (float)(p - n));
        }
        case WF_SPARSE_TERNARY: {
            const uint32_t code = (row[c >> 2] >> ((c & 3) * 2)) & 3;
            return __fmul_rn(scales[r], code == 1 ? 1.0f : (code == 3 ? -1.0f : 0.0f));
        }
        default: return 0.0f;
    }
}

__global__ void dequant_kernel(WeightDesc w, float* __restrict__ out) {
    const size_t total = (size_t)w.rows * w.cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / w.cols), c = (uint32_t)(i % w.cols);
        out[i] = deq_elem(w.fmt, w.data + (size_t)r * w.row_bytes, c, w.row_bytes, w.scales, r);
    }
}

__global__ void q8k_to_f32_kernel(Q8KView q, size_t total, float* __restrict__ out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __fmul_rn(q.d[i >> 8], (float)q.qs[i]);
}

}  // namespace

int launch_dequantize(const WeightDesc& w, float* out, cudaStream_t stream) {
    const size_t total = (size_t)w.rows * w.cols;
    if (total == 0) return ALICE_OK;
    const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 148 * 32);
    dequant_kernel<<<blocks, 256, 0, stream>>>(w, out);
    return cudaGetLastError() == cudaSuccess ? ALICE_OK : ALICE_E_CUDA;
}

void launch_q8k_to_f32(const Q8KView& q8, size_t total, float* out, cudaStream_t stream) {
    if (total == 0) return;
    const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 148 * 8);
    q8k_to_f32_kernel<<<blocks, 256, 0, stream>>>(q8, total, out);
}

}  // namespace alice
