// Device-side ternarization of f32 weight rows and sparsification of ternary rows, bit-exact with
// TernaryRow::from_f32 (ALICE-LLM src/gguf.rs:5207-5245) and SparseTernaryRow::from_ternary_row (src/gguf.rs:5451-5507).
//
// Both reference routines accumulate in index order (an f32 running sum of |w| over the row; an f64 running sum over
// the kept weights in block order and, inside a block, in sorted order), so the bits of the scale depend on that order.
// One thread therefore owns one row and walks it front to back; a warp owns 32 consecutive rows and stages 32 x 32
// tiles of them through shared memory, so that global loads are whole 128-byte lines although every thread reads its
// own row. This is a load-time conversion (once per matrix), not a decode-path kernel.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/alice_cuda.h"
#include "abi_internal.cuh"

namespace alice {
namespace {

constexpr int TILE = 32;

// tile[j][l] = w[(r0 + j) * cols + c0 + l], zero outside the matrix; one warp
__device__ __forceinline__ void load_tile(float (*tile)[TILE + 1], const float* w, uint32_t rows, uint32_t cols, uint32_t r0,
                                          uint32_t c0, uint32_t lane) {
#pragma unroll 4
    for (int j = 0; j < TILE; j++) {
        const uint32_t r = r0 + j, c = c0 + lane;
        tile[j][lane] = (r < rows && c < cols) ? w[(size_t)r * cols + c] : 0.0f;
    }
    __syncwarp();
}

// Device row layout of a ternary matrix: [pos plane | neg plane], planes of pb = ceil(cols / 32) * 4 bytes.
__global__ void __launch_bounds__(128) ternarize_kernel(const float* __restrict__ w, uint32_t rows, uint32_t cols, float ratio,
                                                        uint8_t* __restrict__ out, uint32_t pb, float* __restrict__ scales) {
    __shared__ float tiles[4][TILE][TILE + 1];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float (*tile)[TILE + 1] = tiles[warp];
    const uint32_t r0 = (blockIdx.x * 4 + warp) * TILE, row = r0 + lane;
    if (r0 >= rows) return;
    // pass 1: mean |w| of the row, summed front to back in f32
    float s = 0.0f;
    for (uint32_t c0 = 0; c0 < cols; c0 += TILE) {
        load_tile(tile, w, rows, cols, r0, c0, lane);
        const uint32_t n = min((uint32_t)TILE, cols - c0);
        for (uint32_t i = 0; i < n; i++) s = __fadd_rn(s, fabsf(tile[lane][i]));
        __syncwarp();
    }
    const float threshold = __fmul_rn(ratio, __fdiv_rn(s, (float)cols));
    // pass 2: masks (one 32-bit word of each plane per tile) and the mean magnitude of the kept weights
    float abs_sum = 0.0f;
    uint32_t nz = 0;
    for (uint32_t c0 = 0; c0 < cols; c0 += TILE) {
        load_tile(tile, w, rows, cols, r0, c0, lane);
        const uint32_t n = min((uint32_t)TILE, cols - c0);
        uint32_t pw = 0, nw = 0;
        for (uint32_t i = 0; i < n; i++) {
            const float v = tile[lane][i];
            if (fabsf(v) > threshold) {
                if (v > 0.0f) pw |= 1u << i; else nw |= 1u << i;
                abs_sum = __fadd_rn(abs_sum, fabsf(v));
                nz++;
            }
        }
        if (row < rows) {
            uint8_t* dst = out + (size_t)row * 2 * pb + c0 / 8;
            *reinterpret_cast<uint32_t*>(dst) = pw;
            *reinterpret_cast<uint32_t*>(dst + pb) = nw;
        }
        __syncwarp();
    }
    if (row < rows) scales[row] = nz > 0 ? __fdiv_rn(abs_sum, (float)nz) : 0.0f;
}

// Keeps the n_keep largest |w| among the non-zero weights of every block of 16 (ties: the earlier index, as the
// reference's stable sort does) and packs the result as 2-bit codes, 00 = 0, 01 = +1, 11 = -1 (src/gguf.rs:5432-5450).
__global__ void __launch_bounds__(128) sparsify_kernel(const uint8_t* __restrict__ tern, uint32_t pb, const float* __restrict__ dense_scale,
                                                       const float* __restrict__ w, uint32_t rows, uint32_t cols, uint32_t n_keep,
                                                       uint8_t* __restrict__ out, uint32_t rb, float* __restrict__ scales) {
    __shared__ float tiles[4][TILE][TILE + 1];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float (*tile)[TILE + 1] = tiles[warp];
    const uint32_t r0 = (blockIdx.x * 4 + warp) * TILE, row = r0 + lane;
    if (r0 >= rows) return;
    double abs_sum = 0.0;
    uint32_t nz = 0;
    for (uint32_t c0 = 0; c0 < cols; c0 += TILE) {
        load_tile(tile, w, rows, cols, r0, c0, lane);
        uint32_t pw = 0, nw = 0;
        if (row < rows) {
            const uint8_t* src = tern + (size_t)row * 2 * pb + c0 / 8;
            pw = *reinterpret_cast<const uint32_t*>(src);
            nw = *reinterpret_cast<const uint32_t*>(src + pb);
        }
        for (uint32_t h = 0; h < 2; h++) {                    // the two 16-weight blocks of this tile
            const uint32_t base = c0 + h * 16;
            if (base >= cols) break;
            const uint32_t len = min(16u, cols - base);
            const uint32_t nzmask = ((pw | nw) >> (h * 16)) & 0xffffu;
            const uint32_t keep = min(n_keep, len);
            // selection in sorted order: repeatedly the largest remaining magnitude, the lowest index among equals
            uint32_t left = nzmask, active = 0, sign = 0;
            for (uint32_t k = 0; k < keep && left; k++) {
                float best = -1.0f;
                uint32_t bi = 0;
                for (uint32_t i = 0; i < len; i++) {
                    if (!((left >> i) & 1u)) continue;
                    const float m = fabsf(tile[lane][h * 16 + i]);
                    if (m > best) { best = m; bi = i; }
                }
                left &= ~(1u << bi);
                active |= 1u << bi;
                if ((nw >> (h * 16 + bi)) & 1u) sign |= 1u << bi;
                abs_sum += (double)best;
                nz++;
            }
            if (row < rows) {
                uint32_t packed = 0;
                for (uint32_t i = 0; i < 16; i++) {
                    const uint32_t code = ((active >> i) & 1u) ? (((sign >> i) & 1u) ? 3u : 1u) : 0u;
                    packed |= code << (2 * i);
                }
                *reinterpret_cast<uint32_t*>(out + (size_t)row * rb + (base / 16) * 4) = packed;
            }
        }
        __syncwarp();
    }
    if (row < rows) scales[row] = nz > 0 ? (float)(abs_sum / (double)nz) : dense_scale[row];
}

int new_weights(alice_engine* e, alice::WeightDesc d, size_t data_bytes, void** data, float** scales) {
    cudaError_t err = cudaMalloc(data, data_bytes + 64);
    if (err != cudaSuccess) return alice_cuda_fail(err, "cudaMalloc");
    err = cudaMalloc(reinterpret_cast<void**>(scales), (size_t)d.rows * sizeof(float));
    if (err == cudaSuccess) err = cudaMemsetAsync(*data, 0, data_bytes + 64, e->stream);
    if (err != cudaSuccess) { cudaFree(*data); return alice_cuda_fail(err, "cudaMalloc"); }
    return ALICE_OK;
}

}  // namespace
}  // namespace alice

using namespace alice;

extern "C" {

int32_t alice_ternarize(alice_engine* e, const alice_buf* w, uint32_t rows, uint32_t cols, float threshold_ratio,
                        alice_weights** out) {
    if (!e || !w || !out) return alice_fail(ALICE_E_INVALID, "alice_ternarize: null argument");
    if (rows == 0 || cols == 0) return alice_fail(ALICE_E_SHAPE, "alice_ternarize: empty matrix");
    if (w->len < (size_t)rows * cols) return alice_fail(ALICE_E_SHAPE, "alice_ternarize: buffer holds %zu floats, need %zu", w->len, (size_t)rows * cols);
    cudaError_t err = cudaSetDevice(e->device);
    if (err != cudaSuccess) return alice_cuda_fail(err, "cudaSetDevice");
    const uint32_t pb = ((cols + 31) / 32) * 4;
    WeightDesc d = {};
    d.fmt = WF_TERNARY; d.rows = rows; d.cols = cols; d.row_bytes = 2 * pb;
    void* data = nullptr;
    float* scales = nullptr;
    int rc = new_weights(e, d, (size_t)rows * 2 * pb, &data, &scales);
    if (rc) return rc;
    ternarize_kernel<<<(rows + 127) / 128, 128, 0, e->stream>>>(w->p, rows, cols, threshold_ratio, static_cast<uint8_t*>(data), pb, scales);
    err = cudaGetLastError();
    if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);
    if (err != cudaSuccess) { cudaFree(data); cudaFree(scales); return alice_cuda_fail(err, "alice_ternarize"); }
    d.data = static_cast<const uint8_t*>(data); d.scales = scales;
    *out = new alice_weights{e, d, data, scales};
    alice_engine_retain(e);
    return ALICE_OK;
}

int32_t alice_sparsify(alice_engine* e, const alice_weights* ternary, const alice_buf* w, uint32_t n_keep, alice_weights** out) {
    if (!e || !ternary || !w || !out) return alice_fail(ALICE_E_INVALID, "alice_sparsify: null argument");
    const WeightDesc& t = ternary->d;
    if (t.fmt != WF_TERNARY) return alice_fail(ALICE_E_UNSUPPORTED, "alice_sparsify: the source must be a ternary bit-plane matrix");
    if (w->len < (size_t)t.rows * t.cols) return alice_fail(ALICE_E_SHAPE, "alice_sparsify: buffer holds %zu floats, need %zu", w->len, (size_t)t.rows * t.cols);
    cudaError_t err = cudaSetDevice(e->device);
    if (err != cudaSuccess) return alice_cuda_fail(err, "cudaSetDevice");
    const uint32_t rb = ((t.cols + 15) / 16) * 4;
    WeightDesc d = {};
    d.fmt = WF_SPARSE_TERNARY; d.rows = t.rows; d.cols = t.cols; d.row_bytes = rb;
    void* data = nullptr;
    float* scales = nullptr;
    int rc = new_weights(e, d, (size_t)t.rows * rb, &data, &scales);
    if (rc) return rc;
    sparsify_kernel<<<(t.rows + 127) / 128, 128, 0, e->stream>>>(t.data, t.row_bytes / 2, t.scales, w->p, t.rows, t.cols, n_keep,
                                                                 static_cast<uint8_t*>(data), rb, scales);
    err = cudaGetLastError();
    if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);
    if (err != cudaSuccess) { cudaFree(data); cudaFree(scales); return alice_cuda_fail(err, "alice_sparsify"); }
    d.data = static_cast<const uint8_t*>(data); d.scales = scales;
    *out = new alice_weights{e, d, data, scales};
    alice_engine_retain(e);
    return ALICE_OK;
}

int32_t alice_weights_download(alice_engine* e, const alice_weights* w, uint8_t* rows_out, size_t rows_bytes, float* scales_out) {
    if (!e || !w || !rows_out) return alice_fail(ALICE_E_INVALID, "alice_weights_download: null argument");
    const WeightDesc& d = w->d;
    const size_t need = (size_t)d.rows * d.row_bytes;
    if (rows_bytes < need) return alice_fail(ALICE_E_SHAPE, "alice_weights_download: %zu bytes offered, %zu needed", rows_bytes, need);
    cudaError_t err = cudaSetDevice(e->device);
    if (err == cudaSuccess) err = cudaMemcpyAsync(rows_out, d.data, need, cudaMemcpyDeviceToHost, e->stream);
    if (err == cudaSuccess && scales_out && d.scales) err = cudaMemcpyAsync(scales_out, d.scales, (size_t)d.rows * 4, cudaMemcpyDeviceToHost, e->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);
    if (err != cudaSuccess) return alice_cuda_fail(err, "alice_weights_download");
    return ALICE_OK;
}

}  // extern "C"
