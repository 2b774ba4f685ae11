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

// Quantizes `batch` vectors of `cols` floats (x[k*cols + c]) into the layout above.
// Bit-exact with quantize_row_q8_k (src/gguf.rs:1323-1374).
void launch_quantize_q8k(const float* x, uint32_t cols, uint32_t batch, void* q8k_base, cudaStream_t stream);

}  // namespace alice
