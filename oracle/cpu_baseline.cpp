// Timed CPU baseline: the oracle's restatement of the reference CPU path, compiled
// -O3 -march=native (the reference builds with -C target-cpu=native, .cargo/config.toml) and
// run row-parallel on a persistent pool of worker threads, standing in for rayon's par_iter_mut over output rows
// (ALICE-LLM src/gguf.rs:3661-3675). TEST / BENCHMARK INFRASTRUCTURE ONLY: it is what the GPU
// numbers are placed next to, never something the product calls.
//
// The per-block kernels are the same functions as in alice_oracle.cpp (included below), i.e. the
// scalar bodies the reference's own "avx512" Q4_K kernel consists of (src/gguf.rs:2681-2695);
// the compiler vectorizes them for the host.
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>

#include "alice_oracle.cpp"

namespace {

// A persistent pool (rayon keeps its workers alive between par_iter calls too): the workers sleep on a condition
// variable, a call hands every worker one contiguous row range and waits for all of them.
class Pool {
public:
    explicit Pool(int n) : n_(n) {
        for (int t = 0; t < n; t++) th_.emplace_back([this, t] { work(t); });
    }
    ~Pool() {
        { std::lock_guard<std::mutex> lk(mu_); stop_ = true; gen_++; }
        cv_.notify_all();
        for (auto& t : th_) t.join();
    }
    int size() const { return n_; }
    void run(size_t rows, const std::function<void(size_t, size_t)>& fn) {
        std::unique_lock<std::mutex> lk(mu_);
        fn_ = &fn; rows_ = rows; pending_ = n_; gen_++;
        cv_.notify_all();
        done_.wait(lk, [this] { return pending_ == 0; });
    }
private:
    void work(int t) {
        unsigned seen = 0;
        for (;;) {
            const std::function<void(size_t, size_t)>* fn;
            size_t rows;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return gen_ != seen; });
                seen = gen_;
                if (stop_) return;
                fn = fn_; rows = rows_;
            }
            const size_t r0 = rows * t / n_, r1 = rows * (t + 1) / n_;
            if (r1 > r0) (*fn)(r0, r1);
            { std::lock_guard<std::mutex> lk(mu_); if (--pending_ == 0) done_.notify_one(); }
        }
    }
    int n_;
    std::vector<std::thread> th_;
    std::mutex mu_;
    std::condition_variable cv_, done_;
    const std::function<void(size_t, size_t)>* fn_ = nullptr;
    size_t rows_ = 0;
    int pending_ = 0;
    unsigned gen_ = 0;
    bool stop_ = false;
};

Pool* pool_for(int nthreads) {
    static std::mutex mu;
    static Pool* pool = nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!pool || pool->size() != nthreads) { delete pool; pool = new Pool(nthreads); }
    return pool;
}

template <class Fn>
void par_rows(size_t rows, int nthreads, Fn fn) {
    if (nthreads <= 1) { fn(0, rows); return; }
    std::function<void(size_t, size_t)> f = fn;
    pool_for(nthreads)->run(rows, f);
}

}  // namespace

extern "C" {

// quantized_matvec with `parallel` feature: y = W x over nthreads row ranges.
int base_matvec(uint32_t type, const float* x, const uint8_t* data, size_t nbytes, size_t rows, size_t cols,
                float* y, int nthreads) {
    const size_t row_bytes = nbytes / rows;
    if (type == T_Q4_K || type == T_Q5_K || type == T_Q6_K) {
        size_t nb = cols / QK_K;
        std::vector<float> d8(nb); std::vector<int8_t> q8(nb * QK_K); std::vector<int16_t> bs(nb * 16);
        quantize_row_q8_k(x, nb * QK_K, d8.data(), q8.data(), bs.data());
        par_rows(rows, nthreads, [&](size_t r0, size_t r1) {
            orc_matvec_preq(type, data + r0 * row_bytes, (r1 - r0) * row_bytes, r1 - r0, cols, d8.data(), q8.data(),
                            bs.data(), y + r0);
        });
        return 0;
    }
    par_rows(rows, nthreads, [&](size_t r0, size_t r1) {
        orc_matvec(type, x, data + r0 * row_bytes, (r1 - r0) * row_bytes, r1 - r0, cols, y + r0);
    });
    return 0;
}

// The SwiGLU FFN block of the CPU model (src/llama3.rs:14519-14540): gate/up from one Q8_K input,
// silu(gate)*up, then down.
int base_ffn(uint32_t gu_type, const uint8_t* gate, const uint8_t* up, size_t gu_bytes, uint32_t down_type,
             const uint8_t* down, size_t down_bytes, size_t hidden, size_t ffn, const float* x, float* y,
             int nthreads) {
    std::vector<float> g(ffn), u(ffn);
    base_matvec(gu_type, x, gate, gu_bytes, ffn, hidden, g.data(), nthreads);
    base_matvec(gu_type, x, up, gu_bytes, ffn, hidden, u.data(), nthreads);
    for (size_t i = 0; i < ffn; i++) g[i] = silu(g[i]) * u[i];
    return base_matvec(down_type, g.data(), down, down_bytes, hidden, ffn, y, nthreads);
}

void base_ternary_matvec(const uint8_t* pos, const uint8_t* neg, const float* scales, size_t rows, size_t cols,
                         const float* x, float* y, int nthreads) {
    size_t pb = (cols + 7) / 8;
    par_rows(rows, nthreads, [&](size_t r0, size_t r1) {
        orc_ternary_matvec(pos + r0 * pb, neg + r0 * pb, scales + r0, r1 - r0, cols, x, y + r0);
    });
}

// Llama3Model::forward with the `parallel` feature: the oracle's forward with row-parallel matvecs.
int base_llama_forward(const OrcModel* m, uint32_t token, uint32_t pos, float* logits, int nthreads) {
    return llama_forward(
        *m, token, pos, logits,
        [nthreads](uint32_t t, const float* x, const uint8_t* d, size_t nb, size_t r, size_t c, float* y) {
            return base_matvec(t, x, d, nb, r, c, y, nthreads);
        },
        [nthreads](uint32_t t, const uint8_t* d, size_t nb, size_t r, size_t c, const float* d8, const int8_t* q8,
                   const int16_t* bs, float* y) {
            const size_t row_bytes = nb / r;
            int rc = 0;
            par_rows(r, nthreads, [&](size_t r0, size_t r1) {
                if (orc_matvec_preq(t, d + r0 * row_bytes, (r1 - r0) * row_bytes, r1 - r0, c, d8, q8, bs, y + r0)) rc = -1;
            });
            return rc;
        });
}

int base_hw_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
