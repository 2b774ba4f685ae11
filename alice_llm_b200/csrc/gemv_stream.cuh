// Streaming fused dequantize + matvec for GGUF block formats on sm_100a.
//
// Two CTAs per SM stream the raw weight rows they own, in order, through a ring of shared-memory stages filled by
// untiled TMA bulk copies (cp.async.bulk + mbarrier complete_tx), so the number of bytes in flight does not depend on
// registers. A stage holds up to slots*rps whole consecutive rows (and, for the fused SwiGLU variant, the same rows of
// the second matrix); the rows are dealt to the CTAs in equal shares (to within one row per warp set), each CTA cuts
// its share into stages of nearly equal size (RowWalk). Eight consumer warps decode from shared memory: P = 8/slots warps share a row, each warp set walks
// rps rows per stage, and every lane owns the same KL "unit" positions (column ranges) of every row it ever sees, so
// the activations of those columns are loaded ONCE into registers and no activation traffic touches shared memory
// inside the loop. A ninth warp is the copy producer.
//
// The input arrives already in the form the loop reads (Q8_K blocks for the K-quant formats, f32 otherwise): it was
// prepared once by a small stand-alone kernel launched between producer and consumer (csrc/q8k.cu, csrc/publish.cuh);
// where no such kernel covers the case the CTAs prepare the raw vector themselves (pro_mode).
//
// Row result = fixed-order sum of the P warp partials (deterministic run to run).
#pragma once
#include "common.cuh"
#include "publish.cuh"
#include "q8k.cuh"

namespace alice {

constexpr int NCW = 8;                          // consumer warps per CTA
constexpr int STREAM_THREADS = (NCW + 1) * 32;  // + one producer warp
constexpr int MAX_STAGES = 4;
constexpr int MAX_RPS = 16;                     // rows per warp set per stage (must stay <= 32)

struct StreamArgs {
    const uint8_t* w0;   // weight rows (gate matrix for SwiGLU)
    const uint8_t* w1;   // up matrix for SwiGLU, else null
    Q8KView q8;          // K-quants: the input as Q8_K blocks (global memory); vector k at qs + k*cols, d + k*nb, bsums + k*nb*16
    const float* x;      // f32-activation formats: the input vector(s), x[k*cols + c]
    const float* aux0;   // per-row scales (ternary formats) for w0
    const float* aux1;   // per-row scales for w1
    float* y;            // y[k*y_stride + row]
    int* status;         // device status word (0 = ok)
    uint32_t rows, cols;
    uint32_t row_bytes;  // bytes of one weight row
    uint32_t units;      // units per row (format specific)
    uint32_t P;          // consumer warps per row: 1, 2, 4 or 8
    uint32_t slots;      // warp sets per CTA = NCW / P
    uint32_t rps;        // rows each warp set handles per stage, at most (<= MAX_RPS)
    uint32_t groups;     // number of stage-sized row groups over all CTAs
    uint32_t nstages;
    uint32_t cap;        // bytes reserved per matrix per stage (multiple of 128)
    uint32_t batch;      // input vectors sharing one pass over the weights (batch kernels), else 1
    uint32_t y_stride;   // floats between the outputs of consecutive input vectors
    uint32_t tab_off;    // shared-memory offset of the activation area (Q8_K blocks / f32 vector / bit-plane digit table)
    const uint8_t* tab_global;  // bit-plane kernels: the digit table prepared in global memory (mma_table_kernel), or null
    // pro_mode != 0: x is the raw f32 vector and every CTA prepares its own copy in the activation area
    // (stream_prologue): rms_norm with the weights pro_norm_w into the f32 area at offset 0, then Q8_K blocks at
    // pro_q8_off (K-quant formats); f32-activation formats read the normalised vector (pro_roundtrip: rounded to the
    // Q8_K grid).
    uint32_t pro_mode, pro_roundtrip;
    uint32_t pro_q8_off;
    const float* pro_norm_w;
    float pro_eps;
    // Optional residual epilogue: y[row] = resid[row] + result (resid may alias y)
    const float* resid;
    // Optional greedy-argmax epilogue: atomicMax of (order-preserving bits of y[i]) << 32 | ~i, so the
    // largest value wins and, among equal values, the lowest index. The caller clears it to 0.
    unsigned long long* argmax_key;
    // Up to three matrices of the same format and width share one launch (q, k, v): segment s owns
    // row groups [seg_g0[s], seg_g0[s+1]) and writes y + seg_y[s]. nseg == 1 for a single matrix.
    uint32_t nseg;
    const uint8_t* seg_w[3];
    uint32_t seg_rows[3];
    uint32_t seg_g0[4];
    uint32_t seg_t0[4];  // per-lane kernel: prefix sums of ceil(seg_rows / slots), the "set rows" RowWalk deals out
    uint32_t seg_y[3];
    const float* seg_aux[3];   // per-row scales of each segment's matrix (formats that have them), else null
    // Row-wise staging (tensor-core kernels): instead of one contiguous copy per stage every row is
    // copied on its own, as npieces pieces of piece_len bytes taken at piece_off[p] inside the global row of
    // src_row_bytes bytes, to shared memory rows row_stride bytes apart. That allows a padded (bank-conflict
    // free) row stride and a matvec over a column sub-range of the matrix (row_bytes = npieces * piece_len
    // then describes the sub-row). row_mode == 0: rows are row_bytes apart in both memories (contiguous copy).
    uint32_t row_mode;
    uint32_t row_stride;
    uint32_t src_row_bytes;
    uint32_t npieces;
    uint32_t piece_off[2];
    uint32_t piece_len;
    uint32_t row_pad;    // bytes in front of the first wanted byte of a staged row (piece start rounded down to 16)
    uint32_t x_stride;   // elements between consecutive input vectors (the matrix's full column count)
    // Tensor parallel: every row result is also stored at the same index of the vector of each of npeers other GPUs
    // (peer-mapped memory); the hand-over that tells the peers is a kernel of its own behind this one (csrc/publish.cuh).
    uint32_t npeers;
    float* peer_y[MAX_PEERS];
    long long wait_limit;      // SM cycles a wait inside the kernel may take; 0 = WAIT_CYCLE_LIMIT
};

// Shared-memory header in front of the ring.
struct StreamSmem {
    unsigned long long full[MAX_STAGES];
    unsigned long long empty[MAX_STAGES];
    unsigned long long red[MAX_STAGES][NCW];  // per (stage, slot): partials of the P-1 helper warps posted
    unsigned long long act_bar;               // batch kernels: the activation blocks have landed in shared memory
    float partial[MAX_STAGES][NCW][MAX_RPS][2];  // [stage][warp][row in set][gate|up]
    double norm_part[NCW];
    int abort_flag;
};

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                              int code, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);   // keep the first report
            return false;
        }
    }
    return true;
}

// Sums NV per-lane values across the warp with one butterfly: each halving step trades half of
// the values with the partner lane, so NV-1 shuffles replace 5*NV. On return the lanes
// [i*32/NV, (i+1)*32/NV) all hold the warp total of value i.
template <int NV>
__device__ __forceinline__ float reduce_values(float (&v)[NV], uint32_t lane) {
    static_assert(NV == 1 || NV == 2 || NV == 4 || NV == 8, "NV must be a power of two <= 8");
    int off = 16;
#pragma unroll
    for (int n = NV; n > 1; n >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; i++) {
            const float keep = upper ? v[i + n / 2] : v[i];
            const float send = upper ? v[i] : v[i + n / 2];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
        off >>= 1;
    }
    float r = v[0];
    for (; off > 0; off >>= 1) r += __shfl_xor_sync(0xffffffffu, r, off);
    return r;
}

// Per-CTA streaming state.
struct StreamCtx {
    StreamSmem* sm;
    uint8_t* smem_raw;
    uint32_t ring;          // shared address of stage 0
    uint32_t stage_stride;  // bytes between stages
    uint32_t nstages;
    uint32_t cc;            // chunks streamed so far (producer and consumers keep separate copies in step)
    long long limit;        // cycle budget of one wait
};

// The per-(stage, warp set) barriers collect the P-1 helper warps of a row set. Each barrier expects
// RED_COUNT = lcm(1, 3, 7) arrivals and every helper arrives with weight RED_COUNT / (P - 1). A barrier
// that a stage does not use (no such row set, or no rows left for it) is completed by its own warp, so
// every barrier finishes exactly one phase per stage use and shares the phase of the `full` barrier.
constexpr uint32_t RED_COUNT = 21;
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t n) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(n) : "memory");
}

// Called by every thread of the CTA (one barrier per thread: a single thread initialising all of them costs ~0.6 us
// on the critical path of a small matvec); the caller follows with __syncthreads().
__device__ __forceinline__ void stream_init_ring(StreamSmem* sm, uint32_t nstages) {
    const uint32_t t = threadIdx.x;
    if (t < nstages) mbar_init(smem_u32(&sm->full[t]), 1);
    else if (t < 2 * nstages) mbar_init(smem_u32(&sm->empty[t - nstages]), NCW);
    else if (t < (2 + NCW) * nstages) mbar_init(smem_u32(&sm->red[(t - 2 * nstages) / NCW][(t - 2 * nstages) % NCW]), RED_COUNT);
    else if (t == (2 + NCW) * nstages) {
        mbar_init(smem_u32(&sm->act_bar), 1);
        sm->abort_flag = 0;
    }
    if (t <= (2 + NCW) * nstages) mbar_fence_init();
}

// The row groups (stages) of one CTA of the per-lane kernel, in order; producer and consumers walk them in step.
// A "set row" is `slots` consecutive rows (one per warp set when a stage holds one row per set); segment s owns set
// rows [seg_t0[s], seg_t0[s+1]). CTA c owns the set rows [total*c/grid, total*(c+1)/grid) - shares differ by at most
// one - and cuts the part inside each segment into ceil(T / rps) groups of floor or ceil(T / groups) set rows, so its
// stages are of nearly equal size and no CTA streams a whole stage more than another (with fixed-size groups dealt
// out whole, 1195 groups on 296 CTAs give some CTAs five and most four; measured on the 8B FFN block: 32.2 us per
// block with the even shares, 32.9 us without).
struct RowWalk {
    uint32_t t, t_end, sg, left, base, extra;
    __device__ __forceinline__ void init(const StreamArgs& a) {
        const uint32_t total = a.seg_t0[a.nseg];
        t = (uint32_t)(((uint64_t)total * blockIdx.x) / gridDim.x);
        t_end = (uint32_t)(((uint64_t)total * (blockIdx.x + 1)) / gridDim.x);
        sg = 0; left = 0; base = 0; extra = 0;

    }
    // Next group: segment, first row inside it, rows per warp set. false when the CTA's share is done.
    __device__ __forceinline__ bool next(const StreamArgs& a, uint32_t& seg, uint32_t& r0, uint32_t& rps_g) {
        if (left == 0) {
            if (t >= t_end) return false;
            while (sg + 1 < a.nseg && t >= a.seg_t0[sg + 1]) sg++;
            const uint32_t T = min(t_end, a.seg_t0[sg + 1]) - t;
            const uint32_t G = (T + a.rps - 1) / a.rps;
            base = T / G; extra = T % G; left = G;
        }
        rps_g = base + (extra > 0 ? 1u : 0u);
        if (extra > 0) extra--;
        left--;
        seg = sg; r0 = (t - a.seg_t0[sg]) * a.slots;
        t += rps_g;
        return true;
    }
};

// Producer side of one matvec: streams this CTA's row groups of `a` through the ring. One thread.
__device__ __forceinline__ void stream_produce(const StreamArgs& a, StreamCtx& cx) {
    StreamSmem* sm = cx.sm;
    volatile int* abort_flag = &sm->abort_flag;
    const uint32_t rows_per_group = a.slots * a.rps;
    const bool two = a.w1 != nullptr;
    const uint32_t g0 = (uint32_t)(((uint64_t)a.groups * blockIdx.x) / gridDim.x);
    const uint32_t g1 = (uint32_t)(((uint64_t)a.groups * (blockIdx.x + 1)) / gridDim.x);
    for (uint32_t g = g0; g < g1; g++) {
        const uint32_t s = cx.cc % cx.nstages, use = cx.cc / cx.nstages;
        if (use > 0 && !wait_or_abort(smem_u32(&sm->empty[s]), (use - 1) & 1, abort_flag, a.status, KERR_WAIT_EMPTY, 2 * cx.limit)) return;
        uint32_t sg = 0;
        while (sg + 1 < a.nseg && g >= a.seg_g0[sg + 1]) sg++;
        const uint32_t r0 = (g - a.seg_g0[sg]) * rows_per_group;
        const uint32_t nrow = min(rows_per_group, a.seg_rows[sg] - r0);
        const uint64_t off = (uint64_t)r0 * a.row_bytes;
        const uint64_t a0 = off & ~uint64_t(15);
        const uint32_t cb = (uint32_t)((off - a0) + (uint64_t)nrow * a.row_bytes + 15) & ~15u;
        const uint32_t fb = smem_u32(&sm->full[s]);
        mbar_arrive_expect_tx(fb, two ? 2 * cb : cb);
        bulk_g2s(cx.ring + s * cx.stage_stride, a.seg_w[sg] + a0, cb, fb);
        if (two) bulk_g2s(cx.ring + s * cx.stage_stride + a.cap, a.w1 + a0, cb, fb);
        cx.cc++;
    }
}

// Producer side of the per-lane kernel: the CTA's share of the rows, group by group (RowWalk). One thread.
__device__ __forceinline__ void stream_produce_walk(const StreamArgs& a, StreamCtx& cx) {
    StreamSmem* sm = cx.sm;
    volatile int* abort_flag = &sm->abort_flag;
    const bool two = a.w1 != nullptr;
    RowWalk walk;
    walk.init(a);
    uint32_t sg, r0, rps_g;
    while (walk.next(a, sg, r0, rps_g)) {
        const uint32_t s = cx.cc % cx.nstages, use = cx.cc / cx.nstages;
        if (use > 0 && !wait_or_abort(smem_u32(&sm->empty[s]), (use - 1) & 1, abort_flag, a.status, KERR_WAIT_EMPTY, 2 * cx.limit)) return;
        const uint32_t nrow = min(a.slots * rps_g, a.seg_rows[sg] - r0);
        const uint64_t off = (uint64_t)r0 * a.row_bytes;
        const uint64_t a0 = off & ~uint64_t(15);
        const uint32_t cb = (uint32_t)((off - a0) + (uint64_t)nrow * a.row_bytes + 15) & ~15u;
        const uint32_t fb = smem_u32(&sm->full[s]);
        mbar_arrive_expect_tx(fb, two ? 2 * cb : cb);
        bulk_g2s(cx.ring + s * cx.stage_stride, a.seg_w[sg] + a0, cb, fb);
        if (two) bulk_g2s(cx.ring + s * cx.stage_stride + a.cap, a.w1 + a0, cb, fb);
        cx.cc++;
    }
}

// Producer side in row mode: the whole producer warp takes part, lane l copies rows l, l + 32, ... of the stage.
__device__ __forceinline__ void stream_produce_rows(const StreamArgs& a, StreamCtx& cx) {
    StreamSmem* sm = cx.sm;
    volatile int* abort_flag = &sm->abort_flag;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t rows_per_group = a.slots * a.rps;
    const bool two = a.w1 != nullptr;
    const uint32_t g0 = (uint32_t)(((uint64_t)a.groups * blockIdx.x) / gridDim.x);
    const uint32_t g1 = (uint32_t)(((uint64_t)a.groups * (blockIdx.x + 1)) / gridDim.x);
    for (uint32_t g = g0; g < g1; g++) {
        const uint32_t s = cx.cc % cx.nstages, use = cx.cc / cx.nstages;
        int ok = 1;
        if (lane == 0 && use > 0)
            ok = wait_or_abort(smem_u32(&sm->empty[s]), (use - 1) & 1, abort_flag, a.status, KERR_WAIT_EMPTY, 2 * cx.limit) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return;
        uint32_t sg = 0;
        while (sg + 1 < a.nseg && g >= a.seg_g0[sg + 1]) sg++;
        const uint32_t r0 = (g - a.seg_g0[sg]) * rows_per_group;
        const uint32_t nrow = min(rows_per_group, a.seg_rows[sg] - r0);
        const uint32_t fb = smem_u32(&sm->full[s]);
        if (lane == 0) mbar_arrive_expect_tx(fb, nrow * a.npieces * a.piece_len * (two ? 2u : 1u));
        __syncwarp();   // the byte count is posted before any copy can complete
        const uint32_t stage = cx.ring + s * cx.stage_stride;
        for (uint32_t r = lane; r < nrow; r += 32) {
            const uint64_t src = (uint64_t)(r0 + r) * a.src_row_bytes;
            const uint32_t dst = stage + r * a.row_stride;
            for (uint32_t p = 0; p < a.npieces; p++) {
                bulk_g2s(dst + p * a.piece_len, a.seg_w[sg] + src + a.piece_off[p], a.piece_len, fb);
                if (two) bulk_g2s(dst + a.cap + p * a.piece_len, a.w1 + src + a.piece_off[p], a.piece_len, fb);
            }
        }
        cx.cc++;
    }
}

// After an abort: let copies already issued land before the CTA gives its shared memory back.
__device__ __forceinline__ void stream_drain(StreamCtx& cx) {
    const uint32_t first = cx.cc > cx.nstages ? cx.cc - cx.nstages : 0;
    for (uint32_t c = first; c < cx.cc; c++) mbar_wait(smem_u32(&cx.sm->full[c % cx.nstages]), (c / cx.nstages) & 1);
}

// Row epilogue shared by every consumer: residual, store (here and on the peers), packed argmax key of the row.
template <bool PEER>
__device__ __forceinline__ unsigned long long stream_store_row(const StreamArgs& a, float r, float res, bool has_res, uint32_t yi) {
    if (has_res) r = __fadd_rn(res, r);
    a.y[yi] = r;
    if (PEER) for (uint32_t p = 0; p < a.npeers; p++) a.peer_y[p][yi] = r;
    const uint32_t b = __float_as_uint(r);
    const uint32_t ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return r == r ? ((unsigned long long)ordered << 32) | (0xFFFFFFFFu - yi) : 0ull;
}
__device__ __forceinline__ void stream_argmax(unsigned long long* argmax_key, unsigned long long key, uint32_t lane) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = other > key ? other : key;
    }
    if (lane == 0) atomicMax(argmax_key, key);
}

// Per-CTA input preparation (pro_mode), run by the NCW consumer warps on the raw f32 vector in global memory.
//   norm_w != null: rms_norm (src/llama3.rs:5244-5256) - f64 sum of squares, mean and scale in f32, then
//                   (x * scale) * w - into the f32 area xn (shared memory);
//   q8 != null:     the (normalised) vector -> Q8_K in shared memory at q8 (qs | bsums | d), one warp per
//                   256-element block, exactly the stand-alone quantizer (cols % 256 == 0);
//   roundtrip:      (with norm_w) the normalised vector is replaced by d * q of its Q8_K quantization, which is what
//                   quantized_matvec_preq hands a Q1_0 / Q2_0 matvec (src/gguf.rs:4593-4605).
// Loads travel in rounds (several per thread in flight), so a pass over x costs a few memory round trips.
// Redundant across CTAs, but parallel: a single CTA doing it once for everybody costs a serial chain of ~10 us
// (ticket, loads, reduction, quantization, each a dependent round trip) at the end of the producing kernel.
static __device__ __forceinline__ void stream_prologue(StreamSmem* sm, const float* x, const float* norm_w, float norm_eps, uint32_t cols,
                                                       float* xn, uint8_t* q8, bool roundtrip) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const float* src = x;
    bool src_global = true;
    if (norm_w != nullptr) {
        // a thread's share of x stays in registers between the two passes when it fits in NORM_V float4
        // (cols <= NCW*32*4*NORM_V); the norm weights ride the same memory round trip as x
        constexpr int NORM_V = 4;
        const uint32_t nvec = cols / 4;
        const float4* xg = reinterpret_cast<const float4*>(x);
        const float4* wg = reinterpret_cast<const float4*>(norm_w);
        const bool one_round = nvec <= NCW * 32 * NORM_V;
        float4 xv[NORM_V], wv[NORM_V];
        double ss = 0.0;
#pragma unroll 1
        for (uint32_t base = 0; base < nvec; base += NCW * 32 * NORM_V) {
#pragma unroll
            for (int k = 0; k < NORM_V; k++) {
                const uint32_t i = base + k * NCW * 32 + tid;
                xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < nvec) xv[k] = xg[i];
            }
            if (one_round) {
#pragma unroll
                for (int k = 0; k < NORM_V; k++) {
                    const uint32_t i = k * NCW * 32 + tid;
                    if (i < nvec) wv[k] = __ldg(wg + i);
                }
            }
#pragma unroll
            for (int k = 0; k < NORM_V; k++)
                ss += (double)xv[k].x * (double)xv[k].x + (double)xv[k].y * (double)xv[k].y +
                      (double)xv[k].z * (double)xv[k].z + (double)xv[k].w * (double)xv[k].w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) sm->norm_part[warp] = ss;
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        double tot = 0.0;
#pragma unroll
        for (int w = 0; w < NCW; w++) tot += sm->norm_part[w];
        const float mean = (float)(tot / (double)cols);
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, norm_eps)));
#pragma unroll 1
        for (uint32_t base = 0; base < nvec; base += NCW * 32 * NORM_V) {
#pragma unroll
            for (int k = 0; k < NORM_V; k++) {
                const uint32_t i = base + k * NCW * 32 + tid;
                if (i < nvec) {
                    const float4 v = one_round ? xv[k] : xg[i];
                    const float4 w = one_round ? wv[k] : __ldg(wg + i);
                    reinterpret_cast<float4*>(xn)[i] = make_float4(__fmul_rn(__fmul_rn(v.x, scale), w.x), __fmul_rn(__fmul_rn(v.y, scale), w.y),
                                                                   __fmul_rn(__fmul_rn(v.z, scale), w.z), __fmul_rn(__fmul_rn(v.w, scale), w.w));
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");  // xn complete
        src = xn;
        src_global = false;
        if (roundtrip) {   // xn <- d * q of its own Q8_K quantization, block by block, in place
#pragma unroll 1
            for (uint32_t b = warp; b < cols / QK_K; b += NCW) {
                const Q8KLaneInput in = q8k_load_lane(xn + (size_t)b * QK_K, lane, false);
                q8k_quantize_block_warp<true>(in, lane, nullptr, nullptr, nullptr, xn + (size_t)b * QK_K);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        }
    }
    if (q8 != nullptr) {
        const uint32_t nb = cols / QK_K;
        int8_t* qs_s = reinterpret_cast<int8_t*>(q8);
        int16_t* bs_s = reinterpret_cast<int16_t*>(q8 + (size_t)nb * 256);  // 8-byte aligned for any nb
        float* d_s = reinterpret_cast<float*>(q8 + (size_t)nb * 288);
        // QB blocks per warp per round: their loads travel together (one memory round trip per round when
        // the source is global memory) and their reduction chains interleave
        constexpr int QB = 4;
#pragma unroll 1
        for (uint32_t b0 = warp; b0 < nb; b0 += QB * NCW) {
            Q8KLaneInput in[QB];
#pragma unroll
            for (int i = 0; i < QB; i++) {
                const uint32_t blk = b0 + i * NCW;
                if (blk < nb) in[i] = q8k_load_lane(src + (size_t)blk * QK_K, lane, false);
            }
#pragma unroll
            for (int i = 0; i < QB; i++) {
                const uint32_t blk = b0 + i * NCW;
                if (blk < nb) q8k_quantize_block_warp(in[i], lane, qs_s + (size_t)blk * QK_K, d_s + blk, bs_s + (size_t)blk * 16);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
    }
    (void)src_global;
}

// F supplies:
//   struct Act;                                            per-position activation registers
//   static void load_act(Act&, const StreamArgs&, const Q8KView&, const float* x, bool x_global, uint32_t u, bool valid)
//   static float unit(uint32_t row_smem_addr, uint32_t u, const Act&, const StreamArgs&)   partial dot of unit u
//   static float finish(float v, const StreamArgs&, const float* aux, uint32_t row)   per-row epilogue
// Consumer side of one matvec (the NCW consumer warps of the CTA, threads 0 .. NCW*32-1). Returns false after an abort.
// PLAIN: the matvec is known to use none of the fused extras (residual / argmax epilogue, q/k/v segments, hand-over to
// the next op, peers), so their code is compiled out - the stand-alone matvec entry points run this leaner instance.
template <class F, int KL, bool SWIGLU, bool PEER, bool PLAIN>
__device__ __forceinline__ bool stream_consume(const StreamArgs& a, StreamCtx& cx) {
    StreamSmem* sm = cx.sm;
    volatile int* abort_flag = &sm->abort_flag;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t P = a.P, slots = a.slots;
    const uint32_t slot = warp / P, part = warp % P;
    const float* const resid = PLAIN ? nullptr : a.resid;
    unsigned long long* const argmax_key = PLAIN ? nullptr : a.argmax_key;

    // the input: already prepared in global memory (every lane takes its own columns straight into registers; the
    // loads are L1-cached, so the warp sets of a CTA share one trip to L2), or the raw f32 vector, prepared per CTA
    Q8KView q8 = a.q8;
    const float* xin = a.x;
    if (a.pro_mode) {
        uint8_t* area = cx.smem_raw + a.tab_off;
        float* xn = reinterpret_cast<float*>(area);
        uint8_t* q8a = F::USES_Q8K ? area + a.pro_q8_off : nullptr;
        stream_prologue(sm, a.x, a.pro_norm_w, a.pro_eps, a.cols, xn, q8a, a.pro_roundtrip != 0);
        if (F::USES_Q8K) {
            const uint32_t nb = a.cols / QK_K;
            q8.qs = reinterpret_cast<const int8_t*>(q8a);
            q8.bsums = reinterpret_cast<const int16_t*>(q8a + (size_t)nb * 256);
            q8.d = reinterpret_cast<const float*>(q8a + (size_t)nb * 288);
            q8.nb = nb;
        } else {
            xin = xn;
        }
    }
    typename F::Act act[KL];
#pragma unroll
    for (int k = 0; k < KL; k++) {
        const uint32_t u = ((uint32_t)k * P + part) * 32 + lane;
        F::load_act(act[k], a, q8, xin, false, u, u < a.units);
    }

    // Rows are walked RB at a time so that RB*M independent unit decodes are in flight per lane
    // and one butterfly reduces all of them (NV-1 + log2(32/NV) shuffles instead of 5*NV).
    constexpr int M = SWIGLU ? 2 : 1;
    constexpr int RB = KL == 1 ? (SWIGLU ? 2 : 4) : (KL == 2 ? (SWIGLU ? 1 : 2) : 1);
    constexpr int NV = RB * M;
    constexpr uint32_t LANES_PER_VALUE = 32 / NV;

    RowWalk walk;
    walk.init(a);
    uint32_t sg, r0, rps;
    while (walk.next(a, sg, r0, rps)) {
        const uint32_t s = cx.cc % cx.nstages, ph = (cx.cc / cx.nstages) & 1;
        cx.cc++;
        const uint32_t seg_rows = a.seg_rows[sg];
        const uint32_t pad = (uint32_t)(((uint64_t)r0 * a.row_bytes) & 15);
        const uint32_t set0 = slot * rps;                 // first row (within the stage) of this warp set
        const uint32_t nrow = r0 + set0 < seg_rows ? min(rps, seg_rows - r0 - set0) : 0;
        // the residual this lane will add in the epilogue: requested now, needed after the rows are done
        float res = 0.0f;
        if (resid != nullptr && part == 0 && lane < nrow) res = __ldcg(resid + a.seg_y[sg] + r0 + set0 + lane);
        if (!wait_or_abort(smem_u32(&sm->full[s]), ph, abort_flag, a.status, KERR_WAIT_FULL, cx.limit)) return false;
        const uint32_t sb = cx.ring + s * cx.stage_stride + pad + set0 * a.row_bytes;
        for (uint32_t rr0 = 0; rr0 < nrow; rr0 += RB) {
            float v[NV];
#pragma unroll
            for (int i = 0; i < NV; i++) v[i] = 0.0f;
#pragma unroll
            for (int j = 0; j < RB; j++) {
                if (rr0 + j < nrow) {
                    const uint32_t rb = sb + (rr0 + j) * a.row_bytes;
#pragma unroll
                    for (int k = 0; k < KL; k++) {
                        const uint32_t u = ((uint32_t)k * P + part) * 32 + lane;
                        if (u < a.units) {
                            v[j * M] += F::unit(rb, u, act[k], a);
                            if (SWIGLU) v[j * M + M - 1] += F::unit(rb + a.cap, u, act[k], a);
                        }
                    }
                }
            }
            const float tot = reduce_values<NV>(v, lane);
            const uint32_t vi = lane / LANES_PER_VALUE;   // which of the NV values this lane now holds
            if ((lane % LANES_PER_VALUE) == 0 && rr0 + vi / M < nrow) sm->partial[s][warp][rr0 + vi / M][vi % M] = tot;
        }
        __syncwarp();
        {   // barrier red[s][warp] completes one phase per stage use even when no row set needs it
            const uint32_t own0 = warp * rps;
            const bool used = P > 1 && warp < slots && r0 + own0 < seg_rows;
            if (!used && lane == 0) mbar_arrive_n(smem_u32(&sm->red[s][warp]), RED_COUNT);
        }
        if (nrow > 0) {
            if (part != 0) {
                if (lane == 0) mbar_arrive_n(smem_u32(&sm->red[s][slot]), RED_COUNT / (P - 1));
            } else {
                if (P > 1 && !wait_or_abort(smem_u32(&sm->red[s][slot]), ph, abort_flag, a.status, KERR_WAIT_PARTIALS, cx.limit)) return false;
                unsigned long long key = 0ull;
                float v0 = 0.0f, v1 = 0.0f;
                if (lane < nrow) {
                    for (uint32_t p = 0; p < P; p++) {
                        v0 += sm->partial[s][warp + p][lane][0];
                        if (SWIGLU) v1 += sm->partial[s][warp + p][lane][1];
                    }
                }
                // everything this warp needed from the stage has been read: the producer may refill it while the
                // epilogue runs
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
                if (lane < nrow) {
                    const uint32_t row = r0 + set0 + lane;      // row inside its matrix
                    float r = F::finish(v0, a, a.seg_aux[sg], row);
                    if (SWIGLU) r = silu_ref(r) * F::finish(v1, a, a.aux1, row);
                    key = stream_store_row<PEER>(a, r, res, resid != nullptr, a.seg_y[sg] + row);
                }
                if (argmax_key != nullptr) stream_argmax(argmax_key, key, lane);
                continue;   // this warp has already released the stage
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
    }
    return true;
}

// One matvec per launch.
template <class F, int KL, bool SWIGLU, bool PEER, bool PLAIN>
__global__ void __launch_bounds__(STREAM_THREADS, KL <= 2 ? 2 : 1) stream_gemv_kernel(const __grid_constant__ StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    StreamSmem* sm = reinterpret_cast<StreamSmem*>(smem_raw);
    constexpr uint32_t HDR = (sizeof(StreamSmem) + 127) & ~127u;
    StreamCtx cx;
    cx.sm = sm; cx.smem_raw = smem_raw; cx.ring = smem_u32(smem_raw) + HDR;
    cx.stage_stride = a.cap * (SWIGLU ? 2u : 1u); cx.nstages = a.nstages; cx.cc = 0;
    cx.limit = a.wait_limit > 0 ? a.wait_limit : WAIT_CYCLE_LIMIT;
    stream_init_ring(sm, a.nstages);
    __syncthreads();
    pdl_launch_dependents();
    if ((threadIdx.x >> 5) == NCW) {
        // producer: weights do not depend on the previous kernel, so copies start at once
        if ((threadIdx.x & 31) == 0) {
            stream_produce_walk(a, cx);
            if (sm->abort_flag) stream_drain(cx);
        }
        return;
    }
    pdl_wait();  // activations come from the previous kernel
    stream_consume<F, KL, SWIGLU, PEER, PLAIN>(a, cx);
}

}  // namespace alice
