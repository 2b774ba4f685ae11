// Streaming fused dequantize + matvec for GGUF block formats on sm_100a.
//
// One persistent CTA per SM streams the raw weight rows it owns, in order, through a ring of
// shared-memory stages filled by untiled TMA bulk copies (cp.async.bulk + mbarrier complete_tx),
// so the number of bytes in flight does not depend on registers. A stage holds slots*rps whole
// consecutive rows (and, for the fused SwiGLU variant, the same rows of the second matrix).
// Eight consumer warps decode from shared memory: P = 8/slots warps share a row, each warp set
// walks rps rows per stage, and every lane owns the same KL "unit" positions (column ranges) of
// every row it ever sees, so the activations of those columns are loaded ONCE into registers
// and no activation traffic touches shared memory inside the loop. A ninth warp is the copy
// producer.
//
// Row result = fixed-order sum of the P warp partials (deterministic run to run).
#pragma once
#include "common.cuh"
#include "q8k.cuh"

namespace alice {

constexpr int NCW = 8;                        // consumer warps per CTA
constexpr int STREAM_THREADS = (NCW + 1) * 32;  // + one producer warp
constexpr int MAX_STAGES = 4;
constexpr int MAX_RPS = 16;                   // rows per warp set per stage (must stay <= 32)

struct StreamArgs {
    const uint8_t* w0;   // weight rows (gate matrix for SwiGLU)
    const uint8_t* w1;   // up matrix for SwiGLU, else null
    const void* act;     // Q8KView base (K-quants) or const float* x (f32-activation formats)
    Q8KView q8;          // valid for K-quants
    const float* x;      // valid for f32-activation formats
    const float* aux0;   // per-row scales (ternary formats) for w0
    const float* aux1;   // per-row scales for w1
    float* y;            // y[k*rows + r]
    int* status;         // device status word (0 = ok)
    uint32_t rows, cols;
    uint32_t row_bytes;  // bytes of one weight row
    uint32_t units;      // units per row (format specific)
    uint32_t P;          // consumer warps per row: 1, 2, 4 or 8
    uint32_t slots;      // warp sets per CTA = NCW / P
    uint32_t rps;        // rows each warp set handles per stage (<= MAX_RPS)
    uint32_t groups;     // ceil(rows / (slots * rps)) = number of stage-sized row groups
    uint32_t nstages;
    uint32_t cap;        // bytes reserved per matrix per stage (multiple of 128)
    uint32_t q8_off;     // shared-memory offset of the in-kernel Q8_K area (K-quants with f32 input)
    uint32_t xn_off;     // shared-memory offset of the normalised f32 input (RMSNorm prologue)
    // Optional fused RMSNorm of the input (rms_norm, src/llama3.rs:5244): x <- x * rsqrt(mean(x^2) + eps) * norm_w
    const float* norm_w;
    float norm_eps;
    // With norm_w, for f32-activation formats: round the normalised vector to the Q8_K grid (quantize, then
    // d * q), as the CPU model does on projections it reaches through matvec_preq (src/gguf.rs:4593-4605)
    uint32_t q8k_roundtrip;
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
    uint32_t seg_y[3];
    const float* seg_aux[3];   // per-row scales of each segment's matrix (formats that have them), else null
    // Row-wise staging (bit-plane tensor-core kernels): instead of one contiguous copy per stage every row is
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
    // Tensor parallel without a collective library: every row result is also stored at the same index of the
    // vector of each of npeers other GPUs (peer_y, peer-mapped memory), and a CTA that has finished all its rows
    // adds 1 to peer_flag[p] on every peer (release). wait_flag (in this GPU's memory) guards the INPUT vector:
    // the consumers wait until it has reached (*epoch + 1) * wait_mult - the arrivals of all peers' producing
    // CTAs up to and including this decode step - before reading x, and read x past L1.
    uint32_t npeers;
    float* peer_y[7];
    unsigned int* peer_flag[7];
    const unsigned int* wait_flag;
    uint32_t wait_mult;
    const unsigned int* epoch;
    // The per-layer vectors of a tensor-parallel model travel in tagged form instead (8-byte elements (value, tag),
    // see ll_store): x_ll replaces x as the input, y_ll / peer_y_ll[p] receive the rows of this matvec (this GPU's
    // copy and the peers'), resid_ll replaces resid. A vector is rewritten several times per decode step; write
    // number seq of n per step carries tag *epoch * n + seq + 1, so a reader knows exactly which version it wants.
    const uint2* x_ll;
    uint32_t x_seq, x_n;
    uint2* y_ll;
    uint2* peer_y_ll[7];
    uint32_t y_seq, y_n;
    const uint2* resid_ll;
};

// Where the input vector of a matvec comes from: plain f32 (global, optionally past L1) or a tagged vector.
struct XSrc {
    const float* x;
    const uint2* ll;
    uint32_t tag;
    bool cg;
};
__device__ __forceinline__ XSrc xsrc_of(const StreamArgs& a, bool cg) {
    XSrc s;
    s.x = a.x; s.ll = a.x_ll; s.cg = cg;
    s.tag = a.x_ll ? ld_acquire_sys_u32(a.epoch) * a.x_n + a.x_seq + 1u : 0u;
    return s;
}

// Shared-memory header in front of the ring.
struct StreamSmem {
    unsigned long long full[MAX_STAGES];
    unsigned long long empty[MAX_STAGES];
    unsigned long long red[MAX_STAGES][NCW];  // per (stage, slot): partials of the P-1 helper warps posted
    float partial[MAX_STAGES][NCW][MAX_RPS][2];  // [stage][warp][row in set][gate|up]
    double norm_part[NCW];
    int abort_flag;
    unsigned int peer_done;   // consumer warps that have pushed all their rows to the peers (tensor parallel)
    // multi-matvec kernels: the producer (which runs ahead of the consumers) keeps the arguments of the
    // matvec it is streaming here instead of re-reading them from global memory
    StreamArgs pargs;
};

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                              int code = KERR_WAIT_TIMEOUT, long long limit = WAIT_CYCLE_LIMIT) {
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

constexpr uint32_t MAX_PEERS = 7;

// Consumer warps, before the input vector is read. false = gave up (status recorded).
__device__ __forceinline__ bool stream_wait_input(const StreamArgs& a, StreamSmem* sm) {
    if (a.wait_flag == nullptr) return true;
    if (threadIdx.x == 0) {
        const unsigned int expected = (ld_acquire_sys_u32(a.epoch) + 1u) * a.wait_mult;
        if (!peer_wait(a.wait_flag, expected, a.status, KERR_WAIT_PEER)) sm->abort_flag = 1;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
    return sm->abort_flag == 0;
}
// Consumer warps, after their last row: make the pushed rows visible, then tell every peer. The warps meet on a
// shared-memory counter with a bounded wait (no CTA barrier: after an abort some warps never get here).
__device__ __forceinline__ void stream_signal_peers(const StreamArgs& a, StreamSmem* sm, bool stored) {
    if (a.npeers == 0) return;
    if (stored) __threadfence_system();   // only the warps that finished rows have remote stores in flight
    __syncwarp();
    if ((threadIdx.x & 31) == 0) atomicAdd(&sm->peer_done, 1u);
    if (threadIdx.x == 0) {
        volatile unsigned int* done = &sm->peer_done;
        volatile int* abort_flag = &sm->abort_flag;
        const long long t0 = clock64();
        while (*done < NCW && !*abort_flag && clock64() - t0 < WAIT_CYCLE_LIMIT) {}
        if (*done >= NCW)
            for (uint32_t p = 0; p < a.npeers; p++) red_release_sys_add_u32(a.peer_flag[p], 1u);
    }
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

// F supplies:
//   struct Act;                                            per-position activation registers
//   static constexpr bool USES_Q8K;                        integer dot against Q8_K activations
//   static void load_act(Act&, const StreamArgs&, const float* x, bool x_cg, const Q8KView&, uint32_t u, bool valid)
//   static float unit(uint32_t row_smem_addr, uint32_t u, const Act&, const StreamArgs&)   partial dot of unit u
//   static float finish(float v, const StreamArgs&, const float* aux, uint32_t row)   per-row epilogue
// Per-CTA streaming state that outlives one matvec when several run back to back inside one
// kernel: the ring and its full / empty barriers are shared, `cc` counts the chunks ever pushed
// through it (stage = cc % nstages, phase from cc / nstages).
struct StreamCtx {
    StreamSmem* sm;
    uint8_t* smem_raw;
    uint32_t ring;          // shared address of stage 0
    uint32_t stage_stride;  // bytes between stages
    uint32_t nstages;
    uint32_t cc;            // chunks streamed so far (producer and consumers keep separate copies in step)
    int op;                 // index of the matvec inside a multi-op kernel (error reports)
    bool acts_cg;           // read global activations with ld.global.cg (other SMs rewrite them inside this kernel)
    long long* prof = nullptr;  // optional clock64 stamps of this matvec: [1] prologue done, [2] first stage landed, [3] rows done, [8..15] stage g done
};

// The per-(stage, warp set) barriers collect the P-1 helper warps of a row set. P changes from matvec
// to matvec inside a multi-matvec kernel, so instead of re-initialising them each barrier expects
// RED_COUNT = lcm(1, 3, 7) arrivals and every helper arrives with weight RED_COUNT / (P - 1). A barrier
// that a stage does not use (no such row set, or no rows left for it) is completed by its own warp, so
// every barrier finishes exactly one phase per stage use and shares the phase of the `full` barrier.
constexpr uint32_t RED_COUNT = 21;
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t n) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(n) : "memory");
}

__device__ __forceinline__ void stream_init_ring(StreamSmem* sm, uint32_t nstages) {
    for (uint32_t s = 0; s < nstages; s++) {
        mbar_init(smem_u32(&sm->full[s]), 1);
        mbar_init(smem_u32(&sm->empty[s]), NCW);
        for (uint32_t q = 0; q < NCW; q++) mbar_init(smem_u32(&sm->red[s][q]), RED_COUNT);
    }
    sm->abort_flag = 0;
    sm->peer_done = 0;
    mbar_fence_init();
}

__device__ __forceinline__ float ld_act(const float* p, bool cg) { return cg ? __ldcg(p) : *p; }
// float4 number i4 of the input vector (elements 4*i4 .. 4*i4+3). LL: the vector is in tagged form (the callers
// are compiled twice, so that the plain instance carries none of the polling code).
template <bool LL>
__device__ __forceinline__ float4 x_load4(const XSrc& s, uint32_t i4, StreamSmem* sm, int* status) {
    if (LL) return ll_load4(s.ll + (size_t)i4 * 4, s.tag, &sm->abort_flag, status);
    const float4* p = reinterpret_cast<const float4*>(s.x) + i4;
    return s.cg ? __ldcg(p) : *p;
}

// Producer side of one matvec: streams this CTA's row groups of `a` through the ring. One thread.
// PLAIN: the matvec is known to be a single matrix (no q/k/v segments).
template <bool PLAIN = false>
__device__ __forceinline__ void stream_produce(const StreamArgs& a, StreamCtx& cx) {
    StreamSmem* sm = cx.sm;
    volatile int* abort_flag = &sm->abort_flag;
    const uint32_t rows_per_group = a.slots * a.rps;
    const bool two = a.w1 != nullptr;
    const uint32_t g0 = (uint32_t)(((uint64_t)a.groups * blockIdx.x) / gridDim.x);
    const uint32_t g1 = (uint32_t)(((uint64_t)a.groups * (blockIdx.x + 1)) / gridDim.x);
    for (uint32_t g = g0; g < g1; g++) {
        const uint32_t s = cx.cc % cx.nstages, use = cx.cc / cx.nstages;
        if (use > 0 && !wait_or_abort(smem_u32(&sm->empty[s]), (use - 1) & 1, abort_flag, a.status, KERR_WAIT_EMPTY + (cx.op << 8), 2 * WAIT_CYCLE_LIMIT)) return;
        uint32_t sg = 0;
        if (!PLAIN) while (sg + 1 < a.nseg && g >= a.seg_g0[sg + 1]) sg++;
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
            ok = wait_or_abort(smem_u32(&sm->empty[s]), (use - 1) & 1, abort_flag, a.status, KERR_WAIT_EMPTY + (cx.op << 8), 2 * WAIT_CYCLE_LIMIT) ? 1 : 0;
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

// Input prologue of one matvec, run by the NCW consumer warps. A real function call on purpose: it runs
// once per matvec, so its code is fetched cold every time, and one shared compact copy (rolled loops)
// costs far fewer instruction-cache misses than a copy unrolled into every format's kernel body.
//   norm_w != null: rms_norm (src/llama3.rs:5244-5256) - f64 sum of squares, mean and scale in f32, then
//                   (x * scale) * w - into the f32 area at xn_off;
//   quant:          the (normalised) vector -> Q8_K in shared memory at q8_off (qs | bsums | d), one warp
//                   per 256-element block, exactly the stand-alone quantizer;
//   roundtrip:      (with norm_w) the normalised vector is replaced by d * q of its Q8_K quantization.
// cg: read x with ld.global.cg (other SMs rewrote it inside this kernel).
template <bool LL>
static __device__ __forceinline__ void stream_prologue_body(StreamSmem* sm, uint8_t* smem_raw, const XSrc xs, int* status,
                                                         const float* norm_w, float norm_eps, uint32_t cols, uint32_t xn_off,
                                                         uint32_t q8_off, bool quant, bool roundtrip) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const float* src = xs.x;
    bool src_global = true;
    if (norm_w != nullptr) {
        float* xn = reinterpret_cast<float*>(smem_raw + xn_off);
        // a thread's share of x stays in registers between the two passes when it fits in NORM_V float4
        // (cols <= NCW*32*4*NORM_V); the norm weights ride the same memory round trip as x
        constexpr int NORM_V = 4;
        const uint32_t nvec = cols / 4;
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
                if (i < nvec) xv[k] = x_load4<LL>(xs, i, sm, status);
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
                    const float4 v = one_round ? xv[k] : x_load4<LL>(xs, i, sm, status);
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
    if (quant) {
        const uint32_t nb = cols / QK_K;
        uint8_t* area = smem_raw + q8_off;
        int8_t* qs_s = reinterpret_cast<int8_t*>(area);
        int16_t* bs_s = reinterpret_cast<int16_t*>(area + (size_t)nb * 256);  // 8-byte aligned for any nb
        float* d_s = reinterpret_cast<float*>(area + (size_t)nb * 288);
        // QB blocks per warp per round: their loads travel together (one memory round trip per round when
        // the source is global memory) and their reduction chains interleave
        constexpr int QB = 4;
#pragma unroll 1
        for (uint32_t b0 = warp; b0 < nb; b0 += QB * NCW) {
            Q8KLaneInput in[QB];
#pragma unroll
            for (int i = 0; i < QB; i++) {
                const uint32_t blk = b0 + i * NCW;
                if (blk < nb) {
                    if (src_global) {   // the lane's 8 consecutive elements = float4 numbers 2*(blk*32 + lane), +1
                        in[i].a = x_load4<LL>(xs, 2 * (blk * 32 + lane), sm, status);
                        in[i].b = x_load4<LL>(xs, 2 * (blk * 32 + lane) + 1, sm, status);
                    } else {
                        in[i] = q8k_load_lane(src + (size_t)blk * QK_K, lane, false);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < QB; i++) {
                const uint32_t blk = b0 + i * NCW;
                if (blk < nb) q8k_quantize_block_warp(in[i], lane, qs_s + (size_t)blk * QK_K, d_s + blk, bs_s + (size_t)blk * 16);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
    }
}

// The same as one shared out-of-line copy: for kernels that run many matvecs (every format instance calls it, and
// a copy that stays warm in the instruction cache beats an inlined one that is cold every time).
static __device__ __noinline__ void stream_prologue(StreamSmem* sm, uint8_t* smem_raw, const XSrc xs, int* status, const float* norm_w,
                                                    float norm_eps, uint32_t cols, uint32_t xn_off, uint32_t q8_off,
                                                    bool quant, bool roundtrip) {
    if (xs.ll) stream_prologue_body<true>(sm, smem_raw, xs, status, norm_w, norm_eps, cols, xn_off, q8_off, quant, roundtrip);
    else stream_prologue_body<false>(sm, smem_raw, xs, status, norm_w, norm_eps, cols, xn_off, q8_off, quant, roundtrip);
}

// Consumer side of one matvec (the NCW consumer warps of the CTA, threads 0 .. NCW*32-1).
// Returns false after an abort.
// PLAIN: the matvec is known to use none of the fused extras (RMSNorm prologue, residual / argmax epilogue,
// q/k/v segments), so their code is compiled out - the stand-alone matvec entry points run this leaner instance.
// PEER: the tensor-parallel hand-over (pushed rows, tagged vectors, arrival counters) is compiled in; a single-GPU
// model runs the instance without it.
template <class F, int KL, bool SWIGLU, bool SHARED_PROLOGUE = false, bool PLAIN = false, bool PEER = false>
__device__ __forceinline__ bool stream_consume(const StreamArgs& a, StreamCtx& cx) {
    StreamSmem* sm = cx.sm;
    uint8_t* smem_raw = cx.smem_raw;
    volatile int* abort_flag = &sm->abort_flag;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t P = a.P, slots = a.slots, rps = a.rps;
    const uint32_t rows_per_group = slots * rps;
    const uint32_t slot = warp / P, part = warp % P;
    const bool cg = cx.acts_cg || (PEER && a.wait_flag != nullptr);
    if (PEER && !stream_wait_input(a, sm)) return false;   // rows other GPUs push into x
    const uint32_t y_tag = (PEER && a.y_ll != nullptr) ? ld_acquire_sys_u32(a.epoch) * a.y_n + a.y_seq + 1u : 0u;

    // input prologue (shared by every format, one copy of the code per kernel): RMSNorm into shared
    // memory and / or Q8_K quantization into shared memory
    const bool norm = !PLAIN && a.norm_w != nullptr;
    const float* const resid = PLAIN ? nullptr : a.resid;
    unsigned long long* const argmax_key = PLAIN ? nullptr : a.argmax_key;
    const uint32_t nseg = PLAIN ? 1u : a.nseg;
    const bool quant = F::USES_Q8K && a.q8.qs == nullptr;
    if (norm || quant) {
        XSrc xs;
        if (!PEER) { xs.x = a.x; xs.ll = nullptr; xs.tag = 0; xs.cg = cg; } else xs = xsrc_of(a, cg);
        if (SHARED_PROLOGUE)
            stream_prologue(sm, smem_raw, xs, a.status, PLAIN ? nullptr : a.norm_w, a.norm_eps, a.cols, a.xn_off, a.q8_off, quant,
                            !PLAIN && !F::USES_Q8K && a.q8k_roundtrip != 0);
        else if (PEER && xs.ll)   // tagged input (tensor parallel): the shared out-of-line copy
            stream_prologue(sm, smem_raw, xs, a.status, a.norm_w, a.norm_eps, a.cols, a.xn_off, a.q8_off, quant,
                            !F::USES_Q8K && a.q8k_roundtrip != 0);
        else
            stream_prologue_body<false>(sm, smem_raw, xs, a.status, PLAIN ? nullptr : a.norm_w, a.norm_eps, a.cols, a.xn_off, a.q8_off, quant,
                                        !PLAIN && !F::USES_Q8K && a.q8k_roundtrip != 0);
    }
    const float* x_src = norm ? reinterpret_cast<const float*>(smem_raw + a.xn_off) : a.x;
    const bool x_global = !norm;
    Q8KView q8 = a.q8;
    if (quant) {
        const uint32_t nb = a.cols / QK_K;
        const uint8_t* area = smem_raw + a.q8_off;
        q8.qs = reinterpret_cast<const int8_t*>(area);
        q8.bsums = reinterpret_cast<const int16_t*>(area + (size_t)nb * 256);
        q8.d = reinterpret_cast<const float*>(area + (size_t)nb * 288);
        q8.nb = nb;
    }
    typename F::Act act[KL];
#pragma unroll
    for (int k = 0; k < KL; k++) {
        const uint32_t u = ((uint32_t)k * P + part) * 32 + lane;
        F::load_act(act[k], a, x_src, x_global && cg, q8, u, u < a.units);
    }
    if (cx.prof && threadIdx.x == 0) cx.prof[1] = clock64();

    // Rows are walked RB at a time so that RB*M independent unit decodes are in flight per lane
    // and one butterfly reduces all of them (NV-1 + log2(32/NV) shuffles instead of 5*NV).
    constexpr int M = SWIGLU ? 2 : 1;
    constexpr int RB = KL == 1 ? (SWIGLU ? 2 : 4) : (KL == 2 ? (SWIGLU ? 1 : 2) : 1);
    constexpr int NV = RB * M;
    constexpr uint32_t LANES_PER_VALUE = 32 / NV;

    const uint32_t g0 = (uint32_t)(((uint64_t)a.groups * blockIdx.x) / gridDim.x);
    const uint32_t g1 = (uint32_t)(((uint64_t)a.groups * (blockIdx.x + 1)) / gridDim.x);
    for (uint32_t g = g0; g < g1; g++) {
        const uint32_t s = cx.cc % cx.nstages, ph = (cx.cc / cx.nstages) & 1;
        cx.cc++;
        uint32_t sg = 0;
        while (sg + 1 < nseg && g >= a.seg_g0[sg + 1]) sg++;
        const uint32_t seg_rows = a.seg_rows[sg];
        const uint32_t r0 = (g - a.seg_g0[sg]) * rows_per_group;
        const uint32_t pad = (uint32_t)(((uint64_t)r0 * a.row_bytes) & 15);
        const uint32_t set0 = slot * rps;                 // first row (within the stage) of this warp set
        const uint32_t nrow = r0 + set0 < seg_rows ? min(rps, seg_rows - r0 - set0) : 0;
        // the residual this lane will add in the epilogue: requested now, needed after the rows are done
        float res = 0.0f;
        if (part == 0 && lane < nrow) {
            if (PEER && a.resid_ll != nullptr) res = ll_value(a.resid_ll + a.seg_y[sg] + r0 + set0 + lane);
            else if (resid != nullptr) res = ld_act(resid + a.seg_y[sg] + r0 + set0 + lane, cg);
        }
        if (!wait_or_abort(smem_u32(&sm->full[s]), ph, abort_flag, a.status, KERR_WAIT_FULL + (cx.op << 8))) return false;
        if (cx.prof && threadIdx.x == 0 && g == g0) cx.prof[2] = clock64();
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
                if (P > 1 && !wait_or_abort(smem_u32(&sm->red[s][slot]), ph, abort_flag, a.status, KERR_WAIT_PARTIALS + (cx.op << 8))) return false;
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
                    float r = F::finish(v0, a, PLAIN ? a.aux0 : a.seg_aux[sg], row);
                    if (SWIGLU) r = silu_ref(r) * F::finish(v1, a, a.aux1, row);
                    const uint32_t yi = a.seg_y[sg] + row;
                    if (resid != nullptr || (PEER && a.resid_ll != nullptr)) r = __fadd_rn(res, r);
                    if (PEER && a.y_ll != nullptr) {   // tagged vector: this GPU's copy and the peers'
                        ll_store(a.y_ll + yi, r, y_tag);
                        for (uint32_t p = 0; p < a.npeers; p++) ll_store(a.peer_y_ll[p] + yi, r, y_tag);
                    } else {
                        a.y[yi] = r;
                        if (PEER) for (uint32_t p = 0; p < a.npeers; p++) a.peer_y[p][yi] = r;
                    }
                    const uint32_t b = __float_as_uint(r);
                    const uint32_t ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
                    if (argmax_key != nullptr && r == r) key = ((unsigned long long)ordered << 32) | (0xFFFFFFFFu - yi);
                }
                if (argmax_key != nullptr) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
                        key = other > key ? other : key;
                    }
                    if (lane == 0) atomicMax(argmax_key, key);
                }
                if (cx.prof && threadIdx.x == 0 && g - g0 < 8) cx.prof[8 + g - g0] = clock64();
                continue;   // this warp has already released the stage
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm->empty[s]));
        if (cx.prof && threadIdx.x == 0 && g - g0 < 8) cx.prof[8 + g - g0] = clock64();
    }
    if (cx.prof && threadIdx.x == 0) cx.prof[3] = clock64();
    if (PEER && a.y_ll == nullptr) stream_signal_peers(a, sm, part == 0);
    return true;
}

// One matvec per launch.
template <class F, int KL, bool SWIGLU, bool PLAIN, bool PEER>
__global__ void __launch_bounds__(STREAM_THREADS, KL <= 2 ? 2 : 1) stream_gemv_kernel(const StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    StreamSmem* sm = reinterpret_cast<StreamSmem*>(smem_raw);
    constexpr uint32_t HDR = (sizeof(StreamSmem) + 127) & ~127u;
    StreamCtx cx;
    cx.sm = sm; cx.smem_raw = smem_raw; cx.ring = smem_u32(smem_raw) + HDR;
    cx.stage_stride = a.cap * (SWIGLU ? 2u : 1u); cx.nstages = a.nstages; cx.cc = 0; cx.op = 0; cx.acts_cg = false;
    if (threadIdx.x == 0) stream_init_ring(sm, a.nstages);
    __syncthreads();
    pdl_launch_dependents();
    if ((threadIdx.x >> 5) == NCW) {
        // producer: weights do not depend on the previous kernel, so copies start at once
        if ((threadIdx.x & 31) == 0) {
            stream_produce<PLAIN>(a, cx);
            if (sm->abort_flag) stream_drain(cx);
        }
        return;
    }
    pdl_wait();  // activations come from the previous kernel
    stream_consume<F, KL, SWIGLU, false, PLAIN, PEER>(a, cx);
}

}  // namespace alice
