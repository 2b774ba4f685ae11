// Planning and launch of the streaming matvec kernels (one template instance per format,
// activation positions per lane KL in {1,2,4}, plain / fused SwiGLU).
#include <algorithm>
#include <cstdlib>

#include "../../include/alice_cuda.h"
#include "formats.cuh"
#include "gemv_mma.cuh"
#include "gemv_kq_mma.cuh"
#include "gemv_launch.cuh"
#include "gemv_plan.cuh"

namespace alice {

bool format_uses_q8k(WeightFormat f) { return f == WF_Q4_K || f == WF_Q5_K || f == WF_Q6_K; }

uint32_t ggml_block_bytes(WeightFormat f) {
    switch (f) {
        case WF_Q8_0: return 34; case WF_Q4_K: return 144; case WF_Q5_K: return 176;
        case WF_Q6_K: return 210; case WF_Q1_0: return 18; case WF_Q2_0: return 34;
        default: return 0;
    }
}
uint32_t ggml_block_elems(WeightFormat f) {
    switch (f) {
        case WF_Q8_0: return 32;
        case WF_Q4_K: case WF_Q5_K: case WF_Q6_K: return 256;
        case WF_Q1_0: case WF_Q2_0: return 128;
        default: return 0;
    }
}
uint32_t ggml_row_bytes(WeightFormat f, uint32_t cols) {
    const uint32_t e = ggml_block_elems(f);
    if (e == 0 || cols == 0 || cols % e != 0) return 0;
    return cols / e * ggml_block_bytes(f);
}

namespace {

// Shared memory per CTA: two CTAs share an SM when a lane holds at most two activation positions
// (KL <= 2), else one CTA has the SM to itself (of the 227 KB a CTA may opt in to).
constexpr uint32_t SMEM_BUDGET_2 = 112 * 1024, SMEM_BUDGET_1 = 200 * 1024;
constexpr uint32_t DEFAULT_STAGES = 2;         // measured: a deeper ring buys nothing, larger stages do
constexpr uint32_t HDR_BYTES = (sizeof(StreamSmem) + 127) & ~127u;

uint32_t units_per_row(WeightFormat f, uint32_t cols) {
    switch (f) {
        case WF_Q4_K: case WF_Q5_K: return cols / 64;
        case WF_Q6_K: return cols / 32;
        case WF_Q8_0: return cols / 16;
        case WF_Q1_0: return cols / 32;
        case WF_Q2_0: return cols / 16;
        case WF_TERNARY: case WF_SPARSE_TERNARY: return (cols + 31) / 32;
        default: return 0;
    }
}

// cudaFuncSetAttribute is per device: remember, per kernel instance, the devices it has been raised on.
bool attr_needed(bool (&done)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if (done[dev]) return false;
    done[dev] = true;
    return true;
}

template <class K>
int launch_kernel(K kern, const StreamArgs& a, uint32_t grid, size_t smem, const LaunchCfg& cfg) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(STREAM_THREADS);
    lc.dynamicSmemBytes = smem;
    lc.stream = cfg.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, kern, a) == cudaSuccess ? ALICE_OK : ALICE_E_CUDA;
}

template <class F, int KL, bool SW, bool PEER, bool PLAIN>
int launch_one_v(const StreamArgs& a, uint32_t grid, size_t smem, const LaunchCfg& cfg) {
    static bool attr_done[64] = {};  // per template instance
    auto kern = stream_gemv_kernel<F, KL, SW, PEER, PLAIN>;
    if (attr_needed(attr_done) &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(KL <= 2 ? SMEM_BUDGET_2 : SMEM_BUDGET_1)) != cudaSuccess)
        return ALICE_E_CUDA;
    return launch_kernel(kern, a, grid, smem, cfg);
}

// The instance with the tensor-parallel row push only when the matvec takes part in one.
template <class F, int KL, bool SW>
int launch_one(const StreamArgs& a, uint32_t grid, size_t smem, const LaunchCfg& cfg) {
    const bool peer = a.npeers != 0;
    if (peer) return launch_one_v<F, KL, SW, true, false>(a, grid, smem, cfg);
    const bool plain = !a.resid && !a.argmax_key && a.nseg == 1;
    return plain ? launch_one_v<F, KL, SW, false, true>(a, grid, smem, cfg) : launch_one_v<F, KL, SW, false, false>(a, grid, smem, cfg);
}

template <class F>
int launch_fmt(const StreamArgs& a, uint32_t kl, bool sw, uint32_t grid, size_t smem, const LaunchCfg& cfg) {
    if (sw) {
        if (kl == 1) return launch_one<F, 1, true>(a, grid, smem, cfg);
        if (kl == 2) return launch_one<F, 2, true>(a, grid, smem, cfg);
        return launch_one<F, 4, true>(a, grid, smem, cfg);
    }
    if (kl == 1) return launch_one<F, 1, false>(a, grid, smem, cfg);
    if (kl == 2) return launch_one<F, 2, false>(a, grid, smem, cfg);
    return launch_one<F, 4, false>(a, grid, smem, cfg);
}

// Geometry of the bit-plane tensor-core kernel: 16-row tiles, `slots` tiles per stage, the P = NCW / slots
// warps of a tile split the row's 16-byte groups. Shared memory: header | ring | normalised input (optional) |
// activation digit table (512 B per 128 columns) | per-block sums. Two CTAs per SM when that fits.
// [col_lo, col_lo + col_n) selects a column sub-range of the matrix (the whole row when col_n == cols): a
// matrix whose rows are too wide for shared memory runs as several such launches that accumulate into y.
constexpr uint32_t MMA_BUDGET_2 = 112 * 1024, MMA_BUDGET_1 = 225 * 1024;
int plan_mma(const GemvOp& op, const LaunchCfg& cfg, StreamArgs a, uint32_t col_lo, uint32_t col_n, StreamPlan& pl) {
    const WeightDesc& w0 = *op.w[0];
    const bool sw = op.up != nullptr;
    const uint32_t nmat = sw ? 2 : 1;
    const bool whole = col_lo == 0 && col_n == w0.cols;
    if (!whole && (sw || col_lo % 128 || col_n % 128)) return ALICE_E_SHAPE;
    // the sub-row as the consumer sees it, and where its pieces sit inside the global row
    uint32_t sub_row, npieces, piece_len, piece_off[2] = {0, 0};
    if (w0.fmt == WF_Q1_0 || w0.fmt == WF_Q2_0) {
        const uint32_t bb = w0.fmt == WF_Q1_0 ? 18u : 34u;
        npieces = 1; piece_len = col_n / 128 * bb; piece_off[0] = col_lo / 128 * bb; sub_row = piece_len;
    } else if (w0.fmt == WF_SPARSE_TERNARY) {
        npieces = 1; piece_len = (col_n + 15) / 16 * 4; piece_off[0] = col_lo / 16 * 4; sub_row = piece_len;
    } else {
        const uint32_t plane_full = w0.row_bytes / 2;
        npieces = 2; piece_len = (col_n + 31) / 32 * 4; piece_off[0] = col_lo / 8; piece_off[1] = plane_full + col_lo / 8;
        sub_row = 2 * piece_len;
    }
    const bool row_ok = piece_len % 16 == 0 && w0.row_bytes % 16 == 0 && piece_off[0] % 16 == 0 && piece_off[1] % 16 == 0;
    if (!row_ok && !whole) return ALICE_E_SHAPE;
    // shared-memory row stride: an odd number of 16-byte units, so the 8 rows x 4 words one A-fragment load
    // touches fall into 32 different banks
    uint32_t row_stride = sub_row;
    if (row_ok) { row_stride = (sub_row + 15) & ~15u; if ((row_stride / 16) % 2 == 0) row_stride += 16; }
    a.cols = col_n; a.row_bytes = sub_row; a.row_stride = row_stride; a.row_mode = row_ok ? 1u : 0u;
    a.src_row_bytes = w0.row_bytes; a.npieces = npieces; a.piece_len = piece_len;
    a.piece_off[0] = piece_off[0]; a.piece_off[1] = piece_off[1];
    if (a.x) a.x += col_lo;
    const uint32_t ge = (w0.fmt == WF_Q2_0 || w0.fmt == WF_SPARSE_TERNARY) ? 64u : 128u;   // elements per 16 weight bytes
    const uint32_t ngroups = (col_n + ge - 1) / ge;
    const uint32_t table_bytes = (mma_blob_bytes(ngroups) + 127u) & ~127u;   // digit table, per-block sums, fixed-point unit
    for (uint32_t per_sm = 2; per_sm >= 1; per_sm--) {
        const uint32_t budget = per_sm == 2 ? MMA_BUDGET_2 : MMA_BUDGET_1;
        if (HDR_BYTES + table_bytes >= budget) continue;
        const uint32_t avail = budget - HDR_BYTES - table_bytes;
        const uint32_t ctas = (uint32_t)std::max(cfg.num_sms, 1) * per_sm;
        uint32_t best = 0;
        for (uint32_t slots = NCW; slots >= 1; slots /= 2) {
            const uint32_t cap = (slots * 16 * row_stride + 48 + 127) & ~127u;
            if ((uint64_t)cap * nmat * 2 > avail) continue;
            best = slots;                                      // fits; keep shrinking while the CTAs are short of stages
            uint32_t groups = 0;
            for (uint32_t i = 0; i < op.nw; i++) groups += (op.w[i]->rows + slots * 16 - 1) / (slots * 16);
            if (groups >= 2 * ctas) break;
        }
        if (best == 0) continue;
        const uint32_t slots = best;
        a.slots = slots; a.P = NCW / slots; a.rps = 16;
        a.cap = (slots * 16 * row_stride + 48 + 127) & ~127u;
        const uint32_t stage = a.cap * nmat;
        // as deep a ring as fits: the bytes in flight per SM have to cover memory latency at full bandwidth
        const uint32_t nst = std::min<uint32_t>(MAX_STAGES, avail / stage);
        a.nstages = nst;
        a.nseg = op.nw;
        a.groups = 0;
        for (uint32_t i = 0; i < op.nw; i++) {
            a.seg_w[i] = op.w[i]->data; a.seg_rows[i] = op.w[i]->rows; a.seg_y[i] = op.y_off[i]; a.seg_aux[i] = op.w[i]->scales;
            a.seg_g0[i] = a.groups;
            a.groups += (op.w[i]->rows + slots * 16 - 1) / (slots * 16);
        }
        a.seg_g0[op.nw] = a.groups;
        a.tab_off = HDR_BYTES + nst * stage;
        pl.grid = std::min(ctas, a.groups);
        pl.smem = HDR_BYTES + nst * (size_t)stage + table_bytes;
        pl.kl = 1; pl.swiglu = sw; pl.stage = stage;
        pl.mma = true; pl.ctas_per_sm = per_sm;
        pl.args = a;
        return ALICE_OK;
    }
    return ALICE_E_SHAPE;
}

// Column chunk c of ksplit: whole multiples of `unit` columns (Q1_0: 1024, so that a chunk of a row is a multiple
// of 16 bytes; ternary planes: 128).
void mma_chunk(const WeightDesc& w, uint32_t ksplit, uint32_t c, uint32_t& lo, uint32_t& n) {
    const uint32_t unit = (w.fmt == WF_Q1_0 || w.fmt == WF_Q2_0) ? 1024u : 128u, units = w.cols / unit;
    lo = units * c / ksplit * unit;
    n = units * (c + 1) / ksplit * unit - lo;
}

// Whole row if it fits, else the smallest number of column chunks that does (plain matvec only).
int plan_mma_split(const GemvOp& op, const LaunchCfg& cfg, const StreamArgs& a, StreamPlan& pl) {
    const WeightDesc& w0 = *op.w[0];
    if (plan_mma(op, cfg, a, 0, w0.cols, pl) == ALICE_OK) { pl.ksplit = 1; return ALICE_OK; }
    const uint32_t unit = (w0.fmt == WF_Q1_0 || w0.fmt == WF_Q2_0) ? 1024u : 128u;
    if (w0.cols % unit || op.up) return ALICE_E_SHAPE;
    for (uint32_t ks = 2; ks <= 4; ks++) {
        bool ok = true;
        for (uint32_t c = 0; c < ks && ok; c++) {
            uint32_t lo, n;
            mma_chunk(w0, ks, c, lo, n);
            StreamPlan tmp;
            ok = n > 0 && plan_mma(op, cfg, a, lo, n, tmp) == ALICE_OK;
            if (ok && c == 0) pl = tmp;
        }
        if (ok) { pl.ksplit = ks; return ALICE_OK; }
    }
    return ALICE_E_SHAPE;
}

template <class M, bool SW, int CTAS, bool PEER>
int launch_mma_one(const StreamArgs& a, uint32_t grid, size_t smem, const LaunchCfg& cfg) {
    static bool attr_done[64] = {};  // per template instance
    auto kern = stream_gemv_mma_kernel<M, SW, CTAS, PEER>;
    if (attr_needed(attr_done) &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(CTAS == 2 ? MMA_BUDGET_2 : MMA_BUDGET_1)) != cudaSuccess)
        return ALICE_E_CUDA;
    return launch_kernel(kern, a, grid, smem, cfg);
}

template <class M, bool PEER>
int launch_mma_p(const StreamPlan& pl, const LaunchCfg& cfg) {
    if (pl.swiglu) return pl.ctas_per_sm == 2 ? launch_mma_one<M, true, 2, PEER>(pl.args, pl.grid, pl.smem, cfg)
                                              : launch_mma_one<M, true, 1, PEER>(pl.args, pl.grid, pl.smem, cfg);
    return pl.ctas_per_sm == 2 ? launch_mma_one<M, false, 2, PEER>(pl.args, pl.grid, pl.smem, cfg)
                               : launch_mma_one<M, false, 1, PEER>(pl.args, pl.grid, pl.smem, cfg);
}
// the instance with the tensor-parallel hand-over only when the matvec takes part in one
template <class M>
int launch_mma(const StreamPlan& pl, const LaunchCfg& cfg) {
    const StreamArgs& a = pl.args;
    const bool peer = a.npeers != 0;
    return peer ? launch_mma_p<M, true>(pl, cfg) : launch_mma_p<M, false>(pl, cfg);
}

}  // namespace

// ---- batched K-quant matvec on the int8 tensor cores (csrc/gemv_kq_mma.cuh) --------------------------------------
namespace {
constexpr uint32_t KQ_PART_BYTES = (sizeof(KqPartials) + 127) & ~127u;

uint32_t kq_block_bytes(WeightFormat f) { return f == WF_Q4_K ? 144u : f == WF_Q5_K ? 176u : 210u; }

// Column chunk [col_lo, col_lo + col_n) of the matrix (whole 256-blocks); the whole row when col_n == cols.
int plan_kq(const GemvOp& op, const LaunchCfg& cfg, uint32_t col_lo, uint32_t col_n, StreamPlan& pl) {
    const WeightDesc& w0 = *op.w[0];
    const bool sw = op.up != nullptr;
    const uint32_t nmat = sw ? 2 : 1, bb = kq_block_bytes(w0.fmt), nbc = col_n / 256u;
    if (w0.row_bytes % 16 || col_lo % 256 || col_n % 256 || nbc == 0) return ALICE_E_SHAPE;
    const uint32_t off = col_lo / 256u * bb, pad = off & 15u;
    const uint32_t piece_len = (pad + nbc * bb + 15u) & ~15u;
    uint32_t row_stride = (piece_len + 31u) & ~31u;
    while (row_stride % 128u != 32u && row_stride % 128u != 96u) row_stride += 32u;
    const uint32_t acts = kq_acts_bytes(col_n);
    StreamArgs a = {};
    a.w0 = w0.data; a.w1 = sw ? op.up->data : nullptr;
    a.q8 = *op.q8;
    a.q8.qs += col_lo; a.q8.d += col_lo / 256u; a.q8.bsums += (size_t)(col_lo / 256u) * 16;
    a.y = op.y; a.status = cfg.status;
    a.cols = col_n; a.row_bytes = nbc * bb; a.row_stride = row_stride; a.row_mode = 1; a.src_row_bytes = w0.row_bytes;
    a.npieces = 1; a.piece_len = piece_len; a.piece_off[0] = off - pad; a.row_pad = pad;
    a.batch = op.batch; a.x_stride = w0.cols;
    a.resid = op.resid; a.wait_limit = op.wait_limit;
    uint32_t total_rows = 0;
    for (uint32_t i = 0; i < op.nw; i++) total_rows += op.w[i]->rows;
    a.rows = total_rows; a.y_stride = op.y_stride ? op.y_stride : total_rows;
    for (uint32_t per_sm = 2; per_sm >= 1; per_sm--) {
        const uint32_t budget = per_sm == 2 ? MMA_BUDGET_2 : MMA_BUDGET_1;
        if (HDR_BYTES + KQ_PART_BYTES + acts >= budget) continue;
        const uint32_t avail = budget - HDR_BYTES - KQ_PART_BYTES - acts;
        const uint32_t ctas = (uint32_t)std::max(cfg.num_sms, 1) * per_sm;
        uint32_t best = 0;
        for (uint32_t slots = NCW; slots >= 1; slots /= 2) {
            const uint32_t cap = (slots * 16 * row_stride + 127) & ~127u;
            if ((uint64_t)cap * nmat * 2 > avail || NCW / slots > nbc) continue;
            best = slots;                                      // fits; keep shrinking while the CTAs are short of stages
            uint32_t groups = 0;
            for (uint32_t i = 0; i < op.nw; i++) groups += (op.w[i]->rows + slots * 16 - 1) / (slots * 16);
            if (groups >= 2 * ctas) break;
        }
        if (best == 0) continue;
        a.slots = best; a.P = NCW / best; a.rps = 16;
        a.cap = (best * 16 * row_stride + 127) & ~127u;
        a.nstages = 2;       // the partial-sum area is double buffered by stage
        a.nseg = op.nw;
        a.groups = 0;
        for (uint32_t i = 0; i < op.nw; i++) {
            a.seg_w[i] = op.w[i]->data; a.seg_rows[i] = op.w[i]->rows; a.seg_y[i] = op.y_off[i]; a.seg_aux[i] = nullptr;
            a.seg_g0[i] = a.groups;
            a.groups += (op.w[i]->rows + best * 16 - 1) / (best * 16);
        }
        a.seg_g0[op.nw] = a.groups;
        a.tab_off = HDR_BYTES + KQ_PART_BYTES + 2 * a.cap * nmat;
        pl.grid = std::min(ctas, a.groups);
        pl.smem = (size_t)a.tab_off + acts;
        pl.kl = 1; pl.swiglu = sw; pl.stage = a.cap * nmat; pl.mma = true; pl.ctas_per_sm = per_sm; pl.ksplit = 1;
        pl.args = a;
        return ALICE_OK;
    }
    return ALICE_E_SHAPE;
}

template <class T, bool SW, int CTAS>
int launch_kq_one(const StreamPlan& pl, const LaunchCfg& cfg) {
    static bool attr_done[64] = {};
    auto kern = stream_gemv_kq_kernel<T, SW, CTAS>;
    if (attr_needed(attr_done) &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(CTAS == 2 ? MMA_BUDGET_2 : MMA_BUDGET_1)) != cudaSuccess)
        return ALICE_E_CUDA;
    return launch_kernel(kern, pl.args, pl.grid, pl.smem, cfg);
}
template <class T>
int launch_kq_fmt(const StreamPlan& pl, const LaunchCfg& cfg) {
    if (pl.swiglu) return pl.ctas_per_sm == 2 ? launch_kq_one<T, true, 2>(pl, cfg) : launch_kq_one<T, true, 1>(pl, cfg);
    return pl.ctas_per_sm == 2 ? launch_kq_one<T, false, 2>(pl, cfg) : launch_kq_one<T, false, 1>(pl, cfg);
}

// The whole batch in one pass over the weights: one launch, or one per column chunk when 16 rows of the matrix do not
// fit a stage (a later chunk adds to what the earlier ones left in y). ALICE_E_SHAPE: no such plan (the caller falls
// back to one launch per vector).
int launch_kq_batch(const GemvOp& op, const LaunchCfg& cfg, bool dry, uint32_t* nlaunch) {
    const WeightDesc& w0 = *op.w[0];
    if (!format_uses_q8k(w0.fmt) || !op.q8 || op.argmax_key || op.npeers || op.norm_w) return ALICE_E_SHAPE;
    if (((uintptr_t)op.q8->qs & 15) || w0.cols % 256) return ALICE_E_SHAPE;
    for (uint32_t i = 0; i < op.nw; i++)
        if (op.w[i]->fmt != w0.fmt || op.w[i]->cols != w0.cols || ((uintptr_t)op.w[i]->data & 15)) return ALICE_E_SHAPE;
    if (op.up && (op.nw != 1 || op.up->fmt != w0.fmt || op.up->rows != w0.rows || op.up->cols != w0.cols)) return ALICE_E_SHAPE;
    const uint32_t nbt = w0.cols / 256u;
    for (uint32_t ks = 1; ks <= 8; ks++) {
        if (ks > 1 && op.up) break;          // the fused SwiGLU needs whole rows (silu of the complete gate)
        if (nbt % ks) continue;
        const uint32_t nbc = nbt / ks;
        if ((nbc * 256u) % 16u) continue;
        StreamPlan probe;
        if (plan_kq(op, cfg, 0, nbc * 256u, probe) != ALICE_OK) continue;
        if (nlaunch) *nlaunch = ks;
        if (dry) return ALICE_OK;
        for (uint32_t c = 0; c < ks; c++) {
            StreamPlan pc;
            const int rc = plan_kq(op, cfg, c * nbc * 256u, nbc * 256u, pc);
            if (rc) return rc;
            if (c > 0) pc.args.resid = op.y;
            const int lrc = w0.fmt == WF_Q4_K ? launch_kq_fmt<KqK4<false>>(pc, cfg) : w0.fmt == WF_Q5_K ? launch_kq_fmt<KqK4<true>>(pc, cfg)
                                                                                                        : launch_kq_fmt<KqQ6K>(pc, cfg);
            if (lrc) return lrc;
        }
        return ALICE_OK;
    }
    return ALICE_E_SHAPE;
}
}  // namespace

int plan_stream_gemv(const GemvOp& op, const LaunchCfg& cfg, StreamPlan& pl) {
    if (op.nw < 1 || op.nw > 3 || !op.w[0] || !op.y) return ALICE_E_INVALID;
    const WeightDesc& w0 = *op.w[0];
    const WeightDesc* w1 = op.up;
    const Q8KView* q8 = op.q8;
    const float* x = op.x;
    const bool sw = w1 != nullptr;
    if (sw && op.nw != 1) return ALICE_E_INVALID;
    if (w0.rows == 0 || w0.cols == 0 || !w0.data) return ALICE_E_INVALID;
    if (sw && (w1->fmt != w0.fmt || w1->rows != w0.rows || w1->cols != w0.cols || w1->row_bytes != w0.row_bytes))
        return ALICE_E_SHAPE;
    if (((uintptr_t)w0.data & 15) || (sw && ((uintptr_t)w1->data & 15))) return ALICE_E_INVALID;
    uint32_t total_rows = 0;
    for (uint32_t i = 0; i < op.nw; i++) {
        const WeightDesc* wi = op.w[i];
        if (!wi || !wi->data || ((uintptr_t)wi->data & 15) || wi->rows == 0) return ALICE_E_INVALID;
        if (wi->fmt != w0.fmt || wi->cols != w0.cols || wi->row_bytes != w0.row_bytes) return ALICE_E_SHAPE;
        total_rows += wi->rows;
    }
    // the input arrives prepared: Q8_K blocks for the K-quants, the f32 vector for everything else
    if (format_uses_q8k(w0.fmt)) {
        if (q8 ? q8->qs == nullptr : x == nullptr) return ALICE_E_INVALID;
        if (q8 && q8->nb * 256u != w0.cols) return ALICE_E_SHAPE;
        if (q8 && op.norm_w) return ALICE_E_INVALID;   // the norm needs the f32 vector
    } else if (!x) {
        return ALICE_E_INVALID;
    }
    const uint32_t units = units_per_row(w0.fmt, w0.cols);
    if (units == 0) return ALICE_E_UNSUPPORTED;

    StreamArgs a = {};
    a.w0 = w0.data; a.w1 = sw ? w1->data : nullptr;
    if (q8) a.q8 = *q8;
    a.x = x; a.aux0 = w0.scales; a.aux1 = sw ? w1->scales : nullptr;
    a.y = op.y; a.status = cfg.status;
    a.rows = total_rows; a.cols = w0.cols; a.row_bytes = w0.row_bytes; a.units = units;
    a.batch = 1; a.y_stride = op.y_stride ? op.y_stride : total_rows;
    a.resid = op.resid; a.argmax_key = op.argmax_key;
    a.npeers = std::min<uint32_t>(op.npeers, MAX_PEERS);
    for (uint32_t p = 0; p < a.npeers; p++) a.peer_y[p] = op.peer_y[p];
    a.wait_limit = op.wait_limit;
    a.row_stride = a.row_bytes;   // contiguous staging unless the tensor-core planner says otherwise
    if ((w0.fmt == WF_Q1_0 || w0.fmt == WF_Q2_0 || w0.fmt == WF_TERNARY || w0.fmt == WF_SPARSE_TERNARY) && w0.cols % 4 == 0 &&
        ((uintptr_t)x & 15) == 0 && !op.norm_w && plan_mma_split(op, cfg, a, pl) == ALICE_OK)
        return ALICE_OK;

    // warps per row: just enough lanes for one unit each, at most all eight
    uint32_t P = 1;
    while (P < (uint32_t)NCW && P * 32 < units) P *= 2;
    uint32_t kl = (units + P * 32 - 1) / (P * 32);
    if (kl > 4) return ALICE_E_SHAPE;  // row too wide for the register-resident activation scheme
    if (kl == 3) kl = 4;
    a.P = P; a.slots = NCW / P;

    const uint32_t nmat = sw ? 2 : 1;
    const uint32_t per_sm = kl <= 2 ? 2 : 1;
    const uint32_t full_budget = kl <= 2 ? SMEM_BUDGET_2 : SMEM_BUDGET_1;
    uint32_t nst = cfg.force_stages >= 2 ? std::min<uint32_t>(cfg.force_stages, MAX_STAGES) : DEFAULT_STAGES;
    // activation area: only when the kernel prepares the raw f32 vector itself (normalised f32 copy and / or Q8_K blocks)
    uint32_t act_bytes = 0;
    const bool kq = format_uses_q8k(w0.fmt);
    if ((kq && !q8) || op.norm_w) {
        if (((uintptr_t)x & 15) || (op.norm_w && (((uintptr_t)op.norm_w & 15) || w0.cols % 4))) return ALICE_E_INVALID;
        const uint32_t nb = w0.cols / 256u;
        const uint32_t xn_bytes = op.norm_w ? (w0.cols * 4u + 127u) & ~127u : 0u;
        const uint32_t q8_bytes = kq ? (nb * 292u + 127u) & ~127u : 0u;
        a.pro_mode = 1; a.pro_norm_w = op.norm_w; a.pro_eps = op.norm_eps;
        a.pro_roundtrip = (!kq && op.q8k_roundtrip && op.norm_w && w0.cols % QK_K == 0) ? 1u : 0u;
        a.pro_q8_off = xn_bytes;
        act_bytes = xn_bytes + q8_bytes;
    }
    if (HDR_BYTES + act_bytes + 8192 > full_budget) return ALICE_E_SHAPE;
    const uint32_t budget = full_budget - HDR_BYTES - act_bytes;
    const uint32_t ctas = (uint32_t)std::max(cfg.num_sms, 1) * per_sm;
    // rows per warp set per stage: as many as the ring allows (per-stage costs are amortised over
    // them) while every CTA still gets about two stages of work. Measured on 4096 x 4096 Q4_K in a chain of
    // dependent launches: 7.1 us with four stages per CTA, 5.8 with two, 5.1 with one; the whole decode step
    // is fastest with two (a small matrix is in flight in full after the first copies, so the stage count
    // only sets how many wait -> dot -> reduce hand-overs each warp runs back to back)
    uint32_t rps_bytes = std::max<uint32_t>(1, (budget / nst - 256) / std::max<uint32_t>(1, a.slots * a.row_bytes * nmat));
    uint32_t rps_bal = std::max<uint32_t>(1, (total_rows + a.slots * ctas * 2 - 1) / (a.slots * ctas * 2));
    uint32_t rps = std::min<uint32_t>(std::min(rps_bytes, rps_bal), MAX_RPS);
    if (cfg.force_rps > 0) rps = std::min<uint32_t>(cfg.force_rps, MAX_RPS);
    uint32_t cap, stage;
    for (;;) {
        cap = (a.slots * rps * a.row_bytes + 48 + 127) & ~127u;
        stage = cap * nmat;
        if (stage * nst <= budget) break;
        if (rps > 1) { rps--; continue; }
        if (nst > 2) { nst--; continue; }
        return ALICE_E_SHAPE;  // a single row does not fit twice into shared memory
    }
    a.rps = rps; a.cap = cap; a.nstages = nst;
    a.nseg = op.nw;
    // the rows are dealt out in "set rows" of `slots` rows (RowWalk, csrc/gemv_stream.cuh)
    uint32_t total_sets = 0;
    for (uint32_t i = 0; i < op.nw; i++) {
        a.seg_w[i] = op.w[i]->data; a.seg_rows[i] = op.w[i]->rows; a.seg_y[i] = op.y_off[i]; a.seg_aux[i] = op.w[i]->scales;
        a.seg_t0[i] = total_sets;
        total_sets += (op.w[i]->rows + a.slots - 1) / a.slots;
    }
    for (uint32_t i = op.nw; i < 4; i++) a.seg_t0[i] = total_sets;
    pl.grid = std::min(ctas, total_sets);
    // the number of stages the walk produces, over all CTAs (what alice_plan_query reports)
    a.groups = 0;
    for (uint32_t cta = 0; cta < pl.grid; cta++) {
        uint32_t t = (uint32_t)((uint64_t)total_sets * cta / pl.grid);
        const uint32_t t_end = (uint32_t)((uint64_t)total_sets * (cta + 1) / pl.grid);
        for (uint32_t sg = 0; t < t_end;) {
            while (sg + 1 < op.nw && t >= a.seg_t0[sg + 1]) sg++;
            const uint32_t T = std::min(t_end, a.seg_t0[sg + 1]) - t;
            a.groups += (T + rps - 1) / rps;
            t += T;
        }
    }
    a.tab_off = HDR_BYTES + nst * stage;
    pl.smem = HDR_BYTES + (size_t)nst * stage + act_bytes;
    pl.kl = kl; pl.swiglu = sw; pl.stage = stage;
    pl.mma = false; pl.ksplit = 1; pl.ctas_per_sm = per_sm;
    pl.args = a;
    return ALICE_OK;
}

namespace {

template <int CODE>
int launch_mma_table_code(const float* x, uint32_t cols, uint8_t* blob, uint32_t tsum_blocks, const LaunchCfg& cfg) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((cols + MMA_PREP_ELEMS - 1) / MMA_PREP_ELEMS);
    lc.blockDim = dim3(NCW * 32);
    lc.stream = cfg.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, mma_table_kernel<CODE>, x, cols, blob, tsum_blocks) == cudaSuccess ? ALICE_OK : ALICE_E_CUDA;
}
int launch_mma_table(WeightFormat f, const float* x, uint32_t cols, uint8_t* blob, const LaunchCfg& cfg) {
    switch (f) {
        case WF_Q1_0: return launch_mma_table_code<0>(x, cols, blob, cols / 128, cfg);
        case WF_TERNARY: return launch_mma_table_code<0>(x, cols, blob, 0, cfg);
        case WF_Q2_0: return launch_mma_table_code<1>(x, cols, blob, cols / 128, cfg);
        default: return launch_mma_table_code<2>(x, cols, blob, 0, cfg);
    }
}

// One launch (or, for a bit-plane matvec whose rows are too wide for shared memory, one launch per column chunk)
// for ONE input vector.
int launch_single(const GemvOp& op, const LaunchCfg& cfg) {
    StreamPlan pl;
    const int prc = plan_stream_gemv(op, cfg, pl);
    if (prc) return prc;
    const StreamArgs& a = pl.args;
    const WeightDesc& w0 = *op.w[0];
    if (pl.mma) {
        // one launch per column chunk; a later chunk adds to what the earlier ones left in y, and only the last one
        // sees the final values (argmax epilogue, rows pushed to peers, hand-over to the next op)
        size_t prep_off = 0;
        for (uint32_t c = 0; c < pl.ksplit; c++) {
            StreamPlan pc = pl;
            if (pl.ksplit > 1) {
                uint32_t lo, n;
                mma_chunk(w0, pl.ksplit, c, lo, n);
                StreamArgs base = pl.args;
                base.x = op.x; base.cols = w0.cols; base.row_bytes = w0.row_bytes;
                const int rc = plan_mma(op, cfg, base, lo, n, pc);
                if (rc) return rc;
                if (c > 0) pc.args.resid = op.y;
                if (c + 1 < pl.ksplit) { pc.args.argmax_key = nullptr; pc.args.npeers = 0; }
            }
            // the activation digit table of this (chunk of the) vector, prepared once ahead of the matvec
            const uint32_t ge = (w0.fmt == WF_Q2_0 || w0.fmt == WF_SPARSE_TERNARY) ? 64u : 128u;
            const uint32_t blob = (mma_blob_bytes((pc.args.cols + ge - 1) / ge) + 127u) & ~127u;
            if (op.prep && prep_off + blob <= op.prep_bytes && ((uintptr_t)op.prep & 15) == 0) {
                uint8_t* dst = static_cast<uint8_t*>(op.prep) + prep_off;
                prep_off += blob;
                const int trc = launch_mma_table(w0.fmt, pc.args.x, pc.args.cols, dst, cfg);
                if (trc) return trc;
                pc.args.tab_global = dst;
            }
            const int rc = w0.fmt == WF_Q1_0 ? launch_mma<MmaQ1_0>(pc, cfg) : w0.fmt == WF_Q2_0 ? launch_mma<MmaQ2_0>(pc, cfg)
                         : w0.fmt == WF_TERNARY ? launch_mma<MmaTernary>(pc, cfg) : launch_mma<MmaSparseTernary>(pc, cfg);
            if (rc) return rc;
        }
        return ALICE_OK;
    }
    const uint32_t kl = pl.kl, grid = pl.grid;
    const bool sw = pl.swiglu;
    const size_t smem = pl.smem;
    switch (w0.fmt) {
        case WF_Q4_K: return launch_fmt<FmtQ4K>(a, kl, sw, grid, smem, cfg);
        case WF_Q5_K: return launch_fmt<FmtQ5K>(a, kl, sw, grid, smem, cfg);
        case WF_Q6_K: return launch_fmt<FmtQ6K>(a, kl, sw, grid, smem, cfg);
        case WF_Q8_0: return launch_fmt<FmtQ8_0>(a, kl, sw, grid, smem, cfg);
        case WF_Q1_0: return launch_fmt<FmtQ1_0>(a, kl, sw, grid, smem, cfg);
        case WF_Q2_0: return launch_fmt<FmtQ2_0>(a, kl, sw, grid, smem, cfg);
        case WF_TERNARY: return launch_fmt<FmtTernary>(a, kl, sw, grid, smem, cfg);
        case WF_SPARSE_TERNARY: return launch_fmt<FmtSparseTernary>(a, kl, sw, grid, smem, cfg);
        default: return ALICE_E_UNSUPPORTED;
    }
}

}  // namespace

int launch_stream_gemv_op(const GemvOp& op, const LaunchCfg& cfg) {
    if (op.batch == 0 || op.batch > (uint32_t)MAX_BATCH) return ALICE_E_SHAPE;
    if (op.batch == 1) return launch_single(op, cfg);
    if (op.argmax_key) return ALICE_E_INVALID;
    {   // K-quants with prepared Q8_K input: the int8 tensor-core kernel serves the whole batch in one pass over the weights
        const int brc = launch_kq_batch(op, cfg, false, nullptr);
        if (brc != ALICE_E_SHAPE) return brc;
    }
    // Formats without a batch kernel: one launch per input vector (the weights stream once per vector).
    if (!op.w[0]) return ALICE_E_INVALID;
    uint32_t total_rows = 0;
    for (uint32_t i = 0; i < op.nw && i < 3; i++) if (op.w[i]) total_rows += op.w[i]->rows;
    const uint32_t ys = op.y_stride ? op.y_stride : total_rows;
    const uint32_t cols = op.w[0]->cols, nb = cols / QK_K;
    for (uint32_t k = 0; k < op.batch; k++) {
        GemvOp o = op;
        o.batch = 1;
        Q8KView v;
        if (op.q8) { v = *op.q8; v.qs += (size_t)k * cols; v.d += (size_t)k * nb; v.bsums += (size_t)k * nb * 16; o.q8 = &v; }
        if (op.x) o.x = op.x + (size_t)k * cols;
        o.y = op.y + (size_t)k * ys;
        if (op.resid) o.resid = op.resid + (size_t)k * ys;
        for (uint32_t p = 0; p < op.npeers && p < MAX_PEERS; p++) o.peer_y[p] = op.peer_y[p] + (size_t)k * ys;
        const int rc = launch_single(o, cfg);
        if (rc) return rc;
    }
    return ALICE_OK;
}

size_t mma_prep_bytes(uint32_t cols) {
    // the finest grouping (64 elements per group) and the slack of up to four column chunks, each with its own
    // zero record, sums and unit, rounded to 128 bytes
    return ((size_t)mma_blob_bytes((cols + 63) / 64) + 1024 + 255) & ~size_t(255);
}

int batch_plan(const GemvOp& op, const LaunchCfg& cfg, uint32_t* launches, uint32_t* weight_passes) {
    uint32_t n = 0;
    if (op.batch > 1 && launch_kq_batch(op, cfg, true, &n) == ALICE_OK) { *launches = n; *weight_passes = 1; return ALICE_OK; }
    GemvOp one = op; one.batch = 1;
    StreamPlan pl;
    const int rc = plan_stream_gemv(one, cfg, pl);
    if (rc) return rc;
    *launches = op.batch * pl.ksplit; *weight_passes = op.batch;
    return ALICE_OK;
}

// ---- stand-alone hand-over kernel ----------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(256) publish_vector_kernel(const __grid_constant__ Publish p, int* status) {
    __shared__ double red[8];
    __shared__ int ok;
    pdl_launch_dependents();
    pdl_wait();
    if (p.npeers) {
        if (threadIdx.x == 0) ok = publish_peer_gate(p, status) ? 1 : 0;
        __syncthreads();
        if (!ok) return;
    }
    if (p.dst.qs != nullptr || p.dst.xn != nullptr) publish_vector<8, 1>(p, red, true);
}
}  // namespace

cudaError_t launch_publish_vector(const Publish& p, int* status, cudaStream_t stream, bool pdl) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(1);
    lc.blockDim = dim3(256);
    lc.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, publish_vector_kernel, p, status);
}

}  // namespace alice
