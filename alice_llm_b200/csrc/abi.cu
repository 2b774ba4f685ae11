// extern "C" surface of the library (include/alice_cuda.h): handles, uploads, dispatch.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "abi_internal.cuh"
#include "gemv_plan.cuh"
#include "tp.cuh"

using namespace alice;

namespace {

__device__ __forceinline__ void pdl_wait_abi() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

int cuda_fail(cudaError_t err, const char* what) {
    return fail(err == cudaErrorMemoryAllocation ? ALICE_E_NOMEM : ALICE_E_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

#define CU(call)                                               \
    do {                                                       \
        cudaError_t err__ = (call);                            \
        if (err__ != cudaSuccess) return cuda_fail(err__, #call); \
    } while (0)

bool known_ggml(uint32_t t) { return ggml_block_bytes((WeightFormat)t) != 0; }

LaunchCfg cfg_of(const alice_engine* e) { return alice_cfg_of(e); }

}  // namespace

void alice_engine_retain(alice_engine* e) { e->refs++; }
void alice_engine_release(alice_engine* e) {
    if (--e->refs == 0) delete e;
}
// Before a handle frees device memory the engine's queued work must be done - unless the engine is already gone
// (its destroy synchronised the stream).
static void quiesce(alice_engine* e) {
    cudaSetDevice(e->device);
    if (!e->dead) cudaStreamSynchronize(e->stream);
}

LaunchCfg alice_cfg_of(const alice_engine* e) {
    LaunchCfg c;
    c.stream = e->stream; c.num_sms = e->num_sms; c.status = e->status; c.pdl = e->pdl;
    c.force_rps = e->force_rps; c.force_stages = e->force_stages;
    return c;
}

int alice_fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}
int alice_cuda_fail(cudaError_t err, const char* what) { return cuda_fail(err, what); }

namespace {

Q8KView view_of(const alice_q8k* q, uint32_t k) {
    auto* p = static_cast<uint8_t*>(q->base);
    Q8KView v;
    v.qs = reinterpret_cast<const int8_t*>(p + q->lay.qs_off) + (size_t)k * q->nb * 256;
    v.d = reinterpret_cast<const float*>(p + q->lay.d_off) + (size_t)k * q->nb;
    v.bsums = reinterpret_cast<const int16_t*>(p + q->lay.bsums_off) + (size_t)k * q->nb * 16;
    v.nb = q->nb;
    return v;
}

// Engine scratch grows on demand and is reused by later calls on the same stream.
int ensure_scratch(alice_engine* e, size_t bytes) {
    if (bytes <= e->scratch_bytes) return ALICE_OK;
    CU(cudaStreamSynchronize(e->stream));
    if (e->scratch) CU(cudaFree(e->scratch));
    e->scratch = nullptr; e->scratch_bytes = 0;
    CU(cudaMalloc(&e->scratch, bytes));
    e->scratch_bytes = bytes;
    return ALICE_OK;
}

int ensure_prep(alice_engine* e, size_t bytes) {
    if (bytes <= e->prep_bytes) return ALICE_OK;
    CU(cudaStreamSynchronize(e->stream));
    if (e->prep) CU(cudaFree(e->prep));
    e->prep = nullptr; e->prep_bytes = 0;
    CU(cudaMalloc(&e->prep, bytes));
    e->prep_bytes = bytes;
    return ALICE_OK;
}

int launch_rc(int rc, const char* what) {
    if (rc == ALICE_OK) return rc;
    if (rc == ALICE_E_CUDA) return fail(rc, "%s: launch failed: %s", what, cudaGetErrorString(cudaGetLastError()));
    if (rc == ALICE_E_SHAPE) return fail(rc, "%s: shape not supported by the streaming kernel", what);
    return fail(rc, "%s: error %d", what, rc);
}

}  // namespace

extern "C" {

const char* alice_last_error(void) { return g_err.c_str(); }

uint32_t alice_type_block_bytes(uint32_t t) { return ggml_block_bytes((WeightFormat)t); }
uint32_t alice_type_block_elems(uint32_t t) { return ggml_block_elems((WeightFormat)t); }

int32_t alice_engine_create(int32_t device, alice_engine** out) {
    if (!out) return fail(ALICE_E_INVALID, "alice_engine_create: out is null");
    *out = nullptr;
    int n = 0;
    cudaError_t err = cudaGetDeviceCount(&n);
    if (err != cudaSuccess || n == 0)
        return fail(ALICE_E_CUDA, "alice_engine_create: no CUDA device (%s); this library has no CPU path",
                    cudaGetErrorString(err));
    if (device < 0 || device >= n) return fail(ALICE_E_INVALID, "alice_engine_create: device %d of %d", device, n);
    CU(cudaSetDevice(device));
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return fail(ALICE_E_UNSUPPORTED, "alice_engine_create: device is sm_%d%d; kernels are built for sm_100a",
                    prop.major, prop.minor);
    auto* e = new (std::nothrow) alice_engine();
    if (!e) return fail(ALICE_E_NOMEM, "alice_engine_create: host allocation failed");
    e->device = device;
    e->num_sms = prop.multiProcessorCount;
    err = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking);
    if (err != cudaSuccess) { delete e; return cuda_fail(err, "cudaStreamCreate"); }
    e->own_stream = true;
    err = cudaMalloc(&e->status, sizeof(int));
    if (err == cudaSuccess) err = cudaMemset(e->status, 0, sizeof(int));
    if (err == cudaSuccess) err = cudaMallocHost(reinterpret_cast<void**>(&e->status_host), sizeof(int));
    if (err != cudaSuccess) {
        if (e->status) cudaFree(e->status);
        if (e->status_host) cudaFreeHost(e->status_host);
        cudaStreamDestroy(e->stream); delete e;
        return cuda_fail(err, "status word");
    }
    *out = e;
    return ALICE_OK;
}

int32_t alice_engine_destroy(alice_engine* e) {
    if (!e || e->dead) return ALICE_OK;
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->stream);
    alice::tp_release(e);
    if (e->scratch) cudaFree(e->scratch);
    if (e->prep) cudaFree(e->prep);
    if (e->status) cudaFree(e->status);
    if (e->status_host) cudaFreeHost(e->status_host);
    if (e->own_stream) cudaStreamDestroy(e->stream);
    e->scratch = e->prep = nullptr; e->status = nullptr; e->status_host = nullptr; e->stream = nullptr;
    e->dead = true;               // handles created on this engine may outlive it: they only free their own memory
    alice_engine_release(e);
    return ALICE_OK;
}

int32_t alice_engine_set_stream(alice_engine* e, void* s) {
    if (!e) return fail(ALICE_E_INVALID, "alice_engine_set_stream: null engine");
    CU(cudaStreamSynchronize(e->stream));
    if (e->own_stream) { cudaStreamDestroy(e->stream); e->own_stream = false; }
    e->stream = static_cast<cudaStream_t>(s);
    return ALICE_OK;
}

int32_t alice_engine_set_pdl(alice_engine* e, int32_t on) {
    if (!e) return fail(ALICE_E_INVALID, "alice_engine_set_pdl: null engine");
    e->pdl = on != 0;
    return ALICE_OK;
}

int32_t alice_engine_set_tuning(alice_engine* e, int32_t rps, int32_t stages) {
    if (!e) return fail(ALICE_E_INVALID, "alice_engine_set_tuning: null engine");
    e->force_rps = rps; e->force_stages = stages;
    return ALICE_OK;
}

int32_t alice_engine_set_wait_limit(alice_engine* e, uint64_t sm_cycles) {
    if (!e) return fail(ALICE_E_INVALID, "alice_engine_set_wait_limit: null engine");
    e->wait_limit = (long long)std::min<uint64_t>(sm_cycles, (uint64_t)1 << 40);
    return ALICE_OK;
}

int32_t alice_sync(alice_engine* e) {
    if (!e) return fail(ALICE_E_INVALID, "alice_sync: null engine");
    CU(cudaSetDevice(e->device));
    // the status word rides the same wait: its copy to pinned host memory is queued behind the work
    CU(cudaMemcpyAsync(e->status_host, e->status, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    const int st = *e->status_host;
    if (st != 0) {
        cudaMemset(e->status, 0, sizeof(int));
        static const char* const what[] = {"?", "unspecified wait", "weights did not land in shared memory", "partial sums of a row", "stage release",
                                           "grid barrier", "rows from a tensor-parallel peer"};
        const int code = st & 0xff;
        return fail(ALICE_E_KERNEL, "alice_sync: a kernel wait ran out of its cycle budget (status %d: %s); results of the queued work are void",
                    st, code >= 1 && code <= 6 ? what[code] : what[0]);
    }
    return ALICE_OK;
}

int32_t alice_debug_expire_wait(alice_engine* e) {
    if (!e) return fail(ALICE_E_INVALID, "alice_debug_expire_wait: null engine");
    CU(cudaSetDevice(e->device));
    // scratch: [256 floats source][epoch u32][own flag u32][peer flag u32], all zero: the gate expects
    // (epoch + 1) * 1 = 1 at the own flag, which nothing raises
    int rc = ensure_scratch(e, 4096);
    if (rc) return rc;
    CU(cudaMemsetAsync(e->scratch, 0, 4096, e->stream));
    auto* base = static_cast<uint8_t*>(e->scratch);
    Publish p{};
    p.mode = PUB_VECTOR; p.n = 256; p.batch = 1; p.src = reinterpret_cast<const float*>(base);
    p.npeers = 1;
    p.epoch = reinterpret_cast<const unsigned int*>(base + 1024);
    p.wait_flag = reinterpret_cast<const unsigned int*>(base + 1028);
    p.peer_flag[0] = reinterpret_cast<unsigned int*>(base + 1032);
    p.wait_limit = e->wait_limit;
    CU(launch_publish_vector(p, e->status, e->stream, e->pdl));
    return ALICE_OK;
}

// ---- weights -------------------------------------------------------------------------------

static int make_ggml_desc(const char* who, size_t nbytes, uint32_t type, uint32_t rows, uint32_t cols, WeightDesc& d) {
    if (!known_ggml(type)) return fail(ALICE_E_UNSUPPORTED, "%s: unsupported quantization type %u", who, type);
    const uint32_t rb = ggml_row_bytes((WeightFormat)type, cols);
    if (rows == 0 || rb == 0)
        return fail(ALICE_E_SHAPE, "%s: cols %u is not a whole number of %u-element blocks (rows %u)", who, cols,
                    ggml_block_elems((WeightFormat)type), rows);
    if ((size_t)rows * rb != nbytes)
        return fail(ALICE_E_SHAPE, "%s: %zu bytes given, %u x %u needs %zu", who, nbytes, rows, cols, (size_t)rows * rb);
    d = WeightDesc{};
    d.fmt = (WeightFormat)type; d.rows = rows; d.cols = cols; d.row_bytes = rb;
    return ALICE_OK;
}

int32_t alice_upload_weights(alice_engine* e, const uint8_t* data, size_t nbytes, uint32_t type, uint32_t rows,
                             uint32_t cols, alice_weights** out) {
    if (!e || !data || !out) return fail(ALICE_E_INVALID, "alice_upload_weights: null argument");
    WeightDesc d;
    int rc = make_ggml_desc("alice_upload_weights", nbytes, type, rows, cols, d);
    if (rc) return rc;
    CU(cudaSetDevice(e->device));
    void* p = nullptr;
    CU(cudaMalloc(&p, nbytes + 64));  // tail slack: bulk copies round their end up to 16 bytes
    cudaError_t err = cudaMemcpyAsync(p, data, nbytes, cudaMemcpyHostToDevice, e->stream);
    if (err == cudaSuccess) err = cudaMemsetAsync(static_cast<uint8_t*>(p) + nbytes, 0, 64, e->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);  // the host slice is only borrowed
    if (err != cudaSuccess) { cudaFree(p); return cuda_fail(err, "alice_upload_weights copy"); }
    d.data = static_cast<const uint8_t*>(p);
    *out = new alice_weights{e, d, p, nullptr};
    alice_engine_retain(e);
    return ALICE_OK;
}

int32_t alice_weights_from_device(alice_engine* e, const void* dptr, size_t nbytes, uint32_t type, uint32_t rows,
                                  uint32_t cols, alice_weights** out) {
    if (!e || !dptr || !out) return fail(ALICE_E_INVALID, "alice_weights_from_device: null argument");
    if ((uintptr_t)dptr & 15) return fail(ALICE_E_INVALID, "alice_weights_from_device: pointer not 16-byte aligned");
    WeightDesc d;
    int rc = make_ggml_desc("alice_weights_from_device", nbytes, type, rows, cols, d);
    if (rc) return rc;
    if (nbytes & 15)
        return fail(ALICE_E_SHAPE, "alice_weights_from_device: byte size %zu must be a multiple of 16", nbytes);
    d.data = static_cast<const uint8_t*>(dptr);
    *out = new alice_weights{e, d, nullptr, nullptr};
    alice_engine_retain(e);
    return ALICE_OK;
}

static int upload_rows_and_scales(alice_engine* e, const std::vector<uint8_t>& host, const float* scales,
                                  WeightDesc d, alice_weights** out) {
    CU(cudaSetDevice(e->device));
    void* p = nullptr;
    void* s = nullptr;
    CU(cudaMalloc(&p, host.size() + 64));
    cudaError_t err = cudaMalloc(&s, (size_t)d.rows * sizeof(float));
    if (err == cudaSuccess) err = cudaMemcpyAsync(p, host.data(), host.size(), cudaMemcpyHostToDevice, e->stream);
    if (err == cudaSuccess) err = cudaMemsetAsync(static_cast<uint8_t*>(p) + host.size(), 0, 64, e->stream);
    if (err == cudaSuccess) err = cudaMemcpyAsync(s, scales, (size_t)d.rows * sizeof(float), cudaMemcpyHostToDevice, e->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);
    if (err != cudaSuccess) { cudaFree(p); if (s) cudaFree(s); return cuda_fail(err, "ternary upload"); }
    d.data = static_cast<const uint8_t*>(p);
    d.scales = static_cast<const float*>(s);
    *out = new alice_weights{e, d, p, s};
    alice_engine_retain(e);
    return ALICE_OK;
}

int32_t alice_upload_ternary(alice_engine* e, const uint8_t* pos, const uint8_t* neg, const float* scales,
                             uint32_t rows, uint32_t cols, alice_weights** out) {
    if (!e || !pos || !neg || !scales || !out) return fail(ALICE_E_INVALID, "alice_upload_ternary: null argument");
    if (rows == 0 || cols == 0) return fail(ALICE_E_SHAPE, "alice_upload_ternary: empty matrix");
    // device row = [pos plane | neg plane]; planes padded with zero bits to a whole number of 32-bit words
    const uint32_t src_pb = (cols + 7) / 8, pb = ((cols + 31) / 32) * 4;
    std::vector<uint8_t> host((size_t)rows * 2 * pb, 0);
    const uint8_t tail_mask = (cols % 8) ? (uint8_t)((1u << (cols % 8)) - 1) : 0xFF;
    for (uint32_t r = 0; r < rows; r++) {
        uint8_t* dp = host.data() + (size_t)r * 2 * pb;
        memcpy(dp, pos + (size_t)r * src_pb, src_pb);
        memcpy(dp + pb, neg + (size_t)r * src_pb, src_pb);
        dp[src_pb - 1] &= tail_mask;       // bits past num_cols are never read by the reference
        dp[pb + src_pb - 1] &= tail_mask;
    }
    WeightDesc d = {};
    d.fmt = WF_TERNARY; d.rows = rows; d.cols = cols; d.row_bytes = 2 * pb;
    return upload_rows_and_scales(e, host, scales, d, out);
}

int32_t alice_ternary_from_device(alice_engine* e, const void* rows_dptr, const float* scales_dptr, uint32_t rows,
                                  uint32_t cols, alice_weights** out) {
    if (!e || !rows_dptr || !scales_dptr || !out) return fail(ALICE_E_INVALID, "alice_ternary_from_device: null argument");
    if (rows == 0 || cols == 0) return fail(ALICE_E_SHAPE, "alice_ternary_from_device: empty matrix");
    if ((uintptr_t)rows_dptr & 15) return fail(ALICE_E_INVALID, "alice_ternary_from_device: pointer not 16-byte aligned");
    const uint32_t pb = ((cols + 31) / 32) * 4;
    if (((size_t)rows * 2 * pb) & 15)
        return fail(ALICE_E_SHAPE, "alice_ternary_from_device: rows * row bytes (%zu) must be a multiple of 16", (size_t)rows * 2 * pb);
    WeightDesc d = {};
    d.fmt = WF_TERNARY; d.rows = rows; d.cols = cols; d.row_bytes = 2 * pb;
    d.data = static_cast<const uint8_t*>(rows_dptr);
    d.scales = scales_dptr;
    *out = new alice_weights{e, d, nullptr, nullptr};
    alice_engine_retain(e);
    return ALICE_OK;
}

int32_t alice_upload_sparse_ternary(alice_engine* e, const uint8_t* packed, const float* scales, uint32_t rows,
                                    uint32_t cols, alice_weights** out) {
    if (!e || !packed || !scales || !out) return fail(ALICE_E_INVALID, "alice_upload_sparse_ternary: null argument");
    if (rows == 0 || cols == 0) return fail(ALICE_E_SHAPE, "alice_upload_sparse_ternary: empty matrix");
    const uint32_t rb = ((cols + 15) / 16) * 4;
    std::vector<uint8_t> host(packed, packed + (size_t)rows * rb);
    WeightDesc d = {};
    d.fmt = WF_SPARSE_TERNARY; d.rows = rows; d.cols = cols; d.row_bytes = rb;
    return upload_rows_and_scales(e, host, scales, d, out);
}

int32_t alice_weights_free(alice_weights* w) {
    if (!w) return ALICE_OK;
    if (w->owned_data || w->owned_scales) quiesce(w->e);
    if (w->owned_data) cudaFree(w->owned_data);
    if (w->owned_scales) cudaFree(w->owned_scales);
    alice_engine_release(w->e);
    delete w;
    return ALICE_OK;
}

// ---- f32 buffers ---------------------------------------------------------------------------

int32_t alice_buf_alloc_f32(alice_engine* e, size_t len, alice_buf** out) {
    if (!e || !out) return fail(ALICE_E_INVALID, "alice_buf_alloc_f32: null argument");
    CU(cudaSetDevice(e->device));
    void* p = nullptr;
    CU(cudaMalloc(&p, std::max<size_t>(len, 1) * sizeof(float)));
    cudaError_t err = cudaMemsetAsync(p, 0, std::max<size_t>(len, 1) * sizeof(float), e->stream);
    if (err != cudaSuccess) { cudaFree(p); return cuda_fail(err, "alice_buf_alloc_f32 memset"); }
    *out = new alice_buf{e, static_cast<float*>(p), len, true};
    alice_engine_retain(e);
    return ALICE_OK;
}

int32_t alice_buf_write_f32(alice_engine* e, alice_buf* b, const float* data, size_t len) {
    if (!e || !b || (!data && len)) return fail(ALICE_E_INVALID, "alice_buf_write_f32: null argument");
    if (len > b->len) return fail(ALICE_E_SHAPE, "alice_buf_write_f32: %zu floats into a buffer of %zu", len, b->len);
    CU(cudaMemcpyAsync(b->p, data, len * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));  // the host slice is only borrowed for the call
    return ALICE_OK;
}

int32_t alice_buf_write_f32_async(alice_engine* e, alice_buf* b, const float* data, size_t len) {
    if (!e || !b || (!data && len)) return fail(ALICE_E_INVALID, "alice_buf_write_f32_async: null argument");
    if (len > b->len) return fail(ALICE_E_SHAPE, "alice_buf_write_f32_async: %zu floats into a buffer of %zu", len, b->len);
    CU(cudaMemcpyAsync(b->p, data, len * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    return ALICE_OK;
}

int32_t alice_buf_read_f32_async(alice_engine* e, const alice_buf* b, float* out, size_t len) {
    if (!e || !b || (!out && len)) return fail(ALICE_E_INVALID, "alice_buf_read_f32_async: null argument");
    if (len > b->len) return fail(ALICE_E_SHAPE, "alice_buf_read_f32_async: %zu floats from a buffer of %zu", len, b->len);
    CU(cudaMemcpyAsync(out, b->p, len * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
    return ALICE_OK;
}

int32_t alice_buf_upload_f32(alice_engine* e, const float* data, size_t len, alice_buf** out) {
    int rc = alice_buf_alloc_f32(e, len, out);
    if (rc) return rc;
    rc = alice_buf_write_f32(e, *out, data, len);
    if (rc) { alice_buf_free(*out); *out = nullptr; }
    return rc;
}

int32_t alice_buf_read_f32(alice_engine* e, const alice_buf* b, float* out, size_t len) {
    if (!e || !b || (!out && len)) return fail(ALICE_E_INVALID, "alice_buf_read_f32: null argument");
    if (len > b->len) return fail(ALICE_E_SHAPE, "alice_buf_read_f32: %zu floats from a buffer of %zu", len, b->len);
    CU(cudaMemcpyAsync(out, b->p, len * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    return ALICE_OK;
}

int32_t alice_buf_from_device(alice_engine* e, void* dptr, size_t len, alice_buf** out) {
    if (!e || !dptr || !out) return fail(ALICE_E_INVALID, "alice_buf_from_device: null argument");
    if ((uintptr_t)dptr & 15) return fail(ALICE_E_INVALID, "alice_buf_from_device: pointer not 16-byte aligned");
    *out = new alice_buf{e, static_cast<float*>(dptr), len, false};
    alice_engine_retain(e);
    return ALICE_OK;
}

int32_t alice_buf_free(alice_buf* b) {
    if (!b) return ALICE_OK;
    if (b->owned) {
        quiesce(b->e);
        cudaFree(b->p);
    }
    alice_engine_release(b->e);
    delete b;
    return ALICE_OK;
}

// ---- Q8_K activations ----------------------------------------------------------------------

int32_t alice_q8k_alloc(alice_engine* e, uint32_t cols, uint32_t batch, alice_q8k** out) {
    if (!e || !out) return fail(ALICE_E_INVALID, "alice_q8k_alloc: null argument");
    if (cols == 0 || cols % 256 != 0) return fail(ALICE_E_SHAPE, "alice_q8k_alloc: cols %u is not a multiple of 256", cols);
    if (batch == 0) return fail(ALICE_E_SHAPE, "alice_q8k_alloc: batch 0");
    CU(cudaSetDevice(e->device));
    auto* q = new alice_q8k{e, nullptr, cols, batch, cols / 256, Q8KLayout::make(cols / 256, batch)};
    cudaError_t err = cudaMalloc(&q->base, q->lay.total);
    if (err != cudaSuccess) { delete q; return cuda_fail(err, "alice_q8k_alloc"); }
    alice_engine_retain(e);
    *out = q;
    return ALICE_OK;
}

int32_t alice_quantize_q8k(alice_engine* e, const alice_buf* x, alice_q8k* q) {
    if (!e || !x || !q) return fail(ALICE_E_INVALID, "alice_quantize_q8k: null argument");
    if (x->len < (size_t)q->cols * q->batch)
        return fail(ALICE_E_SHAPE, "alice_quantize_q8k: input has %zu floats, need %zu", x->len, (size_t)q->cols * q->batch);
    launch_quantize_q8k(x->p, q->cols, q->batch, q->base, e->stream, e->pdl);
    CU(cudaGetLastError());
    return ALICE_OK;
}

int32_t alice_q8k_read(alice_engine* e, const alice_q8k* q, float* d, int8_t* qs, int16_t* bsums) {
    if (!e || !q || !d || !qs || !bsums) return fail(ALICE_E_INVALID, "alice_q8k_read: null argument");
    const size_t n = (size_t)q->batch * q->nb;
    auto* p = static_cast<const uint8_t*>(q->base);
    CU(cudaMemcpyAsync(qs, p + q->lay.qs_off, n * 256, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaMemcpyAsync(d, p + q->lay.d_off, n * 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaMemcpyAsync(bsums, p + q->lay.bsums_off, n * 32, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    return ALICE_OK;
}

int32_t alice_q8k_upload(alice_engine* e, const float* d, const int8_t* qs, const int16_t* bsums, uint32_t cols,
                         uint32_t batch, alice_q8k** out) {
    if (!d || !qs || !bsums) return fail(ALICE_E_INVALID, "alice_q8k_upload: null argument");
    int rc = alice_q8k_alloc(e, cols, batch, out);
    if (rc) return rc;
    alice_q8k* q = *out;
    const size_t n = (size_t)batch * q->nb;
    auto* p = static_cast<uint8_t*>(q->base);
    cudaError_t err = cudaMemcpyAsync(p + q->lay.qs_off, qs, n * 256, cudaMemcpyHostToDevice, e->stream);
    if (err == cudaSuccess) err = cudaMemcpyAsync(p + q->lay.d_off, d, n * 4, cudaMemcpyHostToDevice, e->stream);
    if (err == cudaSuccess) err = cudaMemcpyAsync(p + q->lay.bsums_off, bsums, n * 32, cudaMemcpyHostToDevice, e->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);
    if (err != cudaSuccess) { alice_q8k_free(q); *out = nullptr; return cuda_fail(err, "alice_q8k_upload"); }
    return ALICE_OK;
}

int32_t alice_q8k_free(alice_q8k* q) {
    if (!q) return ALICE_OK;
    quiesce(q->e);
    cudaFree(q->base);
    alice_engine_release(q->e);
    delete q;
    return ALICE_OK;
}

// ---- the hot path --------------------------------------------------------------------------

Q8KView view_at(void* base, uint32_t nb, uint32_t batch) {
    const Q8KLayout l = Q8KLayout::make(nb, batch);
    auto* p = static_cast<uint8_t*>(base);
    Q8KView v;
    v.qs = reinterpret_cast<const int8_t*>(p + l.qs_off);
    v.d = reinterpret_cast<const float*>(p + l.d_off);
    v.bsums = reinterpret_cast<const int16_t*>(p + l.bsums_off);
    v.nb = nb;
    return v;
}

// One matvec / fused SwiGLU over `batch` prepared input vectors.
static int run_gemv(alice_engine* e, const alice_weights* w0, const alice_weights* w1, const Q8KView* q8, const float* xf,
                    float* y, uint32_t batch, const char* who, bool may_alloc = true) {
    GemvOp op;
    const WeightFormat f = w0->d.fmt;
    if (f == WF_Q1_0 || f == WF_Q2_0 || f == WF_TERNARY || f == WF_SPARSE_TERNARY) {
        // room for the activation digit table, prepared once ahead of the matvec (csrc/gemv_mma.cuh)
        if (may_alloc) { const int rc = ensure_prep(e, mma_prep_bytes(w0->d.cols)); if (rc) return rc; }
        op.prep = e->prep; op.prep_bytes = e->prep_bytes;
    }
    op.w[0] = &w0->d; op.up = w1 ? &w1->d : nullptr;
    op.q8 = q8; op.x = xf; op.y = y; op.batch = batch;
    op.wait_limit = e->wait_limit;
    return launch_rc(launch_stream_gemv_op(op, cfg_of(e)), who);
}

static int check_pair(const alice_weights* g, const alice_weights* u, const char* who) {
    if (g->d.fmt != u->d.fmt || g->d.rows != u->d.rows || g->d.cols != u->d.cols)
        return fail(ALICE_E_SHAPE, "%s: gate and up differ in format or shape", who);
    return ALICE_OK;
}

// f32 input of a matvec. K-quant weights want it as Q8_K blocks (q4k_matvec = quantize_row_q8_k + q4k_matvec_preq,
// src/gguf.rs:3600-3603): a small quantizer kernel runs ahead of the matvec, which is launched as its programmatic
// dependent - its CTAs become resident and stream weights while the blocks are being written. (Measured on the FFN
// block at 8B shapes: 31.6 us per block this way, 35.5 us with the quantization done inside the matvec kernels.)
static int matvec_common(alice_engine* e, const alice_weights* w0, const alice_weights* w1, const alice_buf* x,
                         alice_buf* y, uint32_t batch, const char* who) {
    if (!e || !w0 || !x || !y) return fail(ALICE_E_INVALID, "%s: null argument", who);
    if (batch == 0 || batch > 8) return fail(ALICE_E_SHAPE, "%s: batch %u outside 1..8", who, batch);
    if (w1) { int rc = check_pair(w0, w1, who); if (rc) return rc; }
    const WeightDesc& d = w0->d;
    if (x->len < (size_t)batch * d.cols) return fail(ALICE_E_SHAPE, "%s: input has %zu floats, need %zu", who, x->len, (size_t)batch * d.cols);
    if (y->len < (size_t)batch * d.rows) return fail(ALICE_E_SHAPE, "%s: output has %zu floats, need %zu", who, y->len, (size_t)batch * d.rows);
    CU(cudaSetDevice(e->device));
    if (!format_uses_q8k(d.fmt)) return run_gemv(e, w0, w1, nullptr, x->p, y->p, batch, who);
    if ((uintptr_t)x->p & 15) return fail(ALICE_E_INVALID, "%s: input vector must be 16-byte aligned", who);
    const uint32_t nb = d.cols / 256;
    int rc = ensure_scratch(e, Q8KLayout::make(nb, batch).total);
    if (rc) return rc;
    launch_quantize_q8k(x->p, d.cols, batch, e->scratch, e->stream, e->pdl);
    CU(cudaGetLastError());
    const Q8KView v = view_at(e->scratch, nb, batch);
    return run_gemv(e, w0, w1, &v, nullptr, y->p, batch, who);
}

static int preq_common(alice_engine* e, const alice_weights* w0, const alice_weights* w1, const alice_q8k* q,
                       alice_buf* y, const char* who) {
    if (!e || !w0 || !q || !y) return fail(ALICE_E_INVALID, "%s: null argument", who);
    if (w1) { int rc = check_pair(w0, w1, who); if (rc) return rc; }
    const WeightDesc& d = w0->d;
    if (q->cols != d.cols) return fail(ALICE_E_SHAPE, "%s: Q8_K input has %u columns, weights %u", who, q->cols, d.cols);
    if (q->batch > 8) return fail(ALICE_E_SHAPE, "%s: batch %u outside 1..8", who, q->batch);
    if (y->len < (size_t)q->batch * d.rows) return fail(ALICE_E_SHAPE, "%s: output too small", who);
    CU(cudaSetDevice(e->device));
    if (format_uses_q8k(d.fmt)) {
        const Q8KView v = view_of(q, 0);
        return run_gemv(e, w0, w1, &v, nullptr, y->p, q->batch, who);
    }
    if (d.fmt == WF_Q1_0 || d.fmt == WF_Q2_0) {
        const size_t total = (size_t)q->batch * d.cols;
        int rc = ensure_scratch(e, total * sizeof(float));
        if (rc) return rc;
        launch_q8k_to_f32(view_of(q, 0), total, static_cast<float*>(e->scratch), e->stream);
        return run_gemv(e, w0, w1, nullptr, static_cast<float*>(e->scratch), y->p, q->batch, who);
    }
    // quantized_matvec_preq panics for every other type (src/gguf.rs:4606)
    return fail(ALICE_E_UNSUPPORTED, "%s: pre-quantized input only for Q4_K/Q5_K/Q6_K/Q1_0/Q2_0", who);
}

int32_t alice_matvec(alice_engine* e, const alice_weights* w, const alice_buf* x, alice_buf* y, uint32_t batch) {
    return matvec_common(e, w, nullptr, x, y, batch, "alice_matvec");
}

int32_t alice_matvec_preq(alice_engine* e, const alice_weights* w, const alice_q8k* q, alice_buf* y) {
    return preq_common(e, w, nullptr, q, y, "alice_matvec_preq");
}

int32_t alice_swiglu(alice_engine* e, const alice_weights* gate, const alice_weights* up, const alice_buf* x,
                     alice_buf* y, uint32_t batch) {
    if (!up) return fail(ALICE_E_INVALID, "alice_swiglu: null argument");
    return matvec_common(e, gate, up, x, y, batch, "alice_swiglu");
}

int32_t alice_swiglu_preq(alice_engine* e, const alice_weights* gate, const alice_weights* up, const alice_q8k* q,
                          alice_buf* y) {
    if (!up) return fail(ALICE_E_INVALID, "alice_swiglu_preq: null argument");
    return preq_common(e, gate, up, q, y, "alice_swiglu_preq");
}

int32_t alice_plan_query(alice_engine* e, const alice_weights* w, int32_t swiglu, int32_t preq, uint32_t* out, uint32_t n_out) {
    if (!e || !w || !out || n_out < 10) return fail(ALICE_E_INVALID, "alice_plan_query: null argument or fewer than 10 outputs");
    GemvOp op;
    op.w[0] = &w->d;
    if (swiglu) op.up = &w->d;
    alignas(16) static float dummy[4];
    Q8KView v{};
    (void)preq;     // the input always reaches the kernel prepared; the plan does not depend on who prepared it
    if (format_uses_q8k(w->d.fmt)) { v.qs = reinterpret_cast<const int8_t*>(dummy); v.nb = w->d.cols / 256; op.q8 = &v; }
    else op.x = dummy;
    op.y = dummy;   // planning never dereferences the vectors
    StreamPlan pl;
    const int rc = plan_stream_gemv(op, cfg_of(e), pl);
    if (rc) return launch_rc(rc, "alice_plan_query");
    const StreamArgs& a = pl.args;
    out[0] = pl.grid; out[1] = a.P; out[2] = a.slots; out[3] = a.rps; out[4] = a.groups; out[5] = a.nstages;
    out[6] = pl.kl; out[7] = pl.mma ? 1u : 0u; out[8] = pl.ksplit; out[9] = pl.ctas_per_sm;
    return ALICE_OK;
}

int32_t alice_batch_plan(alice_engine* e, const alice_weights* w, int32_t swiglu, uint32_t batch, uint32_t* launches, uint32_t* weight_passes) {
    if (!e || !w || !launches || !weight_passes) return fail(ALICE_E_INVALID, "alice_batch_plan: null argument");
    if (batch == 0 || batch > 8) return fail(ALICE_E_SHAPE, "alice_batch_plan: batch %u outside 1..8", batch);
    GemvOp op;
    op.w[0] = &w->d;
    if (swiglu) op.up = &w->d;
    alignas(16) static float dummy[4];
    Q8KView v{};
    if (format_uses_q8k(w->d.fmt)) { v.qs = reinterpret_cast<const int8_t*>(dummy); v.d = dummy; v.bsums = reinterpret_cast<const int16_t*>(dummy); v.nb = w->d.cols / 256; op.q8 = &v; }
    else op.x = dummy;
    op.y = dummy; op.batch = batch;
    return launch_rc(batch_plan(op, cfg_of(e), launches, weight_passes), "alice_batch_plan");
}

int32_t alice_dequantize(alice_engine* e, const alice_weights* w, alice_buf* out) {
    if (!e || !w || !out) return fail(ALICE_E_INVALID, "alice_dequantize: null argument");
    if (out->len < (size_t)w->d.rows * w->d.cols) return fail(ALICE_E_SHAPE, "alice_dequantize: output too small");
    CU(cudaSetDevice(e->device));
    return launch_rc(launch_dequantize(w->d, out->p, e->stream), "alice_dequantize");
}

// ---- host-pointer convenience --------------------------------------------------------------

static alice_engine* g_host_engine = nullptr;
static std::mutex g_host_mu;

static int host_engine(alice_engine** out) {
    if (!g_host_engine) {
        int rc = alice_engine_create(0, &g_host_engine);
        if (rc) return rc;
    }
    *out = g_host_engine;
    return ALICE_OK;
}

int32_t alice_matvec_host(uint32_t type, const uint8_t* data, size_t nbytes, uint32_t rows, uint32_t cols,
                          const float* x, float* y) {
    if (!data || !x || !y) return fail(ALICE_E_INVALID, "alice_matvec_host: null argument");
    std::lock_guard<std::mutex> lk(g_host_mu);
    alice_engine* e;
    int rc = host_engine(&e);
    if (rc) return rc;
    alice_weights* w = nullptr;
    alice_buf *bx = nullptr, *by = nullptr;
    rc = alice_upload_weights(e, data, nbytes, type, rows, cols, &w);
    if (!rc) rc = alice_buf_upload_f32(e, x, cols, &bx);
    if (!rc) rc = alice_buf_alloc_f32(e, rows, &by);
    if (!rc) rc = alice_matvec(e, w, bx, by, 1);
    if (!rc) rc = alice_buf_read_f32(e, by, y, rows);
    if (!rc) rc = alice_sync(e);
    alice_buf_free(by); alice_buf_free(bx); alice_weights_free(w);
    return rc;
}

int32_t alice_dequantize_host(uint32_t type, const uint8_t* data, size_t nbytes, float* out, size_t n_out) {
    if (!data || !out) return fail(ALICE_E_INVALID, "alice_dequantize_host: null argument");
    const uint32_t be = ggml_block_elems((WeightFormat)type);
    if (be == 0) return fail(ALICE_E_UNSUPPORTED, "alice_dequantize_host: unsupported quantization type %u", type);
    if (n_out == 0 || n_out % be != 0 || n_out > 0xFFFFFFFFu)
        return fail(ALICE_E_SHAPE, "alice_dequantize_host: %zu outputs is not a whole number of blocks", n_out);
    std::lock_guard<std::mutex> lk(g_host_mu);
    alice_engine* e;
    int rc = host_engine(&e);
    if (rc) return rc;
    alice_weights* w = nullptr;
    alice_buf* bo = nullptr;
    rc = alice_upload_weights(e, data, nbytes, type, 1, (uint32_t)n_out, &w);
    if (!rc) rc = alice_buf_alloc_f32(e, n_out, &bo);
    if (!rc) rc = alice_dequantize(e, w, bo);
    if (!rc) rc = alice_buf_read_f32(e, bo, out, n_out);
    alice_buf_free(bo); alice_weights_free(w);
    return rc;
}

// ---- pre-quantized Q1_0 / Q2_0 matvec without any allocation -------------------------------------
//
// alice_matvec_preq turns the Q8_K blocks back into f32 (src/gguf.rs:4593-4605) in a scratch
// buffer that the engine obtains with cudaMalloc and grows on demand. Some callers must not reach
// the allocator at all: a serving process that has handed every byte of HBM to its own pool
// (KV-cache arena, a framework's caching allocator) so that cudaMalloc fails; or a decode thread
// that cannot afford cudaMalloc / cudaFree because both synchronise the whole device. For them the
// variant below keeps the f32 scratch in a fixed array that is part of the library image: every
// GPU that loads the library holds ALICE_NOALLOC_MAX_FLOATS * 4 bytes (256 KiB) until the process
// exits.

static __device__ __align__(256) float g_noalloc_scratch[ALICE_NOALLOC_MAX_FLOATS];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address; the
// address of each device's copy is looked up once, with that device current, and cached here.
static float* g_noalloc_ptr[64] = {};
static std::mutex g_noalloc_mu;

static __global__ void q8k_to_f32_noalloc_kernel(Q8KView q, uint32_t total) {
    pdl_wait_abi();
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x)
        g_noalloc_scratch[i] = __fmul_rn(q.d[i >> 8], (float)q.qs[i]);
}

static int noalloc_scratch_for(alice_engine* e, float** out) {
    if (e->device < 0 || e->device >= 64) return fail(ALICE_E_INVALID, "alice_matvec_preq_noalloc: device index %d", e->device);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[e->device]) {
        void* p = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&p, g_noalloc_scratch);  // current device = e->device (set by the caller)
        if (err != cudaSuccess || !p) return cuda_fail(err, "alice_matvec_preq_noalloc: cudaGetSymbolAddress");
        g_noalloc_ptr[e->device] = static_cast<float*>(p);
    }
    *out = g_noalloc_ptr[e->device];
    return ALICE_OK;
}

int32_t alice_matvec_preq_noalloc(alice_engine* e, const alice_weights* w, const alice_q8k* q, alice_buf* y) {
    const char* who = "alice_matvec_preq_noalloc";
    if (!e || !w || !q || !y) return fail(ALICE_E_INVALID, "%s: null argument", who);
    const WeightDesc& d = w->d;
    if (d.fmt != WF_Q1_0 && d.fmt != WF_Q2_0)
        return fail(ALICE_E_UNSUPPORTED, "%s: only Q1_0 / Q2_0 weights need the f32 scratch; use alice_matvec_preq", who);
    if (q->cols != d.cols) return fail(ALICE_E_SHAPE, "%s: Q8_K input has %u columns, weights %u", who, q->cols, d.cols);
    if (q->batch == 0 || q->batch > 8) return fail(ALICE_E_SHAPE, "%s: batch %u outside 1..8", who, q->batch);
    const size_t total = (size_t)q->batch * d.cols;
    if (total > (size_t)ALICE_NOALLOC_MAX_FLOATS)
        return fail(ALICE_E_SHAPE, "%s: batch * cols = %zu floats exceeds the fixed scratch of %d floats", who, total,
                    (int)ALICE_NOALLOC_MAX_FLOATS);
    if (y->len < (size_t)q->batch * d.rows) return fail(ALICE_E_SHAPE, "%s: output too small", who);
    CU(cudaSetDevice(e->device));
    float* scratch = nullptr;
    int rc = noalloc_scratch_for(e, &scratch);
    if (rc) return rc;
    // Every element the matvec reads is rewritten first, so nothing has to be cleared between calls.
    const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 148 * 8);
    q8k_to_f32_noalloc_kernel<<<blocks, 256, 0, e->stream>>>(view_of(q, 0), (uint32_t)total);
    CU(cudaGetLastError());
    return run_gemv(e, w, nullptr, nullptr, scratch, y->p, q->batch, who, false);   // never allocates
}

}  // extern "C"
