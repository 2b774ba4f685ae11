// Shared device helpers for the quantized-matvec kernels (sm_100a).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace alice {

constexpr int QK_K = 256;

// Status codes written by kernels into the engine's device status word.
// low byte: which wait ran out of its cycle budget; higher bits: index of the op inside a multi-op kernel
constexpr int KERR_WAIT_TIMEOUT = 1;   // unspecified wait
constexpr int KERR_WAIT_FULL = 2;      // consumer waiting for a weight stage to land
constexpr int KERR_WAIT_PARTIALS = 3;  // row finalizer waiting for the other warps' partial sums
constexpr int KERR_WAIT_EMPTY = 4;     // producer waiting for a stage to be released
constexpr int KERR_WAIT_GRID = 5;      // grid-wide barrier
constexpr int KERR_WAIT_PEER = 6;      // rows another GPU pushes into this GPU's vector (tensor parallel)

// A wait that has not been satisfied after this many SM clock cycles (about one second) gives
// up, records KERR_WAIT_TIMEOUT and lets the CTA drain and return instead of spinning forever.
constexpr long long WAIT_CYCLE_LIMIT = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ── shared-memory loads by 32-bit shared address ────────────────────────────
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float ldsf(uint32_t a) { return __uint_as_float(lds32(a)); }

// 32-bit word at a shared address that is only 2-byte aligned: two aligned words, funnel shift.
__device__ __forceinline__ uint32_t lds32_u2(uint32_t a) {
    uint32_t base = a & ~3u;
    uint32_t lo = lds32(base), hi = lds32(base + 4);
    return __funnelshift_r(lo, hi, (a & 2u) * 8u);
}

// ── mbarrier + bulk async copy (TMA, untiled) ───────────────────────────────
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: true when the phase completed, false after WAIT_CYCLE_LIMIT cycles.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > WAIT_CYCLE_LIMIT) return false;
    }
    return true;
}
// Contiguous global -> shared copy. Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Programmatic dependent launch: wait for the producing grid / let the dependent grid start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ── cross-GPU hand-over (tensor parallel): peers store rows straight into this GPU's vector and bump a
// counter here; the reader waits (bounded) for the count before it touches the vector ─────────────────
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add_u32(unsigned int* p, unsigned int v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// One thread. true when *flag has reached `expected` (wrap-safe), false after `limit` SM cycles; records `code` in the
// status word then (the first report is kept).
__device__ __forceinline__ bool peer_wait(const unsigned int* flag, unsigned int expected, int* status, int code,
                                          long long limit = WAIT_CYCLE_LIMIT) {
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys_u32(flag) - expected) < 0) {
        if (clock64() - t0 > limit) {
            atomicCAS(status, 0, code);
            return false;
        }
    }
    return true;
}

// ── arithmetic helpers ──────────────────────────────────────────────────────
// u8 x s8 dot of four byte lanes, accumulated into c.
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// IEEE half -> float; identical to the reference's bit-level f16_to_f32 for every non-NaN input.
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// silu as the reference writes it: x / (1 + exp(-x)).
__device__ __forceinline__ float silu_ref(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }

}  // namespace alice
