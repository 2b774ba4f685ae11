// Whole-decode-step kernel: every matvec, the attention and the token hand-over of `nsteps`
// decode steps run inside ONE cooperative launch of 2 CTAs per SM.
//
// Why: at batch 1 a projection streams for only 1-10 us, and a kernel boundary (drain, dependency
// resolution, launch, ring refill) costs about 3 us - as much as the work. Here the producer warp of
// every CTA walks the op list on its own and keeps the shared-memory ring full of the NEXT matvec's
// weights while the consumer warps finish the current one and meet at the grid barrier, so HBM
// never idles across an op boundary. Activations move between ops through global memory (read with
// ld.global.cg, since other SMs rewrite them inside the kernel); ordering is a grid-wide barrier
// (one atomic counter, bounded spin) after every op.
#include "attn_body.cuh"
#include "formats.cuh"
#include "step_kernel.cuh"

namespace alice {

namespace {

// Grid-wide barrier for the consumer warps of all CTAs (all CTAs are co-resident: cooperative launch).
// false = gave up (timeout, or a wait inside this or another CTA aborted); all 256 consumer threads
// of the CTA get the same answer and leave the kernel together, so nobody is left at a named barrier.
__device__ __forceinline__ bool grid_sync(unsigned int* counter, uint32_t& epoch, StreamSmem* sm, int* status) {
    asm volatile("bar.sync 1, 256;" ::: "memory");
    epoch++;
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        const unsigned int target = epoch * gridDim.x;
        const long long t0 = clock64();
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if (v >= target) break;
            if (sm->abort_flag || __ldcg(status) != 0) { sm->abort_flag = 1; break; }
            if (clock64() - t0 > 3 * WAIT_CYCLE_LIMIT) {   // longest: a stall inside a CTA should be what gets reported
                sm->abort_flag = 1;
                atomicCAS(status, 0, KERR_WAIT_GRID + (int)(epoch << 8));
                break;
            }
        }
        __threadfence();
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    return sm->abort_flag == 0;
}

// Each instance is a real function call, so its registers are allocated on their own instead of
// the whole op interpreter paying for the widest one.
template <class F, int KL, bool SW>
__device__ __noinline__ bool consume_call(const StreamArgs& a, StreamCtx& cx) { return stream_consume<F, KL, SW, true>(a, cx); }

__device__ __forceinline__ bool run_gemv(int variant, const StreamArgs& g, StreamCtx& cx) {
    switch (variant) {
        case SV_Q4K_1: return consume_call<FmtQ4K, 1, false>(g, cx);
        case SV_Q4K_1_SW: return consume_call<FmtQ4K, 1, true>(g, cx);
        case SV_Q4K_2: return consume_call<FmtQ4K, 2, false>(g, cx);
        case SV_Q6K_1: return consume_call<FmtQ6K, 1, false>(g, cx);
        case SV_Q6K_2: return consume_call<FmtQ6K, 2, false>(g, cx);
        case SV_Q8_0_1: return consume_call<FmtQ8_0, 1, false>(g, cx);
        case SV_Q8_0_2: return consume_call<FmtQ8_0, 2, false>(g, cx);
        default: return false;
    }
}

// Word-wise copy of one matvec's arguments from the device-resident op list into shared memory.
__device__ __forceinline__ void copy_args(StreamArgs* dst, const StreamArgs* src, uint32_t tid, uint32_t nthreads) {
    static_assert(sizeof(StreamArgs) % 4 == 0, "copied as 32-bit words");
    const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
    uint32_t* d = reinterpret_cast<uint32_t*>(dst);
    for (uint32_t i = tid; i < sizeof(StreamArgs) / 4; i += nthreads) d[i] = __ldg(s + i);
}

// Asynchronous copy (no register round trip, so the issuing warps carry on at once) of one op
// descriptor into shared memory; complete for everybody after cp_async_wait_all() + a CTA barrier.
__device__ __forceinline__ void prefetch_op(StepOp* dst, const StepOp* src, uint32_t tid) {
    static_assert(sizeof(StepOp) % 16 == 0, "copied in 16-byte pieces");
    if (tid < sizeof(StepOp) / 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(reinterpret_cast<uint8_t*>(dst) + tid * 16)),
                     "l"(reinterpret_cast<const uint8_t*>(src) + tid * 16)
                     : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int GROUP>
__device__ __noinline__ void run_attn(const StepOp& op, uint32_t pos, uint8_t* aux, long long* prof) {
    AttnSmem<GROUP>* sh = reinterpret_cast<AttnSmem<GROUP>*>(aux);
    const uint32_t items = op.shape.num_kv_heads * op.nsplit;
    for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        asm volatile("bar.sync 1, 256;" ::: "memory");   // the scratch of the previous item is free
        attn_fused_body<GROUP, true>(op.qkv, op.kc, op.vc, pos, op.shape, op.rope_tab, op.neox, op.nsplit, op.part,
                                     op.tickets, op.attn_out, it % op.shape.num_kv_heads, it / op.shape.num_kv_heads, sh, prof);
    }
}

}  // namespace

__global__ void __launch_bounds__(STREAM_THREADS, 2) decode_step_kernel(const StepArgs sa) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    StreamSmem* sm = reinterpret_cast<StreamSmem*>(smem_raw);
    StreamCtx cx;
    cx.sm = sm; cx.smem_raw = smem_raw; cx.ring = smem_u32(smem_raw) + STREAM_HDR_BYTES;
    cx.stage_stride = sa.stage_stride; cx.nstages = sa.nstages; cx.cc = 0; cx.op = 0; cx.acts_cg = true;
    if (threadIdx.x == 0) stream_init_ring(sm, sa.nstages);
    __syncthreads();

    if ((threadIdx.x >> 5) == NCW) {
        // producer warp: streams the weights of every matvec of every step, never waiting for activations
        const uint32_t lane = threadIdx.x & 31;
        for (uint32_t step = 0; step < sa.nsteps; step++)
            for (uint32_t i = 0; i < sa.nops; i++) {
                if (sa.ops[i].type != SOP_GEMV) continue;
                copy_args(&sm->pargs, &sa.ops[i].g, lane, 32);
                __syncwarp();
                if (lane == 0 && !sm->abort_flag) { cx.op = (int)i; stream_produce(sm->pargs, cx); }
                __syncwarp();
            }
        if (lane == 0 && sm->abort_flag) stream_drain(cx);
        return;
    }

    uint8_t* aux = smem_raw + sa.aux_off;
    StepOp* sops = reinterpret_cast<StepOp*>(smem_raw + sa.ops_off);
    static_assert(sizeof(StepOp) / 16 <= NCW * 32, "one 16-byte piece per consumer thread");
    uint32_t epoch = 0, nop = 0;   // nop: ops started so far; descriptor of op number n sits in sops[n & 1]
    prefetch_op(&sops[0], &sa.ops[0], threadIdx.x);
    cp_async_wait_all();
    asm volatile("bar.sync 1, 256;" ::: "memory");
    for (uint32_t step = 0; step < sa.nsteps; step++) {
        const uint32_t pos = (uint32_t)__ldcg(sa.pos);
        for (uint32_t i = 0; i < sa.nops; i++, nop++) {
            const StepOp& op = sops[nop & 1];
            // the next descriptor travels while this op runs
            if (i + 1 < sa.nops || step + 1 < sa.nsteps) prefetch_op(&sops[(nop + 1) & 1], &sa.ops[i + 1 < sa.nops ? i + 1 : 0], threadIdx.x);
            long long* prof = (sa.prof && blockIdx.x == gridDim.x / 2) ? sa.prof + 16 * i : nullptr;
            cx.prof = prof;
            if (prof && threadIdx.x == 0) prof[0] = clock64();
            if (op.type == SOP_EMBED) {
                // hidden = dequantized Q8_0 row of the current token (src/gguf.rs:990-1004)
                if (blockIdx.x == gridDim.x - 1 && threadIdx.x < 64) rope_table_entry(op.rope_tab, threadIdx.x, pos, op.theta);
                uint32_t t = (uint32_t)__ldcg(sa.token);
                if (t >= op.vocab) t = 0;
                const uint8_t* row = op.table + (size_t)t * (op.cols / 32) * 34;
                for (uint32_t c = blockIdx.x * 256 + threadIdx.x; c < op.cols; c += gridDim.x * 256) {
                    const uint8_t* b = row + (c >> 5) * 34;
                    const float d = f16_bits_to_f32((uint32_t)b[0] | ((uint32_t)b[1] << 8));
                    op.hidden[c] = __fmul_rn(d, (float)(int8_t)b[2 + (c & 31)]);
                }
            } else if (op.type == SOP_GEMV) {
                cx.op = (int)i;
                run_gemv(op.variant, op.g, cx);   // after an abort every warp still walks to the barrier below and leaves there
            } else if (op.type == SOP_ATTN) {
                switch (op.shape.num_heads / op.shape.num_kv_heads) {
                    case 1: run_attn<1>(op, pos, aux, prof); break;
                    case 2: run_attn<2>(op, pos, aux, prof); break;
                    case 4: run_attn<4>(op, pos, aux, prof); break;
                    default: break;
                }
            }
            if (prof && threadIdx.x == 0) prof[4] = clock64();
            cp_async_wait_all();   // own pieces of the next descriptor; the barrier below publishes everybody's
            if (!grid_sync(sa.barrier, epoch, sm, sa.status)) return;
            if (prof && threadIdx.x == 0) prof[5] = clock64();
        }
        // greedy hand-over: the head matvec left the packed maximum; one thread turns it into the next token
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            const unsigned long long k = __ldcg(sa.key);
            if (sa.write_token) {
                const int t = (int)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
                *sa.token = t;
                if (sa.trace) sa.trace[pos] = t;
            }
            *sa.pos = (int)pos + 1;
            *sa.key = 0ull;
        }
        if (!grid_sync(sa.barrier, epoch, sm, sa.status)) return;
    }
}

cudaError_t launch_decode_steps(const StepArgs& sa, uint32_t grid, size_t smem, cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t err = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)STEP_SMEM_BUDGET);
        if (err != cudaSuccess) return err;
        attr_set = true;
    }
    void* args[] = {const_cast<StepArgs*>(&sa)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(decode_step_kernel), dim3(grid), dim3(STREAM_THREADS), args, smem, st);
}

cudaError_t decode_step_max_ctas_per_sm(size_t smem, int* out) {
    cudaError_t err = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)STEP_SMEM_BUDGET);
    if (err != cudaSuccess) return err;
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(out, decode_step_kernel, STREAM_THREADS, smem);
}

int step_variant(WeightFormat f, uint32_t kl, bool swiglu) {
    if (f == WF_Q4_K && kl == 1) return swiglu ? SV_Q4K_1_SW : SV_Q4K_1;
    if (f == WF_Q4_K && kl == 2 && !swiglu) return SV_Q4K_2;
    if (f == WF_Q6_K && !swiglu && (kl == 1 || kl == 2)) return kl == 1 ? SV_Q6K_1 : SV_Q6K_2;
    if (f == WF_Q8_0 && !swiglu && (kl == 1 || kl == 2)) return kl == 1 ? SV_Q8_0_1 : SV_Q8_0_2;
    return -1;
}

}  // namespace alice
