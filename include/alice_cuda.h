/* alice_cuda.h -- C ABI of the B200 (sm_100a) quantized-matvec decode path for ALICE-LLM.
 *
 * This library replaces, for the decode hot path only, the wgpu backend of ALICE-LLM
 * (src/gpu.rs) and the CPU quantized matvec of src/gguf.rs. Weights are uploaded as the raw
 * GGUF blocks and stay on the device; every entry point below names the reference interface
 * it stands in for (file:line in ext-sakamoro/ALICE-LLM v1.6.0).
 *
 * Conventions
 *   - Every function returns an int32_t status: ALICE_OK (0) or a negative ALICE_E_* code.
 *     The reference panics on shape / format violations (src/gguf.rs:4243, src/gpu.rs:721-734);
 *     a binding turns a non-zero status into its language's panic. alice_last_error() gives
 *     the message of the calling thread's last failure.
 *   - No CPU fallback exists: without a CUDA device alice_engine_create fails.
 *   - All device work of an engine is queued on one CUDA stream, in call order (the reference
 *     has a single in-order wgpu queue). Calls on one engine are not thread-safe, like the
 *     reference's Mutex<ModelBackend> usage (src/bin/server.rs:359).
 *   - Batch layout: inputs x[k*cols + c], outputs y[k*rows + r] (src/gpu.rs:1141-1143).
 *   - Kernels that wait on a barrier give up after about one second, record an error in the
 *     engine's device status word and return; alice_sync reports it as ALICE_E_KERNEL.
 */
#ifndef ALICE_CUDA_H
#define ALICE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ALICE_OK 0
#define ALICE_E_INVALID (-1)     /* null pointer, misaligned device pointer, bad handle */
#define ALICE_E_UNSUPPORTED (-2) /* quantization type outside the path */
#define ALICE_E_SHAPE (-3)       /* rows/cols/bytes do not fit the format or each other */
#define ALICE_E_CUDA (-4)        /* a CUDA runtime call failed */
#define ALICE_E_KERNEL (-5)      /* a kernel recorded an error in the status word */
#define ALICE_E_NOMEM (-6)       /* device allocation failed */

/* GGML type ids of the block formats on the path (GgmlType::from_u32, src/gguf.rs:101-122). */
#define ALICE_TYPE_Q8_0 8u
#define ALICE_TYPE_Q4_K 12u
#define ALICE_TYPE_Q5_K 13u
#define ALICE_TYPE_Q6_K 14u
#define ALICE_TYPE_Q1_0 41u
#define ALICE_TYPE_Q2_0 42u

typedef struct alice_engine alice_engine;   /* GpuEngine, src/gpu.rs:320 */
typedef struct alice_weights alice_weights; /* GpuWeightBuffer, src/gpu.rs:302 */
typedef struct alice_buf alice_buf;         /* GpuBuffer (f32 storage), src/gpu.rs:277 */
typedef struct alice_q8k alice_q8k;         /* Vec<BlockQ8K> on the device, src/gguf.rs:1306 */

/* Message of the calling thread's most recent failing call ("" if none). */
const char* alice_last_error(void);

/* Block geometry, GgmlType::block_bytes / elements_per_block (src/gguf.rs:126, :161). 0 = unknown type. */
uint32_t alice_type_block_bytes(uint32_t ggml_type);
uint32_t alice_type_block_elems(uint32_t ggml_type);

/* ---- engine ------------------------------------------------------------------------------ */
/* GpuEngine::new (src/gpu.rs:434). Selects `device`, creates the engine's stream. */
int32_t alice_engine_create(int32_t device, alice_engine** out);
int32_t alice_engine_destroy(alice_engine* e);
/* Queue the engine's work on a caller-owned CUDA stream (cudaStream_t passed as void*), e.g. the
 * current stream of a framework that owns the device buffers. No reference counterpart. */
int32_t alice_engine_set_stream(alice_engine* e, void* cuda_stream);
/* GpuEngine::sync (src/gpu.rs:962): block until queued work is done; ALICE_E_KERNEL if a kernel
 * recorded an error (the status word is cleared). */
int32_t alice_sync(alice_engine* e);
/* Launch dependent kernels with programmatic stream serialization (on by default). */
int32_t alice_engine_set_pdl(alice_engine* e, int32_t enabled);
/* Tuning overrides for the streaming matvec: rows per warp set per stage and ring depth; 0 = automatic. */
int32_t alice_engine_set_tuning(alice_engine* e, int32_t rows_per_set, int32_t stages);
/* Cycle budget (SM clock cycles) of every bounded wait inside the kernels launched from now on; 0 = the default of
 * about one second. A wait that runs out records its code in the engine's status word and the kernel returns;
 * alice_sync then reports ALICE_E_KERNEL and clears the word (the engine stays usable). No reference counterpart. */
int32_t alice_engine_set_wait_limit(alice_engine* e, uint64_t sm_cycles);
/* Self-test of that path, nothing else: queues the tensor-parallel hand-over of a 256-element vector with one "peer"
 * whose flag nobody ever raises (both flags live in scratch memory of this GPU), so the bounded wait runs out after
 * the engine's cycle budget and the kernel returns with status 6 recorded. The next alice_sync reports ALICE_E_KERNEL;
 * work queued afterwards runs normally. Set a short budget first (a few million cycles). No reference counterpart. */
int32_t alice_debug_expire_wait(alice_engine* e);

/* ---- weights ----------------------------------------------------------------------------- */
/* GpuEngine::upload_weights / _q5k / _q6k / _q8_0 / _q1_0 (src/gpu.rs:698-798): raw GGUF blocks,
 * row-major, rows * (cols / block_elems) * block_bytes bytes, copied verbatim (Q8_0 is NOT
 * re-padded to 36 bytes as the wgpu backend does). cols must be a whole number of blocks. */
int32_t alice_upload_weights(alice_engine* e, const uint8_t* data, size_t nbytes, uint32_t ggml_type,
                             uint32_t rows, uint32_t cols, alice_weights** out);
/* Same, for blocks already resident on the device (16-byte aligned, not copied, not owned). */
int32_t alice_weights_from_device(alice_engine* e, const void* device_ptr, size_t nbytes, uint32_t ggml_type,
                                  uint32_t rows, uint32_t cols, alice_weights** out);
/* TernaryMatrix (src/gguf.rs:5190-5202): pos/neg bit planes flattened to [rows][ceil(cols/8)]
 * (bit i%8 of byte i/8), one f32 scale per row. */
int32_t alice_upload_ternary(alice_engine* e, const uint8_t* pos, const uint8_t* neg, const float* scales,
                             uint32_t rows, uint32_t cols, alice_weights** out);
/* Borrowed device-resident ternary matrix in the layout alice_upload_ternary builds on the device: row r =
 * [pos plane | neg plane], each plane ceil(cols/32)*4 bytes (bit c%8 of byte c/8, zero bits past cols), plus
 * one f32 scale per row. No reference counterpart (the reference uploads from host memory only); it lets a
 * host that already holds the planes on the device (or generates them there) skip the round trip. */
int32_t alice_ternary_from_device(alice_engine* e, const void* rows_dptr, const float* scales_dptr, uint32_t rows,
                                  uint32_t cols, alice_weights** out);
/* SparseTernaryMatrix (src/gguf.rs:5425-5445): packed_2bit rows, 4 bytes per 16 columns
 * (00 = 0, 01 = +1, 11 = -1), [rows][ceil(cols/16)*4] bytes, one f32 scale per row. */
int32_t alice_upload_sparse_ternary(alice_engine* e, const uint8_t* packed_2bit, const float* scales,
                                    uint32_t rows, uint32_t cols, alice_weights** out);
int32_t alice_weights_free(alice_weights* w);

/* ---- f32 buffers ------------------------------------------------------------------------- */
/* GpuEngine::alloc_f32 / upload_f32 / write_f32 / read_f32 (src/gpu.rs:667-695, 801-824). */
int32_t alice_buf_alloc_f32(alice_engine* e, size_t len, alice_buf** out);
int32_t alice_buf_upload_f32(alice_engine* e, const float* data, size_t len, alice_buf** out);
int32_t alice_buf_write_f32(alice_engine* e, alice_buf* b, const float* data, size_t len);
int32_t alice_buf_read_f32(alice_engine* e, const alice_buf* b, float* out, size_t len);
/* The same two copies queued on the engine's stream without waiting (GpuEngine::write_f32 is queue.write_buffer in the
 * reference, src/gpu.rs:801, which does not block either): `data` / `out` must stay valid - and should be pinned host
 * memory - until the next alice_sync (or any blocking call) has returned; `out` holds the values only then. With them a
 * host-buffer step costs one synchronisation instead of two. */
int32_t alice_buf_write_f32_async(alice_engine* e, alice_buf* b, const float* data, size_t len);
int32_t alice_buf_read_f32_async(alice_engine* e, const alice_buf* b, float* out, size_t len); /* blocks */
/* Wrap `len` floats of caller-owned device memory (not copied, not owned). */
int32_t alice_buf_from_device(alice_engine* e, void* device_ptr, size_t len, alice_buf** out);
int32_t alice_buf_free(alice_buf* b);

/* ---- Q8_K activations -------------------------------------------------------------------- */
/* quantize_row_q8_k (src/gguf.rs:1323): `batch` vectors of `cols` floats (cols % 256 == 0). */
int32_t alice_q8k_alloc(alice_engine* e, uint32_t cols, uint32_t batch, alice_q8k** out);
int32_t alice_quantize_q8k(alice_engine* e, const alice_buf* x, alice_q8k* q);
/* Copy to host as structure-of-arrays: d[batch*nb], qs[batch*nb*256], bsums[batch*nb*16]. Blocks. */
int32_t alice_q8k_read(alice_engine* e, const alice_q8k* q, float* d, int8_t* qs, int16_t* bsums);
/* Upload host BlockQ8K data given as the same three arrays (for the *_matvec_preq signatures). */
int32_t alice_q8k_upload(alice_engine* e, const float* d, const int8_t* qs, const int16_t* bsums,
                         uint32_t cols, uint32_t batch, alice_q8k** out);
int32_t alice_q8k_free(alice_q8k* q);

/* TernaryRow::from_f32 for every row of an f32 matrix on the device (src/gguf.rs:5207-5245; w[r * cols + c]):
 * threshold = threshold_ratio * mean |w| of the row, masks of the weights above it, scale = their mean magnitude. The
 * masks and scales equal the reference's bit for bit (sums run in its order). *out is a ternary matrix like
 * alice_upload_ternary's. */
int32_t alice_ternarize(alice_engine* e, const alice_buf* w, uint32_t rows, uint32_t cols, float threshold_ratio,
                        alice_weights** out);
/* SparseTernaryRow::from_ternary_row for every row (src/gguf.rs:5451-5507): of the non-zero weights of each block of 16
 * the n_keep largest |w| stay (ties: the earlier one); packed as SparseTernaryMatrix.packed_2bit, scale = mean kept
 * magnitude (the dense scale for a row that keeps nothing). `w` is the f32 matrix `ternary` was made from. */
int32_t alice_sparsify(alice_engine* e, const alice_weights* ternary, const alice_buf* w, uint32_t n_keep, alice_weights** out);
/* The device rows of a weight matrix back on the host (rows * row bytes, the layout the library keeps: raw GGUF blocks;
 * [pos plane | neg plane] per row with planes of ceil(cols / 32) * 4 bytes; packed 2-bit rows of ceil(cols / 16) * 4
 * bytes) and, for the ternary forms, the per-row scales (scales_out may be null). No reference counterpart. */
int32_t alice_weights_download(alice_engine* e, const alice_weights* w, uint8_t* rows_out, size_t rows_bytes, float* scales_out);

/* ---- the hot path ------------------------------------------------------------------------ */
/* quantized_matvec / q4k_matvec / q5k_matvec / q6k_matvec / q8_0_matvec / ternary_matvec /
 * sparse_ternary_matvec (src/gguf.rs:4214, 3600, 3502, 4077, 3811, 5303, 5808) and
 * GpuPass::matvec_* / matvec_auto (src/gpu.rs:1022-1392, 1795-1960): y = W x for `batch`
 * input vectors (1..8). K-quant weights quantize x to Q8_K first, as the CPU path does. */
int32_t alice_matvec(alice_engine* e, const alice_weights* w, const alice_buf* x, alice_buf* y, uint32_t batch);
/* quantized_matvec_preq / q4k_matvec_preq / ... (src/gguf.rs:4574, 3607, 3509, 4084). For Q1_0 /
 * Q2_0 weights the Q8_K blocks are turned back into f32 first (src/gguf.rs:4593-4605). */
int32_t alice_matvec_preq(alice_engine* e, const alice_weights* w, const alice_q8k* q, alice_buf* y);
/* Fused SwiGLU gate/up, swiglu_fused_q4k / _q1_0 dispatch (src/gpu.rs:4711-4721, 5995) and the
 * CPU model's gate/up/silu sequence (src/llama3.rs:14519-14534): y = silu(gate x) * (up x). */
int32_t alice_swiglu(alice_engine* e, const alice_weights* gate, const alice_weights* up, const alice_buf* x,
                     alice_buf* y, uint32_t batch);
int32_t alice_swiglu_preq(alice_engine* e, const alice_weights* gate, const alice_weights* up, const alice_q8k* q,
                          alice_buf* y);
/* dequantize_weight_row / GgufFile::tensor_to_f32 (src/gguf.rs:6168, 574): out[r*cols + c], bit-exact. */
int32_t alice_dequantize(alice_engine* e, const alice_weights* w, alice_buf* out);

/* Launch geometry the planner chooses for one matvec over `w` (fused SwiGLU of two such matrices when swiglu != 0;
 * pre-quantized Q8_K input when preq != 0): out[0..9] = CTAs, warps per row (or per 16-row tile), row sets per CTA,
 * rows per set per stage, stage-sized row groups in total, ring stages, activation units per lane, 1 if the bit-plane
 * tensor-core kernel is used, column chunks, CTAs per SM. A CTA handles about groups / CTAs stages, so a test can
 * assert that a shape really re-uses the ring. No reference counterpart (diagnostic). */
int32_t alice_plan_query(alice_engine* e, const alice_weights* w, int32_t swiglu, int32_t preq, uint32_t* out, uint32_t n_out);

/* How alice_matvec / alice_swiglu run `batch` input vectors over `w`: the number of kernel launches and how many times
 * the weight bytes stream from HBM (1 = the batch kernel decodes every weight once for all vectors, as the reference's
 * *_batch4 shaders do, src/gpu.rs:4759; `batch` = one pass per vector). No reference counterpart (diagnostic). */
int32_t alice_batch_plan(alice_engine* e, const alice_weights* w, int32_t swiglu, uint32_t batch, uint32_t* launches, uint32_t* weight_passes);

/* ---- tensor parallel ------------------------------------------------------------------------ */
/* One engine (one process) per GPU; output rows of every projection are sharded over the group and the
 * full vector is rebuilt on every rank by an NCCL all-gather queued on the engine's stream (the row
 * split is where the reference parallelises a matvec, src/gguf.rs:3664; the reference itself is single
 * device). NCCL is loaded at run time (libnccl.so.2), only when a group is formed.
 * alice_tp_unique_id: rank 0 fills `out` (ALICE_TP_ID_BYTES) and hands it to the other ranks by any
 * means; every rank then calls alice_engine_tp_init (collective: returns when the group is formed).
 * A model created on an engine that belongs to a group takes this rank's row shards (see below). */
#define ALICE_TP_ID_BYTES 128
int32_t alice_tp_unique_id(void* out, size_t nbytes);
int32_t alice_engine_tp_init(alice_engine* e, uint32_t rank, uint32_t world, const void* unique_id, size_t nbytes);
int32_t alice_engine_tp_info(const alice_engine* e, uint32_t* rank, uint32_t* world);

/* ---- decode model ------------------------------------------------------------------------- */
/* GpuModel (src/gpu.rs:2348) for the Llama-style attention + SwiGLU layer stack, i.e. the Llama branch
 * of Llama3Model::forward_with_layer_hook (src/llama3.rs:13632-13687, 14167-14613): per layer
 * rms_norm -> q/k/v matvec -> RoPE -> KV append -> GQA attention -> o matvec + residual ->
 * rms_norm -> fused SwiGLU gate/up -> down matvec + residual; then output norm and head.
 * One decode step is five large kernels per layer (q/k/v, attention, o, gate/up, down) with a small kernel in front of
 * each matvec that prepares its input once (rms_norm, Q8_K blocks or the f32 vector and its digit table), replayed from a
 * CUDA graph; position and token live on the device. K-quant projections use the CPU model's semantics (Q8_K-quantized
 * activations).
 * On an engine that is rank r of a tensor-parallel group of n, the config stays the whole model's and the
 * weight handles are row shards: rows [r*R/n, (r+1)*R/n) of q, k, v, o, gate, up, down and the output
 * head (R = that matrix's row count; contiguous byte ranges of the raw blocks); the embedding table is
 * whole on every rank. The rank keeps the KV cache of its num_kv_heads/n heads only (kv_write / kv_read
 * move rows of kv_dim/n floats). All ranks must make the same calls in the same order. */
typedef struct alice_model alice_model;
typedef struct {                       /* GpuModelConfig, src/gpu.rs:2111-2151 */
    uint32_t num_layers, hidden_dim, intermediate_dim, num_heads, num_kv_heads, head_dim;
    uint32_t vocab_size, max_seq_len;
    float rope_theta, eps;
    uint32_t neox_rope;                /* 0 = pairs (i, i+1) (Llama), 1 = (i, i + d/2) */
} alice_model_config;
typedef struct {                       /* one transformer layer; norms are host arrays of hidden_dim floats */
    const alice_weights *q, *k, *v, *o, *gate, *up, *down;
    const float *attn_norm, *ffn_norm;
} alice_layer_weights;
/* GpuModel::load (src/gpu.rs:2831). Weight handles are borrowed and must outlive the model. The
 * embedding is a Q8_0 table [vocab][hidden] kept quantized; a row is dequantized per token. */
int32_t alice_model_create(alice_engine* e, const alice_model_config* cfg, const alice_layer_weights* layers,
                           const alice_weights* embedding, const float* output_norm, const alice_weights* output,
                           alice_model** out);
int32_t alice_model_destroy(alice_model* m);
/* GpuModel::forward / forward_and_read (src/gpu.rs:5010, 5033): one token at the current position. */
int32_t alice_model_forward(alice_model* m, uint32_t token);
int32_t alice_model_forward_read(alice_model* m, uint32_t token, float* logits);
/* GpuModel::forward_batch / forward_batch_and_read (src/gpu.rs:6020, 6057): n consecutive tokens (1..8; the reference
 * takes exactly 4) in one pass over the weights, token k at position + k attending position + k + 1 rows (causal,
 * src/shaders/attention.wgsl:45); the position advances by n. logits[k * vocab + v]. Together with
 * alice_model_rollback_to this is the verify step of speculative decoding (examples/speculative_dual_gpu.rs:230-322).
 * Single GPU only. */
int32_t alice_model_forward_batch(alice_model* m, const uint32_t* tokens, uint32_t n);
int32_t alice_model_forward_batch_read(alice_model* m, const uint32_t* tokens, uint32_t n, float* logits);
/* Greedy decode loop (Llama3Model::generate's decode loop, src/llama3.rs:16084, with argmax sampling):
 * feeds first_token, then n-1 times the argmax of the previous logits; out_tokens[i] = argmax after
 * step i. No host round trip between steps. */
int32_t alice_model_decode_greedy(alice_model* m, uint32_t first_token, uint32_t n, uint32_t* out_tokens);
int32_t alice_model_read_logits(alice_model* m, float* logits);
/* Tensor parallel without collective calls: after every rank has created its model, each exports a handle to its
 * exchange region (ALICE_TP_HANDLE_BYTES; CUDA IPC, same node), the host gathers the handles of all ranks in rank
 * order and every rank connects. From then on the kernel that produces a sharded vector stores its rows straight
 * into every peer's copy over NVLink; a one-CTA kernel behind it raises one counter per vector on every peer (release)
 * and waits, bounded (ALICE_E_KERNEL on expiry), until all peers have raised the same counter here, then prepares the
 * complete vector for the next op. The consuming kernels read local memory only. The connect result must be the same on every
 * rank (all-reduce the status on the host and rebuild the models if any rank failed: a rank left on NCCL would block
 * in its next all-gather), and the ranks must meet in a host barrier before alice_model_destroy (a peer may still be
 * storing into the region). No reference counterpart (the reference is single device). */
#define ALICE_TP_HANDLE_BYTES 64
int32_t alice_model_tp_export(alice_model* m, void* out, size_t nbytes);
int32_t alice_model_tp_connect(alice_model* m, const void* handles, size_t bytes_per_handle);
/* position / vocab_size / rollback_to / reset (src/gpu.rs:5655, 5660, 5645, 5618). rollback only lowers
 * the position; reset also zeroes the KV cache. */
int32_t alice_model_position(const alice_model* m, uint32_t* pos);
int32_t alice_model_vocab_size(const alice_model* m, uint32_t* vocab);
int32_t alice_model_rollback_to(alice_model* m, uint32_t pos);
int32_t alice_model_reset(alice_model* m);
/* Write / read KV rows of one layer, layout [pos][num_kv_heads * head_dim] as KvCache (src/llama3.rs:4731),
 * and set the position: used to start from a pre-filled context. */
int32_t alice_model_kv_write(alice_model* m, uint32_t layer, uint32_t pos0, uint32_t npos, const float* k, const float* v);
int32_t alice_model_kv_read(alice_model* m, uint32_t layer, uint32_t pos0, uint32_t npos, float* k, float* v);
int32_t alice_model_set_position(alice_model* m, uint32_t pos);

/* ---- no-allocation variant ---------------------------------------------------------------- */
/* Has no counterpart in the reference. alice_matvec_preq for Q1_0 / Q2_0 weights needs an f32 copy
 * of the Q8_K input and takes it from engine scratch obtained with cudaMalloc. This variant is for
 * callers that cannot allocate: a process whose HBM is entirely owned by its own pool (so cudaMalloc
 * would fail), or a decode thread that must not trigger the device-wide synchronisation cudaMalloc /
 * cudaFree imply. The f32 scratch is a fixed array inside the library image instead:
 * ALICE_NOALLOC_MAX_FLOATS floats (256 KiB) resident on every GPU that loads the library, for the
 * life of the process. batch * cols beyond that limit is rejected with ALICE_E_SHAPE; weights other
 * than Q1_0 / Q2_0 with ALICE_E_UNSUPPORTED. The call itself performs no cudaMalloc / cudaFree and
 * calls no allocating library routine. The first call on a device looks up the address of that
 * device's copy of the array (cudaGetSymbolAddress); make that first call before starting any stream
 * capture. Warm-up: with CUDA's lazy module loading the FIRST call per device and weight shape still makes the
 * driver take device memory - the array is materialised by that first address look-up, and each kernel instance's
 * code is loaded at its first launch (so is the opt-in shared-memory attribute). A process that hands all HBM to
 * its own pool must therefore make one call per shape it will use BEFORE the pool takes the memory (or run with
 * CUDA_MODULE_LOADING=EAGER); calls after that warm-up leave the device's free memory unchanged, which the test
 * suite checks with cudaMemGetInfo. It also uses the activation digit table scratch of an earlier alice_matvec /
 * alice_matvec_preq call on the engine when one is there and large enough, and never creates it. All calls share
 * the one array and it keeps the previous call's contents (each call
 * rewrites every element it reads, so nothing needs clearing); two calls whose GPU work overlaps -
 * different streams or engines on one device - race on it. Results equal alice_matvec_preq's. */
#define ALICE_NOALLOC_MAX_FLOATS 65536
int32_t alice_matvec_preq_noalloc(alice_engine* e, const alice_weights* w, const alice_q8k* q, alice_buf* y);

/* ---- host-pointer convenience (the gguf.rs-level signatures) ------------------------------- */
/* quantized_matvec(input, data, qtype, rows, cols, output) (src/gguf.rs:4214): uploads, runs on
 * device 0 through a process-wide engine, reads back. */
int32_t alice_matvec_host(uint32_t ggml_type, const uint8_t* data, size_t nbytes, uint32_t rows, uint32_t cols,
                          const float* x, float* y);
/* dequantize_weight_row(data, qtype, out) (src/gguf.rs:6168) for n_out = whole blocks of one row. */
int32_t alice_dequantize_host(uint32_t ggml_type, const uint8_t* data, size_t nbytes, float* out, size_t n_out);

#ifdef __cplusplus
}
#endif
#endif /* ALICE_CUDA_H */
