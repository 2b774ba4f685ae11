// Device-resident Llama-style decode model over the streaming matvec (alice_model_* of
// include/alice_cuda.h): the GpuModel of ALICE-LLM src/gpu.rs:2348 with the arithmetic of the CPU
// forward (src/llama3.rs:13632-13687, 14167-14613).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "abi_internal.cuh"
#include "attn_body.cuh"
#include "glue.cuh"
#include "tp.cuh"

using namespace alice;

struct alice_model {
    alice_engine* e = nullptr;
    alice_model_config cfg{};
    struct Layer {
        WeightDesc q, k, v, o, gate, up, down;
        float* attn_norm = nullptr;
        float* ffn_norm = nullptr;
    };
    std::vector<Layer> layers;
    WeightDesc emb{}, out{};
    float* out_norm = nullptr;
    // activations, each for up to MAX_BATCH tokens: [k][dim]
    float *hidden = nullptr, *qkv = nullptr, *attn_out = nullptr, *ffn_h = nullptr, *logits = nullptr;
    float *kcache = nullptr, *vcache = nullptr;  // [layer][max_seq][kv_dim]
    float* attn_part = nullptr;
    float* rope_freq = nullptr;  // 1 / theta^(2j / head_dim), j < 64, computed on the host (libm powf, as the CPU path)
    float* rope_tab = nullptr;   // [k][(sin, cos) per rotation pair] at the current positions, rewritten every step
    // Prepared forms of the vectors the matvecs read (csrc/publish.cuh), written once by the kernel that produced the
    // vector: Q8_K blocks for K-quant consumers, f32 (normalised) for the others
    uint8_t *hid_q8 = nullptr, *attn_q8 = nullptr, *ffn_q8 = nullptr;
    float* hid_xn = nullptr;
    uint8_t* prep = nullptr;            // scratch of the bit-plane kernels: the activation digit table of the current input
    size_t prep_bytes = 0;
    unsigned int* attn_tickets = nullptr;
    unsigned long long* argmax_key = nullptr;
    uint32_t nsplit = 1;
    // tensor parallel (engine's group): every projection holds rows [r*R/n, (r+1)*R/n); l* are the local sizes
    uint32_t tp_n = 1, tp_r = 0, lq = 0, lkv = 0, lH = 0, lF = 0, lV = 0;
    unsigned long long* argmax_keys = nullptr;   // one packed maximum per rank (argmax_key = &argmax_keys[tp_r])
    // Exchange region (tensor parallel): hidden | attn_out | ffn_h | logits | keys | flags | epoch in ONE allocation,
    // so one IPC handle maps all of it into the peers. peer_base[p] = that region of the p-th other rank.
    uint8_t* xchg = nullptr;
    size_t xchg_bytes = 0;
    unsigned int* flags = nullptr;      // arrival counters, one per op with an exchanged output (4 per layer + head)
    unsigned int* epoch = nullptr;      // decode steps completed
    bool peer_mode = false;             // peers connected: rows are pushed by the kernels, no collective calls
    uint32_t npeers = 0;
    uint32_t peer_rank[7] = {};
    uint8_t* peer_base[7] = {};
    // device-side state: position, current tokens, tokens chosen per position
    int *d_pos = nullptr, *d_token = nullptr, *d_trace = nullptr;
    uint32_t pos = 0;  // host mirror of *d_pos
    cudaGraphExec_t graph_greedy = nullptr;
    bool graph_tried = false;
    std::vector<void*> owned;
};

namespace {

#define MCU(call)                                                       \
    do {                                                                \
        cudaError_t err__ = (call);                                     \
        if (err__ != cudaSuccess) return alice_cuda_fail(err__, #call); \
    } while (0)

template <class T>
int dev_alloc(alice_model* m, T** p, size_t n) {
    void* q = nullptr;
    cudaError_t err = cudaMalloc(&q, std::max<size_t>(n, 1) * sizeof(T));
    if (err != cudaSuccess) return alice_cuda_fail(err, "alice_model_create: cudaMalloc");
    m->owned.push_back(q);
    *p = static_cast<T*>(q);
    return ALICE_OK;
}

int upload_norm(alice_model* m, float** dst, const float* host, size_t n) {
    int rc = dev_alloc(m, dst, n);
    if (rc) return rc;
    MCU(cudaMemcpy(*dst, host, n * sizeof(float), cudaMemcpyHostToDevice));
    return ALICE_OK;
}

int gemv(alice_model* m, GemvOp& op, const char* what) {
    op.wait_limit = m->e->wait_limit;
    op.prep = m->prep; op.prep_bytes = m->prep_bytes;
    const int rc = launch_stream_gemv_op(op, alice_cfg_of(m->e));
    if (rc == ALICE_OK) return rc;
    return alice_fail(rc, "alice_model: %s matvec failed (%d): %s", what, rc, cudaGetErrorString(cudaGetLastError()));
}

// The CPU model reaches q/k/v and gate/up through matvec_preq with the Q8_K-quantized norm output; for
// Q1_0 / Q2_0 weights that path turns the blocks back into f32 (src/gguf.rs:4593-4605), so those
// projections see the vector rounded to the Q8_K grid.
bool preq_roundtrip(const WeightDesc& w) { return w.fmt == WF_Q1_0 || w.fmt == WF_Q2_0; }

Q8KView q8_view(uint8_t* base, uint32_t n) {
    const Q8KLayout l = Q8KLayout::make(n / 256, MAX_BATCH);
    Q8KView v;
    v.qs = reinterpret_cast<const int8_t*>(base + l.qs_off);
    v.d = reinterpret_cast<const float*>(base + l.d_off);
    v.bsums = reinterpret_cast<const int16_t*>(base + l.bsums_off);
    v.nb = n / 256;
    return v;
}

// The bit-plane tensor-core kernels (Q1_0, Q2_0, ternary formats) take their input as a finished f32 vector in global
// memory, left there by the kernel that produced the vector; the K-quant kernels take Q8_K blocks that a one-CTA kernel
// prepares between producer and consumer; the rest (Q8_0) prepare the raw vector per CTA in their own prologue.
bool wants_prepared(const WeightDesc& w) {
    return (w.fmt == WF_Q1_0 || w.fmt == WF_Q2_0 || w.fmt == WF_TERNARY || w.fmt == WF_SPARSE_TERNARY) && w.cols % 4 == 0;
}
// Which prepared forms of a vector its consumers need from the kernel that produces it.
struct Need { bool q8 = false, xn = false, roundtrip = false; };
void need_of(Need& nd, const WeightDesc& w, bool via_preq) {
    if (!wants_prepared(w)) return;
    nd.xn = true;
    if (via_preq && preq_roundtrip(w)) nd.roundtrip = true;
}
void fill_dst(PublishDst& d, const Need& nd, uint8_t* q8_base, float* xn, uint32_t n) {
    d = PublishDst{};
    if (nd.q8) {
        const Q8KView v = q8_view(q8_base, n);
        d.qs = const_cast<int8_t*>(v.qs); d.d = const_cast<float*>(v.d); d.bsums = const_cast<int16_t*>(v.bsums);
    }
    if (nd.xn) { d.xn = xn; d.roundtrip = nd.roundtrip ? 1u : 0u; }
}

// Queues one decode step for `batch` consecutive tokens (read from d_token[0 .. batch)) on the engine's stream.
// With a tensor-parallel group every matvec computes this rank's rows into its slice of the full vector; the slices
// reach the other ranks either by an NCCL all-gather after the kernel, or (peer mode) by the kernel itself storing its
// rows into every peer's copy, with one flag per vector that a one-CTA kernel behind it raises on the peers and waits for
// here before it prepares the vector for the next op. Attention runs on the rank's own KV heads (its q, k, v rows), so
// only its output needs exchanging (it is the input of the output projection).
int enqueue_step(alice_model* m, uint32_t batch, bool greedy_feed) {
    const alice_model_config& c = m->cfg;
    cudaStream_t st = m->e->stream;
    const bool pdl = m->e->pdl;
    const uint32_t lq = m->lq, lkv = m->lkv, r = m->tp_r, L_n = c.num_layers, n = m->tp_n;
    const uint32_t H = c.hidden_dim, F = c.intermediate_dim, q_dim = c.num_heads * c.head_dim, V = c.vocab_size;
    const AttnShape shape{c.num_heads / n, c.num_kv_heads / n, c.head_dim};
    const bool peer = m->peer_mode, nccl = n > 1 && !peer;
    if (n > 1 && batch > 1) return alice_fail(ALICE_E_UNSUPPORTED, "alice_model: batches of tokens are single-GPU only");
    auto on_peer = [&](uint32_t p, const void* local) { return m->peer_base[p] + (reinterpret_cast<const uint8_t*>(local) - m->xchg); };
    int rc;

    // A whole-vector hand-over: what `consumers` need of vector `src` (length len), after rms_norm with norm_w (or none).
    // A one-CTA kernel behind the producing kernel runs it: on one GPU it prepares the vector; in NCCL mode it follows
    // the all-gather; in peer mode it first hands the pushed rows over (flags), then prepares the vector.
    auto vector_pub = [&](Publish& p, const float* src, uint32_t len, const float* norm_w, const Need& nd, uint8_t* q8_base, float* xn,
                          uint32_t flag_idx) {
        p = Publish{};
        p.mode = PUB_VECTOR; p.n = len; p.batch = batch; p.src = src; p.norm_w = norm_w; p.eps = c.eps;
        fill_dst(p.dst, nd, q8_base, xn, len);
        p.wait_limit = m->e->wait_limit;
        if (peer) {
            p.npeers = m->npeers; p.wait_flag = m->flags + flag_idx; p.epoch = m->epoch;
            for (uint32_t q = 0; q < m->npeers; q++) p.peer_flag[q] = reinterpret_cast<unsigned int*>(on_peer(q, m->flags + flag_idx));
        }
    };
    // after the kernel: NCCL gather + stand-alone preparation
    auto gather_then_publish = [&](float* vec, uint32_t floats_per_rank, Publish& p) -> int {
        if (n == 1) {
            // single GPU: a one-CTA kernel between producer and consumer (the consumer is its programmatic dependent
            // and streams weights meanwhile) instead of the last CTA of the producer doing the same as a serial tail
            if (p.dst.qs || p.dst.xn) { p.mode = PUB_VECTOR; MCU(launch_publish_vector(p, m->e->status, st, pdl)); }
            return ALICE_OK;
        }
        if (peer) {
            // pushed rows: the producing kernel has stored its rows into every peer's copy; a one-CTA kernel behind it
            // (which starts once that kernel and its stores are complete) raises this vector's counter on the peers,
            // waits (bounded) for theirs, and then prepares the now complete vector if the consumer wants it prepared.
            // (The same hand-over run by the producing kernel's last CTA was a serial tail of ~10 us per vector.)
            p.mode = PUB_VECTOR;
            MCU(launch_publish_vector(p, m->e->status, st, pdl));
            return ALICE_OK;
        }
        int g = tp_all_gather(m->e, vec, (size_t)floats_per_rank * sizeof(float));
        if (g) return g;
        if (p.dst.qs || p.dst.xn) { p.mode = PUB_VECTOR; MCU(launch_publish_vector(p, m->e->status, st, pdl)); }
        return ALICE_OK;
    };
    auto push_rows = [&](GemvOp& op, float* vec) {
        if (!peer) return;
        op.npeers = m->npeers;
        for (uint32_t q = 0; q < m->npeers; q++) op.peer_y[q] = reinterpret_cast<float*>(on_peer(q, vec));
    };
    // input of a matvec over `w` that reads the (normalised) hidden state: the prepared f32 vector for the bit-plane
    // tensor-core kernels; for the K-quants ONE shared copy of the Q8_K blocks (of all vectors of a batch), which a
    // one-CTA kernel prepares (norm + Q8_K) ahead of the matvec - the matvec is its programmatic dependent, so its CTAs
    // are resident and streaming weights meanwhile (measured on the 8B decode step: 2.23 ms per token this way, 2.28
    // with every CTA of the matvec normalising and quantizing the vector itself); else the raw vector plus the norm
    // weights, prepared per CTA. `fresh` = the hidden state has changed since the last such preparation.
    Q8KView hid_view = q8_view(m->hid_q8, H);
    auto hidden_input = [&](GemvOp& op, const WeightDesc& w, const float* norm_w, bool via_preq, bool fresh) -> int {
        op.batch = batch;
        if (wants_prepared(w)) { op.x = m->hid_xn; return ALICE_OK; }
        if (format_uses_q8k(w.fmt)) {
            if (fresh) {
                Publish p{};
                p.mode = PUB_VECTOR; p.n = H; p.batch = batch; p.src = m->hidden; p.norm_w = norm_w; p.eps = c.eps;
                Need nd; nd.q8 = true;
                fill_dst(p.dst, nd, m->hid_q8, nullptr, H);
                MCU(launch_publish_vector(p, m->e->status, st, pdl));
            }
            op.q8 = &hid_view;
            return ALICE_OK;
        }
        op.x = m->hidden; op.norm_w = norm_w; op.norm_eps = c.eps; op.q8k_roundtrip = via_preq && preq_roundtrip(w);
        return ALICE_OK;
    };

    // embedding + rotation table + hidden prepared for layer 0
    Need nd0;
    {
        const alice_model::Layer& L = m->layers[0];
        need_of(nd0, L.q, true); need_of(nd0, L.k, true); need_of(nd0, L.v, true);
    }
    EmbedArgs ea{};
    ea.table = m->emb.data; ea.tokens = m->d_token; ea.cols = H; ea.vocab = V; ea.batch = batch; ea.hidden = m->hidden;
    ea.pos = m->d_pos; ea.rope_freq = m->rope_freq; ea.rope_tab = m->rope_tab; ea.status = m->e->status;
    {
        Publish p;
        vector_pub(p, m->hidden, H, m->layers[0].attn_norm, nd0, m->hid_q8, m->hid_xn, 0);
        p.npeers = 0;     // every rank computes the whole embedding row itself
        if (nd0.xn) ea.pub = p;
    }
    MCU(launch_embed_q8_0(ea, st, pdl));

    for (uint32_t l = 0; l < L_n; l++) {
        const alice_model::Layer& L = m->layers[l];
        float* kc = m->kcache + (size_t)l * c.max_seq_len * lkv;
        float* vc = m->vcache + (size_t)l * c.max_seq_len * lkv;
        const uint32_t qkv_stride = lq + 2 * lkv;
        // attention norm (already applied: hid_q8 / hid_xn) + q, k, v projections (src/llama3.rs:14178-14217)
        if (L.q.fmt == L.k.fmt && L.q.fmt == L.v.fmt) {
            GemvOp op; Q8KView view;
            op.w[0] = &L.q; op.w[1] = &L.k; op.w[2] = &L.v; op.nw = 3;
            op.y_off[0] = 0; op.y_off[1] = lq; op.y_off[2] = lq + lkv;
            if ((rc = hidden_input(op, L.q, L.attn_norm, true, true))) return rc;
            op.y = m->qkv; op.y_stride = qkv_stride;
            if ((rc = gemv(m, op, "qkv"))) return rc;
        } else {   // mixed formats (e.g. V kept at higher precision): one launch each
            const WeightDesc* ws[3] = {&L.q, &L.k, &L.v};
            const uint32_t offs[3] = {0, lq, lq + lkv};
            for (int i = 0; i < 3; i++) {
                GemvOp op; Q8KView view;
                op.w[0] = ws[i];
                if ((rc = hidden_input(op, *ws[i], L.attn_norm, true, i == 0))) return rc;
                op.y = m->qkv + offs[i]; op.y_stride = qkv_stride;
                if ((rc = gemv(m, op, "q/k/v"))) return rc;
            }
        }
        // RoPE, KV append, GQA attention and the split combine in one launch (src/llama3.rs:14307-14362)
        const uint32_t group = shape.num_heads / shape.num_kv_heads;
        AttnArgs aa{};
        aa.qkv = m->qkv; aa.kcache = kc; aa.vcache = vc; aa.pos = m->d_pos; aa.shape = shape; aa.rope_tab = m->rope_tab;
        aa.neox = (int)c.neox_rope; aa.nsplit = m->nsplit; aa.part = m->attn_part; aa.tickets = m->attn_tickets;
        aa.attn_out = m->attn_out + (size_t)r * lq; aa.out_stride = q_dim; aa.status = m->e->status;
        Publish attn_pub{};
        // a K-quant output projection takes the attention output as Q8_K: written by the attention kernel itself when a
        // KV head's outputs are whole blocks, else quantized in the projection's own prologue
        const bool per_head_q8 = format_uses_q8k(L.o.fmt) && n == 1 && group % 2 == 0 && q_dim % 256 == 0;
        if (per_head_q8) {
            const Q8KView v = q8_view(m->attn_q8, q_dim);
            aa.q8.qs = const_cast<int8_t*>(v.qs); aa.q8.d = const_cast<float*>(v.d); aa.q8.bsums = const_cast<int16_t*>(v.bsums);
        }
        if (n > 1) {   // tensor parallel: the hand-over of the pushed rows
            Need none;
            vector_pub(attn_pub, m->attn_out, q_dim, nullptr, none, nullptr, nullptr, 4 * l + 0);
        }
        if (peer) {
            aa.npeers = m->npeers;
            for (uint32_t q = 0; q < m->npeers; q++) aa.peer_out[q] = reinterpret_cast<float*>(on_peer(q, m->attn_out)) + (size_t)r * lq;
        }
        MCU(launch_attention(aa, batch, st, pdl));
        if ((rc = gather_then_publish(m->attn_out, lq, attn_pub))) return rc;
        {   // output projection + residual (src/llama3.rs:14423, 14468); leaves hidden prepared for gate / up
            GemvOp op; Q8KView view; Publish p;
            op.w[0] = &L.o;
            if (per_head_q8) { view = q8_view(m->attn_q8, q_dim); op.q8 = &view; } else op.x = m->attn_out;
            op.batch = batch;
            op.resid = m->hidden; op.y = m->hidden; op.y_off[0] = r * m->lH; op.y_stride = H;
            Need nd; need_of(nd, L.gate, true);
            vector_pub(p, m->hidden, H, L.ffn_norm, nd, m->hid_q8, m->hid_xn, 4 * l + 1);
            push_rows(op, m->hidden);
            if ((rc = gemv(m, op, "o_proj"))) return rc;
            if ((rc = gather_then_publish(m->hidden, m->lH, p))) return rc;
        }
        {   // fused SwiGLU gate/up (src/llama3.rs:14497-14534)
            GemvOp op; Publish p;
            op.w[0] = &L.gate; op.up = &L.up;
            if ((rc = hidden_input(op, L.gate, L.ffn_norm, true, true))) return rc;
            op.y = m->ffn_h; op.y_off[0] = r * m->lF; op.y_stride = F;
            // a K-quant down projection takes the SwiGLU output as Q8_K: a small quantizer kernel follows (single GPU;
            // with a tensor-parallel group the down projection prepares the gathered vector in its own prologue)
            const bool down_q8 = n == 1 && format_uses_q8k(L.down.fmt);
            if (n > 1) {
                Need none;
                vector_pub(p, m->ffn_h, F, nullptr, none, nullptr, nullptr, 4 * l + 2);
            }
            push_rows(op, m->ffn_h);
            if ((rc = gemv(m, op, "gate/up"))) return rc;
            if (down_q8) { launch_quantize_q8k(m->ffn_h, F, batch, m->ffn_q8, st, pdl, MAX_BATCH); MCU(cudaGetLastError()); }
            if (n > 1 && (rc = gather_then_publish(m->ffn_h, m->lF, p))) return rc;
        }
        {   // down projection + residual (src/llama3.rs:14536-14555); leaves hidden prepared for the next layer / the head
            GemvOp op; Q8KView view; Publish p;
            op.w[0] = &L.down;
            if (n == 1 && format_uses_q8k(L.down.fmt)) { view = q8_view(m->ffn_q8, F); op.q8 = &view; } else op.x = m->ffn_h;
            op.batch = batch;
            op.resid = m->hidden; op.y = m->hidden; op.y_off[0] = r * m->lH; op.y_stride = H;
            Need nd;
            const float* norm_w;
            if (l + 1 < L_n) {
                const alice_model::Layer& N = m->layers[l + 1];
                need_of(nd, N.q, true); need_of(nd, N.k, true); need_of(nd, N.v, true);
                norm_w = N.attn_norm;
            } else {
                need_of(nd, m->out, false);
                norm_w = m->out_norm;
            }
            vector_pub(p, m->hidden, H, norm_w, nd, m->hid_q8, m->hid_xn, 4 * l + 3);
            push_rows(op, m->hidden);
            if ((rc = gemv(m, op, "down_proj"))) return rc;
            if ((rc = gather_then_publish(m->hidden, m->lH, p))) return rc;
        }
    }
    {   // output head on the prepared (normalised) hidden (src/llama3.rs:14590-14604)
        GemvOp op; Q8KView view; Publish p;
        op.w[0] = &m->out;
        if ((rc = hidden_input(op, m->out, m->out_norm, false, true))) return rc;
        op.y = m->logits; op.y_off[0] = r * m->lV; op.y_stride = V;
        if (batch == 1) op.argmax_key = m->argmax_key;   // greedy sampling: the head kernel leaves the packed maximum of its rows
        if (peer) {
            Need none;
            vector_pub(p, m->logits, V, nullptr, none, nullptr, nullptr, 4 * L_n);
            p.key_src = m->argmax_key;
            for (uint32_t q = 0; q < m->npeers; q++) p.peer_key[q] = reinterpret_cast<unsigned long long*>(on_peer(q, m->argmax_keys)) + r;
            push_rows(op, m->logits);
        }
        if ((rc = gemv(m, op, "output head"))) return rc;
        if (peer) MCU(launch_publish_vector(p, m->e->status, st, pdl));   // logits rows and the argmax key have been pushed: hand over
        if (nccl) {
            if ((rc = tp_all_gather(m->e, m->logits, (size_t)m->lV * sizeof(float)))) return rc;
            if ((rc = tp_all_gather(m->e, m->argmax_keys, sizeof(unsigned long long)))) return rc;
        }
    }
    MCU(launch_finish_step(m->argmax_keys, m->tp_n, m->d_token, m->d_pos, m->d_trace, greedy_feed ? 1 : 0, batch,
                           peer ? m->epoch : nullptr,   // the epoch counts steps whose rows were pushed (it is what the per-vector flags are compared with)
                           st, pdl));
    return ALICE_OK;
}

int check_room(const alice_model* m, uint32_t steps, const char* who) {
    if ((uint64_t)m->pos + steps > m->cfg.max_seq_len)
        return alice_fail(ALICE_E_SHAPE, "%s: position %u + %u steps exceeds max_seq_len %u", who, m->pos, steps,
                          m->cfg.max_seq_len);
    return ALICE_OK;
}

bool same_shape(const WeightDesc& w, uint32_t rows, uint32_t cols) { return w.rows == rows && w.cols == cols; }

}  // namespace

extern "C" {

int32_t alice_model_create(alice_engine* e, const alice_model_config* cfg, const alice_layer_weights* layers,
                           const alice_weights* embedding, const float* output_norm, const alice_weights* output,
                           alice_model** out) {
    const char* who = "alice_model_create";
    if (!e || !cfg || !layers || !embedding || !output_norm || !output || !out) return alice_fail(ALICE_E_INVALID, "%s: null argument", who);
    *out = nullptr;
    const alice_model_config& c = *cfg;
    if (!c.num_layers || !c.hidden_dim || !c.intermediate_dim || !c.num_heads || !c.num_kv_heads || !c.vocab_size || !c.max_seq_len)
        return alice_fail(ALICE_E_SHAPE, "%s: zero dimension in config", who);
    if (c.head_dim != 128) return alice_fail(ALICE_E_SHAPE, "%s: head_dim %u (the attention kernel is built for 128)", who, c.head_dim);
    if (c.num_heads % c.num_kv_heads) return alice_fail(ALICE_E_SHAPE, "%s: num_heads %% num_kv_heads != 0", who);
    const uint32_t group = c.num_heads / c.num_kv_heads;
    if (group != 1 && group != 2 && group != 4 && group != 5 && group != 8)
        return alice_fail(ALICE_E_SHAPE, "%s: %u query heads per KV head not supported (1, 2, 4, 5, 8)", who, group);
    const uint32_t q_dim = c.num_heads * c.head_dim, kv_dim = c.num_kv_heads * c.head_dim;
    // tensor-parallel group of the engine: the weight handles are this rank's row shards
    const uint32_t n = e->tp_world;
    if (c.num_kv_heads % n || c.hidden_dim % n || c.intermediate_dim % n || c.vocab_size % n)
        return alice_fail(ALICE_E_SHAPE, "%s: kv heads %u, hidden %u, ffn %u and vocab %u must all divide by the group size %u", who,
                          c.num_kv_heads, c.hidden_dim, c.intermediate_dim, c.vocab_size, n);
    const uint32_t lq = q_dim / n, lkv = kv_dim / n, lH = c.hidden_dim / n, lF = c.intermediate_dim / n, lV = c.vocab_size / n;
    if (embedding->d.fmt != WF_Q8_0 || !same_shape(embedding->d, c.vocab_size, c.hidden_dim))
        return alice_fail(ALICE_E_SHAPE, "%s: embedding must be Q8_0 [vocab x hidden]", who);
    if (!same_shape(output->d, lV, c.hidden_dim)) return alice_fail(ALICE_E_SHAPE, "%s: output head shape", who);
    MCU(cudaSetDevice(e->device));
    auto* m = new alice_model();
    m->e = e; m->cfg = c; m->emb = embedding->d; m->out = output->d;
    alice_engine_retain(e);
    m->tp_n = n; m->tp_r = e->tp_rank; m->lq = lq; m->lkv = lkv; m->lH = lH; m->lF = lF; m->lV = lV;
    int rc = ALICE_OK;
    for (uint32_t l = 0; l < c.num_layers && !rc; l++) {
        const alice_layer_weights& s = layers[l];
        if (!s.q || !s.k || !s.v || !s.o || !s.gate || !s.up || !s.down || !s.attn_norm || !s.ffn_norm) {
            rc = alice_fail(ALICE_E_INVALID, "%s: layer %u has a null weight", who, l);
            break;
        }
        if (!same_shape(s.q->d, lq, c.hidden_dim) || !same_shape(s.k->d, lkv, c.hidden_dim) ||
            !same_shape(s.v->d, lkv, c.hidden_dim) || !same_shape(s.o->d, lH, q_dim) ||
            !same_shape(s.gate->d, lF, c.hidden_dim) || !same_shape(s.up->d, lF, c.hidden_dim) ||
            !same_shape(s.down->d, lH, c.intermediate_dim) || s.gate->d.fmt != s.up->d.fmt) {
            rc = alice_fail(ALICE_E_SHAPE, "%s: layer %u weight shapes do not match the config (rows are this rank's 1/%u share)", who, l, n);
            break;
        }
        alice_model::Layer L;
        L.q = s.q->d; L.k = s.k->d; L.v = s.v->d; L.o = s.o->d; L.gate = s.gate->d; L.up = s.up->d; L.down = s.down->d;
        rc = upload_norm(m, &L.attn_norm, s.attn_norm, c.hidden_dim);
        if (!rc) rc = upload_norm(m, &L.ffn_norm, s.ffn_norm, c.hidden_dim);
        m->layers.push_back(L);
    }
    m->nsplit = std::max<uint32_t>(1, std::min<uint32_t>(64, (2 * (uint32_t)e->num_sms) / (c.num_kv_heads / n)));
    // (measured on the 8B and 27B decode steps: one wave of 2 CTAs per SM is the optimum; 18 or 64 splits cost 4-10 %)
    const size_t kv_elems = (size_t)c.num_layers * c.max_seq_len * lkv;
    if (!rc) rc = upload_norm(m, &m->out_norm, output_norm, c.hidden_dim);
    constexpr uint32_t B = MAX_BATCH;
    {   // the vectors other ranks need, the argmax keys and the hand-over counters share one allocation
        auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
        const size_t o_hidden = 0, o_attn = o_hidden + up((size_t)B * c.hidden_dim * 4), o_ffn = o_attn + up((size_t)B * q_dim * 4),
                     o_logits = o_ffn + up((size_t)B * c.intermediate_dim * 4), o_keys = o_logits + up((size_t)B * c.vocab_size * 4),
                     o_flags = o_keys + up(8 * 8), o_epoch = o_flags + up(((size_t)4 * c.num_layers + 2) * 4);
        m->xchg_bytes = o_epoch + 256;
        if (!rc) rc = dev_alloc(m, &m->xchg, m->xchg_bytes);
        if (!rc) {
            const cudaError_t zerr = cudaMemset(m->xchg, 0, m->xchg_bytes);
            if (zerr != cudaSuccess) rc = alice_cuda_fail(zerr, "alice_model_create: clearing the exchange region");
            m->hidden = reinterpret_cast<float*>(m->xchg + o_hidden);
            m->attn_out = reinterpret_cast<float*>(m->xchg + o_attn);
            m->ffn_h = reinterpret_cast<float*>(m->xchg + o_ffn);
            m->logits = reinterpret_cast<float*>(m->xchg + o_logits);
            m->argmax_keys = reinterpret_cast<unsigned long long*>(m->xchg + o_keys);
            m->argmax_key = m->argmax_keys + m->tp_r;
            m->flags = reinterpret_cast<unsigned int*>(m->xchg + o_flags);
            m->epoch = reinterpret_cast<unsigned int*>(m->xchg + o_epoch);
        }
    }
    if (!rc) rc = dev_alloc(m, &m->qkv, (size_t)B * (lq + 2 * lkv));
    if (!rc) rc = dev_alloc(m, &m->kcache, kv_elems);
    if (!rc) rc = dev_alloc(m, &m->vcache, kv_elems);
    if (!rc) rc = dev_alloc(m, &m->attn_part, (size_t)B * m->nsplit * (c.num_heads / n) * (c.head_dim + 4));
    if (!rc) rc = dev_alloc(m, &m->attn_tickets, (size_t)B * (c.num_kv_heads / n));
    if (!rc) rc = dev_alloc(m, &m->rope_tab, (size_t)B * 128);
    if (!rc) rc = dev_alloc(m, &m->rope_freq, 64);
    if (!rc) rc = dev_alloc(m, &m->hid_q8, Q8KLayout::make((c.hidden_dim + 255) / 256, B).total);
    if (!rc) rc = dev_alloc(m, &m->attn_q8, Q8KLayout::make((q_dim + 255) / 256, B).total);
    if (!rc) rc = dev_alloc(m, &m->ffn_q8, Q8KLayout::make((c.intermediate_dim + 255) / 256, B).total);
    if (!rc) rc = dev_alloc(m, &m->hid_xn, (size_t)B * c.hidden_dim);
    if (!rc) {
        m->prep_bytes = mma_prep_bytes(std::max({c.hidden_dim, c.intermediate_dim, q_dim}));
        rc = dev_alloc(m, &m->prep, m->prep_bytes);
    }
    if (!rc) rc = dev_alloc(m, &m->d_pos, 1);
    if (!rc) rc = dev_alloc(m, &m->d_token, B);
    if (!rc) rc = dev_alloc(m, &m->d_trace, c.max_seq_len);
    if (!rc) {
        // apply_rope's frequencies (src/llama3.rs:5323-5333): 1 / theta^(i / head_dim) for even i, in f32 with the host's powf
        float freq[64];
        for (int j = 0; j < 64; j++) freq[j] = 1.0f / std::pow(c.rope_theta, (float)(2 * j) / (float)c.head_dim);
        cudaError_t err = cudaMemcpy(m->rope_freq, freq, sizeof freq, cudaMemcpyHostToDevice);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->kcache, 0, kv_elems * 4, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->vcache, 0, kv_elems * 4, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->d_pos, 0, 4, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->attn_tickets, 0, (size_t)B * (c.num_kv_heads / n) * 4, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->d_token, 0, 4 * B, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->d_trace, 0, (size_t)c.max_seq_len * 4, e->stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(e->stream);
        if (err != cudaSuccess) rc = alice_cuda_fail(err, "alice_model_create: clearing state");
    }
    if (rc) { alice_model_destroy(m); return rc; }
    *out = m;
    return ALICE_OK;
}

int32_t alice_model_destroy(alice_model* m) {
    if (!m) return ALICE_OK;
    cudaSetDevice(m->e->device);
    if (!m->e->dead) cudaStreamSynchronize(m->e->stream);
    if (m->graph_greedy) cudaGraphExecDestroy(m->graph_greedy);
    for (uint32_t p = 0; p < m->npeers; p++) cudaIpcCloseMemHandle(m->peer_base[p]);
    for (void* p : m->owned) cudaFree(p);
    alice_engine_release(m->e);
    delete m;
    return ALICE_OK;
}

static int set_tokens(alice_model* m, const uint32_t* tokens, uint32_t n) {
    int t[MAX_BATCH];
    for (uint32_t k = 0; k < n; k++) {
        if (tokens[k] >= m->cfg.vocab_size) return alice_fail(ALICE_E_INVALID, "alice_model: token %u >= vocab %u", tokens[k], m->cfg.vocab_size);
        t[k] = (int)tokens[k];
    }
    MCU(cudaMemcpyAsync(m->d_token, t, 4 * n, cudaMemcpyHostToDevice, m->e->stream));
    MCU(cudaStreamSynchronize(m->e->stream));  // `t` lives on this stack frame
    return ALICE_OK;
}
static int set_token(alice_model* m, uint32_t token) { return set_tokens(m, &token, 1); }

int32_t alice_model_forward(alice_model* m, uint32_t token) {
    if (!m) return alice_fail(ALICE_E_INVALID, "alice_model_forward: null model");
    MCU(cudaSetDevice(m->e->device));
    int rc = check_room(m, 1, "alice_model_forward");
    if (!rc) rc = set_token(m, token);
    if (!rc) rc = enqueue_step(m, 1, false);
    if (!rc) m->pos += 1;
    return rc;
}

int32_t alice_model_forward_batch(alice_model* m, const uint32_t* tokens, uint32_t n) {
    const char* who = "alice_model_forward_batch";
    if (!m || !tokens) return alice_fail(ALICE_E_INVALID, "%s: null argument", who);
    if (n == 0 || n > (uint32_t)MAX_BATCH) return alice_fail(ALICE_E_SHAPE, "%s: %u tokens outside 1..%d", who, n, MAX_BATCH);
    MCU(cudaSetDevice(m->e->device));
    int rc = check_room(m, n, who);
    if (!rc) rc = set_tokens(m, tokens, n);
    if (!rc) rc = enqueue_step(m, n, false);
    if (!rc) m->pos += n;
    return rc;
}

int32_t alice_model_forward_batch_read(alice_model* m, const uint32_t* tokens, uint32_t n, float* logits) {
    if (!logits) return alice_fail(ALICE_E_INVALID, "alice_model_forward_batch_read: null argument");
    int rc = alice_model_forward_batch(m, tokens, n);
    if (rc) return rc;
    MCU(cudaMemcpyAsync(logits, m->logits, (size_t)n * m->cfg.vocab_size * 4, cudaMemcpyDeviceToHost, m->e->stream));
    MCU(cudaStreamSynchronize(m->e->stream));
    return alice_sync(m->e);
}

int32_t alice_model_read_logits(alice_model* m, float* logits) {
    if (!m || !logits) return alice_fail(ALICE_E_INVALID, "alice_model_read_logits: null argument");
    MCU(cudaMemcpyAsync(logits, m->logits, (size_t)m->cfg.vocab_size * 4, cudaMemcpyDeviceToHost, m->e->stream));
    MCU(cudaStreamSynchronize(m->e->stream));
    return alice_sync(m->e);
}

int32_t alice_model_forward_read(alice_model* m, uint32_t token, float* logits) {
    int rc = alice_model_forward(m, token);
    if (rc) return rc;
    return alice_model_read_logits(m, logits);
}

int32_t alice_model_decode_greedy(alice_model* m, uint32_t first_token, uint32_t n, uint32_t* out_tokens) {
    const char* who = "alice_model_decode_greedy";
    if (!m || (!out_tokens && n)) return alice_fail(ALICE_E_INVALID, "%s: null argument", who);
    if (n == 0) return ALICE_OK;
    MCU(cudaSetDevice(m->e->device));
    int rc = check_room(m, n, who);
    if (!rc) rc = set_token(m, first_token);
    if (rc) return rc;
    cudaStream_t st = m->e->stream;
    const uint32_t pos0 = m->pos;
    if (!m->graph_tried) {
        // Capture one step (every kernel reads position and token from device memory) and replay it.
        m->graph_tried = true;
        rc = enqueue_step(m, 1, true);   // eager first step: also sets per-kernel attributes outside capture
        if (rc) return rc;
        m->pos += 1;
        cudaGraph_t g = nullptr;
        if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            const int crc = enqueue_step(m, 1, true);
            cudaError_t err = cudaStreamEndCapture(st, &g);
            if (crc == ALICE_OK && err == cudaSuccess && g) {
                if (cudaGraphInstantiate(&m->graph_greedy, g, 0) != cudaSuccess) m->graph_greedy = nullptr;
            }
            if (g) cudaGraphDestroy(g);
            cudaGetLastError();  // a failed capture only means the steps are launched one by one
        }
    }
    while (m->pos < pos0 + n) {
        if (m->graph_greedy) {
            MCU(cudaGraphLaunch(m->graph_greedy, st));
        } else {
            rc = enqueue_step(m, 1, true);
            if (rc) return rc;
        }
        m->pos += 1;
    }
    static_assert(sizeof(uint32_t) == sizeof(int), "token trace is copied as 32-bit words");
    MCU(cudaMemcpyAsync(out_tokens, m->d_trace + pos0, (size_t)n * 4, cudaMemcpyDeviceToHost, st));
    MCU(cudaStreamSynchronize(st));
    return alice_sync(m->e);
}

int32_t alice_model_tp_export(alice_model* m, void* out, size_t nbytes) {
    if (!m || !out) return alice_fail(ALICE_E_INVALID, "alice_model_tp_export: null argument");
    if (nbytes < sizeof(cudaIpcMemHandle_t)) return alice_fail(ALICE_E_INVALID, "alice_model_tp_export: need %zu bytes", sizeof(cudaIpcMemHandle_t));
    MCU(cudaSetDevice(m->e->device));
    cudaIpcMemHandle_t h;
    MCU(cudaIpcGetMemHandle(&h, m->xchg));
    memset(out, 0, nbytes);
    memcpy(out, &h, sizeof(h));
    return ALICE_OK;
}

int32_t alice_model_tp_connect(alice_model* m, const void* handles, size_t bytes_per_handle) {
    if (!m || !handles) return alice_fail(ALICE_E_INVALID, "alice_model_tp_connect: null argument");
    if (bytes_per_handle < sizeof(cudaIpcMemHandle_t)) return alice_fail(ALICE_E_INVALID, "alice_model_tp_connect: handles of %zu bytes, need %zu", bytes_per_handle, sizeof(cudaIpcMemHandle_t));
    if (m->peer_mode) return alice_fail(ALICE_E_INVALID, "alice_model_tp_connect: already connected");
    if (m->tp_n <= 1) return ALICE_OK;
    MCU(cudaSetDevice(m->e->device));
    MCU(cudaStreamSynchronize(m->e->stream));
    uint32_t k = 0;
    for (uint32_t p = 0; p < m->tp_n; p++) {
        if (p == m->tp_r) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)p * bytes_per_handle, sizeof(h));
        void* base = nullptr;
        const cudaError_t err = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
        if (err != cudaSuccess) {
            for (uint32_t q = 0; q < k; q++) cudaIpcCloseMemHandle(m->peer_base[q]);
            return alice_cuda_fail(err, "alice_model_tp_connect: cudaIpcOpenMemHandle (are the GPUs peer-accessible?)");
        }
        m->peer_base[k] = static_cast<uint8_t*>(base);
        m->peer_rank[k] = p;
        k++;
    }
    m->npeers = k;
    m->peer_mode = true;
    if (m->graph_greedy) { cudaGraphExecDestroy(m->graph_greedy); m->graph_greedy = nullptr; }
    m->graph_tried = false;   // a step captured earlier holds the collective calls
    return ALICE_OK;
}

int32_t alice_model_position(const alice_model* m, uint32_t* pos) {
    if (!m || !pos) return alice_fail(ALICE_E_INVALID, "alice_model_position: null argument");
    *pos = m->pos;
    return ALICE_OK;
}

int32_t alice_model_vocab_size(const alice_model* m, uint32_t* vocab) {
    if (!m || !vocab) return alice_fail(ALICE_E_INVALID, "alice_model_vocab_size: null argument");
    *vocab = m->cfg.vocab_size;
    return ALICE_OK;
}

int32_t alice_model_set_position(alice_model* m, uint32_t pos) {
    if (!m) return alice_fail(ALICE_E_INVALID, "alice_model_set_position: null model");
    if (pos > m->cfg.max_seq_len) return alice_fail(ALICE_E_SHAPE, "alice_model_set_position: %u > max_seq_len %u", pos, m->cfg.max_seq_len);
    const int p = (int)pos;
    MCU(cudaSetDevice(m->e->device));
    MCU(cudaMemcpyAsync(m->d_pos, &p, 4, cudaMemcpyHostToDevice, m->e->stream));
    MCU(cudaStreamSynchronize(m->e->stream));
    m->pos = pos;
    return ALICE_OK;
}

int32_t alice_model_rollback_to(alice_model* m, uint32_t pos) {
    if (!m) return alice_fail(ALICE_E_INVALID, "alice_model_rollback_to: null model");
    if (pos > m->pos) return ALICE_OK;  // only ever lowers the counter (src/gpu.rs:5645-5652)
    return alice_model_set_position(m, pos);
}

int32_t alice_model_reset(alice_model* m) {
    if (!m) return alice_fail(ALICE_E_INVALID, "alice_model_reset: null model");
    const size_t kv_bytes = (size_t)m->cfg.num_layers * m->cfg.max_seq_len * m->lkv * 4;
    MCU(cudaSetDevice(m->e->device));
    MCU(cudaMemsetAsync(m->kcache, 0, kv_bytes, m->e->stream));
    MCU(cudaMemsetAsync(m->vcache, 0, kv_bytes, m->e->stream));
    return alice_model_set_position(m, 0);
}

static int kv_copy(alice_model* m, uint32_t layer, uint32_t pos0, uint32_t npos, float* k, float* v, bool to_device) {
    if (!m || !k || !v) return alice_fail(ALICE_E_INVALID, "alice_model_kv: null argument");
    const alice_model_config& c = m->cfg;
    if (layer >= c.num_layers || (uint64_t)pos0 + npos > c.max_seq_len) return alice_fail(ALICE_E_SHAPE, "alice_model_kv: layer / position out of range");
    const size_t kv_dim = m->lkv;   // this rank's KV heads
    const size_t off = ((size_t)layer * c.max_seq_len + pos0) * kv_dim, bytes = (size_t)npos * kv_dim * 4;
    cudaStream_t st = m->e->stream;
    MCU(cudaSetDevice(m->e->device));
    if (to_device) {
        MCU(cudaMemcpyAsync(m->kcache + off, k, bytes, cudaMemcpyHostToDevice, st));
        MCU(cudaMemcpyAsync(m->vcache + off, v, bytes, cudaMemcpyHostToDevice, st));
    } else {
        MCU(cudaMemcpyAsync(k, m->kcache + off, bytes, cudaMemcpyDeviceToHost, st));
        MCU(cudaMemcpyAsync(v, m->vcache + off, bytes, cudaMemcpyDeviceToHost, st));
    }
    MCU(cudaStreamSynchronize(st));
    return ALICE_OK;
}

int32_t alice_model_kv_write(alice_model* m, uint32_t layer, uint32_t pos0, uint32_t npos, const float* k, const float* v) {
    return kv_copy(m, layer, pos0, npos, const_cast<float*>(k), const_cast<float*>(v), true);
}

int32_t alice_model_kv_read(alice_model* m, uint32_t layer, uint32_t pos0, uint32_t npos, float* k, float* v) {
    return kv_copy(m, layer, pos0, npos, k, v, false);
}

}  // extern "C"
