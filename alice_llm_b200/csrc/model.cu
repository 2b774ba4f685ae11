// Device-resident Llama-style decode model over the streaming matvec (alice_model_* of
// include/alice_cuda.h): the GpuModel of ALICE-LLM src/gpu.rs:2348 with the arithmetic of the CPU
// forward (src/llama3.rs:13632-13687, 14167-14613).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "abi_internal.cuh"
#include "attn_body.cuh"
#include "glue.cuh"
#include "step_kernel.cuh"
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
    // activations
    float *hidden = nullptr, *qkv = nullptr, *attn_out = nullptr, *ffn_h = nullptr, *logits = nullptr;
    float *kcache = nullptr, *vcache = nullptr;  // [layer][max_seq][kv_dim]
    float* attn_part = nullptr;
    float* rope_tab = nullptr;   // (sin, cos) per rotation pair at the current position, rewritten every step
    // Q8_K copy of the attention output, written by the attention kernel for K-quant output projections (single GPU)
    uint8_t* attn_q8 = nullptr;
    Q8KLayout attn_q8_lay{};
    bool attn_q8_ok = false;
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
    unsigned int* flags = nullptr;      // arrival counters, one per op that has an exchanged output (4 per layer + head + keys)
    unsigned int* epoch = nullptr;      // decode steps completed
    uint2 *hidden_ll = nullptr, *attn_ll = nullptr, *ffn_ll = nullptr;   // tagged forms of the per-layer vectors (peer mode)
    bool peer_mode = false;             // peers connected: rows are pushed by the kernels, no collective calls
    uint32_t npeers = 0;
    uint32_t peer_rank[7] = {};
    uint8_t* peer_base[7] = {};
    // device-side state: position, current token, tokens chosen per position
    int *d_pos = nullptr, *d_token = nullptr, *d_trace = nullptr;
    uint32_t pos = 0;  // host mirror of *d_pos
    cudaGraphExec_t graph_greedy = nullptr;
    bool graph_tried = false;
    // whole-step kernel (csrc/step_kernel.cu): op table on the device, its launch geometry
    bool use_step_kernel = false, step_ready = false, step_tried = false;
    StepOp* d_ops = nullptr;
    uint32_t step_nops = 0, step_grid = 0, step_stride = 0, step_aux_off = 0;
    size_t step_smem = 0;
    std::vector<uint32_t> step_types;   // StepOpType per op (host copy, for the debug profile)
    unsigned int* d_barrier = nullptr;
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

int gemv(alice_model* m, const GemvOp& op, const char* what) {
    const int rc = launch_stream_gemv_op(op, alice_cfg_of(m->e));
    if (rc == ALICE_OK) return rc;
    return alice_fail(rc, "alice_model: %s matvec failed (%d): %s", what, rc, cudaGetErrorString(cudaGetLastError()));
}

// The CPU model reaches q/k/v and gate/up through matvec_preq with the Q8_K-quantized norm output; for
// Q1_0 / Q2_0 weights that path turns the blocks back into f32 (src/gguf.rs:4593-4605), so those
// projections see the vector rounded to the Q8_K grid.
bool preq_roundtrip(const WeightDesc& w) { return w.fmt == WF_Q1_0 || w.fmt == WF_Q2_0; }

// In-place all-gather of a row-sharded activation vector (no-op for a single GPU).
int gather(alice_model* m, float* base, uint32_t floats_per_rank) {
    return tp_all_gather(m->e, base, (size_t)floats_per_rank * sizeof(float));
}

// Queues one decode step on the engine's stream. The token is read from *d_token.
// With a tensor-parallel group every matvec computes this rank's rows into its slice of the full vector
// and an all-gather completes it on every rank; attention runs on the rank's own KV heads (its q, k, v
// rows), so only its output needs gathering (it is the input of the output projection).
int enqueue_step(alice_model* m, bool greedy_feed) {
    const alice_model_config& c = m->cfg;
    cudaStream_t st = m->e->stream;
    const bool pdl = m->e->pdl;
    const uint32_t lq = m->lq, lkv = m->lkv, r = m->tp_r, L_n = c.num_layers;
    const AttnShape shape{c.num_heads / m->tp_n, c.num_kv_heads / m->tp_n, c.head_dim};
    const bool peer = m->peer_mode;
    // Peer mode. The per-layer vectors (hidden, attention output, SwiGLU output) travel as tagged vectors: the kernel
    // that produces rows stores (value, tag) into this GPU's copy and every peer's, the kernel that consumes the vector
    // polls for the tag of the version it wants - no fence, no counter. hidden is rewritten 2 L + 1 times per step
    // (embedding, then o and down of every layer), the other two L times. The logits and the argmax keys (once per
    // step) use plain stores + an arrival counter instead.
    // Why nobody overwrites a version that is still being read: a peer's next write into vector V is the epilogue of a
    // matvec whose input needs rows this GPU produces only AFTER all its CTAs have read V (hidden -> peers' down needs
    // this GPU's complete SwiGLU slice, whose CTAs read hidden in their prologue; attention output -> peers' next
    // attention needs this GPU's o / SwiGLU / down rows; SwiGLU output -> peers' next SwiGLU needs this GPU's down rows).
    const uint32_t hid_n = 2 * L_n + 1;
    auto on_peer = [&](uint32_t p, const void* local) { return m->peer_base[p] + (reinterpret_cast<const uint8_t*>(local) - m->xchg); };
    auto push_ll = [&](GemvOp& op, PeerPush& pp, uint2* vec, uint32_t seq, uint32_t n) {
        pp.npeers = m->npeers;
        for (uint32_t p = 0; p < m->npeers; p++) pp.y_ll[p] = reinterpret_cast<uint2*>(on_peer(p, vec));
        op.push = &pp; op.y_ll = vec; op.y_seq = seq; op.y_n = n; op.epoch = m->epoch;
    };
    auto read_ll = [&](GemvOp& op, const uint2* vec, uint32_t seq, uint32_t n) { op.x_ll = vec; op.x_seq = seq; op.x_n = n; op.epoch = m->epoch; };
    const uint32_t f_logits = 4 * L_n, f_keys = f_logits + 1;
    int rc;
    EmbedTag et;
    if (peer) { et.hidden_ll = m->hidden_ll; et.epoch = m->epoch; et.tag_n = hid_n; }
    MCU(launch_embed_q8_0(m->emb.data, m->d_token, c.hidden_dim, c.vocab_size, m->hidden, m->d_pos, c.rope_theta, m->rope_tab, et, st, pdl));
    for (uint32_t l = 0; l < L_n; l++) {
        const alice_model::Layer& L = m->layers[l];
        float* kc = m->kcache + (size_t)l * c.max_seq_len * lkv;
        float* vc = m->vcache + (size_t)l * c.max_seq_len * lkv;
        if (L.q.fmt == L.k.fmt && L.q.fmt == L.v.fmt) {
            // attention norm + q, k, v projections in one launch (src/llama3.rs:14178-14217)
            GemvOp op;
            op.w[0] = &L.q; op.w[1] = &L.k; op.w[2] = &L.v; op.nw = 3;
            op.y_off[0] = 0; op.y_off[1] = lq; op.y_off[2] = lq + lkv;
            op.x = m->hidden; op.norm_w = L.attn_norm; op.norm_eps = c.eps; op.y = m->qkv;
            op.q8k_roundtrip = preq_roundtrip(L.q);
            if (peer) read_ll(op, m->hidden_ll, 2 * l, hid_n);
            if ((rc = gemv(m, op, "qkv"))) return rc;
        } else {   // mixed formats (e.g. V kept at higher precision): one launch each, same norm prologue
            const WeightDesc* ws[3] = {&L.q, &L.k, &L.v};
            const uint32_t offs[3] = {0, lq, lq + lkv};
            for (int i = 0; i < 3; i++) {
                GemvOp op;
                op.w[0] = ws[i]; op.x = m->hidden; op.norm_w = L.attn_norm; op.norm_eps = c.eps;
                op.q8k_roundtrip = preq_roundtrip(*ws[i]);
                op.y = m->qkv + offs[i];
                if (peer) read_ll(op, m->hidden_ll, 2 * l, hid_n);
                if ((rc = gemv(m, op, "q/k/v"))) return rc;
            }
        }
        // RoPE, KV append, GQA attention and the split combine in one launch (src/llama3.rs:14307-14362)
        AttnPeers ap;
        if (peer) {
            ap.npeers = m->npeers;
            ap.out_ll = m->attn_ll + (size_t)r * lq; ap.epoch = m->epoch; ap.tag_seq = l; ap.tag_n = L_n;
            for (uint32_t p = 0; p < m->npeers; p++) ap.peer_ll[p] = reinterpret_cast<uint2*>(on_peer(p, m->attn_ll)) + (size_t)r * lq;
        }
        // a K-quant output projection takes the attention output already in Q8_K (written by the attention kernel)
        const bool o_preq = m->attn_q8_ok && !peer && (L.o.fmt == WF_Q4_K || L.o.fmt == WF_Q5_K || L.o.fmt == WF_Q6_K);
        AttnQ8Out aq;
        Q8KView o_view{};
        if (o_preq) {
            aq.qs = reinterpret_cast<int8_t*>(m->attn_q8 + m->attn_q8_lay.qs_off);
            aq.d = reinterpret_cast<float*>(m->attn_q8 + m->attn_q8_lay.d_off);
            aq.bsums = reinterpret_cast<int16_t*>(m->attn_q8 + m->attn_q8_lay.bsums_off);
            o_view.qs = aq.qs; o_view.d = aq.d; o_view.bsums = aq.bsums; o_view.nb = (c.num_heads * c.head_dim) / 256;
        }
        MCU(launch_attention(m->qkv, kc, vc, m->d_pos, shape, m->rope_tab, (int)c.neox_rope, m->nsplit, m->attn_part,
                             m->attn_tickets, m->attn_out + (size_t)r * lq, ap, aq, st, pdl));
        if (!peer && (rc = gather(m, m->attn_out, lq))) return rc;
        {   // output projection + residual (src/llama3.rs:14423, 14468)
            GemvOp op; PeerPush pp;
            op.w[0] = &L.o; op.x = m->attn_out; op.resid = m->hidden; op.y = m->hidden; op.y_off[0] = r * m->lH;
            if (o_preq) { op.q8 = &o_view; op.x = nullptr; }
            if (peer) { read_ll(op, m->attn_ll, l, L_n); op.resid_ll = m->hidden_ll; push_ll(op, pp, m->hidden_ll, 2 * l + 1, hid_n); }
            if ((rc = gemv(m, op, "o_proj"))) return rc;
            if (!peer && (rc = gather(m, m->hidden, m->lH))) return rc;
        }
        {   // FFN norm + fused SwiGLU gate/up (src/llama3.rs:14497-14534)
            GemvOp op; PeerPush pp;
            op.w[0] = &L.gate; op.up = &L.up; op.x = m->hidden; op.norm_w = L.ffn_norm; op.norm_eps = c.eps;
            op.q8k_roundtrip = preq_roundtrip(L.gate);
            op.y = m->ffn_h; op.y_off[0] = r * m->lF;
            if (peer) { read_ll(op, m->hidden_ll, 2 * l + 1, hid_n); push_ll(op, pp, m->ffn_ll, l, L_n); }
            if ((rc = gemv(m, op, "gate/up"))) return rc;
            if (!peer && (rc = gather(m, m->ffn_h, m->lF))) return rc;
        }
        {   // down projection + residual (src/llama3.rs:14536-14555)
            GemvOp op; PeerPush pp;
            op.w[0] = &L.down; op.x = m->ffn_h; op.resid = m->hidden; op.y = m->hidden; op.y_off[0] = r * m->lH;
            if (peer) { read_ll(op, m->ffn_ll, l, L_n); op.resid_ll = m->hidden_ll; push_ll(op, pp, m->hidden_ll, 2 * l + 2, hid_n); }
            if ((rc = gemv(m, op, "down_proj"))) return rc;
            if (!peer && (rc = gather(m, m->hidden, m->lH))) return rc;
        }
    }
    StepPeers sp;
    {   // output norm + head (src/llama3.rs:14590-14604)
        GemvOp op; PeerPush pp;
        op.w[0] = &m->out; op.x = m->hidden; op.norm_w = m->out_norm; op.norm_eps = c.eps; op.y = m->logits;
        op.y_off[0] = r * m->lV;
        op.argmax_key = m->argmax_key;   // greedy sampling: the head kernel leaves the packed maximum of its rows
        uint32_t head_grid = 0;
        if (peer) {
            read_ll(op, m->hidden_ll, 2 * L_n, hid_n);
            pp.npeers = m->npeers;
            for (uint32_t p = 0; p < m->npeers; p++) {
                pp.y[p] = reinterpret_cast<float*>(on_peer(p, m->logits));
                pp.flag[p] = reinterpret_cast<unsigned int*>(on_peer(p, m->flags + f_logits));
            }
            op.push = &pp;
            const int prc = stream_gemv_final_grid(op, alice_cfg_of(m->e), &head_grid);
            if (prc) return alice_fail(prc, "alice_model: planning the output head failed (%d)", prc);
        }
        if ((rc = gemv(m, op, "output head"))) return rc;
        if (!peer) {
            if ((rc = gather(m, m->logits, m->lV))) return rc;
            if ((rc = tp_all_gather(m->e, m->argmax_keys, sizeof(unsigned long long)))) return rc;
        } else {
            sp.npeers = m->npeers; sp.rank = r;
            for (uint32_t p = 0; p < m->npeers; p++) {
                sp.keys[p] = reinterpret_cast<unsigned long long*>(on_peer(p, m->argmax_keys));
                sp.key_flag[p] = reinterpret_cast<unsigned int*>(on_peer(p, m->flags + f_keys));
            }
            sp.my_key_flag = m->flags + f_keys; sp.my_logits_flag = m->flags + f_logits; sp.logits_mult = m->npeers * head_grid;
            sp.epoch = m->epoch; sp.status = m->e->status;
        }
    }
    MCU(launch_finish_step(m->argmax_keys, m->tp_n, m->d_token, m->d_pos, m->d_trace, greedy_feed ? 1 : 0, sp, st, pdl));
    return ALICE_OK;
}

// The same ops as enqueue_step, as a device-resident list for the whole-step kernel. Leaves
// step_ready false (and the model on the one-launch-per-op path) when an op has no instance there.
static int step_skip(int why) {
    if (getenv("ALICE_DEBUG")) fprintf(stderr, "[alice] whole-step kernel not used (reason %d)\n", why);
    return ALICE_OK;
}

int build_step_ops(alice_model* m) {
    const alice_model_config& c = m->cfg;
    const uint32_t q_dim = c.num_heads * c.head_dim, kv_dim = c.num_kv_heads * c.head_dim;
    const AttnShape shape{c.num_heads, c.num_kv_heads, c.head_dim};
    const uint32_t group = c.num_heads / c.num_kv_heads;
    if (group != 1 && group != 2 && group != 4) return step_skip(1);
    if (m->tp_n > 1) return step_skip(9);   // the whole-step kernel has no collective stage
    std::vector<GemvOp> gops;
    std::vector<int> kind;   // -1 embed, -2 attention(layer), >= 0 index into gops
    std::vector<uint32_t> attn_layer;
    kind.push_back(-1);
    for (uint32_t l = 0; l < c.num_layers; l++) {
        const alice_model::Layer& L = m->layers[l];
        if (!(L.q.fmt == L.k.fmt && L.q.fmt == L.v.fmt)) return step_skip(2);
        GemvOp qkv; qkv.w[0] = &L.q; qkv.w[1] = &L.k; qkv.w[2] = &L.v; qkv.nw = 3;
        qkv.y_off[1] = q_dim; qkv.y_off[2] = q_dim + kv_dim;
        qkv.x = m->hidden; qkv.norm_w = L.attn_norm; qkv.norm_eps = c.eps; qkv.y = m->qkv;
        kind.push_back((int)gops.size()); gops.push_back(qkv);
        kind.push_back(-2); attn_layer.push_back(l);
        GemvOp o; o.w[0] = &L.o; o.x = m->attn_out; o.resid = m->hidden; o.y = m->hidden;
        kind.push_back((int)gops.size()); gops.push_back(o);
        GemvOp gu; gu.w[0] = &L.gate; gu.up = &L.up; gu.x = m->hidden; gu.norm_w = L.ffn_norm; gu.norm_eps = c.eps; gu.y = m->ffn_h;
        kind.push_back((int)gops.size()); gops.push_back(gu);
        GemvOp dn; dn.w[0] = &L.down; dn.x = m->ffn_h; dn.resid = m->hidden; dn.y = m->hidden;
        kind.push_back((int)gops.size()); gops.push_back(dn);
    }
    GemvOp head; head.w[0] = &m->out; head.x = m->hidden; head.norm_w = m->out_norm; head.norm_eps = c.eps;
    head.y = m->logits; head.argmax_key = m->argmax_key;
    kind.push_back((int)gops.size()); gops.push_back(head);

    const LaunchCfg cfg = alice_cfg_of(m->e);
    const uint32_t grid = 2u * (uint32_t)m->e->num_sms;
    // first pass: the auxiliary area (normalised input + in-kernel Q8_K, or the attention scratch)
    uint32_t aux = (uint32_t)((group == 4 ? sizeof(AttnSmem<4>) : group == 2 ? sizeof(AttnSmem<2>) : sizeof(AttnSmem<1>)) + 127) & ~127u;
    PlanLimits probe{2, 48 * 1024, grid};
    for (const GemvOp& g : gops) {
        StreamPlan pl;
        if (plan_stream_gemv(g, cfg, &probe, pl)) return step_skip(3);
        if (pl.kl > 2) return step_skip(4);
        aux = std::max(aux, pl.q8_bytes + pl.xn_bytes);
    }
    const uint32_t ops_bytes = 2 * (uint32_t)sizeof(StepOp);   // the consumers' descriptor double buffer, after the auxiliary area
    const uint32_t stride = ((STEP_SMEM_BUDGET - STREAM_HDR_BYTES - aux - ops_bytes) / 2) & ~127u;
    PlanLimits lim{2, stride, grid};
    const uint32_t aux_off = STREAM_HDR_BYTES + 2 * stride;
    std::vector<StepOp> ops;
    size_t ai = 0;
    for (int k : kind) {
        StepOp op{};
        if (k == -1) {
            op.type = SOP_EMBED; op.table = m->emb.data; op.hidden = m->hidden; op.cols = c.hidden_dim; op.vocab = c.vocab_size; op.theta = c.rope_theta; op.rope_tab = m->rope_tab;
        } else if (k == -2) {
            const uint32_t l = attn_layer[ai++];
            op.type = SOP_ATTN; op.qkv = m->qkv;
            op.kc = m->kcache + (size_t)l * c.max_seq_len * kv_dim; op.vc = m->vcache + (size_t)l * c.max_seq_len * kv_dim;
            op.part = m->attn_part; op.tickets = m->attn_tickets; op.attn_out = m->attn_out;
            op.shape = shape; op.rope_tab = m->rope_tab; op.neox = (int)c.neox_rope; op.nsplit = m->nsplit;
        } else {
            StreamPlan pl;
            if (plan_stream_gemv(gops[k], cfg, &lim, pl)) return step_skip(5);
            const int v = step_variant(gops[k].w[0]->fmt, pl.kl, pl.swiglu);
            if (v < 0) return step_skip(6);
            op.type = SOP_GEMV; op.variant = v; op.g = pl.args;
            op.g.xn_off = aux_off; op.g.q8_off = aux_off + pl.xn_bytes;
        }
        ops.push_back(op);
    }
    int per_sm = 0;
    const size_t smem = aux_off + aux + ops_bytes;
    if (decode_step_max_ctas_per_sm(smem, &per_sm) != cudaSuccess || per_sm < 2) { cudaGetLastError(); return step_skip(7); }
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, m->e->device);
    if (!coop) return step_skip(8);
    int rc = dev_alloc(m, &m->d_ops, ops.size());
    if (!rc) rc = dev_alloc(m, &m->d_barrier, 1);
    if (rc) return rc;
    MCU(cudaMemcpy(m->d_ops, ops.data(), ops.size() * sizeof(StepOp), cudaMemcpyHostToDevice));
    m->step_types.clear();
    for (const StepOp& o : ops) m->step_types.push_back(o.type);
    m->step_nops = (uint32_t)ops.size(); m->step_grid = grid; m->step_stride = stride; m->step_aux_off = aux_off;
    m->step_smem = smem; m->step_ready = true;
    return ALICE_OK;
}

// n decode steps in one cooperative launch of the whole-step kernel.
int run_step_kernel(alice_model* m, uint32_t n, bool greedy_feed) {
    cudaStream_t st = m->e->stream;
    MCU(cudaMemsetAsync(m->d_barrier, 0, sizeof(unsigned int), st));
    StepArgs sa{};
    sa.ops = m->d_ops; sa.nops = m->step_nops; sa.nsteps = n;
    sa.pos = m->d_pos; sa.token = m->d_token; sa.trace = m->d_trace; sa.key = m->argmax_key;
    sa.barrier = m->d_barrier; sa.status = m->e->status; sa.write_token = greedy_feed ? 1 : 0;
    sa.nstages = 2; sa.stage_stride = m->step_stride; sa.aux_off = m->step_aux_off;
    sa.ops_off = (uint32_t)(m->step_smem - 2 * sizeof(StepOp));
    // ALICE_STEP_PROF=1: per-op clock stamps of one CTA during the last step, printed after the launch (debug aid)
    long long* prof = nullptr;
    if (getenv("ALICE_STEP_PROF")) {
        MCU(cudaMalloc(&prof, (size_t)m->step_nops * 16 * sizeof(long long)));
        MCU(cudaMemset(prof, 0, (size_t)m->step_nops * 16 * sizeof(long long)));
    }
    sa.prof = prof;
    MCU(launch_decode_steps(sa, m->step_grid, m->step_smem, st));
    if (prof) {
        std::vector<long long> h((size_t)m->step_nops * 16);
        MCU(cudaStreamSynchronize(st));
        MCU(cudaMemcpy(h.data(), prof, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
        cudaFree(prof);
        fprintf(stderr, "[alice] step profile of one CTA, SM clock cycles\n");
        for (uint32_t i = 0; i < m->step_nops; i++) {
            const long long* p = &h[(size_t)i * 16];
            if (m->step_types[i] == SOP_GEMV) {
                fprintf(stderr, "[alice] %3u matvec    prologue %6lld  first stage %6lld  rows %7lld  grid barrier %6lld  total %7lld  | stages:", i,
                        p[1] - p[0], p[2] - p[1], p[3] - p[2], p[5] - p[4], p[5] - p[0]);
                for (int c = 0; c < 8 && p[8 + c]; c++) fprintf(stderr, " %lld", p[8 + c] - (c ? p[7 + c] : p[2]));
                fprintf(stderr, "\n");
            } else if (m->step_types[i] == SOP_ATTN) {
                fprintf(stderr, "[alice] %3u attention q+rope %6lld  positions %6lld  cta combine %6lld  ticket %6lld  fold %6lld  grid barrier %6lld  total %7lld\n", i,
                        p[1] - p[0], p[2] - p[1], p[3] - p[2], p[6] - p[3], p[4] - p[6], p[5] - p[4], p[5] - p[0]);
            } else {
                fprintf(stderr, "[alice] %3u embedding %6lld  grid barrier %6lld\n", i, p[4] - p[0], p[5] - p[4]);
            }
        }
    }
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
    const size_t kv_elems = (size_t)c.num_layers * c.max_seq_len * lkv;
    if (!rc) rc = upload_norm(m, &m->out_norm, output_norm, c.hidden_dim);
    {   // the vectors other ranks need, the argmax keys and the hand-over counters share one allocation
        auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
        const size_t o_hidden = 0, o_attn = o_hidden + up((size_t)c.hidden_dim * 4), o_ffn = o_attn + up((size_t)q_dim * 4),
                     o_logits = o_ffn + up((size_t)c.intermediate_dim * 4), o_keys = o_logits + up((size_t)c.vocab_size * 4),
                     o_flags = o_keys + up(8 * 8), o_epoch = o_flags + up(((size_t)4 * c.num_layers + 2) * 4),
                     o_hll = o_epoch + 256, o_all = o_hll + up((size_t)c.hidden_dim * 8), o_fll = o_all + up((size_t)q_dim * 8);
        m->xchg_bytes = o_fll + up((size_t)c.intermediate_dim * 8);
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
            m->hidden_ll = reinterpret_cast<uint2*>(m->xchg + o_hll);
            m->attn_ll = reinterpret_cast<uint2*>(m->xchg + o_all);
            m->ffn_ll = reinterpret_cast<uint2*>(m->xchg + o_fll);
        }
    }
    if (!rc) rc = dev_alloc(m, &m->qkv, lq + 2 * lkv);
    if (!rc) rc = dev_alloc(m, &m->kcache, kv_elems);
    if (!rc) rc = dev_alloc(m, &m->vcache, kv_elems);
    if (!rc) rc = dev_alloc(m, &m->attn_part, (size_t)m->nsplit * (c.num_heads / n) * (c.head_dim + 4));
    if (!rc) rc = dev_alloc(m, &m->attn_tickets, c.num_kv_heads / n);
    if (!rc) rc = dev_alloc(m, &m->rope_tab, 128);
    m->attn_q8_lay = Q8KLayout::make(q_dim / 256, 1);
    m->attn_q8_ok = n == 1 && (group % 2) == 0 && q_dim % 256 == 0 && !getenv("ALICE_NO_ATTN_Q8");
    if (!rc && m->attn_q8_ok) rc = dev_alloc(m, &m->attn_q8, m->attn_q8_lay.total);
    if (!rc) rc = dev_alloc(m, &m->d_pos, 1);
    if (!rc) rc = dev_alloc(m, &m->d_token, 1);
    if (!rc) rc = dev_alloc(m, &m->d_trace, c.max_seq_len);
    if (!rc) {
        cudaError_t err = cudaMemsetAsync(m->kcache, 0, kv_elems * 4, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->vcache, 0, kv_elems * 4, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->d_pos, 0, 4, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->attn_tickets, 0, (size_t)(c.num_kv_heads / n) * 4, e->stream);
        if (err == cudaSuccess) err = cudaMemsetAsync(m->d_token, 0, 4, e->stream);
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
    cudaStreamSynchronize(m->e->stream);
    if (m->graph_greedy) cudaGraphExecDestroy(m->graph_greedy);
    for (uint32_t p = 0; p < m->npeers; p++) cudaIpcCloseMemHandle(m->peer_base[p]);
    for (void* p : m->owned) cudaFree(p);
    delete m;
    return ALICE_OK;
}

static int set_token(alice_model* m, uint32_t token) {
    if (token >= m->cfg.vocab_size) return alice_fail(ALICE_E_INVALID, "alice_model: token %u >= vocab %u", token, m->cfg.vocab_size);
    const int t = (int)token;
    MCU(cudaMemcpyAsync(m->d_token, &t, 4, cudaMemcpyHostToDevice, m->e->stream));
    MCU(cudaStreamSynchronize(m->e->stream));  // `t` lives on this stack frame
    return ALICE_OK;
}

int32_t alice_model_forward(alice_model* m, uint32_t token) {
    if (!m) return alice_fail(ALICE_E_INVALID, "alice_model_forward: null model");
    MCU(cudaSetDevice(m->e->device));
    int rc = check_room(m, 1, "alice_model_forward");
    if (!rc) rc = set_token(m, token);
    if (!rc) rc = enqueue_step(m, false);
    if (!rc) m->pos += 1;
    return rc;
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
    if (m->use_step_kernel && !m->step_tried) {
        m->step_tried = true;
        rc = build_step_ops(m);
        if (rc) return rc;
    }
    if (m->use_step_kernel && m->step_ready) {
        rc = run_step_kernel(m, n, true);
        if (rc) return rc;
        m->pos += n;
        MCU(cudaMemcpyAsync(out_tokens, m->d_trace + pos0, (size_t)n * 4, cudaMemcpyDeviceToHost, st));
        MCU(cudaStreamSynchronize(st));
        return alice_sync(m->e);
    }
    if (!m->graph_tried) {
        // Capture one step (every kernel reads position and token from device memory) and replay it.
        m->graph_tried = true;
        rc = enqueue_step(m, true);   // eager first step: also sets per-kernel attributes outside capture
        if (rc) return rc;
        m->pos += 1;
        cudaGraph_t g = nullptr;
        if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            const int crc = enqueue_step(m, true);
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
            rc = enqueue_step(m, true);
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
    for (const alice_model::Layer& L : m->layers)
        for (const WeightDesc* w : {&L.o, &L.down})
            if (w->fmt == WF_Q8_0 || w->fmt == WF_Q2_0 || w->fmt == WF_SPARSE_TERNARY)
                return alice_fail(ALICE_E_UNSUPPORTED, "alice_model_tp_connect: o / down projections in Q8_0, Q2_0 or sparse ternary read their input "
                                                       "directly and cannot take pushed vectors; the model keeps using NCCL all-gathers");
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

int32_t alice_model_use_step_kernel(alice_model* m, int32_t enabled) {
    if (!m) return alice_fail(ALICE_E_INVALID, "alice_model_use_step_kernel: null model");
    m->use_step_kernel = enabled != 0;
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
