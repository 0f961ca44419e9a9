// Llama-2 family decoder: weights, state, one-token forward and the device-resident greedy loop.
//
// Follows Llama2::dispatch (crates/wgml/src/models/llama2/transformer.rs:298-431) and the token
// loop of ChatLlama2::forward (crates/wgml-chat/src/chat_llama2.rs:102-228).  Two schedules:
//   fused    5 launches per layer:  [RMSNorm + Q/K/V products + bias + RoPE + KV append]
//            [split attention]  [O product + residual]  [RMSNorm + gate/up products + SiLU]
//            [down product + residual], then [RMSNorm + output product], argmax.
//   unfused  one launch per reference dispatch, in the reference's order.
// Token id, position, logits and the KV cache live on the device; a decode step is captured
// once into a CUDA graph and replayed per token.
#include "kernels.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

namespace wgb {
void rope_inv_freq(uint32_t head_size, float base, float *out);
}

using namespace wgb;

struct wgb_llama2 {
    wgb_llama2_config cfg;
    int model_type, tp_rank, tp_size;
    uint32_t head_size, kv_mul;
    // per-rank sizes
    uint32_t n_q_local, n_kv_local, q_dim, kv_dim, hidden;
    uint32_t hidden_blk0, hidden_blks;   // this rank's slice of the FFN dimension in 256-column blocks
    struct Layer {
        wgb_quant_matrix *m[7] = {};
        float *v[5] = {};
    };
    std::vector<Layer> layers;
    wgb_quant_matrix *token_embd = nullptr, *output = nullptr;
    float *output_norm = nullptr;
    // state (Llama2State, transformer.rs:17-45)
    float *x = nullptr, *xb = nullptr, *xb2 = nullptr, *hb = nullptr, *hb2 = nullptr, *q = nullptr, *logits = nullptr;
    float *tk = nullptr, *tv = nullptr;      // unfused path: K / V projections before RoPE + append
    // [n_layers][n_kv_local][seq_len][head_size]: head-major, so that the positions of one head are contiguous
    float *key_cache = nullptr, *value_cache = nullptr;
    float *attn_scratch = nullptr;
    uint32_t *attn_counters = nullptr;
    float *rope_freq = nullptr;
    uint32_t *scalars = nullptr;             // token, pos, step
    uint32_t *argmax_scratch = nullptr;
    uint32_t *d_prompt = nullptr, *d_out = nullptr;
    size_t prompt_cap = 0, out_cap = 0;
    uint32_t *h_pinned = nullptr;            // pinned staging of a decode call: [0] status word, [1..2] status polls, [3..] token ids
    size_t pinned_cap = 0;
    StatusPoll poll;
    Uploader up;                             // pipelined weight upload (set_matrix / load_gguf)
    bool loading = false;                    // inside wgb_llama2_load_gguf: the uploads are waited for once, at the end
    // sampling of generated tokens: temperature 0 = greedy (Sampler::sample, models/sampler.rs:32-52)
    float smp_temperature = 0.0f, smp_topp = 0.0f;
    unsigned long long smp_seed = 0;
    void *smp_scratch = nullptr;
    bool fused = true, use_pdl = true;
    cudaGraphExec_t graph = nullptr;
    uint32_t graph_n_prompt = 0;
    uint32_t pos_bound = 0;                  // furthest position the launches being recorded will serve
    uint32_t graph_attn_chunks = 0;          // attention launch shape (attn_sizing_class) the captured graph was built for
    void *comm = nullptr;
    // direct exchange of partial products between the ranks (wgb_llama2_set_exchange)
    int exchange = 0;
    float *mail_peer[PEER_MAX] = {};         // rank p's mailbox as seen from here: [2 * n_layers][tp][dim] floats
    uint32_t *flag_peer[PEER_MAX] = {};      // rank p's flags: [2 * n_layers][tp]
    uint32_t *tickets = nullptr;             // local: one per exchange
    uint32_t *tp_epoch = nullptr;            // local: forwards so far
    bool exchange_external = false;          // mailboxes and flags were mapped by the caller (wgb_llama2_set_exchange_buffers)
    bool vocab_shard = false;                // every rank computes vocab_size / tp_size logits, an all-gather completes them
    int kernels_per_token = 0;
    // per-launch timing of wgb_llama2_profile_step: one event after every launch
    bool profiling = false;
    // per-launch timing inside a graph replay: end-time slot per launch ([0] = start of the step)
    unsigned long long *stamps = nullptr;
    size_t stamps_cap = 0;
    bool stamping = false;
    std::vector<cudaEvent_t> prof_events;
    std::vector<int> prof_kind, prof_layer;
    // batched prompt prefill (wgb_llama2_set_prefill): tile-major copies of the Q4_K layer matrices for the
    // tensor-core product, activation images and the buffers of a pass of PF_TOK positions
    struct Prefill {
        bool enabled = false;
        std::vector<uint8_t *> tiles;        // [layer * 7 + matrix], NULL: no tensor-core path for that matrix
        std::vector<uint8_t> tiles_q6;       // same index: 0 a Q4_K copy, 1 a Q6_K one (its own kernel and image), 2 a Q8_0 one
        uint8_t *img_dim = nullptr, *img_q = nullptr, *img_hidden = nullptr;
        uint8_t *img6 = nullptr;             // Q6_K image of the widest input
        float *x = nullptr, *xn = nullptr, *q = nullptr, *xb = nullptr, *h = nullptr;   // [PF_TOK][dim | q_dim | hidden]
        float *part[3] = {};                 // product slices: [PF_MAX_SPLIT][PF_TOK][max(dim, q_dim, hidden)]
        float *attn_scratch = nullptr;       // prompt attention split over several blocks: partial sums
        uint32_t *attn_counters = nullptr;   //   and arrival counters
        float *red = nullptr;                // tensor parallel: [PF_TOK][dim], a rank's partial product summed over the group
        size_t positions = 0;                // prompt positions that went through it, over all decode calls
    } pf;
};

namespace {

__global__ void bump_kernel(uint32_t *p) { *p += 1; }

__global__ void stamp_kernel(unsigned long long *slot) { stamp_end(slot); }

__global__ void set_scalars_kernel(uint32_t *s, uint32_t token, uint32_t pos, uint32_t step)
{
    s[0] = token;
    s[1] = pos;
    s[2] = step;
}

// Unfused path: bias, RoPE and KV append for one position (the work of the OpAssign / RoPE
// dispatches of transformer.rs:343-365, plus the write into cache column `pos`).
__global__ void qkv_finish_kernel(float *__restrict__ q, const float *__restrict__ tk, const float *__restrict__ tv,
                                  const float *__restrict__ bq, const float *__restrict__ bk, const float *__restrict__ bv,
                                  float *__restrict__ k_cache, float *__restrict__ v_cache, const uint32_t *__restrict__ d_pos,
                                  uint32_t q_dim, uint32_t kv_dim, uint32_t head_size, uint32_t seq_len, int variant,
                                  const float *__restrict__ freq)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;  // pair index over q
    if (2 * i >= q_dim) return;
    const uint32_t pos = *d_pos;
    const uint32_t half = head_size / 2;
    float sn, cs;
    sincosf((float)pos * freq[i % half], &sn, &cs);
    uint32_t ia, ib;
    if (variant == WGB_ROPE_ORIGINAL) { ia = 2 * i; ib = ia + 1; }
    else { ia = i + ((2 * i) / head_size) * half; ib = ia + half; }
    float x = q[ia] + (bq ? bq[ia] : 0.0f), y = q[ib] + (bq ? bq[ib] : 0.0f);
    q[ia] = cs * x - sn * y;
    q[ib] = sn * x + cs * y;
    if (2 * i < kv_dim) {
        // head-major cache: element e of head h at position pos sits at (h * seq_len + pos) * head_size + e
        float *kc = k_cache + (size_t)pos * head_size, *vc = v_cache + (size_t)pos * head_size;
        const size_t da = (size_t)(ia / head_size) * seq_len * head_size + ia % head_size;
        const size_t db = (size_t)(ib / head_size) * seq_len * head_size + ib % head_size;
        x = tk[ia] + (bk ? bk[ia] : 0.0f);
        y = tk[ib] + (bk ? bk[ib] : 0.0f);
        kc[da] = cs * x - sn * y;
        kc[db] = sn * x + cs * y;
        vc[da] = tv[ia] + (bv ? bv[ia] : 0.0f);
        vc[db] = tv[ib] + (bv ? bv[ib] : 0.0f);
    }
}

int dalloc(float **p, size_t n)
{
    WGB_CUDA(cudaMalloc((void **)p, n * sizeof(float)));
    WGB_CUDA(cudaMemset(*p, 0, n * sizeof(float)));
    return WGB_OK;
}

bool fusable(const wgb_llama2 *m)
{
    for (const auto &l : m->layers) {
        for (int i = 0; i < 7; i++)
            if (!l.m[i] || !gemv_fast_supported(l.m[i]->view)) return false;
        const QMat &q = l.m[WGB_L_ATTN_Q]->view, &k = l.m[WGB_L_ATTN_K]->view, &v = l.m[WGB_L_ATTN_V]->view;
        if (q.qtype != k.qtype || q.qtype != v.qtype) return false;
        if (l.m[WGB_L_FFN_GATE]->view.qtype != l.m[WGB_L_FFN_UP]->view.qtype) return false;
    }
    const wgb_quant_matrix *out = m->output ? m->output : m->token_embd;
    return out && gemv_fast_supported(out->view);
}

int check_complete(const wgb_llama2 *m)
{
    for (size_t l = 0; l < m->layers.size(); l++) {
        for (int i = 0; i < 7; i++)
            if (!m->layers[l].m[i]) return fail(WGB_ERR_NOT_FOUND, "layer %zu: matrix %d was never set", l, i);
        for (int i = 0; i < 2; i++)
            if (!m->layers[l].v[i]) return fail(WGB_ERR_NOT_FOUND, "layer %zu: norm vector %d was never set", l, i);
    }
    if (!m->token_embd) return fail(WGB_ERR_NOT_FOUND, "token_embd.weight was never set");
    if (!m->output_norm) return fail(WGB_ERR_NOT_FOUND, "output_norm.weight was never set");
    return WGB_OK;
}

// Plain product out = W . x through the fast kernel when there is one.
int mat_vec(const QMat &w, const float *x, float *out, cudaStream_t s)
{
    if (gemv_fast_supported(w)) {
        GemvArgs a = {};
        a.mat[0] = w;
        a.nmat = 1;
        a.x = x;
        a.epilogue = EPI_STORE;
        a.out = out;
        return launch_gemv(a, s, false);
    }
    return launch_gemv_generic(w, x, out, s);
}

// Profiling: an event after the launch just enqueued, tagged with its kind and layer.
enum { K_EMBED = 0, K_QKV, K_ATTN, K_OPROJ, K_GATE_UP, K_DOWN, K_HEAD, K_OTHER };
int mark(wgb_llama2 *m, cudaStream_t s, int kind, int layer)
{
    if (m->stamping) {   // the launch wrote its own end time; only its tag is kept
        m->prof_kind.push_back(kind);
        m->prof_layer.push_back(layer);
        return WGB_OK;
    }
    if (!m->profiling) return WGB_OK;
    cudaEvent_t e;
    WGB_CUDA(cudaEventCreate(&e));
    WGB_CUDA(cudaEventRecord(e, s));
    m->prof_events.push_back(e);
    m->prof_kind.push_back(kind);
    m->prof_layer.push_back(layer);
    return WGB_OK;
}

// Enqueues one token forward reading token / position from the device scalars.
int enqueue_forward(wgb_llama2 *m, cudaStream_t s, int *nkernels)
{
    const wgb_llama2_config &c = m->cfg;
    const uint32_t *d_token = m->scalars, *d_pos = m->scalars + 1;
    const bool fused = m->fused && fusable(m);
    const bool pdl = m->use_pdl && !m->profiling;
    const bool tp = m->tp_size > 1;
    const int variant = m->model_type == WGB_QWEN2 ? WGB_ROPE_NEOX : WGB_ROPE_ORIGINAL;
    int n = 0;
    // stamping: slot 0 takes the start of the step, slot i the end of the i-th marked launch
    size_t next_stamp = 0;
    auto stamp_slot = [&]() -> unsigned long long * { return m->stamping ? m->stamps + next_stamp++ : nullptr; };
    if (m->stamping) {
        stamp_kernel<<<1, 1, 0, s>>>(stamp_slot());
        WGB_LAUNCH_CHECK("stamp_kernel");
    }
    // Direct exchange between the ranks (fused schedule only): exchange 2l follows attn_output of layer l,
    // 2l + 1 its ffn_down; the next normalising kernel (gate/up, the next layer's q/k/v, the logits) adds
    // the partials.  `pending` is the exchange whose sum the next such kernel has to form.
    const bool direct = tp && m->exchange == 1 && fused;
    int pending = -1;
    auto send_to_peers = [&](GemvArgs &g, int e) {
        g.peer_out.n = (uint32_t)m->tp_size;
        for (int p = 0; p < m->tp_size; p++) {
            g.peer_out.mail[p] = m->mail_peer[p] + ((size_t)e * m->tp_size + m->tp_rank) * c.dim;
            g.peer_out.flag[p] = m->flag_peer[p] + (size_t)e * m->tp_size + m->tp_rank;
        }
        g.peer_out.ticket = m->tickets + e;
        pending = e;
    };
    auto receive_pending = [&](GemvArgs &g) {
        if (pending < 0) return;
        g.peer_in.n = (uint32_t)m->tp_size;
        g.peer_in.mail = m->mail_peer[m->tp_rank] + (size_t)pending * m->tp_size * c.dim;
        g.peer_in.flag = m->flag_peer[m->tp_rank] + (size_t)pending * m->tp_size;
        g.peer_in.epoch = m->tp_epoch;
        g.peer_in.x_out = m->x;
        pending = -1;
    };
    if (direct) {
        bump_kernel<<<1, 1, 0, s>>>(m->tp_epoch);
        WGB_LAUNCH_CHECK("bump_kernel");
    }
    int rc = launch_embed(m->token_embd->view, nullptr, d_token, d_pos, m->x, s);
    if (rc) return rc;
    n++;
    if (!m->stamping) mark(m, s, K_EMBED, -1);
    const size_t cache_stride = (size_t)c.seq_len * m->kv_dim;
    AttnArgs at = {};
    at.p.seq_len = c.seq_len;
    at.p.kv_dim = m->kv_dim;
    at.p.kv_mul = m->kv_mul;
    at.p.n_heads = m->n_q_local;
    at.p.head_size = m->head_size;
    at.p.pos = m->pos_bound;
    at.pos = d_pos;
    at.row_stride = m->head_size;
    at.head_stride = c.seq_len * m->head_size;
    at.q = m->q;
    at.xb = m->xb;
    at.scratch = m->attn_scratch;
    at.counters = m->attn_counters;
    at.err = gemv_status_word();
    for (uint32_t l = 0; l < c.n_layers; l++) {
        const wgb_llama2::Layer &w = m->layers[l];
        float *kc = m->key_cache + l * cache_stride, *vc = m->value_cache + l * cache_stride;
        at.k_cache = kc;
        at.v_cache = vc;
        if (fused) {
            GemvArgs a = {};
            a.mat[0] = w.m[WGB_L_ATTN_Q]->view;
            a.mat[1] = w.m[WGB_L_ATTN_K]->view;
            a.mat[2] = w.m[WGB_L_ATTN_V]->view;
            a.nmat = 3;
            a.x = m->x;
            a.prologue = PRO_RMS;
            a.norm_w = w.v[WGB_L_ATTN_NORM];
            a.eps = c.rms_norm_eps;
            a.epilogue = EPI_QKV_ROPE;
            a.out = m->q;
            a.bias = w.v[WGB_L_ATTN_Q_BIAS];
            a.bias_k = w.v[WGB_L_ATTN_K_BIAS];
            a.bias_v = w.v[WGB_L_ATTN_V_BIAS];
            a.k_cache = kc;
            a.v_cache = vc;
            a.pos = d_pos;
            a.kv_dim = m->kv_dim;
            a.head_size = m->head_size;
            a.kv_row_stride = m->head_size;
            a.kv_head_stride = c.seq_len * m->head_size;
            a.rope_variant = variant;
            a.rope_freq = m->rope_freq;
            a.stamp = stamp_slot();
            receive_pending(a);
            if ((rc = launch_gemv(a, s, pdl))) return rc;
            mark(m, s, K_QKV, l);
            at.stamp = stamp_slot();
            if ((rc = launch_attention(at, s, pdl))) return rc;
            mark(m, s, K_ATTN, l);
            GemvArgs o = {};
            o.mat[0] = w.m[WGB_L_ATTN_OUTPUT]->view;
            o.nmat = 1;
            o.x = m->xb;
            // Tensor parallel: the rank holds a column slice, so its product is a partial sum over the
            // group; rank 0 folds the residual in and the all-reduce leaves the new x on every rank.
            o.epilogue = (!tp || m->tp_rank == 0) ? EPI_RESIDUAL : EPI_STORE;
            o.residual = m->x;
            o.out = tp ? m->xb2 : m->x;
            o.stamp = stamp_slot();
            if (direct) send_to_peers(o, 2 * (int)l);
            if ((rc = launch_gemv(o, s, pdl))) return rc;
            if (tp && !direct && (rc = wgb_comm_all_reduce_sum((wgb_comm *)m->comm, m->xb2, m->x, c.dim, s))) return rc;
            mark(m, s, K_OPROJ, l);
            GemvArgs f = {};
            f.mat[0] = w.m[WGB_L_FFN_GATE]->view;
            f.mat[1] = w.m[WGB_L_FFN_UP]->view;
            f.nmat = 2;
            f.x = m->x;
            f.prologue = PRO_RMS;
            f.norm_w = w.v[WGB_L_FFN_NORM];
            f.eps = c.rms_norm_eps;
            f.epilogue = EPI_SILU_PAIR;
            f.out = m->hb;
            f.stamp = stamp_slot();
            receive_pending(f);
            if ((rc = launch_gemv(f, s, pdl))) return rc;
            mark(m, s, K_GATE_UP, l);
            GemvArgs d = {};
            d.mat[0] = w.m[WGB_L_FFN_DOWN]->view;
            d.nmat = 1;
            d.x = m->hb;
            d.epilogue = (!tp || m->tp_rank == 0) ? EPI_RESIDUAL : EPI_STORE;
            d.residual = m->x;
            d.out = tp ? m->xb2 : m->x;
            d.stamp = stamp_slot();
            if (direct) send_to_peers(d, 2 * (int)l + 1);
            if ((rc = launch_gemv(d, s, pdl))) return rc;
            if (tp && !direct && (rc = wgb_comm_all_reduce_sum((wgb_comm *)m->comm, m->xb2, m->x, c.dim, s))) return rc;
            mark(m, s, K_DOWN, l);
            n += 5;
        } else {
            // transformer.rs:312-407, dispatch by dispatch
            if ((rc = wgb_rms_norm(m->xb, m->x, w.v[WGB_L_ATTN_NORM], c.dim, c.rms_norm_eps, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_L_ATTN_Q]->view, m->xb, m->q, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_L_ATTN_K]->view, m->xb, m->tk, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_L_ATTN_V]->view, m->xb, m->tv, s))) return rc;
            qkv_finish_kernel<<<(m->q_dim / 2 + 127) / 128, 128, 0, s>>>(
                m->q, m->tk, m->tv, w.v[WGB_L_ATTN_Q_BIAS], w.v[WGB_L_ATTN_K_BIAS], w.v[WGB_L_ATTN_V_BIAS], kc, vc, d_pos,
                m->q_dim, m->kv_dim, m->head_size, c.seq_len, variant, m->rope_freq);
            WGB_LAUNCH_CHECK("qkv_finish_kernel");
            if ((rc = launch_attention(at, s, false))) return rc;
            if ((rc = mat_vec(w.m[WGB_L_ATTN_OUTPUT]->view, m->xb, m->xb2, s))) return rc;
            if (tp && (rc = wgb_comm_all_reduce_sum((wgb_comm *)m->comm, m->xb2, m->xb2, c.dim, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->x, m->xb2, c.dim, s))) return rc;
            if ((rc = wgb_rms_norm(m->xb, m->x, w.v[WGB_L_FFN_NORM], c.dim, c.rms_norm_eps, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_L_FFN_GATE]->view, m->xb, m->hb, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_L_FFN_UP]->view, m->xb, m->hb2, s))) return rc;
            if ((rc = wgb_silu(m->hb, m->hb2, m->hidden, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_L_FFN_DOWN]->view, m->hb, m->xb2, s))) return rc;
            if (tp && (rc = wgb_comm_all_reduce_sum((wgb_comm *)m->comm, m->xb2, m->xb2, c.dim, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->x, m->xb2, c.dim, s))) return rc;
            mark(m, s, K_OTHER, l);
            n += 14;
        }
    }
    // The output head.  Its matrix is replicated; with the vocabulary-sharded head a rank multiplies only its run of
    // vocab_size / tp_size rows (a row-range view: every plane is row-major with 16-byte-aligned pitches) into its
    // part of the logits, and an all-gather hands every rank all of them, so that the argmax / the sampler and
    // wgb_llama2_logits see what they see on one GPU.
    QMat outw = (m->output ? m->output : m->token_embd)->view;
    float *head_out = m->logits;
    const bool vshard = tp && m->vocab_shard;
    const uint32_t vocab_local = vshard ? c.vocab_size / (uint32_t)m->tp_size : c.vocab_size;
    if (vshard) {
        WGB_REQUIRE(m->comm, "the vocabulary-sharded head needs a communicator (wgb_llama2_set_comm)");
        const size_t row0 = (size_t)m->tp_rank * vocab_local;
        for (int i = 0; i < outw.nplanes; i++) outw.p[i] += row0 * outw.pitch[i];
        outw.nrows = vocab_local;
        head_out += row0;
    }
    if (fused) {
        GemvArgs a = {};
        a.mat[0] = outw;
        a.nmat = 1;
        a.x = m->x;
        a.prologue = PRO_RMS;
        a.norm_w = m->output_norm;
        a.eps = c.rms_norm_eps;
        a.epilogue = EPI_STORE;
        a.out = head_out;
        a.stamp = stamp_slot();
        receive_pending(a);
        if ((rc = launch_gemv(a, s, pdl))) return rc;
        mark(m, s, K_HEAD, -1);
        n += 1;
    } else {
        if ((rc = wgb_rms_norm(m->xb, m->x, m->output_norm, c.dim, c.rms_norm_eps, s))) return rc;
        if ((rc = mat_vec(outw, m->xb, head_out, s))) return rc;
        mark(m, s, K_HEAD, -1);
        n += 2;
    }
    if (vshard && (rc = wgb_comm_all_gather((wgb_comm *)m->comm, head_out, m->logits, vocab_local, s))) return rc;
    if (nkernels) *nkernels = n;
    return WGB_OK;
}

void prefill_free(wgb_llama2 *m)
{
    for (uint8_t *t : m->pf.tiles) if (t) cudaFree(t);
    m->pf.tiles.clear();
    uint8_t *imgs[] = { m->pf.img_dim, m->pf.img_q, m->pf.img_hidden, m->pf.img6 };
    for (uint8_t *b : imgs) if (b) cudaFree(b);
    float *bufs[] = { m->pf.x, m->pf.xn, m->pf.q, m->pf.xb, m->pf.h, m->pf.part[0], m->pf.part[1], m->pf.part[2], m->pf.red, m->pf.attn_scratch };
    if (m->pf.attn_counters) cudaFree(m->pf.attn_counters);
    for (float *b : bufs) if (b) cudaFree(b);
    m->pf = wgb_llama2::Prefill();
}

// One product of a prefill pass: W . (the `ntok` vectors whose image is `image` and whose values are xf), as
// slices [slice][PF_TOK][stride] in `out`.  Matrices without a tile-major copy (any format but Q4_K) go through
// the matrix-vector kernel once per position.
int prefill_product(wgb_llama2 *m, uint32_t layer, int which, const uint8_t *image, const float *xf, uint32_t xf_stride, uint32_t ntok,
                    float *out, uint32_t stride, uint32_t *nsplit, cudaStream_t s)
{
    const QMat &w = m->layers[layer].m[which]->view;
    const uint8_t *tiles = m->pf.tiles[(size_t)layer * 7 + which];
    if (tiles && m->pf.tiles_q6[(size_t)layer * 7 + which] == 2) {
        *nsplit = prefill_gemm_splits(w.nrows, w.ncols);
        return launch_gemm_q80_tiles(tiles, w.nrows, w.ncols, image, ntok, out, stride, *nsplit, s);
    }
    if (tiles && m->pf.tiles_q6[(size_t)layer * 7 + which] == 1) {
        *nsplit = prefill_gemm_splits(w.nrows, w.ncols);
        int rc = launch_prefill_image6(xf, xf_stride, w.ncols, ntok, m->pf.img6, s);
        if (rc) return rc;
        return launch_gemm_q6k_tiles(tiles, w.nrows, w.ncols, m->pf.img6, ntok, out, stride, *nsplit, s);
    }
    if (tiles) {
        *nsplit = prefill_gemm_splits(w.nrows, w.ncols);
        return launch_gemm_q4k_tiles(tiles, w.nrows, w.ncols, image, ntok, out, stride, *nsplit, s);
    }
    *nsplit = 1;
    for (uint32_t t = 0; t < ntok; t++) {
        int rc = mat_vec(w, xf + (size_t)t * xf_stride, out + (size_t)t * stride, s);
        if (rc) return rc;
    }
    return WGB_OK;
}

// Products of several matrices of a layer with the same input (q / k / v; gate / up), product i as slices in out[i]:
// one launch when all of them have Q4_K tile-major copies, one product after the other otherwise.
int prefill_products(wgb_llama2 *m, uint32_t layer, const int *which, uint32_t n, const uint8_t *image, const float *xf, uint32_t xf_stride,
                     uint32_t ntok, float *const *out, const uint32_t *stride, uint32_t *nsplit, cudaStream_t s)
{
    bool together = n > 1;
    uint32_t rows[3], total_rows = 0;
    const uint8_t *tiles[3];
    for (uint32_t i = 0; i < n; i++) {
        const size_t idx = (size_t)layer * 7 + which[i];
        const QMat &w = m->layers[layer].m[which[i]]->view;
        tiles[i] = m->pf.tiles[idx];
        rows[i] = w.nrows;
        total_rows += w.nrows;
        if (!tiles[i] || m->pf.tiles_q6[idx] || w.ncols != m->layers[layer].m[which[0]]->view.ncols) together = false;
    }
    if (together) {
        const uint32_t K = m->layers[layer].m[which[0]]->view.ncols, ns = prefill_gemm_splits(total_rows, K);
        for (uint32_t i = 0; i < n; i++) nsplit[i] = ns;
        return launch_gemm_q4k_tiles_multi(n, tiles, rows, K, image, ntok, out, stride, ns, s);
    }
    for (uint32_t i = 0; i < n; i++) {
        int rc = prefill_product(m, layer, which[i], image, xf, xf_stride, ntok, out[i], stride[i], &nsplit[i], s);
        if (rc) return rc;
    }
    return WGB_OK;
}

// Prompt positions pos0 .. pos0 + ntok - 1 (tokens d_tokens[0 .. ntok)) through the layer stack in one pass: the
// work of ntok calls of Llama2::dispatch (models/llama2/transformer.rs:298-431) up to the last layer's cache
// rows -- the logits of prompt positions are never looked at (chat_llama2.rs:169-204 samples only once the
// prompt is through), so the final norm and the output matrix are left out.
int prefill_pass(wgb_llama2 *m, cudaStream_t s, const uint32_t *d_tokens, uint32_t pos0, uint32_t ntok)
{
    const wgb_llama2_config &c = m->cfg;
    wgb_llama2::Prefill &pf = m->pf;
    const int variant = m->model_type == WGB_QWEN2 ? WGB_ROPE_NEOX : WGB_ROPE_ORIGINAL;
    const uint32_t dim = c.dim, q_dim = m->q_dim, kv_dim = m->kv_dim, hidden = m->hidden;
    int rc;
    for (uint32_t t = 0; t < ntok; t++)
        if ((rc = launch_embed(m->token_embd->view, nullptr, d_tokens + t, m->scalars + 1, pf.x + (size_t)t * dim, s))) return rc;
    const size_t cache_stride = (size_t)c.seq_len * kv_dim;
    // Tensor parallel: a rank's attn_output / ffn_down products are partial sums over the group (column slices of
    // the matrices); their slices are added up locally, summed over the ranks (one all-reduce of [ntok][dim] per
    // product) and handed on as a single slice.  Every rank then adds the same sum to its copy of x.
    auto across_ranks = [&](const float **part, uint32_t *nsplit) -> int {
        if (m->tp_size == 1) return WGB_OK;
        WGB_CUDA(cudaMemsetAsync(pf.red, 0, (size_t)PF_TOK * dim * sizeof(float), s));
        int r = launch_prefill_norm_image(pf.red, dim, *part, *nsplit, dim, nullptr, 0.0f, dim, ntok, nullptr, nullptr, 0, s);
        if (r) return r;
        if ((r = wgb_comm_all_reduce_sum((wgb_comm *)m->comm, pf.red, pf.red, (size_t)PF_TOK * dim, s))) return r;
        *part = pf.red;
        *nsplit = 1;
        return WGB_OK;
    };
    const float *pending = nullptr;   // slices of the last layer's ffn_down, folded into x by the next norm
    uint32_t pending_split = 0;
    for (uint32_t l = 0; l < c.n_layers; l++) {
        const wgb_llama2::Layer &w = m->layers[l];
        uint32_t nq, nk, nv, no, ng, nu, nd;
        if ((rc = launch_prefill_norm_image(pf.x, dim, pending, pending_split, dim, w.v[WGB_L_ATTN_NORM], c.rms_norm_eps, dim, ntok, pf.img_dim,
                                            pf.xn, dim, s)))
            return rc;
        {
            // q and k (and v, unless the file keeps it in another format) in one launch
            const int which[3] = { WGB_L_ATTN_Q, WGB_L_ATTN_K, WGB_L_ATTN_V };
            const uint32_t strides[3] = { q_dim, kv_dim, kv_dim };
            uint32_t ns[3];
            const bool v_too = pf.tiles[(size_t)l * 7 + WGB_L_ATTN_V] && !pf.tiles_q6[(size_t)l * 7 + WGB_L_ATTN_V];
            if ((rc = prefill_products(m, l, which, v_too ? 3 : 2, pf.img_dim, pf.xn, dim, ntok, pf.part, strides, ns, s))) return rc;
            if (!v_too && (rc = prefill_product(m, l, WGB_L_ATTN_V, pf.img_dim, pf.xn, dim, ntok, pf.part[2], kv_dim, &ns[2], s))) return rc;
            nq = ns[0]; nk = ns[1]; nv = ns[2];
        }
        PrefillQkv qa = {};
        qa.q = pf.part[0]; qa.k = pf.part[1]; qa.v = pf.part[2];
        qa.q_split = nq; qa.k_split = nk; qa.v_split = nv;
        qa.q_stride = q_dim; qa.kv_stride = kv_dim;
        qa.bq = w.v[WGB_L_ATTN_Q_BIAS]; qa.bk = w.v[WGB_L_ATTN_K_BIAS]; qa.bv = w.v[WGB_L_ATTN_V_BIAS];
        qa.q_out = pf.q;
        qa.k_cache = m->key_cache + l * cache_stride;
        qa.v_cache = m->value_cache + l * cache_stride;
        qa.q_dim = q_dim; qa.kv_dim = kv_dim; qa.head_size = m->head_size; qa.seq_len = c.seq_len; qa.pos0 = pos0;
        qa.variant = variant;
        qa.freq = m->rope_freq;
        if ((rc = launch_prefill_rope_append(qa, ntok, s))) return rc;
        const bool attn_image = prefill_attention_writes_image(m->head_size);
        if ((rc = launch_prefill_attention(pf.q, qa.k_cache, qa.v_cache, pf.xb, m->n_q_local, m->head_size, m->kv_mul, m->head_size,
                                           c.seq_len * m->head_size, pos0, ntok,
                                           attn_image ? pf.img_q : nullptr, pf.attn_scratch, pf.attn_counters, s)))
            return rc;
        if (!attn_image && (rc = launch_prefill_norm_image(pf.xb, q_dim, nullptr, 0, 0, nullptr, 0.0f, q_dim, ntok, pf.img_q, nullptr, 0, s))) return rc;
        if ((rc = prefill_product(m, l, WGB_L_ATTN_OUTPUT, pf.img_q, pf.xb, q_dim, ntok, pf.part[0], dim, &no, s))) return rc;
        const float *opart = pf.part[0];
        if ((rc = across_ranks(&opart, &no))) return rc;
        if ((rc = launch_prefill_norm_image(pf.x, dim, opart, no, dim, w.v[WGB_L_FFN_NORM], c.rms_norm_eps, dim, ntok, pf.img_dim, pf.xn, dim, s)))
            return rc;
        {
            const int which[2] = { WGB_L_FFN_GATE, WGB_L_FFN_UP };
            const uint32_t strides[2] = { hidden, hidden };
            uint32_t ns[2];
            if ((rc = prefill_products(m, l, which, 2, pf.img_dim, pf.xn, dim, ntok, pf.part, strides, ns, s))) return rc;
            ng = ns[0]; nu = ns[1];
        }
        if ((rc = launch_prefill_silu_image(pf.part[0], ng, pf.part[1], nu, hidden, hidden, ntok, pf.img_hidden, pf.h, hidden, s))) return rc;
        if ((rc = prefill_product(m, l, WGB_L_FFN_DOWN, pf.img_hidden, pf.h, hidden, ntok, pf.part[2], dim, &nd, s))) return rc;
        pending = pf.part[2];
        pending_split = nd;
        if ((rc = across_ranks(&pending, &pending_split))) return rc;
    }
    // leave the residual stream of the pass complete (nothing reads it; it keeps wgb_llama2_x meaningful for tests)
    if ((rc = launch_prefill_norm_image(pf.x, dim, pending, pending_split, dim, nullptr, 0.0f, dim, ntok, nullptr, nullptr, 0, s))) return rc;
    pf.positions += ntok;
    return WGB_OK;
}

void drop_graph(wgb_llama2 *m)
{
    if (m->graph) cudaGraphExecDestroy(m->graph);
    m->graph = nullptr;
}

// Local counters of the direct exchange: one ticket per exchange and the step count.
int alloc_exchange_counters(wgb_llama2 *m)
{
    const size_t n_ex = 2 * (size_t)m->cfg.n_layers;
    if (!m->tickets) {
        WGB_CUDA(cudaMalloc((void **)&m->tickets, n_ex * sizeof(uint32_t)));
        WGB_CUDA(cudaMemset(m->tickets, 0, n_ex * sizeof(uint32_t)));
    }
    if (!m->tp_epoch) {
        WGB_CUDA(cudaMalloc((void **)&m->tp_epoch, sizeof(uint32_t)));
        WGB_CUDA(cudaMemset(m->tp_epoch, 0, sizeof(uint32_t)));
    }
    return WGB_OK;
}

}  // namespace

WGB_EXPORT int wgb_llama2_create(const wgb_llama2_config *cfg, int model_type, int tp_rank, int tp_size, wgb_llama2 **out)
{
    WGB_REQUIRE(cfg && out, "null argument");
    WGB_REQUIRE(model_type == WGB_LLAMA || model_type == WGB_QWEN2, "unknown model type %d", model_type);
    WGB_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, "bad tensor-parallel rank %d of %d", tp_rank, tp_size);
    const wgb_llama2_config &c = *cfg;
    WGB_REQUIRE(c.dim && c.hidden_dim && c.n_layers && c.n_q_heads && c.n_kv_heads && c.vocab_size && c.seq_len, "zero-sized config");
    WGB_REQUIRE(c.dim % c.n_q_heads == 0 && c.n_q_heads % c.n_kv_heads == 0, "head counts do not divide the model dimension");
    const uint32_t hs = c.dim / c.n_q_heads;
    WGB_REQUIRE(hs % 4 == 0 && hs <= 256, "head size %u unsupported (multiple of 4, at most 256)", hs);
    WGB_REQUIRE(c.dim % 4 == 0 && c.hidden_dim % 4 == 0, "dimensions must be multiples of 4");
    WGB_REQUIRE(c.n_kv_heads % tp_size == 0, "n_kv_heads %u is not a multiple of the tensor-parallel size %d", c.n_kv_heads, tp_size);
    { const int rc0 = gemv_global_init(); if (rc0) return rc0; }
    wgb_llama2 *m = new (std::nothrow) wgb_llama2();
    if (!m) return fail(WGB_ERR_INVALID, "out of host memory");
    m->cfg = c;
    m->model_type = model_type;
    m->tp_rank = tp_rank;
    m->tp_size = tp_size;
    m->head_size = hs;
    m->kv_mul = c.n_q_heads / c.n_kv_heads;
    m->n_kv_local = c.n_kv_heads / tp_size;
    m->n_q_local = m->n_kv_local * m->kv_mul;
    m->q_dim = m->n_q_local * hs;
    m->kv_dim = m->n_kv_local * hs;
    if (tp_size == 1) {
        m->hidden_blk0 = 0;
        m->hidden_blks = 0;
        m->hidden = c.hidden_dim;
    } else {
        if (c.hidden_dim % 256 != 0) { delete m; return fail(WGB_ERR_INVALID, "tensor parallelism needs hidden_dim %% 256 == 0"); }
        const uint32_t nb = c.hidden_dim / 256;
        m->hidden_blk0 = (uint32_t)((uint64_t)nb * tp_rank / tp_size);
        m->hidden_blks = (uint32_t)((uint64_t)nb * (tp_rank + 1) / tp_size) - m->hidden_blk0;
        m->hidden = m->hidden_blks * 256;
        if (m->hidden == 0) { delete m; return fail(WGB_ERR_INVALID, "more ranks than 256-column FFN blocks"); }
    }
    m->layers.resize(c.n_layers);
    int rc = WGB_OK;
    const size_t cache = (size_t)c.n_layers * c.seq_len * m->kv_dim;
    if ((rc = dalloc(&m->x, c.dim)) || (rc = dalloc(&m->xb, c.dim)) || (rc = dalloc(&m->xb2, c.dim)) ||
        (rc = dalloc(&m->hb, m->hidden)) || (rc = dalloc(&m->hb2, m->hidden)) || (rc = dalloc(&m->q, m->q_dim)) ||
        (rc = dalloc(&m->tk, m->kv_dim)) || (rc = dalloc(&m->tv, m->kv_dim)) || (rc = dalloc(&m->logits, c.vocab_size)) ||
        (rc = dalloc(&m->key_cache, cache)) || (rc = dalloc(&m->value_cache, cache)) ||
        (rc = dalloc(&m->attn_scratch, attn_scratch_floats(m->n_q_local, hs, c.seq_len))) ||
        (rc = dalloc(&m->rope_freq, hs / 2 + 4))) {
        wgb_llama2_destroy(m);
        return rc;
    }
    cudaError_t e;
    if ((e = cudaMalloc((void **)&m->attn_counters, (size_t)m->n_q_local * 4)) != cudaSuccess ||
        (e = cudaMemset(m->attn_counters, 0, (size_t)m->n_q_local * 4)) != cudaSuccess ||
        (e = cudaMalloc((void **)&m->scalars, 16)) != cudaSuccess || (e = cudaMemset(m->scalars, 0, 16)) != cudaSuccess ||
        (e = cudaMalloc((void **)&m->argmax_scratch, 64 * 8)) != cudaSuccess) {
        wgb_llama2_destroy(m);
        return cuda_fail(e, "cudaMalloc(model state)");
    }
    std::vector<float> freq(hs / 2);
    rope_inv_freq(hs, c.rope_base_freq, freq.data());
    if ((e = cudaMemcpy(m->rope_freq, freq.data(), freq.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess) {
        wgb_llama2_destroy(m);
        return cuda_fail(e, "cudaMemcpy(rope table)");
    }
    const char *env = getenv("WGB_NO_PDL");
    if (env && env[0] == '1') m->use_pdl = false;
    *out = m;
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_destroy(wgb_llama2 *m)
{
    if (!m) return WGB_OK;
    drop_graph(m);
    prefill_free(m);
    for (auto &l : m->layers) {
        for (auto *q : l.m) wgb_quant_matrix_destroy(q);
        for (auto *v : l.v) if (v) cudaFree(v);
    }
    wgb_quant_matrix_destroy(m->token_embd);
    wgb_quant_matrix_destroy(m->output);
    float *bufs[] = { m->output_norm, m->x, m->xb, m->xb2, m->hb, m->hb2, m->q, m->tk, m->tv, m->logits, m->key_cache,
                      m->value_cache, m->attn_scratch, m->rope_freq };
    for (float *b : bufs) if (b) cudaFree(b);
    if (m->stamps) cudaFree(m->stamps);
    if (m->tickets) cudaFree(m->tickets);
    if (m->tp_epoch) cudaFree(m->tp_epoch);
    m->stamps = nullptr;
    m->tickets = m->tp_epoch = nullptr;
    status_poll_destroy(m->poll);
    m->up.destroy();
    if (m->smp_scratch) cudaFree(m->smp_scratch);
    uint32_t *ubufs[] = { m->attn_counters, m->scalars, m->argmax_scratch, m->d_prompt, m->d_out };
    for (uint32_t *b : ubufs) if (b) cudaFree(b);
    if (m->h_pinned) cudaFreeHost(m->h_pinned);
    delete m;
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_set_matrix(wgb_llama2 *m, int layer, int which, int qtype, const void *h_blocks, size_t nrows,
                                     size_t ncols)
{
    WGB_REQUIRE(m && h_blocks, "null argument");
    if (m->pf.enabled) prefill_free(m);   // its tile-major copies would go stale
    const wgb_llama2_config &c = m->cfg;
    const int bl = block_len(qtype);
    if (!bl) return fail(WGB_ERR_UNSUPPORTED, "unsupported tensor type %d", qtype);
    const uint32_t hs = m->head_size, full_kv = c.n_kv_heads * hs;
    size_t exp_rows, exp_cols, row0 = 0, rows_keep, kb0 = 0, kb_keep;
    wgb_quant_matrix **slot;
    if (layer < 0) {
        WGB_REQUIRE(which == WGB_L_TOKEN_EMBD || which == WGB_L_OUTPUT, "unknown model matrix %d", which);
        exp_rows = c.vocab_size; exp_cols = c.dim; rows_keep = exp_rows; kb_keep = exp_cols / bl;
        slot = which == WGB_L_TOKEN_EMBD ? &m->token_embd : &m->output;
    } else {
        WGB_REQUIRE((uint32_t)layer < c.n_layers && which >= 0 && which < 7, "layer %d / matrix %d out of range", layer, which);
        slot = &m->layers[layer].m[which];
        switch (which) {
        case WGB_L_ATTN_Q: exp_rows = c.dim; exp_cols = c.dim; row0 = (size_t)m->tp_rank * m->q_dim; rows_keep = m->q_dim; kb_keep = exp_cols / bl; break;
        case WGB_L_ATTN_K: case WGB_L_ATTN_V:
            exp_rows = full_kv; exp_cols = c.dim; row0 = (size_t)m->tp_rank * m->kv_dim; rows_keep = m->kv_dim; kb_keep = exp_cols / bl; break;
        case WGB_L_ATTN_OUTPUT:
            exp_rows = c.dim; exp_cols = c.dim; rows_keep = exp_rows;
            WGB_REQUIRE(m->q_dim % bl == 0, "attention slice of %u columns is not a multiple of the block length %d", m->q_dim, bl);
            kb0 = (size_t)m->tp_rank * m->q_dim / bl; kb_keep = m->q_dim / bl; break;
        case WGB_L_FFN_GATE: case WGB_L_FFN_UP:
            exp_rows = c.hidden_dim; exp_cols = c.dim; kb_keep = exp_cols / bl;
            row0 = m->tp_size == 1 ? 0 : (size_t)m->hidden_blk0 * 256; rows_keep = m->hidden; break;
        default:  // WGB_L_FFN_DOWN
            exp_rows = c.dim; exp_cols = c.hidden_dim; rows_keep = exp_rows;
            kb0 = m->tp_size == 1 ? 0 : (size_t)m->hidden_blk0 * 256 / bl; kb_keep = m->hidden / bl; break;
        }
    }
    WGB_REQUIRE(nrows == exp_rows && ncols == exp_cols, "matrix is %zu x %zu, the model expects %zu x %zu", nrows, ncols, exp_rows, exp_cols);
    WGB_REQUIRE(ncols % bl == 0, "ncols %zu is not a multiple of the block length %d", ncols, bl);
    wgb_quant_matrix *q = nullptr;
    int rc = qmat_create_slice_async(m->up, qtype, h_blocks, nrows, ncols, row0, rows_keep, kb0, kb_keep, &q);
    if (rc) return rc;
    // a caller of its own may release h_blocks on return; the GGUF loader keeps the file mapped until it has waited
    if (!m->loading && (rc = m->up.finish())) { wgb_quant_matrix_destroy(q); return rc; }
    wgb_quant_matrix_destroy(*slot);
    *slot = q;
    drop_graph(m);
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_set_vector(wgb_llama2 *m, int layer, int which, const float *h_data, size_t n)
{
    WGB_REQUIRE(m && h_data, "null argument");
    const wgb_llama2_config &c = m->cfg;
    float **slot;
    size_t expect, off = 0, keep;
    if (layer < 0) {
        slot = &m->output_norm;
        expect = keep = c.dim;
    } else {
        WGB_REQUIRE((uint32_t)layer < c.n_layers && which >= 0 && which < 5, "layer %d / vector %d out of range", layer, which);
        slot = &m->layers[layer].v[which];
        if (which == WGB_L_ATTN_NORM || which == WGB_L_FFN_NORM) { expect = keep = c.dim; }
        else if (which == WGB_L_ATTN_Q_BIAS) { expect = c.dim; keep = m->q_dim; off = (size_t)m->tp_rank * m->q_dim; }
        else { expect = (size_t)c.n_kv_heads * m->head_size; keep = m->kv_dim; off = (size_t)m->tp_rank * m->kv_dim; }
    }
    WGB_REQUIRE(n == expect, "vector has %zu entries, the model expects %zu", n, expect);
    if (!*slot) WGB_CUDA(cudaMalloc((void **)slot, keep * sizeof(float)));
    WGB_CUDA(cudaMemcpy(*slot, h_data + off, keep * sizeof(float), cudaMemcpyHostToDevice));
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_config_from_gguf(const wgb_gguf *g, int model_type, wgb_llama2_config *out)
{
    WGB_REQUIRE(g && out, "null argument");
    const char *name = model_type == WGB_QWEN2 ? "qwen2" : "llama";  // models/llama2/mod.rs:19-24
    auto key = [&](const char *suffix) { return std::string(name) + "." + suffix; };
    auto get_u32 = [&](const std::string &k, uint32_t *v) -> int {
        const int64_t i = wgb_gguf_meta_find(g, k.c_str());
        if (i < 0) return fail(WGB_ERR_NOT_FOUND, "missing GGUF key '%s'", k.c_str());
        int type = 0;
        wgb_gguf_meta_type(g, (uint64_t)i, &type, nullptr, nullptr);
        if (type != WGB_META_U32) return fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type for '%s'.", k.c_str());
        uint64_t u = 0;
        wgb_gguf_meta_u64(g, (uint64_t)i, &u);
        *v = (uint32_t)u;
        return WGB_OK;
    };
    auto get_f32 = [&](const std::string &k, float dflt, float *v) -> int {
        const int64_t i = wgb_gguf_meta_find(g, k.c_str());
        if (i < 0) { *v = dflt; return WGB_OK; }
        int type = 0;
        wgb_gguf_meta_type(g, (uint64_t)i, &type, nullptr, nullptr);
        if (type != WGB_META_F32) return fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type for '%s'.", k.c_str());
        double d = 0;
        wgb_gguf_meta_f64(g, (uint64_t)i, &d);
        *v = (float)d;
        return WGB_OK;
    };
    int rc;
    // cpu.rs:79-109
    if ((rc = get_u32(key("embedding_length"), &out->dim)) || (rc = get_u32(key("feed_forward_length"), &out->hidden_dim)) ||
        (rc = get_u32(key("block_count"), &out->n_layers)) || (rc = get_u32(key("attention.head_count"), &out->n_q_heads)) ||
        (rc = get_u32(key("attention.head_count_kv"), &out->n_kv_heads)) || (rc = get_u32(key("context_length"), &out->seq_len)))
        return rc;
    const int64_t ti = wgb_gguf_meta_find(g, "tokenizer.ggml.tokens");
    if (ti < 0) return fail(WGB_ERR_NOT_FOUND, "missing GGUF key 'tokenizer.ggml.tokens'");
    int type = 0;
    uint64_t len = 0;
    wgb_gguf_meta_type(g, (uint64_t)ti, &type, nullptr, &len);
    if (type != WGB_META_ARRAY) return fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type for 'tokenizer.ggml.tokens'.");
    out->vocab_size = (uint32_t)len;
    if ((rc = get_f32(key("rope.freq_base"), 10000.0f, &out->rope_base_freq)) ||
        (rc = get_f32(key("attention.layer_norm_rms_epsilon"), 1.0e-6f, &out->rms_norm_eps)))
        return rc;
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_load_gguf(wgb_llama2 *m, const wgb_gguf *g)
{
    WGB_REQUIRE(m && g, "null argument");
    const wgb_llama2_config &c = m->cfg;
    const uint32_t full_kv = c.n_kv_heads * m->head_size;
    auto find = [&](const std::string &name, bool required, wgb_gguf_tensor *t) -> int {
        const int64_t i = wgb_gguf_tensor_find(g, name.c_str());
        if (i < 0) return required ? fail(WGB_ERR_NOT_FOUND, "missing GGUF tensor '%s'", name.c_str()) : -1;
        const int rc = wgb_gguf_tensor_info(g, (uint64_t)i, t);
        if (rc) return rc;
        if (!t->data) return fail(WGB_ERR_UNSUPPORTED, "tensor '%s' has unsupported type %u", name.c_str(), t->type);
        return WGB_OK;
    };
    auto mat = [&](int layer, int which, const std::string &name, size_t nrows, size_t ncols, bool required) -> int {
        wgb_gguf_tensor t;
        int rc = find(name, required, &t);
        if (rc == -1) return WGB_OK;
        if (rc) return rc;
        if (t.dims[0] * t.dims[1] * t.dims[2] * t.dims[3] != nrows * ncols)
            return fail(WGB_ERR_INVALID, "tensor '%s' has %llu elements, expected %zu x %zu", name.c_str(),
                        (unsigned long long)(t.dims[0] * t.dims[1] * t.dims[2] * t.dims[3]), nrows, ncols);
        return wgb_llama2_set_matrix(m, layer, which, (int)t.type, t.data, nrows, ncols);
    };
    auto vec = [&](int layer, int which, const std::string &name, size_t n, bool required) -> int {
        wgb_gguf_tensor t;
        int rc = find(name, required, &t);
        if (rc == -1) return WGB_OK;
        if (rc) return rc;
        if (t.type != WGB_F32) return fail(WGB_ERR_INVALID, "tensor '%s' must be f32", name.c_str());  // as_f32().unwrap()
        if (t.n_bytes != n * 4) return fail(WGB_ERR_INVALID, "tensor '%s' has %llu bytes, expected %zu", name.c_str(), (unsigned long long)t.n_bytes, n * 4);
        return wgb_llama2_set_vector(m, layer, which, (const float *)t.data, n);
    };
    // Every tensor's bytes are enqueued on the upload stream (pinned ring, repack kernels) without waiting; one
    // wait at the end.  The figures of the batch are kept for wgb_llama2_load_stats.
    m->loading = true;
    struct Done {
        wgb_llama2 *m;
        ~Done() { m->up.finish(); m->loading = false; }
    } done{m};
    int rc;
    for (uint32_t l = 0; l < c.n_layers; l++) {
        const std::string p = "blk." + std::to_string(l) + ".";
        // transformer.rs:161-216
        if ((rc = mat(l, WGB_L_ATTN_Q, p + "attn_q.weight", c.dim, c.dim, true)) ||
            (rc = mat(l, WGB_L_ATTN_K, p + "attn_k.weight", full_kv, c.dim, true)) ||
            (rc = mat(l, WGB_L_ATTN_V, p + "attn_v.weight", full_kv, c.dim, true)) ||
            (rc = mat(l, WGB_L_ATTN_OUTPUT, p + "attn_output.weight", c.dim, c.dim, true)) ||
            (rc = mat(l, WGB_L_FFN_DOWN, p + "ffn_down.weight", c.dim, c.hidden_dim, true)) ||
            (rc = mat(l, WGB_L_FFN_GATE, p + "ffn_gate.weight", c.hidden_dim, c.dim, true)) ||
            (rc = mat(l, WGB_L_FFN_UP, p + "ffn_up.weight", c.hidden_dim, c.dim, true)) ||
            (rc = vec(l, WGB_L_ATTN_NORM, p + "attn_norm.weight", c.dim, true)) ||
            (rc = vec(l, WGB_L_FFN_NORM, p + "ffn_norm.weight", c.dim, true)) ||
            (rc = vec(l, WGB_L_ATTN_Q_BIAS, p + "attn_q.bias", c.dim, false)) ||
            (rc = vec(l, WGB_L_ATTN_K_BIAS, p + "attn_k.bias", full_kv, false)) ||
            (rc = vec(l, WGB_L_ATTN_V_BIAS, p + "attn_v.bias", full_kv, false)))
            return rc;
    }
    // transformer.rs:235-260
    if ((rc = mat(-1, WGB_L_TOKEN_EMBD, "token_embd.weight", c.vocab_size, c.dim, true)) ||
        (rc = mat(-1, WGB_L_OUTPUT, "output.weight", c.vocab_size, c.dim, false)) ||
        (rc = vec(-1, 0, "output_norm.weight", c.dim, true)))
        return rc;
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_set_comm(wgb_llama2 *m, void *comm)
{
    WGB_REQUIRE(m, "null argument");
    WGB_REQUIRE(!comm || (wgb_comm_size((wgb_comm *)comm) == m->tp_size && wgb_comm_rank((wgb_comm *)comm) == m->tp_rank),
                "communicator rank/size does not match the model's tensor-parallel rank %d of %d", m->tp_rank, m->tp_size);
    m->comm = comm;
    drop_graph(m);
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_set_vocab_shard(wgb_llama2 *m, int on)
{
    WGB_REQUIRE(m, "null argument");
    const bool want = on != 0 && m->tp_size > 1;
    if (want)
        WGB_REQUIRE(m->cfg.vocab_size % (uint32_t)m->tp_size == 0, "a vocabulary of %u rows does not split evenly over %d ranks",
                    m->cfg.vocab_size, m->tp_size);
    m->vocab_shard = want;
    drop_graph(m);
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_set_exchange(wgb_llama2 *m, int mode)
{
    WGB_REQUIRE(m && (mode == 0 || mode == 1), "bad argument");
    if (m->tp_size == 1 || mode == 0) {
        m->exchange = 0;
        drop_graph(m);
        return WGB_OK;
    }
    WGB_REQUIRE(m->tp_size <= PEER_MAX, "direct exchange supports at most %d ranks", PEER_MAX);
    if (!m->mail_peer[0]) {
        WGB_REQUIRE(m->comm, "set the communicator first (or map the buffers yourself: wgb_llama2_set_exchange_buffers)");
        size_t mail_bytes = 0, flag_bytes = 0;
        wgb_llama2_exchange_bytes(m, &mail_bytes, &flag_bytes);
        void *peers[PEER_MAX] = {};
        int rc = wgb_comm_shared_alloc((wgb_comm *)m->comm, mail_bytes + flag_bytes, peers);
        if (rc) return rc;
        for (int p = 0; p < m->tp_size; p++) {
            m->mail_peer[p] = (float *)peers[p];
            m->flag_peer[p] = (uint32_t *)((char *)peers[p] + mail_bytes);
        }
    }
    int rc = alloc_exchange_counters(m);
    if (rc) return rc;
    m->exchange = 1;
    drop_graph(m);
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_exchange_bytes(const wgb_llama2 *m, size_t *mail_bytes, size_t *flag_bytes)
{
    WGB_REQUIRE(m && mail_bytes && flag_bytes, "null argument");
    const size_t n_ex = 2 * (size_t)m->cfg.n_layers;
    *mail_bytes = n_ex * m->tp_size * m->cfg.dim * sizeof(float);
    *flag_bytes = n_ex * m->tp_size * sizeof(uint32_t);
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_set_exchange_buffers(wgb_llama2 *m, void *const *d_mail, void *const *d_flags)
{
    WGB_REQUIRE(m && d_mail && d_flags, "null argument");
    WGB_REQUIRE(m->tp_size > 1 && m->tp_size <= PEER_MAX, "direct exchange wants 2..%d ranks, the model has %d", PEER_MAX, m->tp_size);
    WGB_REQUIRE(!m->mail_peer[0] || m->exchange_external, "the exchange buffers of this model were already allocated through its communicator");
    for (int p = 0; p < m->tp_size; p++) {
        WGB_REQUIRE(d_mail[p] && d_flags[p], "rank %d: null buffer", p);
        WGB_REQUIRE(((uintptr_t)d_mail[p] % 16) == 0 && ((uintptr_t)d_flags[p] % 4) == 0, "rank %d: misaligned buffer", p);
    }
    for (int p = 0; p < m->tp_size; p++) {
        m->mail_peer[p] = (float *)d_mail[p];
        m->flag_peer[p] = (uint32_t *)d_flags[p];
    }
    m->exchange_external = true;
    int rc = alloc_exchange_counters(m);
    if (rc) return rc;
    m->exchange = 1;
    drop_graph(m);
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_set_fused(wgb_llama2 *m, int enable)
{
    WGB_REQUIRE(m, "null argument");
    m->fused = enable != 0;
    drop_graph(m);
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_forward(wgb_llama2 *m, uint32_t token, uint32_t pos, void *stream)
{
    WGB_REQUIRE(m, "null argument");
    int rc = check_complete(m);
    if (rc) return rc;
    WGB_REQUIRE(token < m->cfg.vocab_size, "token %u outside a vocabulary of %u", token, m->cfg.vocab_size);
    WGB_REQUIRE(pos < m->cfg.seq_len, "position %u outside a context of %u", pos, m->cfg.seq_len);
    WGB_REQUIRE(m->tp_size == 1 || m->comm || (m->exchange == 1 && m->exchange_external), "tensor-parallel model without a communicator");
    cudaStream_t s = as_stream(stream);
    set_scalars_kernel<<<1, 1, 0, s>>>(m->scalars, token, pos, 0);
    WGB_LAUNCH_CHECK("set_scalars_kernel");
    m->pos_bound = pos;
    return enqueue_forward(m, s, &m->kernels_per_token);
}

// One forward with an event after every launch.  `as_graph`: the launches and event records are captured
// into a CUDA graph and replayed once, so that the gaps between launches are the device's, not the time the
// host needs to issue a launch; otherwise they are issued one by one.
static int profile_once(wgb_llama2 *m, cudaStream_t s, bool as_graph, int cap, int *kinds, int *layers, float *ms, int *n_out)
{
    m->profiling = true;
    m->prof_events.clear();
    m->prof_kind.clear();
    m->prof_layer.clear();
    cudaEvent_t start = nullptr;
    cudaError_t e = cudaEventCreate(&start);
    int rc = WGB_OK;
    if (e == cudaSuccess && as_graph) {
        cudaStream_t cs = nullptr;
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        e = cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal);
        if (e == cudaSuccess) {
            e = cudaEventRecord(start, cs);
            if (e == cudaSuccess) rc = enqueue_forward(m, cs, nullptr);
            cudaError_t e2 = cudaStreamEndCapture(cs, &graph);
            if (e == cudaSuccess) e = e2;
        }
        if (e == cudaSuccess && rc == WGB_OK) e = cudaGraphInstantiate(&exec, graph, 0);
        if (e == cudaSuccess && rc == WGB_OK) e = cudaGraphLaunch(exec, s);
        if (e == cudaSuccess && rc == WGB_OK) e = cudaStreamSynchronize(s);
        if (exec) cudaGraphExecDestroy(exec);
        if (graph) cudaGraphDestroy(graph);
        if (cs) cudaStreamDestroy(cs);
    } else if (e == cudaSuccess) {
        e = cudaEventRecord(start, s);
        if (e == cudaSuccess) rc = enqueue_forward(m, s, nullptr);
        cudaError_t e2 = cudaStreamSynchronize(s);
        if (e == cudaSuccess) e = e2;
    }
    m->profiling = false;
    int n = 0;
    cudaEvent_t prev = start;
    for (size_t i = 0; i < m->prof_events.size(); i++) {
        if (rc == WGB_OK && e == cudaSuccess && n < cap) {
            float t = 0.0f;
            e = cudaEventElapsedTime(&t, prev, m->prof_events[i]);
            kinds[n] = m->prof_kind[i];
            layers[n] = m->prof_layer[i];
            ms[n] = t;
            n++;
        }
        if (prev != start) cudaEventDestroy(prev);
        prev = m->prof_events[i];
    }
    if (prev != start && prev) cudaEventDestroy(prev);
    if (start) cudaEventDestroy(start);
    m->prof_events.clear();
    *n_out = n;
    if (rc) return rc;
    if (e != cudaSuccess) { cudaGetLastError(); return cuda_fail(e, "profile step"); }
    return WGB_OK;
}

// The fused schedule exactly as a decode step runs it (one CUDA graph, programmatic dependent launch), each
// launch leaving its end time in device memory; a launch's time is the distance to its predecessor's end,
// which is what it adds to the step (the embedding copy is counted with the first launch).
static int profile_stamped(wgb_llama2 *m, cudaStream_t s, int cap, int *kinds, int *layers, float *ms, int *n_out)
{
    const size_t need = 5 * (size_t)m->cfg.n_layers + 2;
    if (need > m->stamps_cap) {
        if (m->stamps) cudaFree(m->stamps);
        m->stamps = nullptr;
        m->stamps_cap = 0;
        WGB_CUDA(cudaMalloc((void **)&m->stamps, need * sizeof(unsigned long long)));
        m->stamps_cap = need;
    }
    m->stamping = true;
    m->prof_kind.clear();
    m->prof_layer.clear();
    cudaStream_t cs = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int rc = WGB_OK;
    cudaError_t e = cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
        rc = enqueue_forward(m, cs, nullptr);
        e = cudaStreamEndCapture(cs, &graph);
    }
    m->stamping = false;
    if (e == cudaSuccess && rc == WGB_OK) e = cudaGraphInstantiate(&exec, graph, 0);
    std::vector<unsigned long long> h(need, 0);
    for (int rep = 0; rep < 2 && e == cudaSuccess && rc == WGB_OK; rep++) {   // the second replay is the one read
        e = cudaMemsetAsync(m->stamps, 0, need * sizeof(unsigned long long), s);
        if (e == cudaSuccess) e = cudaGraphLaunch(exec, s);
    }
    if (e == cudaSuccess && rc == WGB_OK) e = cudaMemcpyAsync(h.data(), m->stamps, need * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess && rc == WGB_OK) e = cudaStreamSynchronize(s);
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    if (cs) cudaStreamDestroy(cs);
    int n = 0;
    if (e == cudaSuccess && rc == WGB_OK) {
        for (size_t i = 0; i < m->prof_kind.size() && i + 1 < need && n < cap; i++) {
            kinds[n] = m->prof_kind[i];
            layers[n] = m->prof_layer[i];
            ms[n] = h[i + 1] > h[i] ? (float)((double)(h[i + 1] - h[i]) * 1e-6) : 0.0f;
            n++;
        }
    }
    *n_out = n;
    if (rc) return rc;
    if (e != cudaSuccess) return cuda_fail(e, "stamped profile step");
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_profile_step(wgb_llama2 *m, uint32_t token, uint32_t pos, void *stream, int cap, int *kinds,
                                       int *layers, float *ms, int *n_out)
{
    WGB_REQUIRE(m && kinds && layers && ms && n_out, "null argument");
    int rc = check_complete(m);
    if (rc) return rc;
    WGB_REQUIRE(token < m->cfg.vocab_size && pos < m->cfg.seq_len, "token / position out of range");
    cudaStream_t s = as_stream(stream);
    set_scalars_kernel<<<1, 1, 0, s>>>(m->scalars, token, pos, 0);
    WGB_LAUNCH_CHECK("set_scalars_kernel");
    m->pos_bound = pos;
    if (m->fused && fusable(m) && (m->tp_size == 1 || m->exchange == 1)) return profile_stamped(m, s, cap, kinds, layers, ms, n_out);
    rc = profile_once(m, s, true, cap, kinds, layers, ms, n_out);
    if (rc == WGB_ERR_CUDA) {   // events inside a captured graph unavailable: issue the launches one by one
        set_scalars_kernel<<<1, 1, 0, s>>>(m->scalars, token, pos, 0);
        WGB_LAUNCH_CHECK("set_scalars_kernel");
        rc = profile_once(m, s, false, cap, kinds, layers, ms, n_out);
    }
    return rc;
}

WGB_EXPORT const float *wgb_llama2_logits(const wgb_llama2 *m) { return m ? m->logits : nullptr; }
WGB_EXPORT const float *wgb_llama2_x(const wgb_llama2 *m) { return m ? m->x : nullptr; }
WGB_EXPORT float *wgb_llama2_key_cache(wgb_llama2 *m, uint32_t layer)
{
    return (m && layer < m->cfg.n_layers) ? m->key_cache + (size_t)layer * m->cfg.seq_len * m->kv_dim : nullptr;
}
WGB_EXPORT float *wgb_llama2_value_cache(wgb_llama2 *m, uint32_t layer)
{
    return (m && layer < m->cfg.n_layers) ? m->value_cache + (size_t)layer * m->cfg.seq_len * m->kv_dim : nullptr;
}
WGB_EXPORT int wgb_llama2_kernels_per_token(const wgb_llama2 *m) { return m ? m->kernels_per_token : 0; }

WGB_EXPORT int wgb_llama2_decode(wgb_llama2 *m, const uint32_t *h_prompt, size_t n_prompt, size_t n_gen, uint32_t start_pos,
                                 uint32_t *h_out_tokens, void *stream)
{
    WGB_REQUIRE(m && h_prompt && n_prompt >= 1, "null or empty prompt");
    int rc = check_complete(m);
    if (rc) return rc;
    const size_t total = n_prompt - 1 + n_gen;
    if (total == 0) return WGB_OK;
    WGB_REQUIRE(h_out_tokens, "null output");
    WGB_REQUIRE((size_t)start_pos + total <= m->cfg.seq_len, "%zu steps from position %u overrun a context of %u", total, start_pos,
                m->cfg.seq_len);
    for (size_t i = 0; i < n_prompt; i++)
        WGB_REQUIRE(h_prompt[i] < m->cfg.vocab_size, "prompt token %u outside a vocabulary of %u", h_prompt[i], m->cfg.vocab_size);
    WGB_REQUIRE(m->tp_size == 1 || m->comm || (m->exchange == 1 && m->exchange_external), "tensor-parallel model without a communicator");
    cudaStream_t s = as_stream(stream);
    if (n_prompt > m->prompt_cap) {
        if (m->d_prompt) cudaFree(m->d_prompt);
        m->d_prompt = nullptr;
        m->prompt_cap = 0;
        drop_graph(m);
        WGB_CUDA(cudaMalloc((void **)&m->d_prompt, n_prompt * 4));
        m->prompt_cap = n_prompt;
    }
    if (total > m->out_cap) {
        if (m->d_out) cudaFree(m->d_out);
        m->d_out = nullptr;
        m->out_cap = 0;
        drop_graph(m);
        WGB_CUDA(cudaMalloc((void **)&m->d_out, total * 4));
        m->out_cap = total;
    }
    if (total + 3 > m->pinned_cap) {
        if (m->h_pinned) cudaFreeHost(m->h_pinned);
        m->h_pinned = nullptr;
        m->pinned_cap = 0;
        WGB_CUDA(cudaMallocHost((void **)&m->h_pinned, (total + 3) * 4));
        m->pinned_cap = total + 3;
    }
    // the first token travels as a kernel argument; the rest of the prompt is only read when there is one
    if (n_prompt > 1) WGB_CUDA(cudaMemcpyAsync(m->d_prompt, h_prompt, n_prompt * 4, cudaMemcpyHostToDevice, s));
    // Batched prefill: every prompt position but the last (whose logits choose the first generated token) may go
    // through passes of PF_TOK positions; a remainder shorter than half a pass stays with the token loop.
    size_t done = 0;
    if (m->pf.enabled && n_prompt - 1 >= PF_TOK) {
        const size_t rem = (n_prompt - 1) % PF_TOK;
        const size_t batched = n_prompt - 1 - (rem >= PF_TOK / 2 ? 0 : rem);
        for (; done < batched; done += PF_TOK) {
            const uint32_t nt = (uint32_t)(batched - done < PF_TOK ? batched - done : PF_TOK);
            if ((rc = prefill_pass(m, s, m->d_prompt + done, start_pos + (uint32_t)done, nt))) return rc;
        }
        done = batched;
        // the token loop reports prompt[i + 1] for step i < n_prompt - 1
        WGB_CUDA(cudaMemcpyAsync(m->d_out, m->d_prompt + 1, done * 4, cudaMemcpyDeviceToDevice, s));
    }
    set_scalars_kernel<<<1, 1, 0, s>>>(m->scalars, h_prompt[done], start_pos + (uint32_t)done, (uint32_t)done);
    WGB_LAUNCH_CHECK("set_scalars_kernel");

    LoopState ls = {};
    ls.token = m->scalars;
    ls.pos = m->scalars + 1;
    ls.step = m->scalars + 2;
    ls.prompt = m->d_prompt;
    ls.n_prompt = (uint32_t)n_prompt;
    ls.out_tokens = m->d_out;

    // The attention launch is sized for the furthest position of this call; the captured step is kept until
    // that changes the shape of the launch (once in the life of a sequence).
    m->pos_bound = (uint32_t)((size_t)start_pos + total - 1);
    wgb_attn_params ap = {};
    ap.seq_len = m->cfg.seq_len;
    ap.kv_dim = m->kv_dim;
    ap.kv_mul = m->kv_mul;
    ap.n_heads = m->n_q_local;
    ap.head_size = m->head_size;
    ap.pos = m->pos_bound;
    const int attn_class = attn_sizing_class(ap);
    WGB_REQUIRE(attn_class >= 0, "attention sizing failed");
    if (m->graph && (m->graph_n_prompt != (uint32_t)n_prompt || m->graph_attn_chunks != (uint32_t)attn_class)) drop_graph(m);
    if (!m->graph) {
        // Capture one step on a private stream (capturing on the legacy default stream is not allowed).
        cudaStream_t cs;
        WGB_CUDA(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal);
        if (e == cudaSuccess) {
            int nk = 0;
            rc = enqueue_forward(m, cs, &nk);
            if (!rc && m->smp_temperature == 0.0f) {
                rc = launch_argmax_advance(m->logits, m->cfg.vocab_size, ls, m->argmax_scratch, cs);
                m->kernels_per_token = nk + 2;
            } else if (!rc) {
                rc = launch_sample(m->logits, m->cfg.vocab_size, m->smp_temperature, m->smp_topp, 0.0f, 1, m->smp_seed, m->smp_scratch, nullptr,
                                   &ls, cs);
                m->kernels_per_token = nk + 1;
            }
            e = cudaStreamEndCapture(cs, &graph);
            if (rc) { if (graph) cudaGraphDestroy(graph); cudaStreamDestroy(cs); return rc; }
        }
        if (e == cudaSuccess) e = cudaGraphInstantiate(&m->graph, graph, 0);
        if (graph) cudaGraphDestroy(graph);
        cudaStreamDestroy(cs);
        if (e != cudaSuccess) { m->graph = nullptr; return cuda_fail(e, "CUDA graph capture of a decode step"); }
        m->graph_n_prompt = (uint32_t)n_prompt;
        m->graph_attn_chunks = (uint32_t)attn_class;
    }
    if ((rc = replay_with_status(m->graph, total - done, s, m->h_pinned + 1, m->poll))) return rc;
    // One wait for the ids and the kernels' status word, both through pinned memory.
    WGB_CUDA(cudaMemcpyAsync(m->h_pinned + 3, m->d_out, total * 4, cudaMemcpyDeviceToHost, s));
    m->h_pinned[0] = 0;
    if (gemv_status_word()) WGB_CUDA(cudaMemcpyAsync(m->h_pinned, gemv_status_word(), 4, cudaMemcpyDeviceToHost, s));
    WGB_CUDA(cudaStreamSynchronize(s));
    memcpy(h_out_tokens, m->h_pinned + 3, total * 4);
    return gemv_report_status(m->h_pinned[0]);
}

WGB_EXPORT int wgb_llama2_set_prefill(wgb_llama2 *m, int enable)
{
    WGB_REQUIRE(m, "null argument");
    if (!enable) {
        prefill_free(m);
        return WGB_OK;
    }
    if (m->pf.enabled) return WGB_OK;
    if (m->tp_size != 1 && !m->comm)
        return fail(WGB_ERR_UNSUPPORTED, "batched prefill of a tensor-parallel model sums its partial products with the communicator: call wgb_llama2_set_comm first (rank %d of %d)",
                    m->tp_rank, m->tp_size);
    int rc = check_complete(m);
    if (rc) return rc;
    if ((rc = gemv_global_init())) return rc;
    const wgb_llama2_config &c = m->cfg;
    WGB_REQUIRE(c.dim % 256 == 0 && m->q_dim % 256 == 0 && m->hidden % 256 == 0 && m->kv_dim % 4 == 0 && m->head_size % 4 == 0 && m->head_size <= 256,
                "batched prefill wants widths that are multiples of 256 (dim %u, attention width %u, hidden %u) and a head size up to 256", c.dim,
                m->q_dim, m->hidden);
    wgb_llama2::Prefill &pf = m->pf;
    pf.tiles.assign((size_t)c.n_layers * 7, nullptr);
    pf.tiles_q6.assign((size_t)c.n_layers * 7, 0);
    auto bail = [&](int code) { prefill_free(m); return code; };
    for (uint32_t l = 0; l < c.n_layers; l++)
        for (int i = 0; i < 7; i++) {
            const QMat &w = m->layers[l].m[i]->view;
            if (prefill_tileable(w) && (rc = prefill_tile_major(w, &pf.tiles[(size_t)l * 7 + i], nullptr))) return bail(rc);
            if (prefill_tileable6(w)) {
                if ((rc = prefill_tile_major6(w, &pf.tiles[(size_t)l * 7 + i], nullptr))) return bail(rc);
                pf.tiles_q6[(size_t)l * 7 + i] = 1;
            }
            if (prefill_tileable8(w)) {
                if ((rc = prefill_tile_major8(w, &pf.tiles[(size_t)l * 7 + i], nullptr))) return bail(rc);
                pf.tiles_q6[(size_t)l * 7 + i] = 2;
            }
        }
    auto image = [&](uint8_t **p, uint32_t K) -> int {
        WGB_CUDA(cudaMalloc((void **)p, prefill_image_bytes(K)));
        WGB_CUDA(cudaMemset(*p, 0, prefill_image_bytes(K)));
        return WGB_OK;
    };
    if ((rc = image(&pf.img_dim, c.dim)) || (rc = image(&pf.img_q, m->q_dim)) || (rc = image(&pf.img_hidden, m->hidden))) return bail(rc);
    const size_t widest = std::max<size_t>(std::max<size_t>(c.dim, m->q_dim), m->hidden);
    WGB_CUDA(cudaMalloc((void **)&pf.img6, prefill_image6_bytes((uint32_t)widest)));
    if ((rc = dalloc(&pf.x, (size_t)PF_TOK * c.dim)) || (rc = dalloc(&pf.xn, (size_t)PF_TOK * c.dim)) || (rc = dalloc(&pf.q, (size_t)PF_TOK * m->q_dim)) ||
        (rc = dalloc(&pf.xb, (size_t)PF_TOK * m->q_dim)) || (rc = dalloc(&pf.h, (size_t)PF_TOK * m->hidden)))
        return bail(rc);
    for (int i = 0; i < 3; i++)
        if ((rc = dalloc(&pf.part[i], (size_t)PF_MAX_SPLIT * PF_TOK * widest))) return bail(rc);
    if (m->tp_size > 1 && (rc = dalloc(&pf.red, (size_t)PF_TOK * c.dim))) return bail(rc);
    if ((rc = dalloc(&pf.attn_scratch, prefill_attention_scratch_floats(m->n_q_local, m->head_size)))) return bail(rc);
    {
        const size_t nc = prefill_attention_counters(m->n_q_local);
        cudaError_t e = cudaMalloc((void **)&pf.attn_counters, nc * 4);
        if (e == cudaSuccess) e = cudaMemset(pf.attn_counters, 0, nc * 4);
        if (e != cudaSuccess) { prefill_free(m); return cuda_fail(e, "cudaMalloc(prompt attention counters)"); }
    }
    WGB_CUDA(cudaDeviceSynchronize());
    pf.enabled = true;
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_prefill_positions(const wgb_llama2 *m, size_t *positions)
{
    WGB_REQUIRE(m && positions, "null argument");
    *positions = m->pf.positions;
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_set_sampler(wgb_llama2 *m, float temperature, float topp, uint64_t seed)
{
    WGB_REQUIRE(m, "null argument");
    WGB_REQUIRE(temperature >= 0.0f, "negative temperature %g", temperature);
    if (temperature > 0.0f && !m->smp_scratch) WGB_CUDA(cudaMalloc(&m->smp_scratch, sampler_scratch_bytes(m->cfg.vocab_size)));
    m->smp_temperature = temperature;
    m->smp_topp = topp;
    m->smp_seed = seed;
    drop_graph(m);   // the parameters are baked into the recorded step
    return WGB_OK;
}

WGB_EXPORT int wgb_llama2_load_stats(const wgb_llama2 *m, size_t *bytes, double *seconds)
{
    WGB_REQUIRE(m && bytes && seconds, "null argument");
    *bytes = m->up.total_bytes;
    *seconds = m->up.total_seconds;
    return WGB_OK;
}
