// GPT-2 decoder: weights, state, one-token forward and the device-resident greedy loop.
//
// Follows Gpt2::dispatch (crates/wgml/src/models/gpt2/transformer.rs:265-477) and the loop of
// ChatGpt2::forward (crates/wgml-chat/src/chat_gpt2.rs:43-151).  Matrices stay in their GGUF
// blocks (the reference dequantises them to f32 at load, transformer.rs:133-140).  Schedules:
//   fused    [LayerNorm*g+b + QKV product + bias + split into q / KV append]  [attention]
//            [proj + bias + residual]  [LayerNorm*g+b + fc + bias + GELU]  [proj + bias + residual]
//   unfused  one launch per reference dispatch.
#include "kernels.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

using namespace wgb;

struct wgb_gpt2 {
    wgb_gpt2_params p;
    struct Layer {
        wgb_quant_matrix *m[4] = {};
        float *v[8] = {};
    };
    std::vector<Layer> layers;
    wgb_quant_matrix *wte = nullptr, *wpe = nullptr;
    float *ln_f_g = nullptr, *ln_f_b = nullptr;
    // Gpt2State (transformer.rs:14-68)
    float *layer_input = nullptr, *curr_768 = nullptr, *curr_768_b = nullptr, *curr_2304 = nullptr, *curr_3072 = nullptr,
          *memory_q = nullptr, *logits = nullptr;
    float *key_cache = nullptr, *value_cache = nullptr;  // [n_layer][n_seq][n_embd]
    float *attn_scratch = nullptr;
    uint32_t *attn_counters = nullptr, *scalars = nullptr, *argmax_scratch = nullptr, *d_prompt = nullptr, *d_out = nullptr;
    size_t prompt_cap = 0, out_cap = 0;
    uint32_t *h_pinned = nullptr;            // pinned staging of a decode call: [0] status word, [1..2] status polls, [3..] token ids
    size_t pinned_cap = 0;
    StatusPoll poll;
    // sampling of generated tokens: temperature 0 = greedy (Sampler::sample, models/sampler.rs:32-52)
    float smp_temperature = 0.0f, smp_topp = 0.0f;
    unsigned long long smp_seed = 0;
    void *smp_scratch = nullptr;
    bool fused = true, use_pdl = true;
    cudaGraphExec_t graph = nullptr;
    uint32_t graph_n_prompt = 0;
    int kernels_per_token = 0;
    // batched prompt prefill (wgb_gpt2_set_prefill): tile-major copies of the layer matrices for the tensor-core
    // products, activation images and the buffers of a pass of PF_TOK positions
    struct Prefill {
        bool enabled = false;
        std::vector<uint8_t *> tiles;        // [layer * 4 + matrix], NULL: no tensor-core path for that matrix
        std::vector<uint8_t> kind;           // same index: 0 a Q4_K copy, 1 a Q6_K one, 2 a Q8_0 one
        uint8_t *img_e = nullptr, *img_a = nullptr, *img_h = nullptr, *img6 = nullptr;   // images of n_embd / n_embd / ff_len columns
        float *x = nullptr, *xn = nullptr, *q = nullptr, *xb = nullptr, *h = nullptr;     // [PF_TOK][n_embd | ff_len]
        float *part[3] = {};                 // product slices: [PF_MAX_SPLIT][PF_TOK][max(3 n_embd, ff_len)]
        float *attn_scratch = nullptr;
        uint32_t *attn_counters = nullptr, *pos = nullptr;   // pos: the PF_TOK positions of a pass
        size_t positions = 0;
    } pf;
};

namespace {

__global__ void set_scalars_kernel(uint32_t *s, uint32_t token, uint32_t pos, uint32_t step)
{
    s[0] = token;
    s[1] = pos;
    s[2] = step;
}

// Unfused path: the three Copy dispatches of transformer.rs:329-353 with the position on the device.
__global__ void qkv_split_kernel(const float *__restrict__ qkv, float *__restrict__ q, float *__restrict__ k_cache,
                                 float *__restrict__ v_cache, const uint32_t *__restrict__ d_pos, uint32_t n)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t pos = *d_pos;
    q[i] = qkv[i];
    k_cache[(size_t)pos * n + i] = qkv[n + i];
    v_cache[(size_t)pos * n + i] = qkv[2 * n + i];
}

int dalloc(float **p, size_t n)
{
    WGB_CUDA(cudaMalloc((void **)p, n * sizeof(float)));
    WGB_CUDA(cudaMemset(*p, 0, n * sizeof(float)));
    return WGB_OK;
}

bool fusable(const wgb_gpt2 *m)
{
    for (const auto &l : m->layers)
        for (int i = 0; i < 4; i++)
            if (!l.m[i] || !gemv_fast_supported(l.m[i]->view)) return false;
    return m->wte && gemv_fast_supported(m->wte->view);
}

int check_complete(const wgb_gpt2 *m)
{
    for (size_t l = 0; l < m->layers.size(); l++) {
        for (int i = 0; i < 4; i++)
            if (!m->layers[l].m[i]) return fail(WGB_ERR_NOT_FOUND, "layer %zu: matrix %d was never set", l, i);
        for (int i = 0; i < 8; i++)
            if (!m->layers[l].v[i]) return fail(WGB_ERR_NOT_FOUND, "layer %zu: vector %d was never set", l, i);
    }
    if (!m->wte || !m->wpe) return fail(WGB_ERR_NOT_FOUND, "token_embd.weight / position_embd.weight was never set");
    if (!m->ln_f_g || !m->ln_f_b) return fail(WGB_ERR_NOT_FOUND, "output_norm was never set");
    return WGB_OK;
}

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

int enqueue_forward(wgb_gpt2 *m, cudaStream_t s, int *nkernels)
{
    const wgb_gpt2_params &p = m->p;
    const uint32_t n = p.n_embd;
    const uint32_t *d_token = m->scalars, *d_pos = m->scalars + 1;
    const bool fused = m->fused && fusable(m);
    const bool pdl = m->use_pdl;
    int nk = 0, rc;
    // transformer.rs:277-290
    if ((rc = launch_embed(m->wte->view, &m->wpe->view, d_token, d_pos, m->layer_input, s))) return rc;
    nk++;
    const size_t cache_stride = (size_t)p.n_seq * n;
    AttnArgs at = {};
    at.p.seq_len = p.n_seq;
    at.p.kv_dim = n;
    at.p.kv_mul = 1;
    at.p.n_heads = p.n_head;
    at.p.head_size = n / p.n_head;
    at.pos = d_pos;
    at.q = m->memory_q;
    at.xb = m->curr_768;
    at.scratch = m->attn_scratch;
    at.counters = m->attn_counters;
    at.err = gemv_status_word();
    for (uint32_t l = 0; l < p.n_layer; l++) {
        const wgb_gpt2::Layer &w = m->layers[l];
        float *kc = m->key_cache + l * cache_stride, *vc = m->value_cache + l * cache_stride;
        at.k_cache = kc;
        at.v_cache = vc;
        if (fused) {
            GemvArgs a = {};
            a.mat[0] = w.m[WGB_G_ATTN_QKV]->view;
            a.nmat = 1;
            a.x = m->layer_input;
            a.prologue = PRO_LN;
            a.norm_w = w.v[WGB_G_LN_1_G];
            a.norm_b = w.v[WGB_G_LN_1_B];
            a.epilogue = EPI_QKV_SPLIT;
            a.bias = w.v[WGB_G_ATTN_QKV_B];
            a.out = m->memory_q;
            a.k_cache = kc;
            a.v_cache = vc;
            a.pos = d_pos;
            a.kv_dim = n;
            if ((rc = launch_gemv(a, s, pdl))) return rc;
            if ((rc = launch_attention(at, s, pdl))) return rc;
            GemvArgs o = {};
            o.mat[0] = w.m[WGB_G_ATTN_PROJ]->view;
            o.nmat = 1;
            o.x = m->curr_768;
            o.epilogue = EPI_RESIDUAL;
            o.bias = w.v[WGB_G_ATTN_PROJ_B];
            o.residual = m->layer_input;
            o.out = m->layer_input;
            if ((rc = launch_gemv(o, s, pdl))) return rc;
            GemvArgs f = {};
            f.mat[0] = w.m[WGB_G_MLP_FC]->view;
            f.nmat = 1;
            f.x = m->layer_input;
            f.prologue = PRO_LN;
            f.norm_w = w.v[WGB_G_LN_2_G];
            f.norm_b = w.v[WGB_G_LN_2_B];
            f.epilogue = EPI_GELU;
            f.bias = w.v[WGB_G_MLP_FC_B];
            f.out = m->curr_3072;
            if ((rc = launch_gemv(f, s, pdl))) return rc;
            GemvArgs d = {};
            d.mat[0] = w.m[WGB_G_MLP_PROJ]->view;
            d.nmat = 1;
            d.x = m->curr_3072;
            d.epilogue = EPI_RESIDUAL;
            d.bias = w.v[WGB_G_MLP_PROJ_B];
            d.residual = m->layer_input;
            d.out = m->layer_input;
            if ((rc = launch_gemv(d, s, pdl))) return rc;
            nk += 5;
        } else {
            // transformer.rs:295-452, dispatch by dispatch
            if ((rc = wgb_layernorm(m->curr_768, m->layer_input, n, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_MUL, m->curr_768, w.v[WGB_G_LN_1_G], n, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->curr_768, w.v[WGB_G_LN_1_B], n, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_G_ATTN_QKV]->view, m->curr_768, m->curr_2304, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->curr_2304, w.v[WGB_G_ATTN_QKV_B], 3 * (size_t)n, s))) return rc;
            qkv_split_kernel<<<(n + 127) / 128, 128, 0, s>>>(m->curr_2304, m->memory_q, kc, vc, d_pos, n);
            WGB_LAUNCH_CHECK("qkv_split_kernel");
            if ((rc = launch_attention(at, s, false))) return rc;
            if ((rc = mat_vec(w.m[WGB_G_ATTN_PROJ]->view, m->curr_768, m->curr_768_b, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->curr_768_b, w.v[WGB_G_ATTN_PROJ_B], n, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->curr_768_b, m->layer_input, n, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_COPY, m->layer_input, m->curr_768_b, n, s))) return rc;
            if ((rc = wgb_layernorm(m->curr_768, m->curr_768_b, n, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_MUL, m->curr_768, w.v[WGB_G_LN_2_G], n, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->curr_768, w.v[WGB_G_LN_2_B], n, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_G_MLP_FC]->view, m->curr_768, m->curr_3072, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->curr_3072, w.v[WGB_G_MLP_FC_B], p.ff_len, s))) return rc;
            if ((rc = wgb_unary_inplace(WGB_UNARY_GELU, m->curr_3072, p.ff_len, nullptr, s))) return rc;
            if ((rc = mat_vec(w.m[WGB_G_MLP_PROJ]->view, m->curr_3072, m->curr_768, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->curr_768, w.v[WGB_G_MLP_PROJ_B], n, s))) return rc;
            if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->layer_input, m->curr_768, n, s))) return rc;
            nk += 20;
        }
    }
    if (fused) {
        GemvArgs a = {};
        a.mat[0] = m->wte->view;
        a.nmat = 1;
        a.x = m->layer_input;
        a.prologue = PRO_LN;
        a.norm_w = m->ln_f_g;
        a.norm_b = m->ln_f_b;
        a.epilogue = EPI_STORE;
        a.out = m->logits;
        if ((rc = launch_gemv(a, s, pdl))) return rc;
        nk += 1;
    } else {
        // transformer.rs:457-476
        if ((rc = wgb_layernorm(m->curr_768, m->layer_input, n, s))) return rc;
        if ((rc = wgb_op_assign(WGB_ASSIGN_MUL, m->curr_768, m->ln_f_g, n, s))) return rc;
        if ((rc = wgb_op_assign(WGB_ASSIGN_ADD, m->curr_768, m->ln_f_b, n, s))) return rc;
        if ((rc = mat_vec(m->wte->view, m->curr_768, m->logits, s))) return rc;
        nk += 4;
    }
    if (nkernels) *nkernels = nk;
    return WGB_OK;
}

void prefill_free(wgb_gpt2 *m)
{
    for (uint8_t *t : m->pf.tiles) if (t) cudaFree(t);
    uint8_t *imgs[] = { m->pf.img_e, m->pf.img_a, m->pf.img_h, m->pf.img6 };
    for (uint8_t *b : imgs) if (b) cudaFree(b);
    float *bufs[] = { m->pf.x, m->pf.xn, m->pf.q, m->pf.xb, m->pf.h, m->pf.part[0], m->pf.part[1], m->pf.part[2], m->pf.attn_scratch };
    for (float *b : bufs) if (b) cudaFree(b);
    if (m->pf.attn_counters) cudaFree(m->pf.attn_counters);
    if (m->pf.pos) cudaFree(m->pf.pos);
    m->pf = wgb_gpt2::Prefill();
}

// One product of a prefill pass: W . (the `ntok` vectors whose image is `image` and whose values are xf), as slices
// [slice][PF_TOK][stride] in `out`; matrices without a tile-major copy go through the matrix-vector kernel per position.
int prefill_product(wgb_gpt2 *m, uint32_t layer, int which, const uint8_t *image, const float *xf, uint32_t xf_stride, uint32_t ntok, float *out,
                    uint32_t stride, uint32_t *nsplit, cudaStream_t s)
{
    const QMat &w = m->layers[layer].m[which]->view;
    const size_t idx = (size_t)layer * 4 + which;
    const uint8_t *tiles = m->pf.tiles[idx];
    if (tiles) {
        *nsplit = prefill_gemm_splits(w.nrows, w.ncols);
        if (m->pf.kind[idx] == 2) return launch_gemm_q80_tiles(tiles, w.nrows, w.ncols, image, ntok, out, stride, *nsplit, s);
        if (m->pf.kind[idx] == 1) {
            int rc = launch_prefill_image6(xf, xf_stride, w.ncols, ntok, m->pf.img6, s);
            return rc ? rc : launch_gemm_q6k_tiles(tiles, w.nrows, w.ncols, m->pf.img6, ntok, out, stride, *nsplit, s);
        }
        return launch_gemm_q4k_tiles(tiles, w.nrows, w.ncols, image, ntok, out, stride, *nsplit, s);
    }
    *nsplit = 1;
    for (uint32_t t = 0; t < ntok; t++) {
        int rc = mat_vec(w, xf + (size_t)t * xf_stride, out + (size_t)t * stride, s);
        if (rc) return rc;
    }
    return WGB_OK;
}

// Prompt positions pos0 .. pos0 + ntok - 1 (tokens d_tokens[0 .. ntok)) through the layer stack in one pass: the work
// of ntok calls of Gpt2::dispatch (models/gpt2/transformer.rs:265-477) up to the last layer's cache rows; the final
// LayerNorm and the logits of prompt positions are never looked at (chat_gpt2.rs:43-151 samples after the prompt).
int prefill_pass(wgb_gpt2 *m, cudaStream_t s, const uint32_t *d_tokens, uint32_t pos0, uint32_t ntok)
{
    const wgb_gpt2_params &p = m->p;
    wgb_gpt2::Prefill &pf = m->pf;
    const uint32_t n = p.n_embd, ff = p.ff_len, hs = n / p.n_head;
    int rc;
    if ((rc = launch_prefill_positions(pf.pos, pos0, s))) return rc;
    for (uint32_t t = 0; t < ntok; t++)
        if ((rc = launch_embed(m->wte->view, &m->wpe->view, d_tokens + t, pf.pos + t, pf.x + (size_t)t * n, s))) return rc;
    const size_t cache_stride = (size_t)p.n_seq * n;
    const bool attn_image = prefill_attention_writes_image(hs);
    const float *pending = nullptr, *pending_bias = nullptr;   // the last layer's second projection and its bias
    uint32_t pending_split = 0;
    for (uint32_t l = 0; l < p.n_layer; l++) {
        const wgb_gpt2::Layer &w = m->layers[l];
        float *kc = m->key_cache + l * cache_stride, *vc = m->value_cache + l * cache_stride;
        uint32_t nq, no, nf, nd;
        if ((rc = launch_prefill_ln_image(pf.x, n, pending, pending_split, n, pending_bias, w.v[WGB_G_LN_1_G], w.v[WGB_G_LN_1_B], n, ntok, pf.img_e, pf.xn,
                                          n, s)))
            return rc;
        if ((rc = prefill_product(m, l, WGB_G_ATTN_QKV, pf.img_e, pf.xn, n, ntok, pf.part[0], 3 * n, &nq, s))) return rc;
        if ((rc = launch_prefill_qkv_split(pf.part[0], nq, w.v[WGB_G_ATTN_QKV_B], pf.q, kc, vc, n, pos0, ntok, s))) return rc;
        if ((rc = launch_prefill_attention(pf.q, kc, vc, pf.xb, p.n_head, hs, 1, n, hs, pos0, ntok, attn_image ? pf.img_a : nullptr, pf.attn_scratch,
                                           pf.attn_counters, s)))
            return rc;
        if (!attn_image && (rc = launch_prefill_norm_image(pf.xb, n, nullptr, 0, 0, nullptr, 0.0f, n, ntok, pf.img_a, nullptr, 0, s))) return rc;
        if ((rc = prefill_product(m, l, WGB_G_ATTN_PROJ, pf.img_a, pf.xb, n, ntok, pf.part[1], n, &no, s))) return rc;
        if ((rc = launch_prefill_ln_image(pf.x, n, pf.part[1], no, n, w.v[WGB_G_ATTN_PROJ_B], w.v[WGB_G_LN_2_G], w.v[WGB_G_LN_2_B], n, ntok, pf.img_e,
                                          pf.xn, n, s)))
            return rc;
        if ((rc = prefill_product(m, l, WGB_G_MLP_FC, pf.img_e, pf.xn, n, ntok, pf.part[0], ff, &nf, s))) return rc;
        if ((rc = launch_prefill_gelu_image(pf.part[0], nf, ff, w.v[WGB_G_MLP_FC_B], ff, ntok, pf.img_h, pf.h, ff, s))) return rc;
        if ((rc = prefill_product(m, l, WGB_G_MLP_PROJ, pf.img_h, pf.h, ff, ntok, pf.part[2], n, &nd, s))) return rc;
        pending = pf.part[2];
        pending_bias = w.v[WGB_G_MLP_PROJ_B];
        pending_split = nd;
    }
    // leave the residual stream of the pass complete
    if ((rc = launch_prefill_ln_image(pf.x, n, pending, pending_split, n, pending_bias, nullptr, nullptr, n, ntok, nullptr, nullptr, 0, s))) return rc;
    pf.positions += ntok;
    return WGB_OK;
}

void drop_graph(wgb_gpt2 *m)
{
    if (m->graph) cudaGraphExecDestroy(m->graph);
    m->graph = nullptr;
}

}  // namespace

WGB_EXPORT int wgb_gpt2_create(const wgb_gpt2_params *params, wgb_gpt2 **out)
{
    WGB_REQUIRE(params && out, "null argument");
    const wgb_gpt2_params &p = *params;
    WGB_REQUIRE(p.n_vocab && p.n_seq && p.n_embd && p.n_head && p.n_layer && p.ff_len, "zero-sized parameters");
    WGB_REQUIRE(p.n_embd % p.n_head == 0, "n_embd %u is not a multiple of n_head %u", p.n_embd, p.n_head);
    const uint32_t hs = p.n_embd / p.n_head;
    WGB_REQUIRE(hs % 4 == 0 && hs <= 256, "head size %u unsupported (multiple of 4, at most 256)", hs);
    WGB_REQUIRE(p.attn_b == 0 || p.attn_b == 3 * p.n_embd, "attn_b %u is not 3 * n_embd", p.attn_b);
    { const int rc0 = gemv_global_init(); if (rc0) return rc0; }
    wgb_gpt2 *m = new (std::nothrow) wgb_gpt2();
    if (!m) return fail(WGB_ERR_INVALID, "out of host memory");
    m->p = p;
    m->p.attn_b = 3 * p.n_embd;
    m->layers.resize(p.n_layer);
    int rc;
    const size_t cache = (size_t)p.n_layer * p.n_seq * p.n_embd;
    if ((rc = dalloc(&m->layer_input, p.n_embd)) || (rc = dalloc(&m->curr_768, p.n_embd)) || (rc = dalloc(&m->curr_768_b, p.n_embd)) ||
        (rc = dalloc(&m->curr_2304, 3 * (size_t)p.n_embd)) || (rc = dalloc(&m->curr_3072, p.ff_len)) ||
        (rc = dalloc(&m->memory_q, p.n_embd)) || (rc = dalloc(&m->logits, p.n_vocab)) || (rc = dalloc(&m->key_cache, cache)) ||
        (rc = dalloc(&m->value_cache, cache)) || (rc = dalloc(&m->attn_scratch, attn_scratch_floats(p.n_head, hs, p.n_seq)))) {
        wgb_gpt2_destroy(m);
        return rc;
    }
    cudaError_t e;
    if ((e = cudaMalloc((void **)&m->attn_counters, (size_t)p.n_head * 4)) != cudaSuccess ||
        (e = cudaMemset(m->attn_counters, 0, (size_t)p.n_head * 4)) != cudaSuccess ||
        (e = cudaMalloc((void **)&m->scalars, 16)) != cudaSuccess || (e = cudaMemset(m->scalars, 0, 16)) != cudaSuccess ||
        (e = cudaMalloc((void **)&m->argmax_scratch, 64 * 8)) != cudaSuccess) {
        wgb_gpt2_destroy(m);
        return cuda_fail(e, "cudaMalloc(model state)");
    }
    const char *env = getenv("WGB_NO_PDL");
    if (env && env[0] == '1') m->use_pdl = false;
    *out = m;
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_destroy(wgb_gpt2 *m)
{
    if (!m) return WGB_OK;
    drop_graph(m);
    prefill_free(m);
    for (auto &l : m->layers) {
        for (auto *q : l.m) wgb_quant_matrix_destroy(q);
        for (auto *v : l.v) if (v) cudaFree(v);
    }
    wgb_quant_matrix_destroy(m->wte);
    wgb_quant_matrix_destroy(m->wpe);
    float *bufs[] = { m->ln_f_g, m->ln_f_b, m->layer_input, m->curr_768, m->curr_768_b, m->curr_2304, m->curr_3072, m->memory_q,
                      m->logits, m->key_cache, m->value_cache, m->attn_scratch };
    for (float *b : bufs) if (b) cudaFree(b);
    uint32_t *ubufs[] = { m->attn_counters, m->scalars, m->argmax_scratch, m->d_prompt, m->d_out };
    for (uint32_t *b : ubufs) if (b) cudaFree(b);
    if (m->h_pinned) cudaFreeHost(m->h_pinned);
    status_poll_destroy(m->poll);
    if (m->smp_scratch) cudaFree(m->smp_scratch);
    delete m;
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_set_matrix(wgb_gpt2 *m, int layer, int which, int qtype, const void *h_blocks, size_t nrows, size_t ncols)
{
    WGB_REQUIRE(m && h_blocks, "null argument");
    if (m->pf.enabled) prefill_free(m);   // its tile-major copies would go stale
    const wgb_gpt2_params &p = m->p;
    size_t er, ec;
    wgb_quant_matrix **slot;
    if (layer < 0) {
        WGB_REQUIRE(which == WGB_G_WTE || which == WGB_G_WPE, "unknown model matrix %d", which);
        er = which == WGB_G_WTE ? p.n_vocab : p.n_seq;
        ec = p.n_embd;
        slot = which == WGB_G_WTE ? &m->wte : &m->wpe;
    } else {
        WGB_REQUIRE((uint32_t)layer < p.n_layer && which >= 0 && which < 4, "layer %d / matrix %d out of range", layer, which);
        slot = &m->layers[layer].m[which];
        switch (which) {
        case WGB_G_ATTN_QKV: er = 3 * (size_t)p.n_embd; ec = p.n_embd; break;
        case WGB_G_ATTN_PROJ: er = p.n_embd; ec = p.n_embd; break;
        case WGB_G_MLP_FC: er = p.ff_len; ec = p.n_embd; break;
        default: er = p.n_embd; ec = p.ff_len; break;
        }
    }
    WGB_REQUIRE(nrows == er && ncols == ec, "matrix is %zu x %zu, the model expects %zu x %zu", nrows, ncols, er, ec);
    wgb_quant_matrix *q = nullptr;
    const int rc = qmat_create(qtype, h_blocks, false, nrows, ncols, nullptr, &q);
    if (rc) return rc;
    WGB_CUDA(cudaStreamSynchronize(nullptr));
    wgb_quant_matrix_destroy(*slot);
    *slot = q;
    drop_graph(m);
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_set_vector(wgb_gpt2 *m, int layer, int which, const float *h_data, size_t n)
{
    WGB_REQUIRE(m && h_data, "null argument");
    const wgb_gpt2_params &p = m->p;
    float **slot;
    size_t expect;
    if (layer < 0) {
        WGB_REQUIRE(which == WGB_G_LN_F_G || which == WGB_G_LN_F_B, "unknown model vector %d", which);
        slot = which == WGB_G_LN_F_G ? &m->ln_f_g : &m->ln_f_b;
        expect = p.n_embd;
    } else {
        WGB_REQUIRE((uint32_t)layer < p.n_layer && which >= 0 && which < 8, "layer %d / vector %d out of range", layer, which);
        slot = &m->layers[layer].v[which];
        expect = which == WGB_G_ATTN_QKV_B ? 3 * (size_t)p.n_embd : (which == WGB_G_MLP_FC_B ? p.ff_len : p.n_embd);
    }
    WGB_REQUIRE(n == expect, "vector has %zu entries, the model expects %zu", n, expect);
    if (!*slot) WGB_CUDA(cudaMalloc((void **)slot, n * sizeof(float)));
    WGB_CUDA(cudaMemcpy(*slot, h_data, n * sizeof(float), cudaMemcpyHostToDevice));
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_params_from_gguf(const wgb_gguf *g, wgb_gpt2_params *out)
{
    WGB_REQUIRE(g && out, "null argument");
    auto get_u32 = [&](const char *k, uint32_t *v) -> int {
        const int64_t i = wgb_gguf_meta_find(g, k);
        if (i < 0) return fail(WGB_ERR_NOT_FOUND, "missing GGUF key '%s'", k);
        int type = 0;
        wgb_gguf_meta_type(g, (uint64_t)i, &type, nullptr, nullptr);
        if (type != WGB_META_U32) return fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type for '%s'.", k);
        uint64_t u = 0;
        wgb_gguf_meta_u64(g, (uint64_t)i, &u);
        *v = (uint32_t)u;
        return WGB_OK;
    };
    int rc;
    // gpt2/cpu.rs:36-47
    const int64_t ti = wgb_gguf_meta_find(g, "tokenizer.ggml.tokens");
    if (ti < 0) return fail(WGB_ERR_NOT_FOUND, "missing GGUF key 'tokenizer.ggml.tokens'");
    int type = 0;
    uint64_t len = 0;
    wgb_gguf_meta_type(g, (uint64_t)ti, &type, nullptr, &len);
    if (type != WGB_META_ARRAY) return fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type for 'tokenizer.ggml.tokens'.");
    out->n_vocab = (uint32_t)len;
    if ((rc = get_u32("gpt2.context_length", &out->n_seq)) || (rc = get_u32("gpt2.embedding_length", &out->n_embd)) ||
        (rc = get_u32("gpt2.attention.head_count", &out->n_head)) || (rc = get_u32("gpt2.block_count", &out->n_layer)) ||
        (rc = get_u32("general.file_type", &out->ftype)) || (rc = get_u32("gpt2.feed_forward_length", &out->ff_len)))
        return rc;
    const int64_t bi = wgb_gguf_tensor_find(g, "blk.0.attn_qkv.bias");
    if (bi < 0) return fail(WGB_ERR_NOT_FOUND, "missing GGUF tensor 'blk.0.attn_qkv.bias'");
    wgb_gguf_tensor t;
    if ((rc = wgb_gguf_tensor_info(g, (uint64_t)bi, &t))) return rc;
    out->attn_b = (uint32_t)t.dims[0];
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_load_gguf(wgb_gpt2 *m, const wgb_gguf *g)
{
    WGB_REQUIRE(m && g, "null argument");
    const wgb_gpt2_params &p = m->p;
    auto find = [&](const std::string &name, wgb_gguf_tensor *t) -> int {
        const int64_t i = wgb_gguf_tensor_find(g, name.c_str());
        if (i < 0) return fail(WGB_ERR_NOT_FOUND, "missing GGUF tensor '%s'", name.c_str());
        const int rc = wgb_gguf_tensor_info(g, (uint64_t)i, t);
        if (rc) return rc;
        if (!t->data) return fail(WGB_ERR_UNSUPPORTED, "tensor '%s' has unsupported type %u", name.c_str(), t->type);
        return WGB_OK;
    };
    auto mat = [&](int layer, int which, const std::string &name, size_t nrows, size_t ncols) -> int {
        wgb_gguf_tensor t;
        int rc = find(name, &t);
        if (rc) return rc;
        if (t.dims[0] * t.dims[1] * t.dims[2] * t.dims[3] != nrows * ncols)
            return fail(WGB_ERR_INVALID, "tensor '%s' does not have %zu x %zu elements", name.c_str(), nrows, ncols);
        return wgb_gpt2_set_matrix(m, layer, which, (int)t.type, t.data, nrows, ncols);
    };
    auto vec = [&](int layer, int which, const std::string &name, size_t n) -> int {
        wgb_gguf_tensor t;
        int rc = find(name, &t);
        if (rc) return rc;
        if (t.type != WGB_F32 || t.n_bytes != n * 4) return fail(WGB_ERR_INVALID, "tensor '%s' must be f32 with %zu entries", name.c_str(), n);
        return wgb_gpt2_set_vector(m, layer, which, (const float *)t.data, n);
    };
    int rc;
    const size_t n = p.n_embd;
    for (uint32_t l = 0; l < p.n_layer; l++) {
        const std::string b = "blk." + std::to_string(l) + ".";
        // transformer.rs:115-156
        if ((rc = vec(l, WGB_G_LN_1_G, b + "attn_norm.weight", n)) || (rc = vec(l, WGB_G_LN_1_B, b + "attn_norm.bias", n)) ||
            (rc = vec(l, WGB_G_LN_2_G, b + "ffn_norm.weight", n)) || (rc = vec(l, WGB_G_LN_2_B, b + "ffn_norm.bias", n)) ||
            (rc = mat(l, WGB_G_ATTN_QKV, b + "attn_qkv.weight", 3 * n, n)) || (rc = vec(l, WGB_G_ATTN_QKV_B, b + "attn_qkv.bias", 3 * n)) ||
            (rc = mat(l, WGB_G_ATTN_PROJ, b + "attn_output.weight", n, n)) || (rc = vec(l, WGB_G_ATTN_PROJ_B, b + "attn_output.bias", n)) ||
            (rc = mat(l, WGB_G_MLP_FC, b + "ffn_up.weight", p.ff_len, n)) || (rc = vec(l, WGB_G_MLP_FC_B, b + "ffn_up.bias", p.ff_len)) ||
            (rc = mat(l, WGB_G_MLP_PROJ, b + "ffn_down.weight", n, p.ff_len)) || (rc = vec(l, WGB_G_MLP_PROJ_B, b + "ffn_down.bias", n)))
            return rc;
    }
    // transformer.rs:179-195
    if ((rc = vec(-1, WGB_G_LN_F_G, "output_norm.weight", n)) || (rc = vec(-1, WGB_G_LN_F_B, "output_norm.bias", n)) ||
        (rc = mat(-1, WGB_G_WTE, "token_embd.weight", p.n_vocab, n)) || (rc = mat(-1, WGB_G_WPE, "position_embd.weight", p.n_seq, n)))
        return rc;
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_set_fused(wgb_gpt2 *m, int enable)
{
    WGB_REQUIRE(m, "null argument");
    m->fused = enable != 0;
    drop_graph(m);
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_forward(wgb_gpt2 *m, uint32_t token, uint32_t pos, void *stream)
{
    WGB_REQUIRE(m, "null argument");
    int rc = check_complete(m);
    if (rc) return rc;
    WGB_REQUIRE(token < m->p.n_vocab, "token %u outside a vocabulary of %u", token, m->p.n_vocab);
    WGB_REQUIRE(pos < m->p.n_seq, "position %u outside a context of %u", pos, m->p.n_seq);
    cudaStream_t s = as_stream(stream);
    set_scalars_kernel<<<1, 1, 0, s>>>(m->scalars, token, pos, 0);
    WGB_LAUNCH_CHECK("set_scalars_kernel");
    return enqueue_forward(m, s, &m->kernels_per_token);
}

WGB_EXPORT const float *wgb_gpt2_logits(const wgb_gpt2 *m) { return m ? m->logits : nullptr; }
WGB_EXPORT float *wgb_gpt2_key_cache(wgb_gpt2 *m, uint32_t layer)
{
    return (m && layer < m->p.n_layer) ? m->key_cache + (size_t)layer * m->p.n_seq * m->p.n_embd : nullptr;
}
WGB_EXPORT float *wgb_gpt2_value_cache(wgb_gpt2 *m, uint32_t layer)
{
    return (m && layer < m->p.n_layer) ? m->value_cache + (size_t)layer * m->p.n_seq * m->p.n_embd : nullptr;
}
WGB_EXPORT int wgb_gpt2_kernels_per_token(const wgb_gpt2 *m) { return m ? m->kernels_per_token : 0; }

WGB_EXPORT int wgb_gpt2_decode(wgb_gpt2 *m, const uint32_t *h_prompt, size_t n_prompt, size_t n_gen, uint32_t start_pos,
                               uint32_t *h_out_tokens, void *stream)
{
    WGB_REQUIRE(m && h_prompt && n_prompt >= 1, "null or empty prompt");
    int rc = check_complete(m);
    if (rc) return rc;
    const size_t total = n_prompt - 1 + n_gen;
    if (total == 0) return WGB_OK;
    WGB_REQUIRE(h_out_tokens, "null output");
    WGB_REQUIRE((size_t)start_pos + total <= m->p.n_seq, "%zu steps from position %u overrun a context of %u", total, start_pos, m->p.n_seq);
    for (size_t i = 0; i < n_prompt; i++)
        WGB_REQUIRE(h_prompt[i] < m->p.n_vocab, "prompt token %u outside a vocabulary of %u", h_prompt[i], m->p.n_vocab);
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
    // Batched prefill: every prompt position but the last may go through passes of PF_TOK positions; a remainder
    // shorter than half a pass stays with the token loop.
    size_t done = 0;
    if (m->pf.enabled && n_prompt - 1 >= PF_TOK) {
        const size_t rem = (n_prompt - 1) % PF_TOK;
        const size_t batched = n_prompt - 1 - (rem >= PF_TOK / 2 ? 0 : rem);
        for (; done < batched; done += PF_TOK) {
            const uint32_t nt = (uint32_t)(batched - done < PF_TOK ? batched - done : PF_TOK);
            if ((rc = prefill_pass(m, s, m->d_prompt + done, start_pos + (uint32_t)done, nt))) return rc;
        }
        done = batched;
        WGB_CUDA(cudaMemcpyAsync(m->d_out, m->d_prompt + 1, done * 4, cudaMemcpyDeviceToDevice, s));   // step i reports prompt[i + 1]
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
    if (m->graph && m->graph_n_prompt != (uint32_t)n_prompt) drop_graph(m);
    if (!m->graph) {
        cudaStream_t cs;
        WGB_CUDA(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal);
        if (e == cudaSuccess) {
            int nk = 0;
            rc = enqueue_forward(m, cs, &nk);
            if (!rc && m->smp_temperature == 0.0f) {
                rc = launch_argmax_advance(m->logits, m->p.n_vocab, ls, m->argmax_scratch, cs);
                m->kernels_per_token = nk + 2;
            } else if (!rc) {
                rc = launch_sample(m->logits, m->p.n_vocab, m->smp_temperature, m->smp_topp, 0.0f, 1, m->smp_seed, m->smp_scratch, nullptr,
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

WGB_EXPORT int wgb_gpt2_set_prefill(wgb_gpt2 *m, int enable)
{
    WGB_REQUIRE(m, "null argument");
    if (!enable) {
        prefill_free(m);
        return WGB_OK;
    }
    if (m->pf.enabled) return WGB_OK;
    int rc = check_complete(m);
    if (rc) return rc;
    if ((rc = gemv_global_init())) return rc;
    const wgb_gpt2_params &p = m->p;
    const uint32_t n = p.n_embd, ff = p.ff_len, hs = n / p.n_head;
    WGB_REQUIRE(n % 256 == 0 && ff % 256 == 0 && hs % 4 == 0 && hs <= 256, "batched prefill wants widths that are multiples of 256 (n_embd %u, ff_len %u)", n, ff);
    wgb_gpt2::Prefill &pf = m->pf;
    pf.tiles.assign((size_t)p.n_layer * 4, nullptr);
    pf.kind.assign((size_t)p.n_layer * 4, 0);
    auto bail = [&](int code) { prefill_free(m); return code; };
    for (uint32_t l = 0; l < p.n_layer; l++)
        for (int i = 0; i < 4; i++) {
            const QMat &w = m->layers[l].m[i]->view;
            const size_t idx = (size_t)l * 4 + i;
            if (prefill_tileable(w) && (rc = prefill_tile_major(w, &pf.tiles[idx], nullptr))) return bail(rc);
            if (prefill_tileable6(w)) {
                if ((rc = prefill_tile_major6(w, &pf.tiles[idx], nullptr))) return bail(rc);
                pf.kind[idx] = 1;
            }
            if (prefill_tileable8(w)) {
                if ((rc = prefill_tile_major8(w, &pf.tiles[idx], nullptr))) return bail(rc);
                pf.kind[idx] = 2;
            }
        }
    auto image = [&](uint8_t **ptr, uint32_t K) -> int {
        WGB_CUDA(cudaMalloc((void **)ptr, prefill_image_bytes(K)));
        WGB_CUDA(cudaMemset(*ptr, 0, prefill_image_bytes(K)));
        return WGB_OK;
    };
    if ((rc = image(&pf.img_e, n)) || (rc = image(&pf.img_a, n)) || (rc = image(&pf.img_h, ff))) return bail(rc);
    const size_t widest = std::max<size_t>(3 * (size_t)n, ff);
    if (cudaMalloc((void **)&pf.img6, prefill_image6_bytes((uint32_t)widest)) != cudaSuccess) return bail(fail(WGB_ERR_CUDA, "cudaMalloc(Q6_K image)"));
    if ((rc = dalloc(&pf.x, (size_t)PF_TOK * n)) || (rc = dalloc(&pf.xn, (size_t)PF_TOK * n)) || (rc = dalloc(&pf.q, (size_t)PF_TOK * n)) ||
        (rc = dalloc(&pf.xb, (size_t)PF_TOK * n)) || (rc = dalloc(&pf.h, (size_t)PF_TOK * ff)))
        return bail(rc);
    for (int i = 0; i < 3; i++)
        if ((rc = dalloc(&pf.part[i], (size_t)PF_MAX_SPLIT * PF_TOK * widest))) return bail(rc);
    if ((rc = dalloc(&pf.attn_scratch, prefill_attention_scratch_floats(p.n_head, hs)))) return bail(rc);
    {
        const size_t nc = prefill_attention_counters(p.n_head);
        cudaError_t e = cudaMalloc((void **)&pf.attn_counters, nc * 4);
        if (e == cudaSuccess) e = cudaMemset(pf.attn_counters, 0, nc * 4);
        if (e == cudaSuccess) e = cudaMalloc((void **)&pf.pos, PF_TOK * 4);
        if (e != cudaSuccess) { prefill_free(m); return cuda_fail(e, "cudaMalloc(prompt pass state)"); }
    }
    WGB_CUDA(cudaDeviceSynchronize());
    pf.enabled = true;
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_prefill_positions(const wgb_gpt2 *m, size_t *positions)
{
    WGB_REQUIRE(m && positions, "null argument");
    *positions = m->pf.positions;
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_set_sampler(wgb_gpt2 *m, float temperature, float topp, uint64_t seed)
{
    WGB_REQUIRE(m, "null argument");
    WGB_REQUIRE(temperature >= 0.0f, "negative temperature %g", temperature);
    if (temperature > 0.0f && !m->smp_scratch) WGB_CUDA(cudaMalloc(&m->smp_scratch, sampler_scratch_bytes(m->p.n_vocab)));
    m->smp_temperature = temperature;
    m->smp_topp = topp;
    m->smp_seed = seed;
    drop_graph(m);   // the parameters are baked into the recorded step
    return WGB_OK;
}
