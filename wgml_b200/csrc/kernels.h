// Internal C++ interface between the kernel files and the model / API files of the library.
#pragma once

#include "common.cuh"
#include "qmatrix.cuh"

namespace wgb {

// ---- fused matrix-vector kernel ------------------------------------------------------------

enum Prologue {
    PRO_NONE = 0,  // x used as is
    PRO_RMS = 1,   // x <- (x * 1/sqrt(mean(x^2) + eps)) * norm_w          (RmsNorm, ops/rms_norm.wgsl:58-67)
    PRO_LN = 2     // x <- ((x - mean) * 1/sqrt(var + 1e-5)) * norm_w + norm_b (LayerNorm + Mul + Add)
};

enum Epilogue {
    EPI_STORE = 0,     // out[r] = y (+ bias[r])
    EPI_RESIDUAL = 1,  // out[r] = residual[r] + y (+ bias[r]); out may alias residual
    EPI_SILU_PAIR = 2, // matrices {gate, up}: out[r] = up_r * gate_r / (1 + exp(-gate_r))   (Silu, ops/silu.wgsl:19-27)
    EPI_GELU = 3,      // out[r] = gelu(y + bias[r])                                       (unary.wgsl:50-52)
    EPI_QKV_ROPE = 4,  // matrices {q, k, v}: (+bias), rotate q and k (RoPE), q -> out, k/v -> cache row *pos
    EPI_QKV_SPLIT = 5  // one fused qkv matrix (+bias): rows [0,n) -> out, [n,2n) -> k cache, [2n,3n) -> v cache
};

// Direct exchange of partial products between the ranks of a tensor-parallel group (no collective call):
// the sender's epilogue stores its partial rows into every rank's mailbox (plain stores to peer memory
// over NVLink) and, once per launch, adds one to its flag on every rank; the receiver's prologue waits
// until all `n` flags have reached the step count and adds the `n` partials in rank order.
constexpr int PEER_MAX = 8;
struct PeerOut {
    uint32_t n;                   // ranks (0: write to `out` as usual)
    float *mail[PEER_MAX];        // on rank p: where this rank's partial of this exchange goes
    uint32_t *flag[PEER_MAX];     // on rank p: this rank's flag for this exchange (counts steps)
    uint32_t *ticket;             // local: blocks of this launch that have finished
};
struct PeerIn {
    uint32_t n;                   // ranks (0: read `x` as usual)
    const float *mail;            // local mailbox of this exchange: [n][ncols]
    const uint32_t *flag;         // local flags of this exchange: [n]
    const uint32_t *epoch;        // device scalar: steps so far = the value every flag must have reached
    float *x_out;                 // where block 0 leaves the sum (the residual stream)
};

struct GemvArgs {
    QMat mat[3];
    int nmat;
    const float *x;          // input vector, mat[0].ncols floats
    // prologue
    int prologue;
    const float *norm_w, *norm_b;
    float eps;
    // epilogue
    int epilogue;
    float *out;
    const float *bias;       // optional; for EPI_QKV_ROPE: bias of q
    const float *bias_k, *bias_v;
    const float *residual;
    // EPI_QKV_*: KV cache rows and the position, read on the device
    float *k_cache, *v_cache;   // element (pos, head, e) at pos * kv_row_stride + head * kv_head_stride + e
    uint32_t kv_row_stride, kv_head_stride;   // 0, 0: the reference layout [seq_len][kv_dim] (kv_dim, head_size)
    const uint32_t *pos;        // device scalar
    uint32_t kv_dim, head_size;
    int rope_variant;
    const float *rope_freq;     // head_size/2 inverse frequencies base^(-2j/head_size)
    // launch plan, filled by launch_gemv
    uint32_t rs;            // rows per shared-memory stage
    uint32_t ngroups;       // stages' worth of rows in the launch
    uint32_t nstage;        // ring depth
    uint32_t stage_bytes;
    uint32_t ring_offset;   // of the ring inside dynamic shared memory (after the input image)
    uint32_t kparts;        // column parts = consumer warps that share one row
    uint32_t rparts;        // row parts per stage (a power of two)
    uint32_t rparts_log2;
    uint32_t gq, gk;        // EPI_QKV_ROPE: groups of the q and of the k matrix
    uint32_t rrows;         // rows per consumer task = rs / rparts
    uint32_t row_bytes;     // bytes of one row over all planes
    uint32_t per_block;     // groups of blocks 0 .. rem_blocks-1; the other blocks have one fewer
    uint32_t rem_blocks;    //   (0: every block has per_block)
    uint32_t cps_log2;      // log2 of the copies per stage (planes x parts)
    uint32_t spb;           // stages per producer pass
    uint32_t *err;          // device status word for expired waits
    unsigned long long wait_ns, peer_wait_ns;   // limits of the waits inside the block / for the peers' flags
    unsigned long long *stamp;   // optional: receives the launch's end time (stamp_end)
    PeerOut peer_out;            // EPI_STORE / EPI_RESIDUAL only
    PeerIn peer_in;              // PRO_RMS only
};

// Enqueues one fused kernel.  All matrices must share format and ncols and have a fast path;
// returns WGB_ERR_UNSUPPORTED otherwise so that the caller can fall back to separate ops.
// `pdl` launches with programmatic stream serialization (the kernel prefetches its first
// weights before waiting for its predecessor).
int launch_gemv(const GemvArgs &a, cudaStream_t stream, bool pdl);
bool gemv_fast_supported(const QMat &m);
// One-time per-process set-up of the fused kernels (call outside stream capture).
int gemv_global_init();
// WGB_ERR_TIMEOUT if any bounded wait of a fused kernel expired since the last call (synchronises).
int gemv_check_status();
// The device status word itself (NULL before gemv_global_init) and the error for a value read from it
// (clears the word when v != 0): lets a caller fold the read into its own device-to-host copy.
uint32_t *gemv_status_word();
int gemv_report_status(uint32_t v);

// Replays a captured decode step `total` times on `stream` and reads the device status word every
// STATUS_EVERY launches through `h_slots` (two words of pinned host memory) without draining the stream: the
// copy issued after launch 64k is looked at before launch 64(k + 2) goes out.  When a wait has expired on the
// device, stops launching, drains the stream, clears the word and returns WGB_ERR_TIMEOUT; the launches in
// flight (at most 2 * STATUS_EVERY) finish quickly because kernels do not wait while the word is set.
constexpr size_t STATUS_EVERY = 64;
struct StatusPoll {
    cudaEvent_t ev[2] = { nullptr, nullptr };
};
int replay_with_status(cudaGraphExec_t graph, size_t total, cudaStream_t stream, uint32_t *h_slots, StatusPoll &sp);
void status_poll_destroy(StatusPoll &sp);

// Slow path for any format: one warp per row, dequantising with the exact block formulas.
int launch_gemv_generic(const QMat &m, const float *x, float *out, cudaStream_t stream);

// ---- attention ------------------------------------------------------------------------------
struct AttnArgs {
    wgb_attn_params p;          // with pos != NULL, p.pos is only a bound on the position used to size the launch
    const uint32_t *pos;        // device scalar or NULL
    const float *q, *k_cache, *v_cache;
    // cache element (pos, KV head, e) at pos * row_stride + head * head_stride + e.  0, 0: the reference layout
    // [seq_len][kv_dim] (kv_dim, head_size); head-major caches (head_size, seq_len * head_size) make the rows of a
    // head contiguous, which is what the streaming kernel copies in one piece.
    uint32_t row_stride, head_stride;
    float *xb;
    float *scratch;             // attn_scratch_floats() floats
    uint32_t *counters;         // n_kv_heads counters, zero before the first launch
    unsigned long long *stamp;  // optional: receives the launch's end time (stamp_end)
    uint32_t *err;              // optional: status word for an expired wait of the streaming kernel
};
size_t attn_scratch_floats(uint32_t n_heads, uint32_t head_size, uint32_t seq_len);
uint32_t attn_num_splits(uint32_t seq_len);
int launch_attention(const AttnArgs &a, cudaStream_t stream, bool pdl);
int attn_sizing_class(const wgb_attn_params &p);

// ---- small ops used by the models -------------------------------------------------------------
// x[0..n) = row *d_token of the embedding matrix (+ row *d_pos of `pos_embd` when given).
int launch_embed(const QMat &embd, const QMat *pos_embd, const uint32_t *d_token, const uint32_t *d_pos,
                 float *x, cudaStream_t stream);
// Greedy sampling step kept on the device: next = step+1 < n_prompt ? prompt[step+1] : argmax(logits);
// token <- next, pos <- pos+1, out_tokens[step] <- next, step <- step+1.
struct LoopState {
    uint32_t *token, *pos, *step;       // device scalars
    const uint32_t *prompt;             // device, n_prompt ids
    uint32_t n_prompt;
    uint32_t *out_tokens;               // device
};
int launch_argmax_advance(const float *logits, uint32_t n, const LoopState &ls, uint32_t *scratch,
                          cudaStream_t stream);

// Temperature / top-p draw on the device (sampler.cu).  `scratch` holds sampler_scratch_bytes(n) bytes.  With a
// loop state the kernel is the sampling step of the token loop: forced prompt tokens, then a draw per
// generated position with coin = f(seed, position).
size_t sampler_scratch_bytes(uint32_t n);
int launch_sample(const float *logits, uint32_t n, float temperature, float topp, float coin, int seeded, unsigned long long seed,
                  void *scratch, uint32_t *out_index, const LoopState *ls, cudaStream_t stream);


// ---- batched prompt prefill (prefill.cu) --------------------------------------------------------------
constexpr uint32_t PF_TOK = 8;         // prompt positions per pass
constexpr uint32_t PF_MAX_SPLIT = 8;   // column slices of one product
// Bytes of the activation image per 256-column unit: 16 K-cores x 4 row groups x 128 bytes of digits, then one exponent
// and one sum per 32-column group and position.
constexpr uint32_t prefill_image_unit_bytes() { return 16 * 4 * 128 + 2 * 8 * PF_TOK * 4; }
// Bytes of the fixed-point activation image of PF_TOK vectors of K elements (zero it once: the kernels never
// write its padding rows).
size_t prefill_image_bytes(uint32_t K);
bool prefill_tileable(const QMat &m);
// Tile-major copy of a Q4_K matrix for the tensor-core product (cudaMalloc'd, *out).
int prefill_tile_major(const QMat &m, uint8_t **out, cudaStream_t stream);
uint32_t prefill_gemm_splits(uint32_t nrows, uint32_t K);
// out[slice][position][row] (out_stride floats per position) = the product of the tile-major matrix with the
// `ntok` vectors whose image is `image`, the columns cut into `nsplit` slices.
int launch_gemm_q4k_tiles(const uint8_t *w_tiles, uint32_t nrows, uint32_t K, const uint8_t *image, uint32_t ntok, float *out,
                          uint32_t out_stride, uint32_t nsplit, cudaStream_t stream);
// The same for up to three matrices that share the input (q / k / v, gate / up) in one launch; `nsplit` is common.
int launch_gemm_q4k_tiles_multi(uint32_t nmat, const uint8_t *const *w_tiles, const uint32_t *nrows, uint32_t K, const uint8_t *image,
                                uint32_t ntok, float *const *out, const uint32_t *out_stride, uint32_t nsplit, cudaStream_t stream);
// x[t] (+= the slices of `part` when given, written back); then optionally RMS-normalised with norm_w; the image
// of the result and, with xn, the values.  With neither image nor xn only x is updated.
int launch_prefill_norm_image(float *x, uint32_t x_stride, const float *part, uint32_t nsplit, uint32_t part_stride, const float *norm_w,
                              float eps, uint32_t K, uint32_t ntok, uint8_t *image, float *xn, uint32_t xn_stride, cudaStream_t stream);
int launch_prefill_silu_image(const float *gate, uint32_t gsplit, const float *up, uint32_t usplit, uint32_t stride, uint32_t K,
                              uint32_t ntok, uint8_t *image, float *h, uint32_t h_stride, cudaStream_t stream);
// The Q6_K counterparts (prefill_q6k.cu): the scale is folded into a two-plane weight operand and a super-block's
// MMAs accumulate in tensor memory, which takes an image of the inputs with one exponent per vector and
// super-block (launch_prefill_image6, from the values themselves).
size_t prefill_image6_bytes(uint32_t K);
bool prefill_tileable6(const QMat &m);
int prefill_tile_major6(const QMat &m, uint8_t **out, cudaStream_t stream);
int launch_prefill_image6(const float *x, uint32_t x_stride, uint32_t K, uint32_t ntok, uint8_t *image, cudaStream_t stream);
int launch_gemm_q6k_tiles(const uint8_t *w_tiles, uint32_t nrows, uint32_t K, const uint8_t *image, uint32_t ntok, float *out,
                          uint32_t out_stride, uint32_t nsplit, cudaStream_t stream);
// The Q8_0 counterpart (prefill_q80.cu): the codes are the operand as they are, kept in HBM in the operand's
// shared-memory image; it reads the same activation image as the Q4_K product.
bool prefill_tileable8(const QMat &m);
int prefill_tile_major8(const QMat &m, uint8_t **out, cudaStream_t stream);
int launch_gemm_q80_tiles(const uint8_t *w_tiles, uint32_t nrows, uint32_t K, const uint8_t *image, uint32_t ntok, float *out,
                          uint32_t out_stride, uint32_t nsplit, cudaStream_t stream);
// GPT-2 passes: LayerNorm (two passes, epsilon 1e-5) * gain + bias with the fold of the preceding product and its
// bias; the split of the fused qkv product into q / cache rows ([seq][n] caches); GELU of a product plus bias.
int launch_prefill_ln_image(float *x, uint32_t x_stride, const float *part, uint32_t nsplit, uint32_t part_stride, const float *fold_bias,
                            const float *gain, const float *bias, uint32_t K, uint32_t ntok, uint8_t *image, float *xn, uint32_t xn_stride,
                            cudaStream_t stream);
int launch_prefill_qkv_split(const float *qkv, uint32_t nsplit, const float *bias, float *q_out, float *k_cache, float *v_cache, uint32_t n,
                             uint32_t pos0, uint32_t ntok, cudaStream_t stream);
int launch_prefill_gelu_image(const float *part, uint32_t nsplit, uint32_t stride, const float *bias, uint32_t K, uint32_t ntok, uint8_t *image,
                              float *h, uint32_t h_stride, cudaStream_t stream);
int launch_prefill_positions(uint32_t *positions, uint32_t pos0, cudaStream_t stream);
struct PrefillQkv {
    const float *q, *k, *v;            // product slices: [split][PF_TOK][stride]
    uint32_t q_split, k_split, v_split, q_stride, kv_stride;
    const float *bq, *bk, *bv;         // optional biases
    float *q_out;                      // [ntok][q_dim]
    float *k_cache, *v_cache;          // one layer, head-major
    uint32_t q_dim, kv_dim, head_size, seq_len, pos0;
    int variant;
    const float *freq;
};
int launch_prefill_rope_append(const PrefillQkv &a, uint32_t ntok, cudaStream_t stream);
// With `image` (allowed when prefill_attention_writes_image(head_size)) the kernel also writes the activation image of
// its output, the input of the output projection.
bool prefill_attention_writes_image(uint32_t head_size);
// With scratch (prefill_attention_scratch_floats) and counters (prefill_attention_counters words, zero before the first
// launch; the kernel leaves them zero) long contexts are split over several blocks per (head, pair of positions).
size_t prefill_attention_scratch_floats(uint32_t n_heads, uint32_t head_size);
size_t prefill_attention_counters(uint32_t n_heads);
// Cache row p of KV head g lies at p * row_stride + g * head_stride floats.
int launch_prefill_attention(const float *q, const float *k_cache, const float *v_cache, float *out, uint32_t n_heads, uint32_t head_size,
                             uint32_t kv_mul, uint32_t row_stride, uint32_t head_stride, uint32_t pos0, uint32_t ntok, uint8_t *image,
                             float *scratch, uint32_t *counters, cudaStream_t stream);

}  // namespace wgb
