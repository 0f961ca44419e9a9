/*
 * wgml_b200.h -- C ABI of the B200-native token-loop path behind wgml's operator surface.
 *
 * wgml has no FFI of its own: its operators are Rust structs that record WGSL dispatches into a
 * wgpu compute pass.  Each entry point below replaces one of those Rust interfaces (cited as
 * file:line inside the wgml repository) with a call that enqueues hand-written sm_100a CUDA
 * kernels on a caller-supplied CUDA stream.
 *
 * Conventions
 *  - Every function returns a wgb_status; 0 is success.  Nothing aborts: where the Rust code
 *    panics on an `assert!`, the call returns WGB_ERR_INVALID.  wgb_last_error() gives the
 *    message of the calling thread's last failure.
 *  - `stream` is a `cudaStream_t` passed as `void *` (NULL = the legacy default stream).  Work is
 *    enqueued and the call returns: the counterpart of wgml's "record, then queue.submit".
 *  - Pointers named d_* are device addresses of the current CUDA device, owned by the caller,
 *    as wgml's ops borrow the caller's GpuVector / GpuMatrix buffers.  Vector views are
 *    contiguous: pass `base + offset` for `column(pos)` / `rows(start, n)` views.
 *  - Matrices are row-major with the input dimension contiguous, exactly the byte order of a
 *    GGUF tensor (crates/wgml/src/gguf.rs:148-155).
 *  - There is no CPU fallback: on a machine without a CUDA device every compute entry point
 *    fails with WGB_ERR_CUDA.
 */
#ifndef WGML_B200_H
#define WGML_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    WGB_OK = 0,
    WGB_ERR_INVALID = 1,     /* shape / argument mismatch (a Rust `assert!` in the reference) */
    WGB_ERR_UNSUPPORTED = 2, /* tensor or metadata type the reference does not support either */
    WGB_ERR_CUDA = 3,        /* a CUDA runtime call failed, or no device */
    WGB_ERR_PARSE = 4,       /* malformed GGUF (GgufParseError, gguf.rs:23-37) */
    WGB_ERR_NOT_FOUND = 5,   /* missing GGUF key / tensor (a panic in the reference) */
    WGB_ERR_TIMEOUT = 6      /* a bounded device-side wait gave up */
} wgb_status;

/* ggml tensor type ids (crates/wgml/src/gguf.rs:73-105); the variants of GpuQuantMatrix
 * (crates/wgml/src/quantized_matrix.rs:9-20) plus F16. */
typedef enum {
    WGB_F32 = 0, WGB_F16 = 1, WGB_Q4_0 = 2, WGB_Q4_1 = 3, WGB_Q5_0 = 6, WGB_Q5_1 = 7,
    WGB_Q8_0 = 8, WGB_Q4_K = 12, WGB_Q5_K = 13, WGB_Q6_K = 14, WGB_Q8_K = 15
} wgb_qtype;

const char *wgb_last_error(void);
/* Library version string and the compute capability the kernels were built for ("sm_100a"). */
const char *wgb_version(void);
/* Bytes per block / weights per block of a format (block structs, quantization.rs:13-327). */
int wgb_block_bytes(int qtype);
int wgb_block_len(int qtype);

/* ---- device memory helpers (what wgcore's GpuVector::init / read do for the Rust caller) ---- */
int wgb_malloc(void **d_ptr, size_t bytes);
int wgb_free(void *d_ptr);
int wgb_memcpy_h2d(void *d_dst, const void *h_src, size_t bytes, void *stream);
int wgb_memcpy_d2h(void *h_dst, const void *d_src, size_t bytes, void *stream);
int wgb_memset(void *d_dst, int value, size_t bytes, void *stream);
int wgb_stream_synchronize(void *stream);

/* ---- quantisation ---- */

/* Block*::dequantize for every block of a tensor (quantization.rs:21-378,
 * GgufTensorData::dequantize gguf.rs:114-129; GPU twin ops/quantization_test.wgsl:45-146).
 * d_blocks: raw GGUF blocks; d_out: nblocks * wgb_block_len(qtype) floats.  Bit-exact with the
 * Rust CPU code (every multiply, add and subtract individually rounded). */
int wgb_dequantize(int qtype, const void *d_blocks, size_t nblocks, float *d_out, void *stream);

/* GpuQuantMatrix (quantized_matrix.rs:9-75) as built by GgufTensorData::to_gpu_matrix
 * (gguf.rs:131-184): an nrows x ncols matrix kept in its GGUF blocks on the device.  Unlike the
 * reference there is no dense-f32 fallback when ncols is not a multiple of 64 / 512: any ncols
 * that is a multiple of the format's block length is accepted.  Q8_0 and Q6_K blocks (34 and
 * 210 bytes, only 2-byte aligned) are split into 16-byte aligned planes once, here; the weights
 * they decode to are unchanged. */
typedef struct wgb_quant_matrix wgb_quant_matrix;
int wgb_quant_matrix_create(int qtype, const void *h_blocks, size_t nrows, size_t ncols,
                            void *stream, wgb_quant_matrix **out);
/* Same, from blocks that are already on the device (raw GGUF order). */
int wgb_quant_matrix_create_from_device(int qtype, const void *d_blocks, size_t nrows, size_t ncols,
                                        void *stream, wgb_quant_matrix **out);
int wgb_quant_matrix_destroy(wgb_quant_matrix *m);
/* GpuQuantMatrix::shape (quantized_matrix.rs:37-52) in weights, and the format. */
int wgb_quant_matrix_shape(const wgb_quant_matrix *m, size_t *nrows, size_t *ncols, int *qtype);
/* Dequantise rows [row0, row0+n) to d_out (n * ncols floats), bit-exact as wgb_dequantize. */
int wgb_quant_matrix_dequantize_rows(const wgb_quant_matrix *m, size_t row0, size_t n, float *d_out,
                                     void *stream);

/* GemvQuant::dispatch (ops/gemv_quant.rs:241-348): d_out[nrows] = m * d_v[ncols], f32 in and
 * out, f32 accumulation.  Any nrows (the reference needs nrows % 4 == 0). */
int wgb_gemv_quant(const wgb_quant_matrix *m, const float *d_v, float *d_out, void *stream);
/* The same product over raw GGUF blocks in device memory (no wgb_quant_matrix).  The blocks may be produced by
 * earlier work on the same stream: unlike wgb_gemv_quant on a matrix the library uploaded, this launch does not
 * start reading weights before its predecessor in the stream has completed. */
int wgb_gemv_quant_raw(int qtype, const void *d_blocks, size_t nrows, size_t ncols, const float *d_v,
                       float *d_out, void *stream);

/* The same operator (GemvQuant::dispatch, ops/gemv_quant.rs:241-348) for Q4_K on the tcgen05 tensor-core
 * path: weights kept tile-major (128 rows x one 256-column super-block per bulk copy), nibbles unpacked to
 * bytes in shared memory, eight kind::i8 MMAs per tile and super-block against the three byte digits of
 * the input, accumulators read back from tensor memory one lane per row.  nrows a multiple of 128, ncols a
 * multiple of 256 up to 4096.  Same results as wgb_gemv_quant within f32 rounding.  Measured slower than
 * wgb_gemv_quant for a single input vector (an MMA pays for loading its 128-row operand whatever the
 * number of input columns); the models do not use it. */
typedef struct wgb_q4k_tiles wgb_q4k_tiles;
int wgb_q4k_tiles_create(const void *h_blocks, size_t nrows, size_t ncols, void *stream, wgb_q4k_tiles **out);
int wgb_q4k_tiles_destroy(wgb_q4k_tiles *m);
int wgb_gemv_q4k_tiles(const wgb_q4k_tiles *m, const float *d_v, float *d_out, void *stream);
/* The same product for 1..8 input vectors at once, d_v [n_vec][ncols] -> d_out [n_vec][nrows]: the tensor-core
 * kernel of the batched prompt prefill (wgb_llama2_set_prefill), any number of columns that is a multiple of
 * 256.  In the reference a prompt costs one GemvQuant::dispatch per matrix and position
 * (chat_llama2.rs:104-116); here eight positions share one pass over the weights.  Asynchronous like the other
 * operators; the first call on a matrix allocates its work areas (make it outside stream capture), and calls on
 * one matrix must be ordered on a stream. */
int wgb_gemm_q4k_tiles(wgb_q4k_tiles *m, const float *d_v, size_t n_vec, float *d_out, void *stream);
/* The batched product for Q6_K matrices (BlockQ6K, quantization.rs:225-264): the 16-column scales are folded
 * into a two-plane integer weight operand and a super-block's sixteen MMAs accumulate in tensor memory, with one
 * exponent per input vector and super-block.  h_blocks: raw GGUF blocks, nrows a multiple of 128, ncols of 256. */
typedef struct wgb_q6k_tiles wgb_q6k_tiles;
int wgb_q6k_tiles_create(const void *h_blocks, size_t nrows, size_t ncols, void *stream, wgb_q6k_tiles **out);
int wgb_q6k_tiles_destroy(wgb_q6k_tiles *m);
int wgb_gemm_q6k_tiles(wgb_q6k_tiles *m, const float *d_v, size_t n_vec, float *d_out, void *stream);
/* The batched product for Q8_0 matrices (BlockQ8_0, quantization.rs:29-52): the signed byte codes are the tensor-core
 * operand as they are, kept in HBM in the operand's shared-memory image (128-byte swizzle applied), so a bulk copy
 * lands a unit where the MMAs read it.  h_blocks: raw GGUF blocks, nrows a multiple of 128, ncols of 256. */
typedef struct wgb_q80_tiles wgb_q80_tiles;
int wgb_q80_tiles_create(const void *h_blocks, size_t nrows, size_t ncols, void *stream, wgb_q80_tiles **out);
int wgb_q80_tiles_destroy(wgb_q80_tiles *m);
int wgb_gemm_q80_tiles(wgb_q80_tiles *m, const float *d_v, size_t n_vec, float *d_out, void *stream);
/* Waits for the device and returns WGB_ERR_TIMEOUT if a bounded wait inside a matrix-vector kernel has
 * expired since the last report (stand-alone launches are asynchronous and cannot say so themselves). */
int wgb_device_status(void);

/* ---- normalisation, activations, elementwise ---- */

/* RmsNorm::dispatch (ops/rms_norm.rs:24-53, rms_norm.wgsl:58-67), RmsNormConfig::nudge_factor
 * (rms_norm.rs:17-21) passed as eps: out = (v * 1/sqrt(mean(v^2) + eps)) * w. */
int wgb_rms_norm(float *d_out, const float *d_v, const float *d_w, size_t n, float eps, void *stream);
/* LayerNorm::dispatch (ops/layernorm.rs:18-41, layernorm.wgsl:28-80): (x - mean)/sqrt(var+1e-5),
 * no gain or bias. */
int wgb_layernorm(float *d_out, const float *d_in, size_t n, void *stream);

/* RoPEConfig (ops/rope.rs:26-35); field order and types as the Rust / WGSL struct. */
typedef struct {
    uint32_t head_size;
    uint32_t kv_dim;
    uint32_t pos;
    float base_freq;
} wgb_rope_config;
/* RoPEVariant (ops/rope.rs:10-16) */
typedef enum { WGB_ROPE_ORIGINAL = 0, WGB_ROPE_NEOX = 1 } wgb_rope_variant;
/* RoPE::dispatch (ops/rope.rs:37-76, rope.wgsl:36-77): rotates q and the first kv_dim entries
 * of k in place.  q_len and k_len must be even and q_len >= k_len (rope.rs:51-56). */
int wgb_rope(int variant, const wgb_rope_config *cfg, float *d_q, size_t q_len, float *d_k,
             size_t k_len, void *stream);

/* BatchedMultiqueryAttentionParams (ops/batched_multiquery_attention.rs:26-37). */
typedef struct {
    uint32_t seq_len;
    uint32_t kv_dim;
    uint32_t kv_mul;
    uint32_t n_heads;
    uint32_t head_size;
    uint32_t pos;
} wgb_attn_params;
/* BatchedMultiqueryAttention::dispatch / dispatch_multi (ops/batched_multiquery_attention.rs:
 * 55-139): xb_h = softmax(q_h . K_t / sqrt(head_size), t = 0..=pos) . V_t for every query head.
 * Caches are [seq_len][kv_dim] floats (time step t is the t-th run of kv_dim floats).  d_attn
 * may be NULL; otherwise it receives the attention weights as [n_heads][seq_len] (the layout of
 * the reference's single-kernel path, batched_multiquery_attention.wgsl:48,66). */
int wgb_attention(const wgb_attn_params *p, const float *d_q, const float *d_key_cache,
                  const float *d_value_cache, float *d_attn, float *d_xb, void *stream);

/* wgb_attention without any device allocation.  No counterpart in the reference; it exists for hosts
 * that cannot have cudaMalloc / cudaFree on the call path: a server that has given the whole device to
 * its own memory pool, or a latency-critical loop in which the device-wide synchronisation of an
 * allocation would stall the other streams.  The split-K partial results live in a fixed array that is
 * part of the library image (one copy per device, 8 MiB), so
 *   - shapes that need more are refused with WGB_ERR_INVALID and a message naming the limit:
 *     n_heads * ceil(seq_len / 64) * (head_size + 4) <= WGB_ATTENTION_STATIC_MAX_SCRATCH_FLOATS and
 *     n_heads <= WGB_ATTENTION_STATIC_MAX_HEADS (a 7B-class 32 x 128 head layout fits up to 31 744 cached
 *     positions; 64 heads up to 15 872);
 *   - the first call on a device looks the array up (cudaGetSymbolAddress, with that device current) and, like
 *     the first wgb_attention there, sets the kernels up once (cudaFuncSetAttribute for the shared-memory
 *     opt-in, cudaOccupancyMaxActiveBlocksPerMultiprocessor for the launch shapes): none of these may run while
 *     a stream is capturing, so make that first call before the stream is put into capture mode;
 *   - two calls that may run at the same time (different streams, or different host threads on one
 *     device) share the array and race: keep calls on one device in one stream order.
 * Every call clears its tickets first, so an earlier launch that was cut short cannot disturb it.
 * Results are identical to wgb_attention with d_attn == NULL. */
#define WGB_ATTENTION_STATIC_MAX_SCRATCH_FLOATS (2 * 1024 * 1024)
#define WGB_ATTENTION_STATIC_MAX_HEADS 256
int wgb_attention_static(const wgb_attn_params *p, const float *d_q, const float *d_key_cache,
                         const float *d_value_cache, float *d_xb, void *stream);
/* SoftMax::dispatch (ops/softmax.rs:18-30, softmax.wgsl:31-92): every column of a column-major
 * nrows x ncols matrix (column j starts at d_mat + j * col_stride) replaced by its softmax. */
int wgb_softmax(float *d_mat, size_t nrows, size_t ncols, size_t col_stride, void *stream);
/* Silu::dispatch (ops/silu.rs:18-34, silu.wgsl:19-27): h1 = h2 * h1 / (1 + exp(-h1)). */
int wgb_silu(float *d_h1, const float *d_h2, size_t n, void *stream);

/* UnaryOp (ops/unary.rs:16-38), numbered in declaration order. */
typedef enum {
    WGB_UNARY_ABS = 0, WGB_UNARY_SGN, WGB_UNARY_NEG, WGB_UNARY_STEP, WGB_UNARY_ELU, WGB_UNARY_GELU,
    WGB_UNARY_GELU_QUICK, WGB_UNARY_SILU, WGB_UNARY_TANH, WGB_UNARY_RELU, WGB_UNARY_SIGMOID,
    WGB_UNARY_HARD_SIGMOID, WGB_UNARY_HARD_SWISH, WGB_UNARY_SQR, WGB_UNARY_SQRT, WGB_UNARY_LOG,
    WGB_UNARY_LEAKY_RELU, WGB_UNARY_CLAMP, WGB_UNARY_SCALE, WGB_UNARY_ADD_SCALAR
} wgb_unary_op;
/* Unary::dispatch / UnaryInplace::dispatch (ops/unary.rs:158-193, 229-256; unary.wgsl:116-130).
 * args4 (host pointer to 4 floats) must be given exactly for the ops that take arguments
 * (LeakyRelu, Clamp, Scale, AddScalar), else NULL (unary.rs:172-175). */
int wgb_unary(int op, float *d_dst, const float *d_src, size_t n, const float *args4, void *stream);
int wgb_unary_inplace(int op, float *d_src, size_t n, const float *args4, void *stream);

/* wgebra OpAssign{Add,Mul,Copy} as wgml calls it (models/llama2/transformer.rs:293,343-354,
 * 383-384; models/gpt2/transformer.rs:259-261,277-290): lhs += rhs, lhs *= rhs, lhs = rhs. */
typedef enum { WGB_ASSIGN_ADD = 0, WGB_ASSIGN_MUL = 1, WGB_ASSIGN_COPY = 2 } wgb_assign_kind;
int wgb_op_assign(int kind, float *d_lhs, const float *d_rhs, size_t n, void *stream);

/* Sampler::sample_argmax (models/sampler.rs:54-56) on the device: index of the first maximum
 * of d_v[0..n) written to *d_index. */
int wgb_argmax(const float *d_v, size_t n, uint32_t *d_index, void *stream);
/* Sampler::sample (models/sampler.rs:32-52) on the device, with the reference's `coin = random()` passed
 * in (0 <= coin < 1): logits / temperature, softmax, then Sampler::sample_mult (sampler.rs:62-76) when topp
 * is outside (0, 1) or Sampler::sample_topp (sampler.rs:84-130): candidates >= (1 - topp) / (n - 1),
 * stable sort by decreasing probability, prefix cut where the running sum exceeds topp, inverse CDF at
 * coin * sum.  temperature == 0 is wgb_argmax.  The logits are left untouched; the token id goes to
 * *d_token.  The softmax denominator and the CDF are added in the reference's order (one thread, about 2 ns
 * per vocabulary entry), so the same coin gives the same token up to the last bit of expf. */
int wgb_sample(const float *d_logits, size_t n, float temperature, float topp, float coin, uint32_t *d_token,
               void *stream);
/* The counter-based uniform draw the device-resident token loops use for the token at position `draw`:
 * 24 bits in [0, 1), the form of rand's f32 sample (the reference's generator is unseeded,
 * sampler.rs:42). */
float wgb_sampler_coin(uint64_t seed, uint64_t draw);

/* ---- GGUF ---- */

/* Gguf (gguf.rs:317-322) parsed by Gguf::from_bytes (gguf.rs:452-623).  The file is mapped, not
 * copied: tensor data pointers point into the mapping (or into `bytes`, which must then outlive
 * the handle). */
typedef struct wgb_gguf wgb_gguf;
int wgb_gguf_open(const char *path, wgb_gguf **out);
int wgb_gguf_from_bytes(const void *bytes, size_t len, wgb_gguf **out);
int wgb_gguf_close(wgb_gguf *g);
uint32_t wgb_gguf_version(const wgb_gguf *g);
uint64_t wgb_gguf_tensor_count(const wgb_gguf *g);
uint64_t wgb_gguf_metadata_count(const wgb_gguf *g);
uint32_t wgb_gguf_alignment(const wgb_gguf *g);

/* GgufMetadataValue (gguf.rs:230-245); type ids of MetadataValueType (gguf.rs:332-364). */
typedef enum {
    WGB_META_U8 = 0, WGB_META_I8 = 1, WGB_META_U16 = 2, WGB_META_I16 = 3, WGB_META_U32 = 4,
    WGB_META_I32 = 5, WGB_META_F32 = 6, WGB_META_BOOL = 7, WGB_META_STRING = 8, WGB_META_ARRAY = 9,
    WGB_META_U64 = 10, WGB_META_I64 = 11, WGB_META_F64 = 12
} wgb_meta_type;
/* Index of a key, or -1.  Keys are listed in file order by wgb_gguf_meta_key. */
int64_t wgb_gguf_meta_find(const wgb_gguf *g, const char *key);
const char *wgb_gguf_meta_key(const wgb_gguf *g, uint64_t index);
/* Value type; for arrays *elem_type and *len describe the elements (elem_type WGB_META_ARRAY
 * for nested arrays, whose elements are not exposed). */
int wgb_gguf_meta_type(const wgb_gguf *g, uint64_t index, int *type, int *elem_type, uint64_t *len);
/* Scalar getters: integers and bool widen to 64 bits, floats to double.  WGB_ERR_INVALID when
 * the stored type is of another kind (the reference's unwrap_* accessors panic, gguf.rs:247-295). */
int wgb_gguf_meta_u64(const wgb_gguf *g, uint64_t index, uint64_t *out);
int wgb_gguf_meta_i64(const wgb_gguf *g, uint64_t index, int64_t *out);
int wgb_gguf_meta_f64(const wgb_gguf *g, uint64_t index, double *out);
/* String value: pointer into the file (not NUL-terminated) and its length. */
int wgb_gguf_meta_str(const wgb_gguf *g, uint64_t index, const char **ptr, uint64_t *len);
/* Array element i as integer / double / string. */
int wgb_gguf_meta_arr_u64(const wgb_gguf *g, uint64_t index, uint64_t i, uint64_t *out);
int wgb_gguf_meta_arr_i64(const wgb_gguf *g, uint64_t index, uint64_t i, int64_t *out);
int wgb_gguf_meta_arr_f64(const wgb_gguf *g, uint64_t index, uint64_t i, double *out);
int wgb_gguf_meta_arr_str(const wgb_gguf *g, uint64_t index, uint64_t i, const char **ptr, uint64_t *len);

/* GgufTensor (gguf.rs:297-315). */
typedef struct {
    const char *name;      /* NUL-terminated copy owned by the handle */
    uint32_t n_dims;
    uint64_t dims[4];      /* unused trailing dims are 1, as in the reference (gguf.rs:516) */
    uint32_t type;         /* ggml type id */
    uint64_t offset;       /* absolute offset of the data in the file (gguf.rs:540-542) */
    uint64_t n_bytes;      /* 0 for the block formats the reference leaves unread (gguf.rs:618) */
    const void *data;      /* host pointer to the tensor bytes */
} wgb_gguf_tensor;
int64_t wgb_gguf_tensor_find(const wgb_gguf *g, const char *name);
int wgb_gguf_tensor_info(const wgb_gguf *g, uint64_t index, wgb_gguf_tensor *out);

/* ---- Tokenizers and chat template (host only) ---- */

/* LlamaTokenizer (models/llama2/tokenizer.rs:8-180) from the GGUF metadata keys tokenizer.ggml.tokens,
 * .scores, .bos_token_id, .eos_token_id, .unknown_token_id (tokenizer.rs:23-34).  Text is UTF-8.
 * encode (tokenizer.rs:75-164): spaces become U+2581, one token per character with byte fallback (byte b ->
 * id b + 3), the "<s>" / "</s>" scans, then the best-scoring adjacent pair is merged until none is in the
 * vocabulary.  With out_ids == NULL only *n_out is written (size query).
 * decode (tokenizer.rs:166-177): the text of `token` after `prev_token` (leading white space dropped after
 * id 1, "<0xHH>" pieces become the character of that byte value, U+2581 becomes a space). */
typedef struct wgb_llama_tokenizer wgb_llama_tokenizer;
int wgb_llama_tokenizer_from_gguf(const wgb_gguf *g, wgb_llama_tokenizer **out);
int wgb_llama_tokenizer_destroy(wgb_llama_tokenizer *t);
uint32_t wgb_llama_tokenizer_bos(const wgb_llama_tokenizer *t);
uint32_t wgb_llama_tokenizer_eos(const wgb_llama_tokenizer *t);
uint32_t wgb_llama_tokenizer_unk(const wgb_llama_tokenizer *t);
size_t wgb_llama_tokenizer_vocab_size(const wgb_llama_tokenizer *t);
int wgb_llama_tokenizer_encode(const wgb_llama_tokenizer *t, const char *text, size_t text_len, int bos, int eos,
                               uint32_t *out_ids, size_t cap, size_t *n_out);
int wgb_llama_tokenizer_decode(const wgb_llama_tokenizer *t, uint32_t prev_token, uint32_t token, char *buf, size_t cap,
                               size_t *len);
/* Gpt2Tokenizer (models/gpt2/tokenizer.rs:38-217) from tokenizer.ggml.tokens, .merges, .bos_token_id,
 * .eos_token_id (tokenizer.rs:56-60): "<...>" spans are special tokens (tokenizer.rs:128-139, an unknown one
 * is WGB_ERR_NOT_FOUND where the reference panics), the rest is split by the GPT-2 pattern (tokenizer.rs:75),
 * mapped byte by byte to printable characters (bytes_to_unicode, tokenizer.rs:22-36) and merged by rank.
 * \p{L} and \p{N} are decided exactly for ASCII and by the C library's UTF-8 character tables beyond it. */
typedef struct wgb_gpt2_tokenizer wgb_gpt2_tokenizer;
int wgb_gpt2_tokenizer_from_gguf(const wgb_gguf *g, wgb_gpt2_tokenizer **out);
int wgb_gpt2_tokenizer_destroy(wgb_gpt2_tokenizer *t);
uint32_t wgb_gpt2_tokenizer_bos(const wgb_gpt2_tokenizer *t);
uint32_t wgb_gpt2_tokenizer_eos(const wgb_gpt2_tokenizer *t);
int wgb_gpt2_tokenizer_encode(const wgb_gpt2_tokenizer *t, const char *text, size_t text_len, uint32_t *out_ids, size_t cap,
                              size_t *n_out);
int wgb_gpt2_tokenizer_decode(const wgb_gpt2_tokenizer *t, const uint32_t *tokens, size_t n, char *buf, size_t cap, size_t *len);
/* ChatTemplate::apply (crates/wgml-chat/src/chat_template.rs:27-39) for the default template
 * (LlamaTokenizer::CHAT_TEMPLATE, models/llama2/llama-2-chat.jinja) with minijinja configured as there
 * (trim_blocks, bos_token / eos_token globals): roles[i] in {"system" (first only), "user", "assistant"},
 * alternating from "user" (else WGB_ERR_INVALID with the template's own message).  The white space the
 * template leaves between its tags is part of the rendering and is reproduced.  Templates carried by a GGUF
 * (tokenizer.chat_template, chat_template.rs:18-25) are arbitrary Jinja and are not interpreted. */
int wgb_chat_template_llama2(const char *const *roles, const char *const *contents, size_t n_messages, const char *bos,
                             const char *eos, char *buf, size_t cap, size_t *len);

/* ---- Llama-2 family ---- */

/* Llama2Config (models/llama2/cpu.rs:46-67); usize fields are u32 here. */
typedef struct {
    uint32_t dim;
    uint32_t hidden_dim;
    uint32_t n_layers;
    uint32_t n_q_heads;
    uint32_t n_kv_heads;
    uint32_t vocab_size;
    uint32_t seq_len;
    float rope_base_freq;
    float rms_norm_eps;
} wgb_llama2_config;
/* LlamaModelType (models/llama2/mod.rs:14-32): Qwen2 = q/k/v biases + Neox RoPE. */
typedef enum { WGB_LLAMA = 0, WGB_QWEN2 = 1 } wgb_llama_model_type;
/* Llama2Config::from_gguf_with_model_type (cpu.rs:79-109), same keys and defaults. */
int wgb_llama2_config_from_gguf(const wgb_gguf *g, int model_type, wgb_llama2_config *out);

/* Per-layer matrices / vectors of Llama2LayerWeights (models/llama2/transformer.rs:128-141). */
typedef enum {
    WGB_L_ATTN_Q = 0, WGB_L_ATTN_K, WGB_L_ATTN_V, WGB_L_ATTN_OUTPUT, WGB_L_FFN_GATE, WGB_L_FFN_UP,
    WGB_L_FFN_DOWN
} wgb_llama2_matrix;
typedef enum {
    WGB_L_ATTN_NORM = 0, WGB_L_FFN_NORM, WGB_L_ATTN_Q_BIAS, WGB_L_ATTN_K_BIAS, WGB_L_ATTN_V_BIAS
} wgb_llama2_vector;
/* Model-level tensors of Llama2Weights (transformer.rs:143-148), used with layer = -1. */
typedef enum { WGB_L_TOKEN_EMBD = 0, WGB_L_OUTPUT = 1 } wgb_llama2_model_matrix;

/* Llama2 + Llama2Weights + Llama2State (models/llama2/transformer.rs:17-126,143-148,271-296)
 * for tensor-parallel rank `tp_rank` of `tp_size` (1 GPU: 0 of 1).  The model owns its weights,
 * activations and KV cache on the current device. */
typedef struct wgb_llama2 wgb_llama2;
int wgb_llama2_create(const wgb_llama2_config *cfg, int model_type, int tp_rank, int tp_size,
                      wgb_llama2 **out);
int wgb_llama2_destroy(wgb_llama2 *m);
/* Upload one tensor from host memory (raw GGUF blocks or f32).  Under tensor parallelism the
 * full tensor is passed and the rank keeps its slice.  layer = -1 addresses token_embd / output
 * / output_norm; output defaults to token_embd when never set (transformer.rs:244-257). */
int wgb_llama2_set_matrix(wgb_llama2 *m, int layer, int which, int qtype, const void *h_blocks,
                          size_t nrows, size_t ncols);
int wgb_llama2_set_vector(wgb_llama2 *m, int layer, int which, const float *h_data, size_t n);
/* Llama2Weights::from_gguf (transformer.rs:151-268): same tensor names. */
int wgb_llama2_load_gguf(wgb_llama2 *m, const wgb_gguf *g);
/* Required for tp_size > 1: the communicator of the tensor-parallel group (see wgb_comm_create below);
 * `comm` is a `wgb_comm *`.  The model does not own it. */
int wgb_llama2_set_comm(wgb_llama2 *m, void *comm);
/* 1 (default): fused kernels (norm + matrix product + RoPE / KV append / SiLU / residual in one
 * launch each).  0: one launch per reference dispatch, in the order of Llama2::dispatch
 * (transformer.rs:310-427); also what is used when a layer mixes block formats that have no fused
 * kernel. */
int wgb_llama2_set_fused(wgb_llama2 *m, int enable);
/* Llama2::dispatch + the embedding copy of ChatLlama2::forward_logits (transformer.rs:298-431,
 * crates/wgml-chat/src/chat_llama2.rs:155-213): one token at position pos; logits stay on the
 * device (wgb_llama2_logits). */
int wgb_llama2_forward(wgb_llama2 *m, uint32_t token, uint32_t pos, void *stream);
/* Device pointers into Llama2State (transformer.rs:17-45): logits [vocab_size], x [dim], key / value cache
 * of a layer.  The caches are head-major, [n_kv_heads / tp_size][seq_len][head_size] (the reference keeps
 * [seq_len][kv_dim], transformer.rs:75-80): the positions of one KV head are contiguous, so the attention
 * kernel can move 64 of them with one bulk copy.  Element (pos, head, e) of the reference layout is element
 * (head, pos, e) here. */
const float *wgb_llama2_logits(const wgb_llama2 *m);
const float *wgb_llama2_x(const wgb_llama2 *m);
float *wgb_llama2_key_cache(wgb_llama2 *m, uint32_t layer);
float *wgb_llama2_value_cache(wgb_llama2 *m, uint32_t layer);
/* The token loop of ChatLlama2::forward (chat_llama2.rs:102-121) with the forced-token rule of
 * sample_next_token (crates/wgml-chat/src/sampler.rs:102-107) and greedy sampling
 * (Sampler::sample with temperature 0, models/sampler.rs:33-35), kept on the device: token ids,
 * position, logits, argmax and the KV cache never leave the GPU and every step replays one CUDA
 * graph.  h_prompt: n_prompt >= 1 host token ids, the first fed at position start_pos.
 * h_out_tokens receives n_prompt - 1 + n_gen ids: the token fed at each following position. */
int wgb_llama2_decode(wgb_llama2 *m, const uint32_t *h_prompt, size_t n_prompt, size_t n_gen,
                      uint32_t start_pos, uint32_t *h_out_tokens, void *stream);
/* Weight upload so far: bytes copied host -> device and the wall time the copies took (first byte taken to
 * last repack kernel finished, summed over wgb_llama2_set_matrix calls and wgb_llama2_load_gguf).  The loader
 * replaces the reference's eager element-by-element parse (gguf.rs:539-620, 671-681) by a pipeline: bytes go
 * from the mapped file through a ring of pinned buffers to the device on a copy stream, the repack kernels of
 * the planar formats run behind them, and nothing is waited for until the last tensor is enqueued. */
int wgb_llama2_load_stats(const wgb_llama2 *m, size_t *bytes, double *seconds);
/* Sampling of the generated tokens in wgb_llama2_decode: Sampler::new(vocab, temperature, topp)
 * (models/sampler.rs:21-29; the chat loop uses 0.7 / 0.95, crates/wgml-chat/src/sampler.rs:109-110) with
 * coin = wgb_sampler_coin(seed, position of the sampled token).  temperature 0 (the default) is greedy.
 * The draw happens on the device: no logits leave it. */
int wgb_llama2_set_sampler(wgb_llama2 *m, float temperature, float topp, uint64_t seed);
/* Batched prompt prefill, no counterpart in the reference (its chat loop feeds the prompt one position per
 * Llama2::dispatch, chat_llama2.rs:104-116,169-204, and drops the logits).  Once enabled, wgb_llama2_decode
 * sends every prompt position but the last through passes of eight positions: the Q4_K layer matrices are
 * multiplied on the tensor cores (tcgen05.mma kind::i8 on the same fixed-point image of the activations as the
 * matrix-vector kernels, from tile-major copies of the weights made here, which doubles their memory), the Q6_K
 * and Q8_0 ones by kernels of their own (Q6_K: scales folded into the weight operand; Q8_0: the codes are the operand),
 * other formats through the matrix-vector
 * kernel position by position; RMSNorm, RoPE, the cache rows and causal attention are computed per pass.  Cache rows and everything after the prompt agree with the
 * position-by-position path to the order of the f32 additions.  A tensor-parallel rank sums its partial attn_output
 * and ffn_down products over the group with one all-reduce each per pass and layer (call wgb_llama2_set_comm first,
 * else WGB_ERR_UNSUPPORTED); enable it after the weights are set (setting a matrix disables it). */
int wgb_llama2_set_prefill(wgb_llama2 *m, int enable);
/* Prompt positions that have gone through the batched passes since it was enabled. */
int wgb_llama2_prefill_positions(const wgb_llama2 *m, size_t *positions);
/* Number of kernels one decode step launches (for launch accounting). */
int wgb_llama2_kernels_per_token(const wgb_llama2 *m);
/* Measurement aid, the counterpart of wgcore's GpuTimestamps around a pass
 * (crates/wgml-bench/src/main.rs:201,226-241): the time each launch of one forward adds to the step.
 * Fused schedule on one GPU, or tensor parallel with the direct exchange: the step is replayed from a CUDA graph exactly as wgb_llama2_decode runs it
 * (programmatic dependent launch included) and every launch leaves its end time (%globaltimer) in device
 * memory; a launch's time is the distance from its predecessor's end to its own (the embedding copy is
 * counted with the first launch).  Otherwise (unfused schedule, NCCL exchange): a CUDA event after every
 * launch.  Reports per launch its kind (0 embedding, 1 norm+QKV+RoPE, 2 attention, 3 output projection,
 * 4 norm+gate/up+SiLU, 5 down projection, 6 norm+logits, 7 unfused layer), its layer (-1 outside layers)
 * and the milliseconds.  At most `cap` entries are written; *n_out is their number. */
int wgb_llama2_profile_step(wgb_llama2 *m, uint32_t token, uint32_t pos, void *stream, int cap,
                            int *kinds, int *layers, float *ms, int *n_out);

/* ---- Tensor-parallel group ----
 * No counterpart in the reference, which runs on one device (crates/wgml-bench/src/main.rs:23-36 picks
 * a single adapter); this is what lets Llama-2-70B-sized weights be sharded over several GPUs.  One
 * process per GPU.  Rank 0 makes an id, the host program hands it to the other ranks (MPI,
 * torch.distributed, a file), then every rank calls wgb_comm_create with its device current.
 * Sharding: Q/K/V, gate and up keep the rows of their heads / hidden slice; attn_output and ffn_down
 * keep the matching columns and their partial products are summed over the group (NCCL all-reduce,
 * the residual added by rank 0 before the sum); embeddings, norms and the output matrix are replicated. */
#define WGB_COMM_ID_BYTES 128
typedef struct wgb_comm wgb_comm;
int wgb_comm_unique_id(void *id_out /* WGB_COMM_ID_BYTES */);
int wgb_comm_create(const void *id, int rank, int size, wgb_comm **out);
int wgb_comm_destroy(wgb_comm *c);
int wgb_comm_rank(const wgb_comm *c);
int wgb_comm_size(const wgb_comm *c);
/* d_recv[i] = sum over ranks of d_send[i]; in place when d_send == d_recv. */
int wgb_comm_all_reduce_sum(wgb_comm *c, const float *d_send, float *d_recv, size_t n, void *stream);
/* d_recv[r * n_per_rank + i] = rank r's d_send[i]. */
int wgb_comm_all_gather(wgb_comm *c, const float *d_send, float *d_recv, size_t n_per_rank, void *stream);
/* A zero-filled device buffer of `bytes` on every rank, each mapped into every other rank's address space
 * (CUDA IPC between the processes; peer access over NVLink).  peers_out[p] (size entries, at most
 * WGB_COMM_MAX_PEERS) is rank p's buffer as seen from this rank, peers_out[rank] the local one.
 * Collective; the buffers live as long as the communicator. */
#define WGB_COMM_MAX_PEERS 8
int wgb_comm_shared_alloc(wgb_comm *c, size_t bytes, void **peers_out);
/* Tensor-parallel models exchange the partial products of attn_output / ffn_down either with one NCCL
 * all-reduce each (mode 0, default) or directly (mode 1): the matrix-vector kernel's epilogue stores its
 * partial rows into every rank's mailbox over NVLink and raises a flag, and the next kernel's prologue
 * waits for the tp flags (bounded) and adds the tp partials in rank order while it normalises its input.
 * No collective library call and no extra launch remain on the token path.  Call after
 * wgb_llama2_set_comm and before the first forward; collective (every rank, same mode). */
int wgb_llama2_set_exchange(wgb_llama2 *m, int mode);
/* Vocabulary-sharded output head of a tensor-parallel model (off by default): every rank multiplies only rows
 * [tp_rank, tp_rank + 1) * vocab_size / tp_size of the output matrix -- a view of the replicated matrix, no
 * reload -- and one NCCL all-gather per token gives every rank all the logits, so that the argmax, the
 * sampler and wgb_llama2_logits see what they see on one GPU.  Needs the communicator and a vocabulary that
 * is a multiple of tp_size; no effect on a single-GPU model.  Collective: every rank, same setting, before
 * the next forward.  No counterpart in the reference (one adapter; the head is the last `matmul` of
 * crates/wgml/src/models/llama2/transformer.rs:310-427). */
int wgb_llama2_set_vocab_shard(wgb_llama2 *m, int on);
/* Direct exchange on buffers the host mapped itself (its own CUDA IPC, cuMem fabric or symmetric-memory
 * allocator) instead of wgb_comm_shared_alloc: d_mail[p] / d_flags[p] are rank p's mailbox and flags as
 * seen from this rank, of the sizes wgb_llama2_exchange_bytes gives, zero-filled, 16-byte aligned, valid
 * for the life of the model; entry [tp_rank] is this rank's own.  Selects mode 1; no communicator is
 * needed on the token path.  No counterpart in the reference (wgml runs on one adapter,
 * crates/wgml-chat/src/chat_llama2.rs:168-213). */
int wgb_llama2_exchange_bytes(const wgb_llama2 *m, size_t *mail_bytes, size_t *flag_bytes);
int wgb_llama2_set_exchange_buffers(wgb_llama2 *m, void *const *d_mail, void *const *d_flags);
/* How long a kernel waits for the flags of the other ranks before it gives up, in milliseconds (default
 * 2000; it has to cover the skew between the ranks' host threads).  A wait that runs out leaves a code in
 * the device's status word: the decode call in progress returns WGB_ERR_TIMEOUT within two batches of 64
 * steps, and while the word is set no kernel waits for peers at all, so a missing rank costs one limit,
 * not one per exchange.  After WGB_ERR_TIMEOUT the group's step counts no longer agree: rebuild the
 * models of every rank.  Process-wide.  No counterpart in the reference. */
int wgb_set_wait_limit_ms(unsigned ms);
unsigned wgb_get_wait_limit_ms(void);

/* ---- GPT-2 ---- */

/* Gpt2Params (models/gpt2/cpu.rs:18-33); usize fields are u32 here. */
typedef struct {
    uint32_t n_vocab;
    uint32_t n_seq;
    uint32_t n_embd;
    uint32_t n_head;
    uint32_t n_layer;
    uint32_t ff_len;
    uint32_t attn_b;
    uint32_t ftype;
} wgb_gpt2_params;
/* Gpt2Params::from_gguf (gpt2/cpu.rs:36-47). */
int wgb_gpt2_params_from_gguf(const wgb_gguf *g, wgb_gpt2_params *out);

/* Gpt2LayerWeights (models/gpt2/transformer.rs:70-94). */
typedef enum { WGB_G_ATTN_QKV = 0, WGB_G_ATTN_PROJ, WGB_G_MLP_FC, WGB_G_MLP_PROJ } wgb_gpt2_matrix;
typedef enum {
    WGB_G_LN_1_G = 0, WGB_G_LN_1_B, WGB_G_LN_2_G, WGB_G_LN_2_B, WGB_G_ATTN_QKV_B, WGB_G_ATTN_PROJ_B,
    WGB_G_MLP_FC_B, WGB_G_MLP_PROJ_B
} wgb_gpt2_vector;
/* Gpt2Weights (transformer.rs:96-106), with layer = -1: matrices WTE / WPE (lm_head is WTE,
 * transformer.rs:194-195), vectors LN_F_G / LN_F_B. */
typedef enum { WGB_G_WTE = 0, WGB_G_WPE = 1 } wgb_gpt2_model_matrix;
typedef enum { WGB_G_LN_F_G = 0, WGB_G_LN_F_B = 1 } wgb_gpt2_model_vector;

/* Gpt2 + Gpt2Weights + Gpt2State (models/gpt2/transformer.rs:14-68,96-106,240-263). */
typedef struct wgb_gpt2 wgb_gpt2;
int wgb_gpt2_create(const wgb_gpt2_params *params, wgb_gpt2 **out);
int wgb_gpt2_destroy(wgb_gpt2 *m);
int wgb_gpt2_set_matrix(wgb_gpt2 *m, int layer, int which, int qtype, const void *h_blocks,
                        size_t nrows, size_t ncols);
int wgb_gpt2_set_vector(wgb_gpt2 *m, int layer, int which, const float *h_data, size_t n);
/* Gpt2Weights::from_gguf (transformer.rs:109-205).  Matrices stay quantised (the reference
 * dequantises them to f32 first, transformer.rs:133-140; the products are the same). */
int wgb_gpt2_load_gguf(wgb_gpt2 *m, const wgb_gguf *g);
/* As wgb_llama2_set_fused. */
int wgb_gpt2_set_fused(wgb_gpt2 *m, int enable);
/* Gpt2::dispatch (transformer.rs:265-477). */
int wgb_gpt2_forward(wgb_gpt2 *m, uint32_t token, uint32_t pos, void *stream);
const float *wgb_gpt2_logits(const wgb_gpt2 *m);
float *wgb_gpt2_key_cache(wgb_gpt2 *m, uint32_t layer);
float *wgb_gpt2_value_cache(wgb_gpt2 *m, uint32_t layer);
/* As wgb_llama2_set_sampler. */
int wgb_gpt2_set_sampler(wgb_gpt2 *m, float temperature, float topp, uint64_t seed);
/* Batched prompt prefill as wgb_llama2_set_prefill, for Gpt2::dispatch (models/gpt2/transformer.rs:265-477): passes of
 * eight positions with LayerNorm, the fused qkv product and its split into cache rows, causal attention, the
 * projections and GELU computed per pass; Q8_0 / Q4_K / Q6_K matrices on the tensor cores.  The reference's loop
 * (chat_gpt2.rs:43-151) feeds the prompt one position per dispatch. */
int wgb_gpt2_set_prefill(wgb_gpt2 *m, int enable);
int wgb_gpt2_prefill_positions(const wgb_gpt2 *m, size_t *positions);
/* ChatGpt2::forward's loop (crates/wgml-chat/src/chat_gpt2.rs:43-151), device-resident. */
int wgb_gpt2_decode(wgb_gpt2 *m, const uint32_t *h_prompt, size_t n_prompt, size_t n_gen,
                    uint32_t start_pos, uint32_t *h_out_tokens, void *stream);
int wgb_gpt2_kernels_per_token(const wgb_gpt2 *m);

#ifdef __cplusplus
}
#endif
#endif /* WGML_B200_H */
