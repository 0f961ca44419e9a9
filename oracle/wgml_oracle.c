/*
 * wgml_oracle.c -- CPU restatement of wgml's CPU reference code for the per-token
 * transformer forward (quantised blocks, the ops' `run_cpu` twins, the Llama-2 and GPT-2
 * CPU transformers and the greedy sampler).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared with and
 * the CPU baseline that is timed next to them.  Nothing that ships may call into it.
 *
 * The original is Rust and cannot be built where this repository is developed, so every
 * function below restates, in plain C, the function named in its comment (paths are relative
 * to the wgml repository).  Build with `-O2 -ffp-contract=off`: Rust never contracts `a*b+c`
 * into an FMA, and dequantised weights have to match bit for bit.
 *
 * Third-party arithmetic.  The Rust code performs its reductions with nalgebra 0.33.1
 * (`gemv`, `dot`, `norm_squared`, `axpy`, `mean`, `max`, `imax`).  nalgebra is not part of the
 * wgml tree; the loops here follow its published implementation (src/base/blas.rs: `dot` keeps
 * eight partial sums per column and folds them as (a0+a4)+(a1+a5)+(a2+a6)+(a3+a7) before a
 * scalar tail; `gemv` is one `axpy` per matrix column).  That order cannot be checked offline,
 * so f32 reductions are only ever compared to a tolerance, never bit for bit.
 *
 * Pinning.  Dequantisation is pinned by the deterministic block patterns of the reference's
 * own `dequantization` test (crates/wgml/src/ops/quantization.rs:79-222) evaluated with an
 * independent implementation of the same ggml formats (gguf-py `quants.dequantize`); see
 * tests/golden/.  No reference test stores numeric outputs for GEMV, attention or the
 * transformers: for those the parity is "unpinned" beyond this restatement.  What anchors the
 * reading of the architectures instead is an implementation that shares no code with this one:
 * tests/test_oracle_hf.py compares the Llama (Original RoPE), Qwen2 (Neox RoPE, biases) and
 * GPT-2 forwards below with logits that Hugging Face `transformers` computes in float64 for
 * the same seeded weights (tests/golden/make_hf_golden.py): they agree to 4e-6 on logits of
 * order 3 (Llama, Qwen2) and 3e-5 on logits of order 70 (GPT-2).  That check says nothing about wgml's summation order.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define WGO_API __attribute__((visibility("default")))

/* ggml tensor type ids, crates/wgml/src/gguf.rs:73-105 */
enum {
    WGO_F32 = 0, WGO_F16 = 1, WGO_Q4_0 = 2, WGO_Q4_1 = 3, WGO_Q5_0 = 6, WGO_Q5_1 = 7,
    WGO_Q8_0 = 8, WGO_Q4_K = 12, WGO_Q5_K = 13, WGO_Q6_K = 14, WGO_Q8_K = 15
};

#define QK_K 256
#define K_SCALE_SIZE 12

/* ------------------------------------------------------------------------------------------
 * decode_f16 -- crates/wgml/src/quantization.rs:392-409
 * ---------------------------------------------------------------------------------------- */
WGO_API float wgo_decode_f16(uint16_t half)
{
    uint16_t exp = (half >> 10) & 0x1f;
    uint16_t mant = half & 0x3ff;
    float val;
    if (exp == 0) {
        val = (float)mant * 5.9604644775390625e-8f; /* 2^-24 */
    } else if (exp != 31) {
        val = ((float)mant + 1024.0f) * ldexpf(1.0f, (int)exp - 25);
    } else if (mant == 0) {
        val = INFINITY;
    } else {
        val = NAN;
    }
    return (half & 0x8000) ? -val : val;
}

/* Bytes per block / weights per block; struct layouts of crates/wgml/src/quantization.rs. */
WGO_API int wgo_block_bytes(int qtype)
{
    switch (qtype) {
    case WGO_F32: return 4;
    case WGO_F16: return 2;
    case WGO_Q4_0: return 18;  /* :47-50  */
    case WGO_Q4_1: return 20;  /* :74-78  */
    case WGO_Q5_0: return 22;  /* :103-107 */
    case WGO_Q5_1: return 24;  /* :134-139 */
    case WGO_Q8_0: return 34;  /* :29-32  */
    case WGO_Q4_K: return 144; /* :322-327 */
    case WGO_Q5_K: return 176; /* :249-255 */
    case WGO_Q6_K: return 210; /* :204-209 */
    case WGO_Q8_K: return 292; /* :170-174 */
    default: return 0;
    }
}

WGO_API int wgo_block_len(int qtype)
{
    switch (qtype) {
    case WGO_F32: case WGO_F16: return 1;
    case WGO_Q4_0: case WGO_Q4_1: case WGO_Q5_0: case WGO_Q5_1: case WGO_Q8_0: return 32;
    case WGO_Q4_K: case WGO_Q5_K: case WGO_Q6_K: case WGO_Q8_K: return QK_K;
    default: return 0;
    }
}

static inline uint16_t rd16(const uint8_t *p) { uint16_t v; memcpy(&v, p, 2); return v; }
static inline uint32_t rd32(const uint8_t *p) { uint32_t v; memcpy(&v, p, 4); return v; }

/* BlockQ8_0::dequantize -- quantization.rs:38-41 */
static void deq_q8_0(const uint8_t *b, float *out)
{
    float scale = wgo_decode_f16(rd16(b));
    const int8_t *data = (const int8_t *)(b + 2);
    for (int i = 0; i < 32; i++) out[i] = (float)data[i] * scale;
}

/* BlockQ4_0::dequantize -- quantization.rs:55-68 */
static void deq_q4_0(const uint8_t *b, float *out)
{
    float d = wgo_decode_f16(rd16(b));
    const uint8_t *qs = b + 2;
    for (int j = 0; j < 16; j++) {
        int x0 = (int)(qs[j] & 0x0F) - 8;
        int x1 = (int)(qs[j] >> 4) - 8;
        out[j] = (float)x0 * d;
        out[j + 16] = (float)x1 * d;
    }
}

/* BlockQ4_1::dequantize -- quantization.rs:83-97 */
static void deq_q4_1(const uint8_t *b, float *out)
{
    float d = wgo_decode_f16(rd16(b));
    float m = wgo_decode_f16(rd16(b + 2));
    const uint8_t *qs = b + 4;
    for (int j = 0; j < 16; j++) {
        uint8_t x0 = qs[j] & 0x0F;
        uint8_t x1 = qs[j] >> 4;
        out[j] = (float)x0 * d + m;
        out[j + 16] = (float)x1 * d + m;
    }
}

/* BlockQ5_0::dequantize -- quantization.rs:112-128 */
static void deq_q5_0(const uint8_t *b, float *out)
{
    float d = wgo_decode_f16(rd16(b));
    uint32_t qh = rd32(b + 2);
    const uint8_t *qs = b + 6;
    for (int j = 0; j < 16; j++) {
        uint32_t xh_0 = ((qh >> j) << 4) & 0x10;
        uint32_t xh_1 = (qh >> (j + 12)) & 0x10;
        int x0 = (int)(((uint32_t)qs[j] & 0x0F) | xh_0) - 16;
        int x1 = (int)(((uint32_t)qs[j] >> 4) | xh_1) - 16;
        out[j] = (float)x0 * d;
        out[j + 16] = (float)x1 * d;
    }
}

/* BlockQ5_1::dequantize -- quantization.rs:144-161 */
static void deq_q5_1(const uint8_t *b, float *out)
{
    float d = wgo_decode_f16(rd16(b));
    float m = wgo_decode_f16(rd16(b + 2));
    uint32_t qh = rd32(b + 4);
    const uint8_t *qs = b + 8;
    for (int j = 0; j < 16; j++) {
        uint32_t xh_0 = ((qh >> j) << 4) & 0x10;
        uint32_t xh_1 = (qh >> (j + 12)) & 0x10;
        uint32_t x0 = ((uint32_t)qs[j] & 0x0F) | xh_0;
        uint32_t x1 = ((uint32_t)qs[j] >> 4) | xh_1;
        out[j] = (float)x0 * d + m;
        out[j + 16] = (float)x1 * d + m;
    }
}

/* BlockQ8K::dequantize -- quantization.rs:192-198 (d is a plain f32) */
static void deq_q8_k(const uint8_t *b, float *out)
{
    float d;
    memcpy(&d, b, 4);
    const int8_t *qs = (const int8_t *)(b + 4);
    for (int j = 0; j < QK_K; j++) out[j] = d * (float)qs[j];
}

/* BlockQ6K::dequantize -- quantization.rs:214-243.  `d * sc * q` associates left. */
static void deq_q6_k(const uint8_t *b, float *out)
{
    const uint8_t *ql = b;
    const uint8_t *qh = b + 128;
    const int8_t *scales = (const int8_t *)(b + 192);
    float d = wgo_decode_f16(rd16(b + 208));
    for (int i = 0; i < 2; i++) {
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            uint8_t ql0 = ql[i * 64 + l];
            uint8_t ql32 = ql[i * 64 + l + 32];
            uint8_t h = qh[i * 32 + l];
            int8_t q1 = (int8_t)(((ql0 & 0xF) | (((h >> 0) & 3) << 4))) - 32;
            int8_t q2 = (int8_t)(((ql32 & 0xF) | (((h >> 2) & 3) << 4))) - 32;
            int8_t q3 = (int8_t)(((ql0 >> 4) | (((h >> 4) & 3) << 4))) - 32;
            int8_t q4 = (int8_t)(((ql32 >> 4) | (((h >> 6) & 3) << 4))) - 32;
            out[i * 128 + l + 0] = d * (float)scales[i * 8 + is + 0] * (float)q1;
            out[i * 128 + l + 32] = d * (float)scales[i * 8 + is + 2] * (float)q2;
            out[i * 128 + l + 64] = d * (float)scales[i * 8 + is + 4] * (float)q3;
            out[i * 128 + l + 96] = d * (float)scales[i * 8 + is + 6] * (float)q4;
        }
    }
}

/* get_scale_min_k4 -- quantization.rs:381-389 */
static void get_scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m)
{
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (uint8_t)((q[j + 4] & 0xf) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* BlockQ4K::dequantize -- quantization.rs:347-378.  `d1 * q - m1`: a multiply, then a
 * subtract, each rounded. */
static void deq_q4_k(const uint8_t *b, float *out)
{
    float d = wgo_decode_f16(rd16(b));
    float min = wgo_decode_f16(rd16(b + 2));
    const uint8_t *scales = b + 4;
    const uint8_t *qs = b + 16;
    int is = 0, iq = 0;
    uint8_t sc = 0, m = 0;
    for (int j = 0; j < QK_K; j += 64) {
        get_scale_min_k4(is, scales, &sc, &m);
        float d1 = d * (float)sc;
        float m1 = min * (float)m;
        get_scale_min_k4(is + 1, scales, &sc, &m);
        float d2 = d * (float)sc;
        float m2 = min * (float)m;
        for (int l = 0; l < 32; l++) out[j + l] = d1 * (float)(qs[iq + l] & 0xF) - m1;
        for (int l = 0; l < 32; l++) out[j + l + 32] = d2 * (float)(qs[iq + l] >> 4) - m2;
        iq += 32;
        is += 2;
    }
}

/* BlockQ5K::dequantize -- quantization.rs:275-316 */
static void deq_q5_k(const uint8_t *b, float *out)
{
    float d = wgo_decode_f16(rd16(b));
    float min = wgo_decode_f16(rd16(b + 2));
    const uint8_t *scales = b + 4;
    const uint8_t *qh = b + 16;
    const uint8_t *qs = b + 48;
    int is = 0, iq = 0;
    uint8_t sc = 0, m = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int j = 0; j < QK_K; j += 64) {
        get_scale_min_k4(is, scales, &sc, &m);
        float d1 = d * (float)sc;
        float m1 = min * (float)m;
        get_scale_min_k4(is + 1, scales, &sc, &m);
        float d2 = d * (float)sc;
        float m2 = min * (float)m;
        for (int l = 0; l < 32; l++) {
            uint8_t v = (uint8_t)((qs[iq + l] & 0xF) + ((qh[l] & u1) ? 16 : 0));
            out[j + l] = d1 * (float)v - m1;
        }
        for (int l = 0; l < 32; l++) {
            uint8_t v = (uint8_t)((qs[iq + l] >> 4) + ((qh[l] & u2) ? 16 : 0));
            out[j + l + 32] = d2 * (float)v - m2;
        }
        iq += 32;
        is += 2;
        u1 <<= 2;
        u2 <<= 2;
    }
}

static void deq_block(int qtype, const uint8_t *b, float *out)
{
    switch (qtype) {
    case WGO_F32: memcpy(out, b, 4); break;
    case WGO_F16: out[0] = wgo_decode_f16(rd16(b)); break; /* BlockF16, quantization.rs:21-23 */
    case WGO_Q4_0: deq_q4_0(b, out); break;
    case WGO_Q4_1: deq_q4_1(b, out); break;
    case WGO_Q5_0: deq_q5_0(b, out); break;
    case WGO_Q5_1: deq_q5_1(b, out); break;
    case WGO_Q8_0: deq_q8_0(b, out); break;
    case WGO_Q4_K: deq_q4_k(b, out); break;
    case WGO_Q5_K: deq_q5_k(b, out); break;
    case WGO_Q6_K: deq_q6_k(b, out); break;
    case WGO_Q8_K: deq_q8_k(b, out); break;
    default: break;
    }
}

/* GgufTensorData::dequantize -- crates/wgml/src/gguf.rs:114-129 (block after block). */
WGO_API int wgo_dequantize(int qtype, const void *blocks, size_t nblocks, float *out)
{
    int bb = wgo_block_bytes(qtype), bl = wgo_block_len(qtype);
    if (!bb) return -1;
    const uint8_t *p = (const uint8_t *)blocks;
#pragma omp parallel for schedule(static) if (nblocks > 4096)
    for (size_t i = 0; i < nblocks; i++) deq_block(qtype, p + i * (size_t)bb, out + i * (size_t)bl);
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * nalgebra 0.33.1 primitives (see the header note).
 * ---------------------------------------------------------------------------------------- */
static float na_dot(const float *a, const float *b, size_t n)
{
    float res = 0.0f;
    float acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0, acc4 = 0, acc5 = 0, acc6 = 0, acc7 = 0;
    size_t i = 0;
    while (n - i >= 8) {
        acc0 += a[i + 0] * b[i + 0];
        acc1 += a[i + 1] * b[i + 1];
        acc2 += a[i + 2] * b[i + 2];
        acc3 += a[i + 3] * b[i + 3];
        acc4 += a[i + 4] * b[i + 4];
        acc5 += a[i + 5] * b[i + 5];
        acc6 += a[i + 6] * b[i + 6];
        acc7 += a[i + 7] * b[i + 7];
        i += 8;
    }
    res += acc0 + acc4;
    res += acc1 + acc5;
    res += acc2 + acc6;
    res += acc3 + acc7;
    for (; i < n; i++) res += a[i] * b[i];
    return res;
}

/* One output of `out.gemv(1.0, w, x, 0.0)` for a row of a matrix built with
 * `DMatrix::from_row_slice`: column j contributes (1.0 * x[j]) * w[row][j], added in order. */
static float na_gemv_row(const float *wrow, const float *x, size_t ncols)
{
    float y = x[0] * wrow[0];
    for (size_t j = 1; j < ncols; j++) y += x[j] * wrow[j];
    return y;
}

/* The same product accumulated in double: a second opinion that says on which side of the
 * f32 rounding noise a CUDA result sits. */
static double gemv_row_f64(const float *wrow, const float *x, size_t ncols)
{
    double y = 0.0;
    for (size_t j = 0; j < ncols; j++) y += (double)x[j] * (double)wrow[j];
    return y;
}

/* Test switch: when set, every matrix-vector product of the transformers below is accumulated in double and
 * rounded to f32 once (all else stays f32).  The distance between the two settings is how far f32 summation
 * rounding alone moves the logits of a model -- the yardstick a CUDA result is held against where a deep
 * random network amplifies rounding beyond the flat tolerance. */
static int g_dot_f64 = 0;
WGO_API void wgo_set_dot_f64(int on) { g_dot_f64 = on != 0; }

/* `matmul` of the CPU transformer -- crates/wgml/src/models/llama2/cpu.rs:368-374 -- over a
 * matrix that is still in GGUF blocks: each row is dequantised (exactly as
 * TransformerWeights::from_gguf does once at load, cpu.rs:198-217) and then multiplied.
 * `out64` may be NULL. */
WGO_API int wgo_gemv_quant(int qtype, const void *w, size_t nrows, size_t ncols, const float *x,
                           float *out, double *out64)
{
    int bb = wgo_block_bytes(qtype), bl = wgo_block_len(qtype);
    if (!bb || ncols % (size_t)bl) return -1;
    size_t bpr = ncols / (size_t)bl;
    const uint8_t *p = (const uint8_t *)w;
#pragma omp parallel
    {
        float *row = (float *)malloc(ncols * sizeof(float));
#pragma omp for schedule(static)
        for (size_t r = 0; r < nrows; r++) {
            const float *wr;
            if (qtype == WGO_F32) {
                wr = (const float *)p + r * ncols;
            } else {
                const uint8_t *rb = p + r * bpr * (size_t)bb;
                for (size_t k = 0; k < bpr; k++) deq_block(qtype, rb + k * (size_t)bb, row + k * (size_t)bl);
                wr = row;
            }
            out[r] = g_dot_f64 ? (float)gemv_row_f64(wr, x, ncols) : na_gemv_row(wr, x, ncols);
            if (out64) out64[r] = gemv_row_f64(wr, x, ncols);
        }
        free(row);
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * Ops' CPU twins.
 * ---------------------------------------------------------------------------------------- */

/* RmsNorm::run_cpu -- crates/wgml/src/ops/rms_norm.rs:55-63 (and cpu.rs:338-346).  The Rust
 * twin hard-codes 1e-5; the GPU kernel takes it from RmsNormConfig::nudge_factor
 * (rms_norm.wgsl:62), so it is a parameter here. */
WGO_API void wgo_rms_norm(float *out, const float *a, const float *w, size_t n, float eps)
{
    float rms = 1.0f / sqrtf(na_dot(a, a, n) / (float)n + eps);
    for (size_t i = 0; i < n; i++) out[i] = (a[i] * rms) * w[i];
}

/* LayerNorm::run_cpu -- crates/wgml/src/ops/layernorm.rs:46-54 */
WGO_API void wgo_layernorm(float *res, const float *v, size_t n)
{
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) sum += v[i];
    float mean = sum / (float)n;
    for (size_t i = 0; i < n; i++) res[i] = v[i] - mean;
    float variance = na_dot(res, res, n) / (float)n;
    float scale = 1.0f / sqrtf(variance + 1.0e-5f);
    for (size_t i = 0; i < n; i++) res[i] *= scale;
}

/* RoPE::run_cpu -- crates/wgml/src/ops/rope.rs:79-116 (variant 0, adjacent pairs) and the
 * `main_neox` shader -- crates/wgml/src/ops/rope.wgsl:57-77 (variant 1; it has no CPU twin,
 * so the shader arithmetic is restated).  `base` is 10000 in the CPU twin and
 * RoPEConfig::base_freq on the GPU.  Rotation2::new(a) * (x, y) = (c x - s y, s x + c y). */
WGO_API void wgo_rope(int variant, float *q, size_t q_len, float *k, uint32_t head_size,
                      uint32_t kv_dim, uint32_t pos, float base)
{
    for (size_t i = 0; i < q_len; i += 2) {
        float head_dim = (float)(i % head_size);
        float theta = powf(base, -head_dim / (float)head_size);
        float m_theta = (float)pos * theta;
        float s = sinf(m_theta), c = cosf(m_theta);
        size_t ia, ib;
        if (variant == 0) {
            ia = i;
            ib = i + 1;
        } else {
            size_t pair = i / 2;
            size_t head = i / head_size;
            ia = pair + head * head_size / 2;
            ib = ia + head_size / 2;
        }
        float x = q[ia], y = q[ib];
        q[ia] = c * x - s * y;
        q[ib] = s * x + c * y;
        if (i < kv_dim) {
            x = k[ia];
            y = k[ib];
            k[ia] = c * x - s * y;
            k[ib] = s * x + c * y;
        }
    }
}

/* SoftMax::run_cpu -- crates/wgml/src/ops/softmax.rs:36-49 (== cpu.rs:352-365) */
WGO_API void wgo_softmax(float *vals, size_t n)
{
    float max_val = vals[0];
    for (size_t i = 1; i < n; i++) if (vals[i] > max_val) max_val = vals[i];
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        vals[i] = expf(vals[i] - max_val);
        sum += vals[i];
    }
    for (size_t i = 0; i < n; i++) vals[i] /= sum;
}

/* Silu::run_cpu -- crates/wgml/src/ops/silu.rs:36-47 */
WGO_API void wgo_silu(float *h1, const float *h2, size_t n)
{
    for (size_t i = 0; i < n; i++) {
        float x = h1[i];
        h1[i] = h2[i] * (x / (1.0f + expf(-1.0f * x)));
    }
}

/* UnaryOp::eval -- crates/wgml/src/ops/unary.rs:87-129; op numbering follows the enum order
 * of unary.rs:16-38. */
WGO_API float wgo_unary(int op, float x, const float *args)
{
    float a0 = args ? args[0] : 0.0f, a1 = args ? args[1] : 0.0f;
    switch (op) {
    case 0: return fabsf(x);                                             /* Abs */
    case 1: return isnan(x) ? NAN : copysignf(1.0f, x);                  /* Sgn: f32::signum */
    case 2: return -x;                                                   /* Neg */
    case 3: return x > 0.0f ? 1.0f : 0.0f;                               /* Step */
    case 4: return x > 0.0f ? x : expf(x) - 1.0f;                        /* Elu */
    case 5: {                                                            /* Gelu */
        const float GELU_COEF_A = 0.044715f, SQRT_2_OVER_PI = 0.7978846f;
        return 0.5f * x * (1.0f + tanhf(SQRT_2_OVER_PI * x * (1.0f + GELU_COEF_A * x * x)));
    }
    case 6: return x * (1.0f / (1.0f + expf(-1.702f * x)));              /* GeluQuick */
    case 7: return x / (1.0f + expf(-x));                                /* Silu */
    case 8: return tanhf(x);                                             /* Tanh */
    case 9: return fmaxf(x, 0.0f);                                       /* Relu */
    case 10: return 1.0f / (1.0f + expf(-x));                            /* Sigmoid */
    case 11: return fminf(1.0f, fmaxf(0.0f, (x + 3.0f) / 6.0f));         /* HardSigmoid */
    case 12: return x * fminf(1.0f, fmaxf(0.0f, (x + 3.0f) / 6.0f));     /* HardSwish */
    case 13: return x * x;                                               /* Sqr */
    case 14: return sqrtf(x);                                            /* Sqrt */
    case 15: return logf(x);                                             /* Log */
    case 16: return fmaxf(x, 0.0f) + fminf(x, 0.0f) * a0;                /* LeakyRelu */
    case 17: { float t = x < a0 ? a0 : x; return t > a1 ? a1 : t; }      /* Clamp */
    case 18: return x * a0;                                              /* Scale */
    case 19: return x + a0;                                              /* AddScalar */
    default: return NAN;
    }
}

/* Unary::run_cpu -- unary.rs:196-202 */
WGO_API void wgo_unary_vec(int op, float *vals, size_t n, const float *args)
{
    for (size_t i = 0; i < n; i++) vals[i] = wgo_unary(op, vals[i], args);
}

/* BatchedMultiqueryAttentionParams -- ops/batched_multiquery_attention.rs:26-37 */
typedef struct {
    uint32_t seq_len, kv_dim, kv_mul, n_heads, head_size, pos;
} wgo_attn_params;

/* BatchedMultiqueryAttention::run_cpu -- ops/batched_multiquery_attention.rs:141-195
 * (== Transformer::attention, cpu.rs:486-537).  Caches are kv_dim x seq_len column-major, so
 * time step t is the t-th run of kv_dim floats; `attn` is seq_len x n_heads column-major. */
WGO_API void wgo_attention(const wgo_attn_params *p, const float *q, const float *key_cache,
                           const float *value_cache, float *attn, float *xb)
{
    size_t hs = p->head_size, kv_mul = p->kv_mul;
    for (size_t h = 0; h < p->n_heads; h++) {
        const float *qh = q + h * hs;
        float *att = attn + h * (size_t)p->seq_len;
        for (size_t t = 0; t <= p->pos; t++) {
            const float *kh = key_cache + t * (size_t)p->kv_dim + (h / kv_mul) * hs;
            float score = na_dot(qh, kh, hs);
            score /= sqrtf((float)hs);
            att[t] = score;
        }
        wgo_softmax(att, (size_t)p->pos + 1);
        float *xh = xb + h * hs;
        for (size_t i = 0; i < hs; i++) xh[i] = 0.0f;
        for (size_t t = 0; t <= p->pos; t++) {
            const float *vh = value_cache + t * (size_t)p->kv_dim + (h / kv_mul) * hs;
            float a = att[t];
            for (size_t i = 0; i < hs; i++) xh[i] = a * vh[i] + 1.0f * xh[i]; /* axpy(a, v, 1.0) */
        }
    }
}

/* The counter-based uniform draw of the device token loops (not in the reference, whose generator is unseeded,
 * crates/wgml/src/models/sampler.rs:42): splitmix64 of (seed, draw), top 24 bits, the form of rand's f32 sample. */
WGO_API float wgo_sampler_coin(uint64_t seed, uint64_t draw)
{
    uint64_t z = seed + (draw + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

typedef struct { float prob; size_t index; } wgo_prob_index;
/* `sort_by_key(|pid| OrderedFloat(-pid.prob))` is a stable sort: equal probabilities keep index order. */
static int cmp_prob_desc(const void *a, const void *b)
{
    const wgo_prob_index *x = (const wgo_prob_index *)a, *y = (const wgo_prob_index *)b;
    if (x->prob > y->prob) return -1;
    if (x->prob < y->prob) return 1;
    return x->index < y->index ? -1 : (x->index > y->index ? 1 : 0);
}

/* Sampler::sample -- crates/wgml/src/models/sampler.rs:32-52 with sample_mult :62-76 and sample_topp :84-130;
 * `coin` stands for `random()`.  `logits` is overwritten with the probabilities, as in the reference.
 * slack[0] receives the distance of the deciding comparison from its threshold, relative to the running sum:
 * a draw whose slack is at rounding level may legitimately land on the neighbouring token elsewhere. */
WGO_API size_t wgo_sample(float *logits, size_t n, float temperature, float topp, float coin, float *slack)
{
    if (slack) slack[0] = 1.0f;
    if (temperature == 0.0f) {
        size_t best = 0;
        for (size_t i = 1; i < n; i++) if (logits[i] > logits[best]) best = i;
        return best;
    }
    for (size_t i = 0; i < n; i++) logits[i] /= temperature;
    wgo_softmax(logits, n);
    if (topp <= 0.0f || topp >= 1.0f) {
        float cdf = 0.0f;
        for (size_t i = 0; i < n; i++) {
            float before = cdf;
            cdf += logits[i];
            if (coin < cdf) {
                if (slack) slack[0] = fminf(cdf - coin, i ? coin - before : 1.0f);
                return i;
            }
        }
        if (slack) slack[0] = 0.0f;
        return n - 1;
    }
    wgo_prob_index *pi = (wgo_prob_index *)malloc(n * sizeof(wgo_prob_index));
    size_t n0 = 0;
    float cutoff = (1.0f - topp) / ((float)n - 1.0f);
    for (size_t i = 0; i < n; i++) {
        if (logits[i] >= cutoff) {
            pi[n0].index = i;
            pi[n0].prob = logits[i];
            n0++;
        }
    }
    qsort(pi, n0, sizeof(wgo_prob_index), cmp_prob_desc);
    float cumulative = 0.0f;
    size_t last = n0 - 1;
    for (size_t i = 0; i < n0; i++) {
        cumulative += pi[i].prob;
        if (cumulative > topp) {
            last = i;
            break;
        }
    }
    float r = coin * cumulative, cdf = 0.0f;
    size_t pick = pi[last].index;
    float sl = 0.0f;
    for (size_t i = 0; i <= last; i++) {
        float before = cdf;
        cdf += pi[i].prob;
        if (r < cdf) {
            pick = pi[i].index;
            sl = fminf(cdf - r, i ? r - before : 1.0f) / cumulative;
            break;
        }
    }
    if (slack) slack[0] = sl;
    free(pi);
    return pick;
}

/* Sampler::sample_argmax -- crates/wgml/src/models/sampler.rs:54-56; nalgebra `imax` keeps
 * the first of equal maxima. */
WGO_API size_t wgo_argmax(const float *v, size_t n)
{
    size_t best = 0;
    for (size_t i = 1; i < n; i++) if (v[i] > v[best]) best = i;
    return best;
}

/* ------------------------------------------------------------------------------------------
 * Llama-2 CPU transformer -- crates/wgml/src/models/llama2/cpu.rs:259-562 with the GPU path's
 * extra parameters (crates/wgml/src/models/llama2/transformer.rs:298-431): configurable RMS
 * epsilon and RoPE base, optional q/k/v biases and the Neox rotation used for Qwen2.
 * Matrices stay in their GGUF blocks and are dequantised row by row inside the product,
 * which yields the same numbers as dequantising them all at load.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    int qtype;
    const void *data;
    size_t nrows, ncols;
} wgo_mat;

enum { WGO_ATTN_Q, WGO_ATTN_K, WGO_ATTN_V, WGO_ATTN_OUT, WGO_FFN_GATE, WGO_FFN_UP, WGO_FFN_DOWN,
       WGO_N_LAYER_MATS };
enum { WGO_ATTN_NORM, WGO_FFN_NORM, WGO_Q_BIAS, WGO_K_BIAS, WGO_V_BIAS, WGO_N_LAYER_VECS };

typedef struct {
    wgo_mat m[WGO_N_LAYER_MATS];
    const float *v[WGO_N_LAYER_VECS];
} wgo_llama2_layer;

typedef struct {
    uint32_t dim, hidden_dim, n_layers, n_q_heads, n_kv_heads, vocab_size, seq_len;
    float rope_base_freq, rms_norm_eps;
    int rope_variant; /* 0 Original (Llama), 1 Neox (Qwen2): models/llama2/mod.rs:26-32 */
    wgo_llama2_layer *layers;
    wgo_mat token_embd, output;
    const float *output_norm;
    float *x, *xb, *xb2, *hb, *hb2, *q, *att, *logits, *key_cache, *value_cache, *embd_row;
} wgo_llama2;

WGO_API wgo_llama2 *wgo_llama2_new(uint32_t dim, uint32_t hidden_dim, uint32_t n_layers,
                                   uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t vocab_size,
                                   uint32_t seq_len, float rope_base_freq, float rms_norm_eps,
                                   int rope_variant)
{
    wgo_llama2 *m = (wgo_llama2 *)calloc(1, sizeof(*m));
    m->dim = dim; m->hidden_dim = hidden_dim; m->n_layers = n_layers; m->n_q_heads = n_q_heads;
    m->n_kv_heads = n_kv_heads; m->vocab_size = vocab_size; m->seq_len = seq_len;
    m->rope_base_freq = rope_base_freq; m->rms_norm_eps = rms_norm_eps; m->rope_variant = rope_variant;
    size_t kv_dim = (size_t)dim * n_kv_heads / n_q_heads;
    m->layers = (wgo_llama2_layer *)calloc(n_layers, sizeof(wgo_llama2_layer));
    /* RunState::new -- cpu.rs:305-325 */
    m->x = (float *)calloc(dim, 4); m->xb = (float *)calloc(dim, 4); m->xb2 = (float *)calloc(dim, 4);
    m->hb = (float *)calloc(hidden_dim, 4); m->hb2 = (float *)calloc(hidden_dim, 4);
    m->q = (float *)calloc(dim, 4);
    m->att = (float *)calloc((size_t)seq_len * n_q_heads, 4);
    m->logits = (float *)calloc(vocab_size, 4);
    m->key_cache = (float *)calloc((size_t)n_layers * kv_dim * seq_len, 4);
    m->value_cache = (float *)calloc((size_t)n_layers * kv_dim * seq_len, 4);
    m->embd_row = (float *)calloc(dim, 4);
    return m;
}

WGO_API void wgo_llama2_free(wgo_llama2 *m)
{
    if (!m) return;
    free(m->layers); free(m->x); free(m->xb); free(m->xb2); free(m->hb); free(m->hb2); free(m->q);
    free(m->att); free(m->logits); free(m->key_cache); free(m->value_cache); free(m->embd_row);
    free(m);
}

/* layer < 0 selects the model-level matrices: which 0 = token_embd, 1 = output. */
WGO_API void wgo_llama2_set_matrix(wgo_llama2 *m, int layer, int which, int qtype, const void *data,
                                   size_t nrows, size_t ncols)
{
    wgo_mat mat = { qtype, data, nrows, ncols };
    if (layer < 0) { if (which == 0) m->token_embd = mat; else m->output = mat; }
    else m->layers[layer].m[which] = mat;
}

/* layer < 0: output_norm. */
WGO_API void wgo_llama2_set_vector(wgo_llama2 *m, int layer, int which, const float *data)
{
    if (layer < 0) m->output_norm = data; else m->layers[layer].v[which] = data;
}

WGO_API float *wgo_llama2_logits(wgo_llama2 *m) { return m->logits; }
WGO_API float *wgo_llama2_key_cache(wgo_llama2 *m) { return m->key_cache; }
WGO_API float *wgo_llama2_value_cache(wgo_llama2 *m) { return m->value_cache; }
WGO_API float *wgo_llama2_x(wgo_llama2 *m) { return m->x; }

static void mat_vec(const wgo_mat *w, const float *x, float *out)
{
    wgo_gemv_quant(w->qtype, w->data, w->nrows, w->ncols, x, out, NULL);
}

/* Column `row` of the dim x vocab embedding matrix (cpu.rs:244, :389) = the row-th run of
 * `dim` dequantised values of token_embd.weight. */
static void embedding_row(const wgo_mat *w, size_t row, float *out)
{
    int bb = wgo_block_bytes(w->qtype), bl = wgo_block_len(w->qtype);
    size_t bpr = w->ncols / (size_t)bl;
    const uint8_t *rb = (const uint8_t *)w->data + row * bpr * (size_t)bb;
    for (size_t k = 0; k < bpr; k++) deq_block(w->qtype, rb + k * (size_t)bb, out + k * (size_t)bl);
}

/* One iteration of the layer loop of Transformer::forward -- cpu.rs:392-434 -- on the running
 * activation `x`.  Exposed on its own so that the CPU baseline can time a bounded sample of a
 * model that is too slow to run whole. */
WGO_API void wgo_llama2_layer_forward(wgo_llama2 *m, uint32_t l, uint32_t pos)
{
    size_t dim = m->dim, hidden = m->hidden_dim;
    size_t kv_dim = dim * m->n_kv_heads / m->n_q_heads;
    uint32_t head_size = (uint32_t)(dim / m->n_q_heads);
    {
        wgo_llama2_layer *wl = &m->layers[l];
        float *kc_l = m->key_cache + (size_t)l * kv_dim * m->seq_len;
        float *vc_l = m->value_cache + (size_t)l * kv_dim * m->seq_len;
        float *k_cache = kc_l + (size_t)pos * kv_dim;
        float *v_cache = vc_l + (size_t)pos * kv_dim;
        wgo_rms_norm(m->xb, m->x, wl->v[WGO_ATTN_NORM], dim, m->rms_norm_eps);
        mat_vec(&wl->m[WGO_ATTN_Q], m->xb, m->q);
        mat_vec(&wl->m[WGO_ATTN_K], m->xb, k_cache);
        mat_vec(&wl->m[WGO_ATTN_V], m->xb, v_cache);
        /* transformer.rs:343-354 */
        if (wl->v[WGO_Q_BIAS]) for (size_t i = 0; i < dim; i++) m->q[i] += wl->v[WGO_Q_BIAS][i];
        if (wl->v[WGO_K_BIAS]) for (size_t i = 0; i < kv_dim; i++) k_cache[i] += wl->v[WGO_K_BIAS][i];
        if (wl->v[WGO_V_BIAS]) for (size_t i = 0; i < kv_dim; i++) v_cache[i] += wl->v[WGO_V_BIAS][i];
        wgo_rope(m->rope_variant, m->q, dim, k_cache, head_size, (uint32_t)kv_dim, pos, m->rope_base_freq);
        wgo_attn_params ap = { m->seq_len, (uint32_t)kv_dim, m->n_q_heads / m->n_kv_heads,
                               m->n_q_heads, head_size, pos };
        wgo_attention(&ap, m->q, kc_l, vc_l, m->att, m->xb);
        mat_vec(&wl->m[WGO_ATTN_OUT], m->xb, m->xb2);
        for (size_t i = 0; i < dim; i++) m->x[i] += m->xb2[i];
        wgo_rms_norm(m->xb, m->x, wl->v[WGO_FFN_NORM], dim, m->rms_norm_eps);
        /* ffn_silu -- cpu.rs:543-562 */
        mat_vec(&wl->m[WGO_FFN_GATE], m->xb, m->hb);
        mat_vec(&wl->m[WGO_FFN_UP], m->xb, m->hb2);
        wgo_silu(m->hb, m->hb2, hidden);
        mat_vec(&wl->m[WGO_FFN_DOWN], m->hb, m->xb2);
        for (size_t i = 0; i < dim; i++) m->x[i] += m->xb2[i];
    }
}

/* Final norm and classifier -- cpu.rs:436-443. */
WGO_API void wgo_llama2_head_forward(wgo_llama2 *m)
{
    wgo_rms_norm(m->xb, m->x, m->output_norm, m->dim, m->rms_norm_eps);
    mat_vec(&m->output, m->xb, m->logits);
}

/* Transformer::forward -- cpu.rs:377-444 */
WGO_API void wgo_llama2_forward(wgo_llama2 *m, uint32_t token, uint32_t pos)
{
    embedding_row(&m->token_embd, token, m->x);
    for (uint32_t l = 0; l < m->n_layers; l++) wgo_llama2_layer_forward(m, l, pos);
    wgo_llama2_head_forward(m);
}

/* The token loop of crates/wgml-chat/src/chat_llama2.rs:102-121 with the forced-token rule of
 * crates/wgml-chat/src/sampler.rs:102-107 and greedy sampling (models/sampler.rs:33-35 with
 * temperature 0).  Writes the n_prompt-1 forced tokens followed by n_gen sampled ones, i.e.
 * `out_tokens[i]` is the token fed at position start_pos + i + 1. */
WGO_API void wgo_llama2_decode(wgo_llama2 *m, const uint32_t *prompt, size_t n_prompt, size_t n_gen,
                               uint32_t start_pos, uint32_t *out_tokens, float *top2_margin)
{
    uint32_t token = prompt[0];
    size_t total = n_prompt - 1 + n_gen;
    for (size_t i = 0; i < total; i++) {
        wgo_llama2_forward(m, token, start_pos + (uint32_t)i);
        uint32_t next;
        if (i + 1 < n_prompt) {
            next = prompt[i + 1];
            if (top2_margin) top2_margin[i] = 0.0f;
        } else {
            next = (uint32_t)wgo_argmax(m->logits, m->vocab_size);
            if (top2_margin) {
                float second = -INFINITY;
                for (size_t j = 0; j < m->vocab_size; j++)
                    if (j != next && m->logits[j] > second) second = m->logits[j];
                top2_margin[i] = m->logits[next] - second;
            }
        }
        out_tokens[i] = next;
        token = next;
    }
}

/* ------------------------------------------------------------------------------------------
 * GPT-2 CPU transformer -- crates/wgml/src/models/gpt2/cpu.rs:224-381.
 * ---------------------------------------------------------------------------------------- */
enum { WGO_G_ATTN_QKV, WGO_G_ATTN_PROJ, WGO_G_FC, WGO_G_PROJ, WGO_G_N_MATS };
enum { WGO_G_LN1_G, WGO_G_LN1_B, WGO_G_LN2_G, WGO_G_LN2_B, WGO_G_ATTN_QKV_B, WGO_G_ATTN_PROJ_B,
       WGO_G_FC_B, WGO_G_PROJ_B, WGO_G_N_VECS };

typedef struct {
    wgo_mat m[WGO_G_N_MATS];
    const float *v[WGO_G_N_VECS];
} wgo_gpt2_layer;

typedef struct {
    uint32_t n_vocab, n_seq, n_embd, n_head, n_layer, ff_len;
    wgo_gpt2_layer *layers;
    wgo_mat wte, wpe; /* lm_head = wte transposed (cpu.rs:195-196): logits[r] = wte row r . x */
    const float *ln_f_g, *ln_f_b;
    float *memory_q, *memory_att, *layer_input, *curr_768, *curr_768_b, *curr_2304, *curr_3072,
        *curr_vocab, *key_cache, *value_cache, *tmp;
} wgo_gpt2;

WGO_API wgo_gpt2 *wgo_gpt2_new(uint32_t n_vocab, uint32_t n_seq, uint32_t n_embd, uint32_t n_head,
                               uint32_t n_layer, uint32_t ff_len)
{
    wgo_gpt2 *m = (wgo_gpt2 *)calloc(1, sizeof(*m));
    m->n_vocab = n_vocab; m->n_seq = n_seq; m->n_embd = n_embd; m->n_head = n_head;
    m->n_layer = n_layer; m->ff_len = ff_len;
    m->layers = (wgo_gpt2_layer *)calloc(n_layer, sizeof(wgo_gpt2_layer));
    m->memory_q = (float *)calloc(n_embd, 4);
    m->memory_att = (float *)calloc((size_t)n_seq * n_head, 4);
    m->layer_input = (float *)calloc(n_embd, 4);
    m->curr_768 = (float *)calloc(n_embd, 4);
    m->curr_768_b = (float *)calloc(n_embd, 4);
    m->curr_2304 = (float *)calloc(3 * (size_t)n_embd, 4);
    m->curr_3072 = (float *)calloc(ff_len, 4);
    m->curr_vocab = (float *)calloc(n_vocab, 4);
    m->key_cache = (float *)calloc((size_t)n_layer * n_embd * n_seq, 4);
    m->value_cache = (float *)calloc((size_t)n_layer * n_embd * n_seq, 4);
    m->tmp = (float *)calloc(n_embd, 4);
    return m;
}

WGO_API void wgo_gpt2_free(wgo_gpt2 *m)
{
    if (!m) return;
    free(m->layers); free(m->memory_q); free(m->memory_att); free(m->layer_input); free(m->curr_768);
    free(m->curr_768_b); free(m->curr_2304); free(m->curr_3072); free(m->curr_vocab);
    free(m->key_cache); free(m->value_cache); free(m->tmp);
    free(m);
}

/* layer < 0: which 0 = wte (token_embd), 1 = wpe (position_embd). */
WGO_API void wgo_gpt2_set_matrix(wgo_gpt2 *m, int layer, int which, int qtype, const void *data,
                                 size_t nrows, size_t ncols)
{
    wgo_mat mat = { qtype, data, nrows, ncols };
    if (layer < 0) { if (which == 0) m->wte = mat; else m->wpe = mat; }
    else m->layers[layer].m[which] = mat;
}

/* layer < 0: which 0 = ln_f_g, 1 = ln_f_b. */
WGO_API void wgo_gpt2_set_vector(wgo_gpt2 *m, int layer, int which, const float *data)
{
    if (layer < 0) { if (which == 0) m->ln_f_g = data; else m->ln_f_b = data; }
    else m->layers[layer].v[which] = data;
}

WGO_API float *wgo_gpt2_logits(wgo_gpt2 *m) { return m->curr_vocab; }
WGO_API float *wgo_gpt2_key_cache(wgo_gpt2 *m) { return m->key_cache; }
WGO_API float *wgo_gpt2_value_cache(wgo_gpt2 *m) { return m->value_cache; }

WGO_API void wgo_gpt2_forward(wgo_gpt2 *m, uint32_t embd, uint32_t pos)
{
    size_t n = m->n_embd;
    /* cpu.rs:226-227 */
    embedding_row(&m->wte, embd, m->layer_input);
    embedding_row(&m->wpe, pos, m->tmp);
    for (size_t i = 0; i < n; i++) m->layer_input[i] += m->tmp[i];
    for (uint32_t l = 0; l < m->n_layer; l++) {
        wgo_gpt2_layer *w = &m->layers[l];
        float *kc_l = m->key_cache + (size_t)l * n * m->n_seq;
        float *vc_l = m->value_cache + (size_t)l * n * m->n_seq;
        /* cpu.rs:231-240 */
        wgo_layernorm(m->curr_768, m->layer_input, n);
        for (size_t i = 0; i < n; i++) m->curr_768[i] *= w->v[WGO_G_LN1_G][i];
        for (size_t i = 0; i < n; i++) m->curr_768[i] += w->v[WGO_G_LN1_B][i];
        /* cpu.rs:250-255 */
        mat_vec(&w->m[WGO_G_ATTN_QKV], m->curr_768, m->curr_2304);
        for (size_t i = 0; i < 3 * n; i++) m->curr_2304[i] += w->v[WGO_G_ATTN_QKV_B][i];
        /* cpu.rs:260-289 */
        memcpy(m->memory_q, m->curr_2304, n * 4);
        memcpy(kc_l + (size_t)pos * n, m->curr_2304 + n, n * 4);
        memcpy(vc_l + (size_t)pos * n, m->curr_2304 + 2 * n, n * 4);
        wgo_attn_params ap = { m->n_seq, (uint32_t)n, 1, m->n_head, (uint32_t)(n / m->n_head), pos };
        wgo_attention(&ap, m->memory_q, kc_l, vc_l, m->memory_att, m->curr_768);
        /* cpu.rs:299-310 */
        mat_vec(&w->m[WGO_G_ATTN_PROJ], m->curr_768, m->curr_768_b);
        for (size_t i = 0; i < n; i++) m->curr_768_b[i] += w->v[WGO_G_ATTN_PROJ_B][i];
        for (size_t i = 0; i < n; i++) m->curr_768_b[i] += m->layer_input[i];
        memcpy(m->layer_input, m->curr_768_b, n * 4);
        /* cpu.rs:313-355 */
        wgo_layernorm(m->curr_768, m->curr_768_b, n);
        for (size_t i = 0; i < n; i++) m->curr_768[i] *= w->v[WGO_G_LN2_G][i];
        for (size_t i = 0; i < n; i++) m->curr_768[i] += w->v[WGO_G_LN2_B][i];
        mat_vec(&w->m[WGO_G_FC], m->curr_768, m->curr_3072);
        for (size_t i = 0; i < m->ff_len; i++) m->curr_3072[i] += w->v[WGO_G_FC_B][i];
        wgo_unary_vec(5, m->curr_3072, m->ff_len, NULL);
        mat_vec(&w->m[WGO_G_PROJ], m->curr_3072, m->curr_768);
        for (size_t i = 0; i < n; i++) m->curr_768[i] += w->v[WGO_G_PROJ_B][i];
        /* cpu.rs:358 */
        for (size_t i = 0; i < n; i++) m->layer_input[i] += m->curr_768[i];
    }
    /* cpu.rs:362-377 */
    wgo_layernorm(m->curr_768, m->layer_input, n);
    for (size_t i = 0; i < n; i++) m->curr_768[i] *= m->ln_f_g[i];
    for (size_t i = 0; i < n; i++) m->curr_768[i] += m->ln_f_b[i];
    mat_vec(&m->wte, m->curr_768, m->curr_vocab);
}

/* Token loop of crates/wgml-chat/src/chat_gpt2.rs:43-151, forced prompt tokens then greedy. */
WGO_API void wgo_gpt2_decode(wgo_gpt2 *m, const uint32_t *prompt, size_t n_prompt, size_t n_gen,
                             uint32_t start_pos, uint32_t *out_tokens)
{
    uint32_t token = prompt[0];
    size_t total = n_prompt - 1 + n_gen;
    for (size_t i = 0; i < total; i++) {
        wgo_gpt2_forward(m, token, start_pos + (uint32_t)i);
        uint32_t next = (i + 1 < n_prompt) ? prompt[i + 1] : (uint32_t)wgo_argmax(m->curr_vocab, m->n_vocab);
        out_tokens[i] = next;
        token = next;
    }
}

WGO_API int wgo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

WGO_API void wgo_set_num_threads(int n)
{
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
