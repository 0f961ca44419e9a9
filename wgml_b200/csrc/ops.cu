// Stand-alone operators of wgml's surface (norms, RoPE, softmax, SiLU, unary, op-assign, argmax)
// plus the small device-resident helpers of the token loop (embedding gather, greedy step).
#include "qaccess.cuh"
#include "kernels.h"

#include <cmath>
#include <vector>

namespace wgb {

constexpr int OPS_NT = 256;

static inline int ew_grid(size_t n)
{
    size_t g = (n + OPS_NT - 1) / OPS_NT;
    size_t cap = (size_t)sm_count() * 8;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// RmsNorm (ops/rms_norm.wgsl:36-67): a single block, like the reference's single workgroup.
__global__ void __launch_bounds__(1024) rms_norm_kernel(float *__restrict__ out, const float *__restrict__ v,
                                                        const float *__restrict__ w, uint32_t n, float eps)
{
    __shared__ float red[32];
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += 1024) ss = fmaf(v[i], v[i], ss);
    ss = block_sum<1024>(ss, red);
    const float rms = 1.0f / sqrtf(ss / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += 1024) out[i] = (v[i] * rms) * w[i];
}

// LayerNorm (ops/layernorm.wgsl:28-80): two passes, epsilon 1e-5, no affine part.
__global__ void __launch_bounds__(1024) layernorm_kernel(float *__restrict__ out, const float *__restrict__ v, uint32_t n)
{
    __shared__ float red[32];
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += 1024) s += v[i];
    const float mean = block_sum<1024>(s, red) / (float)n;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += 1024) {
        const float d = v[i] - mean;
        ss = fmaf(d, d, ss);
    }
    ss = block_sum<1024>(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)n + 1.0e-5f);
    for (uint32_t i = threadIdx.x; i < n; i += 1024) out[i] = (v[i] - mean) * scale;
}

// Inverse frequencies of RoPE passed by value (head sizes up to 512).
struct RopeFreq { float f[256]; };

// RoPE (ops/rope.wgsl:36-77) with the bounds checks WebGPU's robust access provides implicitly.
__global__ void rope_kernel(int variant, wgb_rope_config cfg, const __grid_constant__ RopeFreq fr, float *__restrict__ q,
                            uint32_t q_len, float *__restrict__ k, uint32_t k_len)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;  // pair index
    if (2 * i >= q_len) return;
    const uint32_t half = cfg.head_size / 2;
    const float ang = (float)cfg.pos * fr.f[i % half];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    uint32_t ia, ib;
    if (variant == WGB_ROPE_ORIGINAL) {
        ia = 2 * i;
        ib = ia + 1;
    } else {
        const uint32_t head = (2 * i) / cfg.head_size;
        ia = i + head * half;
        ib = ia + half;
    }
    if (ib < q_len) {
        const float x = q[ia], y = q[ib];
        q[ia] = cs * x - sn * y;
        q[ib] = sn * x + cs * y;
    }
    if (2 * i < cfg.kv_dim && ib < k_len) {
        const float x = k[ia], y = k[ib];
        k[ia] = cs * x - sn * y;
        k[ib] = sn * x + cs * y;
    }
}

// SoftMax (ops/softmax.wgsl:31-92): one block per column.
__global__ void __launch_bounds__(OPS_NT) softmax_kernel(float *__restrict__ mat, uint32_t nrows, size_t col_stride)
{
    __shared__ float red[32];
    float *col = mat + (size_t)blockIdx.x * col_stride;
    float m = -INFINITY;
    for (uint32_t i = threadIdx.x; i < nrows; i += OPS_NT) m = fmaxf(m, col[i]);
    m = block_max<OPS_NT>(m, red);
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < nrows; i += OPS_NT) {
        const float e = expf(col[i] - m);
        col[i] = e;
        s += e;
    }
    s = block_sum<OPS_NT>(s, red);
    for (uint32_t i = threadIdx.x; i < nrows; i += OPS_NT) col[i] = col[i] / s;
}

// Silu (ops/silu.wgsl:13-27)
__global__ void silu_kernel(float *__restrict__ h1, const float *__restrict__ h2, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float x = h1[i];
        h1[i] = h2[i] * (x / (1.0f + expf(-1.0f * x)));
    }
}

// UnaryOp::eval (ops/unary.rs:87-129) -- the CPU twin's definitions (signum(0) = 1, accurate tanh).
__device__ __forceinline__ float unary_eval(int op, float x, float a0, float a1)
{
    switch (op) {
    case WGB_UNARY_ABS: return fabsf(x);
    case WGB_UNARY_SGN: return isnan(x) ? x : copysignf(1.0f, x);
    case WGB_UNARY_NEG: return -x;
    case WGB_UNARY_STEP: return x > 0.0f ? 1.0f : 0.0f;
    case WGB_UNARY_ELU: return x > 0.0f ? x : expf(x) - 1.0f;
    case WGB_UNARY_GELU: {
        const float GELU_COEF_A = 0.044715f, SQRT_2_OVER_PI = 0.7978846f;
        return 0.5f * x * (1.0f + tanhf(SQRT_2_OVER_PI * x * (1.0f + GELU_COEF_A * x * x)));
    }
    case WGB_UNARY_GELU_QUICK: return x * (1.0f / (1.0f + expf(-1.702f * x)));
    case WGB_UNARY_SILU: return x / (1.0f + expf(-x));
    case WGB_UNARY_TANH: return tanhf(x);
    case WGB_UNARY_RELU: return fmaxf(x, 0.0f);
    case WGB_UNARY_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case WGB_UNARY_HARD_SIGMOID: return fminf(1.0f, fmaxf(0.0f, (x + 3.0f) / 6.0f));
    case WGB_UNARY_HARD_SWISH: return x * fminf(1.0f, fmaxf(0.0f, (x + 3.0f) / 6.0f));
    case WGB_UNARY_SQR: return x * x;
    case WGB_UNARY_SQRT: return sqrtf(x);
    case WGB_UNARY_LOG: return logf(x);
    case WGB_UNARY_LEAKY_RELU: return fmaxf(x, 0.0f) + fminf(x, 0.0f) * a0;
    case WGB_UNARY_CLAMP: { const float t = x < a0 ? a0 : x; return t > a1 ? a1 : t; }
    case WGB_UNARY_SCALE: return x * a0;
    case WGB_UNARY_ADD_SCALAR: return x + a0;
    default: return x;
    }
}

__global__ void unary_kernel(int op, float *__restrict__ dst, const float *__restrict__ src, size_t n, float a0, float a1)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = unary_eval(op, src[i], a0, a1);
}

__global__ void op_assign_kernel(int kind, float *__restrict__ lhs, const float *__restrict__ rhs, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float r = rhs[i];
        lhs[i] = kind == WGB_ASSIGN_ADD ? lhs[i] + r : (kind == WGB_ASSIGN_MUL ? lhs[i] * r : r);
    }
}

// ---- argmax: first maximum, two stages ------------------------------------------------------
// Key = (value mapped to a monotone unsigned, ~index): the larger key wins, ties go to the lower index.
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t i)
{
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    if (isnan(v)) b = 0;  // NaN never wins (nalgebra's `>` comparison)
    return ((unsigned long long)b << 32) | (uint32_t)(~i);
}

constexpr int ARGMAX_BLOCKS = 64;

__global__ void __launch_bounds__(OPS_NT) argmax_partial_kernel(const float *__restrict__ v, uint32_t n,
                                                                unsigned long long *__restrict__ part)
{
    __shared__ unsigned long long red[OPS_NT / 32];
    pdl_launch_dependents();
    pdl_wait();
    unsigned long long best = 0;
    for (uint32_t i = blockIdx.x * OPS_NT + threadIdx.x; i < n; i += gridDim.x * OPS_NT) {
        const unsigned long long k = argmax_key(__ldcg(v + i), i);
        best = k > best ? k : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < OPS_NT / 32; w++) best = red[w] > best ? red[w] : best;
        part[blockIdx.x] = best;
    }
}

// Final stage.  With a loop state: the greedy step of the token loop (forced prompt tokens as
// crates/wgml-chat/src/sampler.rs:102-107); otherwise the index goes to *out_index.
__global__ void argmax_final_kernel(const unsigned long long *__restrict__ part, int nparts, uint32_t *out_index,
                                    LoopState ls, int have_loop)
{
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0) return;
    unsigned long long best = 0;
    for (int i = 0; i < nparts; i++) {
        const unsigned long long k = __ldcg(part + i);
        best = k > best ? k : best;
    }
    const uint32_t arg = ~(uint32_t)(best & 0xffffffffu);
    if (!have_loop) {
        *out_index = arg;
        return;
    }
    const uint32_t step = *ls.step;
    const uint32_t next = (step + 1 < ls.n_prompt) ? ls.prompt[step + 1] : arg;
    ls.out_tokens[step] = next;
    *ls.token = next;
    *ls.pos = *ls.pos + 1;
    *ls.step = step + 1;
}

// x = embedding row *d_token (+ position row *d_pos), dequantised exactly.
__global__ void embed_kernel(const __grid_constant__ QMat embd, const __grid_constant__ QMat pos_embd, int have_pos,
                             const uint32_t *__restrict__ d_token, const uint32_t *__restrict__ d_pos, float *__restrict__ x)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tok = *d_token;
    const uint32_t pos = have_pos ? *d_pos : 0;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < embd.ncols; c += gridDim.x * blockDim.x) {
        float v = tok < embd.nrows ? qmat_weight_any(embd, tok, c) : 0.0f;
        if (have_pos && pos < pos_embd.nrows) v += qmat_weight_any(pos_embd, pos, c);
        x[c] = v;
    }
}

int launch_embed(const QMat &embd, const QMat *pos_embd, const uint32_t *d_token, const uint32_t *d_pos, float *x,
                 cudaStream_t stream)
{
    QMat pe = pos_embd ? *pos_embd : embd;
    const int grid = (int)((embd.ncols + 127) / 128);
    embed_kernel<<<grid, 128, 0, stream>>>(embd, pe, pos_embd ? 1 : 0, d_token, d_pos, x);
    WGB_LAUNCH_CHECK("embed_kernel");
    return WGB_OK;
}

// scratch: ARGMAX_BLOCKS 64-bit words
int launch_argmax_advance(const float *logits, uint32_t n, const LoopState &ls, uint32_t *scratch, cudaStream_t stream)
{
    unsigned long long *part = reinterpret_cast<unsigned long long *>(scratch);
    argmax_partial_kernel<<<ARGMAX_BLOCKS, OPS_NT, 0, stream>>>(logits, n, part);
    WGB_LAUNCH_CHECK("argmax_partial_kernel");
    argmax_final_kernel<<<1, 32, 0, stream>>>(part, ARGMAX_BLOCKS, nullptr, ls, 1);
    WGB_LAUNCH_CHECK("argmax_final_kernel");
    return WGB_OK;
}

}  // namespace wgb

using namespace wgb;

WGB_EXPORT int wgb_rms_norm(float *d_out, const float *d_v, const float *d_w, size_t n, float eps, void *stream)
{
    WGB_REQUIRE(d_out && d_v && d_w && n > 0, "null or empty argument");
    rms_norm_kernel<<<1, 1024, 0, as_stream(stream)>>>(d_out, d_v, d_w, (uint32_t)n, eps);
    WGB_LAUNCH_CHECK("rms_norm_kernel");
    return WGB_OK;
}

WGB_EXPORT int wgb_layernorm(float *d_out, const float *d_in, size_t n, void *stream)
{
    WGB_REQUIRE(d_out && d_in && n > 0, "null or empty argument");
    layernorm_kernel<<<1, 1024, 0, as_stream(stream)>>>(d_out, d_in, (uint32_t)n);
    WGB_LAUNCH_CHECK("layernorm_kernel");
    return WGB_OK;
}

namespace wgb {
// base^(-(2j)/head_size), evaluated on the host exactly as the CPU reference does
// (`10000.0_f32.powf(-head_dim / head_size as f32)`, ops/rope.rs:97): the device `powf` may differ
// in the last bit, which the position multiplies.
void rope_inv_freq(uint32_t head_size, float base, float *out)
{
    for (uint32_t j = 0; j < head_size / 2; j++) out[j] = powf(base, -(float)(2 * j) / (float)head_size);
}
}  // namespace wgb

WGB_EXPORT int wgb_rope(int variant, const wgb_rope_config *cfg, float *d_q, size_t q_len, float *d_k, size_t k_len,
                        void *stream)
{
    WGB_REQUIRE(cfg && d_q && d_k, "null argument");
    WGB_REQUIRE(variant == WGB_ROPE_ORIGINAL || variant == WGB_ROPE_NEOX, "unknown RoPE variant %d", variant);
    // ops/rope.rs:51-56
    WGB_REQUIRE(q_len % 2 == 0 && k_len % 2 == 0, "RoPE: vector lengths must be even");
    WGB_REQUIRE(q_len >= k_len, "The Query vector must be larger than, or as large as, the Key vector.");
    WGB_REQUIRE(cfg->head_size >= 2 && cfg->head_size % 2 == 0 && cfg->head_size <= 512, "RoPE: head_size %u unsupported", cfg->head_size);
    if (q_len == 0) return WGB_OK;
    RopeFreq fr;
    rope_inv_freq(cfg->head_size, cfg->base_freq, fr.f);
    const uint32_t pairs = (uint32_t)(q_len / 2);
    rope_kernel<<<(pairs + 63) / 64, 64, 0, as_stream(stream)>>>(variant, *cfg, fr, d_q, (uint32_t)q_len, d_k, (uint32_t)k_len);
    WGB_LAUNCH_CHECK("rope_kernel");
    return WGB_OK;
}

WGB_EXPORT int wgb_softmax(float *d_mat, size_t nrows, size_t ncols, size_t col_stride, void *stream)
{
    WGB_REQUIRE(d_mat && col_stride >= nrows, "bad softmax arguments");
    if (nrows == 0 || ncols == 0) return WGB_OK;
    softmax_kernel<<<(unsigned)ncols, OPS_NT, 0, as_stream(stream)>>>(d_mat, (uint32_t)nrows, col_stride);
    WGB_LAUNCH_CHECK("softmax_kernel");
    return WGB_OK;
}

WGB_EXPORT int wgb_silu(float *d_h1, const float *d_h2, size_t n, void *stream)
{
    WGB_REQUIRE(d_h1 && d_h2, "null argument");
    if (n == 0) return WGB_OK;
    silu_kernel<<<ew_grid(n), OPS_NT, 0, as_stream(stream)>>>(d_h1, d_h2, n);
    WGB_LAUNCH_CHECK("silu_kernel");
    return WGB_OK;
}

static int unary_impl(int op, float *dst, const float *src, size_t n, const float *args4, void *stream)
{
    WGB_REQUIRE(dst && src, "null argument");
    WGB_REQUIRE(op >= WGB_UNARY_ABS && op <= WGB_UNARY_ADD_SCALAR, "unknown unary op %d", op);
    const bool has_args = op >= WGB_UNARY_LEAKY_RELU;
    WGB_REQUIRE(has_args == (args4 != nullptr), "Unary ops argument mismatch.");  // ops/unary.rs:172-175
    if (n == 0) return WGB_OK;
    unary_kernel<<<ew_grid(n), OPS_NT, 0, as_stream(stream)>>>(op, dst, src, n, args4 ? args4[0] : 0.0f, args4 ? args4[1] : 0.0f);
    WGB_LAUNCH_CHECK("unary_kernel");
    return WGB_OK;
}

WGB_EXPORT int wgb_unary(int op, float *d_dst, const float *d_src, size_t n, const float *args4, void *stream)
{
    return unary_impl(op, d_dst, d_src, n, args4, stream);
}

WGB_EXPORT int wgb_unary_inplace(int op, float *d_src, size_t n, const float *args4, void *stream)
{
    return unary_impl(op, d_src, d_src, n, args4, stream);
}

WGB_EXPORT int wgb_op_assign(int kind, float *d_lhs, const float *d_rhs, size_t n, void *stream)
{
    WGB_REQUIRE(d_lhs && d_rhs, "null argument");
    WGB_REQUIRE(kind >= WGB_ASSIGN_ADD && kind <= WGB_ASSIGN_COPY, "unknown assign kind %d", kind);
    if (n == 0) return WGB_OK;
    op_assign_kernel<<<ew_grid(n), OPS_NT, 0, as_stream(stream)>>>(kind, d_lhs, d_rhs, n);
    WGB_LAUNCH_CHECK("op_assign_kernel");
    return WGB_OK;
}

WGB_EXPORT int wgb_argmax(const float *d_v, size_t n, uint32_t *d_index, void *stream)
{
    WGB_REQUIRE(d_v && d_index && n > 0 && n <= 0xffffffffull, "bad argmax arguments");
    // partial keys: allocated once per device
    DeviceState *ds = device_state();
    if (!ds) return WGB_ERR_CUDA;
    if (!ds->argmax_part) WGB_CUDA(cudaMalloc((void **)&ds->argmax_part, ARGMAX_BLOCKS * sizeof(unsigned long long)));
    unsigned long long *g_argmax_part = ds->argmax_part;
    argmax_partial_kernel<<<ARGMAX_BLOCKS, OPS_NT, 0, as_stream(stream)>>>(d_v, (uint32_t)n, g_argmax_part);
    WGB_LAUNCH_CHECK("argmax_partial_kernel");
    LoopState none = {};
    argmax_final_kernel<<<1, 32, 0, as_stream(stream)>>>(g_argmax_part, ARGMAX_BLOCKS, d_index, none, 0);
    WGB_LAUNCH_CHECK("argmax_final_kernel");
    return WGB_OK;
}
