// Matrix-vector kernels: the fused kernel used by the models and by GemvQuant, and the generic
// per-format fallback.
//
// Grid: one persistent block of 8 warps per SM.  Work is split into groups of R rows; group
// `g` belongs to warp (g / gridDim.x) % 8 of block g % gridDim.x, so every SM ends up with the
// same number of groups to within one.  Each warp preloads the first step of its first group
// before waiting for the preceding kernel (programmatic dependent launch): weights never depend
// on activations, so their HBM reads overlap the predecessor's tail.
#include "gemv_core.cuh"
#include "kernels.h"

namespace wgb {

constexpr int GEMV_NT = 256;
constexpr int GEMV_WARPS = GEMV_NT / 32;

__device__ __forceinline__ float4 ld_act4(const float *p)
{
    return __ldcg(reinterpret_cast<const float4 *>(p));
}

// Rows (and their matrices) of group gi.  Returns false when the whole group is out of range;
// rows past the end of a matrix are clamped (computed, never stored) and flagged in `valid`.
template <int EPI, int R>
__device__ __forceinline__ bool group_rows(const GemvArgs &a, uint32_t gi, const QMat *(&mats)[R],
                                           uint32_t (&rows)[R], bool (&valid)[R])
{
    if (EPI == EPI_SILU_PAIR) {
        constexpr int P = R / 2;
        const uint32_t n = a.mat[0].nrows;
        if (gi * P >= n) return false;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t row = gi * P + (r % P);
            mats[r] = &a.mat[r / P];
            valid[r] = row < n;
            rows[r] = valid[r] ? row : n - 1;
        }
        return true;
    } else if (EPI == EPI_QKV_ROPE) {
        constexpr int P = R / 2;
        const uint32_t qp = a.mat[0].nrows / 2, kp = a.mat[1].nrows / 2, vp = a.mat[2].nrows / 2;
        if (gi * P >= qp + kp + vp) return false;
        const uint32_t half = a.head_size / 2;
#pragma unroll
        for (int j = 0; j < P; j++) {
            uint32_t p = gi * P + j;
            const bool ok = p < qp + kp + vp;
            if (!ok) p = qp + kp + vp - 1;
            int s = p < qp ? 0 : (p < qp + kp ? 1 : 2);
            const uint32_t lp = p - (s == 0 ? 0 : (s == 1 ? qp : qp + kp));
            uint32_t r0, r1;
            if (s < 2 && a.rope_variant == WGB_ROPE_NEOX) {
                const uint32_t h = lp / half, jj = lp % half;
                r0 = h * a.head_size + jj;
                r1 = r0 + half;
            } else {
                r0 = 2 * lp;
                r1 = r0 + 1;
            }
            mats[2 * j] = mats[2 * j + 1] = &a.mat[s];
            rows[2 * j] = r0;
            rows[2 * j + 1] = r1;
            valid[2 * j] = valid[2 * j + 1] = ok;
        }
        return true;
    } else {
        const uint32_t n = a.mat[0].nrows;
        if (gi * R >= n) return false;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t row = gi * R + r;
            mats[r] = &a.mat[0];
            valid[r] = row < n;
            rows[r] = valid[r] ? row : n - 1;
        }
        return true;
    }
}

template <int R>
__device__ __forceinline__ float pick(const float (&acc)[R], int i)
{
    float v = acc[0];
#pragma unroll
    for (int r = 1; r < R; r++) v = (i == r) ? acc[r] : v;
    return v;
}

__device__ __forceinline__ float gelu_f32(float x)
{
    // UnaryOp::Gelu, crates/wgml/src/ops/unary.rs:106-110
    const float GELU_COEF_A = 0.044715f, SQRT_2_OVER_PI = 0.7978846f;
    return 0.5f * x * (1.0f + tanhf(SQRT_2_OVER_PI * x * (1.0f + GELU_COEF_A * x * x)));
}

template <int EPI, int R>
__device__ __forceinline__ void epilogue(const GemvArgs &a, const QMat *const (&mats)[R], const uint32_t (&rows)[R],
                                         const bool (&valid)[R], const float (&acc)[R], int lane)
{
    if (EPI == EPI_STORE || EPI == EPI_RESIDUAL || EPI == EPI_GELU) {
        if (lane < R) {
            bool ok = valid[0];
            uint32_t row = rows[0];
#pragma unroll
            for (int r = 1; r < R; r++) { ok = (lane == r) ? valid[r] : ok; row = (lane == r) ? rows[r] : row; }
            if (ok) {
                float y = pick<R>(acc, lane);
                if (a.bias) y += a.bias[row];
                if (EPI == EPI_RESIDUAL) y = a.residual[row] + y;
                if (EPI == EPI_GELU) y = gelu_f32(y);
                a.out[row] = y;
            }
        }
    } else if (EPI == EPI_SILU_PAIR) {
        constexpr int P = R / 2;
        if (lane < P) {
            bool ok = valid[0];
            uint32_t row = rows[0];
#pragma unroll
            for (int r = 1; r < P; r++) { ok = (lane == r) ? valid[r] : ok; row = (lane == r) ? rows[r] : row; }
            if (ok) {
                const float g = pick<R>(acc, lane), u = pick<R>(acc, lane + P);
                a.out[row] = u * (g / (1.0f + expf(-g)));
            }
        }
    } else if (EPI == EPI_QKV_ROPE) {
        constexpr int P = R / 2;
        if (lane < P) {
            bool ok = valid[0];
            uint32_t r0 = rows[0], r1 = rows[1];
            const QMat *m = mats[0];
#pragma unroll
            for (int j = 1; j < P; j++) {
                const bool sel = lane == j;
                ok = sel ? valid[2 * j] : ok;
                r0 = sel ? rows[2 * j] : r0;
                r1 = sel ? rows[2 * j + 1] : r1;
                m = sel ? mats[2 * j] : m;
            }
            if (ok) {
                float y0 = pick<R>(acc, 2 * lane), y1 = pick<R>(acc, 2 * lane + 1);
                const int s = (m == &a.mat[0]) ? 0 : ((m == &a.mat[1]) ? 1 : 2);
                const float *bias = s == 0 ? a.bias : (s == 1 ? a.bias_k : a.bias_v);
                if (bias) { y0 += bias[r0]; y1 += bias[r1]; }
                const uint32_t pos = *a.pos;
                if (s < 2) {
                    // RoPE (ops/rope.wgsl:36-77): angle = pos * base^(-(2i % head_size) / head_size)
                    const uint32_t half = a.head_size / 2;
                    const uint32_t fi = (a.rope_variant == WGB_ROPE_NEOX) ? (r0 % a.head_size) : ((r0 / 2) % half);
                    const float ang = (float)pos * a.rope_freq[fi];
                    float sn, cs;
                    sincosf(ang, &sn, &cs);
                    const float t0 = cs * y0 - sn * y1, t1 = sn * y0 + cs * y1;
                    y0 = t0;
                    y1 = t1;
                }
                float *dst = s == 0 ? a.out : ((s == 1 ? a.k_cache : a.v_cache) + (size_t)pos * a.kv_dim);
                dst[r0] = y0;
                dst[r1] = y1;
            }
        }
    } else if (EPI == EPI_QKV_SPLIT) {
        if (lane < R) {
            bool ok = valid[0];
            uint32_t row = rows[0];
#pragma unroll
            for (int r = 1; r < R; r++) { ok = (lane == r) ? valid[r] : ok; row = (lane == r) ? rows[r] : row; }
            if (ok) {
                float y = pick<R>(acc, lane);
                if (a.bias) y += a.bias[row];
                const uint32_t n = a.kv_dim, pos = *a.pos;
                if (row < n) a.out[row] = y;
                else if (row < 2 * n) a.k_cache[(size_t)pos * n + (row - n)] = y;
                else a.v_cache[(size_t)pos * n + (row - 2 * n)] = y;
            }
        }
    }
}

template <int QT, int R, int PRO, int EPI>
__global__ void __launch_bounds__(GEMV_NT) gemv_kernel(const __grid_constant__ GemvArgs a)
{
    using S = Step<QT>;
    extern __shared__ float4 smem4[];
    const uint32_t K = a.mat[0].ncols;
    float *xs = reinterpret_cast<float *>(smem4);
    float *xsum = xs + K;
    float *red = xsum + ((K / 16 + 3) & ~3u);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    uint32_t gi = warp * gridDim.x + blockIdx.x;
    const QMat *mats[R];
    uint32_t rows[R];
    bool valid[R];
    bool have = group_rows<EPI, R>(a, gi, mats, rows, valid);

    // First step of the first group: issued before the dependency wait.
    typename S::Raw cur[R];
    bool cur_act = have && S::active(a.mat[0], 0, lane);
    if (cur_act) {
#pragma unroll
        for (int r = 0; r < R; r++) S::load(cur[r], *mats[r], rows[r], 0, lane);
    }
    pdl_launch_dependents();
    pdl_wait();

    // Prologue: normalisation statistics, then the shared image of the (normalised) input.
    float mean = 0.0f, scale = 1.0f;
    if (PRO == PRO_RMS) {
        float ss = 0.0f;
        for (uint32_t c = threadIdx.x; c < K / 4; c += GEMV_NT) {
            float4 v = ld_act4(a.x + 4 * c);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum<GEMV_NT>(ss, red);
        scale = 1.0f / sqrtf(ss / (float)K + a.eps);
    } else if (PRO == PRO_LN) {
        float s = 0.0f;
        for (uint32_t c = threadIdx.x; c < K / 4; c += GEMV_NT) {
            float4 v = ld_act4(a.x + 4 * c);
            s += (v.x + v.y) + (v.z + v.w);
        }
        mean = block_sum<GEMV_NT>(s, red) / (float)K;
        float ss = 0.0f;
        for (uint32_t c = threadIdx.x; c < K / 4; c += GEMV_NT) {
            float4 v = ld_act4(a.x + 4 * c);
            v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum<GEMV_NT>(ss, red);
        scale = 1.0f / sqrtf(ss / (float)K + 1.0e-5f);
    }
    stage_x<QT, GEMV_NT>(xs, xsum, K, [&](uint32_t c) {
        float4 v = ld_act4(a.x + 4 * c);
        if (PRO == PRO_RMS) {
            const float4 w = __ldg(reinterpret_cast<const float4 *>(a.norm_w) + c);
            v.x = (v.x * scale) * w.x; v.y = (v.y * scale) * w.y; v.z = (v.z * scale) * w.z; v.w = (v.w * scale) * w.w;
        } else if (PRO == PRO_LN) {
            const float4 w = __ldg(reinterpret_cast<const float4 *>(a.norm_w) + c);
            const float4 b = __ldg(reinterpret_cast<const float4 *>(a.norm_b) + c);
            v.x = ((v.x - mean) * scale) * w.x + b.x; v.y = ((v.y - mean) * scale) * w.y + b.y;
            v.z = ((v.z - mean) * scale) * w.z + b.z; v.w = ((v.w - mean) * scale) * w.w + b.w;
        }
        return v;
    });

    while (have) {
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; r++) acc[r] = 0.0f;
        for (uint32_t col0 = 0; col0 < K; col0 += step_cols<QT>()) {
            // Issue the next step's loads before consuming the current one.
            typename S::Raw nxt[R];
            const uint32_t ncol = col0 + step_cols<QT>();
            const bool nxt_act = ncol < K && S::active(a.mat[0], ncol, lane);
            if (nxt_act) {
#pragma unroll
                for (int r = 0; r < R; r++) S::load(nxt[r], *mats[r], rows[r], ncol, lane);
            }
            if (cur_act) {
                typename S::X x;
                S::load_x(x, xs, xsum, col0, lane);
#pragma unroll
                for (int r = 0; r < R; r++) acc[r] += S::dot(cur[r], x, lane);
            }
            cur_act = nxt_act;
#pragma unroll
            for (int r = 0; r < R; r++) cur[r] = nxt[r];
        }
#pragma unroll
        for (int r = 0; r < R; r++) acc[r] = warp_sum(acc[r]);
        epilogue<EPI, R>(a, mats, rows, valid, acc, lane);

        gi += GEMV_WARPS * gridDim.x;
        have = group_rows<EPI, R>(a, gi, mats, rows, valid);
        cur_act = have && S::active(a.mat[0], 0, lane);
        if (cur_act) {
#pragma unroll
            for (int r = 0; r < R; r++) S::load(cur[r], *mats[r], rows[r], 0, lane);
        }
    }
}

// One warp per row, any format and layout, x read from global memory.
template <int QT>
__device__ __forceinline__ float generic_weight(const QMat &m, size_t row, uint32_t col);

template <int QT>
__global__ void __launch_bounds__(256) gemv_generic_kernel(const __grid_constant__ QMat m, const float *__restrict__ x,
                                                           float *__restrict__ out)
{
    constexpr int BL = block_len(QT), BB = block_bytes(QT);
    const int lane = threadIdx.x & 31;
    for (uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5); row < m.nrows; row += gridDim.x * 8) {
        float acc = 0.0f;
        if constexpr (BL == 1) {
            for (uint32_t c = lane; c < m.ncols; c += 32)
                acc = fmaf(dequant_one<QT>(m.p0 + ((size_t)row * m.ncols + c) * BB, 0, 0), x[c], acc);
        } else {
            // lane <-> 32-weight group, so the scale decode is hoisted out of the inner loop
            for (uint32_t grp = lane; grp < m.ncols / 32; grp += 32) {
                constexpr uint32_t GPB = BL / 32;  // 32-weight groups per block
                const uint32_t kb = grp / GPB, g = grp % GPB;
                const size_t blk = (size_t)row * m.bpr + kb;
                float s = 0.0f;
                if (m.planar && QT == WGB_Q8_0) {
                    const uint16_t d = ((const uint16_t *)m.p1)[blk];
                    for (int l = 0; l < 32; l++)
                        s = fmaf(q8_0_value(d, (int8_t)m.p0[(size_t)row * m.ncols + grp * 32 + l]), x[grp * 32 + l], s);
                } else if (m.planar && QT == WGB_Q6_K) {
                    for (int l = 0; l < 32; l++)
                        s = fmaf(q6_k_value(m.p0 + blk * 128, m.p1 + blk * 64, (const int8_t *)(m.p2 + blk * 16),
                                            ((const uint16_t *)m.p3)[blk], g, l),
                                 x[grp * 32 + l], s);
                } else {
                    const uint8_t *b = m.p0 + blk * BB;
                    for (int l = 0; l < 32; l++) s = fmaf(dequant_one<QT>(b, g, l), x[grp * 32 + l], s);
                }
                acc += s;
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) out[row] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------------------------

bool gemv_fast_supported(const QMat &m)
{
    if (!has_fast_path(m.qtype)) return false;
    if (m.qtype == WGB_F32) return m.ncols % 4 == 0 && ((uintptr_t)m.p0 % 16) == 0;
    if (m.qtype == WGB_Q8_0 || m.qtype == WGB_Q6_K) return m.planar != 0;
    return ((uintptr_t)m.p0 % 16) == 0;  // Q4_K raw
}

static size_t gemv_smem_bytes(uint32_t K) { return (size_t)K * 4 + (size_t)((K / 16 + 3) & ~3u) * 4 + 32 * 4; }

template <int QT, int R, int PRO, int EPI>
static int launch_one(const GemvArgs &a, uint32_t ngroups, cudaStream_t stream, bool pdl)
{
    auto kern = gemv_kernel<QT, R, PRO, EPI>;
    const size_t smem = gemv_smem_bytes(a.mat[0].ncols);
    if (smem > 48 * 1024) {
        static thread_local size_t configured = 0;  // per instantiation and thread
        if (smem > configured) {
            if (smem > 227 * 1024) return fail(WGB_ERR_UNSUPPORTED, "input vector of %u floats does not fit shared memory", a.mat[0].ncols);
            WGB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured = smem;
        }
    }
    const uint32_t per_block = (ngroups + GEMV_WARPS - 1) / GEMV_WARPS;
    uint32_t grid = (uint32_t)sm_count();
    if (per_block < grid) grid = per_block;
    if (grid == 0) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GEMV_NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    WGB_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    return WGB_OK;
}

template <int QT>
static int launch_qt(const GemvArgs &a, cudaStream_t stream, bool pdl)
{
    constexpr int R = 4;
    const uint32_t n0 = a.mat[0].nrows;
    switch (a.epilogue) {
    case EPI_STORE:
        if (a.prologue == PRO_NONE) return launch_one<QT, R, PRO_NONE, EPI_STORE>(a, (n0 + R - 1) / R, stream, pdl);
        if (a.prologue == PRO_RMS) return launch_one<QT, R, PRO_RMS, EPI_STORE>(a, (n0 + R - 1) / R, stream, pdl);
        return launch_one<QT, R, PRO_LN, EPI_STORE>(a, (n0 + R - 1) / R, stream, pdl);
    case EPI_RESIDUAL:
        if (a.prologue != PRO_NONE) break;
        return launch_one<QT, R, PRO_NONE, EPI_RESIDUAL>(a, (n0 + R - 1) / R, stream, pdl);
    case EPI_SILU_PAIR:
        if (a.prologue != PRO_RMS || a.nmat != 2) break;
        return launch_one<QT, R, PRO_RMS, EPI_SILU_PAIR>(a, (n0 + R / 2 - 1) / (R / 2), stream, pdl);
    case EPI_GELU:
        if (a.prologue != PRO_LN) break;
        return launch_one<QT, R, PRO_LN, EPI_GELU>(a, (n0 + R - 1) / R, stream, pdl);
    case EPI_QKV_ROPE: {
        if (a.prologue != PRO_RMS || a.nmat != 3) break;
        const uint32_t pairs = (a.mat[0].nrows + a.mat[1].nrows + a.mat[2].nrows) / 2;
        return launch_one<QT, R, PRO_RMS, EPI_QKV_ROPE>(a, (pairs + R / 2 - 1) / (R / 2), stream, pdl);
    }
    case EPI_QKV_SPLIT:
        if (a.prologue != PRO_LN) break;
        return launch_one<QT, R, PRO_LN, EPI_QKV_SPLIT>(a, (n0 + R - 1) / R, stream, pdl);
    }
    return fail(WGB_ERR_UNSUPPORTED, "no fused kernel for prologue %d / epilogue %d", a.prologue, a.epilogue);
}

int launch_gemv(const GemvArgs &a, cudaStream_t stream, bool pdl)
{
    for (int i = 0; i < a.nmat; i++) {
        if (!gemv_fast_supported(a.mat[i])) return fail(WGB_ERR_UNSUPPORTED, "no fast kernel for tensor type %d", a.mat[i].qtype);
        if (a.mat[i].qtype != a.mat[0].qtype || a.mat[i].ncols != a.mat[0].ncols)
            return fail(WGB_ERR_UNSUPPORTED, "fused matrices differ in format or width");
    }
    switch (a.mat[0].qtype) {
    case WGB_Q4_K: return launch_qt<WGB_Q4_K>(a, stream, pdl);
    case WGB_Q6_K: return launch_qt<WGB_Q6_K>(a, stream, pdl);
    case WGB_Q8_0: return launch_qt<WGB_Q8_0>(a, stream, pdl);
    case WGB_F32: return launch_qt<WGB_F32>(a, stream, pdl);
    }
    return fail(WGB_ERR_UNSUPPORTED, "no fast kernel for tensor type %d", a.mat[0].qtype);
}

int launch_gemv_generic(const QMat &m, const float *x, float *out, cudaStream_t stream)
{
    uint32_t grid = (m.nrows + 7) / 8;
    const uint32_t cap = (uint32_t)sm_count() * 8;
    if (grid > cap) grid = cap;
#define WGB_GENERIC_CASE(T) case T: gemv_generic_kernel<T><<<grid, 256, 0, stream>>>(m, x, out); break;
    switch (m.qtype) {
        WGB_GENERIC_CASE(WGB_F32) WGB_GENERIC_CASE(WGB_F16) WGB_GENERIC_CASE(WGB_Q4_0) WGB_GENERIC_CASE(WGB_Q4_1)
        WGB_GENERIC_CASE(WGB_Q5_0) WGB_GENERIC_CASE(WGB_Q5_1) WGB_GENERIC_CASE(WGB_Q8_0) WGB_GENERIC_CASE(WGB_Q4_K)
        WGB_GENERIC_CASE(WGB_Q5_K) WGB_GENERIC_CASE(WGB_Q6_K) WGB_GENERIC_CASE(WGB_Q8_K)
    default: return fail(WGB_ERR_UNSUPPORTED, "unsupported tensor type %d", m.qtype);
    }
#undef WGB_GENERIC_CASE
    WGB_LAUNCH_CHECK("gemv_generic_kernel");
    return WGB_OK;
}

}  // namespace wgb

using namespace wgb;

static int gemv_dispatch(const QMat &m, const float *d_v, float *d_out, cudaStream_t stream)
{
    WGB_REQUIRE(d_v && d_out, "null argument");
    if (gemv_fast_supported(m) && ((uintptr_t)d_v % 16) == 0) {
        GemvArgs a = {};
        a.mat[0] = m;
        a.nmat = 1;
        a.x = d_v;
        a.prologue = PRO_NONE;
        a.epilogue = EPI_STORE;
        a.out = d_out;
        return launch_gemv(a, stream, false);
    }
    return launch_gemv_generic(m, d_v, d_out, stream);
}

WGB_EXPORT int wgb_gemv_quant(const wgb_quant_matrix *m, const float *d_v, float *d_out, void *stream)
{
    WGB_REQUIRE(m, "null matrix");
    return gemv_dispatch(m->view, d_v, d_out, as_stream(stream));
}

WGB_EXPORT int wgb_gemv_quant_raw(int qtype, const void *d_blocks, size_t nrows, size_t ncols, const float *d_v,
                                  float *d_out, void *stream)
{
    const int bl = block_len(qtype);
    if (!bl) return fail(WGB_ERR_UNSUPPORTED, "unsupported tensor type %d", qtype);
    WGB_REQUIRE(d_blocks && nrows > 0 && ncols > 0 && ncols % bl == 0, "bad matrix shape %zu x %zu", nrows, ncols);
    QMat m = {};
    m.qtype = qtype;
    m.planar = 0;
    m.nrows = (uint32_t)nrows;
    m.ncols = (uint32_t)ncols;
    m.bpr = (uint32_t)(ncols / bl);
    m.p0 = (const uint8_t *)d_blocks;
    return gemv_dispatch(m, d_v, d_out, as_stream(stream));
}
