// Matrix-vector kernels: the fused, TMA-fed kernel used by the models and by GemvQuant, and the
// generic per-format fallback.
//
// Fused kernel.  One persistent block per SM: eight consumer warps and one producer warp.
//   * Rows are taken in groups of `rs` (2..8) that lie contiguously in HBM.  The producer streams
//     group after group into a ring of shared-memory stages with one bulk asynchronous copy
//     (cp.async.bulk, completion on an mbarrier) per plane of the group, running as many stages
//     ahead as the ring holds.  It starts before the kernel waits for its predecessor in the stream
//     (programmatic dependent launch): weights never depend on activations, so a kernel fills its
//     ring -- the whole matrix, for the small ones -- while the previous kernel is still finishing.
//   * The consumers build the shared image of the (normalised) input vector once.  They are split
//     into slots of `wk` warps; the warps of a slot each own one column step of the matrix (so their
//     part of the input stays in registers for the whole kernel) and together take every nslot-th
//     stage.  The per-row partial sums of the column steps meet in shared memory behind a barrier
//     private to the slot; the slot's first warp adds them and runs the epilogue (bias, residual,
//     SiLU gate, GELU, RoPE + KV-cache append), one lane per output row.  Slots never wait for each
//     other, so several stages are in work at any time.
//   * Group g belongs to block g % gridDim.x, so every SM gets the same number of groups to within
//     one; rs is chosen per launch for the best balance.
// Every mbarrier wait is bounded: after ~2^22 polls a waiter records an error code in the launch's
// status word and carries on with whatever is in shared memory, so the kernel always terminates.
#include "gemv_core.cuh"
#include "kernels.h"
#include "qaccess.cuh"

#include <cstdio>
#include <cstdlib>

namespace wgb {

#ifndef WGB_GEMV_NCONS
#define WGB_GEMV_NCONS 16
#endif
#ifndef WGB_GEMV_MINBLOCKS
#define WGB_GEMV_MINBLOCKS 1
#endif
#ifndef WGB_GEMV_SMEM_KB
#define WGB_GEMV_SMEM_KB 200
#endif
constexpr int GEMV_NCONS = WGB_GEMV_NCONS;          // consumer warps
constexpr int GEMV_MAX_SLOTS = 8;                   // mini-slots of consumer warps
constexpr int GEMV_CONS_THREADS = GEMV_NCONS * 32;
constexpr int GEMV_NT = GEMV_CONS_THREADS + 32;     // + producer warp
constexpr int GEMV_MAX_RS = 8;                      // rows per stage
constexpr int GEMV_MAX_STAGES = 16;
constexpr uint32_t GEMV_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ float4 ld_act4(const float *p)
{
    return __ldcg(reinterpret_cast<const float4 *>(p));
}

__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GEMV_CONS_THREADS) : "memory"); }
// Barrier among the `nthreads` threads of consumer slot `slot` (named barriers 2..2+GEMV_MAX_SLOTS-1).
__device__ __forceinline__ void slot_sync(uint32_t slot, uint32_t nthreads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(slot + 2), "r"(nthreads) : "memory");
}

// Sum / max over the 256 consumer threads (named barrier 1); every consumer gets the result.
__device__ __forceinline__ float cons_sum(float v, float *red)
{
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    cons_sync();
    if (lane == 0) red[warp] = v;
    cons_sync();
    float t = (lane < GEMV_NCONS) ? red[lane] : 0.0f;
    static_assert(GEMV_NCONS <= 32, "one partial per consumer warp");
    return warp_sum(t);
}

// ---- mbarrier / bulk-copy primitives ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; on expiry records `code` in *err and returns false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t *err, uint32_t code)
{
    for (uint32_t i = 0; i < GEMV_WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    if (err) atomicExch(err, code);
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- groups ------------------------------------------------------------------------------------
struct Part {
    int mat;
    uint32_t row0;
};

// Parts (1 or 2 runs of `n` consecutive rows of one matrix) of group gi; returns the number of parts,
// 0 past the end.
template <int EPI>
__device__ __forceinline__ int group_parts(const GemvArgs &a, uint32_t gi, Part (&parts)[2], uint32_t &n)
{
    const uint32_t rs = a.rs;
    if (gi >= a.ngroups) return 0;
    if (EPI == EPI_SILU_PAIR) {
        const uint32_t h = rs / 2, r0 = gi * h, nr = a.mat[0].nrows;
        n = min(h, nr - r0);
        parts[0] = { 0, r0 };
        parts[1] = { 1, r0 };
        return 2;
    } else if (EPI == EPI_QKV_ROPE) {
        const uint32_t gq = a.mat[0].nrows / rs, gk = a.mat[1].nrows / rs;
        const int s = gi < gq ? 0 : (gi < gq + gk ? 1 : 2);
        const uint32_t lg = gi - (s == 0 ? 0 : (s == 1 ? gq : gq + gk));
        if (s < 2 && a.rope_variant == WGB_ROPE_NEOX) {
            const uint32_t h2 = rs / 2, half = a.head_size / 2, lp = lg * h2;
            const uint32_t r0 = (lp / half) * a.head_size + lp % half;
            n = h2;
            parts[0] = { s, r0 };
            parts[1] = { s, r0 + half };
            return 2;
        }
        n = rs;
        parts[0] = { s, lg * rs };
        return 1;
    } else {
        const uint32_t r0 = gi * rs, nr = a.mat[0].nrows;
        n = min(rs, nr - r0);
        parts[0] = { 0, r0 };
        return 1;
    }
}

__device__ __forceinline__ float gelu_f32(float x)
{
    // UnaryOp::Gelu, crates/wgml/src/ops/unary.rs:106-110
    const float GELU_COEF_A = 0.044715f, SQRT_2_OVER_PI = 0.7978846f;
    return 0.5f * x * (1.0f + tanhf(SQRT_2_OVER_PI * x * (1.0f + GELU_COEF_A * x * x)));
}

// RoPE (ops/rope.wgsl:36-77): angle = pos * base^(-(2i % head_size) / head_size) for pair (r0, r1).
__device__ __forceinline__ void rope_pair(const GemvArgs &a, uint32_t r0, uint32_t pos, float &y0, float &y1)
{
    const uint32_t half = a.head_size / 2;
    const uint32_t fi = (a.rope_variant == WGB_ROPE_NEOX) ? (r0 % a.head_size) : ((r0 / 2) % half);
    float sn, cs;
    sincosf((float)pos * a.rope_freq[fi], &sn, &cs);
    const float t0 = cs * y0 - sn * y1, t1 = sn * y0 + cs * y1;
    y0 = t0;
    y1 = t1;
}

// Output units of a group (a unit = the stage rows that make one output: a row, or a pair) and the
// stage rows of unit u.
template <int EPI>
__device__ __forceinline__ uint32_t group_units(const Part (&parts)[2], int nparts, uint32_t n)
{
    if (EPI == EPI_QKV_ROPE && nparts == 1 && parts[0].mat < 2) return n / 2;   // adjacent pairs
    return n;
}
template <int EPI>
__device__ __forceinline__ void unit_rows(const Part (&parts)[2], int nparts, uint32_t n, uint32_t u, uint32_t &ra, uint32_t &rb)
{
    if (EPI == EPI_SILU_PAIR || (EPI == EPI_QKV_ROPE && nparts == 2)) { ra = u; rb = n + u; }
    else if (EPI == EPI_QKV_ROPE && parts[0].mat < 2) { ra = 2 * u; rb = 2 * u + 1; }
    else { ra = u; rb = u; }
}

// Row slot that owns stage row j (the slot of the unit the row belongs to).
template <int EPI>
__device__ __forceinline__ uint32_t row_slot_of(const Part (&parts)[2], int nparts, uint32_t n, uint32_t j, uint32_t rsl)
{
    uint32_t u;
    if (EPI == EPI_SILU_PAIR || (EPI == EPI_QKV_ROPE && nparts == 2)) u = j >= n ? j - n : j;
    else if (EPI == EPI_QKV_ROPE && parts[0].mat < 2) u = j / 2;
    else u = j;
    return u % rsl;
}

// Epilogue of output unit t of a group; `sum(r)` gives the finished dot product of stage row r.
template <int EPI, typename SumF>
__device__ __forceinline__ void group_epilogue(const GemvArgs &a, const Part (&parts)[2], int nparts, uint32_t n, uint32_t t, SumF sum)
{
    if (EPI == EPI_STORE || EPI == EPI_RESIDUAL || EPI == EPI_GELU) {
        if (t < n) {
            const uint32_t row = parts[0].row0 + t;
            float y = sum(t);
            if (a.bias) y += a.bias[row];
            if (EPI == EPI_RESIDUAL) y = a.residual[row] + y;
            if (EPI == EPI_GELU) y = gelu_f32(y);
            a.out[row] = y;
        }
    } else if (EPI == EPI_SILU_PAIR) {
        if (t < n) {
            const float g = sum(t), u = sum(n + t);
            a.out[parts[0].row0 + t] = u * (g / (1.0f + expf(-g)));
        }
    } else if (EPI == EPI_QKV_ROPE) {
        const int s = parts[0].mat;
        const float *bias = s == 0 ? a.bias : (s == 1 ? a.bias_k : a.bias_v);
        const uint32_t pos = *a.pos;
        float *dst = s == 0 ? a.out : ((s == 1 ? a.k_cache : a.v_cache) + (size_t)pos * a.kv_dim);
        if (s == 2) {
            if (t < n) {
                const uint32_t row = parts[0].row0 + t;
                dst[row] = sum(t) + (bias ? bias[row] : 0.0f);
            }
        } else if (nparts == 2) {  // Neox: pairs (r0 + t, r0 + t + head_size/2)
            if (t < n) {
                const uint32_t r0 = parts[0].row0 + t, r1 = parts[1].row0 + t;
                float y0 = sum(t) + (bias ? bias[r0] : 0.0f), y1 = sum(n + t) + (bias ? bias[r1] : 0.0f);
                rope_pair(a, r0, pos, y0, y1);
                dst[r0] = y0;
                dst[r1] = y1;
            }
        } else if (t < n / 2) {  // Original: adjacent pairs
            const uint32_t r0 = parts[0].row0 + 2 * t;
            float y0 = sum(2 * t) + (bias ? bias[r0] : 0.0f), y1 = sum(2 * t + 1) + (bias ? bias[r0 + 1] : 0.0f);
            rope_pair(a, r0, pos, y0, y1);
            dst[r0] = y0;
            dst[r0 + 1] = y1;
        }
    } else if (EPI == EPI_QKV_SPLIT) {
        if (t < n) {
            const uint32_t row = parts[0].row0 + t, d = a.kv_dim, pos = *a.pos;
            float y = sum(t);
            if (a.bias) y += a.bias[row];
            if (row < d) a.out[row] = y;
            else if (row < 2 * d) a.k_cache[(size_t)pos * d + (row - d)] = y;
            else a.v_cache[(size_t)pos * d + (row - 2 * d)] = y;
        }
    }
}

template <int QT, int PRO, int EPI>
__global__ void __launch_bounds__(GEMV_NT, WGB_GEMV_MINBLOCKS) gemv_kernel(const __grid_constant__ GemvArgs a)
{
    using S = Step<QT>;
    constexpr int NPL = QT == WGB_Q6_K ? 4 : (QT == WGB_Q8_0 ? 2 : 1);   // planes of the format
    extern __shared__ uint4 smem4[];
    __shared__ float red[32];
    __shared__ float part[GEMV_MAX_STAGES][GEMV_MAX_RS][GEMV_NCONS];
    __shared__ __align__(8) unsigned long long bars[2 * GEMV_MAX_STAGES];

    const uint32_t K = a.mat[0].ncols;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t nstage = a.nstage;
    uint8_t *smem = reinterpret_cast<uint8_t *>(smem4);
    const uint32_t ring = smem_addr(smem + a.ring_offset);
    const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[GEMV_MAX_STAGES]);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < nstage; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, a.wk * a.rslots);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
#ifndef WGB_DBG_NOPDL
    pdl_launch_dependents();
#endif

    // bytes per row over all planes, and the offset of each plane inside a part of n rows
    uint32_t row_bytes = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) row_bytes += a.mat[0].pitch[i];

    if (warp == GEMV_NCONS) {
        // ------------------------------ producer ------------------------------
        const int nplanes = a.mat[0].nplanes;
        uint32_t it = 0, s = 0, phase = 1;   // parity of the previous use of ring slot s
        for (uint32_t gi = blockIdx.x; gi < a.ngroups; gi += gridDim.x, it++, s = (s + 1 == nstage) ? 0 : s + 1, phase ^= (s == 0)) {
            if (it >= nstage) mbar_wait(empty0 + 8 * s, phase, a.err, 2);
            Part parts[2];
            uint32_t n = 0;
            const int nparts = group_parts<EPI>(a, gi, parts, n);
            const uint32_t stage = ring + s * a.stage_bytes;
            if (lane == 0) mbar_expect_tx(full0 + 8 * s, nparts * n * row_bytes);
            __syncwarp();
            if (lane < nparts * nplanes) {
                const int pi = lane / nplanes, pl = lane % nplanes;
                const QMat &m = a.mat[parts[pi].mat];
                uint32_t off = pi * n * row_bytes;
                for (int q = 0; q < pl; q++) off += n * m.pitch[q];
                bulk_copy_g2s(stage + off, m.p[pl] + (size_t)parts[pi].row0 * m.pitch[pl], n * m.pitch[pl], full0 + 8 * s);
            }
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
#ifndef WGB_DBG_NOPDL
    pdl_wait();
#endif
    float mean = 0.0f, scale = 1.0f;
    if (PRO == PRO_RMS) {
        float ss = 0.0f;
        for (uint32_t c = threadIdx.x; c < K / 4; c += GEMV_CONS_THREADS) {
            float4 v = ld_act4(a.x + 4 * c);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = cons_sum(ss, red);
        scale = 1.0f / sqrtf(ss / (float)K + a.eps);
    } else if (PRO == PRO_LN) {
        float s = 0.0f;
        for (uint32_t c = threadIdx.x; c < K / 4; c += GEMV_CONS_THREADS) {
            float4 v = ld_act4(a.x + 4 * c);
            s += (v.x + v.y) + (v.z + v.w);
        }
        mean = cons_sum(s, red) / (float)K;
        float ss = 0.0f;
        for (uint32_t c = threadIdx.x; c < K / 4; c += GEMV_CONS_THREADS) {
            float4 v = ld_act4(a.x + 4 * c);
            v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = cons_sum(ss, red);
        scale = 1.0f / sqrtf(ss / (float)K + 1.0e-5f);
    }
    stage_x<QT, GEMV_CONS_THREADS>(smem, K, [&](uint32_t c) {
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
    cons_sync();

    const XImage im = ximage_carve(QT, K, smem);
    const uint32_t kunits = QT == WGB_F32 ? K : a.mat[0].bpr;   // what Step::active() compares against
    const uint32_t nsteps = (K + step_cols<QT>() - 1) / step_cols<QT>();
    // Mini-slots of wk warps: `nss` stage slots (stages in work at once) x `rsl` row slots (shares of
    // a stage's output units).
    const uint32_t wk = a.wk, nss = a.nslot, rsl = a.rslots;
    const uint32_t kw = warp % wk, slot = warp / wk;
    const uint32_t sslot = slot / rsl, rslot = slot % rsl;
    const bool working = (uint32_t)warp < wk * nss * rsl;
    const bool single = nsteps <= wk;   // this warp's only column step: keep its x in registers
    typename S::X x;
    if (working && single && S::active(kunits, kw * step_cols<QT>(), lane)) S::load_x(x, im, kw * step_cols<QT>(), lane);

    if (!working) return;

    // Stage slot `sslot` takes every nss-th stage of this block.
    uint32_t s = sslot % nstage, phase = (sslot / nstage) & 1;   // ring slot and parity of stage `it`
    for (uint32_t it = sslot, gi = blockIdx.x + sslot * gridDim.x; gi < a.ngroups;
         it += nss, gi += nss * gridDim.x, s += nss, phase ^= (s >= nstage), s -= (s >= nstage) ? nstage : 0) {
        Part parts[2];
        uint32_t n = 0;
        const int nparts = group_parts<EPI>(a, gi, parts, n);
        const uint32_t nrows = nparts * n;
        const uint32_t nunits = group_units<EPI>(parts, nparts, n);
        const bool paired = EPI == EPI_SILU_PAIR || (EPI == EPI_QKV_ROPE && parts[0].mat < 2);
        const uint32_t stage = ring + s * a.stage_bytes;
#ifdef WGB_DBG_TIMING
        long long t0 = clock64();
#endif
        mbar_wait(full0 + 8 * s, phase, a.err, 1);
#ifdef WGB_DBG_TIMING
        long long t1 = clock64();
#endif
#ifndef WGB_DBG_NOCOMPUTE
        // first shared-memory byte of row 0 of each part in each plane
        uint32_t base[2][NPL];
#pragma unroll
        for (int pi = 0; pi < 2; pi++) {
            uint32_t off = stage + pi * n * row_bytes;
#pragma unroll
            for (int q = 0; q < NPL; q++) {
                base[pi][q] = off;
                off += n * a.mat[0].pitch[q];
            }
        }
        if (single) {
            // Two rows at a time (the two rows of a pair unit, or two single-row units): independent
            // chains for the scheduler to interleave.
            const uint32_t col0 = kw * step_cols<QT>();
            const bool act = S::active(kunits, col0, lane);
            for (uint32_t u = rslot; u < nunits; u += paired ? rsl : 2 * rsl) {
                uint32_t j, j1;
                if (paired) unit_rows<EPI>(parts, nparts, n, u, j, j1);
                else { j = u; j1 = min(u + rsl, nunits - 1); if (u + rsl >= nunits) j1 = j; }
                float v0 = 0.0f, v1 = 0.0f;
                if (act) {
                    uint32_t r0[4], r1[4];
                    const uint32_t p0 = j >= n ? 1 : 0, p1 = j1 >= n ? 1 : 0;
#pragma unroll
                    for (int q = 0; q < NPL; q++) {
                        r0[q] = base[p0][q] + (j - p0 * n) * a.mat[0].pitch[q];
                        r1[q] = base[p1][q] + (j1 - p1 * n) * a.mat[0].pitch[q];
                    }
                    v0 = S::dot(r0, col0, x, lane);
                    v1 = S::dot(r1, col0, x, lane);
                }
#ifdef WGB_DBG_NOSUM
                if (v0 + v1 == 1.2345e-30f) part[s][j][kw] = v0;
#else
                v0 = warp_sum(v0);
                v1 = warp_sum(v1);
                if (lane == 0) {
                    part[s][j][kw] = v0;
                    part[s][j1][kw] = v1;
                }
#endif
            }
        } else {
            float acc[GEMV_MAX_RS];
#pragma unroll
            for (int j = 0; j < GEMV_MAX_RS; j++) acc[j] = 0.0f;
            for (uint32_t ks = kw; ks < nsteps; ks += wk) {
                const uint32_t col0 = ks * step_cols<QT>();
                if (S::active(kunits, col0, lane)) {
                    S::load_x(x, im, col0, lane);
#pragma unroll
                    for (int j = 0; j < GEMV_MAX_RS; j++) {
                        if ((uint32_t)j < nrows && row_slot_of<EPI>(parts, nparts, n, j, rsl) == rslot) {
                            const uint32_t pi = (uint32_t)j >= n ? 1 : 0;
                            uint32_t rowp[4];
#pragma unroll
                            for (int q = 0; q < NPL; q++) rowp[q] = base[pi][q] + (j - pi * n) * a.mat[0].pitch[q];
                            acc[j] += S::dot(rowp, col0, x, lane);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < GEMV_MAX_RS; j++) {
                if ((uint32_t)j < nrows && row_slot_of<EPI>(parts, nparts, n, j, rsl) == rslot) {
                    const float v = warp_sum(acc[j]);
                    if (lane == 0) part[s][j][kw] = v;
                }
            }
        }
#endif
#ifdef WGB_DBG_TIMING
        long long t2 = clock64();
#endif
        // hand the partial sums of the column steps to the slot's first warp
        (void)nrows;
#ifndef WGB_DBG_NOSYNC
        if (wk > 1) slot_sync(slot, wk * 32);
        else __syncwarp();
#endif
        if (kw == 0) {
            // Read the partial sums first, release the stage, then write the outputs: the release must
            // not wait for the global stores of the epilogue.
            const uint32_t u = rslot + (uint32_t)lane * rsl;
            uint32_t ra = 0, rb = 0;
            float ya = 0.0f, yb = 0.0f;
            if (u < nunits) {
                unit_rows<EPI>(parts, nparts, n, u, ra, rb);
                for (uint32_t k = 0; k < wk; k++) {
                    ya += part[s][ra][k];
                    yb += part[s][rb][k];
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
#ifndef WGB_DBG_NOEPI
            group_epilogue<EPI>(a, parts, nparts, n, u, [&](uint32_t r) { return r == ra ? ya : yb; });
#endif
        } else if (lane == 0) {
            mbar_arrive(empty0 + 8 * s);   // this warp is done with the stage and its partial sums
        }
#ifdef WGB_DBG_TIMING
        long long t3 = clock64();
        if (lane == 0 && a.dbg) {
            atomicAdd(a.dbg + 0, (unsigned long long)(t1 - t0));
            atomicAdd(a.dbg + 1, (unsigned long long)(t2 - t1));
            atomicAdd(a.dbg + 2, (unsigned long long)(t3 - t2));
            atomicAdd(a.dbg + 3, 1ull);
        }
#endif
    }
}

// One warp per row, any format and layout, x read from global memory.
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
                acc = fmaf(dequant_one<QT>(m.p[0] + ((size_t)row * m.ncols + c) * BB, 0, 0), x[c], acc);
        } else {
            // lane <-> 32-weight group, so the scale decode is hoisted out of the inner loop
            for (uint32_t grp = lane; grp < m.ncols / 32; grp += 32) {
                constexpr uint32_t GPB = BL / 32;  // 32-weight groups per block
                const uint32_t kb = grp / GPB, g = grp % GPB;
                float s = 0.0f;
                if (m.planar) {
                    for (int l = 0; l < 32; l++) s = fmaf(qmat_weight<QT>(m, row, grp * 32 + l), x[grp * 32 + l], s);
                } else {
                    const uint8_t *b = m.p[0] + (size_t)row * m.pitch[0] + (size_t)kb * BB;
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
    for (int i = 0; i < m.nplanes; i++)
        if (((uintptr_t)m.p[i] % 16) != 0 || m.pitch[i] % 16 != 0) return false;
    if (m.qtype == WGB_F32) return m.ncols % 4 == 0;
    if (m.ncols % 32 != 0) return false;
    if (m.qtype == WGB_Q8_0 || m.qtype == WGB_Q6_K) return m.planar != 0;
    return true;  // Q4_K raw
}

// Device status word shared by all launches of the process: 0, or the code of the first bounded
// wait that expired (1 consumer, 2 producer).
static uint32_t *g_err = nullptr;
static int ensure_err()
{
    if (g_err) return WGB_OK;
    WGB_CUDA(cudaMalloc((void **)&g_err, sizeof(uint32_t)));
    WGB_CUDA(cudaMemset(g_err, 0, sizeof(uint32_t)));
    return WGB_OK;
}

int gemv_check_status()
{
    if (!g_err) return WGB_OK;
    uint32_t v = 0;
    WGB_CUDA(cudaMemcpy(&v, g_err, sizeof(v), cudaMemcpyDeviceToHost));
    if (v) {
        cudaMemset(g_err, 0, sizeof(uint32_t));
        return fail(WGB_ERR_TIMEOUT, "a bounded wait inside a matrix-vector kernel expired (code %u)", v);
    }
    return WGB_OK;
}

static uint32_t steps_of(int qt, uint32_t K)
{
    const uint32_t sc = qt == WGB_Q4_K ? step_cols<WGB_Q4_K>() : qt == WGB_Q6_K ? step_cols<WGB_Q6_K>()
                      : qt == WGB_Q8_0 ? step_cols<WGB_Q8_0>() : step_cols<WGB_F32>();
    return (K + sc - 1) / sc;
}

// Chooses rows per stage, ring depth and grid; fills the plan fields of `a`.  Returns false when the
// shapes do not fit the kernel's assumptions.
static bool plan(GemvArgs &a, size_t &smem_bytes, uint32_t &grid)
{
    const QMat &m0 = a.mat[0];
    uint32_t row_bytes = 0;
    for (int i = 0; i < m0.nplanes; i++) row_bytes += m0.pitch[i];
    const uint32_t sms = (uint32_t)sm_count();
    // rows (or pairs of rows) that must stay together
    uint32_t total_rows = 0;
    for (int i = 0; i < a.nmat; i++) total_rows += a.mat[i].nrows;
    const bool pairs = a.epilogue == EPI_SILU_PAIR || a.epilogue == EPI_QKV_ROPE;
    const size_t image = (ximage_bytes(m0.qtype, m0.ncols) + 127) & ~(size_t)127;
    const size_t budget_max = (size_t)WGB_GEMV_SMEM_KB * 1024, budget_hard = 200 * 1024;
    const uint32_t nsteps = steps_of(m0.qtype, m0.ncols);
    const uint32_t wk = nsteps < (uint32_t)GEMV_NCONS ? nsteps : (uint32_t)GEMV_NCONS;
    uint32_t slots = GEMV_NCONS / wk;             // mini-slots of wk warps
    if (slots > GEMV_MAX_SLOTS) slots = GEMV_MAX_SLOTS;
    const uint32_t nslot = slots >= 4 ? 2 : 1;      // stage slots
    const uint32_t rslots = slots / nslot;          // row slots per stage
    uint32_t best_rs = 0;
    double best_score = -1.0;
    for (uint32_t rs = GEMV_MAX_RS; rs >= 1; rs--) {
        if (pairs && (rs & 1)) continue;
        const size_t stage = ((size_t)rs * row_bytes + 127) & ~(size_t)127;
        if (image + (nslot + 3) * stage > budget_max && rs > (pairs ? 2u : 1u)) continue;   // ring: stages in work + 3 in flight
        if (image + 2 * stage > budget_hard) continue;
        if (a.epilogue == EPI_QKV_ROPE) {
            bool ok = true;
            for (int i = 0; i < 3; i++) ok = ok && a.mat[i].nrows % rs == 0;
            if (a.rope_variant == WGB_ROPE_NEOX) ok = ok && (a.head_size / 2) % (rs / 2) == 0;
            if (!ok) continue;
        }
        uint32_t groups;
        if (a.epilogue == EPI_SILU_PAIR) groups = (m0.nrows + rs / 2 - 1) / (rs / 2);
        else if (a.epilogue == EPI_QKV_ROPE) groups = total_rows / rs;
        else groups = (m0.nrows + rs - 1) / rs;
        const uint32_t per = (groups + sms - 1) / sms;
        // balance across SMs, discounted for small stages (fixed cost per stage ~ 2 KB of streaming)
        const double score = (double)groups / ((double)per * sms) * ((double)stage / ((double)stage + 2048.0));
        if (score > best_score + 1e-9) { best_score = score; best_rs = rs; }
    }
    if (!best_rs) return false;
    a.rs = best_rs;
    if (a.epilogue == EPI_SILU_PAIR) a.ngroups = (m0.nrows + best_rs / 2 - 1) / (best_rs / 2);
    else if (a.epilogue == EPI_QKV_ROPE) a.ngroups = total_rows / best_rs;
    else a.ngroups = (m0.nrows + best_rs - 1) / best_rs;
    a.stage_bytes = (uint32_t)(((size_t)best_rs * row_bytes + 127) & ~(size_t)127);
    grid = a.ngroups < sms ? a.ngroups : sms;
    const uint32_t per_block = (a.ngroups + grid - 1) / grid;
    const size_t budget = image + (nslot + 3) * (size_t)a.stage_bytes > budget_max ? budget_hard : budget_max;
    uint32_t ns = (uint32_t)((budget - image) / a.stage_bytes);
    if (ns > GEMV_MAX_STAGES) ns = GEMV_MAX_STAGES;
    if (ns > per_block) ns = per_block;
    if (ns < 1) ns = 1;
    a.nstage = ns;
    a.ring_offset = (uint32_t)image;
    a.wk = wk;
    a.nslot = nslot;
    a.rslots = rslots;
    smem_bytes = image + (size_t)ns * a.stage_bytes;
    return true;
}

template <int QT>
static int set_smem_attr()
{
    const int bytes = 200 * 1024;
#define WGB_ATTR(PRO, EPI) WGB_CUDA(cudaFuncSetAttribute(gemv_kernel<QT, PRO, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes))
    WGB_ATTR(PRO_NONE, EPI_STORE);
    WGB_ATTR(PRO_RMS, EPI_STORE);
    WGB_ATTR(PRO_LN, EPI_STORE);
    WGB_ATTR(PRO_NONE, EPI_RESIDUAL);
    WGB_ATTR(PRO_RMS, EPI_SILU_PAIR);
    WGB_ATTR(PRO_LN, EPI_GELU);
    WGB_ATTR(PRO_RMS, EPI_QKV_ROPE);
    WGB_ATTR(PRO_LN, EPI_QKV_SPLIT);
#undef WGB_ATTR
    return WGB_OK;
}

// One-time set-up of the fused kernels on the current device: the status word and the opt-in to
// large dynamic shared memory.  Must first run outside stream capture (model creation does).
int gemv_global_init()
{
    static bool done = false;
    if (done) return WGB_OK;
    int rc = ensure_err();
    if (rc) return rc;
    if ((rc = set_smem_attr<WGB_Q4_K>()) || (rc = set_smem_attr<WGB_Q6_K>()) || (rc = set_smem_attr<WGB_Q8_0>()) ||
        (rc = set_smem_attr<WGB_F32>()))
        return rc;
    done = true;
    return WGB_OK;
}

template <int QT, int PRO, int EPI>
static int launch_one(GemvArgs &a, cudaStream_t stream, bool pdl)
{
    auto kern = gemv_kernel<QT, PRO, EPI>;
    size_t smem = 0;
    uint32_t grid = 0;
    if (!plan(a, smem, grid)) return fail(WGB_ERR_UNSUPPORTED, "matrix shape does not fit the fused kernel");
    int rc = gemv_global_init();
    if (rc) return rc;
    a.err = g_err;
#ifdef WGB_DBG_TIMING
    static unsigned long long *dbg = nullptr;
    if (!dbg) { cudaMalloc((void **)&dbg, 64); cudaMemset(dbg, 0, 64); }
    if (getenv("WGB_DBG_DUMP")) {
        unsigned long long h[4];
        cudaMemcpy(h, dbg, 32, cudaMemcpyDeviceToHost);
        if (h[3]) fprintf(stderr, "timing: stages=%llu wait=%.0f compute=%.0f tail=%.0f cycles/stage/warp\n", h[3], (double)h[0] / h[3], (double)h[1] / h[3], (double)h[2] / h[3]);
        cudaMemset(dbg, 0, 64);
    }
    a.dbg = dbg;
#endif
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
    if (getenv("WGB_DBG_PLAN"))
        fprintf(stderr, "gemv plan: qt=%d rows=%u K=%u rs=%u ngroups=%u nstage=%u stage=%u ring_off=%u wk=%u grid=%u smem=%zu\n", QT,
                a.mat[0].nrows, a.mat[0].ncols, a.rs, a.ngroups, a.nstage, a.stage_bytes, a.ring_offset, a.wk * 10000 + a.nslot * 100 + a.rslots, grid, smem);
    WGB_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    return WGB_OK;
}

template <int QT>
static int launch_qt(GemvArgs &a, cudaStream_t stream, bool pdl)
{
    switch (a.epilogue) {
    case EPI_STORE:
        if (a.prologue == PRO_NONE) return launch_one<QT, PRO_NONE, EPI_STORE>(a, stream, pdl);
        if (a.prologue == PRO_RMS) return launch_one<QT, PRO_RMS, EPI_STORE>(a, stream, pdl);
        return launch_one<QT, PRO_LN, EPI_STORE>(a, stream, pdl);
    case EPI_RESIDUAL:
        if (a.prologue != PRO_NONE) break;
        return launch_one<QT, PRO_NONE, EPI_RESIDUAL>(a, stream, pdl);
    case EPI_SILU_PAIR:
        if (a.prologue != PRO_RMS || a.nmat != 2) break;
        return launch_one<QT, PRO_RMS, EPI_SILU_PAIR>(a, stream, pdl);
    case EPI_GELU:
        if (a.prologue != PRO_LN) break;
        return launch_one<QT, PRO_LN, EPI_GELU>(a, stream, pdl);
    case EPI_QKV_ROPE:
        if (a.prologue != PRO_RMS || a.nmat != 3) break;
        return launch_one<QT, PRO_RMS, EPI_QKV_ROPE>(a, stream, pdl);
    case EPI_QKV_SPLIT:
        if (a.prologue != PRO_LN) break;
        return launch_one<QT, PRO_LN, EPI_QKV_SPLIT>(a, stream, pdl);
    }
    return fail(WGB_ERR_UNSUPPORTED, "no fused kernel for prologue %d / epilogue %d", a.prologue, a.epilogue);
}

int launch_gemv(const GemvArgs &args, cudaStream_t stream, bool pdl)
{
    GemvArgs a = args;
    for (int i = 0; i < a.nmat; i++) {
        if (!gemv_fast_supported(a.mat[i])) return fail(WGB_ERR_UNSUPPORTED, "no fast kernel for tensor type %d", a.mat[i].qtype);
        if (a.mat[i].qtype != a.mat[0].qtype || a.mat[i].ncols != a.mat[0].ncols)
            return fail(WGB_ERR_UNSUPPORTED, "fused matrices differ in format or width");
    }
    if (((uintptr_t)a.x % 16) != 0) return fail(WGB_ERR_UNSUPPORTED, "input vector is not 16-byte aligned");
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
    qmat_set_pitches(m);
    m.p[0] = (const uint8_t *)d_blocks;
    return gemv_dispatch(m, d_v, d_out, as_stream(stream));
}
