// Matrix-vector kernels: the fused, TMA-fed kernel used by the models and by GemvQuant, and the
// generic per-format fallback.
//
// Fused kernel.  One persistent block per SM with three roles: eighteen consumer warps, a producer
// warp and an epilogue warp.
//   * Rows are taken in groups of `rs` (1..8) that lie contiguously in HBM.  The producer streams
//     group after group into a ring of shared-memory stages with one bulk asynchronous copy
//     (cp.async.bulk, completion on an mbarrier) per plane of the group, running as many stages
//     ahead as the ring holds and handling several stages per pass, one per group of lanes.  It
//     starts before the kernel waits for its predecessor in the stream (programmatic dependent
//     launch): weights never depend on activations.
//   * The consumers build the shared image of the (normalised) input vector once.  Consumer warp w
//     owns column part w % kp of the matrix for the whole kernel, so its share of the input stays in
//     registers; the warps of one column part form ncl = 18 / kp "lanes" that take the (stage, row
//     part) tasks of the block in turn.  A task is `rrows` rows of one stage: the warp computes the
//     partial dot products (the loop over rows fully unrolled, so that the loads of later rows overlap
//     the arithmetic of earlier ones), folds them across its lanes with a transposing butterfly (9
//     shuffles for up to 8 rows), writes them to shared memory and arrives on the stage's `done`
//     barrier.  Consumers never wait for each other or for the epilogue.
//   * The epilogue warp waits for `done`, adds the column parts of every row in a fixed order,
//     releases the stage to the producer and applies the epilogue (bias, residual, SiLU gate, GELU,
//     RoPE + KV-cache append), one lane per output unit.  Its global loads (bias, residual, position)
//     are issued before the wait, so they overlap the consumers' work on the stage.
//   * Group g belongs to block g % gridDim.x, so every SM gets the same number of groups to within
//     one; rs and the row split are chosen per launch (see plan()).
// Every mbarrier wait is bounded: after ~2^22 polls a waiter records an error code in the launch's
// status word and carries on with whatever is in shared memory, so the kernel always terminates.
#include "async_copy.cuh"
#include "gemv_core.cuh"
#include "kernels.h"
#include "qaccess.cuh"

#include <cstdio>
#include <cstdlib>
#include <type_traits>

namespace wgb {

// Consumer warps per block.  Registers are allocated per scheduler partition (a quarter of the register file
// each, warps dealt round-robin): 18 consumers + producer + epilogue = 20 warps put five warps on every
// partition, which leaves 96 registers per thread -- the same as 17 to 19 warps would -- so 18 is the most
// consumers that budget buys.
#ifndef WGB_GEMV_NCONS
#define WGB_GEMV_NCONS 16
#endif
constexpr int GEMV_NCONS = WGB_GEMV_NCONS;
constexpr int GEMV_CONS_THREADS = GEMV_NCONS * 32;
constexpr int GEMV_PRODUCER = GEMV_NCONS;           // warp index of the producer
constexpr int GEMV_EPILOGUE = GEMV_NCONS + 1;       // warp index of the epilogue warp
constexpr int GEMV_NT = (GEMV_EPILOGUE + 1) * 32;
constexpr int GEMV_MAX_RS = 8;                      // rows per stage
constexpr int GEMV_TASK_ROWS = 4;                   // rows per consumer task, at most
constexpr int GEMV_MAX_STAGES = 24;
constexpr uint32_t GEMV_ROPE_TAB = 128;             // pair indices with a precomputed rotation
constexpr size_t GEMV_SMEM_BUDGET = 200 * 1024;     // dynamic shared memory per block

__device__ __forceinline__ float4 ld_act4(const float *p)
{
    return __ldcg(reinterpret_cast<const float4 *>(p));
}

__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GEMV_CONS_THREADS) : "memory"); }

// Sum over the consumer threads (named barrier 1); every consumer gets the result.
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

// Sums acc[0..8) over the lanes of the warp.  Lane l returns the total of row
// 4 * bit4(l) + 2 * bit3(l) + bit2(l); the four lanes that share bits 2..4 hold the same value.
__device__ __forceinline__ float warp_sum8(const float (&acc)[8], int lane)
{
    float a4[4], a2[2];
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float keep = h16 ? acc[i + 4] : acc[i], send = h16 ? acc[i] : acc[i + 4];
        a4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const float keep = h8 ? a4[i + 2] : a4[i], send = h8 ? a4[i] : a4[i + 2];
        a2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const float keep = h4 ? a2[1] : a2[0], send = h4 ? a2[0] : a2[1];
    float v = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

// The same for R = 4, 2, 1 rows: the total of row r ends up in the lanes whose top log2(R) bits spell r.
template <int R>
__device__ __forceinline__ float warp_sum_rows(const float (&acc)[R], int lane)
{
    static_assert(R == 1 || R == 2 || R == 4 || R == 8, "rows per task");
    if constexpr (R == 8) {
        return warp_sum8(acc, lane);
    } else if constexpr (R == 4) {
        const bool h16 = lane & 16, h8 = lane & 8;
        float a2[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const float keep = h16 ? acc[i + 2] : acc[i], send = h16 ? acc[i] : acc[i + 2];
            a2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
        const float keep = h8 ? a2[1] : a2[0], send = h8 ? a2[0] : a2[1];
        float v = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        return v;
    } else if constexpr (R == 2) {
        const bool h16 = lane & 16;
        float v = (h16 ? acc[1] : acc[0]) + __shfl_xor_sync(0xffffffffu, h16 ? acc[0] : acc[1], 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    } else {
        return warp_sum(acc[0]);
    }
}

// Stages per pass of the epilogue warp and of the producer warp.  The lanes of a warp may be held at a
// reconvergence point until all of them have left their wait, so a pass must be assumed to finish only
// when every stage in it has: the epilogue pass that frees a slot must never contain a stage whose copy
// the producer can only issue in a pass that needs that very slot.  epilogue_batch + producer_batch <=
// nstage + 1 rules the cycle out; the producer also leaves half of the ring queued while it waits.
__host__ __device__ inline uint32_t epilogue_batch(uint32_t nstage) { return nstage >= 8 ? 4u : (nstage >= 4 ? 2u : 1u); }
__host__ __device__ inline uint32_t producer_batch(uint32_t nstage, uint32_t copies_per_stage)
{
    uint32_t b = nstage / 2;
    if (b > 32 / copies_per_stage) b = 32 / copies_per_stage;
    return b < 1 ? 1 : b;
}

// ---- groups ------------------------------------------------------------------------------------
struct Part {
    int mat;
    uint32_t row0;
};

// Parts (1 or 2 runs of `n` consecutive rows of one matrix) of group gi; returns the number of parts,
// 0 past the end.
__device__ __forceinline__ int group_parts(const GemvArgs &a, const int EPI, uint32_t gi, Part (&parts)[2], uint32_t &n)
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
        const uint32_t gq = a.gq, gk = a.gk;
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

// Output units of a group (a unit = the stage rows that make one output: a row, or a pair) and the
// stage rows of unit u.
__device__ __forceinline__ uint32_t group_units(const int EPI, const Part (&parts)[2], int nparts, uint32_t n)
{
    if (EPI == EPI_QKV_ROPE && nparts == 1 && parts[0].mat < 2) return n / 2;   // adjacent pairs
    return n;
}
__device__ __forceinline__ void unit_rows(const int EPI, const Part (&parts)[2], int nparts, uint32_t n, uint32_t u, uint32_t &ra, uint32_t &rb)
{
    if (EPI == EPI_SILU_PAIR || (EPI == EPI_QKV_ROPE && nparts == 2)) { ra = u; rb = n + u; }
    else if (EPI == EPI_QKV_ROPE && parts[0].mat < 2) { ra = 2 * u; rb = 2 * u + 1; }
    else { ra = u; rb = u; }
}

// What the epilogue of one output unit needs besides the dot products; gathered before the unit's
// sums are ready so that the global loads overlap the consumers' work.
struct EpiCtx {
    bool on;            // the lane has a unit
    uint32_t r0, r1;    // output rows of the unit (matrix row indices)
    uint32_t d0, d1;    // EPI_QKV_ROPE: their offsets from `dst`
    float b0, b1;       // bias of r0 / r1, or the residual in b1 for EPI_RESIDUAL
    float sn, cs;       // RoPE rotation
    float *dst;         // EPI_QKV_*: where the rows of the unit go
};

__device__ __forceinline__ EpiCtx epi_prepare(const GemvArgs &a, const int EPI, const Part (&parts)[2], int nparts, uint32_t n, uint32_t t,
                                              uint32_t nunits, const float2 *rope_tab)
{
    EpiCtx c = {};
    c.on = t < nunits;
    if (!c.on) return c;
    if (EPI == EPI_STORE || EPI == EPI_RESIDUAL || EPI == EPI_GELU) {
        c.r0 = parts[0].row0 + t;
        if (a.bias) c.b0 = a.bias[c.r0];
        if (EPI == EPI_RESIDUAL) c.b1 = a.residual[c.r0];
    } else if (EPI == EPI_SILU_PAIR) {
        c.r0 = parts[0].row0 + t;
    } else if (EPI == EPI_QKV_ROPE) {
        const int s = parts[0].mat;
        const float *bias = s == 0 ? a.bias : (s == 1 ? a.bias_k : a.bias_v);
        const uint32_t pos = *a.pos;
        const uint32_t rstr = a.kv_row_stride ? a.kv_row_stride : a.kv_dim;
        c.dst = s == 0 ? a.out : ((s == 1 ? a.k_cache : a.v_cache) + (size_t)pos * rstr);
        if (s == 2) {
            c.r0 = c.r1 = parts[0].row0 + t;
        } else if (nparts == 2) {   // Neox: pairs (r0 + t, r0 + t + head_size / 2)
            c.r0 = parts[0].row0 + t;
            c.r1 = parts[1].row0 + t;
        } else {                    // Original: adjacent pairs
            c.r0 = parts[0].row0 + 2 * t;
            c.r1 = c.r0 + 1;
        }
        // where rows r0 / r1 land: q as is, k / v by (head, element) in the cache's layout
        c.d0 = c.r0;
        c.d1 = c.r1;
        if (s != 0 && a.kv_row_stride) {
            c.d0 = (c.r0 / a.head_size) * a.kv_head_stride + c.r0 % a.head_size;
            c.d1 = (c.r1 / a.head_size) * a.kv_head_stride + c.r1 % a.head_size;
        }
        if (bias) {
            c.b0 = bias[c.r0];
            c.b1 = bias[c.r1];
        }
        if (s < 2) {
            // RoPE (ops/rope.wgsl:36-77): angle = pos * base^(-(2i % head_size) / head_size) for pair (r0, r1)
            const uint32_t half = a.head_size / 2;
            const uint32_t fi = (a.rope_variant == WGB_ROPE_NEOX) ? (c.r0 % a.head_size) : ((c.r0 / 2) % half);
            if (half <= GEMV_ROPE_TAB) {
                const float2 r = rope_tab[fi];
                c.cs = r.x;
                c.sn = r.y;
            } else {
                sincosf((float)pos * a.rope_freq[fi], &c.sn, &c.cs);
            }
        }
    } else if (EPI == EPI_QKV_SPLIT) {
        const uint32_t row = parts[0].row0 + t, d = a.kv_dim, pos = *a.pos;
        c.r0 = row;
        if (a.bias) c.b0 = a.bias[row];
        if (row < d) c.dst = a.out + row;
        else if (row < 2 * d) c.dst = a.k_cache + (size_t)pos * d + (row - d);
        else c.dst = a.v_cache + (size_t)pos * d + (row - 2 * d);
    }
    return c;
}

// ya / yb: finished dot products of the unit's first / second stage row.
__device__ __forceinline__ void epi_finish(const GemvArgs &a, const int EPI, const Part (&parts)[2], const EpiCtx &c, float ya, float yb)
{
    if (!c.on) return;
    if (EPI == EPI_STORE || EPI == EPI_RESIDUAL || EPI == EPI_GELU) {
        float y = ya;
        if (a.bias) y += c.b0;
        if (EPI == EPI_RESIDUAL) y = c.b1 + y;
        if (EPI == EPI_GELU) y = gelu_f32(y);
        if ((EPI == EPI_STORE || EPI == EPI_RESIDUAL) && a.peer_out.n) {
            for (uint32_t p = 0; p < a.peer_out.n; p++) a.peer_out.mail[p][c.r0] = y;   // every rank's mailbox, own included
        } else {
            a.out[c.r0] = y;
        }
    } else if (EPI == EPI_SILU_PAIR) {
        a.out[c.r0] = yb * (ya / (1.0f + expf(-ya)));
    } else if (EPI == EPI_QKV_ROPE) {
        if (parts[0].mat == 2) {
            c.dst[c.d0] = ya + c.b0;
        } else {
            const float y0 = ya + c.b0, y1 = yb + c.b1;
            c.dst[c.d0] = c.cs * y0 - c.sn * y1;
            c.dst[c.d1] = c.sn * y0 + c.cs * y1;
        }
    } else if (EPI == EPI_QKV_SPLIT) {
        *c.dst = ya + c.b0;
    }
}

// One kernel per block format, prologue and epilogue.  The launches of a decode step alternate between
// kernels and evict one another's code from the instruction caches (measured: +0.7 us per launch when two
// kernels alternate, +1.7 us with four), so what matters is how little code one launch executes: a single
// kernel with the prologue and epilogue chosen at run time shares its hot loop between launches but was
// measured 13 % slower over a 7B decode step (more code per launch, a worse register allocation).
template <int QT, int PRO_T, int EPI_T>
__global__ void __launch_bounds__(GEMV_NT, 1) gemv_kernel(const __grid_constant__ GemvArgs a)
{
    using S = Step<QT>;
    constexpr int PRO = PRO_T, EPI = EPI_T;
    constexpr int NPL = QT == WGB_Q6_K ? 4 : (QT == WGB_Q8_0 ? 2 : 1);   // planes of the format
    extern __shared__ uint4 smem4[];
    __shared__ float red[32];
    __shared__ float part[GEMV_MAX_STAGES][GEMV_NCONS][GEMV_MAX_RS];    // [stage][column part][stage row]
    __shared__ __align__(16) float lane_part[GEMV_NCONS][GEMV_TASK_ROWS][32];   // [consumer warp][task row][lane]
    __shared__ __align__(8) unsigned long long bars[3 * GEMV_MAX_STAGES];
    __shared__ float2 rope_tab[GEMV_ROPE_TAB];     // (cos, sin) per pair index of a head (EPI_QKV_ROPE)

    const uint32_t K = a.mat[0].ncols;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t nstage = a.nstage;
    uint8_t *smem = reinterpret_cast<uint8_t *>(smem4);
    const uint32_t ring = smem_addr(smem + a.ring_offset);
    const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[GEMV_MAX_STAGES]),
                   done0 = smem_addr(&bars[2 * GEMV_MAX_STAGES]);
    const uint32_t kp = a.kparts, rparts = a.rparts;

    // one thread per barrier: initialising them one after the other would cost a microsecond
    if (threadIdx.x < 3 * nstage) {
        const uint32_t kind = threadIdx.x / nstage, s = threadIdx.x - kind * nstage;
        mbar_init((kind == 0 ? full0 : (kind == 1 ? empty0 : done0)) + 8 * s, kind == 2 ? kp * rparts : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    const uint32_t row_bytes = a.row_bytes;
    // stages of this block (the grid never exceeds the number of groups)
    const uint32_t nst = a.per_block - ((a.rem_blocks != 0 && blockIdx.x >= a.rem_blocks) ? 1u : 0u);

    if (warp == GEMV_PRODUCER) {
        // ------------------------------ producer ------------------------------
        // Waiting for a free slot, arming its barrier and issuing a copy is a dependent chain of several
        // hundred cycles, so the warp runs it for several stages at once: the lanes form groups of `cps`
        // (copies per stage), one group per stage of a pass; the first lane of a group waits and arms,
        // every lane issues one copy.
        const uint32_t nplanes = (uint32_t)NPL;
        const uint32_t cps = 1u << a.cps_log2;                   // copies per stage: 1, 2, 4 or 8
        const uint32_t spb = a.spb;                              // stages per pass
        const uint32_t sb = (uint32_t)lane >> a.cps_log2, ci = (uint32_t)lane & (cps - 1);
        const uint32_t gmask = ((1u << cps) - 1u) << (sb * cps);
        if (sb >= spb) return;
        uint32_t s = sb % nstage, round = sb / nstage;           // ring slot of stage `it` and its use count
        for (uint32_t it = sb; it < nst; it += spb) {
            Part parts[2];
            uint32_t n = 0;
            const int nparts = group_parts(a, EPI, blockIdx.x + it * gridDim.x, parts, n);
            if (ci == 0) {
                if (round) mbar_wait(empty0 + 8 * s, (round - 1) & 1, a.err, 2, a.wait_ns);
                mbar_expect_tx(full0 + 8 * s, nparts * n * row_bytes);
            }
            __syncwarp(gmask);
            if (ci < (uint32_t)nparts * nplanes) {
                const uint32_t pi = ci / nplanes, pl = ci % nplanes;   // nplanes is a compile-time power of two
                // a stage holds plane after plane; within a plane, the rows of part 0 then those of part 1
                const QMat &m = a.mat[parts[pi].mat];
                uint32_t off = pi * n * m.pitch[pl];
                for (uint32_t q = 0; q < pl; q++) off += (uint32_t)nparts * n * m.pitch[q];
                bulk_copy_g2s(ring + s * a.stage_bytes + off, m.p[pl] + (size_t)parts[pi].row0 * m.pitch[pl], n * m.pitch[pl],
                              full0 + 8 * s);
            }
            s += spb;
            while (s >= nstage) { s -= nstage; round++; }
        }
        return;
    }

    if (warp == GEMV_EPILOGUE) {
        // ------------------------------ epilogue ------------------------------
        // Up to four stages per pass: lanes 8k..8k+7 take stage it0 + k, one lane per output unit.
        pdl_wait();
        if (EPI == EPI_QKV_ROPE) {
            // rotation of every pair index of a head at this position (ops/rope.wgsl:36-77)
            const uint32_t half = a.head_size / 2;
            if (half <= GEMV_ROPE_TAB) {
                const float pos = (float)*a.pos;
                for (uint32_t i = lane; i < half; i += 32) {
                    float sn, cs;
                    sincosf(pos * a.rope_freq[i], &sn, &cs);
                    rope_tab[i] = make_float2(cs, sn);
                }
            }
            __syncwarp();
        }
        const uint32_t nb = epilogue_batch(nstage);
        const uint32_t sub = (uint32_t)lane >> 3, ul = (uint32_t)lane & 7;
        const uint32_t gmask = 0xffu << (8 * sub);
        uint32_t s = sub % nstage, phase = (sub / nstage) & 1;   // ring slot and parity of stage it0 + sub
        float rms_scale = 1.0f;
        bool have_scale = false;
        for (uint32_t it0 = 0; it0 < nst; it0 += nb, s += nb) {
            while (s >= nstage) {
                s -= nstage;
                phase ^= 1;
            }
            const uint32_t it = it0 + sub;
            if (sub >= nb || it >= nst) continue;
            Part parts[2];
            uint32_t n = 0;
            const int nparts = group_parts(a, EPI, blockIdx.x + it * gridDim.x, parts, n);
            const uint32_t nunits = group_units(EPI, parts, nparts, n);
            const EpiCtx c = epi_prepare(a, EPI, parts, nparts, n, ul, nunits, rope_tab);
            uint32_t ra = 0, rb = 0;
            if (c.on) unit_rows(EPI, parts, nparts, n, ul, ra, rb);
            mbar_wait(done0 + 8 * s, phase, a.err, 3, a.wait_ns);
            if (PRO == PRO_RMS && !have_scale) {
                // every consumer warp wrote its sum of squares before its first arrival on a `done` barrier
                float ss = 0.0f;
#pragma unroll
                for (int w = 0; w < GEMV_NCONS; w++) ss += red[w];
                rms_scale = 1.0f / sqrtf(ss / (float)K + a.eps);
                have_scale = true;
            }
            float ya = 0.0f, yb = 0.0f;
            if (c.on) {
                for (uint32_t k = 0; k < kp; k++) {
                    ya += part[s][k][ra];
                    yb += part[s][k][rb];
                }
                if (PRO == PRO_RMS) {
                    ya *= rms_scale;
                    yb *= rms_scale;
                }
            }
            __syncwarp(gmask);
            if (ul == 0) mbar_arrive(empty0 + 8 * s);   // stage and partial sums may be overwritten
            epi_finish(a, EPI, parts, c, ya, yb);
        }
        if ((EPI == EPI_STORE || EPI == EPI_RESIDUAL) && a.peer_out.n) {
            // The block's partial rows are on their way to the peers; the last block of the launch raises
            // this rank's flag everywhere once every block's stores are visible system-wide.
            __threadfence_system();
            __syncwarp();
            uint32_t last = 0;
            if (lane == 0) {
                const uint32_t t = atomicAdd(a.peer_out.ticket, 1u);
                last = (t == gridDim.x - 1);
                if (last) *a.peer_out.ticket = 0;   // ready for the next step
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence_system();
                if ((uint32_t)lane < a.peer_out.n) atomicAdd_system(a.peer_out.flag[lane], 1u);
            }
        }
        if (lane == 0) stamp_end(a.stamp);
        return;
    }

    // ------------------------------ consumers ------------------------------
    // What the task loop needs and the input does not decide is worked out while the launch before drains.
    const uint32_t ncl = GEMV_NCONS / kp;                 // "lanes" of warps per column part
    const XImage im = ximage_carve(QT, K, smem);
    const uint32_t kunits = QT == WGB_F32 ? K : a.mat[0].bpr;   // what Step::active() compares against
    const uint32_t nsteps = (K + step_cols<QT>() - 1) / step_cols<QT>();
    const uint32_t kw = (uint32_t)warp % kp, cl = (uint32_t)warp / kp;
    // The norm weights are parameters, not products of the launch before: their (cold, HBM-latency) loads
    // are issued ahead of the dependency wait and are in registers by the time the input can be read.
    // A thread owns units of eight consecutive inputs (two float4 chunks), u = threadIdx.x + i * GEMV_CONS_THREADS;
    // the first XU of them live in registers from one round of loads to the staging: all of them up to 8192
    // columns, up to 12288 where the kernel has no norm parameters to hold.
    constexpr uint32_t XU = PRO_T == PRO_NONE ? 3 : 2, WU = PRO_T == PRO_NONE ? 1 : 2;
    const uint32_t nchunk = K / 4, nunit = (nchunk + 1) / 2;
    float4 wc[2 * WU], bc[2 * WU];
    if (PRO != PRO_NONE) {
#pragma unroll
        for (uint32_t i = 0; i < WU; i++) {
            const uint32_t c = 2 * (threadIdx.x + i * GEMV_CONS_THREADS);
#pragma unroll
            for (uint32_t h = 0; h < 2; h++) {
                if (c + h < nchunk) {
                    wc[2 * i + h] = __ldg(reinterpret_cast<const float4 *>(a.norm_w) + c + h);
                    if (PRO == PRO_LN) bc[2 * i + h] = __ldg(reinterpret_cast<const float4 *>(a.norm_b) + c + h);
                }
            }
        }
    }
    pdl_wait();
    float4 xc[2 * XU];
    const bool gather = PRO == PRO_RMS && a.peer_in.n != 0;
    if (gather) {
        // Partial products from every rank: wait for the flags, then add in rank order.  The wait is bounded
        // in time (a.peer_wait_ns); a wait that runs out leaves code 6 in the status word, and while the word
        // is non-zero no launch waits at all, so one missing rank costs one limit, not one per exchange.
        if (threadIdx.x < a.peer_in.n) {
            const uint32_t want = __ldcg(a.peer_in.epoch);
            const uint32_t *f = a.peer_in.flag + threadIdx.x;
            bool ok = false, give_up = a.err && ld_relaxed_u32(a.err) != 0;
            unsigned long long t0 = 0;
            for (uint32_t i = 0; !ok && !give_up; i++) {
                uint32_t v;
                asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                ok = (int32_t)(v - want) >= 0;
                if (!ok && (i & 31u) == 31u) {
                    const unsigned long long t = global_ns();
                    if (!t0) t0 = t;
                    give_up = t - t0 > a.peer_wait_ns || (a.err && ld_relaxed_u32(a.err) != 0);
                }
            }
            if (!ok && a.err) atomicCAS(a.err, 0u, 6u);
            asm volatile("fence.acq_rel.sys;" ::: "memory");
        }
        cons_sync();
    }
    auto load_chunk = [&](uint32_t c) {
        if (!gather) return ld_act4(a.x + 4 * c);
        float4 v = __ldcg(reinterpret_cast<const float4 *>(a.peer_in.mail) + c);
        for (uint32_t r = 1; r < a.peer_in.n; r++) {
            const float4 w = __ldcg(reinterpret_cast<const float4 *>(a.peer_in.mail + (size_t)r * K) + c);
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        if (blockIdx.x == 0) reinterpret_cast<float4 *>(a.peer_in.x_out)[c] = v;
        return v;
    };
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (uint32_t i = 0; i < XU; i++) {
        const uint32_t c = 2 * (threadIdx.x + i * GEMV_CONS_THREADS);
        xc[2 * i] = c < nchunk ? load_chunk(c) : zero4;
        xc[2 * i + 1] = c + 1 < nchunk ? load_chunk(c + 1) : zero4;
    }
    // Units past the ones held in registers (longer rows) are read again where needed.
    const uint32_t u_tail = threadIdx.x + XU * GEMV_CONS_THREADS;
    float mean = 0.0f, scale = 1.0f;
    if (PRO == PRO_RMS) {
        float ss = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < 2 * XU; i++) ss += xc[i].x * xc[i].x + xc[i].y * xc[i].y + xc[i].z * xc[i].z + xc[i].w * xc[i].w;
        for (uint32_t u = u_tail; u < nunit; u += GEMV_CONS_THREADS) {
            for (uint32_t c = 2 * u; c < min(2 * u + 2, nchunk); c++) {
                const float4 v = load_chunk(c);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        // The scale is one factor for the whole vector, so it commutes with the dot products: the input is
        // staged as x * w, the warps' sums of squares go to `red`, and the epilogue warp multiplies every
        // finished dot product by 1 / sqrt(mean square + eps).  No block-wide reduction ahead of the staging.
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
    } else if (PRO == PRO_LN) {
        float sm = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < 2 * XU; i++) sm += (xc[i].x + xc[i].y) + (xc[i].z + xc[i].w);   // chunks past the end are zero
        for (uint32_t u = u_tail; u < nunit; u += GEMV_CONS_THREADS) {
            for (uint32_t c = 2 * u; c < min(2 * u + 2, nchunk); c++) {
                const float4 v = load_chunk(c);
                sm += (v.x + v.y) + (v.z + v.w);
            }
        }
        mean = cons_sum(sm, red) / (float)K;
        float ss = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < 2 * XU; i++) {
            if (2 * (threadIdx.x + (i / 2) * GEMV_CONS_THREADS) + (i & 1) < nchunk) {
                const float dx = xc[i].x - mean, dy = xc[i].y - mean, dz = xc[i].z - mean, dw = xc[i].w - mean;
                ss += dx * dx + dy * dy + dz * dz + dw * dw;
            }
        }
        for (uint32_t u = u_tail; u < nunit; u += GEMV_CONS_THREADS) {
            for (uint32_t c = 2 * u; c < min(2 * u + 2, nchunk); c++) {
                float4 v = load_chunk(c);
                v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        ss = cons_sum(ss, red);
        scale = 1.0f / sqrtf(ss / (float)K + 1.0e-5f);
    }
    {
        const XWriter<QT> xw(smem, K);
        auto transform = [&](float4 v, const float4 w, const float4 b) {
            if (PRO == PRO_RMS) {
                v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
            } else if (PRO == PRO_LN) {
                v.x = ((v.x - mean) * scale) * w.x + b.x; v.y = ((v.y - mean) * scale) * w.y + b.y;
                v.z = ((v.z - mean) * scale) * w.z + b.z; v.w = ((v.w - mean) * scale) * w.w + b.w;
            }
            return v;
        };
        auto param = [&](const float *p, uint32_t c, bool in) {
            return in ? __ldg(reinterpret_cast<const float4 *>(p) + c) : zero4;
        };
        // whole warps go round together (the writer shuffles): the bound is per warp, not per lane
        const uint32_t warp_u0 = (uint32_t)warp * 32;
#pragma unroll
        for (uint32_t i = 0; i < XU; i++) {
            if (warp_u0 + i * GEMV_CONS_THREADS < nunit) {
                const uint32_t u = threadIdx.x + i * GEMV_CONS_THREADS, c = 2 * u;
                const bool in = c < nchunk, inb = c + 1 < nchunk;
                float4 w0 = zero4, w1 = zero4, b0 = zero4, b1 = zero4;
                if (i < WU) {
                    w0 = wc[2 * i]; w1 = wc[2 * i + 1];
                    b0 = bc[2 * i]; b1 = bc[2 * i + 1];
                } else if (PRO != PRO_NONE) {
                    w0 = param(a.norm_w, c, in); w1 = param(a.norm_w, c + 1, inb);
                    if (PRO == PRO_LN) { b0 = param(a.norm_b, c, in); b1 = param(a.norm_b, c + 1, inb); }
                }
                xw.put8(u, transform(xc[2 * i], w0, b0), transform(xc[2 * i + 1], w1, b1), in, inb);
            }
        }
        for (uint32_t u0 = warp_u0 + XU * GEMV_CONS_THREADS; u0 < nunit; u0 += GEMV_CONS_THREADS) {
            const uint32_t u = u0 + lane, c = 2 * u;
            const bool in = c < nchunk, inb = c + 1 < nchunk;
            float4 va = zero4, vb = zero4, w0 = zero4, w1 = zero4, b0 = zero4, b1 = zero4;
            if (in) va = load_chunk(c);
            if (inb) vb = load_chunk(c + 1);
            if (PRO != PRO_NONE) { w0 = param(a.norm_w, c, in); w1 = param(a.norm_w, c + 1, inb); }
            if (PRO == PRO_LN) { b0 = param(a.norm_b, c, in); b1 = param(a.norm_b, c + 1, inb); }
            xw.put8(u, transform(va, w0, b0), transform(vb, w1, b1), in, inb);
        }
    }
    cons_sync();

    if ((uint32_t)warp >= kp * ncl) return;               // warps left over when kp does not divide the consumers
    typename S::X x;
    // prefix[q]: bytes of planes 0..q-1 of one row (a stage holds plane after plane, see the producer)
    uint32_t prefix[NPL];
    {
        uint32_t acc = 0;
#pragma unroll
        for (int q = 0; q < NPL; q++) {
            prefix[q] = acc;
            acc += a.mat[0].pitch[q];
        }
    }

    // Task loop.  A task is up to GEMV_TASK_ROWS rows of one stage, taken one at a time by a rolled loop whose
    // body -- one call of the format's dot product -- is the whole hot path of the kernel: two kilobytes of
    // code that every warp of the block shares in the instruction caches.  (Unrolled over the rows the loop ran
    // with "no instruction" as its first stall reason, and the launches of a decode step evict one another's
    // code, so whatever a launch executes it first has to fetch.)  Nothing in the body depends on the lane:
    // a lane past the end of the row works on the row's first unit with an all-zero input instead of sitting
    // out.  Each lane leaves its partial sum of a row in shared memory; after the last row the warp adds the
    // 32 partials of every row: lane l takes four partials of row l / 8, three butterfly steps do the rest.
    // For every shape the models use the matrix has no more column steps than there are consumer warps, so the
    // loop over steps makes one trip and the warp's part of the input is loaded once per kernel.
    constexpr int R = GEMV_TASK_ROWS;
    static_assert(R == 4, "the reduction below reads four partials per lane of four rows");
    const uint32_t Rn = a.rrows;
    float *my_part = &lane_part[warp][0][0];
    uint32_t held = ~0u;   // column step whose part of the input is in `x`
    int lane_d = lane;
    uint32_t s = 0, phase = 0, it_prev = 0;
    for (uint32_t t = cl; t < nst * rparts; t += ncl) {
        const uint32_t it = t >> a.rparts_log2, rp = t & (rparts - 1);
        s += it - it_prev;
        it_prev = it;
        while (s >= nstage) {
            s -= nstage;
            phase ^= 1;
        }
        uint32_t nrows = a.rs;   // rows in this stage: fewer only in the last group of a matrix
        if (EPI != EPI_QKV_ROPE) {
            Part parts[2];
            uint32_t n = 0;
            const int nparts = group_parts(a, EPI, blockIdx.x + it * gridDim.x, parts, n);
            nrows = nparts * n;
        }
        const uint32_t j0 = rp * Rn;
        const uint32_t jn = min(Rn, nrows > j0 ? nrows - j0 : 0u);
        const uint32_t stage = ring + s * a.stage_bytes;
        mbar_wait(full0 + 8 * s, phase, a.err, 1, a.wait_ns);
        for (uint32_t ks = kw; ks < nsteps; ks += kp) {
            const uint32_t col0 = ks * step_cols<QT>();
            if (held != ks) {
                const bool on = S::active(kunits, col0, lane);
                lane_d = on ? lane : S::lane0(lane);
                if (on) S::load_x(x, im, col0, lane);
                else zero_x(x);
                held = ks;
            }
            uint32_t r[4];
#pragma unroll
            for (int q = 0; q < NPL; q++) r[q] = stage + nrows * prefix[q] + j0 * a.mat[0].pitch[q];
            const bool first = ks == kw;
#pragma unroll 1
            for (uint32_t j = 0; j < jn; j++) {
                float v = S::dot(r, col0, x, lane_d);
                if (!first) v += my_part[j * 32 + lane];
                my_part[j * 32 + lane] = v;
#pragma unroll
                for (int q = 0; q < NPL; q++) r[q] += a.mat[0].pitch[q];
            }
        }
        __syncwarp();
        const float4 p4 = reinterpret_cast<const float4 *>(my_part)[lane];   // partials 4 (l % 8) .. + 3 of row l / 8
        float v = (p4.x + p4.y) + (p4.z + p4.w);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        if ((lane & 7) == 0 && (uint32_t)(lane >> 3) < jn) part[s][kw][j0 + (lane >> 3)] = v;
        __syncwarp();
        if (lane == 0) mbar_arrive(done0 + 8 * s);
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

// Device status word shared by all launches on one device: 0, or the code of the first bounded wait that
// expired (1 consumer, 2 producer, 3 epilogue, 6 flags of the tensor-parallel peers, 7 / 8 streaming
// attention, 16+ tensor-memory kernel).  While it is non-zero the kernels do not wait for peers at all.
static bool g_trace_plan = false;   // WGML_B200_TRACE_PLAN=1 prints the plan of every launch to stderr

uint32_t *gemv_status_word()
{
    DeviceState *d = device_state();
    return d ? d->err : nullptr;
}

int gemv_report_status(uint32_t v)
{
    if (!v) return WGB_OK;
    uint32_t *w = gemv_status_word();
    if (w) cudaMemset(w, 0, sizeof(uint32_t));
    return fail(WGB_ERR_TIMEOUT, "a bounded wait inside a kernel expired (code %u%s)", v,
                v == 6 ? ": a rank of the tensor-parallel group did not deliver its partial products in time" : "");
}

int gemv_check_status()
{
    uint32_t *w = gemv_status_word();
    if (!w) return WGB_OK;
    uint32_t v = 0;
    WGB_CUDA(cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost));
    return gemv_report_status(v);
}

int replay_with_status(cudaGraphExec_t graph, size_t total, cudaStream_t stream, uint32_t *h_slots, StatusPoll &sp)
{
    uint32_t *word = gemv_status_word();
    for (int k = 0; k < 2; k++)
        if (!sp.ev[k]) WGB_CUDA(cudaEventCreateWithFlags(&sp.ev[k], cudaEventDisableTiming));
    h_slots[0] = h_slots[1] = 0;
    uint32_t seen = 0;
    for (size_t i = 0; i < total && !seen; i++) {
        if (word && i && i % STATUS_EVERY == 0) {
            const int k = (int)((i / STATUS_EVERY) & 1);
            if (i >= 2 * STATUS_EVERY) {
                WGB_CUDA(cudaEventSynchronize(sp.ev[k]));
                seen = h_slots[k];
                if (seen) break;
            }
            WGB_CUDA(cudaMemcpyAsync(h_slots + k, word, 4, cudaMemcpyDeviceToHost, stream));
            WGB_CUDA(cudaEventRecord(sp.ev[k], stream));
        }
        WGB_CUDA(cudaGraphLaunch(graph, stream));
    }
    if (seen) {
        WGB_CUDA(cudaStreamSynchronize(stream));
        return gemv_report_status(seen);
    }
    return WGB_OK;
}

void status_poll_destroy(StatusPoll &sp)
{
    for (int k = 0; k < 2; k++) {
        if (sp.ev[k]) cudaEventDestroy(sp.ev[k]);
        sp.ev[k] = nullptr;
    }
}

static uint32_t steps_of(int qt, uint32_t K)
{
    const uint32_t sc = qt == WGB_Q4_K ? step_cols<WGB_Q4_K>() : qt == WGB_Q6_K ? step_cols<WGB_Q6_K>()
                      : qt == WGB_Q8_0 ? step_cols<WGB_Q8_0>() : step_cols<WGB_F32>();
    return (K + sc - 1) / sc;
}

// Chooses rows per stage, the row split, ring depth and grid; fills the plan fields of `a`.  Returns
// false when the shapes do not fit the kernel's assumptions.
//
// Candidates are (rs rows per stage, rparts row parts per stage); a consumer task is rrows = rs / rparts
// rows of one column part, and the ncl = 18 / kparts warps of a column part take the tasks of the block
// in turn.  The time of the launch is that of its fullest block: ceil(tasks / ncl) rounds of
// (rrows + 1/2) row products, the half row standing for the wait, reduction and hand-off of a task.
// That is divided by how much of the ~80 KB per SM that must be in flight to cover HBM latency at full
// bandwidth the ring can hold beyond the stages the consumers are working on, and by a mild preference
// for larger copies.
static bool plan(GemvArgs &a, size_t &smem_bytes, uint32_t &grid)
{
    const QMat &m0 = a.mat[0];
    uint32_t row_bytes = 0;
    for (int i = 0; i < m0.nplanes; i++) row_bytes += m0.pitch[i];
    const uint32_t sms = (uint32_t)sm_count();
    uint32_t total_rows = 0;
    for (int i = 0; i < a.nmat; i++) total_rows += a.mat[i].nrows;
    const bool pairs = a.epilogue == EPI_SILU_PAIR || a.epilogue == EPI_QKV_ROPE;
    const size_t image = (ximage_bytes(m0.qtype, m0.ncols) + 127) & ~(size_t)127;
    if (image + 256 > GEMV_SMEM_BUDGET) return false;
    const uint32_t nsteps = steps_of(m0.qtype, m0.ncols);
    const uint32_t kp = nsteps < (uint32_t)GEMV_NCONS ? nsteps : (uint32_t)GEMV_NCONS;
    const uint32_t ncl = GEMV_NCONS / kp;
    const double want_in_flight = 80.0 * 1024;

    auto groups_of = [&](uint32_t rs) -> uint32_t {
        if (a.epilogue == EPI_SILU_PAIR) return (m0.nrows + rs / 2 - 1) / (rs / 2);
        if (a.epilogue == EPI_QKV_ROPE) return total_rows / rs;
        return (m0.nrows + rs - 1) / rs;
    };

    uint32_t best_rs = 0, best_rp = 0, best_ns = 0;
    double best_cost = 1e300;
    for (uint32_t rs = GEMV_MAX_RS; rs >= 1; rs--) {
        if (pairs && (rs & 1)) continue;
        const size_t stage = ((size_t)rs * row_bytes + 127) & ~(size_t)127;
        if (image + 2 * stage > GEMV_SMEM_BUDGET && rs > (pairs ? 2u : 1u)) continue;
        if (image + stage > GEMV_SMEM_BUDGET) continue;
        if (a.epilogue == EPI_QKV_ROPE) {
            bool ok = true;
            for (int i = 0; i < 3; i++) ok = ok && a.mat[i].nrows % rs == 0;
            if (a.rope_variant == WGB_ROPE_NEOX) ok = ok && (a.head_size / 2) % (rs / 2) == 0;
            if (!ok) continue;
        }
        const uint32_t groups = groups_of(rs);
        const uint32_t g = groups < sms ? groups : sms;
        const uint32_t per = (groups + g - 1) / g;
        uint32_t ns = (uint32_t)((GEMV_SMEM_BUDGET - image) / stage);
        if (ns > GEMV_MAX_STAGES) ns = GEMV_MAX_STAGES;
        if (ns > per) ns = per;
        for (uint32_t rparts = 1; rparts <= 8; rparts *= 2) {
            if (rs % rparts) continue;
            const uint32_t rrows = rs / rparts;
            if (rrows > (uint32_t)GEMV_TASK_ROWS) continue;
            const uint32_t in_work = (ncl + rparts - 1) / rparts + 1;   // stages the consumers hold at a time
            double flight;
            if (ns >= per) flight = 1.0;                                // the block's whole share fits in the ring
            else {
                const double bytes = ns > in_work ? (double)(ns - in_work) * stage : 0.25 * stage;
                flight = bytes >= want_in_flight ? 1.0 : bytes / want_in_flight;
            }
            const uint32_t rounds = (per * rparts + ncl - 1) / ncl;
            const double copy = (double)stage / ((double)stage + 512.0);
            const double cost = (double)rounds * ((double)rrows + 0.5) / (flight * copy);
            if (cost < best_cost - 1e-9) {
                best_cost = cost;
                best_rs = rs;
                best_rp = rparts;
                best_ns = ns;
            }
        }
    }
    if (!best_rs) return false;
    a.rs = best_rs;
    a.rparts = best_rp;
    a.rparts_log2 = best_rp == 1 ? 0 : (best_rp == 2 ? 1 : (best_rp == 4 ? 2 : 3));
    if (a.epilogue == EPI_QKV_ROPE) {
        a.gq = a.mat[0].nrows / best_rs;
        a.gk = a.mat[1].nrows / best_rs;
    }
    a.rrows = best_rs / best_rp;
    a.kparts = kp;
    a.ngroups = groups_of(best_rs);
    a.stage_bytes = (uint32_t)(((size_t)best_rs * row_bytes + 127) & ~(size_t)127);
    grid = a.ngroups < sms ? a.ngroups : sms;
    a.nstage = best_ns < 1 ? 1 : best_ns;
    a.ring_offset = (uint32_t)image;
    a.row_bytes = row_bytes;
    a.per_block = (a.ngroups + grid - 1) / grid;
    a.rem_blocks = a.ngroups % grid;
    const uint32_t cps = (uint32_t)m0.nplanes * (pairs ? 2u : 1u);
    a.cps_log2 = cps == 1 ? 0 : (cps == 2 ? 1 : (cps == 4 ? 2 : 3));
    // One producer pass takes about as long as 24 KB of streaming at full HBM rate: no more stages per
    // pass than that needs, so that the ring stays as full as possible.
    a.spb = (24576u + a.stage_bytes - 1) / a.stage_bytes;
    if (a.spb > producer_batch(a.nstage, cps)) a.spb = producer_batch(a.nstage, cps);
    smem_bytes = image + (size_t)a.nstage * a.stage_bytes;
    return true;
}

// The prologue / epilogue combinations the models use, each its own kernel.
#define WGB_GEMV_VARIANTS(F)                                                                                   \
    F(PRO_NONE, EPI_STORE) F(PRO_RMS, EPI_STORE) F(PRO_LN, EPI_STORE) F(PRO_NONE, EPI_RESIDUAL) F(PRO_RMS, EPI_SILU_PAIR) \
    F(PRO_LN, EPI_GELU) F(PRO_RMS, EPI_QKV_ROPE) F(PRO_LN, EPI_QKV_SPLIT)

template <int QT>
static int set_smem_attr()
{
#define WGB_ATTR(PRO, EPI) WGB_CUDA(cudaFuncSetAttribute(gemv_kernel<QT, PRO, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMV_SMEM_BUDGET));
    WGB_GEMV_VARIANTS(WGB_ATTR)
#undef WGB_ATTR
    return WGB_OK;
}

// One-time set-up of the fused kernels on the current device: the status word and the opt-in to
// large dynamic shared memory.  Must first run outside stream capture (model creation does).
int gemv_global_init()
{
    DeviceState *d = device_state();
    if (!d) return WGB_ERR_CUDA;
    if (d->gemv_attrs) return WGB_OK;
    if (!d->err) {
        WGB_CUDA(cudaMalloc((void **)&d->err, sizeof(uint32_t)));
        WGB_CUDA(cudaMemset(d->err, 0, sizeof(uint32_t)));
    }
    const char *tp = getenv("WGML_B200_TRACE_PLAN");
    g_trace_plan = tp && tp[0] == '1';
    int rc;
    if ((rc = set_smem_attr<WGB_Q4_K>()) || (rc = set_smem_attr<WGB_Q6_K>()) || (rc = set_smem_attr<WGB_Q8_0>()) ||
        (rc = set_smem_attr<WGB_F32>()))
        return rc;
    d->gemv_attrs = true;
    return WGB_OK;
}

template <int QT>
static int launch_one(GemvArgs &a, cudaStream_t stream, bool pdl)
{
    void (*kern)(const GemvArgs) = nullptr;
#define WGB_PICK(PRO, EPI) if (a.prologue == PRO && a.epilogue == EPI) kern = gemv_kernel<QT, PRO, EPI>;
    WGB_GEMV_VARIANTS(WGB_PICK)
#undef WGB_PICK
    if (!kern) return fail(WGB_ERR_UNSUPPORTED, "no fused kernel for prologue %d / epilogue %d", a.prologue, a.epilogue);
    size_t smem = 0;
    uint32_t grid = 0;
    if (!plan(a, smem, grid)) return fail(WGB_ERR_UNSUPPORTED, "matrix shape does not fit the fused kernel");
    int rc = gemv_global_init();
    if (rc) return rc;
    a.err = gemv_status_word();
    const WaitLimits wl = wait_limits();
    a.wait_ns = wl.local_ns;
    a.peer_wait_ns = wl.peer_ns;
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
    if (g_trace_plan)
        fprintf(stderr, "gemv plan: qt=%d rows=%u K=%u rs=%u rparts=%u kparts=%u ngroups=%u nstage=%u stage=%u grid=%u smem=%zu\n", QT,
                a.mat[0].nrows, a.mat[0].ncols, a.rs, a.rparts, a.kparts, a.ngroups, a.nstage, a.stage_bytes, grid, smem);
    WGB_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    return WGB_OK;
}

template <int QT>
static int launch_qt(GemvArgs &a, cudaStream_t stream, bool pdl)
{
    // the combinations the kernel is written for
    bool ok = false;
    switch (a.epilogue) {
    case EPI_STORE: ok = a.prologue == PRO_NONE || a.prologue == PRO_RMS || a.prologue == PRO_LN; break;
    case EPI_RESIDUAL: ok = a.prologue == PRO_NONE; break;
    case EPI_SILU_PAIR: ok = a.prologue == PRO_RMS && a.nmat == 2; break;
    case EPI_GELU: ok = a.prologue == PRO_LN; break;
    case EPI_QKV_ROPE: ok = a.prologue == PRO_RMS && a.nmat == 3; break;
    case EPI_QKV_SPLIT: ok = a.prologue == PRO_LN; break;
    }
    if (!ok) return fail(WGB_ERR_UNSUPPORTED, "no fused kernel for prologue %d / epilogue %d", a.prologue, a.epilogue);
    return launch_one<QT>(a, stream, pdl);
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

static int gemv_dispatch(const QMat &m, const float *d_v, float *d_out, cudaStream_t stream, bool early_weights)
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
        // Programmatic dependent launch: the kernel streams its first weights while the previous launch in the
        // stream is still draining, and waits for it (griddepcontrol.wait) before it reads d_v or writes d_out.
        // Only for matrices the library uploaded itself: blocks in caller memory may be the output of that
        // previous launch and must not be read before it has completed.
        return launch_gemv(a, stream, early_weights);
    }
    return launch_gemv_generic(m, d_v, d_out, stream);
}

WGB_EXPORT int wgb_gemv_quant(const wgb_quant_matrix *m, const float *d_v, float *d_out, void *stream)
{
    WGB_REQUIRE(m, "null matrix");
    return gemv_dispatch(m->view, d_v, d_out, as_stream(stream), m->storage != nullptr);
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
    return gemv_dispatch(m, d_v, d_out, as_stream(stream), false);
}
