// Warp-level quantised dot products: R matrix rows against one input vector held in shared
// memory.  These are the inner loops of every matrix-vector kernel of the library.
//
// A warp owns R rows and walks the K dimension in steps; in each step every lane owns a fixed
// slice of the columns (a run of codes that shares its sub-block scale), keeps the matching x
// values in registers and reuses them for all R rows.  Weight bytes are fetched with 128-bit
// loads straight from HBM (each byte is used once, so nothing is staged); x comes from shared
// memory through a bank-conflict-free swizzle.  Codes are unpacked in registers, accumulated in
// f32 and folded across the warp with shuffles.
//
// Algebra used instead of materialising every weight:
//   Q4_K  sum_l (d*sc*q_l - dmin*m) x_l = d*sc * sum_l q_l x_l  -  dmin*m * sum_l x_l
//   Q6_K  sum_l d*sc*(q_l - 32) x_l     = d*sc * (sum_l q_l x_l - 32 * sum_l x_l)
// with the per-16-column sums of x precomputed once per thread block.
#pragma once

#include "dequant.cuh"
#include "qmatrix.cuh"

namespace wgb {

__device__ __forceinline__ uint4 ldg_stream(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint2 ldg_stream8(const void *p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ uint16_t ldg_stream2(const void *p)
{
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// Byte k (0..3) of a word as float; unsigned and signed.
__device__ __forceinline__ float u8f(uint32_t w, int k) { return (float)((w >> (8 * k)) & 0xffu); }
__device__ __forceinline__ float s8f(uint32_t w, int k) { return (float)(int8_t)(w >> (8 * k)); }

// ---------------------------------------------------------------------------------------------
// Shared-memory image of the input vector.
//   xs   : K floats, stored in 16-byte chunks at swizzled positions (swz<QT>(chunk))
//   xsum : K/16 floats, sum of each run of 16 consecutive inputs
// The swizzle permutes chunks inside aligned groups of 8 so that the 8 lanes served together
// by one 128-bit shared load hit 8 different bank groups for the lane->column map of QT.
// ---------------------------------------------------------------------------------------------
template <int QT>
__device__ __forceinline__ uint32_t swz(uint32_t c)
{
    if (QT == WGB_Q4_K) return c ^ ((c >> 4) & 7u);
    if (QT == WGB_Q6_K) return c ^ (((c >> 6) & 1u) | (((c >> 5) & 1u) << 1));
    if (QT == WGB_Q8_0) return c ^ ((c >> 3) & 7u);
    return c;
}

template <int QT>
__device__ __forceinline__ float4 xs_chunk(const float *xs, uint32_t c)
{
    return reinterpret_cast<const float4 *>(xs)[swz<QT>(c)];
}

// Columns one warp step covers.
template <int QT>
__host__ __device__ constexpr uint32_t step_cols()
{
    return QT == WGB_Q4_K ? 2048u : QT == WGB_Q6_K ? 2048u : QT == WGB_Q8_0 ? 1024u : 128u;
}

// Whether a fast path exists for the format / layout.
__host__ __device__ constexpr bool has_fast_path(int qt)
{
    return qt == WGB_Q4_K || qt == WGB_Q6_K || qt == WGB_Q8_0 || qt == WGB_F32;
}

// ---------------------------------------------------------------------------------------------
// Per-format step: `Raw` holds one row's bytes for one step; load() issues the global loads,
// dot() consumes them.  `col0` is the first column of the step; lanes whose slice starts beyond
// K contribute nothing (their loads are skipped).
// ---------------------------------------------------------------------------------------------
template <int QT>
struct Step;

// Q4_K, raw 144-byte super-blocks: 4 lanes per super-block, lane g owns its 64-column group
// (32 bytes of qs: low nibbles = first 32 columns, high nibbles = next 32).
template <>
struct Step<WGB_Q4_K> {
    struct Raw { uint4 hdr, q0, q1; };
    struct X { float lo[32], hi[32]; float slo, shi; };

    __device__ static __forceinline__ bool active(const QMat &m, uint32_t col0, int lane)
    {
        return (col0 >> 8) + (lane >> 2) < m.bpr;
    }
    __device__ static __forceinline__ void load(Raw &r, const QMat &m, uint32_t row, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 8) + (lane >> 2), g = lane & 3;
        const uint8_t *blk = m.p0 + ((size_t)row * m.bpr + kb) * 144;
        r.hdr = ldg_stream(blk);
        r.q0 = ldg_stream(blk + 16 + g * 32);
        r.q1 = ldg_stream(blk + 32 + g * 32);
    }
    __device__ static __forceinline__ void load_x(X &x, const float *xs, const float *xsum, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 8) + (lane >> 2), g = lane & 3;
        const uint32_t c0 = kb * 64 + g * 16;
#pragma unroll
        for (int t = 0; t < 8; t++) {
            float4 a = xs_chunk<WGB_Q4_K>(xs, c0 + t), b = xs_chunk<WGB_Q4_K>(xs, c0 + 8 + t);
            x.lo[4 * t] = a.x; x.lo[4 * t + 1] = a.y; x.lo[4 * t + 2] = a.z; x.lo[4 * t + 3] = a.w;
            x.hi[4 * t] = b.x; x.hi[4 * t + 1] = b.y; x.hi[4 * t + 2] = b.z; x.hi[4 * t + 3] = b.w;
        }
        const float4 s = reinterpret_cast<const float4 *>(xsum)[kb * 4 + g];
        x.slo = s.x + s.y;
        x.shi = s.z + s.w;
    }
    __device__ static __forceinline__ float dot(const Raw &r, const X &x, int lane)
    {
        const uint32_t g = lane & 3;
        // Six-bit scale / min of sub-blocks 2g and 2g+1 (get_scale_min_k4, quantization.rs:381-389),
        // two at a time in the 16-bit halves of a word.
        const uint32_t sh = (g & 1) * 16;
        const uint32_t a = r.hdr.y >> sh, b = r.hdr.z >> sh, t = r.hdr.w >> sh;
        uint32_t sc16, m16;
        if (g < 2) {
            sc16 = a & 0x3f3fu;
            m16 = b & 0x3f3fu;
        } else {
            sc16 = (t & 0x0f0fu) | ((a & 0xc0c0u) >> 2);
            m16 = ((t >> 4) & 0x0f0fu) | ((b & 0xc0c0u) >> 2);
        }
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&r.hdr.x));
        float s_lo = 0.0f, s_hi = 0.0f;
        const uint32_t q[8] = { r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w };
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const uint32_t lo = q[w] & 0x0f0f0f0fu, hi = (q[w] >> 4) & 0x0f0f0f0fu;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                s_lo = fmaf(u8f(lo, k), x.lo[4 * w + k], s_lo);
                s_hi = fmaf(u8f(hi, k), x.hi[4 * w + k], s_hi);
            }
        }
        const float pos = (float)(sc16 & 0xffu) * s_lo + (float)(sc16 >> 8) * s_hi;
        const float neg = (float)(m16 & 0xffu) * x.slo + (float)(m16 >> 8) * x.shi;
        return dm.x * pos - dm.y * neg;
    }
};

// Q6_K, planar: 4 lanes per super-block; lane (i, lb) owns, in half i, the 16 positions
// l0 = 16*lb .. +15 of each of the four 32-column runs (ql[l], ql[l+32] nibbles + qh bit pairs).
template <>
struct Step<WGB_Q6_K> {
    struct Raw { uint4 a, b, h; uint2 sc; uint16_t d; };
    struct X { float v[4][16]; float s[4]; };

    __device__ static __forceinline__ bool active(const QMat &m, uint32_t col0, int lane)
    {
        return (col0 >> 8) + (lane >> 2) < m.bpr;
    }
    __device__ static __forceinline__ void load(Raw &r, const QMat &m, uint32_t row, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 8) + (lane >> 2), i = (lane >> 1) & 1, lb = lane & 1;
        const size_t blk = (size_t)row * m.bpr + kb;
        const uint8_t *ql = m.p0 + blk * 128 + i * 64 + lb * 16;
        r.a = ldg_stream(ql);
        r.b = ldg_stream(ql + 32);
        r.h = ldg_stream(m.p1 + blk * 64 + i * 32 + lb * 16);
        r.sc = ldg_stream8(m.p2 + blk * 16 + i * 8);
        r.d = ldg_stream2(m.p3 + blk * 2);
    }
    __device__ static __forceinline__ void load_x(X &x, const float *xs, const float *xsum, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 8) + (lane >> 2), i = (lane >> 1) & 1, lb = lane & 1;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t c0 = kb * 64 + i * 32 + j * 8 + lb * 4;
#pragma unroll
            for (int t = 0; t < 4; t++) {
                float4 a = xs_chunk<WGB_Q6_K>(xs, c0 + t);
                x.v[j][4 * t] = a.x; x.v[j][4 * t + 1] = a.y; x.v[j][4 * t + 2] = a.z; x.v[j][4 * t + 3] = a.w;
            }
            x.s[j] = xsum[kb * 16 + i * 8 + j * 2 + lb];
        }
    }
    __device__ static __forceinline__ float dot(const Raw &r, const X &x, int lane)
    {
        const uint32_t lb = lane & 1;
        const uint32_t A[4] = { r.a.x, r.a.y, r.a.z, r.a.w }, B[4] = { r.b.x, r.b.y, r.b.z, r.b.w },
                       H[4] = { r.h.x, r.h.y, r.h.z, r.h.w };
        float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t q0 = (A[w] & 0x0f0f0f0fu) | ((H[w] << 4) & 0x30303030u);
            const uint32_t q1 = (B[w] & 0x0f0f0f0fu) | ((H[w] << 2) & 0x30303030u);
            const uint32_t q2 = ((A[w] >> 4) & 0x0f0f0f0fu) | (H[w] & 0x30303030u);
            const uint32_t q3 = ((B[w] >> 4) & 0x0f0f0f0fu) | ((H[w] >> 2) & 0x30303030u);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                s0 = fmaf(u8f(q0, k), x.v[0][4 * w + k], s0);
                s1 = fmaf(u8f(q1, k), x.v[1][4 * w + k], s1);
                s2 = fmaf(u8f(q2, k), x.v[2][4 * w + k], s2);
                s3 = fmaf(u8f(q3, k), x.v[3][4 * w + k], s3);
            }
        }
        // int8 scales i*8 + lb + {0, 2, 4, 6}
        const uint32_t lo = r.sc.x >> (8 * lb), hi = r.sc.y >> (8 * lb);
        float acc = s8f(lo, 0) * (s0 - 32.0f * x.s[0]);
        acc = fmaf(s8f(lo, 2), s1 - 32.0f * x.s[1], acc);
        acc = fmaf(s8f(hi, 0), s2 - 32.0f * x.s[2], acc);
        acc = fmaf(s8f(hi, 2), s3 - 32.0f * x.s[3], acc);
        return __half2float(__ushort_as_half(r.d)) * acc;
    }
};

// Q8_0, planar: one lane per 32-column block.
template <>
struct Step<WGB_Q8_0> {
    struct Raw { uint4 q0, q1; uint16_t d; };
    struct X { float v[32]; };

    __device__ static __forceinline__ bool active(const QMat &m, uint32_t col0, int lane)
    {
        return (col0 >> 5) + lane < m.bpr;
    }
    __device__ static __forceinline__ void load(Raw &r, const QMat &m, uint32_t row, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 5) + lane;
        const uint8_t *qs = m.p0 + (size_t)row * m.ncols + kb * 32;
        r.q0 = ldg_stream(qs);
        r.q1 = ldg_stream(qs + 16);
        r.d = ldg_stream2(m.p1 + ((size_t)row * m.bpr + kb) * 2);
    }
    __device__ static __forceinline__ void load_x(X &x, const float *xs, const float *, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 5) + lane;
#pragma unroll
        for (int t = 0; t < 8; t++) {
            float4 a = xs_chunk<WGB_Q8_0>(xs, kb * 8 + t);
            x.v[4 * t] = a.x; x.v[4 * t + 1] = a.y; x.v[4 * t + 2] = a.z; x.v[4 * t + 3] = a.w;
        }
    }
    __device__ static __forceinline__ float dot(const Raw &r, const X &x, int)
    {
        const uint32_t q[8] = { r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w };
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; w++)
#pragma unroll
            for (int k = 0; k < 4; k++) s = fmaf(s8f(q[w], k), x.v[4 * w + k], s);
        return __half2float(__ushort_as_half(r.d)) * s;
    }
};

// Dense f32 (ncols a multiple of 4): one lane per 4 columns.
template <>
struct Step<WGB_F32> {
    struct Raw { uint4 w; };
    struct X { float4 v; };

    __device__ static __forceinline__ bool active(const QMat &m, uint32_t col0, int lane)
    {
        return col0 + lane * 4 < m.ncols;
    }
    __device__ static __forceinline__ void load(Raw &r, const QMat &m, uint32_t row, uint32_t col0, int lane)
    {
        r.w = ldg_stream(m.p0 + ((size_t)row * m.ncols + col0 + lane * 4) * 4);
    }
    __device__ static __forceinline__ void load_x(X &x, const float *xs, const float *, uint32_t col0, int lane)
    {
        x.v = xs_chunk<WGB_F32>(xs, (col0 >> 2) + lane);
    }
    __device__ static __forceinline__ float dot(const Raw &r, const X &x, int)
    {
        return __uint_as_float(r.w.x) * x.v.x + __uint_as_float(r.w.y) * x.v.y +
               __uint_as_float(r.w.z) * x.v.z + __uint_as_float(r.w.w) * x.v.w;
    }
};

// R rows (possibly of R different matrices of the same format and width) against xs.
// `rows[r]` must be valid row indices of `mats[r]`.  Returns, in every lane, the R sums.
template <int QT, int R>
__device__ __forceinline__ void warp_dot_rows(const QMat *const (&mats)[R], const uint32_t (&rows)[R],
                                              const float *xs, const float *xsum, float (&acc)[R])
{
    using S = Step<QT>;
    const int lane = threadIdx.x & 31;
    const QMat &m0 = *mats[0];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.0f;
    for (uint32_t col0 = 0; col0 < m0.ncols; col0 += step_cols<QT>()) {
        if (S::active(m0, col0, lane)) {
            typename S::Raw raw[R];
#pragma unroll
            for (int r = 0; r < R; r++) S::load(raw[r], *mats[r], rows[r], col0, lane);
            typename S::X x;
            S::load_x(x, xs, xsum, col0, lane);
#pragma unroll
            for (int r = 0; r < R; r++) acc[r] += S::dot(raw[r], x, lane);
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = warp_sum(acc[r]);
}

// Writes v[0..K) (already normalised / transformed by the caller through `f`) into the swizzled
// shared image and builds the 16-column sums.  Called by all NT threads of the block; ends with a
// barrier.  K must be a multiple of 4; `xsum` needs ceil(K/16) floats.
template <int QT, int NT, typename F>
__device__ __forceinline__ void stage_x(float *xs, float *xsum, uint32_t K, F f)
{
    for (uint32_t c = threadIdx.x; c < K / 4; c += NT)
        reinterpret_cast<float4 *>(xs)[swz<QT>(c)] = f(c);
    __syncthreads();
    if (QT == WGB_Q4_K || QT == WGB_Q6_K) {
        for (uint32_t s = threadIdx.x; s < K / 16; s += NT) {
            float t = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float4 a = xs_chunk<QT>(xs, s * 4 + j);
                t += (a.x + a.y) + (a.z + a.w);
            }
            xsum[s] = t;
        }
        __syncthreads();
    }
}

}  // namespace wgb
