// Warp-level quantised dot products: rows of a matrix staged in shared memory against one input vector
// held in shared memory.  These are the inner loops of the fused matrix-vector kernel (gemv.cu).
//
// A warp walks the K dimension in steps; in each step every lane owns a fixed slice of the columns (a run
// of codes that shares its sub-block scale), keeps the matching part of x in registers and reuses it for
// every row it is given.  Weight bytes come from the stage the producer warp filled with bulk copies
// (128-bit shared loads); x comes from the shared image through a bank-conflict-free swizzle.  Partial sums
// are f32 and are folded across the warp by the caller.
//
// Arithmetic.  At 7.7 TB/s a B200 streams ~1.4e13 four-bit codes per second, more than its
// integer pipe can turn into floats one by one, so the inner product of the codes of one
// 32-column sub-block with x is taken in integers instead:
//   x of a 32-column group is written as X * 2^e with a shared exponent and a 24-bit signed X
//   (|X| <= 2^22, rounded to nearest: within one bit of f32 precision for the largest element), X is split into
//   three bytes X = 65536 d2 + 256 d1 + d0, and  sum_l q_l X_l  is three dp4a chains over the
//   packed codes (which are dp4a operands as they come out of the mask), exact in int32.
// The exact integer S then enters the f32 algebra of the format:
//   Q4_K  sum_l (d*sc*q_l - dmin*m) x_l = d*sc * 2^e S  -  dmin*m * sum_l x_l
//   Q6_K  sum_l d*sc*(q_l - 32) x_l     = d*sc * (2^e S - 32 * sum_l x_l)
//   Q8_0  sum_l d*q_l x_l               = d * 2^e S
// with the per-16-column sums of x (f32, from the unrounded x) computed once per thread block.
// Dense f32 matrices use plain f32 FMAs.
#pragma once

#include "dequant.cuh"
#include "qmatrix.cuh"

namespace wgb {

__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)  // a unsigned bytes, b signed bytes
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c)  // a signed bytes, b unsigned bytes
{
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Integer -> f32 without the conversion unit: adding the integer to the bit pattern of 2^23 (resp. 1.5 * 2^23)
// yields the float 2^23 + v exactly, and one FP32 subtraction removes the offset.  Valid for 0 <= v < 2^23
// (resp. |v| < 2^22).  Used where the range is known to fit; sums of digit products go through cvt below.
__device__ __forceinline__ float u2f(uint32_t v) { return __uint_as_float(v + 0x4b000000u) - 8388608.0f; }
__device__ __forceinline__ float i2f(int v) { return __uint_as_float((uint32_t)v + 0x4b400000u) - 12582912.0f; }

// Unsigned byte k of a word as f32: one byte permute drops it into the mantissa of 2^23.
__device__ __forceinline__ float byte2f(uint32_t w, int k)
{
    return __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7440 + k)) - 8388608.0f;
}

// 65536 s2 + 256 s1 + s0 as f32 for the three digit sums of one scale group.  The two low digits are joined in
// the integer unit (|256 s1 + s0| < 2^30 for every format here) and the conversion unit is used twice: its rate
// (a sixteenth of the integer pipe's) is ample at two conversions per 32 or 64 weights, and the pair costs
// four issue slots where the offset trick costs eight.  The result is the correctly rounded f32 of each part
// and one fused multiply-add, i.e. within an ulp of the exact sum.
__device__ __forceinline__ float combine3(int s2, int s1, int s0)
{
    return fmaf(__int2float_rn(s2), 65536.0f, __int2float_rn(s1 * 256 + s0));
}
__device__ __forceinline__ float combine3s(int s2, int s1, int s0) { return combine3(s2, s1, s0); }

// Sign-extended byte k of a word, as f32.
__device__ __forceinline__ float s8f(uint32_t w, int k) { return __int2float_rn((int)(signed char)(w >> (8 * k))); }

// ---------------------------------------------------------------------------------------------
// Shared-memory image of the input vector (built once per thread block by stage_x).
//   quantised formats:  d0, d1, d2  K bytes each: the three byte digits of X, element order,
//                                   16-byte chunks at swizzled positions (swz<QT>)
//                       xscale      K/32 floats: 2^e of every 32-column group
//                       xsum        K/16 floats: f32 sum of every 16 consecutive inputs
//   f32:                xf          K floats
// The swizzle permutes chunks inside aligned groups of 8 so that the 8 lanes served together by one
// 128-bit shared load hit 8 different bank groups for the lane->column map of QT.
// ---------------------------------------------------------------------------------------------
struct XImage {
    const uint4 *d0, *d1, *d2;
    const float *xscale, *xsum, *xf;
};

__host__ __device__ constexpr size_t ximage_bytes(int qt, uint32_t K)
{
    return qt == WGB_F32 ? (size_t)K * 4 : 3 * (size_t)((K + 127) & ~127u) + (size_t)((K / 32 + 3) & ~3u) * 4 + (size_t)((K / 16 + 3) & ~3u) * 4;
}

__device__ __forceinline__ XImage ximage_carve(int qt, uint32_t K, void *smem)
{
    XImage im = {};
    if (qt == WGB_F32) {
        im.xf = reinterpret_cast<const float *>(smem);
        return im;
    }
    const size_t plane = (K + 127) & ~127u;
    uint8_t *p = reinterpret_cast<uint8_t *>(smem);
    im.d0 = reinterpret_cast<const uint4 *>(p);
    im.d1 = reinterpret_cast<const uint4 *>(p + plane);
    im.d2 = reinterpret_cast<const uint4 *>(p + 2 * plane);
    im.xscale = reinterpret_cast<const float *>(p + 3 * plane);
    im.xsum = im.xscale + ((K / 32 + 3) & ~3u);
    return im;
}

// Position of 16-element chunk c of a digit plane.
template <int QT>
__device__ __forceinline__ uint32_t swz(uint32_t c)
{
    if (QT == WGB_Q4_K) return c ^ ((c >> 3) & 3u);          // lanes (kb, g): c = kb*16 + g*4 + t
    if (QT == WGB_Q6_K) return c ^ (((c >> 3) & 3u) << 1);   // lanes (kb, i, lb): c = kb*16 + i*8 + j*2 + lb
    if (QT == WGB_Q8_0) return c ^ ((c >> 3) & 1u);          // lanes kb: c = kb*2 + t
    return c;
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
// Per-format step over rows staged in shared memory.  A step covers step_cols<QT>() columns; lane l
// owns a fixed slice of them.  load_x() brings the lane's part of the input image into registers
// (reused for every row of the step); dot() reads the lane's slice of one staged row -- `rowp[i]` is
// the shared-memory address of the row's first byte in plane i -- and returns its partial sum.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr)
{
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

template <int QT>
struct Step;

// All-zero input registers: what a lane past the end of the row multiplies its (valid, in-row) weights by.
template <typename X>
__device__ __forceinline__ void zero_x(X &x)
{
    uint32_t *w = reinterpret_cast<uint32_t *>(&x);
#pragma unroll
    for (int i = 0; i < (int)(sizeof(X) / 4); i++) w[i] = 0u;
}

// Q4_K, raw 144-byte super-blocks: 4 lanes per super-block, lane g owns its 64-column group
// (32 bytes of qs: low nibbles = first 32 columns, high nibbles = next 32).
template <>
struct Step<WGB_Q4_K> {
    struct X { uint4 d0[4], d1[4], d2[4]; float e_lo, e_hi, s_lo, s_hi; };

    __device__ static __forceinline__ bool active(uint32_t bpr, uint32_t col0, int lane)
    {
        return (col0 >> 8) + (lane >> 2) < bpr;
    }
    // The lane of the step's first unit that plays the same part as `lane` (always inside the row).
    __device__ static __forceinline__ int lane0(int lane) { return lane & 3; }
    __device__ static __forceinline__ void load_x(X &x, const XImage &im, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 8) + (lane >> 2), g = lane & 3;
        const uint32_t c0 = kb * 16 + g * 4;
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const uint32_t c = swz<WGB_Q4_K>(c0 + t);
            x.d0[t] = im.d0[c];
            x.d1[t] = im.d1[c];
            x.d2[t] = im.d2[c];
        }
        const float2 e = reinterpret_cast<const float2 *>(im.xscale)[kb * 4 + g];
        x.e_lo = e.x;
        x.e_hi = e.y * 0.0625f;   // the high nibbles enter the sums as 16 * code
        const float4 s = reinterpret_cast<const float4 *>(im.xsum)[kb * 4 + g];
        x.s_lo = s.x + s.y;
        x.s_hi = s.z + s.w;
    }
    __device__ static __forceinline__ float dot(const uint32_t (&rowp)[4], uint32_t col0, const X &x, int lane)
    {
        const uint32_t kb = (col0 >> 8) + (lane >> 2), g = lane & 3;
        const uint32_t blk = rowp[0] + kb * 144;
        const uint4 hdr = lds128(blk), q0 = lds128(blk + 16 + g * 32), q1 = lds128(blk + 32 + g * 32);
        // Six-bit scale / min of sub-blocks 2g and 2g+1 (get_scale_min_k4, quantization.rs:381-389) as the four
        // bytes (sc_lo, sc_hi, m_lo, m_hi) of one word, without a branch: with j = 2g, 2g+1
        //   g < 2:  sc = scales[j] & 63,                        m = scales[j+4] & 63
        //   g >= 2: sc = (scales[j+4] & 15) | (scales[j-4] >> 6) << 4,  m = (scales[j+4] >> 4) | (scales[j] >> 6) << 4
        // Both cases read bytes 2(g&1), 2(g&1)+1 of hdr.y (scales 0..3) and of hdr.z (4..7); the second also
        // those bytes of hdr.w (8..11).  The selectors and masks depend on the lane only.
        const uint32_t b0 = 2u * (g & 1u);
        const uint32_t sel_yz = (b0) | ((b0 + 1u) << 4) | ((b0 + 4u) << 8) | ((b0 + 5u) << 12);   // (y[b0], y[b0+1], z[b0], z[b0+1])
        const uint32_t yz = __byte_perm(hdr.y, hdr.z, sel_yz);
        const uint32_t t2 = __byte_perm(hdr.w, hdr.w >> 4, sel_yz);                                 // (w[b0], w[b0+1], (w>>4)[b0], (w>>4)[b0+1])
        const bool high = g >= 2;
        const uint32_t scm = ((high ? t2 : yz) & (high ? 0x0f0f0f0fu : 0x3f3f3f3fu)) | ((yz >> 2) & (high ? 0x30303030u : 0u));
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        const uint32_t q[8] = { q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w };
        // columns 0..31 of the group sit in digit chunks 0,1 (low nibbles), 32..63 in chunks 2,3
        const uint32_t *d0 = reinterpret_cast<const uint32_t *>(x.d0), *d1 = reinterpret_cast<const uint32_t *>(x.d1),
                       *d2 = reinterpret_cast<const uint32_t *>(x.d2);
        int l0 = 0, l1 = 0, l2 = 0, h0 = 0, h1 = 0, h2 = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            // high nibbles stay in place (16 * code): the factor 1/16 is applied to the finished sum
            const uint32_t lo = q[w] & 0x0f0f0f0fu, hi = q[w] & 0xf0f0f0f0u;
            l0 = dp4a_uu(lo, d0[w], l0);
            l1 = dp4a_uu(lo, d1[w], l1);
            l2 = dp4a_us(lo, d2[w], l2);
            h0 = dp4a_uu(hi, d0[8 + w], h0);
            h1 = dp4a_uu(hi, d1[8 + w], h1);
            h2 = dp4a_us(hi, d2[8 + w], h2);
        }
        // |256 l1 + l0| <= 257 * 32 * 15 * 255 < 2^25; the high-nibble sums are 16 times larger: < 2^29
        const float s_lo = combine3(l2, l1, l0) * x.e_lo, s_hi = combine3(h2, h1, h0) * x.e_hi;   // e_hi holds 2^e / 16
        const float pos = fmaf(byte2f(scm, 0), s_lo, byte2f(scm, 1) * s_hi);
        const float neg = fmaf(byte2f(scm, 2), x.s_lo, byte2f(scm, 3) * x.s_hi);
        return fmaf(dm.x, pos, -(dm.y * neg));
    }
};

// Q6_K, planar: 4 lanes per super-block; lane (i, lb) owns, in half i, the 16 positions
// l0 = 16*lb .. +15 of each of the four 32-column runs (ql[l], ql[l+32] nibbles + qh bit pairs).
template <>
struct Step<WGB_Q6_K> {
    struct X { uint4 d0[4], d1[4], d2[4]; float e[4], s[4]; };

    __device__ static __forceinline__ bool active(uint32_t bpr, uint32_t col0, int lane)
    {
        return (col0 >> 8) + (lane >> 2) < bpr;
    }
    __device__ static __forceinline__ int lane0(int lane) { return lane & 3; }
    __device__ static __forceinline__ void load_x(X &x, const XImage &im, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 8) + (lane >> 2), i = (lane >> 1) & 1, lb = lane & 1;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t c = swz<WGB_Q6_K>(kb * 16 + i * 8 + j * 2 + lb);
            x.d0[j] = im.d0[c];
            x.d1[j] = im.d1[c];
            x.d2[j] = im.d2[c];
            x.e[j] = im.xscale[kb * 8 + i * 4 + j];
            x.s[j] = im.xsum[kb * 16 + i * 8 + j * 2 + lb];
        }
    }
    __device__ static __forceinline__ float dot(const uint32_t (&rowp)[4], uint32_t col0, const X &x, int lane)
    {
        const uint32_t kb = (col0 >> 8) + (lane >> 2), i = (lane >> 1) & 1, lb = lane & 1;
        const uint32_t ql = rowp[0] + kb * 128 + i * 64 + lb * 16;
        const uint4 ra = lds128(ql), rb = lds128(ql + 32), rh = lds128(rowp[1] + kb * 64 + i * 32 + lb * 16);
        const uint2 rsc = lds64(rowp[2] + kb * 16 + i * 8);
        const uint32_t rd = lds16(rowp[3] + kb * 2);
        const uint32_t A[4] = { ra.x, ra.y, ra.z, ra.w }, B[4] = { rb.x, rb.y, rb.z, rb.w }, H[4] = { rh.x, rh.y, rh.z, rh.w };
        const uint32_t *d0 = reinterpret_cast<const uint32_t *>(x.d0), *d1 = reinterpret_cast<const uint32_t *>(x.d1),
                       *d2 = reinterpret_cast<const uint32_t *>(x.d2);
        int s[4][3] = {};
#pragma unroll
        for (int w = 0; w < 4; w++) {
            uint32_t q[4];
            q[0] = (A[w] & 0x0f0f0f0fu) | ((H[w] << 4) & 0x30303030u);
            q[1] = (B[w] & 0x0f0f0f0fu) | ((H[w] << 2) & 0x30303030u);
            q[2] = ((A[w] >> 4) & 0x0f0f0f0fu) | (H[w] & 0x30303030u);
            q[3] = ((B[w] >> 4) & 0x0f0f0f0fu) | ((H[w] >> 2) & 0x30303030u);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                s[j][0] = dp4a_uu(q[j], d0[4 * j + w], s[j][0]);
                s[j][1] = dp4a_uu(q[j], d1[4 * j + w], s[j][1]);
                s[j][2] = dp4a_us(q[j], d2[4 * j + w], s[j][2]);
            }
        }
        // int8 scales i*8 + lb + {0, 2, 4, 6}
        const uint32_t lo = rsc.x >> (8 * lb), hi = rsc.y >> (8 * lb);
        float acc = s8f(lo, 0) * (combine3(s[0][2], s[0][1], s[0][0]) * x.e[0] - 32.0f * x.s[0]);
        acc = fmaf(s8f(lo, 2), combine3(s[1][2], s[1][1], s[1][0]) * x.e[1] - 32.0f * x.s[1], acc);
        acc = fmaf(s8f(hi, 0), combine3(s[2][2], s[2][1], s[2][0]) * x.e[2] - 32.0f * x.s[2], acc);
        acc = fmaf(s8f(hi, 2), combine3(s[3][2], s[3][1], s[3][0]) * x.e[3] - 32.0f * x.s[3], acc);
        return __half2float(__ushort_as_half((uint16_t)rd)) * acc;
    }
};

// Q8_0, planar: one lane per 32-column block.
template <>
struct Step<WGB_Q8_0> {
    struct X { uint4 d0[2], d1[2], d2[2]; float e; };

    __device__ static __forceinline__ bool active(uint32_t bpr, uint32_t col0, int lane)
    {
        return (col0 >> 5) + lane < bpr;
    }
    __device__ static __forceinline__ int lane0(int) { return 0; }
    __device__ static __forceinline__ void load_x(X &x, const XImage &im, uint32_t col0, int lane)
    {
        const uint32_t kb = (col0 >> 5) + lane;
#pragma unroll
        for (int t = 0; t < 2; t++) {
            const uint32_t c = swz<WGB_Q8_0>(kb * 2 + t);
            x.d0[t] = im.d0[c];
            x.d1[t] = im.d1[c];
            x.d2[t] = im.d2[c];
        }
        x.e = im.xscale[kb];
    }
    __device__ static __forceinline__ float dot(const uint32_t (&rowp)[4], uint32_t col0, const X &x, int lane)
    {
        const uint32_t kb = (col0 >> 5) + lane;
        const uint4 q0 = lds128(rowp[0] + kb * 32), q1 = lds128(rowp[0] + kb * 32 + 16);
        const uint32_t rd = lds16(rowp[1] + kb * 2);
        const uint32_t q[8] = { q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w };
        const uint32_t *d0 = reinterpret_cast<const uint32_t *>(x.d0), *d1 = reinterpret_cast<const uint32_t *>(x.d1),
                       *d2 = reinterpret_cast<const uint32_t *>(x.d2);
        int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            s0 = dp4a_su(q[w], d0[w], s0);
            s1 = dp4a_su(q[w], d1[w], s1);
            s2 = dp4a_ss(q[w], d2[w], s2);
        }
        return __half2float(__ushort_as_half((uint16_t)rd)) * (combine3s(s2, s1, s0) * x.e);
    }
};

// Dense f32 (ncols a multiple of 4): one lane per 4 columns.  `bpr` is the number of columns.
template <>
struct Step<WGB_F32> {
    struct X { float4 v; };

    __device__ static __forceinline__ bool active(uint32_t ncols, uint32_t col0, int lane)
    {
        return col0 + lane * 4 < ncols;
    }
    __device__ static __forceinline__ int lane0(int) { return 0; }
    __device__ static __forceinline__ void load_x(X &x, const XImage &im, uint32_t col0, int lane)
    {
        x.v = reinterpret_cast<const float4 *>(im.xf)[(col0 >> 2) + lane];
    }
    __device__ static __forceinline__ float dot(const uint32_t (&rowp)[4], uint32_t col0, const X &x, int lane)
    {
        const uint4 w = lds128(rowp[0] + (col0 + lane * 4) * 4);
        return __uint_as_float(w.x) * x.v.x + __uint_as_float(w.y) * x.v.y + __uint_as_float(w.z) * x.v.z +
               __uint_as_float(w.w) * x.v.w;
    }
};

// Writer of the shared image.  put(c, v, in) stores float4 chunk c (columns 4c .. 4c+3, already normalised /
// transformed by the caller); it is called by whole warps (all 32 lanes, converged), lane l with chunk c0 + l, so
// that 8 consecutive lanes hold one 32-column group; `in` is false for lanes past the end of the vector (whole
// groups of 8 lanes are in or out together because K is a multiple of 32).  The caller synchronises the block
// afterwards.  K must be a multiple of 32 for the quantised formats, of 4 for f32.
template <int QT>
struct XWriter {
    uint32_t *d0, *d1, *d2;
    float *xscale, *xsum;
    float4 *xf;

    __device__ __forceinline__ XWriter(void *smem, uint32_t K)
    {
        xf = reinterpret_cast<float4 *>(smem);
        const size_t plane = (K + 127) & ~127u;
        uint8_t *p = reinterpret_cast<uint8_t *>(smem);
        d0 = reinterpret_cast<uint32_t *>(p);
        d1 = reinterpret_cast<uint32_t *>(p + plane);
        d2 = reinterpret_cast<uint32_t *>(p + 2 * plane);
        xscale = reinterpret_cast<float *>(p + 3 * plane);
        xsum = xscale + ((K / 32 + 3) & ~3u);
    }

    // Eight consecutive values at once: float4 chunks c = 2u (va) and 2u + 1 (vb) of the thread's unit u; lane l
    // of a warp calls with unit u0 + l, so that four consecutive lanes hold one 32-column group and two hold a
    // 16-column run.  Half the shuffles of put() per value and one 64-bit store per digit plane.  `inb`: chunk
    // 2u + 1 exists (only a dense f32 vector can end in the middle of a unit).
    __device__ __forceinline__ void put8(uint32_t u, const float4 va, const float4 vb, bool in, bool inb) const
    {
        const uint32_t c = 2 * u;
        if (QT == WGB_F32) {
            if (in) xf[c] = va;
            if (in && inb) xf[c + 1] = vb;
            return;
        }
        float m = fmaxf(fmaxf(fmaxf(fabsf(va.x), fabsf(va.y)), fmaxf(fabsf(va.z), fabsf(va.w))),
                        fmaxf(fmaxf(fabsf(vb.x), fabsf(vb.y)), fmaxf(fabsf(vb.z), fabsf(vb.w))));
        float sum = ((va.x + va.y) + (va.z + va.w)) + ((vb.x + vb.y) + (vb.z + vb.w));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        uint32_t ex = (__float_as_uint(m) >> 23) & 0xffu;
        ex = ex < 24u ? 24u : (ex > 253u ? 253u : ex);
        const float up = __uint_as_float((275u - ex) << 23);    // 2^(148 - ex), see put()
        auto fix = [&](float v) { return (int)(__float_as_uint(fmaf(v, up, 12582912.0f)) - 0x4b400000u); };
        const int A0 = fix(va.x), A1 = fix(va.y), A2 = fix(va.z), A3 = fix(va.w);
        const int B0 = fix(vb.x), B1 = fix(vb.y), B2 = fix(vb.z), B3 = fix(vb.w);
        if (in) {
            const uint32_t a01 = __byte_perm(A0, A1, 0x5410), a23 = __byte_perm(A2, A3, 0x5410);
            const uint32_t a01h = __byte_perm(A0, A1, 0x7632), a23h = __byte_perm(A2, A3, 0x7632);
            const uint32_t b01 = __byte_perm(B0, B1, 0x5410), b23 = __byte_perm(B2, B3, 0x5410);
            const uint32_t b01h = __byte_perm(B0, B1, 0x7632), b23h = __byte_perm(B2, B3, 0x7632);
            // chunks 2u and 2u + 1 sit side by side inside one (swizzled) 16-byte chunk of every digit plane
            const uint32_t pos = swz<QT>(c >> 2) * 4 + (c & 3);
            *reinterpret_cast<uint2 *>(d0 + pos) = make_uint2(__byte_perm(a01, a23, 0x6420), __byte_perm(b01, b23, 0x6420));
            *reinterpret_cast<uint2 *>(d1 + pos) = make_uint2(__byte_perm(a01, a23, 0x7531), __byte_perm(b01, b23, 0x7531));
            *reinterpret_cast<uint2 *>(d2 + pos) = make_uint2(__byte_perm(a01h, a23h, 0x6420), __byte_perm(b01h, b23h, 0x6420));
            if ((u & 3) == 0) xscale[u >> 2] = __uint_as_float((ex - 21u) << 23);   // 2^(ex - 148)
            if ((u & 1) == 0) xsum[u >> 1] = sum;
        }
    }

    __device__ __forceinline__ void put(uint32_t c, const float4 v, bool in) const
    {
        if (QT == WGB_F32) {
            if (in) xf[c] = v;
            return;
        }
        float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        float sum = (v.x + v.y) + (v.z + v.w);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
        // |v| < 2^(ex-126) for the biased exponent ex of the group maximum, so X = v * 2^(148-ex) stays
        // within +-2^22 after rounding and its third byte is a valid signed digit
        uint32_t ex = (__float_as_uint(m) >> 23) & 0xffu;
        ex = ex < 24u ? 24u : (ex > 253u ? 253u : ex);
        const float up = __uint_as_float((275u - ex) << 23);    // 2^(148 - ex)
        // round to nearest even through the 1.5 * 2^23 offset (|v * up| <= 2^22)
        const int X0 = (int)(__float_as_uint(fmaf(v.x, up, 12582912.0f)) - 0x4b400000u),
                  X1 = (int)(__float_as_uint(fmaf(v.y, up, 12582912.0f)) - 0x4b400000u),
                  X2 = (int)(__float_as_uint(fmaf(v.z, up, 12582912.0f)) - 0x4b400000u),
                  X3 = (int)(__float_as_uint(fmaf(v.w, up, 12582912.0f)) - 0x4b400000u);
        if (in) {
            // digit k of the four values packed into one word
            const uint32_t a01 = __byte_perm(X0, X1, 0x5410), a23 = __byte_perm(X2, X3, 0x5410);  // bytes 0,1 of each
            const uint32_t b01 = __byte_perm(X0, X1, 0x7632), b23 = __byte_perm(X2, X3, 0x7632);  // bytes 2,3 of each
            const uint32_t w0 = __byte_perm(a01, a23, 0x6420), w1 = __byte_perm(a01, a23, 0x7531);
            const uint32_t w2 = __byte_perm(b01, b23, 0x6420);
            const uint32_t pos = swz<QT>(c >> 2) * 4 + (c & 3);
            d0[pos] = w0;
            d1[pos] = w1;
            d2[pos] = w2;
            if ((c & 7) == 0) xscale[c >> 3] = __uint_as_float((ex - 21u) << 23);   // 2^(ex - 148)
            if ((c & 3) == 0) xsum[c >> 2] = sum;
        }
    }
};

}  // namespace wgb
