// Bit-exact dequantisation of GGUF blocks, 32 weights at a time.
//
// Every function restates one `Block*::dequantize` of crates/wgml/src/quantization.rs with the
// same operation order.  Products and sums use __fmul_rn / __fadd_rn / __fsub_rn, which nvcc
// never contracts into an FMA, so each operation rounds once, as the Rust code does.
#pragma once

#include "common.cuh"

namespace wgb {

// decode_f16 -- quantization.rs:392-409.  Finite values and infinities are exact conversions;
// any NaN becomes the canonical quiet NaN with the half's sign, as `f32::NAN` negated does.
__device__ __forceinline__ float decode_f16(uint16_t h)
{
    if ((h & 0x7c00u) == 0x7c00u && (h & 0x03ffu) != 0u)
        return __uint_as_float(0x7fc00000u | ((uint32_t)(h & 0x8000u) << 16));
    return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ uint16_t ld16(const uint8_t *p) { return (uint16_t)p[0] | ((uint16_t)p[1] << 8); }
__device__ __forceinline__ uint32_t ld32(const uint8_t *p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

// get_scale_min_k4 -- quantization.rs:381-389
__device__ __forceinline__ void get_scale_min_k4(int j, const uint8_t *q, uint8_t &d, uint8_t &m)
{
    if (j < 4) {
        d = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// BlockQ8_0::dequantize -- quantization.rs:38-41, one weight.
__device__ __forceinline__ float q8_0_value(uint16_t scale_bits, int8_t q)
{
    return __fmul_rn((float)q, decode_f16(scale_bits));
}

// BlockQ6K::dequantize -- quantization.rs:214-243, weight l of group g, with the four fields of
// the block passed separately so that split (planar) storage can use it too.
__device__ __forceinline__ float q6_k_value(const uint8_t *ql, const uint8_t *qh, const int8_t *scales,
                                            uint16_t d_bits, int g, int l)
{
    const int i = g >> 2, sub = g & 3;
    float d = decode_f16(d_bits);
    uint8_t h = qh[i * 32 + l];
    uint8_t lo = ql[i * 64 + l + ((sub & 1) ? 32 : 0)];
    uint8_t nib = (sub & 2) ? (lo >> 4) : (lo & 0xF);
    int q = (int)(int8_t)(nib | (((h >> (2 * sub)) & 3) << 4)) - 32;
    float sc = (float)scales[i * 8 + (l >> 4) + 2 * sub];
    return __fmul_rn(__fmul_rn(d, sc), (float)q);
}

// Weight `l` (0..31) of 32-weight group `g` of the block at `b` (raw GGUF byte order).
// Groups: one per block for the 32-weight formats, eight per 256-weight super-block.
template <int QT>
__device__ __forceinline__ float dequant_one(const uint8_t *b, int g, int l)
{
    if (QT == WGB_Q8_0) {
        return q8_0_value(ld16(b), (int8_t)b[2 + l]);
    } else if (QT == WGB_Q4_0) {  // :55-68
        float d = decode_f16(ld16(b));
        uint8_t q = b[2 + (l & 15)];
        int x = (l < 16) ? (int)(q & 0x0F) - 8 : (int)(q >> 4) - 8;
        return __fmul_rn((float)x, d);
    } else if (QT == WGB_Q4_1) {  // :83-97
        float d = decode_f16(ld16(b)), m = decode_f16(ld16(b + 2));
        uint8_t q = b[4 + (l & 15)];
        uint32_t x = (l < 16) ? (q & 0x0Fu) : (q >> 4);
        return __fadd_rn(__fmul_rn((float)x, d), m);
    } else if (QT == WGB_Q5_0) {  // :112-128
        float d = decode_f16(ld16(b));
        uint32_t qh = ld32(b + 2);
        int j = l & 15;
        uint8_t q = b[6 + j];
        uint32_t xh = (l < 16) ? (((qh >> j) << 4) & 0x10u) : ((qh >> (j + 12)) & 0x10u);
        uint32_t lo = (l < 16) ? (q & 0x0Fu) : (uint32_t)(q >> 4);
        return __fmul_rn((float)((int)(lo | xh) - 16), d);
    } else if (QT == WGB_Q5_1) {  // :144-161
        float d = decode_f16(ld16(b)), m = decode_f16(ld16(b + 2));
        uint32_t qh = ld32(b + 4);
        int j = l & 15;
        uint8_t q = b[8 + j];
        uint32_t xh = (l < 16) ? (((qh >> j) << 4) & 0x10u) : ((qh >> (j + 12)) & 0x10u);
        uint32_t lo = (l < 16) ? (q & 0x0Fu) : (uint32_t)(q >> 4);
        return __fadd_rn(__fmul_rn((float)(lo | xh), d), m);
    } else if (QT == WGB_Q8_K) {  // :192-198
        float d = __uint_as_float(ld32(b));
        return __fmul_rn(d, (float)(int8_t)b[4 + g * 32 + l]);
    } else if (QT == WGB_Q6_K) {
        return q6_k_value(b, b + 128, (const int8_t *)(b + 192), ld16(b + 208), g, l);
    } else if (QT == WGB_Q4_K) {  // :347-378
        float d = decode_f16(ld16(b)), mn = decode_f16(ld16(b + 2));
        uint8_t sc, m;
        get_scale_min_k4(g, b + 4, sc, m);
        float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(mn, (float)m);
        uint8_t q = b[16 + (g >> 1) * 32 + l];
        uint8_t nib = (g & 1) ? (q >> 4) : (q & 0xF);
        return __fsub_rn(__fmul_rn(d1, (float)nib), m1);
    } else if (QT == WGB_Q5_K) {  // :275-316
        float d = decode_f16(ld16(b)), mn = decode_f16(ld16(b + 2));
        uint8_t sc, m;
        get_scale_min_k4(g, b + 4, sc, m);
        float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(mn, (float)m);
        uint8_t q = b[48 + (g >> 1) * 32 + l];
        uint8_t nib = (g & 1) ? (q >> 4) : (q & 0xF);
        uint8_t v = (uint8_t)(nib + (((b[16 + l] >> g) & 1) ? 16 : 0));
        return __fsub_rn(__fmul_rn(d1, (float)v), m1);
    } else if (QT == WGB_F16) {  // BlockF16, :21-23
        return decode_f16(ld16(b));
    } else {  // F32
        return __uint_as_float(ld32(b));
    }
}

}  // namespace wgb
