// Q4_K matrix-vector product on the fifth-generation tensor cores (tcgen05.mma kind::i8, accumulators in
// tensor memory).  Same operator as GemvQuant::dispatch (crates/wgml/src/ops/gemv_quant.rs:241-348) for
// Q4_K matrices whose row count is a multiple of 128 and whose column count is a multiple of 256 up to
// TC_MAX_K; the weights are kept tile-major so that one bulk copy brings one super-block column of 128 rows.
//
// Decomposition.  The input vector is quantised once per block into three signed byte digits per element
// with one power-of-two exponent per 32 columns (the same fixed-point image as the dp4a kernel, 23 bits).
// For a tile of 128 rows and one super-block column (256 columns) the worker threads unpack the nibbles to
// unsigned bytes in shared memory (A operand, 128 x 256, K-major, 128-byte swizzle, two K panels of 16 KB),
// and one thread issues eight MMAs, one per 32-column sub-block: D[128 rows x 16] = A[128 x 32] * B[32 x 16],
// where columns 0..2 of B are the digits (columns 3..7 zero, 8..15 alias 0..7; B is K-major without
// swizzle).  The threads of row r read that row of the eight results from tensor memory and apply, in FP32,
// the digit weights, the group exponent, the six-bit sub-block scale and the min term (get_scale_min_k4,
// crates/wgml/src/quantization.rs:381-389).
//
// Measured on a B200: one MMA of this shape takes about 190 cycles whatever N is, which caps this kernel at
// about 3 TB/s of packed weights over 148 SMs, below the dp4a kernel; it pays only with many input vectors.
//
// Pipeline per block: warp 0 streams (tile, column) units into a ring with bulk copies; warp 1 owns the
// tensor memory allocation and issues the MMAs; sixteen worker warps (four per quarter of the rows, one
// 32-byte chunk of each row per thread) unpack unit n and then finish unit n - 1 while the MMAs of unit n
// are issued and run (two operand buffers, two sets of accumulator columns).
// Every wait is bounded; the first that expires records a code and every loop of the block winds down.
#include "kernels.h"
#include "tc_common.cuh"

namespace wgb {

constexpr uint32_t TC_MAX_K = 4096;
constexpr uint32_t TC_RING = 6;
constexpr uint32_t TC_WPQ = 4;                                // worker warps per quarter of the tile's rows
constexpr uint32_t TC_CPT = 4 / TC_WPQ;                       // 32-byte chunks (pairs of sub-blocks) per thread
constexpr uint32_t TC_WORKER_WARPS = 4 * TC_WPQ;
constexpr uint32_t TC_NT = 32 * (2 + TC_WORKER_WARPS);
constexpr uint32_t TC_TMEM_COLS = 256;                        // 128 per unit in flight: eight results of 16 columns

// shared-memory map (dynamic, 1024-byte aligned by the launch)
constexpr uint32_t TC_OFF_B = 0;                               // digits: K / 16 core matrices of 128 bytes
constexpr uint32_t TC_OFF_E = TC_OFF_B + TC_MAX_K * 8;         // K / 32 exponents (odd ones carry the 1/16 of high nibbles)
constexpr uint32_t TC_OFF_S = TC_OFF_E + TC_MAX_K / 32 * 4;    // K / 32 sums of the inputs
constexpr uint32_t TC_OFF_A = TC_OFF_S + TC_MAX_K / 32 * 4;    // two operand buffers (units alternate)
constexpr uint32_t TC_OFF_RING = TC_OFF_A + 2 * TC_A_BYTES;
constexpr uint32_t TC_SMEM = TC_OFF_RING + TC_RING * TC_UNIT_BYTES;
static_assert(TC_OFF_A % 1024 == 0 && TC_OFF_RING % 1024 == 0, "operand buffers on 1 KB boundaries");
static_assert(TC_SMEM <= 220 * 1024, "shared memory budget");

struct TcArgs {
    const uint8_t *w;     // tile-major blocks: [tile][column][128 rows][144 bytes]
    const float *x;
    float *out;
    uint32_t nrows, K;
    uint32_t *err;
};

// Fixed-point image of the input: thread g quantises the 32 inputs of group g.
__device__ __forceinline__ void tc_stage_group(uint8_t *smem, const float *x, uint32_t g)
{
    float v[32];
    const float4 *src = reinterpret_cast<const float4 *>(x + 32 * g);
    float m = 0.0f, sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float4 q = __ldcg(src + i);
        v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
        m = fmaxf(m, fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w))));
        sum += (q.x + q.y) + (q.z + q.w);
    }
    // |v| < 2^(ex - 126), so X = v * 2^(148 - ex) stays within +-2^22 after rounding
    uint32_t ex = (__float_as_uint(m) >> 23) & 0xffu;
    ex = ex < 24u ? 24u : (ex > 253u ? 253u : ex);
    const float up = __uint_as_float((275u - ex) << 23), down = __uint_as_float((ex - 21u) << 23);
    uint32_t dig[3][8];
#pragma unroll
    for (int wd = 0; wd < 8; wd++) {
        uint32_t d0 = 0, d1 = 0, d2 = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            // round to nearest even through the 1.5 * 2^23 offset; with 0x8080 added, bytes 0 and 1 are
            // the signed digits plus 128 and byte 2 is the signed top digit
            const uint32_t y = __float_as_uint(fmaf(v[4 * wd + b], up, 12582912.0f)) - 0x4b400000u + 0x8080u;
            d0 |= ((y & 0xffu) ^ 0x80u) << (8 * b);
            d1 |= (((y >> 8) & 0xffu) ^ 0x80u) << (8 * b);
            d2 |= ((y >> 16) & 0xffu) << (8 * b);
        }
        dig[0][wd] = d0; dig[1][wd] = d1; dig[2][wd] = d2;
    }
    const uint32_t base = smem_addr(smem + TC_OFF_B) + (2 * g) * 128;   // two 16-column core matrices per group
#pragma unroll
    for (int core = 0; core < 2; core++)
#pragma unroll
        for (int n = 0; n < 3; n++)
            sts128(base + core * 128 + n * 16, dig[n][4 * core], dig[n][4 * core + 1], dig[n][4 * core + 2], dig[n][4 * core + 3]);
    reinterpret_cast<float *>(smem + TC_OFF_E)[g] = (g & 1) ? down * 0.0625f : down;
    reinterpret_cast<float *>(smem + TC_OFF_S)[g] = sum;
}

__global__ void __launch_bounds__(TC_NT, 1) gemv_q4k_tc_kernel(const __grid_constant__ TcArgs a)
{
    extern __shared__ uint8_t tc_smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * TC_RING + 2];
    __shared__ float rowpart[TC_WPQ][TC_TILE_ROWS];
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t dead_flag;
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    volatile uint32_t *dead = &dead_flag;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nkb = a.K / 256, ntiles = a.nrows / TC_TILE_ROWS;
    auto bar_full = [&](uint32_t s) { return smem_addr(&bars[s]); };
    auto bar_empty = [&](uint32_t s) { return smem_addr(&bars[TC_RING + s]); };
    auto bar_done = [&](uint32_t u) { return smem_addr(&bars[2 * TC_RING + u]); };
    // tiles of this block: blockIdx.x, blockIdx.x + gridDim.x, ...; unit n = column n % nkb of tile n / nkb
    const uint32_t my_tiles = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    const uint32_t total = my_tiles * nkb;

    if (threadIdx.x == 0) {
        dead_flag = 0;
        for (uint32_t s = 0; s < TC_RING; s++) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 32 * TC_WORKER_WARPS);
        }
        mbar_init(bar_done(0), 1);
        mbar_init(bar_done(1), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // zero the digit operand (rows 3..7 of every core matrix stay zero)
    for (uint32_t i = threadIdx.x; i < TC_MAX_K * 8 / 16; i += TC_NT) reinterpret_cast<uint4 *>(smem + TC_OFF_B)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            bool ok = true;
            for (uint32_t n = 0; n < total && ok; n++) {
                const uint32_t tile = blockIdx.x + (n / nkb) * gridDim.x, kb = n % nkb;
                const uint32_t s = n % TC_RING, round = n / TC_RING;
                if (round) ok = tc_wait(bar_empty(s), (round - 1) & 1, dead, a.err, 11);
                if (!ok) break;
                mbar_expect_tx(bar_full(s), TC_UNIT_BYTES);
                bulk_copy_g2s(smem_addr(smem + TC_OFF_RING) + s * TC_UNIT_BYTES,
                              a.w + ((size_t)tile * nkb + kb) * TC_UNIT_BYTES, TC_UNIT_BYTES, bar_full(s));
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issue ------------------------------
        // Unit n is complete in its operand buffer once all worker threads have arrived at hardware barrier
        // 3 + n % 2 (they do not wait there); this warp does wait there, then one thread issues the unit's
        // eight MMAs into accumulator columns 128 (n % 2) ... and commits them to the unit's barrier.
        // The descriptors are worked out once: a single thread issues, and its own instruction stream is what
        // bounds the rate.  The start-address field is the low 14 bits in units of 16 bytes; the offsets added
        // below stay inside it (shared memory ends below 2^18).
        const uint32_t idesc = tc_idesc(16);
        const uint64_t adesc0 = tc_smem_desc_sw128(smem_addr(smem + TC_OFF_A), 1024);
        const uint64_t bdesc0 = tc_smem_desc(smem_addr(smem + TC_OFF_B), 128, 0);
        uint32_t kb = 0;
        for (uint32_t n = 0; n < total; n++) {
            const uint32_t u = n & 1;
            if (u) asm volatile("bar.sync 4, %0;" ::"n"(32 * TC_WORKER_WARPS + 32) : "memory");
            else asm volatile("bar.sync 3, %0;" ::"n"(32 * TC_WORKER_WARPS + 32) : "memory");
            if (lane == 0 && !*dead) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ad = adesc0 + (uint64_t)(u * (TC_A_BYTES >> 4));
                const uint64_t bd = bdesc0 + (uint64_t)(kb * ((256 / 16) * 128 >> 4));
                const uint32_t dcol = tmem_base + u * 128;
#pragma unroll
                for (uint32_t j = 0; j < 8; j++)
                    tc_mma(dcol + 16 * j, ad + (uint64_t)(((j >> 2) * 16384 + (j & 3) * 32) >> 4), bd + (uint64_t)((j * 256) >> 4), idesc);
                tc_commit(bar_done(u));
            }
            __syncwarp();
            kb = kb + 1 == nkb ? 0 : kb + 1;
        }
    } else {
        // ------------------------------ workers ------------------------------
        // Thread (quarter, lane, sub): row r = 32 quarter + lane of the tile (the quarter of tensor memory
        // its warp may read), 32-byte chunks sub * TC_CPT .. of that row (sub-blocks 2c and 2c + 1 each).
        const uint32_t w = warp - 2, sub = w / 4, quarter = warp & 3, r = quarter * 32 + lane;
        for (uint32_t grp = threadIdx.x - 64; grp < a.K / 32; grp += 32 * TC_WORKER_WARPS) tc_stage_group(smem, a.x, grp);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, %0;" ::"n"(32 * TC_WORKER_WARPS) : "memory");
        const float *e = reinterpret_cast<const float *>(smem + TC_OFF_E), *xs = reinterpret_cast<const float *>(smem + TC_OFF_S);
        const uint32_t arow = smem_addr(smem + TC_OFF_A) + (r >> 3) * 1024 + (r & 7) * 128;
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
        const uint32_t ring = smem_addr(smem + TC_OFF_RING) + r * 144;
        // Step n unpacks unit n into operand buffer n % 2, tells the MMA warp (an arrival at a hardware
        // barrier, without waiting), and goes on to finish unit n - 1, whose MMAs were issued a step ago.
        // Buffer n % 2 is free again by then: finishing unit n - 2 waited for its MMAs.  The two barrier
        // numbers alternate so that an early arrival for unit n + 1 cannot be counted for unit n.
        float rowacc = 0.0f;
        bool ok = true;
        // After an expired wait (`ok` false, warp-uniform) the loop keeps its shape, so that every thread still
        // meets every hardware barrier, but waits for nothing and computes nothing.
        for (uint32_t n = 0; n <= total; n++) {
            if (n < total) {
                const uint32_t slot = n % TC_RING, u = n & 1;
                if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_full(slot), (n / TC_RING) & 1, dead, a.err, 13));
                const uint32_t raw = ring + slot * TC_UNIT_BYTES;
                // nibbles -> bytes: low nibbles are sub-block 2c, high nibbles (left as 16 * code) sub-block
                // 2c + 1; sub-block j lies in K panel j / 4 (16 KB) at bytes 32 (j % 4) .. + 31 of the row,
                // 16-byte chunks swizzled by the row index
#pragma unroll
                for (uint32_t cc = 0; cc < (ok ? TC_CPT : 0u); cc++) {
                    const uint32_t c = TC_CPT * sub + cc;
#pragma unroll
                    for (uint32_t core = 0; core < 2; core++) {
                        const uint4 q = lds128(raw + 16 + 32 * c + 16 * core);
                        const uint32_t jl = 2 * c, jh = 2 * c + 1;
                        sts128(arow + u * TC_A_BYTES + (jl >> 2) * 16384 + (((2 * (jl & 3) + core) ^ (r & 7)) << 4),
                               q.x & 0x0f0f0f0fu, q.y & 0x0f0f0f0fu, q.z & 0x0f0f0f0fu, q.w & 0x0f0f0f0fu);
                        sts128(arow + u * TC_A_BYTES + (jh >> 2) * 16384 + (((2 * (jh & 3) + core) ^ (r & 7)) << 4),
                               q.x & 0xf0f0f0f0u, q.y & 0xf0f0f0f0u, q.z & 0xf0f0f0f0u, q.w & 0xf0f0f0f0u);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                if (u) asm volatile("bar.arrive 4, %0;" ::"n"(32 * TC_WORKER_WARPS + 32) : "memory");
                else asm volatile("bar.arrive 3, %0;" ::"n"(32 * TC_WORKER_WARPS + 32) : "memory");
            }
            if (n >= 1) {
                const uint32_t m = n - 1, slot = m % TC_RING, u = m & 1, kb = m % nkb;
                const uint32_t raw = ring + slot * TC_UNIT_BYTES;
                const uint4 hdr = lds128(raw);
                const uint32_t sc_lo = hdr.y & 0x3f3f3f3fu, m_lo = hdr.z & 0x3f3f3f3fu;
                const uint32_t sc_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
                const uint32_t m_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
                const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
                if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_done(u), (m >> 1) & 1, dead, a.err, 14));
                int d[2 * TC_CPT][4] = {};
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (uint32_t q = 0; q < 2 * TC_CPT; q++) tc_ld4(taddr + u * 128 + 16 * (2 * TC_CPT * sub + q), d[q]);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                }
                float acc = 0.0f, neg = 0.0f;
#pragma unroll
                for (uint32_t cc = 0; cc < TC_CPT; cc++) {
                    // six-bit scales and mins of sub-blocks 2c, 2c + 1 in the low bytes of a word each
                    const uint32_t c = TC_CPT * sub + cc, sh = (c & 1) * 16;
                    const uint32_t scw = (c < 2 ? sc_lo : sc_hi) >> sh, mw = (c < 2 ? m_lo : m_hi) >> sh;
                    const float2 e2 = reinterpret_cast<const float2 *>(e)[kb * 4 + c], s2 = reinterpret_cast<const float2 *>(xs)[kb * 4 + c];
                    // |digit sum| <= 32 * 240 * 128 < 2^22: the offset conversion is exact
                    const float f0 = fmaf(i2f(d[2 * cc][2]), 65536.0f, fmaf(i2f(d[2 * cc][1]), 256.0f, i2f(d[2 * cc][0])));
                    const float f1 = fmaf(i2f(d[2 * cc + 1][2]), 65536.0f, fmaf(i2f(d[2 * cc + 1][1]), 256.0f, i2f(d[2 * cc + 1][0])));
                    acc = fmaf(f0, byte2f(scw, 0) * e2.x, acc);
                    acc = fmaf(f1, byte2f(scw, 1) * e2.y, acc);
                    neg = fmaf(byte2f(mw, 0), s2.x, neg);
                    neg = fmaf(byte2f(mw, 1), s2.y, neg);
                }
                rowacc += dm.x * acc - dm.y * neg;
                mbar_arrive(bar_empty(slot));
                if (kb == nkb - 1) {
                    // the row's total: its TC_WPQ threads' parts, added in a fixed order
                    rowpart[sub][r] = rowacc;
                    rowacc = 0.0f;
                    asm volatile("bar.sync 2, %0;" ::"n"(32 * TC_WORKER_WARPS) : "memory");
                    if (sub == 0 && ok) {
                        float t = rowpart[0][r];
#pragma unroll
                        for (uint32_t q = 1; q < TC_WPQ; q++) t += rowpart[q][r];
                        const uint32_t tile = blockIdx.x + (m / nkb) * gridDim.x;
                        a.out[(size_t)tile * TC_TILE_ROWS + r] = t;
                    }
                    asm volatile("bar.sync 2, %0;" ::"n"(32 * TC_WORKER_WARPS) : "memory");
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

// Raw row-major Q4_K blocks -> [tile][column][row in tile][144 bytes].  One thread per 16 bytes.
__global__ void q4k_tile_major_kernel(const uint4 *__restrict__ raw, uint4 *__restrict__ tiled, uint32_t nrows, uint32_t nkb)
{
    const size_t total = (size_t)nrows * nkb * 9;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t part = (uint32_t)(i % 9);
        const size_t blk = i / 9;
        const uint32_t kb = (uint32_t)(blk % nkb), row = (uint32_t)(blk / nkb);
        const uint32_t tile = row / TC_TILE_ROWS, r = row % TC_TILE_ROWS;
        tiled[(((size_t)tile * nkb + kb) * TC_TILE_ROWS + r) * 9 + part] = raw[i];
    }
}

}  // namespace wgb

using namespace wgb;

struct wgb_q4k_tiles {
    uint8_t *w;
    uint32_t nrows, ncols;
    // work areas of the batched product, made by its first call: activation image and product slices
    uint8_t *image;
    float *part;
};

WGB_EXPORT int wgb_q4k_tiles_create(const void *h_blocks, size_t nrows, size_t ncols, void *stream, wgb_q4k_tiles **out)
{
    WGB_REQUIRE(h_blocks && out, "null argument");
    WGB_REQUIRE(nrows > 0 && nrows % TC_TILE_ROWS == 0, "the tensor-core path wants a multiple of %u rows, got %zu", TC_TILE_ROWS, nrows);
    WGB_REQUIRE(ncols > 0 && ncols % 256 == 0, "the tensor-core path wants a multiple of 256 columns, got %zu", ncols);
    int rc = gemv_global_init();
    if (rc) return rc;
    DeviceState *ds = device_state();
    if (!ds) return WGB_ERR_CUDA;
    if (!ds->tiles_attrs) {
        WGB_CUDA(cudaFuncSetAttribute(gemv_q4k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(TC_SMEM + 1024)));
        ds->tiles_attrs = true;
    }
    const size_t bytes = nrows * (ncols / 256) * 144;
    cudaStream_t st = as_stream(stream);
    wgb_q4k_tiles *m = new (std::nothrow) wgb_q4k_tiles();
    if (!m) return fail(WGB_ERR_INVALID, "out of host memory");
    uint8_t *d_raw = nullptr;
    cudaError_t e = cudaMalloc((void **)&m->w, bytes);
    if (e == cudaSuccess) e = cudaMalloc((void **)&d_raw, bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_raw, h_blocks, bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) {
        q4k_tile_major_kernel<<<(unsigned)((bytes / 16 + 255) / 256 < 65535 * 16 ? (bytes / 16 + 255) / 256 : 65535 * 16), 256, 0, st>>>((const uint4 *)d_raw, (uint4 *)m->w, (uint32_t)nrows, (uint32_t)(ncols / 256));
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (d_raw) cudaFree(d_raw);
    if (e != cudaSuccess) {
        if (m->w) cudaFree(m->w);
        delete m;
        return cuda_fail(e, "Q4_K tile-major upload");
    }
    m->nrows = (uint32_t)nrows;
    m->ncols = (uint32_t)ncols;
    *out = m;
    return WGB_OK;
}


WGB_EXPORT int wgb_q4k_tiles_destroy(wgb_q4k_tiles *m)
{
    if (!m) return WGB_OK;
    cudaFree(m->w);
    if (m->image) cudaFree(m->image);
    if (m->part) cudaFree(m->part);
    delete m;
    return WGB_OK;
}

WGB_EXPORT int wgb_gemv_q4k_tiles(const wgb_q4k_tiles *m, const float *d_v, float *d_out, void *stream)
{
    WGB_REQUIRE(m && d_v && d_out, "null argument");
    WGB_REQUIRE(m->ncols <= TC_MAX_K, "the single-vector tensor-core kernel keeps the whole input image in shared memory: up to %u columns, got %u",
                TC_MAX_K, m->ncols);
    TcArgs a = {};
    a.w = m->w;
    a.x = d_v;
    a.out = d_out;
    a.nrows = m->nrows;
    a.K = m->ncols;
    a.err = gemv_status_word();
    const uint32_t ntiles = m->nrows / TC_TILE_ROWS;
    const uint32_t grid = ntiles < (uint32_t)sm_count() ? ntiles : (uint32_t)sm_count();
    gemv_q4k_tc_kernel<<<grid, TC_NT, TC_SMEM + 1024, as_stream(stream)>>>(a);
    WGB_LAUNCH_CHECK("gemv_q4k_tc_kernel");
    return WGB_OK;
}

// The same product for up to eight input vectors at once (the kernel of the batched prompt prefill, prefill.cu):
// d_v [n_vec][ncols] -> d_out [n_vec][nrows].  The first call on a matrix allocates its work areas (activation
// image, product slices), so make it outside stream capture; calls on one matrix must be ordered on a stream.
WGB_EXPORT int wgb_gemm_q4k_tiles(wgb_q4k_tiles *m, const float *d_v, size_t n_vec, float *d_out, void *stream)
{
    WGB_REQUIRE(m && d_v && d_out, "null argument");
    WGB_REQUIRE(n_vec >= 1 && n_vec <= PF_TOK, "between 1 and %u input vectors, got %zu", PF_TOK, n_vec);
    cudaStream_t st = as_stream(stream);
    const uint32_t ns = prefill_gemm_splits(m->nrows, m->ncols);
    if (!m->image) {
        uint8_t *image = nullptr;
        float *part = nullptr;
        cudaError_t e = cudaMalloc((void **)&image, prefill_image_bytes(m->ncols));
        if (e == cudaSuccess) e = cudaMalloc((void **)&part, (size_t)PF_MAX_SPLIT * PF_TOK * m->nrows * sizeof(float));
        if (e == cudaSuccess) e = cudaMemset(image, 0, prefill_image_bytes(m->ncols));
        if (e != cudaSuccess) {
            if (image) cudaFree(image);
            if (part) cudaFree(part);
            return cuda_fail(e, "work areas of the batched product");
        }
        m->image = image;
        m->part = part;
    }
    WGB_CUDA(cudaMemsetAsync(d_out, 0, n_vec * m->nrows * sizeof(float), st));
    // image of the inputs (they are not written: no slices are folded into them)
    int rc = launch_prefill_norm_image(const_cast<float *>(d_v), m->ncols, nullptr, 0, 0, nullptr, 0.0f, m->ncols, (uint32_t)n_vec, m->image, nullptr, 0, st);
    if (!rc) rc = launch_gemm_q4k_tiles(m->w, m->nrows, m->ncols, m->image, (uint32_t)n_vec, m->part, m->nrows, ns, st);
    // d_out (zero) += the slices
    if (!rc) rc = launch_prefill_norm_image(d_out, m->nrows, m->part, ns, m->nrows, nullptr, 0.0f, m->nrows, (uint32_t)n_vec, nullptr, nullptr, 0, st);
    return rc;
}

// Waits for the device and reports whether a bounded wait inside any matrix-vector kernel has expired since
// the last report (stand-alone launches are asynchronous and cannot return that themselves).
WGB_EXPORT int wgb_device_status(void)
{
    WGB_CUDA(cudaDeviceSynchronize());
    return gemv_check_status();
}
