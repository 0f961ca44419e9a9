// Batched prompt prefill: up to eight prompt positions per pass through the layer stack, with the Q4_K
// matrix products on the fifth-generation tensor cores.
//
// The reference feeds the prompt through its decode path one token at a time (wgml-chat/src/chat_llama2.rs:
// 104-116, 169-204: every prompt position is a full Llama2::dispatch whose logits are thrown away).  Here a pass
// takes eight positions: each weight is read once for the eight, and the products run as tcgen05.mma kind::i8
// on the fixed-point image of the activations that the batch-1 kernels use (three signed byte digits per
// element, one power-of-two exponent per 32 columns), so a prompt position costs what the reference's CPU twin
// computes for it (models/llama2/cpu.rs:83-178) up to the order of the f32 additions.
//
// Matrix product (gemm_q4k_tc_kernel).  Weights tile-major as for the single-vector tensor-core kernel
// (gemv_tc.cu).  Work item = (tile of 128 rows, slice of the super-block columns); an item's units (one
// super-block column each: 18 KB of weights and the 8.5 KB slice of the activation image that goes with it)
// stream through a ring of shared-memory stages.  Eight warps unpack the nibbles of a unit into the A operand
// (128 x 256 bytes, 128-byte swizzle), one thread issues eight MMAs per unit (one per 32-column sub-block;
// M = 128, N = 32: rows 8 d + t of the B operand hold digit d of position t, rows 24..31 are zero, K = 32) into
// 256 columns of tensor memory (two such sets alternate), and eight other warps read the sums back
// (tcgen05.ld), apply digit weights, exponents, six-bit scales and the min term in FP32 and keep one running
// sum per position.  The three roles only meet through barriers, so the unpacking of unit n + 1, the MMAs of
// unit n and the finishing of unit n - 1 overlap.  Each item leaves its partial rows in out[slice][position][row]; whoever consumes the
// product adds the slices in a fixed order, so results do not depend on the schedule.
// Every wait is bounded in time; after an expired wait the loops keep their shape (all hardware barriers are
// still met) but do nothing, and a code is left in the device's status word.
#include "kernels.h"
#include "tc_common.cuh"

#include <cstdlib>

namespace wgb {

constexpr uint32_t TB_IMG_DIGITS = 16 * 4 * 128;                          // 16 K-cores x 4 row groups x 128 bytes
constexpr uint32_t TB_IMG_BYTES = TB_IMG_DIGITS + 2 * 8 * PF_TOK * 4;     // + exponents and sums [group][position]
constexpr uint32_t TB_STAGE = TB_IMG_BYTES + TC_UNIT_BYTES;
constexpr uint32_t TB_RING = 4;
constexpr uint32_t TB_UNPACK_WARPS = 8;                                   // build the A operand of unit n
constexpr uint32_t TB_FINISH_WARPS = 8;                                   // read unit n - 1's sums and apply scales
constexpr uint32_t TB_NT = 32 * (2 + TB_UNPACK_WARPS + TB_FINISH_WARPS);     // 4 + 16 and 8 + 16 warps measured 4-8 % slower
static_assert(16 % TB_UNPACK_WARPS == 0 && TB_UNPACK_WARPS % 4 == 0 && 32 % TB_FINISH_WARPS == 0 && TB_FINISH_WARPS % 4 == 0 && TB_FINISH_WARPS <= 16,
              "whole chunks per unpacking thread, whole sub-block pairs per finishing thread, four warps per quarter of the rows");
constexpr uint32_t TB_TMEM_COLS = 512;                                    // two sets of eight 32-column results
constexpr uint32_t TB_OFF_A = 0;                                          // two operand buffers (units alternate)
constexpr uint32_t TB_OFF_RING = TB_OFF_A + 2 * TC_A_BYTES;
constexpr uint32_t TB_SMEM = TB_OFF_RING + TB_RING * TB_STAGE;
static_assert(PF_TOK == 8, "one core matrix (eight rows) per digit");
static_assert(TB_IMG_BYTES == prefill_image_unit_bytes(), "the image layout other kernels rely on");
static_assert(TB_STAGE % 128 == 0 && TB_IMG_BYTES % 16 == 0, "stages keep the operand alignment");
static_assert(TB_SMEM + 1024 + 20 * 1024 <= 227 * 1024, "shared memory budget (dynamic + static)");

bool pdl_enabled()
{
    static const bool on = [] {
        const char *env = getenv("WGB_NO_PDL");
        return !(env && env[0] == '1');
    }();
    return on;
}

size_t prefill_image_bytes(uint32_t K) { return (size_t)(K / 256) * TB_IMG_BYTES; }

// Up to three matrices with the same input (q / k / v, gate / up) share a launch: their tiles are numbered through.
struct TbArgs {
    const uint8_t *w[3];      // tile-major blocks: [tile][column][128 rows][144 bytes]
    float *out[3];            // [nsplit][PF_TOK][out_stride]
    uint32_t tile0[3];        // first tile of each matrix in the launch's numbering (tile0[0] = 0)
    uint32_t out_stride[3];
    uint32_t nmat, ntiles;    // matrices, tiles over all of them
    const uint8_t *img;       // activation image: [column][TB_IMG_BYTES]
    uint32_t nkb, nsplit, ntok;
    uint32_t *err;
};
// Matrix of a tile in the launch's numbering.
__device__ __forceinline__ uint32_t tb_matrix_of(const TbArgs &a, uint32_t tile)
{
    return (a.nmat > 2 && tile >= a.tile0[2]) ? 2u : (a.nmat > 1 && tile >= a.tile0[1]) ? 1u : 0u;
}

__global__ void __launch_bounds__(TB_NT, 1) gemm_q4k_tc_kernel(const __grid_constant__ TbArgs a)
{
    extern __shared__ uint8_t tb_smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * TB_RING + 4];
    __shared__ float rowpart[TB_FINISH_WARPS / 4][PF_TOK][TC_TILE_ROWS];
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t dead_flag;
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)tb_smem_raw + 1023) & ~(uintptr_t)1023);
    volatile uint32_t *dead = &dead_flag;

    pdl_launch_dependents();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nkb = a.nkb, nsplit = a.nsplit, nitems = a.ntiles * nsplit;
    auto bar_full = [&](uint32_t s) { return smem_addr(&bars[s]); };
    auto bar_empty = [&](uint32_t s) { return smem_addr(&bars[TB_RING + s]); };
    auto bar_done = [&](uint32_t u) { return smem_addr(&bars[2 * TB_RING + u]); };        // the unit's MMAs have completed
    auto bar_tfree = [&](uint32_t u) { return smem_addr(&bars[2 * TB_RING + 2 + u]); };   // its accumulators have been read
    auto stage = [&](uint32_t s) { return smem_addr(smem + TB_OFF_RING) + s * TB_STAGE; };
    uint32_t total = 0;
    for (uint32_t i = blockIdx.x; i < nitems; i += gridDim.x) {
        const uint32_t sp = i % nsplit;
        total += (sp + 1) * nkb / nsplit - sp * nkb / nsplit;
    }

    if (threadIdx.x == 0) {
        dead_flag = 0;
        for (uint32_t s = 0; s < TB_RING; s++) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 32 * (TB_UNPACK_WARPS + TB_FINISH_WARPS));
        }
        for (uint32_t u = 0; u < 2; u++) {
            mbar_init(bar_done(u), 1);
            mbar_init(bar_tfree(u), 32 * TB_FINISH_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(TB_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    // barriers and tensor memory are set up while the preceding launch (which writes the image) still runs
    pdl_wait();

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0 && total) {
            UnitWalk w;
            w.set(blockIdx.x, nsplit, nkb);
            bool ok = true;
            for (uint32_t n = 0; n < total && ok; n++) {
                const uint32_t s = n % TB_RING, round = n / TB_RING;
                if (round) ok = tc_wait(bar_empty(s), (round - 1) & 1, dead, a.err, 21);
                if (!ok) break;
                mbar_expect_tx(bar_full(s), TB_STAGE);
                bulk_copy_g2s(stage(s), a.img + (size_t)w.kb * TB_IMG_BYTES, TB_IMG_BYTES, bar_full(s));
                const uint32_t mi = tb_matrix_of(a, w.tile);
                bulk_copy_g2s(stage(s) + TB_IMG_BYTES, a.w[mi] + ((size_t)(w.tile - a.tile0[mi]) * nkb + w.kb) * TC_UNIT_BYTES, TC_UNIT_BYTES,
                              bar_full(s));
                w.next(nsplit, nkb, gridDim.x);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issue ------------------------------
        // Unit n is complete in operand buffer n % 2 once all unpacking threads have arrived at hardware barrier
        // 3 + n % 2 (they do not wait there); this warp waits there, then one thread -- once the accumulators of
        // unit n - 2 have been read -- issues the unit's eight MMAs into accumulator columns 256 (n % 2) ... and
        // commits them to the unit's barrier.  The B operand is read in place from the unit's stage (K-major, no
        // swizzle: core matrices of eight positions x 16 columns, the four row groups of a K-core 128 bytes apart,
        // K-cores 512 bytes apart).
        const uint32_t idesc = tc_idesc(32);
        const uint64_t adesc0 = tc_smem_desc_sw128(smem_addr(smem + TB_OFF_A), 1024);
        bool ok = true;
        for (uint32_t n = 0; n < total; n++) {
            const uint32_t u = n & 1, s = n % TB_RING;
            if (u) asm volatile("bar.sync 4, %0;" ::"n"(32 * TB_UNPACK_WARPS + 32) : "memory");
            else asm volatile("bar.sync 3, %0;" ::"n"(32 * TB_UNPACK_WARPS + 32) : "memory");
            if (lane == 0 && ok && !*dead) {
                ok = tc_wait(bar_full(s), (n / TB_RING) & 1, dead, a.err, 22);
                if (ok && n >= 2) ok = tc_wait(bar_tfree(u), ((n - 2) >> 1) & 1, dead, a.err, 25);
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ad = adesc0 + (uint64_t)(u * (TC_A_BYTES >> 4));
                    const uint64_t bd = tc_smem_desc(stage(s), 512, 128);
                    const uint32_t dcol = tmem_base + u * 256;
#pragma unroll
                    for (uint32_t j = 0; j < 8; j++)
                        tc_mma(dcol + 32 * j, ad + (uint64_t)(((j >> 2) * 16384 + (j & 3) * 32) >> 4), bd + (uint64_t)((j * 1024) >> 4), idesc);
                    tc_commit(bar_done(u));
                }
            }
            __syncwarp();
        }
    } else if (warp < 2 + TB_UNPACK_WARPS) {
        // ------------------------------ unpacking ------------------------------
        // Thread (quarter, lane, half): row r = 32 quarter + lane of the tile, 32-byte chunks 2 half and 2 half + 1
        // of that row's nibbles (chunk c = sub-blocks 2 c and 2 c + 1).  Unit n goes into operand buffer n % 2 as
        // soon as its stage is full and the MMAs of unit n - 2 have read the buffer; the thread then tells the
        // MMA warp (an arrival at a hardware barrier, without waiting) and is done with the stage.
        const uint32_t half = (warp - 2) >> 2, r = (warp & 3) * 32 + lane;
        const uint32_t arow = smem_addr(smem + TB_OFF_A) + (r >> 3) * 1024 + (r & 7) * 128;
        bool ok = true;
        // After an expired wait (`ok` false, warp-uniform) the loop keeps its shape, so that every thread still meets
        // every hardware barrier, but waits for nothing and computes nothing.
        for (uint32_t n = 0; n < total; n++) {
            const uint32_t slot = n % TB_RING, u = n & 1;
            if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_full(slot), (n / TB_RING) & 1, dead, a.err, 23));
            if (ok && n >= 2) ok = __all_sync(0xffffffffu, tc_wait(bar_done(u), ((n - 2) >> 1) & 1, dead, a.err, 26));
            const uint32_t raw = stage(slot) + TB_IMG_BYTES + r * 144;
            if (ok) {
                // nibbles -> bytes: low nibbles are sub-block 2 c, high nibbles (left as 16 * code) sub-block 2 c + 1;
                // sub-block j lies in K panel j / 4 (16 KB) at bytes 32 (j % 4) .. + 31 of the row, 16-byte chunks
                // swizzled by the row index
#pragma unroll
                for (uint32_t cc = 0; cc < 16 / TB_UNPACK_WARPS; cc++) {
                    const uint32_t c = (16 / TB_UNPACK_WARPS) * half + cc;
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
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (u) asm volatile("bar.arrive 4, %0;" ::"n"(32 * TB_UNPACK_WARPS + 32) : "memory");
            else asm volatile("bar.arrive 3, %0;" ::"n"(32 * TB_UNPACK_WARPS + 32) : "memory");
            mbar_arrive(bar_empty(slot));   // the stage is free once the finishing threads have arrived too
        }
    } else {
        // ------------------------------ finishing ------------------------------
        // Thread (quarter, lane, half): row r = 32 quarter + lane (the quarter of tensor memory its warp may read),
        // sub-blocks 4 half .. 4 half + 3 of the unit.  It reads the row's digit sums of those sub-blocks for the
        // eight positions, frees the accumulators for unit m + 2, and applies scales, exponents and mins.
        const uint32_t half = (warp - 2 - TB_UNPACK_WARPS) >> 2, quarter = warp & 3, r = quarter * 32 + lane;
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
        float rowacc[PF_TOK];
#pragma unroll
        for (uint32_t t = 0; t < PF_TOK; t++) rowacc[t] = 0.0f;
        bool ok = true;
        UnitWalk fin;
        fin.set(blockIdx.x, nsplit, nkb);
        for (uint32_t m = 0; m < total; m++) {
            const uint32_t slot = m % TB_RING, u = m & 1;
            if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_full(slot), (m / TB_RING) & 1, dead, a.err, 27));
            const uint32_t img = stage(slot), raw = img + TB_IMG_BYTES + r * 144;
            uint4 hdr = make_uint4(0u, 0u, 0u, 0u);
            if (ok) hdr = lds128(raw);
            const uint32_t sc_lo = hdr.y & 0x3f3f3f3fu, m_lo = hdr.z & 0x3f3f3f3fu;
            const uint32_t sc_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
            const uint32_t m_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
            const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
            if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_done(u), (m >> 1) & 1, dead, a.err, 24));
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                constexpr uint32_t SPT = 32 / TB_FINISH_WARPS;   // sub-blocks per thread
#pragma unroll
                for (uint32_t cc = 0; cc < SPT / 2; cc++) {
                    // sub-blocks j0 = SPT half + 2 cc and j0 + 1: their six loads are issued before the one wait; the
                    // exponents and sums of the two groups are fetched from the stage meanwhile
                    const uint32_t j0 = SPT * half + 2 * cc;
                    // six-bit scales and mins of sub-blocks j0, j0 + 1 in the two low bytes
                    const uint32_t scw = ((j0 & 4) ? sc_hi : sc_lo) >> (8 * (j0 & 3)), mw = ((j0 & 4) ? m_hi : m_lo) >> (8 * (j0 & 3));
                    int d[2][3][8];
#pragma unroll
                    for (uint32_t q = 0; q < 2; q++)
#pragma unroll
                        for (uint32_t dg = 0; dg < 3; dg++) tc_ld8(taddr + u * 256 + 32 * (j0 + q) + 8 * dg, d[q][dg]);
                    float ev[2][8], sv[2][8];
#pragma unroll
                    for (uint32_t q = 0; q < 2; q++) {
                        const uint32_t eo = img + TB_IMG_DIGITS + (j0 + q) * PF_TOK * 4;   // one float per position
                        const uint4 e0 = lds128(eo), e1 = lds128(eo + 16), s0 = lds128(eo + 8 * PF_TOK * 4), s1 = lds128(eo + 8 * PF_TOK * 4 + 16);
                        ev[q][0] = __uint_as_float(e0.x); ev[q][1] = __uint_as_float(e0.y); ev[q][2] = __uint_as_float(e0.z); ev[q][3] = __uint_as_float(e0.w);
                        ev[q][4] = __uint_as_float(e1.x); ev[q][5] = __uint_as_float(e1.y); ev[q][6] = __uint_as_float(e1.z); ev[q][7] = __uint_as_float(e1.w);
                        sv[q][0] = __uint_as_float(s0.x); sv[q][1] = __uint_as_float(s0.y); sv[q][2] = __uint_as_float(s0.z); sv[q][3] = __uint_as_float(s0.w);
                        sv[q][4] = __uint_as_float(s1.x); sv[q][5] = __uint_as_float(s1.y); sv[q][6] = __uint_as_float(s1.z); sv[q][7] = __uint_as_float(s1.w);
                    }
                    // the block's d and dmin folded into the sub-blocks' scales and mins once per unit
                    const float sc0 = dm.x * byte2f(scw, 0), sc1 = dm.x * byte2f(scw, 1);
                    const float mn0 = -dm.y * byte2f(mw, 0), mn1 = -dm.y * byte2f(mw, 1);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (cc == SPT / 2 - 1) {
                        // every accumulator column this thread reads is in registers: unit m + 2 may overwrite them
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        mbar_arrive(bar_tfree(u));
                    }
#pragma unroll
                    for (uint32_t t = 0; t < PF_TOK; t++) {
                        // the two low digit sums are joined in the integer unit (|.| < 2^31) and take one conversion;
                        // the product of scale and exponent is exact in the exponent (a power of two)
                        const float f0 = fmaf(__int2float_rn(d[0][2][t]), 65536.0f, __int2float_rn(d[0][1][t] * 256 + d[0][0][t]));
                        const float f1 = fmaf(__int2float_rn(d[1][2][t]), 65536.0f, __int2float_rn(d[1][1][t] * 256 + d[1][0][t]));
                        const float mins = fmaf(mn0, sv[0][t], mn1 * sv[1][t]);
                        rowacc[t] += fmaf(f0, sc0 * ev[0][t], fmaf(f1, sc1 * ev[1][t], mins));
                    }
                }
            }
            mbar_arrive(bar_empty(slot));
            if (fin.last()) {
                // the rows' totals over this item's columns: the two threads of a row, in a fixed order
#pragma unroll
                for (uint32_t t = 0; t < PF_TOK; t++) {
                    rowpart[half][t][r] = rowacc[t];
                    rowacc[t] = 0.0f;
                }
                asm volatile("bar.sync 2, %0;" ::"n"(32 * TB_FINISH_WARPS) : "memory");
                if (ok) {
                    constexpr uint32_t NP = TB_FINISH_WARPS / 4, TPT = PF_TOK / NP;   // parts of a row, positions per thread
                    const uint32_t mi = tb_matrix_of(a, fin.tile);
                    float *outp = a.out[mi] + (size_t)(fin.tile - a.tile0[mi]) * TC_TILE_ROWS + r;
                    const uint32_t ostride = a.out_stride[mi];
#pragma unroll
                    for (uint32_t tt = 0; tt < TPT; tt++) {
                        const uint32_t t = TPT * half + tt;
                        float v = rowpart[0][t][r];
#pragma unroll
                        for (uint32_t q = 1; q < NP; q++) v += rowpart[q][t][r];
                        if (t < a.ntok) outp[((size_t)fin.sp * PF_TOK + t) * ostride] = v;
                    }
                }
                asm volatile("bar.sync 2, %0;" ::"n"(32 * TB_FINISH_WARPS) : "memory");
            }
            fin.next(nsplit, nkb, gridDim.x);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TB_TMEM_COLS) : "memory");
    }
}

// Column slices per tile: enough items to fill the machine, at least three units per item, and the count whose
// last wave is fullest.
uint32_t prefill_gemm_splits(uint32_t nrows, uint32_t K)
{
    const uint32_t ntiles = nrows / TC_TILE_ROWS, nkb = K / 256, sms = (uint32_t)sm_count();
    uint32_t best = 1;
    float best_cost = 1e30f;
    for (uint32_t s = 1; s <= PF_MAX_SPLIT && (s == 1 || nkb / s >= 3); s++) {
        const uint32_t items = ntiles * s, waves = (items + sms - 1) / sms;
        // time ~ waves x (units per item + a fixed cost per item of about two units)
        const float cost = (float)waves * ((float)((nkb + s - 1) / s) + 2.0f);
        if (cost < best_cost - 1e-3f) { best_cost = cost; best = s; }
    }
    return best;
}

int launch_gemm_q4k_tiles_multi(uint32_t nmat, const uint8_t *const *w_tiles, const uint32_t *nrows, uint32_t K, const uint8_t *image,
                                uint32_t ntok, float *const *out, const uint32_t *out_stride, uint32_t nsplit, cudaStream_t stream)
{
    WGB_REQUIRE(nmat >= 1 && nmat <= 3 && K % 256 == 0 && ntok >= 1 && ntok <= PF_TOK && nsplit >= 1 && nsplit <= K / 256,
                "batched product: %u matrices, %u columns, %u positions, %u slices", nmat, K, ntok, nsplit);
    DeviceState *ds = device_state();
    if (!ds) return WGB_ERR_CUDA;
    if (!ds->prefill_attrs) {
        WGB_CUDA(cudaFuncSetAttribute(gemm_q4k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(TB_SMEM + 1024)));
        ds->prefill_attrs = true;
    }
    TbArgs a = {};
    for (uint32_t i = 0; i < nmat; i++) {
        WGB_REQUIRE(nrows[i] > 0 && nrows[i] % TC_TILE_ROWS == 0, "batched product: %u rows", nrows[i]);
        a.w[i] = w_tiles[i];
        a.out[i] = out[i];
        a.out_stride[i] = out_stride[i];
        a.tile0[i] = a.ntiles;
        a.ntiles += nrows[i] / TC_TILE_ROWS;
    }
    a.nmat = nmat;
    a.img = image;
    a.nkb = K / 256;
    a.nsplit = nsplit;
    a.ntok = ntok;
    a.err = gemv_status_word();
    const uint32_t items = a.ntiles * nsplit, sms = (uint32_t)sm_count();
    WGB_CUDA(launch_pdl(gemm_q4k_tc_kernel, dim3(items < sms ? items : sms), dim3(TB_NT), TB_SMEM + 1024, stream, a));
    return WGB_OK;
}

int launch_gemm_q4k_tiles(const uint8_t *w_tiles, uint32_t nrows, uint32_t K, const uint8_t *image, uint32_t ntok, float *out,
                          uint32_t out_stride, uint32_t nsplit, cudaStream_t stream)
{
    return launch_gemm_q4k_tiles_multi(1, &w_tiles, &nrows, K, image, ntok, &out, &out_stride, nsplit, stream);
}

// ---- activation image ---------------------------------------------------------------------------------

// Eight threads per (position, 32-column group), four consecutive values each (`v`): writes the three digits of
// the values, and (first thread of the eight) the group's exponent -- odd groups carry the 1/16 of the high
// nibbles -- and the sum of its values.  The eight threads are consecutive lanes of a warp and all take part.
__device__ __forceinline__ void image_quad(uint8_t *__restrict__ image, uint32_t t, uint32_t g, uint32_t j, float4 v)
{
    float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
    }
    // |v| < 2^(ex - 126), so X = v * 2^(148 - ex) stays within +-2^22 after rounding
    uint32_t ex = (__float_as_uint(m) >> 23) & 0xffu;
    ex = ex < 24u ? 24u : (ex > 253u ? 253u : ex);
    const float up = __uint_as_float((275u - ex) << 23), down = __uint_as_float((ex - 21u) << 23);
    const float vv[4] = { v.x, v.y, v.z, v.w };
    uint32_t d0 = 0, d1 = 0, d2 = 0;
#pragma unroll
    for (int b = 0; b < 4; b++) {
        // round to nearest even through the 1.5 * 2^23 offset; with 0x8080 added, bytes 0 and 1 are the signed
        // digits plus 128 and byte 2 is the signed top digit
        const uint32_t y = __float_as_uint(fmaf(vv[b], up, 12582912.0f)) - 0x4b400000u + 0x8080u;
        d0 |= ((y & 0xffu) ^ 0x80u) << (8 * b);
        d1 |= (((y >> 8) & 0xffu) ^ 0x80u) << (8 * b);
        d2 |= ((y >> 16) & 0xffu) << (8 * b);
    }
    // values 4 j .. 4 j + 3 of the group: K-core 2 (g % 8) + j / 4 of the unit, bytes 4 (j % 4) .. of row t
    uint8_t *unit = image + (size_t)(g >> 3) * TB_IMG_BYTES;
    uint8_t *kc = unit + ((g & 7) * 2 + (j >> 2)) * 512 + t * 16 + (j & 3) * 4;
    *reinterpret_cast<uint32_t *>(kc) = d0;
    *reinterpret_cast<uint32_t *>(kc + 128) = d1;
    *reinterpret_cast<uint32_t *>(kc + 256) = d2;
    if (j == 0) {
        float *es = reinterpret_cast<float *>(unit + TB_IMG_DIGITS);
        es[(g & 7) * PF_TOK + t] = (g & 1) ? down * 0.0625f : down;
        es[8 * PF_TOK + (g & 7) * PF_TOK + t] = sum;
    }
}

// x = residual (+ the slices of a product); optionally written back; optionally RMS-normalised (RmsNorm,
// ops/rms_norm.wgsl:36-67: (x * 1/sqrt(mean(x^2) + eps)) * w); its image, and optionally the values themselves.
// One block per position; positions >= ntok get an all-zero image.  K is a multiple of 32, so the eight threads of
// a group are always whole.
__global__ void __launch_bounds__(1024) prefill_norm_image_kernel(float *__restrict__ x, uint32_t x_stride, const float *__restrict__ part,
                                                                 uint32_t nsplit, uint32_t part_stride, const float *__restrict__ norm_w,
                                                                 float eps, uint32_t K, uint32_t ntok, uint8_t *__restrict__ image,
                                                                 float *__restrict__ xn, uint32_t xn_stride)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t t = blockIdx.x;
    __shared__ float red[32];
    __shared__ float scale_s;
    if (t >= ntok) {
        for (uint32_t i = threadIdx.x; i < K / 4; i += 1024) image_quad(image, t, i >> 3, i & 7, make_float4(0.f, 0.f, 0.f, 0.f));
        return;
    }
    float *xr = x + (size_t)t * x_stride;
    if (part || norm_w) {
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x * 4; i < K; i += 4096) {
            float4 v = *reinterpret_cast<const float4 *>(xr + i);
            for (uint32_t s = 0; s < (part ? nsplit : 0u); s++) {
                const float4 p = *reinterpret_cast<const float4 *>(part + ((size_t)s * PF_TOK + t) * part_stride + i);
                v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
            }
            if (part) *reinterpret_cast<float4 *>(xr + i) = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.0f;
            for (int i = 0; i < 32; i++) tot += red[i];
            scale_s = 1.0f / sqrtf(tot / (float)K + eps);
        }
        __syncthreads();
    }
    if (!image) return;
    const float scale = norm_w ? scale_s : 1.0f;
    // the same thread reads back what it wrote above (element 4 (threadIdx.x + 1024 k))
    for (uint32_t i = threadIdx.x; i < K / 4; i += 1024) {
        float4 v = *reinterpret_cast<const float4 *>(xr + 4 * i);
        if (norm_w) {
            const float4 w = *reinterpret_cast<const float4 *>(norm_w + 4 * i);
            v.x = (v.x * scale) * w.x; v.y = (v.y * scale) * w.y; v.z = (v.z * scale) * w.z; v.w = (v.w * scale) * w.w;
        }
        if (xn) *reinterpret_cast<float4 *>(xn + (size_t)t * xn_stride + 4 * i) = v;
        image_quad(image, t, i >> 3, i & 7, v);
    }
}

// h = up * gate / (1 + exp(-gate)) (Silu, ops/silu.wgsl:19-27) from the slices of the two products; its image and,
// optionally, the values.  One thread per four columns.
__global__ void __launch_bounds__(256) prefill_silu_image_kernel(const float *__restrict__ gate, uint32_t gsplit, const float *__restrict__ upv,
                                                                 uint32_t usplit, uint32_t stride, uint32_t K, uint32_t ntok,
                                                                 uint8_t *__restrict__ image, float *__restrict__ h, uint32_t h_stride)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t t = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
    if (i >= K / 4) return;   // K / 4 is a multiple of 8: the eight threads of a group leave together
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t < ntok) {
        float4 a = v, b = v;
        for (uint32_t s = 0; s < gsplit; s++) {
            const float4 p = *reinterpret_cast<const float4 *>(gate + ((size_t)s * PF_TOK + t) * stride + 4 * i);
            a.x += p.x; a.y += p.y; a.z += p.z; a.w += p.w;
        }
        for (uint32_t s = 0; s < usplit; s++) {
            const float4 p = *reinterpret_cast<const float4 *>(upv + ((size_t)s * PF_TOK + t) * stride + 4 * i);
            b.x += p.x; b.y += p.y; b.z += p.z; b.w += p.w;
        }
        v.x = b.x * (a.x / (1.0f + expf(-a.x)));
        v.y = b.y * (a.y / (1.0f + expf(-a.y)));
        v.z = b.z * (a.z / (1.0f + expf(-a.z)));
        v.w = b.w * (a.w / (1.0f + expf(-a.w)));
        if (h) *reinterpret_cast<float4 *>(h + (size_t)t * h_stride + 4 * i) = v;
    }
    image_quad(image, t, i >> 3, i & 7, v);
}

int launch_prefill_norm_image(float *x, uint32_t x_stride, const float *part, uint32_t nsplit, uint32_t part_stride, const float *norm_w,
                              float eps, uint32_t K, uint32_t ntok, uint8_t *image, float *xn, uint32_t xn_stride, cudaStream_t stream)
{
    WGB_REQUIRE(K % 128 == 0 && ntok <= PF_TOK, "activation image of %u columns (whole warps of four-column threads), %u positions", K, ntok);
    WGB_CUDA(launch_pdl(prefill_norm_image_kernel, dim3(image ? PF_TOK : ntok), dim3(1024), 0, stream, x, x_stride, part, nsplit, part_stride, norm_w,
                        eps, K, ntok, image, xn, xn_stride));
    return WGB_OK;
}

int launch_prefill_silu_image(const float *gate, uint32_t gsplit, const float *up, uint32_t usplit, uint32_t stride, uint32_t K,
                              uint32_t ntok, uint8_t *image, float *h, uint32_t h_stride, cudaStream_t stream)
{
    WGB_REQUIRE(K % 128 == 0 && ntok <= PF_TOK, "activation image of %u columns (whole warps of four-column threads), %u positions", K, ntok);
    WGB_CUDA(launch_pdl(prefill_silu_image_kernel, dim3((K / 4 + 255) / 256, PF_TOK), dim3(256), 0, stream, gate, gsplit, up, usplit, stride, K, ntok,
                        image, h, h_stride));
    return WGB_OK;
}

// ---- GPT-2 passes: LayerNorm, fused-qkv split, GELU ---------------------------------------------------------

// x (+= the slices of a product and its bias, written back); then LayerNorm (ops/layernorm.wgsl:28-80: two passes,
// epsilon 1e-5) times gain plus bias (the Mul / Add dispatches of models/gpt2/transformer.rs:295-310, 372-386);
// its image and the values.  One 1024-thread block per position; positions >= ntok get an all-zero image.
__global__ void __launch_bounds__(1024) prefill_ln_image_kernel(float *__restrict__ x, uint32_t x_stride, const float *__restrict__ part,
                                                                uint32_t nsplit, uint32_t part_stride, const float *__restrict__ fold_bias,
                                                                const float *__restrict__ gain, const float *__restrict__ bias, uint32_t K,
                                                                uint32_t ntok, uint8_t *__restrict__ image, float *__restrict__ xn,
                                                                uint32_t xn_stride)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t t = blockIdx.x;
    __shared__ float red[32];
    __shared__ float stat_s;
    if (t >= ntok) {
        for (uint32_t i = threadIdx.x; i < K / 4; i += 1024) image_quad(image, t, i >> 3, i & 7, make_float4(0.f, 0.f, 0.f, 0.f));
        return;
    }
    float *xr = x + (size_t)t * x_stride;
    auto block_total = [&](float v) {
        v = warp_sum(v);
        __syncthreads();   // red[] and stat_s of the previous use have been read
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.0f;
            for (int i = 0; i < 32; i++) tot += red[i];
            stat_s = tot;
        }
        __syncthreads();
        return stat_s;
    };
    float sm = 0.0f;
    for (uint32_t i = threadIdx.x * 4; i < K; i += 4096) {
        float4 v = *reinterpret_cast<const float4 *>(xr + i);
        if (part) {
            for (uint32_t s = 0; s < nsplit; s++) {
                const float4 p = *reinterpret_cast<const float4 *>(part + ((size_t)s * PF_TOK + t) * part_stride + i);
                v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
            }
            if (fold_bias) {
                const float4 b = *reinterpret_cast<const float4 *>(fold_bias + i);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            *reinterpret_cast<float4 *>(xr + i) = v;
        }
        sm += (v.x + v.y) + (v.z + v.w);
    }
    if (!image) return;   // only the fold was wanted
    const float mean = block_total(sm) / (float)K;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x * 4; i < K; i += 4096) {   // the same thread reads back what it wrote above
        const float4 v = *reinterpret_cast<const float4 *>(xr + i);
        const float dx = v.x - mean, dy = v.y - mean, dz = v.z - mean, dw = v.w - mean;
        ss = fmaf(dx, dx, ss); ss = fmaf(dy, dy, ss); ss = fmaf(dz, dz, ss); ss = fmaf(dw, dw, ss);
    }
    const float scale = 1.0f / sqrtf(block_total(ss) / (float)K + 1.0e-5f);
    for (uint32_t i = threadIdx.x; i < K / 4; i += 1024) {
        float4 v = *reinterpret_cast<const float4 *>(xr + 4 * i);
        const float4 g = *reinterpret_cast<const float4 *>(gain + 4 * i), b = *reinterpret_cast<const float4 *>(bias + 4 * i);
        v.x = ((v.x - mean) * scale) * g.x + b.x; v.y = ((v.y - mean) * scale) * g.y + b.y;
        v.z = ((v.z - mean) * scale) * g.z + b.z; v.w = ((v.w - mean) * scale) * g.w + b.w;
        if (xn) *reinterpret_cast<float4 *>(xn + (size_t)t * xn_stride + 4 * i) = v;
        image_quad(image, t, i >> 3, i & 7, v);
    }
}

int launch_prefill_ln_image(float *x, uint32_t x_stride, const float *part, uint32_t nsplit, uint32_t part_stride, const float *fold_bias,
                            const float *gain, const float *bias, uint32_t K, uint32_t ntok, uint8_t *image, float *xn, uint32_t xn_stride,
                            cudaStream_t stream)
{
    WGB_REQUIRE(K % 128 == 0 && ntok <= PF_TOK && (!image || (gain && bias)), "LayerNorm image of %u columns, %u positions", K, ntok);
    WGB_CUDA(launch_pdl(prefill_ln_image_kernel, dim3(image ? PF_TOK : ntok), dim3(1024), 0, stream, x, x_stride, part, nsplit, part_stride, fold_bias,
                        gain, bias, K, ntok, image, xn, xn_stride));
    return WGB_OK;
}

// The three Copy dispatches of models/gpt2/transformer.rs:329-353 for a batch of positions, with the bias of the fused
// qkv product: rows [0, n) -> q_out[t], [n, 2n) -> key cache row pos0 + t, [2n, 3n) -> value cache row ([seq][n] caches).
__global__ void __launch_bounds__(256) prefill_qkv_split_kernel(const float *__restrict__ qkv, uint32_t nsplit, const float *__restrict__ bias,
                                                                float *__restrict__ q_out, float *__restrict__ k_cache,
                                                                float *__restrict__ v_cache, uint32_t n, uint32_t pos0)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t i = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    if (i >= 3 * n) return;
    float v = 0.0f;
    for (uint32_t s = 0; s < nsplit; s++) v += qkv[((size_t)s * PF_TOK + t) * (3 * n) + i];
    if (bias) v += bias[i];
    if (i < n) q_out[(size_t)t * n + i] = v;
    else if (i < 2 * n) k_cache[(size_t)(pos0 + t) * n + (i - n)] = v;
    else v_cache[(size_t)(pos0 + t) * n + (i - 2 * n)] = v;
}

int launch_prefill_qkv_split(const float *qkv, uint32_t nsplit, const float *bias, float *q_out, float *k_cache, float *v_cache, uint32_t n,
                             uint32_t pos0, uint32_t ntok, cudaStream_t stream)
{
    WGB_CUDA(launch_pdl(prefill_qkv_split_kernel, dim3((3 * n + 255) / 256, ntok), dim3(256), 0, stream, qkv, nsplit, bias, q_out, k_cache, v_cache, n,
                        pos0));
    return WGB_OK;
}

// h = gelu(product + bias) (Unary GELU, ops/unary.wgsl:50-52: 0.5 x (1 + tanh(0.7978846 x (1 + 0.044715 x^2)))) from
// the slices of the product; its image and, optionally, the values.  One thread per four columns.
__device__ __forceinline__ float gelu_ref(float x)
{
    return 0.5f * x * (1.0f + tanhf(0.7978846f * x * (1.0f + 0.044715f * x * x)));
}
__global__ void __launch_bounds__(256) prefill_gelu_image_kernel(const float *__restrict__ part, uint32_t nsplit, uint32_t stride,
                                                                 const float *__restrict__ bias, uint32_t K, uint32_t ntok,
                                                                 uint8_t *__restrict__ image, float *__restrict__ h, uint32_t h_stride)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t t = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
    if (i >= K / 4) return;   // K / 4 is a multiple of 32: whole warps leave together
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t < ntok) {
        for (uint32_t s = 0; s < nsplit; s++) {
            const float4 p = *reinterpret_cast<const float4 *>(part + ((size_t)s * PF_TOK + t) * stride + 4 * i);
            v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        if (bias) {
            const float4 b = *reinterpret_cast<const float4 *>(bias + 4 * i);
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        }
        v.x = gelu_ref(v.x); v.y = gelu_ref(v.y); v.z = gelu_ref(v.z); v.w = gelu_ref(v.w);
        if (h) *reinterpret_cast<float4 *>(h + (size_t)t * h_stride + 4 * i) = v;
    }
    image_quad(image, t, i >> 3, i & 7, v);
}

int launch_prefill_gelu_image(const float *part, uint32_t nsplit, uint32_t stride, const float *bias, uint32_t K, uint32_t ntok, uint8_t *image,
                              float *h, uint32_t h_stride, cudaStream_t stream)
{
    WGB_REQUIRE(K % 128 == 0 && ntok <= PF_TOK, "activation image of %u columns (whole warps of four-column threads), %u positions", K, ntok);
    WGB_CUDA(launch_pdl(prefill_gelu_image_kernel, dim3((K / 4 + 255) / 256, PF_TOK), dim3(256), 0, stream, part, nsplit, stride, bias, K, ntok, image, h,
                        h_stride));
    return WGB_OK;
}

// positions[t] = pos0 + t (the learned positional rows of a pass are looked up through device scalars)
__global__ void prefill_positions_kernel(uint32_t *positions, uint32_t pos0)
{
    if (threadIdx.x < PF_TOK) positions[threadIdx.x] = pos0 + threadIdx.x;
}
int launch_prefill_positions(uint32_t *positions, uint32_t pos0, cudaStream_t stream)
{
    prefill_positions_kernel<<<1, 32, 0, stream>>>(positions, pos0);
    WGB_LAUNCH_CHECK("prefill_positions_kernel");
    return WGB_OK;
}

// ---- RoPE + KV append for a batch of positions ------------------------------------------------------

// The work of the OpAssign / RoPE dispatches of models/llama2/transformer.rs:343-365 and the write into the cache
// rows, for positions pos0 .. pos0 + ntok - 1: q, k, v are sums of product slices (+ bias); q is rotated into
// `q_out`, k rotated into the key cache, v copied into the value cache (head-major caches: element e of head h
// at position p sits at (h * seq_len + p) * head_size + e).
__global__ void __launch_bounds__(128) prefill_rope_append_kernel(PrefillQkv a)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t i = blockIdx.x * 128 + threadIdx.x, t = blockIdx.y;   // pair index over q
    if (2 * i >= a.q_dim) return;
    const uint32_t pos = a.pos0 + t, half = a.head_size / 2;
    float sn, cs;
    sincosf((float)pos * a.freq[i % half], &sn, &cs);
    uint32_t ia, ib;
    if (a.variant == WGB_ROPE_ORIGINAL) { ia = 2 * i; ib = ia + 1; }
    else { ia = i + ((2 * i) / a.head_size) * half; ib = ia + half; }
    auto gather = [&](const float *p, uint32_t nsplit, uint32_t stride, const float *bias, uint32_t idx) {
        float v = 0.0f;
        for (uint32_t s = 0; s < nsplit; s++) v += p[((size_t)s * PF_TOK + t) * stride + idx];
        return v + (bias ? bias[idx] : 0.0f);
    };
    float x = gather(a.q, a.q_split, a.q_stride, a.bq, ia), y = gather(a.q, a.q_split, a.q_stride, a.bq, ib);
    a.q_out[(size_t)t * a.q_dim + ia] = cs * x - sn * y;
    a.q_out[(size_t)t * a.q_dim + ib] = sn * x + cs * y;
    if (2 * i < a.kv_dim) {
        float *kc = a.k_cache + (size_t)pos * a.head_size, *vc = a.v_cache + (size_t)pos * a.head_size;
        const size_t da = (size_t)(ia / a.head_size) * a.seq_len * a.head_size + ia % a.head_size;
        const size_t db = (size_t)(ib / a.head_size) * a.seq_len * a.head_size + ib % a.head_size;
        x = gather(a.k, a.k_split, a.kv_stride, a.bk, ia);
        y = gather(a.k, a.k_split, a.kv_stride, a.bk, ib);
        kc[da] = cs * x - sn * y;
        kc[db] = sn * x + cs * y;
        vc[da] = gather(a.v, a.v_split, a.kv_stride, a.bv, ia);
        vc[db] = gather(a.v, a.v_split, a.kv_stride, a.bv, ib);
    }
}

int launch_prefill_rope_append(const PrefillQkv &a, uint32_t ntok, cudaStream_t stream)
{
    WGB_CUDA(launch_pdl(prefill_rope_append_kernel, dim3((a.q_dim / 2 + 127) / 128, ntok), dim3(128), 0, stream, a));
    return WGB_OK;
}

// ---- causal attention of a batch of positions ----------------------------------------------------------

// BatchedMultiqueryAttention (ops/batched_multiquery_attention.wgsl:38-99) for positions pos0 + t, t < ntok, each
// attending to cache rows 0 .. pos0 + t.  One block per (query head, group of TQ = 2, 4 or 8 positions); the block walks the
// cache rows in chunks of 256 with a running maximum and sum (rescaled), one thread per row for the scores, one
// thread per value column (times a quarter of the chunk's rows) for the weighted sum.
constexpr uint32_t PA_TQ_MIN = 2;    // positions per block: 2, 4 or 8 (more on longer contexts: a block's positions share its cache reads)
constexpr uint32_t PA_CHUNK = 256;
constexpr uint32_t PA_MAX_SPLIT = 8; // blocks that may share the rows of one (head, pair of positions)
template <uint32_t TQ>
__global__ void __launch_bounds__(256) prefill_attention_kernel(const float *__restrict__ q, const float *__restrict__ k_cache,
                                                                const float *__restrict__ v_cache, float *__restrict__ out, uint32_t q_dim,
                                                                uint32_t head_size, uint32_t kv_mul, uint32_t row_stride, uint32_t head_stride,
                                                                uint32_t pos0, uint32_t ntok, uint8_t *__restrict__ image,
                                                                float *__restrict__ scratch, uint32_t *__restrict__ counters)
{
    extern __shared__ float pa_smem[];
    pdl_launch_dependents();
    pdl_wait();
    // blockIdx.z: which of gridDim.z interleaved subsets of the 256-row chunks this block walks (long contexts)
    const uint32_t h = blockIdx.x, t0 = blockIdx.y * TQ, nz = gridDim.z, z = blockIdx.z;
    if (t0 >= ntok) {
        // with an image the grid covers all PF_TOK positions: the unused ones get zero digits
        if (image && z == 0)
            for (uint32_t i = threadIdx.x; i < TQ * head_size / 4; i += 256)
                image_quad(image, t0 + i / (head_size / 4), (h * head_size + 4 * (i % (head_size / 4))) >> 5, i & 7, make_float4(0.f, 0.f, 0.f, 0.f));
        return;
    }
    const uint32_t nq = ntok - t0 < TQ ? ntok - t0 : TQ;
    float *qs = pa_smem;                          // [TQ][head_size]
    float *sc = qs + TQ * head_size;           // [TQ][PA_CHUNK]
    float *accs = sc + TQ * PA_CHUNK;          // [4][TQ][head_size]
    __shared__ float red[TQ][8];
    __shared__ float m_run[TQ], l_run[TQ], m_new[TQ], resc[TQ];
    // cache row p of KV head g at p * row_stride + g * head_stride (head-major caches: head_size, seq_len * head_size;
    // the reference layout [seq_len][kv_dim]: kv_dim, head_size)
    const float *kh = k_cache + (size_t)(h / kv_mul) * head_stride;
    const float *vh = v_cache + (size_t)(h / kv_mul) * head_stride;
    const float inv_sqrt = 1.0f / sqrtf((float)head_size);
    for (uint32_t i = threadIdx.x; i < TQ * head_size; i += 256) {
        const uint32_t tq = i / head_size, e = i % head_size;
        qs[i] = tq < nq ? q[(size_t)(t0 + tq) * q_dim + h * head_size + e] : 0.0f;
    }
    if (threadIdx.x < TQ) { m_run[threadIdx.x] = -INFINITY; l_run[threadIdx.x] = 0.0f; }
    // value columns: thread = (quarter of the chunk's rows, column group); head sizes up to 256 (four columns each)
    const uint32_t cg = threadIdx.x & 63, rq = threadIdx.x >> 6;
    float4 acc[TQ];
#pragma unroll
    for (uint32_t tq = 0; tq < TQ; tq++) acc[tq] = make_float4(0.f, 0.f, 0.f, 0.f);
    __syncthreads();
    const uint32_t last = pos0 + t0 + nq - 1;     // furthest row any of the block's positions attends to
    for (uint32_t c0 = z * PA_CHUNK; c0 <= last; c0 += nz * PA_CHUNK) {
        // scores of row c0 + thread for the block's positions
        const uint32_t row = c0 + threadIdx.x;
        float s[TQ];
#pragma unroll
        for (uint32_t tq = 0; tq < TQ; tq++) s[tq] = 0.0f;
        if (row <= last) {
            const float4 *kr = reinterpret_cast<const float4 *>(kh + (size_t)row * row_stride);
#pragma unroll 8
            for (uint32_t e = 0; e < head_size / 4; e++) {
                const float4 kv = kr[e];
#pragma unroll
                for (uint32_t tq = 0; tq < TQ; tq++) {
                    const float4 qv = *reinterpret_cast<const float4 *>(qs + tq * head_size + 4 * e);
                    s[tq] += kv.x * qv.x + kv.y * qv.y + kv.z * qv.z + kv.w * qv.w;
                }
            }
        }
#pragma unroll
        for (uint32_t tq = 0; tq < TQ; tq++) {
            const bool live = tq < nq && row <= pos0 + t0 + tq;
            s[tq] = live ? s[tq] * inv_sqrt : -INFINITY;
            const float mx = warp_max(s[tq]);
            if ((threadIdx.x & 31) == 0) red[tq][threadIdx.x >> 5] = mx;
        }
        __syncthreads();
        if (threadIdx.x < TQ) {
            float mx = m_run[threadIdx.x];
            for (int i = 0; i < 8; i++) mx = fmaxf(mx, red[threadIdx.x][i]);
            m_new[threadIdx.x] = mx;
            resc[threadIdx.x] = mx == -INFINITY ? 1.0f : expf(m_run[threadIdx.x] - mx);
            m_run[threadIdx.x] = mx;
        }
        __syncthreads();
#pragma unroll
        for (uint32_t tq = 0; tq < TQ; tq++) {
            const float p = s[tq] == -INFINITY ? 0.0f : expf(s[tq] - m_new[tq]);
            sc[tq * PA_CHUNK + threadIdx.x] = p;
            const float ps = warp_sum(p);
            if ((threadIdx.x & 31) == 0) red[tq][threadIdx.x >> 5] = ps;   // the maxima in red[] were consumed before the last barrier
        }
        __syncthreads();
        if (threadIdx.x < TQ) {
            float tot = 0.0f;
            for (int i = 0; i < 8; i++) tot += red[threadIdx.x][i];
            l_run[threadIdx.x] = l_run[threadIdx.x] * resc[threadIdx.x] + tot;
        }
        // weighted values: rows c0 + 64 rq .. + 63 of the chunk, columns 4 cg .. + 3
#pragma unroll
        for (uint32_t tq = 0; tq < TQ; tq++) {
            const float rs = resc[tq];
            acc[tq].x *= rs; acc[tq].y *= rs; acc[tq].z *= rs; acc[tq].w *= rs;
        }
        if (4 * cg < head_size) {
            const uint32_t r_end = min(c0 + 64 * (rq + 1), last + 1);
#pragma unroll 4
            for (uint32_t rr = c0 + 64 * rq; rr < r_end; rr++) {
                const float4 vv = *reinterpret_cast<const float4 *>(vh + (size_t)rr * row_stride + 4 * cg);
#pragma unroll
                for (uint32_t tq = 0; tq < TQ; tq++) {
                    const float p = sc[tq * PA_CHUNK + (rr - c0)];
                    acc[tq].x = fmaf(p, vv.x, acc[tq].x); acc[tq].y = fmaf(p, vv.y, acc[tq].y);
                    acc[tq].z = fmaf(p, vv.z, acc[tq].z); acc[tq].w = fmaf(p, vv.w, acc[tq].w);
                }
            }
        }
        __syncthreads();   // sc[], red[] and resc[] are rewritten by the next chunk
    }
    if (4 * cg < head_size) {
#pragma unroll
        for (uint32_t tq = 0; tq < TQ; tq++) *reinterpret_cast<float4 *>(accs + ((size_t)rq * TQ + tq) * head_size + 4 * cg) = acc[tq];
    }
    __syncthreads();
    if (nz > 1) {
        // Several blocks share the rows of this (head, pair of positions): each leaves its unnormalised sum, maximum
        // and denominator in scratch, and the last to arrive (a counter that wraps back to zero) merges them in the
        // order of blockIdx.z, so the result does not depend on which block that is.
        __shared__ uint32_t s_last;
        const uint32_t pstride = head_size + 4;   // per position: head_size sums, maximum, denominator
        float *mine = scratch + (((size_t)h * gridDim.y + blockIdx.y) * nz + z) * TQ * pstride;
        for (uint32_t i = threadIdx.x; i < TQ * head_size / 4; i += 256) {
            const uint32_t tq = i / (head_size / 4), e4 = i % (head_size / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t r4 = 0; r4 < 4; r4++) {
                const float4 p = *reinterpret_cast<const float4 *>(accs + ((size_t)r4 * TQ + tq) * head_size + 4 * e4);
                v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
            }
            *reinterpret_cast<float4 *>(mine + tq * pstride + 4 * e4) = v;
        }
        if (threadIdx.x < TQ) {
            mine[threadIdx.x * pstride + head_size] = m_run[threadIdx.x];
            mine[threadIdx.x * pstride + head_size + 1] = l_run[threadIdx.x];
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicInc(counters + h * gridDim.y + blockIdx.y, nz - 1) == nz - 1;
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        const float *all = scratch + ((size_t)h * gridDim.y + blockIdx.y) * nz * TQ * pstride;
        for (uint32_t i = threadIdx.x; i < TQ * head_size / 4; i += 256) {
            const uint32_t tq = i / (head_size / 4), e4 = i % (head_size / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tq < nq) {
                float mx = -INFINITY;
                for (uint32_t zz = 0; zz < nz; zz++) mx = fmaxf(mx, __ldcg(all + ((size_t)zz * TQ + tq) * pstride + head_size));
                float den = 0.0f;
                for (uint32_t zz = 0; zz < nz; zz++) {
                    const float *p = all + ((size_t)zz * TQ + tq) * pstride;
                    const float mz = __ldcg(p + head_size);
                    if (mz == -INFINITY) continue;   // a subset without a row this position attends to
                    const float wgt = expf(mz - mx);
                    const float4 a4 = __ldcg(reinterpret_cast<const float4 *>(p + 4 * e4));
                    den = fmaf(wgt, __ldcg(p + head_size + 1), den);
                    v.x = fmaf(wgt, a4.x, v.x); v.y = fmaf(wgt, a4.y, v.y); v.z = fmaf(wgt, a4.z, v.z); v.w = fmaf(wgt, a4.w, v.w);
                }
                v.x /= den; v.y /= den; v.z /= den; v.w /= den;
                *reinterpret_cast<float4 *>(out + (size_t)(t0 + tq) * q_dim + h * head_size + 4 * e4) = v;
            }
            if (image) image_quad(image, t0 + tq, (h * head_size + 4 * e4) >> 5, e4 & 7, v);
        }
        return;
    }
    // the block's output, four columns per thread; with `image` (head sizes that are multiples of 64, so that whole
    // warps take part) also its slice of the activation image of the output projection's input
    for (uint32_t i = threadIdx.x; i < TQ * head_size / 4; i += 256) {
        const uint32_t tq = i / (head_size / 4), e4 = i % (head_size / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tq < nq) {
            for (uint32_t r4 = 0; r4 < 4; r4++) {
                const float4 p = *reinterpret_cast<const float4 *>(accs + ((size_t)r4 * TQ + tq) * head_size + 4 * e4);
                v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
            }
            const float l = l_run[tq];
            v.x /= l; v.y /= l; v.z /= l; v.w /= l;
            *reinterpret_cast<float4 *>(out + (size_t)(t0 + tq) * q_dim + h * head_size + 4 * e4) = v;
        }
        if (image) image_quad(image, t0 + tq, (h * head_size + 4 * e4) >> 5, e4 & 7, v);
    }
}

bool prefill_attention_writes_image(uint32_t head_size) { return head_size % 64 == 0; }

size_t prefill_attention_scratch_floats(uint32_t n_heads, uint32_t head_size)
{
    return (size_t)n_heads * PF_TOK * PA_MAX_SPLIT * (head_size + 4);   // per (head, position, block): sums, maximum, denominator
}
size_t prefill_attention_counters(uint32_t n_heads) { return (size_t)n_heads * (PF_TOK / PA_TQ_MIN); }

template <uint32_t TQ>
static int launch_prefill_attention_tq(const float *q, const float *k_cache, const float *v_cache, float *out, uint32_t n_heads, uint32_t head_size,
                                       uint32_t kv_mul, uint32_t row_stride, uint32_t head_stride, uint32_t pos0, uint32_t ntok, uint8_t *image,
                                       float *scratch, uint32_t *counters, uint32_t chunks, cudaStream_t stream)
{
    const size_t smem = (size_t)(TQ * head_size + TQ * PA_CHUNK + 4 * TQ * head_size) * sizeof(float);
    // Long contexts: the chunks of a (head, group of positions) are dealt to several blocks, enough to fill the machine
    // about twice, at most one block per chunk.
    const uint32_t groups = (ntok + TQ - 1) / TQ;
    uint32_t nz = 1;
    if (scratch && counters) {
        const uint32_t want = (2u * (uint32_t)sm_count()) / (n_heads * groups);
        nz = want < 1 ? 1u : want;
        if (nz > chunks) nz = chunks;
        if (nz > PA_MAX_SPLIT) nz = PA_MAX_SPLIT;
    }
    WGB_CUDA(launch_pdl(prefill_attention_kernel<TQ>, dim3(n_heads, image ? PF_TOK / TQ : groups, nz), dim3(256), smem, stream, q, k_cache, v_cache, out,
                        n_heads * head_size, head_size, kv_mul, row_stride, head_stride, pos0, ntok, image, scratch, counters));
    return WGB_OK;
}

int launch_prefill_attention(const float *q, const float *k_cache, const float *v_cache, float *out, uint32_t n_heads, uint32_t head_size,
                             uint32_t kv_mul, uint32_t row_stride, uint32_t head_stride, uint32_t pos0, uint32_t ntok, uint8_t *image,
                             float *scratch, uint32_t *counters, cudaStream_t stream)
{
    WGB_REQUIRE(!image || prefill_attention_writes_image(head_size), "prompt attention writes the image only for head sizes that are multiples of 64, got %u",
                head_size);
    WGB_REQUIRE(head_size % 4 == 0 && head_size <= 256 && ntok >= 1 && ntok <= PF_TOK, "prompt attention: head size %u, %u positions", head_size,
                ntok);
    // Positions per block: two on short contexts (most blocks), four and eight as the cache rows to read grow, provided
    // the chunks can still be dealt to enough blocks.
    const uint32_t chunks = (pos0 + ntok + PA_CHUNK - 1) / PA_CHUNK;
    const bool split = scratch && counters;
    if (split && chunks >= 8 && head_size <= 128)
        return launch_prefill_attention_tq<8>(q, k_cache, v_cache, out, n_heads, head_size, kv_mul, row_stride, head_stride, pos0, ntok, image, scratch, counters, chunks, stream);
    if (split && chunks >= 3)
        return launch_prefill_attention_tq<4>(q, k_cache, v_cache, out, n_heads, head_size, kv_mul, row_stride, head_stride, pos0, ntok, image, scratch, counters, chunks, stream);
    return launch_prefill_attention_tq<2>(q, k_cache, v_cache, out, n_heads, head_size, kv_mul, row_stride, head_stride, pos0, ntok, image, scratch, counters, chunks, stream);
}

// Raw row-major Q4_K blocks -> [tile][column][row in tile][144 bytes].  One thread per 16 bytes.
__global__ void prefill_tile_major_kernel(const uint4 *__restrict__ raw, uint4 *__restrict__ tiled, uint32_t nrows, uint32_t nkb)
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

int prefill_tile_major(const QMat &m, uint8_t **out, cudaStream_t stream)
{
    WGB_REQUIRE(m.qtype == WGB_Q4_K && !m.planar && m.nrows % TC_TILE_ROWS == 0 && m.ncols % 256 == 0, "not a tileable Q4_K matrix");
    const size_t bytes = (size_t)m.nrows * m.bpr * 144;
    WGB_CUDA(cudaMalloc((void **)out, bytes));
    const size_t blocks = (bytes / 16 + 255) / 256;
    prefill_tile_major_kernel<<<(unsigned)(blocks < 65535u * 16u ? blocks : 65535u * 16u), 256, 0, stream>>>((const uint4 *)m.p[0], (uint4 *)*out,
                                                                                                             m.nrows, m.bpr);
    WGB_LAUNCH_CHECK("prefill_tile_major_kernel");
    return WGB_OK;
}

bool prefill_tileable(const QMat &m) { return m.qtype == WGB_Q4_K && !m.planar && m.nrows % TC_TILE_ROWS == 0 && m.ncols % 256 == 0; }

}  // namespace wgb
