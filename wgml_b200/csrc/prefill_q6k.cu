// Batched tensor-core product for Q6_K matrices: the Q6_K counterpart of gemm_q4k_tc_kernel (prefill.cu), used by
// the batched prompt prefill for the matrices a Q4_K_M-style file keeps in Q6_K (attn_v and ffn_down of half the
// layers).  Same operator as GemvQuant::dispatch (crates/wgml/src/ops/gemv_quant.rs:241-348) for up to eight
// input vectors at once; block format and dequantisation as BlockQ6K::dequantize
// (crates/wgml/src/quantization.rs:225-264): value = d * scale[16-column group] * (q - 32).
//
// A Q6_K scale covers 16 columns, half the K extent of one kind::i8 MMA, so it cannot be applied after the MMA as
// in the Q4_K kernel.  It is folded into the weight operand instead: w = scale * (q - 32) is an integer of at
// most 13 bits, written as two byte planes w = 256 hi + lo (lo unsigned, hi signed), and a 256-column
// super-block costs sixteen MMAs (two planes x eight 32-column sub-blocks) that ACCUMULATE in tensor memory:
// Dlo, Dhi [128 rows x 32].  That needs one exponent per input vector for the whole super-block (not one per 32
// columns), so this kernel takes its own image of the activations: three signed byte digits per element against
// the largest magnitude among the 256 columns.  An element's error is below 2^-23 of that maximum, which keeps
// a product within 1e-6 of its output RMS for inputs whose maximum is within a few thousand times their RMS.
// The epilogue per super-block is small: hi and lo sums joined in the integer unit, three conversions, one FMA
// with d * exponent per (row, input vector); one thread per row does it for the eight vectors, so a row's
// running sums live in registers and go straight to the output at the end of an item.
//
// Pipeline as in the Q4_K kernel: producer warp (bulk copies into a ring of stages: the super-block's slice of
// the image and 26 KB of weights), one warp issuing the MMAs, sixteen warps that build the two operand planes of
// unit n, four warps that finish unit n - 1; the roles meet only through barriers.  Bounded waits throughout.
#include "kernels.h"
#include "tc_common.cuh"

namespace wgb {

constexpr uint32_t T6_UNIT_BYTES = TC_TILE_ROWS * 210;                  // ql 128 x 128, qh 128 x 64, scales 128 x 16, d 128 x 2
constexpr uint32_t T6_OFF_QH = TC_TILE_ROWS * 128;
constexpr uint32_t T6_OFF_SC = T6_OFF_QH + TC_TILE_ROWS * 64;
constexpr uint32_t T6_OFF_D = T6_OFF_SC + TC_TILE_ROWS * 16;
constexpr uint32_t T6_IMG_DIGITS = 3 * 16 * 128;                        // 3 digits x 16 K-cores x (8 vectors x 16 bytes)
constexpr uint32_t T6_IMG_BYTES = T6_IMG_DIGITS + PF_TOK * 4;           // + one exponent per vector
constexpr uint32_t T6_STAGE = T6_IMG_BYTES + T6_UNIT_BYTES;
constexpr uint32_t T6_RING = 3;
constexpr uint32_t T6_WORKER_WARPS = 16;                                // build the two operand planes of unit n
constexpr uint32_t T6_FINISH_WARPS = 4;                                 // one thread per row reads unit n - 1's sums
constexpr uint32_t T6_NT = 32 * (2 + T6_WORKER_WARPS + T6_FINISH_WARPS);
constexpr uint32_t T6_TMEM_COLS = 128;                                  // two units x (Dlo, Dhi) x 32 columns
constexpr uint32_t T6_A_BYTES = 2 * TC_A_BYTES;                         // lo plane, hi plane
constexpr uint32_t T6_OFF_RING = 2 * T6_A_BYTES;
constexpr uint32_t T6_SMEM = T6_OFF_RING + T6_RING * T6_STAGE;
static_assert(T6_STAGE % 16 == 0 && T6_IMG_BYTES % 16 == 0, "bulk copies and descriptors want 16-byte granules");
// the MMA reads B rows 24..31 (it has no 24-row shape) from the 2 KB after the digits: they must lie in the stage
static_assert(T6_IMG_DIGITS + 2048 <= T6_STAGE, "the unused fourth row group of the B operand stays inside the stage");
static_assert(T6_SMEM + 1024 + 256 <= 227 * 1024, "shared memory budget");

size_t prefill_image6_bytes(uint32_t K) { return (size_t)(K / 256) * T6_IMG_BYTES; }

struct T6Args {
    const uint8_t *w;     // tile-major units: [tile][column][T6_UNIT_BYTES]
    const uint8_t *img;   // activation image: [column][T6_IMG_BYTES]
    float *out;           // [nsplit][PF_TOK][out_stride]
    uint32_t nrows, nkb, nsplit, ntok, out_stride;
    uint32_t *err;
};

__global__ void __launch_bounds__(T6_NT, 1) gemm_q6k_tc_kernel(const __grid_constant__ T6Args a)
{
    extern __shared__ uint8_t t6_smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * T6_RING + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t dead_flag;
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)t6_smem_raw + 1023) & ~(uintptr_t)1023);
    volatile uint32_t *dead = &dead_flag;

    pdl_launch_dependents();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nkb = a.nkb, nsplit = a.nsplit, nitems = (a.nrows / TC_TILE_ROWS) * nsplit;
    auto bar_full = [&](uint32_t s) { return smem_addr(&bars[s]); };
    auto bar_empty = [&](uint32_t s) { return smem_addr(&bars[T6_RING + s]); };
    auto bar_done = [&](uint32_t u) { return smem_addr(&bars[2 * T6_RING + u]); };        // the unit's MMAs have completed
    auto bar_tfree = [&](uint32_t u) { return smem_addr(&bars[2 * T6_RING + 2 + u]); };   // its accumulators have been read
    auto stage = [&](uint32_t s) { return smem_addr(smem + T6_OFF_RING) + s * T6_STAGE; };
    uint32_t total = 0;
    for (uint32_t i = blockIdx.x; i < nitems; i += gridDim.x) {
        const uint32_t sp = i % nsplit;
        total += (sp + 1) * nkb / nsplit - sp * nkb / nsplit;
    }

    if (threadIdx.x == 0) {
        dead_flag = 0;
        for (uint32_t s = 0; s < T6_RING; s++) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 32 * (T6_WORKER_WARPS + T6_FINISH_WARPS));
        }
        for (uint32_t u = 0; u < 2; u++) {
            mbar_init(bar_done(u), 1);
            mbar_init(bar_tfree(u), 32 * T6_FINISH_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(T6_TMEM_COLS) : "memory");
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
                const uint32_t s = n % T6_RING, round = n / T6_RING;
                if (round) ok = tc_wait(bar_empty(s), (round - 1) & 1, dead, a.err, 31);
                if (!ok) break;
                mbar_expect_tx(bar_full(s), T6_STAGE);
                bulk_copy_g2s(stage(s), a.img + (size_t)w.kb * T6_IMG_BYTES, T6_IMG_BYTES, bar_full(s));
                bulk_copy_g2s(stage(s) + T6_IMG_BYTES, a.w + ((size_t)w.tile * nkb + w.kb) * T6_UNIT_BYTES, T6_UNIT_BYTES, bar_full(s));
                w.next(nsplit, nkb, gridDim.x);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issue ------------------------------
        // Unit n: once all workers have arrived at hardware barrier 3 + n % 2, one thread issues eight MMAs per
        // plane (M = 128, N = 32, K = 32; the first of a plane overwrites, the others accumulate) into
        // columns 64 (n % 2) (lo) and 64 (n % 2) + 32 (hi), and commits them to the unit's barrier.  B is read in
        // place from the stage: K-major, no swizzle, core matrices of eight vectors x 16 columns, K-cores 128 bytes
        // apart, the digits (row groups) 2 KB apart.
        const uint32_t idesc_lo = tc_idesc(32, 0), idesc_hi = tc_idesc(32, 1);
        const uint64_t adesc0 = tc_smem_desc_sw128(smem_addr(smem), 1024);
        for (uint32_t n = 0; n < total; n++) {
            const uint32_t u = n & 1, s = n % T6_RING;
            if (u) asm volatile("bar.sync 4, %0;" ::"n"(32 * T6_WORKER_WARPS + 32) : "memory");
            else asm volatile("bar.sync 3, %0;" ::"n"(32 * T6_WORKER_WARPS + 32) : "memory");
            if (lane == 0 && !*dead && tc_wait(bar_full(s), (n / T6_RING) & 1, dead, a.err, 32) &&
                (n < 2 || tc_wait(bar_tfree(u), ((n - 2) >> 1) & 1, dead, a.err, 35))) {   // the accumulators of unit n - 2 have been read
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t bd = tc_smem_desc(stage(s), 128, 2048);
                const uint32_t dcol = tmem_base + u * 64;
#pragma unroll
                for (uint32_t plane = 0; plane < 2; plane++) {
                    const uint64_t ad = adesc0 + (uint64_t)((u * T6_A_BYTES + plane * TC_A_BYTES) >> 4);
#pragma unroll
                    for (uint32_t j = 0; j < 8; j++)
                        tc_mma_acc(dcol + 32 * plane, ad + (uint64_t)(((j >> 2) * 16384 + (j & 3) * 32) >> 4), bd + (uint64_t)((j * 256) >> 4),
                                   plane ? idesc_hi : idesc_lo, j ? 1u : 0u);
                }
                tc_commit(bar_done(u));
            }
            __syncwarp();
        }
    } else if (warp < 2 + T6_WORKER_WARPS) {
        // ------------------------------ operand ------------------------------
        // Thread (quarter, lane, sub): row r = 32 quarter + lane of the tile, 32-weight groups sub and 4 + sub of the
        // row's super-block (columns 32 sub .. of each 128-column half, the layout of BlockQ6K::dequantize).  Unit n
        // goes into operand buffer n % 2 once its stage is full and the MMAs of unit n - 2 have read the buffer.
        const uint32_t w = warp - 2, sub = w / 4, quarter = warp & 3, r = quarter * 32 + lane;
        const uint32_t arow = smem_addr(smem) + (r >> 3) * 1024 + (r & 7) * 128;
        const uint32_t nib_shift = 4 * (sub >> 1), h_shift = 2 * sub;
        bool ok = true;
        // After an expired wait (`ok` false, warp-uniform) the loop keeps its shape, so that every thread still meets
        // every hardware barrier, but waits for nothing and computes nothing.
        for (uint32_t n = 0; n < total; n++) {
            const uint32_t slot = n % T6_RING, u = n & 1;
            if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_full(slot), (n / T6_RING) & 1, dead, a.err, 33));
            if (ok && n >= 2) ok = __all_sync(0xffffffffu, tc_wait(bar_done(u), ((n - 2) >> 1) & 1, dead, a.err, 36));
            const uint32_t wbase = stage(slot) + T6_IMG_BYTES;
            if (ok) {
                const uint4 scq = lds128(wbase + T6_OFF_SC + r * 16);   // the row's sixteen int8 scales
#pragma unroll
                for (uint32_t half = 0; half < 2; half++) {
#pragma unroll
                    for (uint32_t c = 0; c < 2; c++) {
                        // weights l = 16 c .. 16 c + 15 of group 4 half + sub: low or high nibbles of ql[64 half +
                        // 32 (sub & 1) + l], two more bits from qh[32 half + l] >> 2 sub, scale 8 half + 2 sub + c
                        // (the 16-byte pieces of a row's ql, and of a pair of rows' qh, are stored at piece index ^ row
                        // bits, so that the eight lanes of a quarter warp read eight different bank groups)
                        const uint4 qlq = lds128(wbase + r * 128 + (((4 * half + 2 * (sub & 1) + c) ^ (r & 7)) << 4));
                        const uint4 qhq = lds128(wbase + T6_OFF_QH + (r >> 1) * 128 + (((4 * (r & 1) + 2 * half + c) ^ ((r >> 1) & 7)) << 4));
                        // scale 8 half + 2 sub + c: word 2 half + sub / 2 of the sixteen, byte 2 (sub % 2) + c
                        const uint32_t sw = (sub >> 1) ? (half ? scq.w : scq.y) : (half ? scq.z : scq.x);
                        const int s = (int)(signed char)((sw >> (8 * (2 * (sub & 1) + c))) & 0xffu);
                        const int cst = -0x00200020 * s;   // (q1 - 32, q0 - 32) * s = (q1, q0) * s - (32, 32) * s
                        const uint32_t qlw[4] = { qlq.x, qlq.y, qlq.z, qlq.w }, qhw[4] = { qhq.x, qhq.y, qhq.z, qhq.w };
                        uint32_t lo[4], hi[4];
#pragma unroll
                        for (uint32_t k = 0; k < 4; k++) {
                            const uint32_t q = ((qlw[k] >> nib_shift) & 0x0f0f0f0fu) | (((qhw[k] >> h_shift) & 0x03030303u) << 4);
                            // two 16-bit lanes per word: q0 | q1 << 16 and q2 | q3 << 16, times the scale; a negative low
                            // lane has borrowed one from the high lane, which is given back
                            int r0 = (int)__byte_perm(q, 0u, 0x4140) * s + cst, r1 = (int)__byte_perm(q, 0u, 0x4342) * s + cst;
                            r0 += (r0 & 0x8000) << 1;
                            r1 += (r1 & 0x8000) << 1;
                            lo[k] = __byte_perm((uint32_t)r0, (uint32_t)r1, 0x6420);
                            hi[k] = __byte_perm((uint32_t)r0, (uint32_t)r1, 0x7531);
                        }
                        // columns 128 half + 32 sub + 16 c ..: K panel `half`, 16-byte chunk 2 sub + c of the row (swizzled)
                        const uint32_t off = u * T6_A_BYTES + half * 16384 + (((2 * sub + c) ^ (r & 7)) << 4);
                        sts128(arow + off, lo[0], lo[1], lo[2], lo[3]);
                        sts128(arow + off + TC_A_BYTES, hi[0], hi[1], hi[2], hi[3]);
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (u) asm volatile("bar.arrive 4, %0;" ::"n"(32 * T6_WORKER_WARPS + 32) : "memory");
            else asm volatile("bar.arrive 3, %0;" ::"n"(32 * T6_WORKER_WARPS + 32) : "memory");
            mbar_arrive(bar_empty(slot));   // the stage is free once the finishing threads have arrived too
        }
    } else {
        // ------------------------------ finishing ------------------------------
        // One thread per row (r = 32 quarter + lane, the quarter of tensor memory its warp may read): the row's lo and
        // hi digit sums of unit m for the eight input vectors, joined, converted and added to the row's running sums.
        const uint32_t quarter = warp & 3, r = quarter * 32 + lane;
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
        float rowacc[PF_TOK];
#pragma unroll
        for (uint32_t t = 0; t < PF_TOK; t++) rowacc[t] = 0.0f;
        bool ok = true;
        UnitWalk fin;
        fin.set(blockIdx.x, nsplit, nkb);
        for (uint32_t m = 0; m < total; m++) {
            const uint32_t slot = m % T6_RING, u = m & 1;
            if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_full(slot), (m / T6_RING) & 1, dead, a.err, 37));
            const uint32_t img = stage(slot), wbase = img + T6_IMG_BYTES;
            // d of the row's block and the exponents of the eight input vectors
            uint32_t dbits = 0;
            uint4 ea = make_uint4(0u, 0u, 0u, 0u), eb = ea;
            if (ok) {
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dbits) : "r"(wbase + T6_OFF_D + r * 2));
                ea = lds128(img + T6_IMG_DIGITS);
                eb = lds128(img + T6_IMG_DIGITS + 16);
            }
            const float d = __half2float(__ushort_as_half((unsigned short)dbits));
            const float ev[PF_TOK] = { __uint_as_float(ea.x), __uint_as_float(ea.y), __uint_as_float(ea.z), __uint_as_float(ea.w),
                                       __uint_as_float(eb.x), __uint_as_float(eb.y), __uint_as_float(eb.z), __uint_as_float(eb.w) };
            if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_done(u), (m >> 1) & 1, dead, a.err, 34));
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                int dl[3][8], dh[3][8];
#pragma unroll
                for (uint32_t dg = 0; dg < 3; dg++) {
                    tc_ld8(taddr + u * 64 + 8 * dg, dl[dg]);
                    tc_ld8(taddr + u * 64 + 32 + 8 * dg, dh[dg]);
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(bar_tfree(u));   // unit m + 2 may overwrite the accumulators
#pragma unroll
                for (uint32_t t = 0; t < PF_TOK; t++) {
                    // |hi| <= 256 * 16 * 128 and |lo| <= 256 * 255 * 128: 256 hi + lo stays below 2^28
                    const int t0 = dh[0][t] * 256 + dl[0][t], t1 = dh[1][t] * 256 + dl[1][t], t2 = dh[2][t] * 256 + dl[2][t];
                    const float f = fmaf(__int2float_rn(t2), 65536.0f, fmaf(__int2float_rn(t1), 256.0f, __int2float_rn(t0)));
                    rowacc[t] = fmaf(f, d * ev[t], rowacc[t]);
                }
            }
            mbar_arrive(bar_empty(slot));
            if (fin.last()) {
#pragma unroll
                for (uint32_t t = 0; t < PF_TOK; t++) {
                    if (ok && t < a.ntok) a.out[((size_t)fin.sp * PF_TOK + t) * a.out_stride + (size_t)fin.tile * TC_TILE_ROWS + r] = rowacc[t];
                    rowacc[t] = 0.0f;
                }
            }
            fin.next(nsplit, nkb, gridDim.x);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T6_TMEM_COLS) : "memory");
    }
}

int launch_gemm_q6k_tiles(const uint8_t *w_tiles, uint32_t nrows, uint32_t K, const uint8_t *image, uint32_t ntok, float *out,
                          uint32_t out_stride, uint32_t nsplit, cudaStream_t stream)
{
    WGB_REQUIRE(nrows % TC_TILE_ROWS == 0 && K % 256 == 0 && ntok >= 1 && ntok <= PF_TOK && nsplit >= 1 && nsplit <= K / 256,
                "batched Q6_K product: %u x %u, %u vectors, %u slices", nrows, K, ntok, nsplit);
    DeviceState *ds = device_state();
    if (!ds) return WGB_ERR_CUDA;
    if (!ds->prefill6_attrs) {
        WGB_CUDA(cudaFuncSetAttribute(gemm_q6k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(T6_SMEM + 1024)));
        ds->prefill6_attrs = true;
    }
    T6Args a = {};
    a.w = w_tiles;
    a.img = image;
    a.out = out;
    a.nrows = nrows;
    a.nkb = K / 256;
    a.nsplit = nsplit;
    a.ntok = ntok;
    a.out_stride = out_stride;
    a.err = gemv_status_word();
    const uint32_t items = nrows / TC_TILE_ROWS * nsplit, sms = (uint32_t)sm_count();
    WGB_CUDA(launch_pdl(gemm_q6k_tc_kernel, dim3(items < sms ? items : sms), dim3(T6_NT), T6_SMEM + 1024, stream, a));
    return WGB_OK;
}

// Image of `ntok` vectors x [t][K] for the Q6_K product: one warp per (super-block column, vector), eight values
// per lane.  Vectors >= ntok get zero digits.
__global__ void __launch_bounds__(256) prefill_image6_kernel(const float *__restrict__ x, uint32_t x_stride, uint32_t nkb, uint32_t ntok,
                                                             uint8_t *__restrict__ image)
{
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t wid = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wid >= nkb * PF_TOK) return;
    const uint32_t kb = wid / PF_TOK, t = wid % PF_TOK;
    float v[8] = { 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f };
    if (t < ntok) {
        const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)t * x_stride + 256 * kb + 8 * lane);
        const float4 a = src[0], b = src[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(v[i]));
    m = warp_max(m);
    // |v| < 2^(ex - 126), so X = v * 2^(148 - ex) stays within +-2^22 after rounding
    uint32_t ex = (__float_as_uint(m) >> 23) & 0xffu;
    ex = ex < 24u ? 24u : (ex > 253u ? 253u : ex);
    const float up = __uint_as_float((275u - ex) << 23), down = __uint_as_float((ex - 21u) << 23);
    uint32_t dig[3][2];
#pragma unroll
    for (int wd = 0; wd < 2; wd++) {
        uint32_t d0 = 0, d1 = 0, d2 = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            // round to nearest even through the 1.5 * 2^23 offset; with 0x8080 added, bytes 0 and 1 are the signed
            // digits plus 128 and byte 2 is the signed top digit
            const uint32_t y = __float_as_uint(fmaf(v[4 * wd + b], up, 12582912.0f)) - 0x4b400000u + 0x8080u;
            d0 |= ((y & 0xffu) ^ 0x80u) << (8 * b);
            d1 |= (((y >> 8) & 0xffu) ^ 0x80u) << (8 * b);
            d2 |= ((y >> 16) & 0xffu) << (8 * b);
        }
        dig[0][wd] = d0; dig[1][wd] = d1; dig[2][wd] = d2;
    }
    // values 8 lane .. 8 lane + 7: K-core lane / 2, bytes 8 (lane % 2) .. of row t; digit g 2 KB further on
    uint8_t *unit = image + (size_t)kb * T6_IMG_BYTES;
    uint8_t *p = unit + (lane >> 1) * 128 + t * 16 + (lane & 1) * 8;
#pragma unroll
    for (int g = 0; g < 3; g++) *reinterpret_cast<uint2 *>(p + g * 2048) = make_uint2(dig[g][0], dig[g][1]);
    if (lane == 0) reinterpret_cast<float *>(unit + T6_IMG_DIGITS)[t] = down;
}

int launch_prefill_image6(const float *x, uint32_t x_stride, uint32_t K, uint32_t ntok, uint8_t *image, cudaStream_t stream)
{
    WGB_REQUIRE(K % 256 == 0 && ntok <= PF_TOK, "Q6_K activation image of %u columns, %u vectors", K, ntok);
    const uint32_t warps = K / 256 * PF_TOK;
    WGB_CUDA(launch_pdl(prefill_image6_kernel, dim3((warps * 32 + 255) / 256), dim3(256), 0, stream, x, x_stride, K / 256, ntok, image));
    return WGB_OK;
}

// Planar Q6_K matrix (qmatrix.cuh) -> [tile][column][ql 128 x 128 | qh 128 x 64 | scales 128 x 16 | d 128 x 2], the
// 16-byte pieces of ql rows and qh row pairs permuted (piece index ^ row bits) for conflict-free shared-memory reads.
__global__ void prefill_tile_major6_kernel(QMat m, uint8_t *__restrict__ tiled)
{
    const uint32_t nkb = m.bpr;
    const size_t units = (size_t)(m.nrows / TC_TILE_ROWS) * nkb;
    // 13 sixteen-byte pieces per row and unit (8 of ql, 4 of qh, 1 of scales), then the d of the row
    const size_t total = units * TC_TILE_ROWS * 14;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t piece = (uint32_t)(i % 14);
        const size_t ru = i / 14;
        const uint32_t r = (uint32_t)(ru % TC_TILE_ROWS);
        const size_t unit = ru / TC_TILE_ROWS;
        const uint32_t kb = (uint32_t)(unit % nkb), tile = (uint32_t)(unit / nkb);
        const size_t row = (size_t)tile * TC_TILE_ROWS + r;
        uint8_t *dst = tiled + unit * T6_UNIT_BYTES;
        if (piece < 8)
            reinterpret_cast<uint4 *>(dst + r * 128)[piece ^ (r & 7)] = reinterpret_cast<const uint4 *>(m.p[0] + row * m.pitch[0] + (size_t)kb * 128)[piece];
        else if (piece < 12)
            reinterpret_cast<uint4 *>(dst + T6_OFF_QH + (r >> 1) * 128)[(4 * (r & 1) + piece - 8) ^ ((r >> 1) & 7)] =
                reinterpret_cast<const uint4 *>(m.p[1] + row * m.pitch[1] + (size_t)kb * 64)[piece - 8];
        else if (piece == 12)
            *reinterpret_cast<uint4 *>(dst + T6_OFF_SC + r * 16) = *reinterpret_cast<const uint4 *>(m.p[2] + row * m.pitch[2] + (size_t)kb * 16);
        else
            *reinterpret_cast<uint16_t *>(dst + T6_OFF_D + r * 2) = *reinterpret_cast<const uint16_t *>(m.p[3] + row * m.pitch[3] + (size_t)kb * 2);
    }
}

bool prefill_tileable6(const QMat &m) { return m.qtype == WGB_Q6_K && m.planar && m.nrows % TC_TILE_ROWS == 0 && m.ncols % 256 == 0; }

int prefill_tile_major6(const QMat &m, uint8_t **out, cudaStream_t stream)
{
    WGB_REQUIRE(prefill_tileable6(m), "not a tileable Q6_K matrix");
    const size_t bytes = (size_t)m.nrows * m.bpr * 210;
    WGB_CUDA(cudaMalloc((void **)out, bytes));
    const size_t threads = (size_t)m.nrows * m.bpr * 14, blocks = (threads + 255) / 256;
    prefill_tile_major6_kernel<<<(unsigned)(blocks < 65535u * 16u ? blocks : 65535u * 16u), 256, 0, stream>>>(m, *out);
    WGB_LAUNCH_CHECK("prefill_tile_major6_kernel");
    return WGB_OK;
}

}  // namespace wgb

using namespace wgb;

// Stand-alone entry points (tests and measurement): a Q6_K matrix in the tile-major layout and its batched product.
struct wgb_q6k_tiles {
    uint8_t *w;
    uint32_t nrows, ncols;
    uint8_t *image;   // work areas, made by the first product
    float *part;
};

WGB_EXPORT int wgb_q6k_tiles_create(const void *h_blocks, size_t nrows, size_t ncols, void *stream, wgb_q6k_tiles **out)
{
    WGB_REQUIRE(h_blocks && out, "null argument");
    WGB_REQUIRE(nrows > 0 && nrows % TC_TILE_ROWS == 0, "the tensor-core path wants a multiple of %u rows, got %zu", TC_TILE_ROWS, nrows);
    WGB_REQUIRE(ncols > 0 && ncols % 256 == 0, "the tensor-core path wants a multiple of 256 columns, got %zu", ncols);
    int rc = gemv_global_init();
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    wgb_quant_matrix *planar = nullptr;
    if ((rc = qmat_create(WGB_Q6_K, h_blocks, false, nrows, ncols, st, &planar))) return rc;
    wgb_q6k_tiles *m = new (std::nothrow) wgb_q6k_tiles();
    if (!m) {
        wgb_quant_matrix_destroy(planar);
        return fail(WGB_ERR_INVALID, "out of host memory");
    }
    rc = prefill_tile_major6(planar->view, &m->w, st);
    cudaError_t e = cudaStreamSynchronize(st);
    wgb_quant_matrix_destroy(planar);
    if (!rc && e != cudaSuccess) rc = cuda_fail(e, "Q6_K tile-major upload");
    if (rc) {
        if (m->w) cudaFree(m->w);
        delete m;
        return rc;
    }
    m->nrows = (uint32_t)nrows;
    m->ncols = (uint32_t)ncols;
    *out = m;
    return WGB_OK;
}

WGB_EXPORT int wgb_q6k_tiles_destroy(wgb_q6k_tiles *m)
{
    if (!m) return WGB_OK;
    cudaFree(m->w);
    if (m->image) cudaFree(m->image);
    if (m->part) cudaFree(m->part);
    delete m;
    return WGB_OK;
}

WGB_EXPORT int wgb_gemm_q6k_tiles(wgb_q6k_tiles *m, const float *d_v, size_t n_vec, float *d_out, void *stream)
{
    WGB_REQUIRE(m && d_v && d_out, "null argument");
    WGB_REQUIRE(n_vec >= 1 && n_vec <= PF_TOK, "between 1 and %u input vectors, got %zu", PF_TOK, n_vec);
    cudaStream_t st = as_stream(stream);
    const uint32_t ns = prefill_gemm_splits(m->nrows, m->ncols);
    if (!m->image) {
        uint8_t *image = nullptr;
        float *part = nullptr;
        cudaError_t e = cudaMalloc((void **)&image, prefill_image6_bytes(m->ncols));
        if (e == cudaSuccess) e = cudaMalloc((void **)&part, (size_t)PF_MAX_SPLIT * PF_TOK * m->nrows * sizeof(float));
        if (e != cudaSuccess) {
            if (image) cudaFree(image);
            if (part) cudaFree(part);
            return cuda_fail(e, "work areas of the batched product");
        }
        m->image = image;
        m->part = part;
    }
    WGB_CUDA(cudaMemsetAsync(d_out, 0, n_vec * m->nrows * sizeof(float), st));
    int rc = launch_prefill_image6(d_v, m->ncols, m->ncols, (uint32_t)n_vec, m->image, st);
    if (!rc) rc = launch_gemm_q6k_tiles(m->w, m->nrows, m->ncols, m->image, (uint32_t)n_vec, m->part, m->nrows, ns, st);
    // d_out (zero) += the slices
    if (!rc) rc = launch_prefill_norm_image(d_out, m->nrows, m->part, ns, m->nrows, nullptr, 0.0f, m->nrows, (uint32_t)n_vec, nullptr, nullptr, 0, st);
    return rc;
}
