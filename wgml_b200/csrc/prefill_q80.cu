// Batched tensor-core product for Q8_0 matrices: the Q8_0 counterpart of gemm_q4k_tc_kernel (prefill.cu).  Same
// operator as GemvQuant::dispatch (crates/wgml/src/ops/gemv_quant.rs:241-348) for up to eight input vectors at once;
// block format as BlockQ8_0::dequantize (crates/wgml/src/quantization.rs:29-52): value = d * code, 32 signed byte
// codes per f16 scale.
//
// The codes are the A operand as they are (signed bytes), so the weights are kept in HBM in the operand's own
// shared-memory image: per (tile of 128 rows, 256-column unit) two K panels of 128 rows x 128 bytes with the
// 128-byte swizzle already applied, followed by the rows' eight f16 scales.  A bulk copy lands a unit in its ring
// stage and the MMAs read it there: no unpacking, no operand buffers, no proxy fence.  One thread issues eight
// MMAs per unit (one per 32-column block: M = 128, N = 32, K = 32) into 256 columns of tensor memory (two sets
// alternate); eight warps read the sums back and apply block scale x input exponent per position.  The input
// image is the one of the Q4_K kernel (three signed byte digits per element, one power-of-two exponent per 32
// columns; its odd groups carry a factor 1/16 meant for Q4_K's high nibbles, which is multiplied back here).
// Work items, column slices and the bounded waits as in the Q4_K kernel.
#include "kernels.h"
#include "tc_common.cuh"

namespace wgb {

constexpr uint32_t T8_CODES = TC_TILE_ROWS * 256;                        // the A operand of a unit
constexpr uint32_t T8_UNIT_BYTES = T8_CODES + TC_TILE_ROWS * 16;         // + eight f16 scales per row
constexpr uint32_t T8_IMG_DIGITS = 16 * 4 * 128;                         // as TB_IMG_* of prefill.cu
constexpr uint32_t T8_IMG_BYTES = T8_IMG_DIGITS + 2 * 8 * PF_TOK * 4;
constexpr uint32_t T8_STAGE = (T8_UNIT_BYTES + T8_IMG_BYTES + 1023) / 1024 * 1024;   // stages stay on 1 KB boundaries
constexpr uint32_t T8_RING = 4;
constexpr uint32_t T8_FINISH_WARPS = 8;
constexpr uint32_t T8_NT = 32 * (2 + T8_FINISH_WARPS);
constexpr uint32_t T8_TMEM_COLS = 512;
constexpr uint32_t T8_SMEM = T8_RING * T8_STAGE;
static_assert(T8_IMG_BYTES == prefill_image_unit_bytes(), "the Q8_0 kernel reads the Q4_K kernel's activation image");
static_assert(T8_UNIT_BYTES % 16 == 0 && T8_SMEM + 1024 + 12 * 1024 <= 227 * 1024, "copy granules and shared memory budget");

struct T8Args {
    const uint8_t *w;     // tile-major units: [tile][column][T8_UNIT_BYTES]
    const uint8_t *img;   // activation image: [column][T8_IMG_BYTES]
    float *out;           // [nsplit][PF_TOK][out_stride]
    uint32_t nrows, nkb, nsplit, ntok, out_stride;
    uint32_t *err;
};

__global__ void __launch_bounds__(T8_NT, 1) gemm_q80_tc_kernel(const __grid_constant__ T8Args a)
{
    extern __shared__ uint8_t t8_smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * T8_RING + 4];
    __shared__ float rowpart[T8_FINISH_WARPS / 4][PF_TOK][TC_TILE_ROWS];
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t dead_flag;
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)t8_smem_raw + 1023) & ~(uintptr_t)1023);
    volatile uint32_t *dead = &dead_flag;

    pdl_launch_dependents();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nkb = a.nkb, nsplit = a.nsplit, nitems = (a.nrows / TC_TILE_ROWS) * nsplit;
    auto bar_full = [&](uint32_t s) { return smem_addr(&bars[s]); };
    auto bar_empty = [&](uint32_t s) { return smem_addr(&bars[T8_RING + s]); };
    auto bar_done = [&](uint32_t u) { return smem_addr(&bars[2 * T8_RING + u]); };        // the unit's MMAs have completed
    auto bar_tfree = [&](uint32_t u) { return smem_addr(&bars[2 * T8_RING + 2 + u]); };   // its accumulators have been read
    auto stage = [&](uint32_t s) { return smem_addr(smem) + s * T8_STAGE; };
    uint32_t total = 0;
    for (uint32_t i = blockIdx.x; i < nitems; i += gridDim.x) {
        const uint32_t sp = i % nsplit;
        total += (sp + 1) * nkb / nsplit - sp * nkb / nsplit;
    }

    if (threadIdx.x == 0) {
        dead_flag = 0;
        for (uint32_t s = 0; s < T8_RING; s++) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 32 * T8_FINISH_WARPS);   // the finishing threads arrive after the unit's MMAs have completed
        }
        for (uint32_t u = 0; u < 2; u++) {
            mbar_init(bar_done(u), 1);
            mbar_init(bar_tfree(u), 32 * T8_FINISH_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(T8_TMEM_COLS) : "memory");
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
                const uint32_t s = n % T8_RING, round = n / T8_RING;
                if (round) ok = tc_wait(bar_empty(s), (round - 1) & 1, dead, a.err, 41);
                if (!ok) break;
                mbar_expect_tx(bar_full(s), T8_UNIT_BYTES + T8_IMG_BYTES);
                bulk_copy_g2s(stage(s), a.w + ((size_t)w.tile * nkb + w.kb) * T8_UNIT_BYTES, T8_UNIT_BYTES, bar_full(s));
                bulk_copy_g2s(stage(s) + T8_UNIT_BYTES, a.img + (size_t)w.kb * T8_IMG_BYTES, T8_IMG_BYTES, bar_full(s));
                w.next(nsplit, nkb, gridDim.x);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issue ------------------------------
        // One thread: as soon as unit n's stage is full and the accumulators of unit n - 2 have been read, eight
        // MMAs (A: the stage's codes, 128-byte swizzle; B: the stage's slice of the image, K-major without swizzle,
        // the four row groups of a K-core 128 bytes apart, K-cores 512 bytes apart) into columns 256 (n % 2) ...,
        // committed to the unit's barrier.
        if (lane == 0) {
            const uint32_t idesc = tc_idesc(32, 1);
            bool ok = true;
            for (uint32_t n = 0; n < total && ok; n++) {
                const uint32_t u = n & 1, s = n % T8_RING;
                ok = tc_wait(bar_full(s), (n / T8_RING) & 1, dead, a.err, 42);
                if (ok && n >= 2) ok = tc_wait(bar_tfree(u), ((n - 2) >> 1) & 1, dead, a.err, 45);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ad = tc_smem_desc_sw128(stage(s), 1024);
                const uint64_t bd = tc_smem_desc(stage(s) + T8_UNIT_BYTES, 512, 128);
                const uint32_t dcol = tmem_base + u * 256;
#pragma unroll
                for (uint32_t j = 0; j < 8; j++)
                    tc_mma(dcol + 32 * j, ad + (uint64_t)(((j >> 2) * 16384 + (j & 3) * 32) >> 4), bd + (uint64_t)((j * 1024) >> 4), idesc);
                tc_commit(bar_done(u));
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ finishing ------------------------------
        // Thread (quarter, lane, half): row r = 32 quarter + lane (the quarter of tensor memory its warp may read),
        // blocks 4 half .. 4 half + 3 of the unit's eight.
        const uint32_t half = (warp - 2) >> 2, quarter = warp & 3, r = quarter * 32 + lane;
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
        float rowacc[PF_TOK];
#pragma unroll
        for (uint32_t t = 0; t < PF_TOK; t++) rowacc[t] = 0.0f;
        bool ok = true;
        UnitWalk fin;
        fin.set(blockIdx.x, nsplit, nkb);
        for (uint32_t m = 0; m < total; m++) {
            const uint32_t slot = m % T8_RING, u = m & 1;
            if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_full(slot), (m / T8_RING) & 1, dead, a.err, 43));
            const uint32_t img = stage(slot) + T8_UNIT_BYTES;
            // the row's eight block scales; odd blocks take back the 1/16 that the image's odd groups carry
            uint4 sc = make_uint4(0u, 0u, 0u, 0u);
            if (ok) sc = lds128(stage(slot) + T8_CODES + r * 16);
            const uint32_t scw = half ? sc.z : sc.x, scw2 = half ? sc.w : sc.y;   // blocks 4 half + {0, 1} and + {2, 3}
            if (ok) ok = __all_sync(0xffffffffu, tc_wait(bar_done(u), (m >> 1) & 1, dead, a.err, 44));
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (uint32_t cc = 0; cc < 2; cc++) {
                    const uint32_t j0 = 4 * half + 2 * cc;
                    int d[2][3][8];
#pragma unroll
                    for (uint32_t q = 0; q < 2; q++)
#pragma unroll
                        for (uint32_t dg = 0; dg < 3; dg++) tc_ld8(taddr + u * 256 + 32 * (j0 + q) + 8 * dg, d[q][dg]);
                    float ev[2][8];
#pragma unroll
                    for (uint32_t q = 0; q < 2; q++) {
                        const uint32_t eo = img + T8_IMG_DIGITS + (j0 + q) * PF_TOK * 4;   // one exponent per position
                        const uint4 e0 = lds128(eo), e1 = lds128(eo + 16);
                        ev[q][0] = __uint_as_float(e0.x); ev[q][1] = __uint_as_float(e0.y); ev[q][2] = __uint_as_float(e0.z); ev[q][3] = __uint_as_float(e0.w);
                        ev[q][4] = __uint_as_float(e1.x); ev[q][5] = __uint_as_float(e1.y); ev[q][6] = __uint_as_float(e1.z); ev[q][7] = __uint_as_float(e1.w);
                    }
                    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(cc ? &scw2 : &scw));
                    const float sc0 = dd.x, sc1 = dd.y * 16.0f;   // j0 is even
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (cc == 1) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        mbar_arrive(bar_tfree(u));   // unit m + 2 may overwrite the accumulators
                    }
#pragma unroll
                    for (uint32_t t = 0; t < PF_TOK; t++) {
                        // |digit sum| <= 32 * 128 * 128 < 2^20; the two low ones are joined before their conversion
                        const float f0 = fmaf(__int2float_rn(d[0][2][t]), 65536.0f, __int2float_rn(d[0][1][t] * 256 + d[0][0][t]));
                        const float f1 = fmaf(__int2float_rn(d[1][2][t]), 65536.0f, __int2float_rn(d[1][1][t] * 256 + d[1][0][t]));
                        rowacc[t] += fmaf(f0, sc0 * ev[0][t], f1 * (sc1 * ev[1][t]));
                    }
                }
            }
            mbar_arrive(bar_empty(slot));
            if (fin.last()) {
#pragma unroll
                for (uint32_t t = 0; t < PF_TOK; t++) {
                    rowpart[half][t][r] = rowacc[t];
                    rowacc[t] = 0.0f;
                }
                asm volatile("bar.sync 2, %0;" ::"n"(32 * T8_FINISH_WARPS) : "memory");
                if (ok) {
                    constexpr uint32_t NP = T8_FINISH_WARPS / 4, TPT = PF_TOK / NP;
#pragma unroll
                    for (uint32_t tt = 0; tt < TPT; tt++) {
                        const uint32_t t = TPT * half + tt;
                        float v = rowpart[0][t][r];
#pragma unroll
                        for (uint32_t q = 1; q < NP; q++) v += rowpart[q][t][r];
                        if (t < a.ntok) a.out[((size_t)fin.sp * PF_TOK + t) * a.out_stride + (size_t)fin.tile * TC_TILE_ROWS + r] = v;
                    }
                }
                asm volatile("bar.sync 2, %0;" ::"n"(32 * T8_FINISH_WARPS) : "memory");
            }
            fin.next(nsplit, nkb, gridDim.x);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T8_TMEM_COLS) : "memory");
    }
}

int launch_gemm_q80_tiles(const uint8_t *w_tiles, uint32_t nrows, uint32_t K, const uint8_t *image, uint32_t ntok, float *out,
                          uint32_t out_stride, uint32_t nsplit, cudaStream_t stream)
{
    WGB_REQUIRE(nrows % TC_TILE_ROWS == 0 && K % 256 == 0 && ntok >= 1 && ntok <= PF_TOK && nsplit >= 1 && nsplit <= K / 256,
                "batched Q8_0 product: %u x %u, %u vectors, %u slices", nrows, K, ntok, nsplit);
    DeviceState *ds = device_state();
    if (!ds) return WGB_ERR_CUDA;
    if (!ds->prefill8_attrs) {
        WGB_CUDA(cudaFuncSetAttribute(gemm_q80_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(T8_SMEM + 1024)));
        ds->prefill8_attrs = true;
    }
    T8Args a = {};
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
    WGB_CUDA(launch_pdl(gemm_q80_tc_kernel, dim3(items < sms ? items : sms), dim3(T8_NT), T8_SMEM + 1024, stream, a));
    return WGB_OK;
}

// Planar Q8_0 matrix (qmatrix.cuh: codes [rows][K], f16 scales [rows][K / 32]) -> per (tile, 256-column unit) the A
// operand image (two K panels of 128 rows x 128 bytes, 16-byte pieces of row r stored at piece index ^ (r % 8))
// followed by the rows' eight scales.  One thread per 16 bytes.
__global__ void prefill_tile_major8_kernel(QMat m, uint8_t *__restrict__ tiled)
{
    const uint32_t nkb = m.ncols / 256;
    const size_t units = (size_t)(m.nrows / TC_TILE_ROWS) * nkb;
    const size_t total = units * TC_TILE_ROWS * 17;   // 16 pieces of codes and one of scales per row and unit
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t piece = (uint32_t)(i % 17);
        const size_t ru = i / 17;
        const uint32_t r = (uint32_t)(ru % TC_TILE_ROWS);
        const size_t unit = ru / TC_TILE_ROWS;
        const uint32_t kb = (uint32_t)(unit % nkb), tile = (uint32_t)(unit / nkb);
        const size_t row = (size_t)tile * TC_TILE_ROWS + r;
        uint8_t *dst = tiled + unit * T8_UNIT_BYTES;
        if (piece < 16) {
            const uint4 v = *reinterpret_cast<const uint4 *>(m.p[0] + row * m.pitch[0] + (size_t)kb * 256 + piece * 16);
            const uint32_t panel = piece >> 3, c = piece & 7;
            *reinterpret_cast<uint4 *>(dst + panel * 16384 + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)) = v;
        } else {
            *reinterpret_cast<uint4 *>(dst + T8_CODES + r * 16) = *reinterpret_cast<const uint4 *>(m.p[1] + row * m.pitch[1] + (size_t)kb * 16);
        }
    }
}

bool prefill_tileable8(const QMat &m) { return m.qtype == WGB_Q8_0 && m.planar && m.nrows % TC_TILE_ROWS == 0 && m.ncols % 256 == 0; }

int prefill_tile_major8(const QMat &m, uint8_t **out, cudaStream_t stream)
{
    WGB_REQUIRE(prefill_tileable8(m), "not a tileable Q8_0 matrix");
    const size_t units = (size_t)(m.nrows / TC_TILE_ROWS) * (m.ncols / 256);
    WGB_CUDA(cudaMalloc((void **)out, units * T8_UNIT_BYTES));
    const size_t threads = units * TC_TILE_ROWS * 17, blocks = (threads + 255) / 256;
    prefill_tile_major8_kernel<<<(unsigned)(blocks < 65535u * 16u ? blocks : 65535u * 16u), 256, 0, stream>>>(m, *out);
    WGB_LAUNCH_CHECK("prefill_tile_major8_kernel");
    return WGB_OK;
}

}  // namespace wgb

using namespace wgb;

// Stand-alone entry points (tests and measurement): a Q8_0 matrix in the tile-major layout and its batched product.
struct wgb_q80_tiles {
    uint8_t *w;
    uint32_t nrows, ncols;
    uint8_t *image;   // work areas, made by the first product
    float *part;
};

WGB_EXPORT int wgb_q80_tiles_create(const void *h_blocks, size_t nrows, size_t ncols, void *stream, wgb_q80_tiles **out)
{
    WGB_REQUIRE(h_blocks && out, "null argument");
    WGB_REQUIRE(nrows > 0 && nrows % TC_TILE_ROWS == 0, "the tensor-core path wants a multiple of %u rows, got %zu", TC_TILE_ROWS, nrows);
    WGB_REQUIRE(ncols > 0 && ncols % 256 == 0, "the tensor-core path wants a multiple of 256 columns, got %zu", ncols);
    int rc = gemv_global_init();
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    wgb_quant_matrix *planar = nullptr;
    if ((rc = qmat_create(WGB_Q8_0, h_blocks, false, nrows, ncols, st, &planar))) return rc;
    wgb_q80_tiles *m = new (std::nothrow) wgb_q80_tiles();
    if (!m) {
        wgb_quant_matrix_destroy(planar);
        return fail(WGB_ERR_INVALID, "out of host memory");
    }
    rc = prefill_tile_major8(planar->view, &m->w, st);
    cudaError_t e = cudaStreamSynchronize(st);
    wgb_quant_matrix_destroy(planar);
    if (!rc && e != cudaSuccess) rc = cuda_fail(e, "Q8_0 tile-major upload");
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

WGB_EXPORT int wgb_q80_tiles_destroy(wgb_q80_tiles *m)
{
    if (!m) return WGB_OK;
    cudaFree(m->w);
    if (m->image) cudaFree(m->image);
    if (m->part) cudaFree(m->part);
    delete m;
    return WGB_OK;
}

WGB_EXPORT int wgb_gemm_q80_tiles(wgb_q80_tiles *m, const float *d_v, size_t n_vec, float *d_out, void *stream)
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
    int rc = launch_prefill_norm_image(const_cast<float *>(d_v), m->ncols, nullptr, 0, 0, nullptr, 0.0f, m->ncols, (uint32_t)n_vec, m->image, nullptr, 0, st);
    if (!rc) rc = launch_gemm_q80_tiles(m->w, m->nrows, m->ncols, m->image, (uint32_t)n_vec, m->part, m->nrows, ns, st);
    if (!rc) rc = launch_prefill_norm_image(d_out, m->nrows, m->part, ns, m->nrows, nullptr, 0.0f, m->nrows, (uint32_t)n_vec, nullptr, nullptr, 0, st);
    return rc;
}
