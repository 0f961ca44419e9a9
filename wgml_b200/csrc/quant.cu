// Dequantisation kernels and the quantised-matrix object (upload, planar repack, row dequant).
#include "qaccess.cuh"

#include <algorithm>
#include <cstring>
#include <ctime>
#include <new>

namespace wgb {

// ---------------------------------------------------------------------------------------------
// Kernels
// ---------------------------------------------------------------------------------------------

// One thread per weight of a raw block stream (the role of ops/quantization_test.wgsl:45-146).
template <int QT>
__global__ void dequant_raw_kernel(const uint8_t *__restrict__ blocks, size_t nweights, float *__restrict__ out)
{
    constexpr int BL = block_len(QT), BB = block_bytes(QT);
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < nweights;
         e += (size_t)gridDim.x * blockDim.x) {
        size_t blk = e / BL;
        int r = (int)(e % BL);
        out[e] = dequant_one<QT>(blocks + blk * BB, r >> 5, r & 31);
    }
}

// Rows [row0, row0+n) (or the single row *d_row when d_row != NULL) to dense f32.
template <int QT>
__global__ void dequant_rows_kernel(QMat m, size_t row0, size_t n, const uint32_t *d_row, float *__restrict__ out)
{
    if (d_row) row0 = *d_row;
    const size_t total = n * (size_t)m.ncols;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        size_t r = e / m.ncols;
        uint32_t c = (uint32_t)(e % m.ncols);
        size_t row = row0 + r;
        out[e] = row < m.nrows ? qmat_weight<QT>(m, row, c) : 0.0f;
    }
}

// Raw Q8_0 blocks (row-major, bpr per row) -> planes.  One thread per block.
__global__ void repack_q8_0_kernel(const uint8_t *__restrict__ raw, size_t nblocks, QMat m)
{
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nblocks;
         b += (size_t)gridDim.x * blockDim.x) {
        const size_t row = b / m.bpr, kb = b % m.bpr;
        const uint8_t *s = raw + b * 34;
        reinterpret_cast<uint16_t *>(const_cast<uint8_t *>(m.p[1]) + row * m.pitch[1])[kb] = ld16(s);
        uint32_t *dst = reinterpret_cast<uint32_t *>(const_cast<uint8_t *>(m.p[0]) + row * m.pitch[0] + kb * 32);
#pragma unroll
        for (int i = 0; i < 8; i++) dst[i] = ld32(s + 2 + 4 * i);
    }
}

// Raw Q6_K blocks -> planes.  One thread per 4 bytes of a block's 208 data bytes + its d.
__global__ void repack_q6_k_kernel(const uint8_t *__restrict__ raw, size_t nblocks, QMat m)
{
    const size_t total = nblocks * 53;  // 52 words of ql/qh/scales + one slot for d
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        const size_t b = e / 53, row = b / m.bpr, kb = b % m.bpr;
        const int w = (int)(e % 53);
        const uint8_t *s = raw + b * 210;
        uint8_t *ql = const_cast<uint8_t *>(m.p[0]) + row * m.pitch[0] + kb * 128;
        uint8_t *qh = const_cast<uint8_t *>(m.p[1]) + row * m.pitch[1] + kb * 64;
        uint8_t *sc = const_cast<uint8_t *>(m.p[2]) + row * m.pitch[2] + kb * 16;
        if (w < 32) reinterpret_cast<uint32_t *>(ql)[w] = ld32(s + 4 * w);
        else if (w < 48) reinterpret_cast<uint32_t *>(qh)[w - 32] = ld32(s + 4 * w);
        else if (w < 52) reinterpret_cast<uint32_t *>(sc)[w - 48] = ld32(s + 4 * w);
        else reinterpret_cast<uint16_t *>(const_cast<uint8_t *>(m.p[3]) + row * m.pitch[3])[kb] = ld16(s + 208);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------

static inline int grid_for(size_t n, int threads)
{
    size_t g = (n + threads - 1) / threads;
    size_t cap = (size_t)sm_count() * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

static bool is_supported(int qtype) { return block_bytes(qtype) != 0; }

#define WGB_QT_SWITCH(qtype, CALL)                                                        \
    switch (qtype) {                                                                      \
    case WGB_F32: { constexpr int QT = WGB_F32; CALL; } break;                            \
    case WGB_F16: { constexpr int QT = WGB_F16; CALL; } break;                            \
    case WGB_Q4_0: { constexpr int QT = WGB_Q4_0; CALL; } break;                          \
    case WGB_Q4_1: { constexpr int QT = WGB_Q4_1; CALL; } break;                          \
    case WGB_Q5_0: { constexpr int QT = WGB_Q5_0; CALL; } break;                          \
    case WGB_Q5_1: { constexpr int QT = WGB_Q5_1; CALL; } break;                          \
    case WGB_Q8_0: { constexpr int QT = WGB_Q8_0; CALL; } break;                          \
    case WGB_Q4_K: { constexpr int QT = WGB_Q4_K; CALL; } break;                          \
    case WGB_Q5_K: { constexpr int QT = WGB_Q5_K; CALL; } break;                          \
    case WGB_Q6_K: { constexpr int QT = WGB_Q6_K; CALL; } break;                          \
    case WGB_Q8_K: { constexpr int QT = WGB_Q8_K; CALL; } break;                          \
    default: return fail(WGB_ERR_UNSUPPORTED, "unsupported tensor type %d", qtype);       \
    }

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Fills the pitches and plane pointers of `v` (qtype, planar, bpr set) for `nrows` rows stored at `base`;
// returns the bytes needed.
static size_t layout_planes(size_t nrows, uint8_t *base, QMat &v)
{
    qmat_set_pitches(v);
    size_t off = 0;
    for (int i = 0; i < 4; i++) {
        v.p[i] = i < v.nplanes ? base + off : nullptr;
        if (i < v.nplanes) off += align_up(nrows * (size_t)v.pitch[i], 256);
    }
    return off;
}

static int repack_from_device_raw(int qtype, const uint8_t *d_raw, size_t nb, const QMat &v, cudaStream_t stream)
{
    if (qtype == WGB_Q8_0) {
        repack_q8_0_kernel<<<grid_for(nb, 256), 256, 0, stream>>>(d_raw, nb, v);
    } else {
        repack_q6_k_kernel<<<grid_for(nb * 53, 256), 256, 0, stream>>>(d_raw, nb, v);
    }
    WGB_LAUNCH_CHECK("repack kernel");
    return WGB_OK;
}

int qmat_create_slice(int qtype, const void *h_blocks, size_t nrows, size_t ncols, size_t row0,
                      size_t nrows_keep, size_t kb0, size_t bpr_keep, cudaStream_t stream,
                      wgb_quant_matrix **out)
{
    if (!is_supported(qtype)) return fail(WGB_ERR_UNSUPPORTED, "unsupported tensor type %d", qtype);
    const int bl = block_len(qtype), bb = block_bytes(qtype);
    WGB_REQUIRE(out && h_blocks, "null argument");
    WGB_REQUIRE(ncols % bl == 0, "ncols %zu is not a multiple of the block length %d", ncols, bl);
    const size_t bpr = ncols / bl;
    WGB_REQUIRE(row0 + nrows_keep <= nrows && kb0 + bpr_keep <= bpr && nrows_keep > 0 && bpr_keep > 0,
                "slice outside the matrix");
    const bool planar = (qtype == WGB_Q8_0 || qtype == WGB_Q6_K);
    wgb_quant_matrix *m = new (std::nothrow) wgb_quant_matrix();
    if (!m) return fail(WGB_ERR_INVALID, "out of host memory");
    m->view.qtype = qtype;
    m->view.planar = planar;
    m->view.nrows = (uint32_t)nrows_keep;
    m->view.bpr = (uint32_t)bpr_keep;
    m->view.ncols = (uint32_t)(bpr_keep * bl);
    QMat tmp = m->view;
    m->bytes = layout_planes(nrows_keep, nullptr, tmp);
    cudaError_t e = cudaMalloc(&m->storage, m->bytes);
    if (e != cudaSuccess) { delete m; return cuda_fail(e, "cudaMalloc(quant matrix)"); }
    if (planar) e = cudaMemsetAsync(m->storage, 0, m->bytes, stream);  // pitch padding
    if (e != cudaSuccess) { cudaFree(m->storage); delete m; return cuda_fail(e, "cudaMemset(quant matrix)"); }
    layout_planes(nrows_keep, (uint8_t *)m->storage, m->view);

    const size_t raw_bytes = nrows_keep * bpr_keep * bb;
    uint8_t *d_raw = planar ? nullptr : (uint8_t *)m->storage;
    int rc = WGB_OK;
    if (planar) {
        e = cudaMalloc((void **)&d_raw, raw_bytes);
        if (e != cudaSuccess) { cudaFree(m->storage); delete m; return cuda_fail(e, "cudaMalloc(repack staging)"); }
    }
    const uint8_t *src = (const uint8_t *)h_blocks + (row0 * bpr + kb0) * bb;
    if (bpr_keep == bpr) e = cudaMemcpyAsync(d_raw, src, raw_bytes, cudaMemcpyHostToDevice, stream);
    else e = cudaMemcpy2DAsync(d_raw, bpr_keep * bb, src, bpr * bb, bpr_keep * bb, nrows_keep,
                               cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) rc = cuda_fail(e, "cudaMemcpy(quant matrix upload)");
    if (rc == WGB_OK && planar) rc = repack_from_device_raw(qtype, d_raw, nrows_keep * bpr_keep, m->view, stream);
    if (planar) {
        cudaError_t e2 = cudaStreamSynchronize(stream);
        if (rc == WGB_OK && e2 != cudaSuccess) rc = cuda_fail(e2, "repack");
        cudaFree(d_raw);
    }
    if (rc != WGB_OK) { cudaFree(m->storage); delete m; return rc; }
    *out = m;
    return WGB_OK;
}

static double now_s()
{
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

int Uploader::init()
{
    if (stream) return WGB_OK;
    WGB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    for (int i = 0; i < NBUF; i++) {
        WGB_CUDA(cudaMallocHost((void **)&h_buf[i], BUF_BYTES));
        WGB_CUDA(cudaEventCreateWithFlags(&free_ev[i], cudaEventDisableTiming));
    }
    return WGB_OK;
}

void Uploader::destroy()
{
    if (stream) cudaStreamSynchronize(stream);
    for (int i = 0; i < NBUF; i++) {
        if (h_buf[i]) cudaFreeHost(h_buf[i]);
        if (free_ev[i]) cudaEventDestroy(free_ev[i]);
        h_buf[i] = nullptr;
        free_ev[i] = nullptr;
        used[i] = false;
    }
    if (d_raw) cudaFree(d_raw);
    d_raw = nullptr;
    d_raw_cap = 0;
    if (stream) cudaStreamDestroy(stream);
    stream = nullptr;
}

int Uploader::reserve_raw(size_t n)
{
    if (n <= d_raw_cap) return WGB_OK;
    WGB_CUDA(cudaStreamSynchronize(stream));   // a repack may still read the old buffer
    if (d_raw) cudaFree(d_raw);
    d_raw = nullptr;
    d_raw_cap = 0;
    WGB_CUDA(cudaMalloc((void **)&d_raw, n));
    d_raw_cap = n;
    return WGB_OK;
}

int Uploader::copy_rows(uint8_t *d_dst, const uint8_t *h_src, size_t run_bytes, size_t src_stride, size_t rows)
{
    int rc = init();
    if (rc) return rc;
    if (bytes == 0) t0 = now_s();
    // contiguous source: one long run
    if (run_bytes == src_stride || rows == 1) {
        run_bytes *= rows;
        rows = 1;
    }
    size_t done_rows = 0, done_in_row = 0;   // progress: whole rows, plus bytes inside a row longer than a buffer
    while (done_rows < rows) {
        const int b = next;
        next = (next + 1) % NBUF;
        if (used[b]) WGB_CUDA(cudaEventSynchronize(free_ev[b]));
        size_t fill = 0;
        const size_t dst_off = done_rows * run_bytes + done_in_row;
        if (run_bytes > BUF_BYTES) {
            fill = std::min(BUF_BYTES, run_bytes - done_in_row);
            memcpy(h_buf[b], h_src + done_rows * src_stride + done_in_row, fill);
            done_in_row += fill;
            if (done_in_row == run_bytes) {
                done_in_row = 0;
                done_rows++;
            }
        } else {
            const size_t n = std::min(rows - done_rows, BUF_BYTES / run_bytes);
            for (size_t r = 0; r < n; r++) memcpy(h_buf[b] + r * run_bytes, h_src + (done_rows + r) * src_stride, run_bytes);
            fill = n * run_bytes;
            done_rows += n;
        }
        WGB_CUDA(cudaMemcpyAsync(d_dst + dst_off, h_buf[b], fill, cudaMemcpyHostToDevice, stream));
        WGB_CUDA(cudaEventRecord(free_ev[b], stream));
        used[b] = true;
        bytes += fill;
    }
    return WGB_OK;
}

int Uploader::finish()
{
    if (!stream) return WGB_OK;
    WGB_CUDA(cudaStreamSynchronize(stream));
    if (bytes) {
        total_seconds += now_s() - t0;
        total_bytes += bytes;
        bytes = 0;
    }
    return WGB_OK;
}

int qmat_create_slice_async(Uploader &up, int qtype, const void *h_blocks, size_t nrows, size_t ncols, size_t row0,
                            size_t nrows_keep, size_t kb0, size_t bpr_keep, wgb_quant_matrix **out)
{
    if (!is_supported(qtype)) return fail(WGB_ERR_UNSUPPORTED, "unsupported tensor type %d", qtype);
    const int bl = block_len(qtype), bb = block_bytes(qtype);
    WGB_REQUIRE(out && h_blocks, "null argument");
    WGB_REQUIRE(ncols % bl == 0, "ncols %zu is not a multiple of the block length %d", ncols, bl);
    const size_t bpr = ncols / bl;
    WGB_REQUIRE(row0 + nrows_keep <= nrows && kb0 + bpr_keep <= bpr && nrows_keep > 0 && bpr_keep > 0,
                "slice outside the matrix");
    int rc = up.init();
    if (rc) return rc;
    const bool planar = (qtype == WGB_Q8_0 || qtype == WGB_Q6_K);
    wgb_quant_matrix *m = new (std::nothrow) wgb_quant_matrix();
    if (!m) return fail(WGB_ERR_INVALID, "out of host memory");
    m->view.qtype = qtype;
    m->view.planar = planar;
    m->view.nrows = (uint32_t)nrows_keep;
    m->view.bpr = (uint32_t)bpr_keep;
    m->view.ncols = (uint32_t)(bpr_keep * bl);
    QMat tmp = m->view;
    m->bytes = layout_planes(nrows_keep, nullptr, tmp);
    cudaError_t e = cudaMalloc(&m->storage, m->bytes);
    if (e != cudaSuccess) { delete m; return cuda_fail(e, "cudaMalloc(quant matrix)"); }
    layout_planes(nrows_keep, (uint8_t *)m->storage, m->view);
    const size_t raw_bytes = nrows_keep * bpr_keep * bb;
    uint8_t *d_raw = (uint8_t *)m->storage;
    if (planar) {
        rc = up.reserve_raw(raw_bytes);
        if (rc == WGB_OK && (e = cudaMemsetAsync(m->storage, 0, m->bytes, up.stream)) != cudaSuccess) rc = cuda_fail(e, "cudaMemset(quant matrix)");
        d_raw = up.d_raw;
    }
    const uint8_t *src = (const uint8_t *)h_blocks + (row0 * bpr + kb0) * bb;
    if (rc == WGB_OK) rc = up.copy_rows(d_raw, src, bpr_keep * bb, bpr * bb, nrows_keep);
    if (rc == WGB_OK && planar) rc = repack_from_device_raw(qtype, d_raw, nrows_keep * bpr_keep, m->view, up.stream);
    if (rc != WGB_OK) {
        cudaStreamSynchronize(up.stream);
        cudaFree(m->storage);
        delete m;
        return rc;
    }
    *out = m;
    return WGB_OK;
}

int qmat_create(int qtype, const void *blocks, bool src_on_device, size_t nrows, size_t ncols,
                cudaStream_t stream, wgb_quant_matrix **out)
{
    if (!src_on_device) return qmat_create_slice(qtype, blocks, nrows, ncols, 0, nrows, 0,
                                                 block_len(qtype) ? ncols / block_len(qtype) : 0, stream, out);
    if (!is_supported(qtype)) return fail(WGB_ERR_UNSUPPORTED, "unsupported tensor type %d", qtype);
    const int bl = block_len(qtype), bb = block_bytes(qtype);
    WGB_REQUIRE(out && blocks, "null argument");
    WGB_REQUIRE(ncols % bl == 0 && nrows > 0 && ncols > 0, "ncols %zu is not a multiple of the block length %d", ncols, bl);
    const size_t bpr = ncols / bl;
    const bool planar = (qtype == WGB_Q8_0 || qtype == WGB_Q6_K);
    wgb_quant_matrix *m = new (std::nothrow) wgb_quant_matrix();
    if (!m) return fail(WGB_ERR_INVALID, "out of host memory");
    m->view.qtype = qtype;
    m->view.planar = planar;
    m->view.nrows = (uint32_t)nrows;
    m->view.bpr = (uint32_t)bpr;
    m->view.ncols = (uint32_t)ncols;
    QMat tmp = m->view;
    m->bytes = layout_planes(nrows, nullptr, tmp);
    cudaError_t e = cudaMalloc(&m->storage, m->bytes);
    if (e != cudaSuccess) { delete m; return cuda_fail(e, "cudaMalloc(quant matrix)"); }
    if (planar) e = cudaMemsetAsync(m->storage, 0, m->bytes, stream);  // pitch padding
    if (e != cudaSuccess) { cudaFree(m->storage); delete m; return cuda_fail(e, "cudaMemset(quant matrix)"); }
    layout_planes(nrows, (uint8_t *)m->storage, m->view);
    int rc = WGB_OK;
    if (planar) rc = repack_from_device_raw(qtype, (const uint8_t *)blocks, nrows * bpr, m->view, stream);
    else {
        e = cudaMemcpyAsync(m->storage, blocks, nrows * bpr * bb, cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) rc = cuda_fail(e, "cudaMemcpy(quant matrix)");
    }
    if (rc != WGB_OK) { cudaFree(m->storage); delete m; return rc; }
    *out = m;
    return WGB_OK;
}

int qmat_dequantize_rows(const QMat &m, size_t row0, size_t n, float *d_out, cudaStream_t stream)
{
    WGB_REQUIRE(row0 + n <= m.nrows, "rows [%zu, %zu) outside a matrix of %u rows", row0, row0 + n, m.nrows);
    if (n == 0) return WGB_OK;
    const size_t total = n * (size_t)m.ncols;
    WGB_QT_SWITCH(m.qtype, (dequant_rows_kernel<QT><<<grid_for(total, 256), 256, 0, stream>>>(m, row0, n, nullptr, d_out)));
    WGB_LAUNCH_CHECK("dequant_rows_kernel");
    return WGB_OK;
}

int qmat_dequantize_row_indirect(const QMat &m, const uint32_t *d_row, float *d_out, cudaStream_t stream)
{
    WGB_QT_SWITCH(m.qtype, (dequant_rows_kernel<QT><<<grid_for(m.ncols, 256), 256, 0, stream>>>(m, 0, 1, d_row, d_out)));
    WGB_LAUNCH_CHECK("dequant_rows_kernel");
    return WGB_OK;
}

}  // namespace wgb

using namespace wgb;

WGB_EXPORT int wgb_block_bytes(int qtype) { return block_bytes(qtype); }
WGB_EXPORT int wgb_block_len(int qtype) { return block_len(qtype); }

WGB_EXPORT int wgb_dequantize(int qtype, const void *d_blocks, size_t nblocks, float *d_out, void *stream)
{
    if (nblocks == 0) return WGB_OK;
    WGB_REQUIRE(d_blocks && d_out, "null argument");
    const size_t nweights = nblocks * (size_t)block_len(qtype);
    WGB_QT_SWITCH(qtype, (dequant_raw_kernel<QT><<<grid_for(nweights, 256), 256, 0, as_stream(stream)>>>(
                             (const uint8_t *)d_blocks, nweights, d_out)));
    WGB_LAUNCH_CHECK("dequant_raw_kernel");
    return WGB_OK;
}

WGB_EXPORT int wgb_quant_matrix_create(int qtype, const void *h_blocks, size_t nrows, size_t ncols,
                                       void *stream, wgb_quant_matrix **out)
{
    return qmat_create(qtype, h_blocks, false, nrows, ncols, as_stream(stream), out);
}

WGB_EXPORT int wgb_quant_matrix_create_from_device(int qtype, const void *d_blocks, size_t nrows, size_t ncols,
                                                   void *stream, wgb_quant_matrix **out)
{
    return qmat_create(qtype, d_blocks, true, nrows, ncols, as_stream(stream), out);
}

WGB_EXPORT int wgb_quant_matrix_destroy(wgb_quant_matrix *m)
{
    if (!m) return WGB_OK;
    if (m->storage) cudaFree(m->storage);
    delete m;
    return WGB_OK;
}

WGB_EXPORT int wgb_quant_matrix_shape(const wgb_quant_matrix *m, size_t *nrows, size_t *ncols, int *qtype)
{
    WGB_REQUIRE(m, "null matrix");
    if (nrows) *nrows = m->view.nrows;
    if (ncols) *ncols = m->view.ncols;
    if (qtype) *qtype = m->view.qtype;
    return WGB_OK;
}

WGB_EXPORT int wgb_quant_matrix_dequantize_rows(const wgb_quant_matrix *m, size_t row0, size_t n, float *d_out,
                                                void *stream)
{
    WGB_REQUIRE(m && d_out, "null argument");
    return qmat_dequantize_rows(m->view, row0, n, d_out, as_stream(stream));
}
