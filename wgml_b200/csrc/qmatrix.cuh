// Device-side view of a quantised matrix (the counterpart of wgml's GpuQuantMatrix,
// crates/wgml/src/quantized_matrix.rs:9-75) and its storage layouts in HBM.
//
// Layouts
//   raw     blocks in GGUF order, row-major [nrows][blocks_per_row][block_bytes].  Used as is for
//           every format whose block size is a multiple of 16 bytes (Q4_K: 144, Q5_K: 176) and for
//           the formats that only have the generic kernel.
//   planar  the fields of each block split into planes so that every vector load and every bulk
//           copy of whole rows is 16-byte aligned.  Every plane is row-major with a row pitch that
//           is a multiple of 16 bytes (the 2-byte scale planes are padded up to it).
//             Q8_0: p[0] = int8 codes  [nrows][ncols]          p[1] = f16 scales [nrows][bpr (+pad)]
//             Q6_K: p[0] = ql [nrows][bpr][128]  p[1] = qh [nrows][bpr][64]
//                   p[2] = int8 scales [nrows][bpr][16]        p[3] = f16 d [nrows][bpr (+pad)]
#pragma once

#include "common.cuh"

namespace wgb {

struct QMat {
    int qtype;
    int planar;
    uint32_t nrows, ncols, bpr;  // bpr = blocks per row = ncols / block_len(qtype)
    int nplanes;
    uint32_t pitch[4];           // bytes per row of each plane
    const uint8_t *p[4];
};

// Fills nplanes / pitch for a matrix of `bpr` blocks per row.
__host__ __device__ inline void qmat_set_pitches(QMat &m)
{
    m.pitch[0] = m.pitch[1] = m.pitch[2] = m.pitch[3] = 0;
    if (!m.planar) {
        m.nplanes = 1;
        m.pitch[0] = m.bpr * (uint32_t)block_bytes(m.qtype);
    } else if (m.qtype == WGB_Q8_0) {
        m.nplanes = 2;
        m.pitch[0] = m.bpr * 32;
        m.pitch[1] = (m.bpr * 2 + 15) & ~15u;
    } else {  // Q6_K
        m.nplanes = 4;
        m.pitch[0] = m.bpr * 128;
        m.pitch[1] = m.bpr * 64;
        m.pitch[2] = m.bpr * 16;
        m.pitch[3] = (m.bpr * 2 + 15) & ~15u;
    }
}

}  // namespace wgb

// Host-side owner of a QMat (opaque to C callers).
struct wgb_quant_matrix {
    wgb::QMat view;
    void *storage;   // one cudaMalloc holding every plane (NULL when the matrix wraps caller memory)
    size_t bytes;
};

namespace wgb {

// Pipelined host -> device upload of tensor bytes that live in pageable memory (a memory-mapped GGUF file):
// the bytes go through a small ring of pinned buffers, so that the host's copy out of the mapping (page
// faults, file reads), the DMA of the buffer before and the repack kernel of the tensor before overlap on one
// copy stream; nothing waits for a tensor until finish().  The counterpart of the reference's eager
// element-by-element parse (crates/wgml/src/gguf.rs:539-620, read_array_unaligned :671-681).
struct Uploader {
    static constexpr int NBUF = 3;
    static constexpr size_t BUF_BYTES = (size_t)64 << 20;
    cudaStream_t stream = nullptr;
    uint8_t *h_buf[NBUF] = {};
    cudaEvent_t free_ev[NBUF] = {};
    bool used[NBUF] = {};
    int next = 0;
    uint8_t *d_raw = nullptr;      // device staging of the raw blocks of a tensor that is repacked on the device
    size_t d_raw_cap = 0;
    size_t bytes = 0;              // uploaded since the last finish()
    double t0 = 0.0;               // when the first byte of the batch was taken
    size_t total_bytes = 0;        // over all finished batches
    double total_seconds = 0.0;    //   and their wall time, first byte to finish()

    int init();
    void destroy();
    // `rows` runs of `run_bytes` bytes, `src_stride` apart in host memory, laid end to end at d_dst.
    int copy_rows(uint8_t *d_dst, const uint8_t *h_src, size_t run_bytes, size_t src_stride, size_t rows);
    int reserve_raw(size_t n);
    int finish();                  // waits for everything enqueued; closes the timing batch
};

// Builds a matrix from raw GGUF blocks.  `src_on_device` says where `blocks` lives.  Planar
// formats are repacked on the device; the temporary raw copy is released before returning.
int qmat_create(int qtype, const void *blocks, bool src_on_device, size_t nrows, size_t ncols,
                cudaStream_t stream, wgb_quant_matrix **out);
// Same, but only rows [row0, row0 + nrows_keep) and, within each row, blocks
// [kb0, kb0 + bpr_keep) are kept (tensor-parallel slices).  `blocks` is in host memory.
int qmat_create_slice(int qtype, const void *h_blocks, size_t nrows, size_t ncols, size_t row0,
                      size_t nrows_keep, size_t kb0, size_t bpr_keep, cudaStream_t stream,
                      wgb_quant_matrix **out);
// The same through an Uploader: returns as soon as the copies and the repack are enqueued on the uploader's
// stream; the matrix may be used after up.finish() (or by work ordered after that stream).
int qmat_create_slice_async(Uploader &up, int qtype, const void *h_blocks, size_t nrows, size_t ncols, size_t row0,
                            size_t nrows_keep, size_t kb0, size_t bpr_keep, wgb_quant_matrix **out);
int qmat_dequantize_rows(const QMat &m, size_t row0, size_t n, float *d_out, cudaStream_t stream);
// Device-side variant whose first row is read from *d_row (token id kept on the device).
int qmat_dequantize_row_indirect(const QMat &m, const uint32_t *d_row, float *d_out, cudaStream_t stream);

}  // namespace wgb
