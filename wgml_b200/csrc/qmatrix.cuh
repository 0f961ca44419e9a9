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

// Builds a matrix from raw GGUF blocks.  `src_on_device` says where `blocks` lives.  Planar
// formats are repacked on the device; the temporary raw copy is released before returning.
int qmat_create(int qtype, const void *blocks, bool src_on_device, size_t nrows, size_t ncols,
                cudaStream_t stream, wgb_quant_matrix **out);
// Same, but only rows [row0, row0 + nrows_keep) and, within each row, blocks
// [kb0, kb0 + bpr_keep) are kept (tensor-parallel slices).  `blocks` is in host memory.
int qmat_create_slice(int qtype, const void *h_blocks, size_t nrows, size_t ncols, size_t row0,
                      size_t nrows_keep, size_t kb0, size_t bpr_keep, cudaStream_t stream,
                      wgb_quant_matrix **out);
int qmat_dequantize_rows(const QMat &m, size_t row0, size_t n, float *d_out, cudaStream_t stream);
// Device-side variant whose first row is read from *d_row (token id kept on the device).
int qmat_dequantize_row_indirect(const QMat &m, const uint32_t *d_row, float *d_out, cudaStream_t stream);

}  // namespace wgb
