// Exact (bit-for-bit) value of one weight of a quantised matrix in either storage layout.
#pragma once

#include "dequant.cuh"
#include "qmatrix.cuh"

namespace wgb {

template <int QT>
__device__ __forceinline__ float qmat_weight(const QMat &m, size_t row, uint32_t col)
{
    constexpr int BL = block_len(QT), BB = block_bytes(QT);
    const uint32_t kb = col / BL, r = col % BL;
    if (QT == WGB_Q8_0) {
        if (m.planar) {
            const uint16_t s = reinterpret_cast<const uint16_t *>(m.p[1] + row * m.pitch[1])[kb];
            return q8_0_value(s, (int8_t)m.p[0][row * m.pitch[0] + col]);
        }
    } else if (QT == WGB_Q6_K) {
        if (m.planar)
            return q6_k_value(m.p[0] + row * m.pitch[0] + kb * 128, m.p[1] + row * m.pitch[1] + kb * 64,
                              (const int8_t *)(m.p[2] + row * m.pitch[2] + kb * 16),
                              reinterpret_cast<const uint16_t *>(m.p[3] + row * m.pitch[3])[kb], r >> 5, r & 31);
    }
    return dequant_one<QT>(m.p[0] + row * m.pitch[0] + (size_t)kb * BB, r >> 5, r & 31);
}

__device__ inline float qmat_weight_any(const QMat &m, size_t row, uint32_t col)
{
    switch (m.qtype) {
    case WGB_F32: return qmat_weight<WGB_F32>(m, row, col);
    case WGB_F16: return qmat_weight<WGB_F16>(m, row, col);
    case WGB_Q4_0: return qmat_weight<WGB_Q4_0>(m, row, col);
    case WGB_Q4_1: return qmat_weight<WGB_Q4_1>(m, row, col);
    case WGB_Q5_0: return qmat_weight<WGB_Q5_0>(m, row, col);
    case WGB_Q5_1: return qmat_weight<WGB_Q5_1>(m, row, col);
    case WGB_Q8_0: return qmat_weight<WGB_Q8_0>(m, row, col);
    case WGB_Q4_K: return qmat_weight<WGB_Q4_K>(m, row, col);
    case WGB_Q5_K: return qmat_weight<WGB_Q5_K>(m, row, col);
    case WGB_Q6_K: return qmat_weight<WGB_Q6_K>(m, row, col);
    case WGB_Q8_K: return qmat_weight<WGB_Q8_K>(m, row, col);
    }
    return 0.0f;
}

}  // namespace wgb
