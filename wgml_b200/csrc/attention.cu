// Decode attention over the KV cache: one query position against keys / values 0..=pos.
//
// Semantics: BatchedMultiqueryAttention (crates/wgml/src/ops/batched_multiquery_attention.rs:141-195,
// batched_multiquery_attention.wgsl:38-99): score_t = (q_h . k_t) / sqrt(head_size), softmax with
// the maximum subtracted, xb_h = sum_t p_t v_t; query head h reads KV head h / kv_mul.
//
// Split kernel (the hot path): grid (time chunks of 64, KV heads).  A block computes, for every
// query head of its KV head, the scores of its chunk, the chunk maximum, the exponentials and the
// weighted sum of its 64 value rows; (max, sum, vector) go to a scratch buffer.  The block that
// finishes last for a KV head (an atomic ticket, nobody waits) merges the chunks.  K and V rows
// are read once for all kv_mul query heads.
//
// Long contexts (more chunks than blocks fit in one wave) take the streaming kernel further down: one block
// per SM walks a run of chunks with a producer warp feeding K / V tiles through shared memory.
//
// Full kernel (API path that returns the attention weights): one block per query head, the
// probabilities are materialised in the caller's [n_heads][seq_len] buffer.
#include "async_copy.cuh"
#include "kernels.h"

#include <algorithm>
#include <mutex>

namespace wgb {

constexpr int ATT_NT = 256;
constexpr int ATT_WARPS = ATT_NT / 32;
constexpr int ATT_CHUNK = 64;
constexpr int ATT_TPW = ATT_CHUNK / ATT_WARPS;  // time steps per warp

uint32_t attn_num_splits(uint32_t seq_len) { return (seq_len + ATT_CHUNK - 1) / ATT_CHUNK; }

size_t attn_scratch_floats(uint32_t n_heads, uint32_t head_size, uint32_t seq_len)
{
    return (size_t)n_heads * attn_num_splits(seq_len) * (head_size + 4);
}

// QH = query heads per KV head handled at once; VC = float4 chunks of a head per lane (1: head
// sizes up to 128, 2: up to 256).
// MULTI: a block may get several chunks (long contexts, few heads) and keeps a running softmax over them;
// otherwise every block has exactly one chunk and the loop below collapses.
// The merge of a head's chunks by its last block.
template <int QH, int VC>
__device__ __forceinline__ void attn_merge_chunks(const AttnArgs &a, uint32_t kvh, uint32_t hq0, uint32_t kv_mul, uint32_t hs, uint32_t nchunk,
                                               uint32_t max_splits, uint32_t nsplit_active, float (*s_red)[ATT_WARPS], float (*s_Mw)[ATT_WARPS],
                                               float (*s_acc)[QH][VC * 128 + 4])
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if constexpr (QH > 1 || VC > 1) {
        // Grouped queries / wide heads (kernels whose register count decides their blocks per SM): two passes over
        // the scratch.  The chunk maxima first (one thread per chunk), then warp w folds chunks w, w + 8, ... for
        // every output element, and the eight partial results meet in shared memory.  The chunk -> warp assignment
        // is fixed, so the result does not depend on timing.
        __shared__ float s_M[QH];
#pragma unroll
        for (int j = 0; j < QH; j++) {
            float m = -INFINITY;
            if (hq0 + j < kv_mul) {
                const float *base = a.scratch + (size_t)(kvh * kv_mul + hq0 + j) * max_splits * (hs + 4);
                for (uint32_t sp = threadIdx.x; sp < nsplit_active; sp += ATT_NT) m = fmaxf(m, __ldcg(base + (size_t)sp * (hs + 4) + hs));
            }
            m = warp_max(m);
            if (lane == 0) s_red[j][warp] = m;
        }
        __syncthreads();
        if (threadIdx.x < QH) {
            float m = s_red[threadIdx.x][0];
#pragma unroll
            for (int w = 1; w < ATT_WARPS; w++) m = fmaxf(m, s_red[threadIdx.x][w]);
            s_M[threadIdx.x] = m;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < QH; j++) {
            if (hq0 + j >= kv_mul) continue;   // uniform over the block
            const float *base = a.scratch + (size_t)(kvh * kv_mul + hq0 + j) * max_splits * (hs + 4);
            const float M = s_M[j];
            float4 o[VC];
#pragma unroll
            for (int c = 0; c < VC; c++) o[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            float L = 0.0f;
            for (uint32_t sp = warp; sp < nsplit_active; sp += ATT_WARPS) {
                const float *row = base + (size_t)sp * (hs + 4);
                const float w = expf(__ldcg(row + hs) - M);
                L = fmaf(__ldcg(row + hs + 1), w, L);
#pragma unroll
                for (int c = 0; c < VC; c++) {
                    const uint32_t ch = lane + 32 * c;
                    if (ch < nchunk) {
                        const float4 v = __ldcg(reinterpret_cast<const float4 *>(row) + ch);
                        o[c].x = fmaf(v.x, w, o[c].x);
                        o[c].y = fmaf(v.y, w, o[c].y);
                        o[c].z = fmaf(v.z, w, o[c].z);
                        o[c].w = fmaf(v.w, w, o[c].w);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < VC; c++) {
                const uint32_t ch = lane + 32 * c;
                if (ch < nchunk) reinterpret_cast<float4 *>(&s_acc[warp][j][0])[ch] = o[c];
            }
            if (lane == 0) s_red[j][warp] = L;
        }
        __syncthreads();
        for (uint32_t e = threadIdx.x; e < QH * hs; e += ATT_NT) {
            const uint32_t j = e / hs, i = e % hs;
            if (hq0 + j >= kv_mul) continue;
            float L = 0.0f, o = 0.0f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; w++) {
                L += s_red[j][w];
                o += s_acc[w][j][i];
            }
            a.xb[(size_t)(kvh * kv_mul + hq0 + j) * hs + i] = o / L;
        }
        return;
    }
    // One query head, head size <= 128: one pass over the scratch.  Warp w folds chunks w, w + 8, ...
    // with a running maximum (a row's vector, maximum and denominator come in one round trip), and the eight warps'
    // (vector, maximum, denominator) triples meet in shared memory.  The chunk -> warp assignment and the order of
    // the additions are fixed, so the result does not depend on timing.
#pragma unroll
    for (int j = 0; j < QH; j++) {
        if (hq0 + j >= kv_mul) continue;   // uniform over the block
        const float *base = a.scratch + (size_t)(kvh * kv_mul + hq0 + j) * max_splits * (hs + 4);
        float4 o[VC];
#pragma unroll
        for (int c = 0; c < VC; c++) o[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        float Mw = -INFINITY, Lw = 0.0f;
        for (uint32_t sp = warp; sp < nsplit_active; sp += ATT_WARPS) {
            const float *row = base + (size_t)sp * (hs + 4);
            const float ms = __ldcg(row + hs), ls = __ldcg(row + hs + 1);
            float4 v[VC];
#pragma unroll
            for (int c = 0; c < VC; c++) {
                const uint32_t ch = lane + 32 * c;
                v[c] = ch < nchunk ? __ldcg(reinterpret_cast<const float4 *>(row) + ch) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            const float mn = fmaxf(Mw, ms);
            const float rs = expf(Mw - mn), w = expf(ms - mn);   // rs = 0 at the warp's first chunk (Mw = -inf)
            Mw = mn;
            Lw = fmaf(Lw, rs, ls * w);
#pragma unroll
            for (int c = 0; c < VC; c++) {
                o[c].x = fmaf(o[c].x, rs, v[c].x * w);
                o[c].y = fmaf(o[c].y, rs, v[c].y * w);
                o[c].z = fmaf(o[c].z, rs, v[c].z * w);
                o[c].w = fmaf(o[c].w, rs, v[c].w * w);
            }
        }
#pragma unroll
        for (int c = 0; c < VC; c++) {
            const uint32_t ch = lane + 32 * c;
            if (ch < nchunk) reinterpret_cast<float4 *>(&s_acc[warp][j][0])[ch] = o[c];
        }
        if (lane == 0) {
            s_Mw[j][warp] = Mw;
            s_red[j][warp] = Lw;
        }
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < QH * hs; e += ATT_NT) {
        const uint32_t j = e / hs, i = e % hs;
        if (hq0 + j >= kv_mul) continue;
        float M = s_Mw[j][0];
#pragma unroll
        for (int w = 1; w < ATT_WARPS; w++) M = fmaxf(M, s_Mw[j][w]);
        float L = 0.0f, o = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) {
            const float f = expf(s_Mw[j][w] - M);   // 0 for a warp without a chunk
            L = fmaf(s_red[j][w], f, L);
            o = fmaf(s_acc[w][j][i], f, o);
        }
        a.xb[(size_t)(kvh * kv_mul + hq0 + j) * hs + i] = o / L;
    }
}

// One query head per KV head and head sizes up to 128 (the 7B shape): three blocks per SM, so that the chunks of a
// context of 800 positions are all resident at once.  (Left to itself the kernel takes 85 registers, two blocks per
// SM, and a launch is 1.2 us shorter while its blocks fit one wave -- 576 positions for 32 heads -- but a second
// wave costs 2.5 us, more than the streaming kernel.)
template <int QH, int VC, bool MULTI>
__global__ void __launch_bounds__(ATT_NT, (QH == 1 && VC == 1) ? 3 : 0) attn_split_kernel(const __grid_constant__ AttnArgs a)
{
    __shared__ float s_score[QH][ATT_CHUNK];
    __shared__ float s_red[QH][ATT_WARPS];
    __shared__ float s_acc[ATT_WARPS][QH][VC * 128 + 4];
    __shared__ uint32_t s_last;

    pdl_launch_dependents();
    // The position and every cache row before it were written by earlier steps, so they are read before the
    // wait for the preceding launch (which produces q and the cache row of this position): the DRAM round
    // trip of the first chunk overlaps the hand-over between the launches.
    const uint32_t pos = a.pos ? *a.pos : a.p.pos;
    const uint32_t hs = a.p.head_size, kv_mul = a.p.kv_mul;
    const uint32_t rstr = a.row_stride ? a.row_stride : a.p.kv_dim, hstr = a.row_stride ? a.head_stride : hs;
    const uint32_t split = blockIdx.x, kvh = blockIdx.y;
    // The grid has a fixed number of splits (chosen so that all blocks are resident at once); the chunks of
    // ATT_CHUNK positions up to `pos` are dealt to them in runs of `cpb`.
    const uint32_t nchunks_active = pos / ATT_CHUNK + 1;
    const uint32_t max_splits = gridDim.x;
    const uint32_t cpb = MULTI ? (nchunks_active + max_splits - 1) / max_splits : 1u;
    const uint32_t nsplit_active = (nchunks_active + cpb - 1) / cpb;
    if (split >= nsplit_active) {
        if (threadIdx.x == 0) stamp_end(a.stamp);
        return;
    }
    const uint32_t ck_begin = split * cpb, ck_end = MULTI ? min(ck_begin + cpb, nchunks_active) : ck_begin + 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t nchunk = hs / 4;  // float4 chunks per head
    const float inv_sqrt = sqrtf((float)hs);

    // Every warp owns ATT_TPW consecutive time steps of a chunk.  All of their K and V rows are requested up
    // front (independent loads, one DRAM round trip for the whole chunk), then consumed.
    float4 kr[ATT_TPW][VC], vr[ATT_TPW][VC];
    auto load_rows = [&](uint32_t t0, bool before_wait) {
        const float *kbase = a.k_cache + (size_t)t0 * rstr + (size_t)kvh * hstr;
        const float *vbase = a.v_cache + (size_t)t0 * rstr + (size_t)kvh * hstr;
#pragma unroll
        for (int i = 0; i < ATT_TPW; i++) {
            const uint32_t tl = warp * ATT_TPW + i;
#pragma unroll
            for (int c = 0; c < VC; c++) {
                const uint32_t ch = lane + 32 * c;
                const float4 *kp = reinterpret_cast<const float4 *>(kbase + (size_t)tl * rstr) + ch;
                const float4 *vp = reinterpret_cast<const float4 *>(vbase + (size_t)tl * rstr) + ch;
                if (before_wait) {   // rows of earlier steps only
                    const bool ok = t0 + tl < pos && ch < nchunk;
                    kr[i][c] = ok ? __ldcs(kp) : make_float4(0.f, 0.f, 0.f, 0.f);
                    vr[i][c] = ok ? __ldcs(vp) : make_float4(0.f, 0.f, 0.f, 0.f);
                } else if (ch < nchunk) {
                    if (t0 + tl < pos) {
                        kr[i][c] = __ldcs(kp);
                        vr[i][c] = __ldcs(vp);
                    } else if (t0 + tl == pos) {   // the row of this position, written by the preceding launch
                        kr[i][c] = __ldcg(kp);
                        vr[i][c] = __ldcg(vp);
                    } else {
                        kr[i][c] = make_float4(0.f, 0.f, 0.f, 0.f);
                        vr[i][c] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                } else {
                    kr[i][c] = make_float4(0.f, 0.f, 0.f, 0.f);
                    vr[i][c] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
    };
    load_rows(ck_begin * ATT_CHUNK, true);
    pdl_wait();

    // query heads of this KV head: h = kvh * kv_mul + j, j = hq0 .. hq0 + QH - 1 (looped by caller grid.z)
    const uint32_t hq0 = blockIdx.z * QH;
    float4 q[QH][VC];
#pragma unroll
    for (int j = 0; j < QH; j++)
#pragma unroll
        for (int c = 0; c < VC; c++) {
            const uint32_t ch = lane + 32 * c;
            q[j][c] = (ch < nchunk && hq0 + j < kv_mul)
                          ? __ldcg(reinterpret_cast<const float4 *>(a.q + (size_t)(kvh * kv_mul + hq0 + j) * hs) + ch)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }

    // Running softmax state over the block's chunks (rescaled whenever the maximum grows).
    float M[QH], L[QH];
    float4 acc[QH][VC];
#pragma unroll
    for (int j = 0; j < QH; j++) {
        M[j] = -INFINITY;
        L[j] = 0.0f;
#pragma unroll
        for (int c = 0; c < VC; c++) acc[j][c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    for (uint32_t ck = ck_begin; ck < ck_end; ck++) {
        const uint32_t t0 = ck * ATT_CHUNK;
        const uint32_t nt = min((uint32_t)ATT_CHUNK, pos + 1 - t0);
        if (MULTI && ck != ck_begin) {
            load_rows(t0, false);
        } else {
            // the first chunk was requested before the wait; fetch the row of this position if it lies here
#pragma unroll
            for (int i = 0; i < ATT_TPW; i++) {
                const uint32_t tl = warp * ATT_TPW + i;
                if (t0 + tl == pos) {
#pragma unroll
                    for (int c = 0; c < VC; c++) {
                        const uint32_t ch = lane + 32 * c;
                        if (ch < nchunk) {
                            kr[i][c] = __ldcg(reinterpret_cast<const float4 *>(a.k_cache + (size_t)pos * rstr + (size_t)kvh * hstr) + ch);
                            vr[i][c] = __ldcg(reinterpret_cast<const float4 *>(a.v_cache + (size_t)pos * rstr + (size_t)kvh * hstr) + ch);
                        }
                    }
                }
            }
        }
        // Pass 1: scores of the chunk.
#pragma unroll
        for (int j = 0; j < QH; j++) {
            float part[ATT_TPW];
#pragma unroll
            for (int i = 0; i < ATT_TPW; i++) {
                float p = 0.0f;
#pragma unroll
                for (int c = 0; c < VC; c++)
                    p += q[j][c].x * kr[i][c].x + q[j][c].y * kr[i][c].y + q[j][c].z * kr[i][c].z + q[j][c].w * kr[i][c].w;
                part[i] = p;
            }
            // ATT_TPW sums over the warp at once: each halving step folds two partials into one lane half
            // (8 -> 4 -> 2 -> 1 values per lane in 3 steps, then 2 plain steps): 7 + 2 shuffles instead of 40.
            static_assert(ATT_TPW == 8, "the folding below is written for 8 time steps per warp");
            float f4[4], f2[2], f1;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const bool up = lane & 16;
                const float keep = up ? part[2 * i + 1] : part[2 * i], give = up ? part[2 * i] : part[2 * i + 1];
                f4[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
            }
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const bool up = lane & 8;
                const float keep = up ? f4[2 * i + 1] : f4[2 * i], give = up ? f4[2 * i] : f4[2 * i + 1];
                f2[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
            }
            {
                const bool up = lane & 4;
                const float keep = up ? f2[1] : f2[0], give = up ? f2[0] : f2[1];
                f1 = keep + __shfl_xor_sync(0xffffffffu, give, 4);
            }
            f1 += __shfl_xor_sync(0xffffffffu, f1, 2);
            f1 += __shfl_xor_sync(0xffffffffu, f1, 1);
            // lane l now holds the sum of time step i = (bit4 of l) + 2 * (bit3) + 4 * (bit2)
            if ((lane & 3) == 0) {
                const uint32_t i = ((lane >> 4) & 1) | (((lane >> 3) & 1) << 1) | (((lane >> 2) & 1) << 2);
                const uint32_t tl = warp * ATT_TPW + i;
                if (tl < nt) s_score[j][tl] = f1 / inv_sqrt;
            }
        }
        __syncthreads();

        // Chunk maximum per query head, then exponentials against the running maximum and their sum.
#pragma unroll
        for (int j = 0; j < QH; j++) {
            float m = -INFINITY;
            for (uint32_t tl = threadIdx.x; tl < nt; tl += ATT_NT) m = fmaxf(m, s_score[j][tl]);
            m = warp_max(m);
            if (lane == 0) s_red[j][warp] = m;
        }
        __syncthreads();
        float rescale[QH];
#pragma unroll
        for (int j = 0; j < QH; j++) {
            float m = s_red[j][0];
#pragma unroll
            for (int w = 1; w < ATT_WARPS; w++) m = fmaxf(m, s_red[j][w]);
            const float mn = MULTI ? fmaxf(M[j], m) : m;
            rescale[j] = MULTI ? expf(M[j] - mn) : 0.0f;   // 0 for the first chunk (M = -inf)
            M[j] = mn;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < QH; j++) {
            float sm = 0.0f;
            for (uint32_t tl = threadIdx.x; tl < nt; tl += ATT_NT) {
                const float e = expf(s_score[j][tl] - M[j]);
                s_score[j][tl] = e;
                sm += e;
            }
            sm = warp_sum(sm);
            if (lane == 0) s_red[j][warp] = sm;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < QH; j++) {
            float sm = 0.0f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; w++) sm += s_red[j][w];
            L[j] = MULTI ? fmaf(L[j], rescale[j], sm) : sm;
            if (MULTI) {
#pragma unroll
                for (int c = 0; c < VC; c++) {
                    acc[j][c].x *= rescale[j];
                    acc[j][c].y *= rescale[j];
                    acc[j][c].z *= rescale[j];
                    acc[j][c].w *= rescale[j];
                }
            }
        }

        // Pass 2: weighted sum of the value rows.
#pragma unroll
        for (int i = 0; i < ATT_TPW; i++) {
            const uint32_t tl = warp * ATT_TPW + i;
            if (tl < nt) {
#pragma unroll
                for (int c = 0; c < VC; c++) {
                    const float4 v = vr[i][c];
#pragma unroll
                    for (int j = 0; j < QH; j++) {
                        const float p = s_score[j][tl];
                        acc[j][c].x = fmaf(p, v.x, acc[j][c].x);
                        acc[j][c].y = fmaf(p, v.y, acc[j][c].y);
                        acc[j][c].z = fmaf(p, v.z, acc[j][c].z);
                        acc[j][c].w = fmaf(p, v.w, acc[j][c].w);
                    }
                }
            }
        }
        if (MULTI) __syncthreads();   // the scores and the reduction scratch are reused by the next chunk
    }
#pragma unroll
    for (int j = 0; j < QH; j++)
#pragma unroll
        for (int c = 0; c < VC; c++) {
            const uint32_t ch = lane + 32 * c;
            if (ch < nchunk) reinterpret_cast<float4 *>(&s_acc[warp][j][0])[ch] = acc[j][c];
        }
    __syncthreads();

    // Partial result of this block -> scratch [head][split][hs + 4] = {vector, max, sum}.
    for (uint32_t e = threadIdx.x; e < QH * hs; e += ATT_NT) {
        const uint32_t j = e / hs, i = e % hs;
        if (hq0 + j >= kv_mul) continue;
        float sv = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) sv += s_acc[w][j][i];
        const uint32_t h = kvh * kv_mul + hq0 + j;
        a.scratch[((size_t)h * max_splits + split) * (hs + 4) + i] = sv;
    }
    if (threadIdx.x < QH && hq0 + threadIdx.x < kv_mul) {
        const uint32_t h = kvh * kv_mul + hq0 + threadIdx.x;
        float *dst = a.scratch + ((size_t)h * max_splits + split) * (hs + 4) + hs;
        float m = M[0], sm = L[0];
#pragma unroll
        for (int j = 1; j < QH; j++) { m = (threadIdx.x == j) ? M[j] : m; sm = (threadIdx.x == j) ? L[j] : sm; }
        dst[0] = m;
        dst[1] = sm;
    }

    // Ticket: the last block of this (KV head, query-head group) merges all chunks.
    __threadfence();
    __syncthreads();
    uint32_t *counter = a.counters + kvh * gridDim.z + blockIdx.z;
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(counter, 1u);
        s_last = (ticket == nsplit_active - 1);
        if (s_last) *counter = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!s_last) {
        if (threadIdx.x == 0) stamp_end(a.stamp);
        return;
    }
    __threadfence();
    __shared__ float s_Mw[QH][ATT_WARPS];
    attn_merge_chunks<QH, VC>(a, kvh, hq0, kv_mul, hs, nchunk, max_splits, nsplit_active, s_red, s_Mw, s_acc);
    if (threadIdx.x == 0) stamp_end(a.stamp);
}

// One block per query head; writes the attention weights.
__global__ void __launch_bounds__(ATT_NT) attn_full_kernel(const __grid_constant__ AttnArgs a, float *__restrict__ attn)
{
    __shared__ float red[32];
    const uint32_t pos = a.pos ? *a.pos : a.p.pos;
    const uint32_t hs = a.p.head_size;
    const uint32_t rstr = a.row_stride ? a.row_stride : a.p.kv_dim, hstr = a.row_stride ? a.head_stride : hs;
    const uint32_t h = blockIdx.x, kvh = h / a.p.kv_mul;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float *att = attn + (size_t)h * a.p.seq_len;
    const float *qh = a.q + (size_t)h * hs;
    const float sq = sqrtf((float)hs);
    for (uint32_t t = warp; t <= pos; t += ATT_WARPS) {
        const float *k = a.k_cache + (size_t)t * rstr + (size_t)kvh * hstr;
        float s = 0.0f;
        for (uint32_t i = lane; i < hs; i += 32) s = fmaf(qh[i], k[i], s);
        s = warp_sum(s);
        if (lane == 0) att[t] = s / sq;
    }
    __syncthreads();
    float m = -INFINITY;
    for (uint32_t t = threadIdx.x; t <= pos; t += ATT_NT) m = fmaxf(m, att[t]);
    m = block_max<ATT_NT>(m, red);
    float sum = 0.0f;
    for (uint32_t t = threadIdx.x; t <= pos; t += ATT_NT) {
        const float e = expf(att[t] - m);
        att[t] = e;
        sum += e;
    }
    sum = block_sum<ATT_NT>(sum, red);
    for (uint32_t t = threadIdx.x; t <= pos; t += ATT_NT) att[t] = att[t] / sum;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < hs; i += ATT_NT) {
        float o = 0.0f;
        for (uint32_t t = 0; t <= pos; t++) o = fmaf(att[t], a.v_cache[(size_t)t * rstr + (size_t)kvh * hstr + i], o);
        a.xb[(size_t)h * hs + i] = o;
    }
}

// ---------------------------------------------------------------------------------------------
// Streaming kernel (long contexts; head sizes up to 128).  Grid (splits, KV heads, query-head groups) with
// one block per SM; a block owns a run of 64-position chunks of one KV head and all QH query heads that
// share it.  A producer warp streams the K and V rows of chunk after chunk into a two-stage ring of shared
// memory with bulk asynchronous copies (one per cache row, completion on an mbarrier), so the DRAM round
// trip of the next chunk overlaps the arithmetic of the current one; eight consumer warps score the chunk
// (8 positions per warp); each warp keeps its own running softmax and weighted value sum over its positions,
// so nothing inside the loop synchronises the warps, and the eight are merged once at the end.  The block's
// (vector, max, sum) goes to the scratch buffer and the last block of a head merges, as in the split kernel.
// Every barrier wait is bounded (status codes 7 producer, 8 consumer).
// ---------------------------------------------------------------------------------------------
constexpr int ATS_STAGES = 2;
constexpr int ATS_NT = ATT_NT + 32;   // consumer warps + the producer warp

__device__ __forceinline__ void att_cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(ATT_NT) : "memory"); }

template <int QH>
__global__ void __launch_bounds__(ATS_NT, 1) attn_stream_kernel(const __grid_constant__ AttnArgs a)
{
    extern __shared__ uint4 ring4[];   // ATS_STAGES x (K tile | V tile), a tile = ATT_CHUNK rows of head_size floats
    __shared__ float s_sc[ATT_WARPS][QH][ATT_TPW];   // a warp's scores of the chunk in work
    __shared__ float s_red[QH][ATT_WARPS], s_sum[QH][ATT_WARPS];
    __shared__ float s_M[QH];
    __shared__ __align__(8) unsigned long long bars[2 * ATS_STAGES];
    __shared__ uint32_t s_last;

    const uint32_t pos = a.pos ? *a.pos : a.p.pos;   // written by an earlier step: readable before the wait
    const uint32_t hs = a.p.head_size, kv_mul = a.p.kv_mul;
    const uint32_t rstr = a.row_stride ? a.row_stride : a.p.kv_dim, hstr = a.row_stride ? a.head_stride : hs;
    const uint32_t split = blockIdx.x, kvh = blockIdx.y, hq0 = blockIdx.z * QH;
    const uint32_t nchunks_active = pos / ATT_CHUNK + 1;
    const uint32_t max_splits = gridDim.x;
    const uint32_t cpb = (nchunks_active + max_splits - 1) / max_splits;
    const uint32_t nsplit_active = (nchunks_active + cpb - 1) / cpb;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (split >= nsplit_active) {
        if (threadIdx.x == 0) stamp_end(a.stamp);
        return;
    }
    const uint32_t ck_begin = split * cpb, ck_end = min(ck_begin + cpb, nchunks_active);
    const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[ATS_STAGES]);
    if (threadIdx.x < 2 * ATS_STAGES) {
        mbar_init(smem_addr(&bars[threadIdx.x]), threadIdx.x < ATS_STAGES ? 1 : ATT_WARPS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    const uint32_t row_bytes = hs * 4, tile_bytes = ATT_CHUNK * row_bytes, stage_bytes = 2 * tile_bytes;
    const uint32_t ring = smem_addr(ring4);

    if (warp == ATT_WARPS) {
        // ------------------------------ producer ------------------------------
        for (uint32_t ck = ck_begin, n = 0; ck < ck_end; ck++, n++) {
            const uint32_t s = n % ATS_STAGES;
            if (n >= ATS_STAGES) mbar_wait(empty0 + 8 * s, ((n / ATS_STAGES) - 1) & 1, a.err, 7);
            const uint32_t t0 = ck * ATT_CHUNK;
            const uint32_t nt = min((uint32_t)ATT_CHUNK, pos + 1 - t0);
            // every row before `pos` was written by an earlier step; the row of `pos` by the preceding launch
            if (t0 + nt - 1 == pos) pdl_wait();
            if (lane == 0) mbar_expect_tx(full0 + 8 * s, 2 * nt * row_bytes);
            __syncwarp();
            const float *kbase = a.k_cache + (size_t)t0 * rstr + (size_t)kvh * hstr;
            const float *vbase = a.v_cache + (size_t)t0 * rstr + (size_t)kvh * hstr;
            const uint32_t dst = ring + s * stage_bytes;
            if (rstr == hs) {
                // head-major cache: the rows of the chunk are one contiguous run, one copy per tile
                if (lane == 0) bulk_copy_g2s(dst, kbase, nt * row_bytes, full0 + 8 * s);
                if (lane == 1) bulk_copy_g2s(dst + tile_bytes, vbase, nt * row_bytes, full0 + 8 * s);
            } else {
                for (uint32_t r = lane; r < nt; r += 32) {
                    bulk_copy_g2s(dst + r * row_bytes, kbase + (size_t)r * rstr, row_bytes, full0 + 8 * s);
                    bulk_copy_g2s(dst + tile_bytes + r * row_bytes, vbase + (size_t)r * rstr, row_bytes, full0 + 8 * s);
                }
            }
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    // Every warp keeps its own running softmax over the positions it owns (8 per chunk), so the warps never
    // synchronise inside the loop; their (max, sum, vector) triples are merged once at the end.
    pdl_wait();
    const uint32_t nchunk = hs / 4;  // float4 chunks per head (at most 32: one per lane)
    const float inv_sqrt = sqrtf((float)hs);
    const bool on = (uint32_t)lane < nchunk;
    float4 q[QH];
#pragma unroll
    for (int j = 0; j < QH; j++)
        q[j] = (on && hq0 + j < kv_mul) ? __ldcg(reinterpret_cast<const float4 *>(a.q + (size_t)(kvh * kv_mul + hq0 + j) * hs) + lane)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
    float M[QH], L[QH];
    float4 acc[QH];
#pragma unroll
    for (int j = 0; j < QH; j++) {
        M[j] = -INFINITY;
        L[j] = 0.0f;
        acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const unsigned char *ringp = reinterpret_cast<const unsigned char *>(ring4);
    float *my_sc = &s_sc[warp][0][0];

    for (uint32_t ck = ck_begin, n = 0; ck < ck_end; ck++, n++) {
        const uint32_t s = n % ATS_STAGES;
        const uint32_t t0 = ck * ATT_CHUNK;
        const uint32_t nt = min((uint32_t)ATT_CHUNK, pos + 1 - t0);
        mbar_wait(full0 + 8 * s, (n / ATS_STAGES) & 1, a.err, 8);
        const float4 *kt = reinterpret_cast<const float4 *>(ringp + (size_t)s * stage_bytes);
        const float4 *vt = reinterpret_cast<const float4 *>(ringp + (size_t)s * stage_bytes + tile_bytes);
        if ((uint32_t)warp * ATT_TPW < nt) {   // the warp has positions in this chunk
            // scores of the warp's 8 positions for every query head -> the warp's corner of shared memory
            float4 rows[ATT_TPW];
#pragma unroll
            for (int i = 0; i < ATT_TPW; i++) {
                const uint32_t tl = warp * ATT_TPW + i;
                rows[i] = (on && tl < nt) ? kt[tl * nchunk + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < QH; j++) {
                float part[ATT_TPW];
#pragma unroll
                for (int i = 0; i < ATT_TPW; i++)
                    part[i] = q[j].x * rows[i].x + q[j].y * rows[i].y + q[j].z * rows[i].z + q[j].w * rows[i].w;
                // 8 sums over the warp at once (8 -> 4 -> 2 -> 1 values per lane, then two plain steps)
                float f4[4], f2[2], f1;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const bool up = lane & 16;
                    const float keep = up ? part[2 * i + 1] : part[2 * i], give = up ? part[2 * i] : part[2 * i + 1];
                    f4[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
                }
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const bool up = lane & 8;
                    const float keep = up ? f4[2 * i + 1] : f4[2 * i], give = up ? f4[2 * i] : f4[2 * i + 1];
                    f2[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
                }
                {
                    const bool up = lane & 4;
                    const float keep = up ? f2[1] : f2[0], give = up ? f2[0] : f2[1];
                    f1 = keep + __shfl_xor_sync(0xffffffffu, give, 4);
                }
                f1 += __shfl_xor_sync(0xffffffffu, f1, 2);
                f1 += __shfl_xor_sync(0xffffffffu, f1, 1);
                if ((lane & 3) == 0) {
                    const uint32_t i = ((lane >> 4) & 1) | (((lane >> 3) & 1) << 1) | (((lane >> 2) & 1) << 2);
                    my_sc[j * ATT_TPW + i] = (warp * ATT_TPW + i < nt) ? f1 / inv_sqrt : -INFINITY;
                }
            }
            __syncwarp();
            // the value rows take the registers of the key rows
#pragma unroll
            for (int i = 0; i < ATT_TPW; i++) {
                const uint32_t tl = warp * ATT_TPW + i;
                rows[i] = (on && tl < nt) ? vt[tl * nchunk + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < QH; j++) {
                const float sv = my_sc[j * ATT_TPW + (lane & 7)];   // lane l looks after position l % 8
                float m = sv;
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
                const float mn = fmaxf(M[j], m);          // finite: position 0 of the warp is valid
                const float rs = expf(M[j] - mn);         // 0 at the warp's first chunk (M = -inf)
                const float e = expf(sv - mn);            // 0 for positions past the end
                M[j] = mn;
                float psum = 0.0f;
                acc[j].x *= rs;
                acc[j].y *= rs;
                acc[j].z *= rs;
                acc[j].w *= rs;
#pragma unroll
                for (int i = 0; i < ATT_TPW; i++) {
                    const float p = __shfl_sync(0xffffffffu, e, i);
                    psum += p;
                    acc[j].x = fmaf(p, rows[i].x, acc[j].x);
                    acc[j].y = fmaf(p, rows[i].y, acc[j].y);
                    acc[j].z = fmaf(p, rows[i].z, acc[j].z);
                    acc[j].w = fmaf(p, rows[i].w, acc[j].w);
                }
                L[j] = fmaf(L[j], rs, psum);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);   // this warp is done with the stage
    }

    // Merge of the eight warps.  Every copy has landed and been consumed: the ring now holds their vectors.
    float *s_acc = reinterpret_cast<float *>(ring4);   // [ATT_WARPS][QH][hs + 4]
    const uint32_t astr = hs + 4;
    att_cons_sync();
#pragma unroll
    for (int j = 0; j < QH; j++) {
        if (on) reinterpret_cast<float4 *>(s_acc + ((size_t)warp * QH + j) * astr)[lane] = acc[j];
        if (lane == 0) {
            s_red[j][warp] = M[j];
            s_sum[j][warp] = L[j];
        }
    }
    att_cons_sync();
    for (uint32_t e = threadIdx.x; e < QH * hs; e += ATT_NT) {
        const uint32_t j = e / hs, i = e % hs;
        if (hq0 + j >= kv_mul) continue;
        float mb = s_red[j][0];
#pragma unroll
        for (int w = 1; w < ATT_WARPS; w++) mb = fmaxf(mb, s_red[j][w]);
        float sv = 0.0f, lb = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) {
            const float f = expf(s_red[j][w] - mb);   // 0 for a warp that had no positions
            sv = fmaf(s_acc[((size_t)w * QH + j) * astr + i], f, sv);
            lb = fmaf(s_sum[j][w], f, lb);
        }
        float *dst = a.scratch + ((size_t)(kvh * kv_mul + hq0 + j) * max_splits + split) * (hs + 4);
        dst[i] = sv;
        if (i == 0) {
            dst[hs] = mb;
            dst[hs + 1] = lb;
        }
    }

    // Ticket: the last block of this (KV head, query-head group) merges all splits.
    __threadfence();
    att_cons_sync();
    uint32_t *counter = a.counters + kvh * gridDim.z + blockIdx.z;
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(counter, 1u);
        s_last = (ticket == nsplit_active - 1);
        if (s_last) *counter = 0;  // ready for the next launch
    }
    att_cons_sync();
    if (!s_last) {
        if (threadIdx.x == 0) stamp_end(a.stamp);
        return;
    }
    __threadfence();
#pragma unroll
    for (int j = 0; j < QH; j++) {
        float m = -INFINITY;
        if (hq0 + j < kv_mul) {
            const float *base = a.scratch + (size_t)(kvh * kv_mul + hq0 + j) * max_splits * (hs + 4);
            for (uint32_t sp = threadIdx.x; sp < nsplit_active; sp += ATT_NT) m = fmaxf(m, __ldcg(base + (size_t)sp * (hs + 4) + hs));
        }
        m = warp_max(m);
        if (lane == 0) s_red[j][warp] = m;
    }
    att_cons_sync();
    if (threadIdx.x < QH) {
        float m = s_red[threadIdx.x][0];
#pragma unroll
        for (int w = 1; w < ATT_WARPS; w++) m = fmaxf(m, s_red[threadIdx.x][w]);
        s_M[threadIdx.x] = m;
    }
    att_cons_sync();
#pragma unroll
    for (int j = 0; j < QH; j++) {
        if (hq0 + j >= kv_mul) continue;   // uniform over the block
        const float *base = a.scratch + (size_t)(kvh * kv_mul + hq0 + j) * max_splits * (hs + 4);
        const float Mj = s_M[j];
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        float Lw = 0.0f;
        for (uint32_t sp = warp; sp < nsplit_active; sp += ATT_WARPS) {
            const float *row = base + (size_t)sp * (hs + 4);
            const float w = expf(__ldcg(row + hs) - Mj);
            Lw = fmaf(__ldcg(row + hs + 1), w, Lw);
            if (on) {
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(row) + lane);
                o.x = fmaf(v.x, w, o.x);
                o.y = fmaf(v.y, w, o.y);
                o.z = fmaf(v.z, w, o.z);
                o.w = fmaf(v.w, w, o.w);
            }
        }
        if (on) reinterpret_cast<float4 *>(s_acc + ((size_t)warp * QH + j) * astr)[lane] = o;
        if (lane == 0) s_red[j][warp] = Lw;
    }
    att_cons_sync();
    for (uint32_t e = threadIdx.x; e < QH * hs; e += ATT_NT) {
        const uint32_t j = e / hs, i = e % hs;
        if (hq0 + j >= kv_mul) continue;
        float Lt = 0.0f, o = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) {
            Lt += s_red[j][w];
            o += s_acc[((size_t)w * QH + j) * astr + i];
        }
        a.xb[(size_t)(kvh * kv_mul + hq0 + j) * hs + i] = o / Lt;
    }
    if (threadIdx.x == 0) stamp_end(a.stamp);
}

template <int QH>
static int launch_stream(const AttnArgs &a, uint32_t nchunks, uint32_t n_kv, uint32_t zgroups, cudaStream_t stream, bool pdl)
{
    const size_t smem = (size_t)ATS_STAGES * 2 * ATT_CHUNK * a.p.head_size * sizeof(float);
    static bool ready[MAX_DEVICES] = {};   // per instantiation and device
    const int dev = current_device();
    if (dev < 0) return WGB_ERR_CUDA;
    if (!ready[dev]) {
        WGB_CUDA(cudaFuncSetAttribute(attn_stream_kernel<QH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ATS_STAGES * 2 * ATT_CHUNK * 128 * sizeof(float))));
        ready[dev] = true;
    }
    uint32_t splits = (uint32_t)sm_count() / (n_kv * zgroups);   // one block per SM
    if (splits < 1) splits = 1;
    if (splits > nchunks) splits = nchunks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, n_kv, zgroups);
    cfg.blockDim = dim3(ATS_NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    WGB_CUDA(cudaLaunchKernelEx(&cfg, attn_stream_kernel<QH>, a));
    return WGB_OK;
}

// Long contexts with head sizes up to 128 and at most two query heads per KV head.
static int launch_stream_any(const AttnArgs &a, uint32_t nchunks, cudaStream_t stream, bool pdl)
{
    const uint32_t n_kv = a.p.n_heads / a.p.kv_mul;
    if (a.p.kv_mul == 2) return launch_stream<2>(a, nchunks, n_kv, 1, stream, pdl);
    return launch_stream<1>(a, nchunks, n_kv, 1, stream, pdl);
}

template <int QH, int VC>
static int launch_split(const AttnArgs &a, uint32_t nchunks, uint32_t nchunks_hint, uint32_t n_kv, uint32_t zgroups,
                        cudaStream_t stream, bool pdl)
{
    // One chunk per block while all blocks of such a grid are resident at once (a second wave would double
    // the latency); beyond that, as many splits as fit and several chunks per block.
    static int occ_single[MAX_DEVICES] = {}, occ_multi[MAX_DEVICES] = {};   // per instantiation and device
    const int dev = current_device();
    if (dev < 0) return a.q ? WGB_ERR_CUDA : -1;
    if (!occ_single[dev]) {
        int one = 0, many = 0;
        WGB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&one, attn_split_kernel<QH, VC, false>, ATT_NT, 0));
        WGB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&many, attn_split_kernel<QH, VC, true>, ATT_NT, 0));
        occ_multi[dev] = many < 1 ? 1 : many;
        occ_single[dev] = one < 1 ? 1 : one;
    }
    const int per_sm_single = occ_single[dev], per_sm_multi = occ_multi[dev];
    const uint32_t heads = n_kv * zgroups;
    if (!a.q) {   // sizing query (attn_sizing_class): no launch
        return (uint64_t)nchunks_hint * heads > (uint64_t)per_sm_single * (uint32_t)sm_count() ? 1 : 0;
    }
    // `nchunks_hint`: chunks up to the furthest position this launch is expected to serve (performance only:
    // either kernel is correct for any position inside the cache).
    const bool multi = (uint64_t)nchunks_hint * heads > (uint64_t)per_sm_single * (uint32_t)sm_count();
    // Up to two query heads per KV head the streaming kernel is bandwidth-bound and wins; with more, the
    // arithmetic per cache byte grows (8 heads: 4 FMA per byte) and its eight consumer warps per SM hide
    // less latency than two resident blocks of the chunk-walking split kernel.
    if (multi && VC == 1 && a.p.kv_mul <= 2) return launch_stream_any(a, nchunks, stream, pdl);
    uint32_t splits = nchunks;
    if (multi) {
        splits = (uint32_t)per_sm_multi * (uint32_t)sm_count() / heads;
        if (splits < 1) splits = 1;
        if (splits > nchunks) splits = nchunks;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, n_kv, zgroups);
    cfg.blockDim = dim3(ATT_NT);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (multi) WGB_CUDA(cudaLaunchKernelEx(&cfg, attn_split_kernel<QH, VC, true>, a));
    else WGB_CUDA(cudaLaunchKernelEx(&cfg, attn_split_kernel<QH, VC, false>, a));
    return WGB_OK;
}

// `a.counters` must hold n_kv_heads * ceil(kv_mul / QH) zeroed words (QH as chosen below) and `a.scratch`
// attn_scratch_floats() floats.
int launch_attention(const AttnArgs &a, cudaStream_t stream, bool pdl)
{
    const wgb_attn_params &p = a.p;
    WGB_REQUIRE(p.head_size % 4 == 0 && p.head_size <= 256 && p.head_size > 0, "head_size %u unsupported", p.head_size);
    WGB_REQUIRE(p.kv_mul > 0 && p.n_heads % p.kv_mul == 0, "n_heads %u not a multiple of kv_mul %u", p.n_heads, p.kv_mul);
    const uint32_t n_kv = p.n_heads / p.kv_mul;
    const uint32_t nchunks = attn_num_splits(p.seq_len);
    // With the position on the device, p.pos is the caller's bound on it (0: unknown, assume a short context).
    const uint32_t nh = std::min(nchunks, p.pos / ATT_CHUNK + 1);
    const bool big = p.head_size > 128;
    // query heads per block: the largest of 4 / 2 / 1 that divides nothing away (tail heads masked)
    const uint32_t qh = p.kv_mul >= 4 ? 4 : (p.kv_mul >= 2 ? 2 : 1);
    const uint32_t zg = (p.kv_mul + qh - 1) / qh;
    if (qh == 4) return big ? launch_split<4, 2>(a, nchunks, nh, n_kv, zg, stream, pdl) : launch_split<4, 1>(a, nchunks, nh, n_kv, zg, stream, pdl);
    if (qh == 2) return big ? launch_split<2, 2>(a, nchunks, nh, n_kv, zg, stream, pdl) : launch_split<2, 1>(a, nchunks, nh, n_kv, zg, stream, pdl);
    return big ? launch_split<1, 2>(a, nchunks, nh, n_kv, zg, stream, pdl) : launch_split<1, 1>(a, nchunks, nh, n_kv, zg, stream, pdl);
}

// 0 / 1: which of the two launch shapes launch_attention picks for positions up to p.pos (a caller that
// records launches for later replay re-records when the class changes); negative on error.
int attn_sizing_class(const wgb_attn_params &p)
{
    AttnArgs a = {};
    a.p = p;
    a.pos = reinterpret_cast<const uint32_t *>(&a);   // "position on the device": p.pos is the bound
    const int r = launch_attention(a, nullptr, false);
    return r > 1 ? -1 : r;
}

}  // namespace wgb

using namespace wgb;

WGB_EXPORT int wgb_attention(const wgb_attn_params *p, const float *d_q, const float *d_key_cache,
                             const float *d_value_cache, float *d_attn, float *d_xb, void *stream)
{
    WGB_REQUIRE(p && d_q && d_key_cache && d_value_cache && d_xb, "null argument");
    WGB_REQUIRE(p->pos < p->seq_len, "pos %u outside a cache of %u positions", p->pos, p->seq_len);
    WGB_REQUIRE(p->kv_mul > 0 && p->n_heads % p->kv_mul == 0 && p->kv_dim == (p->n_heads / p->kv_mul) * p->head_size,
                "inconsistent attention parameters");
    AttnArgs a = {};
    a.p = *p;
    a.pos = nullptr;
    a.q = d_q;
    a.k_cache = d_key_cache;
    a.v_cache = d_value_cache;
    a.xb = d_xb;
    if (d_attn) {
        attn_full_kernel<<<p->n_heads, ATT_NT, 0, as_stream(stream)>>>(a, d_attn);
        WGB_LAUNCH_CHECK("attn_full_kernel");
        return WGB_OK;
    }
    WGB_REQUIRE(p->head_size % 4 == 0 && p->head_size <= 256, "head_size %u unsupported", p->head_size);
    // Scratch of the stand-alone op: per device, grown on demand and kept for the life of the process.
    DeviceState *ds = device_state();
    if (!ds) return WGB_ERR_CUDA;
    const size_t need = attn_scratch_floats(p->n_heads, p->head_size, p->seq_len);
    if (need > ds->attn_scratch_floats) {
        WGB_CUDA(cudaStreamSynchronize(as_stream(stream)));
        if (ds->attn_scratch) cudaFree(ds->attn_scratch);
        ds->attn_scratch = nullptr;
        ds->attn_scratch_floats = 0;
        WGB_CUDA(cudaMalloc((void **)&ds->attn_scratch, need * sizeof(float)));
        ds->attn_scratch_floats = need;
    }
    if (p->n_heads > ds->attn_ncounters) {
        WGB_CUDA(cudaStreamSynchronize(as_stream(stream)));
        if (ds->attn_counters) cudaFree(ds->attn_counters);
        ds->attn_counters = nullptr;
        ds->attn_ncounters = 0;
        WGB_CUDA(cudaMalloc((void **)&ds->attn_counters, p->n_heads * sizeof(uint32_t)));
        WGB_CUDA(cudaMemset(ds->attn_counters, 0, p->n_heads * sizeof(uint32_t)));
        ds->attn_ncounters = p->n_heads;
    }
    a.scratch = ds->attn_scratch;
    a.counters = ds->attn_counters;
    return launch_attention(a, as_stream(stream), false);
}

// ---------------------------------------------------------------------------------------------
// Attention entry point that never allocates.
//
// wgb_attention keeps its split-K scratch in device memory that it allocates (and regrows) on demand.
// Some hosts cannot have that on the call path: a server that has handed the whole device to its own
// memory pool has nothing left for cudaMalloc to take, and in a latency-critical loop the device-wide
// synchronisation inside cudaMalloc / cudaFree stalls every other stream.  This variant runs the same
// kernels on scratch that is part of the loaded module: two file-scope __device__ arrays of fixed size.
// Shapes whose scratch would not fit are rejected, never served from another buffer.
// ---------------------------------------------------------------------------------------------
#define WGB_ATTN_STATIC_DEVICES 64

static __device__ __align__(256) float g_static_scratch[WGB_ATTENTION_STATIC_MAX_SCRATCH_FLOATS];
static __device__ __align__(256) uint32_t g_static_counters[WGB_ATTENTION_STATIC_MAX_HEADS];

namespace {

struct StaticScratch {
    float *scratch = nullptr;
    uint32_t *counters = nullptr;
};
StaticScratch g_static[WGB_ATTN_STATIC_DEVICES];   // per device: every device has its own copy of the arrays
std::mutex g_static_mutex;

__global__ void clear_words_kernel(uint32_t *p, uint32_t n)
{
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) p[i] = 0;
}

// Resolves the arrays' addresses on the current device the first time the device is seen.
int static_scratch(StaticScratch *out)
{
    int dev = -1;
    WGB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= WGB_ATTN_STATIC_DEVICES) return fail(WGB_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static[dev].scratch) {
        float *s = nullptr;
        uint32_t *c = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&s, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(attention scratch)");
        e = cudaGetSymbolAddress((void **)&c, g_static_counters);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(attention counters)");
        g_static[dev].scratch = s;
        g_static[dev].counters = c;
    }
    *out = g_static[dev];
    return WGB_OK;
}

}  // namespace

WGB_EXPORT int wgb_attention_static(const wgb_attn_params *p, const float *d_q, const float *d_key_cache,
                                    const float *d_value_cache, float *d_xb, void *stream)
{
    WGB_REQUIRE(p && d_q && d_key_cache && d_value_cache && d_xb, "null argument");
    WGB_REQUIRE(p->pos < p->seq_len, "pos %u outside a cache of %u positions", p->pos, p->seq_len);
    WGB_REQUIRE(p->kv_mul > 0 && p->n_heads % p->kv_mul == 0 && p->kv_dim == (p->n_heads / p->kv_mul) * p->head_size,
                "inconsistent attention parameters");
    WGB_REQUIRE(p->head_size % 4 == 0 && p->head_size <= 256 && p->head_size > 0, "head_size %u unsupported", p->head_size);
    const size_t need = attn_scratch_floats(p->n_heads, p->head_size, p->seq_len);
    if (need > (size_t)WGB_ATTENTION_STATIC_MAX_SCRATCH_FLOATS)
        return fail(WGB_ERR_INVALID,
                    "wgb_attention_static: %u heads x %u positions x head size %u need %zu scratch floats, the built-in "
                    "scratch holds %d; use wgb_attention",
                    p->n_heads, p->seq_len, p->head_size, need, WGB_ATTENTION_STATIC_MAX_SCRATCH_FLOATS);
    if (p->n_heads > (uint32_t)WGB_ATTENTION_STATIC_MAX_HEADS)
        return fail(WGB_ERR_INVALID, "wgb_attention_static: %u heads, the built-in scratch serves at most %d; use wgb_attention",
                    p->n_heads, WGB_ATTENTION_STATIC_MAX_HEADS);
    StaticScratch ss;
    int rc = static_scratch(&ss);
    if (rc) return rc;
    cudaStream_t s = as_stream(stream);
    // The tickets must start at zero.  The kernel leaves them there, but a launch that was cut short
    // (a failed launch further up the stream, a process that reuses the context) must not poison this one.
    clear_words_kernel<<<1, 256, 0, s>>>(ss.counters, p->n_heads);
    WGB_LAUNCH_CHECK("clear_words_kernel");
    AttnArgs a = {};
    a.p = *p;
    a.pos = nullptr;
    a.q = d_q;
    a.k_cache = d_key_cache;
    a.v_cache = d_value_cache;
    a.xb = d_xb;
    a.scratch = ss.scratch;
    a.counters = ss.counters;
    return launch_attention(a, s, false);
}
