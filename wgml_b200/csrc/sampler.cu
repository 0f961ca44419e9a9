// Temperature / top-p sampling on the device, so that non-greedy decoding needs no vocabulary-sized copy to
// the host either.
//
// Semantics: Sampler::sample (crates/wgml/src/models/sampler.rs:32-131): logits /= temperature, softmax with the
// maximum subtracted (ops/softmax.rs:36-49), then either the plain inverse-CDF walk in index order
// (`sample_mult`, topp outside (0, 1)) or nucleus sampling (`sample_topp`): candidates with probability
// >= (1 - topp) / (n - 1), sorted by decreasing probability (a stable sort: equal probabilities keep index
// order), cut where the running sum first exceeds topp, and the inverse-CDF walk over that prefix with
// r = coin * running sum.  temperature == 0 is the greedy argmax.  The reference draws `coin` from an unseeded
// generator; here it is a counter-based draw (seed, position), the same 24-bit form as rand's f32 sample, so a
// sequence can be reproduced and resumed.
//
// One block does a whole draw.  The maximum and the exponentials are computed in parallel; their sum is taken
// by ONE thread in index order, as the reference does: a sequential f32 sum of 32000 to 50257 nearly equal terms
// is off by up to 1e-4 relative (the rounding is biased, not random), every probability inherits that factor,
// and a tree sum -- more accurate -- would move the draws of flat distributions to other tokens than the
// reference's.  The sequential passes read the values through shared memory in double-buffered chunks filled
// by the other warps (about 2 ns per term: 0.1 ms for a 50257-token vocabulary).  Candidates are compacted in
// index order; a bitonic sort of 64-bit keys (probability bits descending, index ascending: the order the
// reference's stable sort produces) runs in shared memory for up to 4096 candidates and in global scratch
// beyond; the two prefix walks are done by one thread in the reference's order of additions.
#include "kernels.h"

namespace wgb {

constexpr int SMP_NT = 1024;
constexpr uint32_t SMP_SMEM_KEYS = 4096;

__host__ __device__ inline float sampler_coin(unsigned long long seed, unsigned long long draw)
{
    unsigned long long z = seed + (draw + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);   // 24 bits in [0, 1)
}

__device__ __forceinline__ float block_reduce_max(float v, float *red)
{
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = (threadIdx.x & 31) < SMP_NT / 32 ? red[threadIdx.x & 31] : -INFINITY;
    return warp_max(t);
}
__device__ __forceinline__ float block_reduce_sum(float v, float *red)
{
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = (threadIdx.x & 31) < SMP_NT / 32 ? red[threadIdx.x & 31] : 0.0f;
    return warp_sum(t);
}

// Bitonic sort, ascending, of `n` (a power of two) 64-bit keys by the whole block.
__device__ void block_bitonic(unsigned long long *keys, uint32_t n)
{
    for (uint32_t k = 2; k <= n; k <<= 1) {
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            for (uint32_t i = threadIdx.x; i < n; i += SMP_NT) {
                const uint32_t l = i ^ j;
                if (l > i) {
                    const unsigned long long a = keys[i], b = keys[l];
                    const bool up = (i & k) == 0;
                    if ((a > b) == up) {
                        keys[i] = b;
                        keys[l] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
}

// Calls op(i, v[i]) for i = 0, 1, ... in order from thread 0 until it returns false or i reaches n; the other
// warps stream v through the two halves of `buf` (2 * SEQ_CHUNK floats of shared memory).  Block-wide call.
constexpr uint32_t SEQ_CHUNK = 4096;
template <typename Op>
__device__ void sequential_pass(const float *v, uint32_t n, float *buf, uint32_t *stop, Op op)
{
    const uint32_t nchunks = (n + SEQ_CHUNK - 1) / SEQ_CHUNK;
    if (threadIdx.x == 0) *stop = 0;
    __syncthreads();
    for (uint32_t c = 0; c <= nchunks; c++) {
        if (threadIdx.x >= 32 && c < nchunks) {
            float *dst = buf + (c & 1) * SEQ_CHUNK;
            const uint32_t base = c * SEQ_CHUNK;
            for (uint32_t i = threadIdx.x - 32; i < SEQ_CHUNK; i += SMP_NT - 32)
                dst[i] = base + i < n ? v[base + i] : 0.0f;
        } else if (threadIdx.x == 0 && c > 0) {
            const float *src = buf + ((c - 1) & 1) * SEQ_CHUNK;
            const uint32_t base = (c - 1) * SEQ_CHUNK, cnt = min(SEQ_CHUNK, n - base);
            bool go = true;
            uint32_t i = 0;
            for (; go && i + 8 <= cnt; i += 8) {
                float t[8];
#pragma unroll
                for (int k = 0; k < 8; k++) t[k] = src[i + k];
#pragma unroll
                for (int k = 0; k < 8; k++) go = go && op(base + i + k, t[k]);
            }
            for (; go && i < cnt; i++) go = op(base + i, src[i]);
            if (!go) *stop = 1;
        }
        __syncthreads();
        if (*stop) break;
    }
    __syncthreads();
}

struct SampleArgs {
    const float *logits;
    uint32_t n;
    float temperature, topp;
    float coin;                       // used when `seeded` is 0
    int seeded;                       // 1: coin = sampler_coin(seed, *ls.pos + 1) (the position the token will occupy)
    unsigned long long seed;
    float *prob;                      // scratch: n floats
    unsigned long long *keys;         // scratch: next power of two >= n 64-bit words
    uint32_t *out_index;              // stand-alone use
    LoopState ls;                     // token loop (have_loop)
    int have_loop;
};

__global__ void __launch_bounds__(SMP_NT) sample_kernel(const __grid_constant__ SampleArgs a)
{
    __shared__ float red[32];
    __shared__ uint32_t s_count[SMP_NT / 32];
    __shared__ uint32_t s_n0, s_token, s_stop;
    __shared__ float s_sum;
    __shared__ unsigned long long s_keys[SMP_SMEM_KEYS];   // also the chunk buffers of the sequential passes
    static_assert(SMP_SMEM_KEYS * sizeof(unsigned long long) >= 2 * SEQ_CHUNK * sizeof(float), "chunk buffers alias the keys");
    float *seq_buf = reinterpret_cast<float *>(s_keys);
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t n = a.n;
    uint32_t step = 0;
    if (a.have_loop) {
        // forced prompt tokens (crates/wgml-chat/src/sampler.rs:102-107): nothing to sample
        step = *a.ls.step;
        if (step + 1 < a.ls.n_prompt) {
            if (threadIdx.x == 0) {
                const uint32_t next = a.ls.prompt[step + 1];
                a.ls.out_tokens[step] = next;
                *a.ls.token = next;
                *a.ls.pos = *a.ls.pos + 1;
                *a.ls.step = step + 1;
            }
            return;
        }
    }
    const float coin = a.seeded ? sampler_coin(a.seed, (unsigned long long)(*a.ls.pos) + 1ull) : a.coin;
    // logits / temperature, maximum, exponentials, sum
    float m = -INFINITY;
    for (uint32_t i = threadIdx.x; i < n; i += SMP_NT) m = fmaxf(m, __ldcg(a.logits + i) / a.temperature);
    m = block_reduce_max(m, red);
    for (uint32_t i = threadIdx.x; i < n; i += SMP_NT) a.prob[i] = expf(__ldcg(a.logits + i) / a.temperature - m);
    __syncthreads();
    {
        float acc = 0.0f;   // thread 0 only
        sequential_pass(a.prob, n, seq_buf, &s_stop, [&](uint32_t, float e) {
            acc += e;
            return true;
        });
        if (threadIdx.x == 0) s_sum = acc;
        __syncthreads();
    }
    const float sum = s_sum;
    const bool nucleus = a.topp > 0.0f && a.topp < 1.0f;
    if (!nucleus) {
        // sample_mult: inverse CDF in index order, the additions in the reference's order
        float cdf = 0.0f;
        uint32_t pick = n - 1;
        sequential_pass(a.prob, n, seq_buf, &s_stop, [&](uint32_t i, float e) {
            cdf += e / sum;
            if (coin < cdf) {
                pick = i;
                return false;
            }
            return true;
        });
        if (threadIdx.x == 0) s_token = pick;
    } else {
        // candidates p >= cutoff, compacted in index order: thread t owns the contiguous run [t * per, (t + 1) * per)
        const float cutoff = (1.0f - a.topp) / ((float)n - 1.0f);
        const uint32_t per = (n + SMP_NT - 1) / SMP_NT;
        const uint32_t i0 = min(threadIdx.x * per, n), i1 = min(i0 + per, n);
        uint32_t mine = 0;
        for (uint32_t i = i0; i < i1; i++) mine += (a.prob[i] / sum >= cutoff) ? 1u : 0u;
        // block-wide exclusive scan of the counts
        uint32_t incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
            if ((threadIdx.x & 31) >= (uint32_t)o) incl += v;
        }
        if ((threadIdx.x & 31) == 31) s_count[threadIdx.x >> 5] = incl;
        __syncthreads();
        if (threadIdx.x < 32) {
            uint32_t v = s_count[threadIdx.x], w = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t u = __shfl_up_sync(0xffffffffu, w, o);
                if (threadIdx.x >= (uint32_t)o) w += u;
            }
            s_count[threadIdx.x] = w - v;   // exclusive prefix of the warp totals
            if (threadIdx.x == 31) s_n0 = w;
        }
        __syncthreads();
        const uint32_t n0 = s_n0;
        uint32_t npad = 1;
        while (npad < n0) npad <<= 1;
        unsigned long long *keys = npad <= SMP_SMEM_KEYS ? s_keys : a.keys;
        uint32_t at = s_count[threadIdx.x >> 5] + incl - mine;
        for (uint32_t i = i0; i < i1; i++) {
            const float p = a.prob[i] / sum;
            if (p >= cutoff) {
                // ascending key order = probability descending (p >= 0: its bits order like its value), index ascending
                keys[at++] = ((unsigned long long)(~__float_as_uint(p)) << 32) | i;
            }
        }
        for (uint32_t i = n0 + threadIdx.x; i < npad; i += SMP_NT) keys[i] = ~0ull;
        __syncthreads();
        block_bitonic(keys, npad);
        if (threadIdx.x == 0) {
            // running sum until it exceeds topp, then the inverse CDF over that prefix (sampler.rs:104-127)
            float cumulative = 0.0f;
            uint32_t last = n0 ? n0 - 1 : 0;
            for (uint32_t i = 0; i < n0; i++) {
                cumulative += __uint_as_float(~(uint32_t)(keys[i] >> 32));
                if (cumulative > a.topp) {
                    last = i;
                    break;
                }
            }
            const float r = coin * cumulative;
            float cdf = 0.0f;
            uint32_t pick = n0 ? (uint32_t)(keys[last] & 0xffffffffu) : 0u;
            for (uint32_t i = 0; i <= last && n0; i++) {
                cdf += __uint_as_float(~(uint32_t)(keys[i] >> 32));
                if (r < cdf) {
                    pick = (uint32_t)(keys[i] & 0xffffffffu);
                    break;
                }
            }
            s_token = pick;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t next = s_token;
        if (a.have_loop) {
            a.ls.out_tokens[step] = next;
            *a.ls.token = next;
            *a.ls.pos = *a.ls.pos + 1;
            *a.ls.step = step + 1;
        } else {
            *a.out_index = next;
        }
    }
}

size_t sampler_scratch_bytes(uint32_t n)
{
    size_t npad = 1;
    while (npad < n) npad <<= 1;
    return (size_t)n * sizeof(float) + 256 + npad * sizeof(unsigned long long);
}

// Enqueues one draw.  `scratch` holds sampler_scratch_bytes(n) bytes.  With a loop state the kernel is the
// sampling step of the token loop (forced prompt tokens, then a seeded draw per generated position).
int launch_sample(const float *logits, uint32_t n, float temperature, float topp, float coin, int seeded, unsigned long long seed,
                  void *scratch, uint32_t *out_index, const LoopState *ls, cudaStream_t stream)
{
    SampleArgs a = {};
    a.logits = logits;
    a.n = n;
    a.temperature = temperature;
    a.topp = topp;
    a.coin = coin;
    a.seeded = seeded;
    a.seed = seed;
    a.prob = reinterpret_cast<float *>(scratch);
    a.keys = reinterpret_cast<unsigned long long *>(reinterpret_cast<char *>(scratch) + (((size_t)n * sizeof(float) + 255) & ~(size_t)255));
    a.out_index = out_index;
    if (ls) {
        a.ls = *ls;
        a.have_loop = 1;
    }
    sample_kernel<<<1, SMP_NT, 0, stream>>>(a);
    WGB_LAUNCH_CHECK("sample_kernel");
    return WGB_OK;
}

}  // namespace wgb

using namespace wgb;

WGB_EXPORT float wgb_sampler_coin(uint64_t seed, uint64_t draw) { return sampler_coin(seed, draw); }

WGB_EXPORT int wgb_sample(const float *d_logits, size_t n, float temperature, float topp, float coin, uint32_t *d_token,
                          void *stream)
{
    WGB_REQUIRE(d_logits && d_token && n > 0 && n <= 0x7fffffffull, "bad sampler arguments");
    WGB_REQUIRE(temperature >= 0.0f && coin >= 0.0f && coin < 1.0f, "temperature %g / coin %g out of range", temperature, coin);
    if (temperature == 0.0f) return wgb_argmax(d_logits, n, d_token, stream);   // Sampler::sample, sampler.rs:33-35
    DeviceState *ds = device_state();
    if (!ds) return WGB_ERR_CUDA;
    const size_t need = sampler_scratch_bytes((uint32_t)n);
    if (need > ds->sampler_scratch_bytes) {
        WGB_CUDA(cudaStreamSynchronize(as_stream(stream)));
        if (ds->sampler_scratch) cudaFree(ds->sampler_scratch);
        ds->sampler_scratch = nullptr;
        ds->sampler_scratch_bytes = 0;
        WGB_CUDA(cudaMalloc((void **)&ds->sampler_scratch, need));
        ds->sampler_scratch_bytes = need;
    }
    return launch_sample(d_logits, (uint32_t)n, temperature, topp, coin, 0, 0, ds->sampler_scratch, d_token, nullptr, as_stream(stream));
}
