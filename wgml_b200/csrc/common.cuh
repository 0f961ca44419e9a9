// Shared declarations of the wgml_b200 library: status handling, block geometry, warp helpers.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include <string>

#include "../../include/wgml_b200.h"

#define WGB_EXPORT extern "C" __attribute__((visibility("default")))

namespace wgb {

// Records the message returned by wgb_last_error() for the calling thread and returns `code`.
int fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
int cuda_fail(cudaError_t e, const char *what);

#define WGB_CUDA(call)                                                     \
    do {                                                                   \
        cudaError_t e__ = (call);                                          \
        if (e__ != cudaSuccess) return ::wgb::cuda_fail(e__, #call);       \
    } while (0)

// After a kernel launch: launch-configuration errors surface here, not at the next sync.
#define WGB_LAUNCH_CHECK(what)                                             \
    do {                                                                   \
        cudaError_t e__ = cudaGetLastError();                              \
        if (e__ != cudaSuccess) return ::wgb::cuda_fail(e__, what);        \
    } while (0)

#define WGB_REQUIRE(cond, ...)                                             \
    do {                                                                   \
        if (!(cond)) return ::wgb::fail(WGB_ERR_INVALID, __VA_ARGS__);     \
    } while (0)

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// Per-device state.  Everything the library sets up once per device (the status word of the bounded waits,
// opt-ins to large dynamic shared memory, occupancy figures, scratch of the stand-alone ops) hangs off the
// current device's entry, so a process may drive several devices.  Entries are created under a mutex; the
// calls of one device must still come from one host thread at a time (the C ABI is not thread-safe).
constexpr int MAX_DEVICES = 64;
struct DeviceState {
    int ordinal = -1;
    int sms = 0;
    uint32_t *err = nullptr;              // device status word: 0, or the code of the first bounded wait that expired
    bool gemv_attrs = false;              // fused matrix-vector kernels opted in to large dynamic shared memory
    bool tiles_attrs = false;             // the same for the tensor-memory kernel
    bool prefill_attrs = false;           // the same for the batched tensor-memory kernel
    bool prefill6_attrs = false;          // the same for its Q6_K counterpart
    bool prefill8_attrs = false;          // and its Q8_0 counterpart
    float *attn_scratch = nullptr;        // scratch of the stand-alone attention op, grown on demand
    size_t attn_scratch_floats = 0;
    uint32_t *attn_counters = nullptr;
    size_t attn_ncounters = 0;
    unsigned long long *argmax_part = nullptr;   // partial keys of the stand-alone argmax
    float *sampler_scratch = nullptr;     // work area of the stand-alone sampler
    size_t sampler_scratch_bytes = 0;
};
// Entry of the current device (created on first use), or NULL with the error recorded.
DeviceState *device_state();
// Ordinal of the current device in [0, MAX_DEVICES), or -1 with the error recorded.
int current_device();

// Number of SMs of the current device (148 on B200).
int sm_count();

// Limits of the device-side waits, in nanoseconds of %globaltimer.  `peer`: how long a kernel waits for the
// flags of the other ranks of a tensor-parallel group (wgb_set_wait_limit_ms; default 2 s, which has to cover
// the skew between the ranks' hosts).  `local`: waits inside one thread block (shared-memory barriers fed by
// the block's own warps and bulk copies); longer than `peer`, because a block's warps may themselves be held
// by a peer wait.
struct WaitLimits { unsigned long long peer_ns, local_ns; };
WaitLimits wait_limits();

__host__ __device__ constexpr int block_bytes(int qtype)
{
    return qtype == WGB_F32 ? 4 : qtype == WGB_F16 ? 2 : qtype == WGB_Q4_0 ? 18 : qtype == WGB_Q4_1 ? 20
         : qtype == WGB_Q5_0 ? 22 : qtype == WGB_Q5_1 ? 24 : qtype == WGB_Q8_0 ? 34 : qtype == WGB_Q4_K ? 144
         : qtype == WGB_Q5_K ? 176 : qtype == WGB_Q6_K ? 210 : qtype == WGB_Q8_K ? 292 : 0;
}

__host__ __device__ constexpr int block_len(int qtype)
{
    return (qtype == WGB_F32 || qtype == WGB_F16) ? 1
         : (qtype == WGB_Q4_0 || qtype == WGB_Q4_1 || qtype == WGB_Q5_0 || qtype == WGB_Q5_1 || qtype == WGB_Q8_0) ? 32
         : (qtype == WGB_Q4_K || qtype == WGB_Q5_K || qtype == WGB_Q6_K || qtype == WGB_Q8_K) ? 256 : 0;
}

#ifdef __CUDACC__
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a thread block of NT threads (NT a multiple of 32, <= 1024); every thread gets the
// result.  `red` is shared scratch of at least 32 floats; safe to call repeatedly.
template <int NT>
__device__ __forceinline__ float block_sum(float v, float *red)
{
    v = warp_sum(v);
    if (NT == 32) return v;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < NT / 32) ? red[lane] : 0.0f;
    return warp_sum(t);
}

template <int NT>
__device__ __forceinline__ float block_max(float v, float *red)
{
    v = warp_max(v);
    if (NT == 32) return v;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < NT / 32) ? red[lane] : -INFINITY;
    return warp_max(t);
}

// Programmatic dependent launch (sm_90+): `pdl_wait` blocks until the preceding kernel in the
// stream has completed and its writes are visible; `pdl_launch_dependents` lets the following
// kernel start its independent prologue.  Both are no-ops for a kernel launched without the
// programmatic-serialization attribute.
// Rule for every read placed BEFORE pdl_wait: it may touch only memory that no launch still in flight can
// write -- weights, launch parameters, and KV-cache rows of positions earlier than this step's (the rows at the
// current position are written by the step's own q/k/v launch and are read after the wait).  Activations,
// the token / position scalars, flags, tickets and the status word are always read after the wait.  A kernel
// launched with the attribute whose predecessor was launched with it too must itself wait before it exits,
// otherwise its successor's wait no longer covers the predecessor.
// End-of-launch time stamp for per-launch timing inside a graph replay: the latest %globaltimer (ns) over
// the blocks of a launch.  Called by one thread per block after its last store; a NULL slot costs a branch.
__device__ __forceinline__ void stamp_end(unsigned long long *slot)
{
    if (!slot) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    atomicMax(slot, t);
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// Launch with programmatic stream serialization allowed: the grid may be scheduled while its predecessor in the
// stream still runs, so the kernel must call pdl_wait() before it touches anything the predecessor writes (and
// before it exits).  WGB_NO_PDL=1 in the environment turns the attribute off (plain stream order).
bool pdl_enabled();
template <typename... P, typename... A>
inline cudaError_t launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}
#endif

}  // namespace wgb
