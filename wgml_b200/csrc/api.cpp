// Status handling and the device-memory helpers of the C ABI.
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

namespace wgb {

static thread_local char g_error[512] = "";

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char *what)
{
    snprintf(g_error, sizeof(g_error), "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    // Clear the sticky "last error" of non-fatal failures so that later launches report their own.
    cudaGetLastError();
    return WGB_ERR_CUDA;
}

static DeviceState *g_devices[MAX_DEVICES] = {};
static std::mutex g_devices_mutex;
static std::atomic<unsigned> g_peer_wait_ms{2000};

int current_device()
{
    int dev = -1;
    const cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { cuda_fail(e, "cudaGetDevice"); return -1; }
    if (dev < 0 || dev >= MAX_DEVICES) { fail(WGB_ERR_UNSUPPORTED, "device ordinal %d outside 0..%d", dev, MAX_DEVICES - 1); return -1; }
    return dev;
}

DeviceState *device_state()
{
    const int dev = current_device();
    if (dev < 0) return nullptr;
    std::lock_guard<std::mutex> lock(g_devices_mutex);
    if (!g_devices[dev]) {
        int n = 0;
        const cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || n <= 0) { cuda_fail(e, "cudaDeviceGetAttribute(multiprocessor count)"); return nullptr; }
        DeviceState *d = new (std::nothrow) DeviceState();
        if (!d) { fail(WGB_ERR_INVALID, "out of host memory"); return nullptr; }
        d->ordinal = dev;
        d->sms = n;
        g_devices[dev] = d;
    }
    return g_devices[dev];
}

int sm_count()
{
    const DeviceState *d = device_state();
    return d ? d->sms : 148;  // B200; the fallback is only reached when no device answers, and then every launch fails anyway
}

WaitLimits wait_limits()
{
    const unsigned long long peer = (unsigned long long)g_peer_wait_ms.load() * 1000000ull;
    return { peer, peer + 2000000000ull };
}

}  // namespace wgb

using namespace wgb;

WGB_EXPORT const char *wgb_last_error(void) { return g_error; }
WGB_EXPORT const char *wgb_version(void) { return "wgml_b200 0.2 (sm_100a)"; }

WGB_EXPORT int wgb_set_wait_limit_ms(unsigned ms)
{
    WGB_REQUIRE(ms >= 1 && ms <= 600000u, "wait limit of %u ms outside 1 ms .. 10 min", ms);
    g_peer_wait_ms.store(ms);
    return WGB_OK;
}

WGB_EXPORT unsigned wgb_get_wait_limit_ms(void) { return g_peer_wait_ms.load(); }

WGB_EXPORT int wgb_malloc(void **d_ptr, size_t bytes)
{
    WGB_REQUIRE(d_ptr, "null argument");
    *d_ptr = nullptr;
    if (bytes == 0) return WGB_OK;
    WGB_CUDA(cudaMalloc(d_ptr, bytes));
    return WGB_OK;
}

WGB_EXPORT int wgb_free(void *d_ptr)
{
    if (d_ptr) WGB_CUDA(cudaFree(d_ptr));
    return WGB_OK;
}

WGB_EXPORT int wgb_memcpy_h2d(void *d_dst, const void *h_src, size_t bytes, void *stream)
{
    if (bytes == 0) return WGB_OK;
    WGB_REQUIRE(d_dst && h_src, "null argument");
    WGB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return WGB_OK;
}

WGB_EXPORT int wgb_memcpy_d2h(void *h_dst, const void *d_src, size_t bytes, void *stream)
{
    if (bytes == 0) return WGB_OK;
    WGB_REQUIRE(h_dst && d_src, "null argument");
    WGB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return WGB_OK;
}

WGB_EXPORT int wgb_memset(void *d_dst, int value, size_t bytes, void *stream)
{
    if (bytes == 0) return WGB_OK;
    WGB_REQUIRE(d_dst, "null argument");
    WGB_CUDA(cudaMemsetAsync(d_dst, value, bytes, as_stream(stream)));
    return WGB_OK;
}

WGB_EXPORT int wgb_stream_synchronize(void *stream)
{
    WGB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return WGB_OK;
}
