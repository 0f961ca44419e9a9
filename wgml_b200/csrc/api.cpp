// Status handling and the device-memory helpers of the C ABI.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstring>

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

int sm_count()
{
    static int cached = 0;
    if (cached > 0) return cached;
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return 148;  // B200; only reached when no device answers, and then every launch fails anyway
    }
    cached = n;
    return n;
}

}  // namespace wgb

using namespace wgb;

WGB_EXPORT const char *wgb_last_error(void) { return g_error; }
WGB_EXPORT const char *wgb_version(void) { return "wgml_b200 0.1 (sm_100a)"; }

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
