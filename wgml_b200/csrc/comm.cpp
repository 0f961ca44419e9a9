// Tensor-parallel communicator: a thin wrapper over NCCL, resolved at run time so that the
// single-GPU library has no link-time dependency on it.  One process per GPU; every rank of the
// group calls wgb_comm_create with the same 128-byte id (made by rank 0 with wgb_comm_unique_id and
// handed to the others by the host program, e.g. through torch.distributed or MPI).
#include "kernels.h"

#include <dlfcn.h>
#include <nccl.h>

#include <mutex>
#include <vector>

namespace {

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    const char *(*GetLastError)(ncclComm_t) = nullptr;
};

NcclApi g_nccl;
std::once_flag g_once;
std::string g_load_error;

void load_nccl()
{
    // A process that already uses NCCL (PyTorch does) gets that copy back for the same soname.
    const char *names[] = { "libnccl.so.2", "libnccl.so" };
    for (const char *n : names) {
        g_nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.lib) break;
    }
    if (!g_nccl.lib) {
        g_load_error = std::string("cannot load libnccl.so.2: ") + dlerror();
        return;
    }
    bool ok = true;
    auto sym = [&](const char *name) {
        void *p = dlsym(g_nccl.lib, name);
        if (!p) {
            ok = false;
            g_load_error = std::string("libnccl lacks ") + name;
        }
        return p;
    };
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))sym("ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))sym("ncclCommInitRank");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))sym("ncclCommDestroy");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))sym("ncclAllReduce");
    g_nccl.AllGather = (decltype(g_nccl.AllGather))sym("ncclAllGather");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))sym("ncclGetErrorString");
    g_nccl.GetLastError = (decltype(g_nccl.GetLastError))dlsym(g_nccl.lib, "ncclGetLastError");   // optional
    if (!ok) {
        dlclose(g_nccl.lib);
        g_nccl.lib = nullptr;
    }
}

int need_nccl()
{
    std::call_once(g_once, load_nccl);
    if (!g_nccl.lib) return wgb::fail(WGB_ERR_UNSUPPORTED, "%s", g_load_error.c_str());
    return WGB_OK;
}

int nccl_fail(ncclResult_t r, const char *what, ncclComm_t comm)
{
    const char *detail = (g_nccl.GetLastError && comm) ? g_nccl.GetLastError(comm) : "";
    return wgb::fail(WGB_ERR_CUDA, "%s: %s %s", what, g_nccl.GetErrorString(r), detail ? detail : "");
}

}  // namespace

struct wgb_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, size = 1;
    struct Shared {
        void *local;
        void *peer[WGB_COMM_MAX_PEERS];
    };
    std::vector<Shared> shared;   // buffers opened on the peers (wgb_comm_shared_alloc)
};

static_assert(sizeof(ncclUniqueId) == WGB_COMM_ID_BYTES, "id size in the public header");

WGB_EXPORT int wgb_comm_unique_id(void *id_out)
{
    WGB_REQUIRE(id_out, "null argument");
    int rc = need_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId", nullptr);
    memcpy(id_out, &id, sizeof(id));
    return WGB_OK;
}

WGB_EXPORT int wgb_comm_create(const void *id, int rank, int size, wgb_comm **out)
{
    WGB_REQUIRE(id && out, "null argument");
    WGB_REQUIRE(size >= 1 && rank >= 0 && rank < size, "bad rank %d of %d", rank, size);
    int rc = need_nccl();
    if (rc) return rc;
    wgb_comm *c = new (std::nothrow) wgb_comm();
    if (!c) return wgb::fail(WGB_ERR_INVALID, "out of host memory");
    ncclUniqueId nid;
    memcpy(&nid, id, sizeof(nid));
    ncclResult_t r = g_nccl.CommInitRank(&c->comm, size, nid, rank);
    if (r != ncclSuccess) {
        delete c;
        return nccl_fail(r, "ncclCommInitRank", nullptr);
    }
    c->rank = rank;
    c->size = size;
    *out = c;
    return WGB_OK;
}

WGB_EXPORT int wgb_comm_destroy(wgb_comm *c)
{
    if (!c) return WGB_OK;
    for (auto &sh : c->shared) {
        for (int p = 0; p < c->size; p++)
            if (p != c->rank && sh.peer[p]) cudaIpcCloseMemHandle(sh.peer[p]);
        if (sh.local) cudaFree(sh.local);
    }
    if (c->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
    delete c;
    return WGB_OK;
}

WGB_EXPORT int wgb_comm_rank(const wgb_comm *c) { return c ? c->rank : 0; }
WGB_EXPORT int wgb_comm_size(const wgb_comm *c) { return c ? c->size : 1; }

WGB_EXPORT int wgb_comm_all_reduce_sum(wgb_comm *c, const float *d_send, float *d_recv, size_t n, void *stream)
{
    WGB_REQUIRE(c && d_send && d_recv, "null argument");
    ncclResult_t r = g_nccl.AllReduce(d_send, d_recv, n, ncclFloat32, ncclSum, c->comm, wgb::as_stream(stream));
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce", c->comm);
    return WGB_OK;
}

WGB_EXPORT int wgb_comm_all_gather(wgb_comm *c, const float *d_send, float *d_recv, size_t n_per_rank, void *stream)
{
    WGB_REQUIRE(c && d_send && d_recv, "null argument");
    ncclResult_t r = g_nccl.AllGather(d_send, d_recv, n_per_rank, ncclFloat32, c->comm, wgb::as_stream(stream));
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllGather", c->comm);
    return WGB_OK;
}

// A zero-filled device buffer of `bytes` on every rank, each mapped into every other rank's address space
// (CUDA IPC; the ranks are separate processes on GPUs of one node with peer access over NVLink).
// peers_out[p] is rank p's buffer as seen from this rank; peers_out[rank] is the local one.  Collective:
// every rank calls it with the same size.  The buffers belong to the communicator.
WGB_EXPORT int wgb_comm_shared_alloc(wgb_comm *c, size_t bytes, void **peers_out)
{
    WGB_REQUIRE(c && peers_out && bytes > 0, "null argument");
    WGB_REQUIRE(c->size <= WGB_COMM_MAX_PEERS, "shared buffers support at most %d ranks", WGB_COMM_MAX_PEERS);
    wgb_comm::Shared sh = {};
    WGB_CUDA(cudaMalloc(&sh.local, bytes));
    cudaError_t e = cudaMemset(sh.local, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t mine;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&mine, sh.local);
    unsigned char *d_send = nullptr, *d_recv = nullptr;
    std::vector<cudaIpcMemHandle_t> all((size_t)c->size);
    if (e == cudaSuccess) e = cudaMalloc((void **)&d_send, sizeof(mine));
    if (e == cudaSuccess) e = cudaMalloc((void **)&d_recv, sizeof(mine) * (size_t)c->size);
    if (e == cudaSuccess) e = cudaMemcpy(d_send, &mine, sizeof(mine), cudaMemcpyHostToDevice);
    int rc = WGB_OK;
    if (e == cudaSuccess) {
        // the zero fill above is complete on every rank before any rank learns a handle
        ncclResult_t r = g_nccl.AllGather(d_send, d_recv, sizeof(mine), ncclUint8, c->comm, (cudaStream_t)0);
        if (r != ncclSuccess) rc = nccl_fail(r, "ncclAllGather(ipc handles)", c->comm);
    }
    if (e == cudaSuccess && rc == WGB_OK) e = cudaStreamSynchronize((cudaStream_t)0);
    if (e == cudaSuccess && rc == WGB_OK) e = cudaMemcpy(all.data(), d_recv, sizeof(mine) * (size_t)c->size, cudaMemcpyDeviceToHost);
    if (d_send) cudaFree(d_send);
    if (d_recv) cudaFree(d_recv);
    for (int p = 0; p < c->size && e == cudaSuccess && rc == WGB_OK; p++) {
        if (p == c->rank) sh.peer[p] = sh.local;
        else e = cudaIpcOpenMemHandle(&sh.peer[p], all[(size_t)p], cudaIpcMemLazyEnablePeerAccess);
    }
    if (e != cudaSuccess || rc != WGB_OK) {
        for (int p = 0; p < c->size; p++)
            if (p != c->rank && sh.peer[p]) cudaIpcCloseMemHandle(sh.peer[p]);
        cudaFree(sh.local);
        return rc != WGB_OK ? rc : wgb::cuda_fail(e, "shared buffer set-up (CUDA IPC)");
    }
    c->shared.push_back(sh);
    for (int p = 0; p < c->size; p++) peers_out[p] = sh.peer[p];
    return WGB_OK;
}
