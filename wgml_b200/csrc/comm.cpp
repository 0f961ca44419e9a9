// Tensor-parallel communicator: a thin wrapper over NCCL, resolved at run time so that the
// single-GPU library has no link-time dependency on it.  One process per GPU; every rank of the
// group calls wgb_comm_create with the same 128-byte id (made by rank 0 with wgb_comm_unique_id and
// handed to the others by the host program, e.g. through torch.distributed or MPI).
#include "kernels.h"

#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

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
