// Collectives for the tensor-parallel decoder: a thin layer over NCCL, loaded at run time so the
// library has no link-time dependency on it.  The reference has no multi-GPU code at all (its only
// cross-device move is Tensor.To through a host array, src/NeuralSharp/Tensor.cs:244-253); this is new.
//
// One process per GPU: rank 0 creates an id (ns_comm_unique_id), the host program hands the 128 bytes
// to the other ranks by its own means (torch.distributed, a file, MPI), every rank calls
// ns_comm_init_rank.  Collectives are queued on the device object's stream and can be captured in a
// CUDA graph.  Errors: every NCCL result other than success becomes NS_ERR_COMM with NCCL's text;
// ns_comm_abort tears the communicator down without waiting for peers (use it after a peer failed).
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include "ns_common.cuh"

namespace {

typedef struct ncclComm* ncclComm_t;
struct NcclUniqueId { char internal[128]; };
// values of nccl.h (stable across NCCL 2.x)
enum { NCCL_SUCCESS = 0, NCCL_IN_PROGRESS = 7 };
enum { NCCL_INT32 = 2, NCCL_FLOAT32 = 7, NCCL_BFLOAT16 = 9 };
enum { NCCL_SUM = 0, NCCL_MAX = 2 };

struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GetVersion)(int*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

NcclApi g_nccl;
std::mutex g_nccl_lock;

int load_nccl()
{
    std::lock_guard<std::mutex> guard(g_nccl_lock);
    if (g_nccl.lib) return NS_OK;
    // An NCCL the process has loaded already (for instance the one bundled with PyTorch) is used as is: the
    // dynamic loader keeps one library per soname.  NS_B200_NCCL_LIB names a specific file.
    const char* names[] = {getenv("NS_B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* lib = nullptr;
    for (const char* n : names) {
        if (n == nullptr || n[0] == 0) continue;
        lib = dlopen(n, RTLD_NOW | RTLD_NOLOAD);
        if (!lib) lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
        if (lib) break;
    }
    NS_REQUIRE(lib != nullptr, NS_ERR_COMM, "NCCL is not available: %s", dlerror());
#define NS_SYM(field, name)                                                        \
    *reinterpret_cast<void**>(&g_nccl.field) = dlsym(lib, name);                   \
    NS_REQUIRE(g_nccl.field != nullptr, NS_ERR_COMM, "NCCL symbol %s is missing", name)
    NS_SYM(GetUniqueId, "ncclGetUniqueId");
    NS_SYM(CommInitRank, "ncclCommInitRank");
    NS_SYM(CommDestroy, "ncclCommDestroy");
    NS_SYM(CommAbort, "ncclCommAbort");
    NS_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    NS_SYM(AllReduce, "ncclAllReduce");
    NS_SYM(AllGather, "ncclAllGather");
    NS_SYM(GetVersion, "ncclGetVersion");
    NS_SYM(GetErrorString, "ncclGetErrorString");
#undef NS_SYM
    g_nccl.lib = lib;
    return NS_OK;
}

int nccl_check(int r, const char* call)
{
    if (r == NCCL_SUCCESS) return NS_OK;
    return ns_fail(NS_ERR_COMM, "%s failed: %s (%d)", call, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?", r);
}

int nccl_type(int dtype, int* out)
{
    switch (dtype) {
        case NS_F32: *out = NCCL_FLOAT32; return NS_OK;
        case NS_BF16: *out = NCCL_BFLOAT16; return NS_OK;
        case NS_I32: *out = NCCL_INT32; return NS_OK;
        default: return ns_fail(NS_ERR_ARGUMENT, "collectives support NS_F32, NS_BF16 and NS_I32 (got %d)", dtype);
    }
}

}  // namespace

struct NsComm {
    ncclComm_t comm = nullptr;
    int rank = 0, size = 1;
};

extern "C" int ns_comm_unique_id(void* id128)
{
    NS_REQUIRE(id128 != nullptr, NS_ERR_ARGUMENT, "ns_comm_unique_id: buffer is null");
    int rc = load_nccl();
    if (rc != NS_OK) return rc;
    NcclUniqueId id;
    rc = nccl_check(g_nccl.GetUniqueId(&id), "ncclGetUniqueId");
    if (rc != NS_OK) return rc;
    memcpy(id128, &id, sizeof(id));
    return NS_OK;
}

extern "C" int ns_comm_init_rank(ns_device_t h, const void* id128, int rank, int size, ns_comm_t* out)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NS_REQUIRE(id128 && out, NS_ERR_ARGUMENT, "ns_comm_init_rank: null argument");
    NS_REQUIRE(size >= 1 && rank >= 0 && rank < size, NS_ERR_ARGUMENT, "ns_comm_init_rank: bad rank %d of %d", rank, size);
    rc = load_nccl();
    if (rc != NS_OK) return rc;
    NcclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    NsComm* c = new NsComm();
    c->rank = rank; c->size = size;
    rc = nccl_check(g_nccl.CommInitRank(&c->comm, size, id, rank), "ncclCommInitRank");
    if (rc != NS_OK) { delete c; return rc; }
    *out = reinterpret_cast<ns_comm_t>(c);
    return NS_OK;
}

extern "C" int ns_comm_info(ns_comm_t ch, int* rank, int* size, int* nccl_version)
{
    NsComm* c = reinterpret_cast<NsComm*>(ch);
    NS_REQUIRE(c != nullptr, NS_ERR_ARGUMENT, "ns_comm_info: communicator is null");
    if (rank) *rank = c->rank;
    if (size) *size = c->size;
    if (nccl_version && g_nccl.GetVersion) g_nccl.GetVersion(nccl_version);
    return NS_OK;
}

extern "C" int ns_allreduce(ns_device_t h, ns_comm_t ch, uint64_t buf, int64_t count, int dtype)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NsComm* c = reinterpret_cast<NsComm*>(ch);
    NS_REQUIRE(c && buf && count >= 0, NS_ERR_ARGUMENT, "ns_allreduce: bad argument");
    int t;
    rc = nccl_type(dtype, &t);
    if (rc != NS_OK) return rc;
    if (count == 0 || c->size == 1) return NS_OK;
    void* p = reinterpret_cast<void*>(buf);
    return nccl_check(g_nccl.AllReduce(p, p, (size_t)count, t, NCCL_SUM, c->comm, d->stream), "ncclAllReduce");
}

extern "C" int ns_allgather(ns_device_t h, ns_comm_t ch, uint64_t src, uint64_t dst, int64_t count, int dtype)
{
    NsDevice* d = ns_dev(h);
    int rc = ns_device_make_current(d);
    if (rc != NS_OK) return rc;
    NsComm* c = reinterpret_cast<NsComm*>(ch);
    NS_REQUIRE(c && src && dst && count >= 0, NS_ERR_ARGUMENT, "ns_allgather: bad argument");
    int t;
    rc = nccl_type(dtype, &t);
    if (rc != NS_OK) return rc;
    if (count == 0) return NS_OK;
    return nccl_check(g_nccl.AllGather(reinterpret_cast<const void*>(src), reinterpret_cast<void*>(dst), (size_t)count, t, c->comm, d->stream),
                      "ncclAllGather");
}

extern "C" int ns_comm_async_error(ns_comm_t ch, int* nccl_result)
{
    NsComm* c = reinterpret_cast<NsComm*>(ch);
    NS_REQUIRE(c && nccl_result, NS_ERR_ARGUMENT, "ns_comm_async_error: null argument");
    return nccl_check(g_nccl.CommGetAsyncError(c->comm, nccl_result), "ncclCommGetAsyncError");
}

extern "C" int ns_comm_abort(ns_comm_t ch)
{
    NsComm* c = reinterpret_cast<NsComm*>(ch);
    if (!c) return NS_OK;
    int rc = c->comm ? nccl_check(g_nccl.CommAbort(c->comm), "ncclCommAbort") : NS_OK;
    delete c;
    return rc;
}

extern "C" int ns_comm_destroy(ns_comm_t ch)
{
    NsComm* c = reinterpret_cast<NsComm*>(ch);
    if (!c) return NS_OK;
    int rc = c->comm ? nccl_check(g_nccl.CommDestroy(c->comm), "ncclCommDestroy") : NS_OK;
    delete c;
    return rc;
}
