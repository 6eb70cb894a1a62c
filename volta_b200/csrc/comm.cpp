// NCCL plumbing for sharded optimizers: one process per GPU, parameters exchanged over
// NVLink 5 / NVSwitch.  libnccl is resolved at run time (dlopen) so that a single-GPU
// user needs no NCCL at all and a host that already loaded its own libnccl.so.2 (for
// example through torch) shares that copy instead of getting a second one.
#include <dlfcn.h>
#include <string.h>

#include "engine.h"

namespace vb {

namespace {

// The handful of NCCL entry points used, declared with the public NCCL 2.x signatures.
typedef struct ncclComm *ncclComm_t;
typedef struct {
    char internal[128];
} ncclUniqueId;
typedef int ncclResult_t;   // ncclSuccess == 0
typedef int ncclDataType_t; // ncclFloat32 == 7
constexpr ncclDataType_t kNcclFloat = 7;
constexpr ncclDataType_t kNcclUint8 = 1;

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;  // optional: teardown after a failed collective
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, int /*ncclRedOp_t*/, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int *) = nullptr;
};

NcclApi g_api;
bool g_api_tried = false;

int load_api()
{
    if (g_api.handle) return VB_OK;
    if (g_api_tried) return fail(VB_ERR_NCCL, "libnccl.so.2 could not be loaded");
    g_api_tried = true;
    const char *names[] = {getenv("VB_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
    void *h = nullptr;
    for (const char *n : names) {
        if (!n || !*n) continue;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return fail(VB_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
    g_api.handle = h;
#define VB_SYM(field, name)                                                          \
    *(void **)(&g_api.field) = dlsym(h, name);                                       \
    if (!g_api.field) {                                                              \
        g_api.handle = nullptr;                                                      \
        return fail(VB_ERR_NCCL, "libnccl has no symbol %s", name);                  \
    }
    VB_SYM(GetUniqueId, "ncclGetUniqueId")
    VB_SYM(CommInitRank, "ncclCommInitRank")
    VB_SYM(CommDestroy, "ncclCommDestroy")
    VB_SYM(AllGather, "ncclAllGather")
    VB_SYM(Broadcast, "ncclBroadcast")
    VB_SYM(AllReduce, "ncclAllReduce")
    VB_SYM(GroupStart, "ncclGroupStart")
    VB_SYM(GroupEnd, "ncclGroupEnd")
    VB_SYM(GetErrorString, "ncclGetErrorString")
    VB_SYM(GetVersion, "ncclGetVersion")
#undef VB_SYM
    *(void **)(&g_api.CommAbort) = dlsym(h, "ncclCommAbort");
    return VB_OK;
}

#define VB_NCCL(expr)                                                                     \
    do {                                                                                  \
        ncclResult_t _r = (expr);                                                         \
        if (_r != 0)                                                                      \
            return fail(VB_ERR_NCCL, "%s failed: %s (%d)", #expr, g_api.GetErrorString(_r), _r); \
    } while (0)
// The same for collectives on an engine's communicator: remembers the failure for teardown.
#define VB_NCCL_ON(eng, expr)                                                             \
    do {                                                                                  \
        ncclResult_t _r = (expr);                                                         \
        if (_r != 0) {                                                                    \
            (eng)->comm->failed = true;                                                   \
            return fail(VB_ERR_NCCL, "%s failed: %s (%d)", #expr, g_api.GetErrorString(_r), _r); \
        }                                                                                 \
    } while (0)

}  // namespace

struct Comm {
    ncclComm_t comm = nullptr;
    float *d_token = nullptr;  // one float: the payload of the barrier all-reduce
    bool failed = false;       // a collective returned an error: tear down with ncclCommAbort
};

int comm_unique_id(void *id128)
{
    VB_TRY(load_api());
    ncclUniqueId id;
    VB_NCCL(g_api.GetUniqueId(&id));
    memcpy(id128, &id, sizeof(id));
    return VB_OK;
}

int comm_init(vb_engine *eng, const void *id128, int rank, int world)
{
    VB_TRY(load_api());
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    Comm *c = new Comm();
    ncclResult_t r = g_api.CommInitRank(&c->comm, world, id, rank);
    if (r != 0) {
        delete c;
        return fail(VB_ERR_NCCL, "ncclCommInitRank failed: %s (%d)", g_api.GetErrorString(r), r);
    }
    eng->comm = c;
    eng->rank = rank;
    eng->world = world;
    return VB_OK;
}

void comm_destroy(vb_engine *eng)
{
    if (eng->comm) {
        // ncclCommDestroy waits for outstanding collectives; after a failed one they may never
        // finish (a peer is gone), so the communicator is aborted instead
        if (eng->comm->comm && eng->comm->failed && g_api.CommAbort) g_api.CommAbort(eng->comm->comm);
        else if (eng->comm->comm && g_api.CommDestroy) g_api.CommDestroy(eng->comm->comm);
        if (eng->comm->d_token) cudaFree(eng->comm->d_token);
        delete eng->comm;
        eng->comm = nullptr;
    }
}

// In-place all-gather: rank r's slice is base[r*count, (r+1)*count).
int comm_all_gather_inplace(vb_engine *eng, float *base, int64_t count)
{
    if (!eng->comm) return fail(VB_ERR_STATE, "engine has no communicator");
    VB_NCCL_ON(eng, g_api.AllGather(base + (int64_t)eng->rank * count, base, (size_t)count, kNcclFloat,
                                    eng->comm->comm, eng->stream));
    return VB_OK;
}

// The same for a buffer addressed in bytes (the bf16 copies of the parameters).
int comm_all_gather_inplace_bytes(vb_engine *eng, void *base, int64_t bytes)
{
    if (!eng->comm) return fail(VB_ERR_STATE, "engine has no communicator");
    VB_NCCL_ON(eng, g_api.AllGather((char *)base + (int64_t)eng->rank * bytes, base, (size_t)bytes, kNcclUint8,
                                    eng->comm->comm, eng->stream));
    return VB_OK;
}

// A one-float all-reduce used as a stream-ordered barrier across the ranks: it completes on
// a rank only after every rank's stream has reached it, i.e. after all work the other ranks
// enqueued before it (their update kernels and the peer stores in them) has finished.  The
// default fence of a fused step is the flag barrier of exchange_fence.cu; this one is selected by
// VB_EXCHANGE_FENCE=nccl for comparison (its wait has no bound).
int comm_barrier(vb_engine *eng)
{
    if (!eng->comm) return fail(VB_ERR_STATE, "engine has no communicator");
    if (!eng->comm->d_token) {
        VB_CUDA(cudaMalloc(&eng->comm->d_token, sizeof(float)));
        VB_CUDA(cudaMemsetAsync(eng->comm->d_token, 0, sizeof(float), eng->stream));
    }
    VB_NCCL_ON(eng, g_api.AllReduce(eng->comm->d_token, eng->comm->d_token, 1, kNcclFloat, 0 /*ncclSum*/,
                                    eng->comm->comm, eng->stream));
    return VB_OK;
}

// One grouped launch of broadcasts (Muon: every matrix from the rank that owns it).
int comm_group_broadcast(vb_engine *eng, const BcastItem *items, int64_t n_items)
{
    if (!eng->comm) return fail(VB_ERR_STATE, "engine has no communicator");
    if (n_items == 0) return VB_OK;
    VB_NCCL(g_api.GroupStart());
    for (int64_t i = 0; i < n_items; ++i) {
        ncclResult_t r = g_api.Broadcast(items[i].ptr, items[i].ptr, (size_t)items[i].count,
                                         items[i].elem_bytes == 4 ? kNcclFloat : kNcclUint8, items[i].root,
                                         eng->comm->comm, eng->stream);
        if (r != 0) {
            g_api.GroupEnd();
            eng->comm->failed = true;
            return fail(VB_ERR_NCCL, "ncclBroadcast failed: %s (%d)", g_api.GetErrorString(r), r);
        }
    }
    VB_NCCL_ON(eng, g_api.GroupEnd());
    return VB_OK;
}

}  // namespace vb
