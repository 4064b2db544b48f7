// Data-parallel gradient exchange: one NCCL communicator per process (one
// process per GPU), all-reduces issued on a dedicated communication stream that
// is event-ordered after the compute stream, so that reductions of finished
// gradient buckets overlap the rest of the backward pass.  The reference is
// single-process; this is the one exchange step its training loop needs when the
// batch is sharded (parameter-gradient sum, scaled by 1/world in znn_sgd_step).
//
// NCCL is loaded with dlopen so that the library works without it on one GPU.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include "common.cuh"

namespace znn {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
};

static NcclApi g_nccl;

static int load_nccl()
{
    if (g_nccl.handle) return ZNN_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return fail(ZNN_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
#define ZNN_SYM(field, name)                                                         \
    do {                                                                             \
        *(void**)(&g_nccl.field) = dlsym(h, name);                                   \
        if (!g_nccl.field) return fail(ZNN_ERR_NCCL, "symbol %s missing in libnccl", name); \
    } while (0)
    ZNN_SYM(GetUniqueId, "ncclGetUniqueId");
    ZNN_SYM(CommInitRank, "ncclCommInitRank");
    ZNN_SYM(AllReduce, "ncclAllReduce");
    ZNN_SYM(Broadcast, "ncclBroadcast");
    ZNN_SYM(CommDestroy, "ncclCommDestroy");
    ZNN_SYM(CommAbort, "ncclCommAbort");
    ZNN_SYM(GetErrorString, "ncclGetErrorString");
    ZNN_SYM(GetVersion, "ncclGetVersion");
#undef ZNN_SYM
    g_nccl.handle = h;
    return ZNN_OK;
}

#define ZNN_NCCL_OK(expr)                                                                       \
    do {                                                                                        \
        ncclResult_t _r = (expr);                                                               \
        if (_r != ncclSuccess)                                                                  \
            return ::znn::fail(ZNN_ERR_NCCL, "%s failed: %s", #expr, g_nccl.GetErrorString(_r)); \
    } while (0)

struct DpState {
    bool ready = false;
    int world = 1, rank = 0;
    ncclComm_t comm = nullptr;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_ready = nullptr;  // compute -> comm
    cudaEvent_t ev_done = nullptr;   // comm -> compute
    bool outstanding = false;
};

static DpState g_dp;

}  // namespace znn

using namespace znn;

extern "C" {

int znn_dp_unique_id(char* out128)
{
    ZNN_REQUIRE(out128, "out128 is NULL");
    int rc = load_nccl();
    if (rc) return rc;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
    ncclUniqueId id;
    ZNN_NCCL_OK(g_nccl.GetUniqueId(&id));
    memcpy(out128, &id, sizeof(id));
    return ZNN_OK;
}

int znn_dp_init(int world, int rank, const char* id128)
{
    ZNN_REQUIRE(world >= 1 && rank >= 0 && rank < world, "bad world/rank %d/%d", world, rank);
    ZNN_REQUIRE(!g_dp.ready, "znn_dp_init called twice");
    if (!stream()) return fail(ZNN_ERR_CUDA, "call znn_init before znn_dp_init");
    g_dp.world = world;
    g_dp.rank = rank;
    if (world > 1) {
        ZNN_REQUIRE(id128, "id128 is NULL");
        int rc = load_nccl();
        if (rc) return rc;
        ncclUniqueId id;
        memcpy(&id, id128, sizeof(id));
        ZNN_NCCL_OK(g_nccl.CommInitRank(&g_dp.comm, world, id, rank));
        ZNN_CUDA_OK(cudaStreamCreateWithFlags(&g_dp.comm_stream, cudaStreamNonBlocking));
        ZNN_CUDA_OK(cudaEventCreateWithFlags(&g_dp.ev_ready, cudaEventDisableTiming));
        ZNN_CUDA_OK(cudaEventCreateWithFlags(&g_dp.ev_done, cudaEventDisableTiming));
    }
    g_dp.ready = true;
    return ZNN_OK;
}

int znn_dp_world(int* world, int* rank)
{
    if (world) *world = g_dp.ready ? g_dp.world : 1;
    if (rank) *rank = g_dp.ready ? g_dp.rank : 0;
    return ZNN_OK;
}

int znn_dp_allreduce_async(float* buf, size_t count)
{
    if (!g_dp.ready || g_dp.world == 1 || count == 0) return ZNN_OK;
    ZNN_REQUIRE(buf, "buf is NULL");
    // everything queued on the compute stream so far (the writers of this bucket) comes first
    ZNN_CUDA_OK(cudaEventRecord(g_dp.ev_ready, stream()));
    ZNN_CUDA_OK(cudaStreamWaitEvent(g_dp.comm_stream, g_dp.ev_ready, 0));
    ZNN_NCCL_OK(g_nccl.AllReduce(buf, buf, count, ncclFloat, ncclSum, g_dp.comm, g_dp.comm_stream));
    g_dp.outstanding = true;
    return ZNN_OK;
}

int znn_dp_join(void)
{
    if (!g_dp.ready || g_dp.world == 1 || !g_dp.outstanding) return ZNN_OK;
    ZNN_CUDA_OK(cudaEventRecord(g_dp.ev_done, g_dp.comm_stream));
    ZNN_CUDA_OK(cudaStreamWaitEvent(stream(), g_dp.ev_done, 0));
    g_dp.outstanding = false;
    return ZNN_OK;
}

int znn_dp_allreduce(float* buf, size_t count)
{
    int rc = znn_dp_allreduce_async(buf, count);
    if (rc) return rc;
    return znn_dp_join();
}

int znn_dp_broadcast(float* buf, size_t count, int root)
{
    if (!g_dp.ready || g_dp.world == 1 || count == 0) return ZNN_OK;
    ZNN_CUDA_OK(cudaEventRecord(g_dp.ev_ready, stream()));
    ZNN_CUDA_OK(cudaStreamWaitEvent(g_dp.comm_stream, g_dp.ev_ready, 0));
    ZNN_NCCL_OK(g_nccl.Broadcast(buf, buf, count, ncclFloat, root, g_dp.comm, g_dp.comm_stream));
    g_dp.outstanding = true;
    return znn_dp_join();
}

int znn_dp_finalize(void)
{
    if (!g_dp.ready) return ZNN_OK;
    if (g_dp.world > 1) {
        cudaStreamSynchronize(g_dp.comm_stream);
        g_nccl.CommDestroy(g_dp.comm);
        cudaEventDestroy(g_dp.ev_ready);
        cudaEventDestroy(g_dp.ev_done);
        cudaStreamDestroy(g_dp.comm_stream);
    }
    g_dp = DpState();
    return ZNN_OK;
}

}  // extern "C"
