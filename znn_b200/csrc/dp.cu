// Data-parallel gradient exchange: one NCCL communicator per device (one process per GPU, or one process that drives
// several GPUs), all-reduces issued on a dedicated communication stream that is event-ordered after the compute
// stream, so that reductions of finished gradient buckets overlap the rest of the backward pass.  The reference is
// single-process; this is the one exchange step its training loop needs when the batch is sharded (parameter-gradient
// sum, scaled by 1/world in znn_sgd_step).
//
// Failure handling: with a timeout set (znn_dp_set_timeout_ms) the communicator is created non-blocking; every NCCL
// call and znn_dp_wait poll ncclCommGetAsyncError against a host deadline, and on an error or an expired deadline the
// communicator is aborted (ncclCommAbort) so that no rank stays blocked on a peer that is gone.
//
// NCCL is loaded with dlopen so that the library works without it on one GPU.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <chrono>
#include <thread>

#include "common.cuh"

namespace znn {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
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
    ZNN_SYM(CommInitRankConfig, "ncclCommInitRankConfig");
    ZNN_SYM(CommInitAll, "ncclCommInitAll");
    ZNN_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    ZNN_SYM(GroupStart, "ncclGroupStart");
    ZNN_SYM(GroupEnd, "ncclGroupEnd");
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

constexpr int kDpMaxDev = 16;

struct DpState {
    bool ready = false;
    int world = 1, rank = 0;
    ncclComm_t comm = nullptr;
    bool nonblocking = false;
    bool aborted = false;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_ready = nullptr;  // compute -> comm
    cudaEvent_t ev_done = nullptr;   // comm -> compute
    bool outstanding = false;
};

// one state per device; the calling thread's current device selects it
static DpState g_dp[kDpMaxDev];
static long long g_timeout_ms = 0;   // 0 = blocking communicator, no host deadline

static DpState* dp_cur()
{
    int d = -1;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kDpMaxDev) return nullptr;
    return &g_dp[d];
}

static int dp_abort(DpState& s, const char* why)
{
    if (s.comm && !s.aborted) {
        g_nccl.CommAbort(s.comm);   // frees the communicator; pending operations of this rank end with an error
        s.comm = nullptr;
        s.aborted = true;
    }
    return fail(ZNN_ERR_NCCL, "communicator aborted: %s", why);
}

// After a call on a non-blocking communicator: poll until NCCL has taken the operation (or failed), at most until the
// host deadline.  On a blocking communicator the result is final already.
static int dp_settle(DpState& s, ncclResult_t r, const char* what)
{
    if (r == ncclSuccess) return ZNN_OK;
    if (r != ncclInProgress || !s.nonblocking) return fail(ZNN_ERR_NCCL, "%s failed: %s", what, g_nccl.GetErrorString(r));
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        ncclResult_t st = ncclSuccess;
        const ncclResult_t q = g_nccl.CommGetAsyncError(s.comm, &st);
        if (q != ncclSuccess) return dp_abort(s, "ncclCommGetAsyncError failed");
        if (st == ncclSuccess) return ZNN_OK;
        if (st != ncclInProgress) {
            char msg[160];
            snprintf(msg, sizeof(msg), "%s: %s", what, g_nccl.GetErrorString(st));
            return dp_abort(s, msg);
        }
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (g_timeout_ms > 0 && ms > g_timeout_ms) {
            char msg[160];
            snprintf(msg, sizeof(msg), "%s still in progress after %lld ms", what, (long long)ms);
            return dp_abort(s, msg);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

static int dp_make_streams(DpState& s)
{
    ZNN_CUDA_OK(cudaStreamCreateWithFlags(&s.comm_stream, cudaStreamNonBlocking));
    ZNN_CUDA_OK(cudaEventCreateWithFlags(&s.ev_ready, cudaEventDisableTiming));
    ZNN_CUDA_OK(cudaEventCreateWithFlags(&s.ev_done, cudaEventDisableTiming));
    return ZNN_OK;
}

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
    const ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return fail(ZNN_ERR_NCCL, "ncclGetUniqueId failed: %s", g_nccl.GetErrorString(r));
    memcpy(out128, &id, sizeof(id));
    return ZNN_OK;
}

int znn_dp_set_timeout_ms(long long ms)
{
    ZNN_REQUIRE(ms >= 0, "timeout must be >= 0 (0 = blocking communicator, no deadline)");
    g_timeout_ms = ms;
    return ZNN_OK;
}

int znn_dp_init(int world, int rank, const char* id128)
{
    ZNN_REQUIRE(world >= 1 && rank >= 0 && rank < world, "bad world/rank %d/%d", world, rank);
    if (!stream()) return fail(ZNN_ERR_CUDA, "call znn_init before znn_dp_init");
    DpState* sp = dp_cur();
    ZNN_REQUIRE(sp, "no current device");
    DpState& s = *sp;
    ZNN_REQUIRE(!s.ready, "znn_dp_init called twice on this device");
    s.world = world;
    s.rank = rank;
    if (world > 1) {
        ZNN_REQUIRE(id128, "id128 is NULL");
        int rc = load_nccl();
        if (rc) return rc;
        ncclUniqueId id;
        memcpy(&id, id128, sizeof(id));
        if (g_timeout_ms > 0) {
            ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
            cfg.blocking = 0;
            s.nonblocking = true;
            const ncclResult_t r = g_nccl.CommInitRankConfig(&s.comm, world, id, rank, &cfg);
            if ((rc = dp_settle(s, r, "ncclCommInitRankConfig"))) return rc;
        } else {
            const ncclResult_t r = g_nccl.CommInitRank(&s.comm, world, id, rank);
            if (r != ncclSuccess) return fail(ZNN_ERR_NCCL, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(r));
        }
        if ((rc = dp_make_streams(s))) return rc;
    }
    s.ready = true;
    return ZNN_OK;
}

int znn_dp_init_all(int ndev)
{
    ZNN_REQUIRE(ndev >= 1 && ndev <= kDpMaxDev, "ndev must be 1..%d", kDpMaxDev);
    int have = 0;
    ZNN_CUDA_OK(cudaGetDeviceCount(&have));
    ZNN_REQUIRE(ndev <= have, "ndev %d exceeds the %d visible devices", ndev, have);
    for (int d = 0; d < ndev; d++) ZNN_REQUIRE(!g_dp[d].ready, "device %d already has a communicator", d);
    int prev = 0;
    ZNN_CUDA_OK(cudaGetDevice(&prev));
    int rc = ZNN_OK;
    ncclComm_t comms[kDpMaxDev];
    if (ndev > 1) {
        if ((rc = load_nccl())) return rc;
        int devs[kDpMaxDev];
        for (int d = 0; d < ndev; d++) devs[d] = d;
        const ncclResult_t r = g_nccl.CommInitAll(comms, ndev, devs);
        if (r != ncclSuccess) return fail(ZNN_ERR_NCCL, "ncclCommInitAll failed: %s", g_nccl.GetErrorString(r));
    }
    for (int d = 0; d < ndev && rc == ZNN_OK; d++) {
        rc = znn_init(d);
        if (rc) break;
        DpState& s = g_dp[d];
        s.world = ndev;
        s.rank = d;
        if (ndev > 1) {
            s.comm = comms[d];
            rc = dp_make_streams(s);
        }
        s.ready = (rc == ZNN_OK);
    }
    cudaSetDevice(prev);
    return rc;
}

int znn_dp_group_begin(void)
{
    int rc = load_nccl();
    if (rc) return rc;
    const ncclResult_t r = g_nccl.GroupStart();
    if (r != ncclSuccess) return fail(ZNN_ERR_NCCL, "ncclGroupStart failed: %s", g_nccl.GetErrorString(r));
    return ZNN_OK;
}

int znn_dp_group_end(void)
{
    int rc = load_nccl();
    if (rc) return rc;
    const ncclResult_t r = g_nccl.GroupEnd();
    if (r != ncclSuccess && r != ncclInProgress) return fail(ZNN_ERR_NCCL, "ncclGroupEnd failed: %s", g_nccl.GetErrorString(r));
    return ZNN_OK;
}

int znn_dp_world(int* world, int* rank)
{
    DpState* s = dp_cur();
    const bool ok = s && s->ready;
    if (world) *world = ok ? s->world : 1;
    if (rank) *rank = ok ? s->rank : 0;
    return ZNN_OK;
}

int znn_dp_allreduce_async(float* buf, size_t count)
{
    DpState* sp = dp_cur();
    if (!sp || !sp->ready || sp->world == 1 || count == 0) return ZNN_OK;
    DpState& s = *sp;
    ZNN_REQUIRE(buf, "buf is NULL");
    if (s.aborted) return fail(ZNN_ERR_NCCL, "the communicator was aborted; call znn_dp_finalize and initialise again");
    // everything queued on the compute stream so far (the writers of this bucket) comes first
    ZNN_CUDA_OK(cudaEventRecord(s.ev_ready, stream()));
    ZNN_CUDA_OK(cudaStreamWaitEvent(s.comm_stream, s.ev_ready, 0));
    const int rc = dp_settle(s, g_nccl.AllReduce(buf, buf, count, ncclFloat, ncclSum, s.comm, s.comm_stream), "ncclAllReduce");
    if (rc) return rc;
    s.outstanding = true;
    return ZNN_OK;
}

int znn_dp_join(void)
{
    DpState* sp = dp_cur();
    if (!sp || !sp->ready || sp->world == 1 || !sp->outstanding) return ZNN_OK;
    DpState& s = *sp;
    if (s.aborted) return fail(ZNN_ERR_NCCL, "the communicator was aborted");
    ZNN_CUDA_OK(cudaEventRecord(s.ev_done, s.comm_stream));
    ZNN_CUDA_OK(cudaStreamWaitEvent(stream(), s.ev_done, 0));
    s.outstanding = false;
    return ZNN_OK;
}

int znn_dp_wait(long long timeout_ms)
{
    DpState* sp = dp_cur();
    if (!sp || !sp->ready || sp->world == 1) return ZNN_OK;
    DpState& s = *sp;
    if (s.aborted) return fail(ZNN_ERR_NCCL, "the communicator was aborted");
    ZNN_CUDA_OK(cudaEventRecord(s.ev_done, s.comm_stream));
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t q = cudaEventQuery(s.ev_done);
        if (q == cudaSuccess) return ZNN_OK;
        if (q != cudaErrorNotReady) {
            cudaGetLastError();
            return dp_abort(s, "the communication stream reported a CUDA error");
        }
        ncclResult_t st = ncclSuccess;
        if (g_nccl.CommGetAsyncError(s.comm, &st) != ncclSuccess || (st != ncclSuccess && st != ncclInProgress))
            return dp_abort(s, "NCCL reported an asynchronous error");
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (timeout_ms > 0 && ms > timeout_ms) return dp_abort(s, "reductions still pending at the host deadline");
        std::this_thread::sleep_for(std::chrono::microseconds(100));
    }
}

int znn_dp_abort(void)
{
    DpState* sp = dp_cur();
    if (!sp || !sp->ready || sp->world == 1 || sp->aborted) return ZNN_OK;
    if (sp->comm) {
        g_nccl.CommAbort(sp->comm);
        sp->comm = nullptr;
    }
    sp->aborted = true;
    sp->outstanding = false;
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
    DpState* sp = dp_cur();
    if (!sp || !sp->ready || sp->world == 1 || count == 0) return ZNN_OK;
    DpState& s = *sp;
    if (s.aborted) return fail(ZNN_ERR_NCCL, "the communicator was aborted");
    ZNN_CUDA_OK(cudaEventRecord(s.ev_ready, stream()));
    ZNN_CUDA_OK(cudaStreamWaitEvent(s.comm_stream, s.ev_ready, 0));
    const int rc = dp_settle(s, g_nccl.Broadcast(buf, buf, count, ncclFloat, root, s.comm, s.comm_stream), "ncclBroadcast");
    if (rc) return rc;
    s.outstanding = true;
    return znn_dp_join();
}

int znn_dp_finalize(void)
{
    DpState* sp = dp_cur();
    if (!sp || !sp->ready) return ZNN_OK;
    DpState& s = *sp;
    if (s.world > 1) {
        if (s.comm_stream && !s.aborted) cudaStreamSynchronize(s.comm_stream);
        if (s.comm) g_nccl.CommDestroy(s.comm);
        if (s.ev_ready) cudaEventDestroy(s.ev_ready);
        if (s.ev_done) cudaEventDestroy(s.ev_done);
        if (s.comm_stream) cudaStreamDestroy(s.comm_stream);
    }
    s = DpState();
    return ZNN_OK;
}

}  // extern "C"
