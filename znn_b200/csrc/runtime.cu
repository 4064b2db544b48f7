// Runtime part of the shim: device selection, stream, allocation, copies,
// error text, device status word, GEMM scratch.
#include <stdarg.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace znn {

static thread_local char t_err[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}

constexpr int kMaxDev = 16;

// Scratch blocks of one stream: slot 0 GEMM planes / partials / row-op partials, slot 1 conv im2col, slot 2 device
// copies of host operands.  Work on one stream is ordered, so one set per (device, stream) can be reused call after
// call; two host threads that launch on different streams get different sets and never share scratch.
struct ScratchSet {
    cudaStream_t st = nullptr;
    bool used = false;
    void* ws[3] = {nullptr, nullptr, nullptr};
    size_t ws_bytes[3] = {0, 0, 0};
    unsigned* counters = nullptr;   // kScratchCounters zeroed words for kernels that let their last block finish a reduction
};
constexpr int kMaxScratchSets = 16;

struct DeviceState {
    bool ready = false;
    cudaStream_t own_stream = nullptr;
    int* status = nullptr;  // device int
    ScratchSet sets[kMaxScratchSets];
    unsigned long long ws_generation = 0;   // bumped whenever a scratch block moves (is freed and allocated anew)
    int sms = 0;
};

static DeviceState g_dev[kMaxDev];
static thread_local long long t_launches = 0;

void count_launch() { t_launches++; }
long long launches_and_reset(int reset)
{
    const long long v = t_launches;
    if (reset) t_launches = 0;
    return v;
}
static std::mutex g_mu;
static thread_local cudaStream_t t_user_stream = nullptr;
static thread_local bool t_has_user_stream = false;

static DeviceState* cur(bool create)
{
    int d = -1;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDev) return nullptr;
    DeviceState& s = g_dev[d];
    if (!s.ready && create) {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!s.ready) {
            if (cudaStreamCreateWithFlags(&s.own_stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
            if (cudaMalloc((void**)&s.status, sizeof(int)) != cudaSuccess) return nullptr;
            if (cudaMemset(s.status, 0, sizeof(int)) != cudaSuccess) return nullptr;
            cudaDeviceProp prop;
            if (cudaGetDeviceProperties(&prop, d) != cudaSuccess) return nullptr;
            s.sms = prop.multiProcessorCount;
            s.ready = true;
        }
    }
    return s.ready ? &s : nullptr;
}

cudaStream_t stream()
{
    if (t_has_user_stream) return t_user_stream;
    DeviceState* s = cur(true);
    return s ? s->own_stream : nullptr;
}

int* device_status_word()
{
    DeviceState* s = cur(true);
    return s ? s->status : nullptr;
}

int sm_count()
{
    DeviceState* s = cur(true);
    return s ? s->sms : 0;
}

static ScratchSet* scratch_set(DeviceState* s, cudaStream_t st)
{
    for (int i = 0; i < kMaxScratchSets; i++)
        if (s->sets[i].used && s->sets[i].st == st) return &s->sets[i];
    std::lock_guard<std::mutex> lk(g_mu);
    for (int i = 0; i < kMaxScratchSets; i++)
        if (s->sets[i].used && s->sets[i].st == st) return &s->sets[i];
    for (int i = 0; i < kMaxScratchSets; i++)
        if (!s->sets[i].used) {
            s->sets[i].st = st;
            s->sets[i].used = true;
            return &s->sets[i];
        }
    return nullptr;
}

void* workspace_slot(int slot, size_t bytes)
{
    DeviceState* s = cur(true);
    if (!s || slot < 0 || slot > 2) return nullptr;
    const cudaStream_t st = stream();
    ScratchSet* set = scratch_set(s, st);
    if (!set) {
        set_error("more than %d streams with their own scratch on one device", kMaxScratchSets);
        return nullptr;
    }
    if (bytes <= set->ws_bytes[slot]) return set->ws[slot];
    // Growing is refused while the stream is being captured: the synchronisation and the allocation below are not
    // capturable, and a captured kernel must never hold a block that a later call may free.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) {
        set_error("scratch block would have to grow to %zu bytes during stream capture (run the step once eagerly, or "
                  "call znn_gemm_workspace_reserve, before capturing)", bytes);
        return nullptr;
    }
    // Growing: everything queued so far may still read the old block.
    cudaStreamSynchronize(st);
    if (set->ws[slot]) cudaFree(set->ws[slot]);
    set->ws[slot] = nullptr;
    set->ws_bytes[slot] = 0;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        s->ws_generation++;
    }
    size_t want = bytes + (bytes >> 3);
    if (cudaMalloc(&set->ws[slot], want) != cudaSuccess) {
        cudaGetLastError();
        want = bytes;
        if (cudaMalloc(&set->ws[slot], want) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
    }
    set->ws_bytes[slot] = want;
    return set->ws[slot];
}

unsigned* scratch_counters()
{
    DeviceState* s = cur(true);
    if (!s) return nullptr;
    ScratchSet* set = scratch_set(s, stream());
    if (!set) return nullptr;
    if (!set->counters) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream(), &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) return nullptr;
        std::lock_guard<std::mutex> lk(g_mu);
        if (!set->counters) {
            unsigned* c = nullptr;
            if (cudaMalloc((void**)&c, kScratchCounters * sizeof(unsigned)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
            if (cudaMemset(c, 0, kScratchCounters * sizeof(unsigned)) != cudaSuccess) { cudaFree(c); cudaGetLastError(); return nullptr; }
            set->counters = c;
        }
    }
    return set->counters;
}

unsigned long long workspace_generation()
{
    DeviceState* s = cur(true);
    return s ? s->ws_generation : 0;
}

// Host-side fault injection for tests: the n-th kernel launch from now (of any host thread) is reported as failed.
static long long g_fail_after = -1;
bool inject_launch_failure()
{
    if (g_fail_after < 0) return false;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_fail_after < 0) return false;
    if (g_fail_after-- == 0) {
        g_fail_after = -1;
        return true;
    }
    return false;
}
void set_fail_after(long long n) { std::lock_guard<std::mutex> lk(g_mu); g_fail_after = n; }

void* workspace(size_t bytes) { return workspace_slot(0, bytes); }

long long launches_and_reset(int reset);

}  // namespace znn

using namespace znn;

extern "C" {

int znn_device_count(int* count)
{
    ZNN_REQUIRE(count, "count is NULL");
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) {
        *count = 0;
        return fail(ZNN_ERR_CUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
    }
    return ZNN_OK;
}

int znn_init(int device)
{
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail(ZNN_ERR_CUDA, "no CUDA device: %s (this library has no CPU fallback)",
                    e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    ZNN_REQUIRE(device >= 0 && device < n && device < kMaxDev, "device %d out of range (have %d)", device, n);
    ZNN_CUDA_OK(cudaSetDevice(device));
    cudaDeviceProp prop;
    ZNN_CUDA_OK(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(ZNN_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);
    if (!cur(true)) return fail(ZNN_ERR_CUDA, "could not create per-device state");
    return ZNN_OK;
}

int znn_set_device(int device)
{
    // per-host-thread current device, as cudaSetDevice; the per-device state is created on first use
    return znn_init(device);
}

int znn_set_stream(void* cuda_stream)
{
    t_user_stream = (cudaStream_t)cuda_stream;
    t_has_user_stream = (cuda_stream != nullptr);
    return ZNN_OK;
}

int znn_get_stream(void** cuda_stream)
{
    ZNN_REQUIRE(cuda_stream, "cuda_stream is NULL");
    *cuda_stream = (void*)stream();
    return ZNN_OK;
}

int znn_sync(void)
{
    ZNN_CUDA_OK(cudaStreamSynchronize(stream()));
    return ZNN_OK;
}

int znn_malloc(void** ptr, size_t bytes)
{
    ZNN_REQUIRE(ptr, "ptr is NULL");
    *ptr = nullptr;
    if (bytes == 0) return ZNN_OK;
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(e == cudaErrorMemoryAllocation ? ZNN_ERR_NOMEM : ZNN_ERR_CUDA, "cudaMalloc(%zu): %s", bytes,
                    cudaGetErrorString(e));
    }
    return ZNN_OK;
}

int znn_free(void* ptr)
{
    if (!ptr) return ZNN_OK;
    ZNN_CUDA_OK(cudaFree(ptr));
    return ZNN_OK;
}

int znn_memset(void* ptr, int value, size_t bytes)
{
    if (bytes == 0) return ZNN_OK;
    ZNN_CUDA_OK(cudaMemsetAsync(ptr, value, bytes, stream()));
    return ZNN_OK;
}

int znn_memcpy_h2d(void* dst, const void* src, size_t bytes)
{
    if (bytes == 0) return ZNN_OK;
    ZNN_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream()));
    return ZNN_OK;
}

int znn_memcpy_d2h(void* dst, const void* src, size_t bytes)
{
    if (bytes == 0) return ZNN_OK;
    ZNN_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream()));
    ZNN_CUDA_OK(cudaStreamSynchronize(stream()));
    return ZNN_OK;
}

int znn_memcpy_d2h_async(void* dst, const void* src, size_t bytes)
{
    if (bytes == 0) return ZNN_OK;
    ZNN_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream()));
    return ZNN_OK;
}

int znn_memcpy_d2d(void* dst, const void* src, size_t bytes)
{
    if (bytes == 0) return ZNN_OK;
    ZNN_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream()));
    return ZNN_OK;
}

int znn_memcpy2d_d2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows)
{
    if (width_bytes == 0 || rows == 0) return ZNN_OK;
    ZNN_CUDA_OK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDeviceToDevice, stream()));
    return ZNN_OK;
}

int znn_last_error(char* buf, size_t buflen)
{
    ZNN_REQUIRE(buf && buflen > 0, "buf is NULL");
    strncpy(buf, t_err, buflen - 1);
    buf[buflen - 1] = 0;
    return ZNN_OK;
}

int znn_device_status(int* status, int clear)
{
    ZNN_REQUIRE(status, "status is NULL");
    int* w = device_status_word();
    if (!w) return fail(ZNN_ERR_CUDA, "no device state");
    ZNN_CUDA_OK(cudaStreamSynchronize(stream()));
    ZNN_CUDA_OK(cudaMemcpy(status, w, sizeof(int), cudaMemcpyDeviceToHost));
    if (clear && *status) ZNN_CUDA_OK(cudaMemset(w, 0, sizeof(int)));
    return ZNN_OK;
}

int znn_workspace_generation(unsigned long long* generation)
{
    ZNN_REQUIRE(generation, "generation is NULL");
    *generation = workspace_generation();
    return ZNN_OK;
}

int znn_debug_fail_after(long long n)
{
    set_fail_after(n);
    return ZNN_OK;
}

int znn_launch_count(long long* count, int reset)
{
    ZNN_REQUIRE(count, "count is NULL");
    *count = launches_and_reset(reset);
    return ZNN_OK;
}

int znn_gemm_workspace_reserve(size_t bytes)
{
    if (!workspace(bytes)) return fail(ZNN_ERR_NOMEM, "could not reserve %zu bytes of GEMM scratch", bytes);
    return ZNN_OK;
}

}  // extern "C"
