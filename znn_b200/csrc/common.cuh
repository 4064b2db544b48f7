// Shared helpers for the znn CUDA shim (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/znn_cuda.h"

namespace znn {

// Per-host-thread error text, returned by znn_last_error().
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

// The stream every kernel of the calling host thread is launched on.
cudaStream_t stream();

// Device status word (one int per device, zero-initialised).  Kernels OR a
// ZNN_DEV_* bit into it when a bounded wait expires; znn_device_status() reads it.
int* device_status_word();

// Shim-owned scratch for GEMM operand planes; grows on demand.
void* workspace(size_t bytes);
// slot 1 is a second, independent block for callers that hold scratch across a GEMM call (conv im2col);
// slot 2 holds the device copies of host operands (znn_sgemm_host, znn_matmul_host_fwd_bwd)
void* workspace_slot(int slot, size_t bytes);

// kScratchCounters zero-initialised words per (device, stream), for kernels whose last block to finish completes a
// reduction: such a kernel counts its blocks with atomicAdd and must leave the words it used at zero again.  nullptr
// when they cannot be had (first use during a stream capture): callers then take their two-kernel form.
constexpr int kScratchCounters = 4096;
unsigned* scratch_counters();

int sm_count();

// Counts the reallocations of scratch blocks on the current device: a holder of raw scratch addresses (a captured
// CUDA graph) compares it with the value it saw when it took them.
unsigned long long workspace_generation();

// Test aid (znn_debug_fail_after): true once, for the launch the injected failure was armed for.
bool inject_launch_failure();

// Kernel-launch counter of the calling host thread (read by znn_launch_count).
void count_launch();

#define ZNN_CUDA_OK(expr)                                                              \
    do {                                                                               \
        cudaError_t _e = (expr);                                                       \
        if (_e != cudaSuccess)                                                         \
            return ::znn::fail(ZNN_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,           \
                               cudaGetErrorString(_e), __FILE__, __LINE__);            \
    } while (0)

#define ZNN_LAUNCH_OK(name)                                                            \
    do {                                                                               \
        cudaError_t _e = cudaGetLastError();                                           \
        if (_e != cudaSuccess)                                                         \
            return ::znn::fail(ZNN_ERR_CUDA, "launch of %s failed: %s", name,          \
                               cudaGetErrorString(_e));                                \
        ::znn::count_launch();                                                         \
        if (::znn::inject_launch_failure())                                            \
            return ::znn::fail(ZNN_ERR_CUDA, "launch of %s failed: injected failure (znn_debug_fail_after)", name); \
    } while (0)

#define ZNN_REQUIRE(cond, ...)                                                         \
    do {                                                                               \
        if (!(cond)) return ::znn::fail(ZNN_ERR_INVALID, __VA_ARGS__);                 \
    } while (0)

static inline int ceil_div(long a, long b) { return (int)((a + b - 1) / b); }

}  // namespace znn
