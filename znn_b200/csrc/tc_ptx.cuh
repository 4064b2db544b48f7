// PTX wrappers shared by the tensor-core kernels (sm_100a): mbarriers with bounded waits, TMA loads, tcgen05
// allocation / MMA / commit / load, cluster helpers and shared-memory matrix descriptors.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace znn {

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Time base of the bounded waits: the SM's own 64-bit cycle counter.  (%globaltimer is not used: its 64-bit read
// is not guaranteed to be consistent when the low word wraps, every 4.29 s, and a torn read makes an elapsed time of
// seconds out of nothing.)  4e9 cycles are 2.0 s at the 1.965 GHz maximum clock, 2.7 s at 1.5 GHz.
__device__ __forceinline__ uint64_t wait_clock() { return (uint64_t)clock64(); }
constexpr uint64_t kWaitLimitCycles = 4000000000ull;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// The suspend-time hint lets the hardware park the thread until the phase completes (or the hint runs out) instead
// of returning at once: waiting roles then leave the issue slots and the shared-memory port to the working warps.
constexpr uint32_t kWaitSuspendNs = 20000;
#ifndef ZNN_WAIT_SLEEP_NS
#define ZNN_WAIT_SLEEP_NS 128   // back-off between polls of a long wait; 0 = keep polling
#endif
#ifndef ZNN_WAIT_FAST_POLLS
#define ZNN_WAIT_FAST_POLLS 8   // polls before a wait counts as long
#endif
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kWaitSuspendNs)
        : "memory");
    return ok;
}

// One look at the barrier without suspending the thread.
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Waits at most `limit` SM cycles (default 4e9, ~2 s); false on expiry.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit = kWaitLimitCycles)
{
    if (mbar_try_wait(bar, parity)) return true;
#pragma unroll 1
    for (int i = 0; i < ZNN_WAIT_FAST_POLLS; i++)
        if (mbar_try_wait(bar, parity)) return true;
    // a long wait: poll less often, so that waiting roles leave issue slots and the shared-memory port alone
    const uint64_t t0 = wait_clock();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; i++) {
            if (mbar_try_wait(bar, parity)) return true;
            if (ZNN_WAIT_SLEEP_NS > 0) __nanosleep(ZNN_WAIT_SLEEP_NS);
        }
        if (wait_clock() - t0 > limit) return false;
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// CTA-pair form: the mbarrier may live in the peer CTA (the pair's leader).
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
{
    if (CTAS == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}

template <int CTAS>
__device__ __forceinline__ void tmem_relinquish()
{
    if (CTAS == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    if (CTAS == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

template <int CTAS>
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    if (CTAS == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
}

// Arrive on an mbarrier once all previously issued MMAs of this thread are done.
__device__ __forceinline__ void umma_commit_1cta(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Pair form: arrives on the barrier at the same offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(mask)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float (&v)[32])
{
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// The same load without the wait: two loads can be in flight before one tmem_ld_wait2.  The registers may not be read
// before the wait; the wait therefore takes them as in-out operands, which keeps every use behind it.
__device__ __forceinline__ void tmem_ld_32x32_issue(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait2(uint32_t (&a)[32], uint32_t (&b)[32])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]), "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]), "+r"(a[16]), "+r"(a[17]), "+r"(a[18]), "+r"(a[19]), "+r"(a[20]), "+r"(a[21]), "+r"(a[22]), "+r"(a[23]), "+r"(a[24]), "+r"(a[25]), "+r"(a[26]), "+r"(a[27]), "+r"(a[28]), "+r"(a[29]), "+r"(a[30]), "+r"(a[31]) : : "memory");
    asm volatile("" : "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]), "+r"(b[8]), "+r"(b[9]), "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15]), "+r"(b[16]), "+r"(b[17]), "+r"(b[18]), "+r"(b[19]), "+r"(b[20]), "+r"(b[21]), "+r"(b[22]), "+r"(b[23]), "+r"(b[24]), "+r"(b[25]), "+r"(b[26]), "+r"(b[27]), "+r"(b[28]), "+r"(b[29]), "+r"(b[30]), "+r"(b[31]) : : "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank)
{
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (32 fp32) with the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                       // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                       // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}

// kind::tf32 instruction descriptor: D fp32, A/B tf32, both K-major.
__host__ __device__ constexpr uint32_t make_tf32_idesc(int mma_m, int mma_n)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}


__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr)
{
    // Default semantics (release at CTA scope): what the waiting side consumes is this CTA's own shared or tensor
    // memory, read by this SM's tensor-core half, so nothing has to be made visible cluster-wide.  The cluster-scope
    // form costs a memory barrier per arrival, which serialised the converter warps (measured: "membar" was the
    // top stall reason and short-K batched products ran 2x slower).
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kWaitSuspendNs)
        : "memory");
    return ok;
}

__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint32_t bar, uint32_t parity, uint64_t limit = kWaitLimitCycles)
{
    if (mbar_try_wait_cluster(bar, parity)) return true;
#pragma unroll 1
    for (int i = 0; i < ZNN_WAIT_FAST_POLLS; i++)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    // a long wait: poll less often, so that waiting roles leave issue slots and the shared-memory port alone
    const uint64_t t0 = wait_clock();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; i++) {
            if (mbar_try_wait_cluster(bar, parity)) return true;
            if (ZNN_WAIT_SLEEP_NS > 0) __nanosleep(ZNN_WAIT_SLEEP_NS);
        }
        if (wait_clock() - t0 > limit) return false;
    }
}

// MN-major tile (32-bit elements): the only shared-memory layout the tensor core takes is the
// 128-byte swizzle with 32-byte atoms (TMA: SWIZZLE_128B_ATOM_32B).  Each TMA box is 32 M/N
// elements (one 128-byte row) x 32 k-rows = 4096 bytes; swizzle atoms are 4 k-rows (512 bytes),
// so one K = 8 instruction spans two atoms.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(4096 >> 4) << 16;  // leading byte offset: next 32-wide M/N group (next box)
    d |= (uint64_t)(512 >> 4) << 32;   // stride byte offset: next atom of 4 k-rows
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;            // SWIZZLE_128B_BASE32B
    return d;
}

__host__ __device__ constexpr uint32_t make_tf32_idesc_major(int mma_m, int mma_n, bool a_mn, bool b_mn)
{
    return make_tf32_idesc(mma_m, mma_n) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16);
}

// The same wait without the back-off between polls, for roles on a latency-critical path with few warps per SM (each
// poll may still be parked by the hardware until the phase completes).  Bounded like the others.
__device__ __forceinline__ bool mbar_wait_bounded_tight(uint32_t bar, uint32_t parity, uint64_t limit = kWaitLimitCycles)
{
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = wait_clock();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (wait_clock() - t0 > limit) return false;
    }
}

// One lane of the (converged) warp; the same lane every time it is asked for.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
        "elect.sync rx|px, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, px;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// 4-d tiled TMA load (no multicast); the box lands in this CTA's shared memory and signals this CTA's mbarrier.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// CTA-pair form of the 4-d load: the box lands in this CTA's shared memory, the mbarrier (a shared::cluster address) may
// be the pair leader's, so that one barrier collects the bytes of both CTAs.  No multicast.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// CTA-pair MMA whose A operand lies in tensor memory (K-major: lane = row, one column per tf32 element, the same
// columns in both CTAs of the pair); B comes from shared memory through a descriptor.
__device__ __forceinline__ void umma_tf32_ts_pair(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 columns of 32-bit values from registers to tensor memory (thread i of the warp writes lane base + i)
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

}  // namespace znn
