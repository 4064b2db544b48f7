// Fused causal self-attention on the 5th-generation tensor cores (sm_100a), forward and backward, at fp32 accuracy.
//
// Replaces the reference's chain transposeND x4 -> batchMatMul -> mulScalar -> mask -> add -> softmax -> batchMatMul ->
// transposeND (src/nn.zig:796-906; the operator arms are src/autodiff.zig:485-531, :1054-1076, :1117-1182): the score
// and probability matrices (B*nh*T*T floats each) never reach memory.  Q, K, V, O and their gradients are read and
// written where the projections leave them ([B, T, nh, hs] or [B, nh, T, hs]: row pitch and head / batch strides are
// arguments), so no head split or merge copy is needed either.
//
// One kernel template, four instantiations.  A work unit is 256 "rows" of one (batch, head) slice, held by a CTA pair
// (cta_group::2, 128 rows per CTA), against a stream of 64-wide "column" blocks:
//
//   forward   rows = queries, columns = keys     S = Q.K^T                   P = softmax (online)     O  += P.V
//   dQ        rows = queries, columns = keys     S = Q.K^T, dP = dO.V^T      dS = P o (dP - D)        dQ += dS.K
//   dK        rows = keys,    columns = queries  S^T = K.Q^T, dP^T = V.dO^T  dS^T                     dK += dS^T.Q
//   dV        rows = keys,    columns = queries  S^T = K.Q^T                 P^T                      dV += P^T.dO
//
// Every product is 3xTF32 (lo*hi + hi*lo + hi*hi of a hi/lo split, as in the GEMM kernels).
//  * The row operand X1 of the first product (Q or K) lives in TENSOR MEMORY for the whole unit: the transform warps
//    fetch their rows from global memory (whole 128-byte lines per access, handed to the thread that owns the row
//    through a small shared-memory stage), split them and store hi and lo with tcgen05.st; the product takes its A
//    operand from there.  (With A in shared memory a 256 x 64 x 8 instruction reads 4 KB of A per SM for 44 cycles of math, which
//    saturates the shared-memory port and starves TMA and the converter warps: measured.)
//  * The second row operand of dQ / dK (dO or V) does not fit in tensor memory beside the rest and stays in shared
//    memory (TMA + converter warps), as do all column operands: Y (K-major, for the first products) and Z (MN-major,
//    for the second product), hi = the raw tile from TMA, lo written next to it by converter warps.
//  * The first products land in tensor memory, where eight transform warps (two threads per row, 32 columns each) turn
//    them into the left operand W of the second product -- hi in place over S, lo beside it -- which the tensor core
//    again reads from tensor memory.  Each block's second product starts a fresh accumulator that the transform warps
//    add into fp32 registers (round to nearest; the tensor core's own accumulation truncates), rescaled in the forward
//    when the running row maximum moves.  Two S buffers let block c+1's first products run while block c is transformed.
//  * The MMA issuer issues P1(g) (first products of block g) and P2(g - 1) in whichever order their inputs arrive: while
//    it waits for block g's tile it issues the previous block's second product as soon as the transform warps have
//    handed it over, so a late tile does not hold back work that is ready (the two use different score buffers).
//  * Between units the pipeline drains; what shortens that: the next unit's rows are prefetched during the last block
//    and stored to tensor memory right after that block's hand-off, and the unit's result rows leave as whole lines.
//
// Causal structure: forward and dQ walk the key blocks 0 .. diagonal; dK and dV walk the query blocks diagonal .. end;
// elements above the diagonal are masked by index (the reference adds -1e9, which makes exp exactly 0).
// No TMA multicast.  Every mbarrier wait is bounded (status word + early exit, as in the GEMM kernels).
#include "tc_ptx.cuh"
#include "../../include/znn_debug.h"

#include <math.h>
#include <math_constants.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

namespace znn {

enum { ATT_FWD = 0, ATT_BWD_Q = 1, ATT_BWD_K = 2, ATT_BWD_V = 3 };

struct AttnParams {
    int T, hs, nslices, nh;
    int nrb, ncb;                 // 256-row blocks and 64-column blocks per slice
    int t_first;                  // 1: tensor-map coordinates are (d, t, h, b); 0: (d, h, t, b) (the smaller stride first)
    float scale, c2;              // c2 = scale * log2(e): the softmax runs in base 2
    long long ld, stride_h, stride_b;   // row pitch, head stride, batch stride of Q / K / V / O and gradients, in floats
    const float* x1;              // the row operand kept in tensor memory: Q (forward, dQ) or K (dK, dV)
    float* out;                   // O, dQ, dK or dV
    float* lse;                   // [nslices, T] base-2 log-sum-exp of the scaled scores: written by the forward, read by the others
    const float* dvec;            // [nslices, T] D = rowsum(dO o O) (dQ and dK)
    int accumulate;               // backward: 1 = add into out (the reference's +=), 0 = store
    int planes;                   // 1: the remainder (lo) parts of the shared-memory operands come precomputed through their own
                                  // tensor maps: TMA fills both halves of a stage and signals the MMA issuer's barrier directly
    int* status;
    int issue_in_order;           // 1: the MMA issuer keeps the fixed order P1(g), P2(g-1), P1(g+1), ... (A/B switch)
    const int* sched;             // [pairs][sched_k] the units of every CTA pair in the order it takes them, -1 after the last; or NULL
    int sched_k;                  // entries per pair (at most kAttSchedMax)
    unsigned long long wait_limit;
};

constexpr int kAttThreads = 512;   // warp 0 TMA, warp 1 MMA + TMEM, warps 2-7 converters, warps 8-15 transform
constexpr int kAttConvWarps = 6, kAttConvWarp0 = 2, kAttXfWarp0 = 8, kAttXfWarps = 8;
constexpr int kRowsPerCta = 128, kColBlock = 64;
constexpr int kAttSchedMax = 32;   // units per CTA pair a schedule table may hold (a copy of the pair's row lives in shared memory)

template <int MODE>
struct AttnCfg {
    static constexpr int NX = (MODE == ATT_BWD_Q || MODE == ATT_BWD_K) ? 2 : 1;   // first products per block
    static constexpr int kXTile = kRowsPerCta * 64 * 4;        // one plane (hi or lo) of the shared-memory row operand
    static constexpr int kXBytes = NX == 2 ? 2 * kXTile : 0;   // X2 (dO or V) of dQ / dK
    static constexpr int kYTile = 32 * 64 * 4;                 // this CTA's 32 of the block's 64 columns x 64 floats
    static constexpr int kYStage = NX * 2 * kYTile;
    static constexpr int kZTile = 64 * 32 * 4;                 // 64 contraction rows x this CTA's 32 output columns
    static constexpr int kZStage = 2 * kZTile;
#ifndef ZNN_ATT_STAGES1
#define ZNN_ATT_STAGES1 3      // ring stages of forward and dV; six measured no faster (and slower at 256 positions)
#endif
    static constexpr int NYS = NX == 2 ? 3 : ZNN_ATT_STAGES1;
    static constexpr int NZS = NX == 2 ? 3 : ZNN_ATT_STAGES1;
    static constexpr int kBarOff = kXBytes + NYS * kYStage + NZS * kZStage;
    static constexpr int kExchBytes = MODE == ATT_FWD ? 2048 : 0;   // row-maximum exchange between the two threads of a row
    // Row staging of the transform warps (rows enter and leave through full 128-byte lines although a thread owns a whole
    // row): per warp kStageRows rows of 8 float4 at a pitch of 9 float4 (conflict-free both ways).  32 rows where shared
    // memory allows, 8 rows (four passes) next to the 64 KB row operand of dQ / dK.
#ifndef ZNN_ATT_STAGE_ROWS1
#define ZNN_ATT_STAGE_ROWS1 32
#endif
    static constexpr int kStageRows = NX == 2 ? 8 : ZNN_ATT_STAGE_ROWS1;
    static constexpr int kStageWarpBytes = kStageRows * 144;
    static constexpr int kStageOff = kBarOff + 512 + kExchBytes;
    // dK and dV: the block's per-column statistics (log-sum-exp, D), fetched one column per lane ahead of the block and
    // passed round the warp here
    static constexpr int kColStatOff = kStageOff + kAttXfWarps * kStageWarpBytes;
    static constexpr int kColStatBytes = (MODE == ATT_BWD_K || MODE == ATT_BWD_V) ? kAttXfWarps * 256 : 0;
    static constexpr int kSmemBytes = kBarOff + 1024 /*alignment*/ + 512 /*barriers*/ + kExchBytes + kAttXfWarps * kStageWarpBytes + kColStatBytes;
    static_assert(kSmemBytes <= 232448, "shared memory budget");
    // tensor-memory columns (512 allocated): X1 hi | X1 lo | S / W_hi [2] | then, forward and dV: W_lo [2], accumulator [2];
    // dQ and dK: dP [2], W_lo [1], accumulator [1]
    static constexpr int NWB = NX == 2 ? 1 : 2;                // W_lo / accumulator buffers
    static constexpr uint32_t kColXhi = 0, kColXlo = 64, kColS = 128;
    static constexpr uint32_t kColDp = 256;
    static constexpr uint32_t kColWlo = NX == 2 ? 384 : 256;
    static constexpr uint32_t kColAcc = NX == 2 ? 448 : 384;
};

struct AttnUnit {
    int slice, b, h, row0, cb0, nb;   // row0: first row of the pair's 256-row block; column blocks cb0 .. cb0 + nb - 1
};

template <int MODE>
__device__ __forceinline__ AttnUnit attn_unit(const AttnParams& p, int u)
{
    AttnUnit d;
    const int rbi = u / p.nslices;            // dearest row blocks first
    d.slice = u - rbi * p.nslices;
    d.b = d.slice / p.nh;
    d.h = d.slice - d.b * p.nh;
    if (MODE == ATT_FWD || MODE == ATT_BWD_Q) {
        const int rb = p.nrb - 1 - rbi;
        d.row0 = rb * 256;
        d.cb0 = 0;
        const int last = min(p.T, d.row0 + 256);   // columns 0 .. last - 1 can be visible to these rows
        d.nb = (last + kColBlock - 1) / kColBlock;
    } else {
        d.row0 = rbi * 256;
        d.cb0 = d.row0 / kColBlock;
        d.nb = p.ncb - d.cb0;
    }
    return d;
}

// Optional role profile (compile with -DZNN_ATTN_PROFILE; off in the product build): CTA pair 0's leader adds up, per
// role, the cycles spent inside each kind of wait and the cycles of the whole role loop into g_attn_prof, which
// znn_debug_attn_profile reads: [0] MMA loop, [1] x waits, [2] y_conv, [3] w_ready, [4] z_conv, [5] acc_empty, [6] issue of
// the first products, [7] issue of the second products; [8] transform loop, [9] s_full, [10] acc_full, [11] row operand
// load; [12] producer loop, [13] its waits; [14] converter loop, [15] its waits, [17] fence + arrival; transform:
// [18] score load, [19] W store + hand-off, [20] accumulator drain, [21] load-to-hand-off of one block.  The life of ring
// slot 0 of the Y stream, summed over its tiles ([11] of them): [5] commit of the products that free the slot -> producer
// sees it empty, [16] loads issued -> converter sees the bytes, [24] conversion, [30] converter's hand-off done -> MMA
// issuer past its wait (slack when the issuer arrives late).
__device__ long long g_attn_prof[32];
#ifdef ZNN_ATTN_PROFILE
#define ATT_PROF_T0 const long long prof_t0 = clock64();
#define ATT_PROF_WAIT(slot, expr) [&]() { const long long t_ = clock64(); const bool r_ = (expr); prof_acc[slot] += clock64() - t_; return r_; }()
#define ATT_PROF_END(slot)                                                                         \
    if (prof_on) {                                                                                 \
        prof_acc[slot] += clock64() - prof_t0;                                                     \
        for (int i_ = 0; i_ < 32; i_++)                                                            \
            if (prof_acc[i_]) atomicAdd((unsigned long long*)&g_attn_prof[i_], (unsigned long long)prof_acc[i_]); \
    }
#define ATT_PROF_MARK2(name) const long long name = clock64();
#define ATT_PROF_ADD2(slot, name) prof_acc[slot] += clock64() - name;
#else
#define ATT_PROF_MARK2(name)
#define ATT_PROF_ADD2(slot, name)
#define ATT_PROF_T0
#define ATT_PROF_WAIT(slot, expr) (expr)
#define ATT_PROF_END(slot)
#endif

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void split_hi_lo(float x, uint32_t& hi, uint32_t& lo)
{
    hi = __float_as_uint(x) & 0xFFFFE000u;                   // exactly a TF32 value
    lo = __float_as_uint(x - __uint_as_float(hi));           // exact in fp32, at most 2^-10 |x|
}

template <int MODE>
__global__ void __launch_bounds__(kAttThreads, 1)
attn_kernel(const __grid_constant__ CUtensorMap mx2, const __grid_constant__ CUtensorMap my1,
            const __grid_constant__ CUtensorMap my2, const __grid_constant__ CUtensorMap mz,
            const __grid_constant__ CUtensorMap mx2l, const __grid_constant__ CUtensorMap my1l,
            const __grid_constant__ CUtensorMap my2l, const __grid_constant__ CUtensorMap mzl, const AttnParams p)
{
    using Cfg = AttnCfg<MODE>;
    constexpr int NX = Cfg::NX, NYS = Cfg::NYS, NZS = Cfg::NZS, NWB = Cfg::NWB;
    constexpr uint32_t kColS = Cfg::kColS, kColDp = Cfg::kColDp, kColWlo = Cfg::kColWlo, kColAcc = Cfg::kColAcc;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t x_base = smem_base, y_base = x_base + Cfg::kXBytes, z_base = y_base + NYS * Cfg::kYStage;
    const uint32_t bar_base = smem_base + Cfg::kBarOff;
    // barriers.  "full": TMA -> converters (own CTA); "conv": converters of both CTAs -> MMA issuer (leader CTA);
    // "empty": MMA commit -> TMA producers (both CTAs); x1_ready: transform warps of both CTAs -> MMA issuer;
    // s_full / acc_full: MMA commit -> transform warps (both CTAs); w_ready: transform warps of both CTAs -> MMA issuer.
    // (w_ready of block g also tells that the accumulator and W_lo buffers block g will use have been drained: the same
    // warps drained them earlier in program order.)
    int bi = 0;
    const uint32_t x_full = bar_base + 8u * bi++, x_conv = bar_base + 8u * bi++, x_empty = bar_base + 8u * bi++;
    const uint32_t x1_ready = bar_base + 8u * bi++;
    const uint32_t y_full0 = bar_base + 8u * bi; bi += NYS;
    const uint32_t y_conv0 = bar_base + 8u * bi; bi += NYS;
    const uint32_t y_empty0 = bar_base + 8u * bi; bi += NYS;
    const uint32_t z_full0 = bar_base + 8u * bi; bi += NZS;
    const uint32_t z_conv0 = bar_base + 8u * bi; bi += NZS;
    const uint32_t z_empty0 = bar_base + 8u * bi; bi += NZS;
    const uint32_t s_full0 = bar_base + 8u * bi; bi += 2;
    const uint32_t w_ready0 = bar_base + 8u * bi; bi += 2;
    const uint32_t acc_full0 = bar_base + 8u * bi; bi += 2;
    const int kWordOff = 8 * bi;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + Cfg::kBarOff + kWordOff);
    const uint32_t tmem_slot_addr = bar_base + kWordOff;
    volatile uint32_t* abort_slot = tmem_slot + 1;
    const uint32_t abort_slot_addr = tmem_slot_addr + 4;

    // the warp index through a shuffle: the compiler then knows it is the same in all lanes, and the code of the MMA
    // warp below (executed by all its lanes, with one elected lane issuing) stays on the uniform datapath
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int cta_rank = (int)cluster_ctarank();
    const bool leader = (cta_rank == 0);
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int total_units = p.nslices * p.nrb;
    const int kbh = p.hs >> 5;                    // 32-float k-blocks across the head dimension (1 or 2)
    // The k-th unit of this CTA pair, or -1.  Units are numbered dearest first.  With a schedule table (made on the host:
    // every unit, dearest first, goes to the pair with the least work so far) the pair's row of the table is read from
    // shared memory; without one, round k deals units k * npairs .. to the pairs in alternating direction, so that a pair
    // that got a dear unit in one round gets a cheap one in the next.  At 96 slices x 1024 positions the busiest pair
    // then has 56 blocks in 5 or 6 units, with the table 52-53, against a mean of 51.9.
    const int* const sched_s = reinterpret_cast<const int*>(smem_gen + Cfg::kBarOff + 256);   // kAttSchedMax entries
    const bool have_sched = p.sched != nullptr;
    auto unit_of = [&](int k) -> int {
        if (have_sched) return k < p.sched_k ? sched_s[k] : -1;
        const int u = k * npairs + ((k & 1) ? npairs - 1 - pair : pair);
        return u < total_units ? u : -1;
    };
#ifdef ZNN_ATTN_PROFILE
    volatile long long* const tstamp = reinterpret_cast<volatile long long*>(smem_gen + Cfg::kBarOff + 512 - 128);   // 16 slots
    const bool prof_on = (pair == 0 && cta_rank == 0 && lane == 0 && (warp <= 3 || warp == kAttXfWarp0));
    const int pslot = (warp == 3) ? 8 : 0;     // the second converter warp (a Z tile; the second Y tile in dQ / dK) reports in slots 22..25
    long long prof_acc[32];      // in registers; written once at the end of the role
#pragma unroll
    for (int i = 0; i < 32; i++) prof_acc[i] = 0;
#endif

    if (have_sched && threadIdx.x >= 32 && threadIdx.x < 32 + kAttSchedMax) {
        const int k = threadIdx.x - 32;
        reinterpret_cast<int*>(smem_gen + Cfg::kBarOff + 256)[k] = k < p.sched_k ? p.sched[(size_t)pair * p.sched_k + k] : -1;
    }
    if (threadIdx.x == 0) {
        static_assert(8 * (4 + 3 * NYS + 3 * NZS + 6) + 8 <= 256, "barrier block overflows into the schedule row");
        static_assert(256 + 4 * kAttSchedMax <= 512 - 128, "schedule row overflows into the profile stamps");
        mbar_init(x_full, 1);
        mbar_init(x_conv, p.planes ? 1 : kAttConvWarps * 2);   // planes: the leader's producer arrives, TMA brings the bytes
        mbar_init(x_empty, 1);
        mbar_init(x1_ready, kAttXfWarps * 2);
        for (int s = 0; s < NYS; s++) {
            mbar_init(y_full0 + 8u * s, 1);
            mbar_init(y_conv0 + 8u * s, p.planes ? 1 : 2 * NX * NX);   // per CTA: one warp per tile (forward, dV), two per tile (dQ, dK)
            mbar_init(y_empty0 + 8u * s, 1);
        }
        for (int s = 0; s < NZS; s++) {
            mbar_init(z_full0 + 8u * s, 1);
            mbar_init(z_conv0 + 8u * s, p.planes ? 1 : 2 * NX);
            mbar_init(z_empty0 + 8u * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(s_full0 + 8u * b, 1);
            mbar_init(w_ready0 + 8u * b, kAttXfWarps * 2);
            mbar_init(acc_full0 + 8u * b, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (leader) {
            const uint32_t prior = (uint32_t)(*reinterpret_cast<volatile int*>(p.status));
            *abort_slot = prior;
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(mapa_shared(abort_slot_addr, 1)), "r"(prior) : "memory");
        }
    }
    if (warp == 1) {
        tmem_alloc<2>(tmem_slot_addr, 512);
        tmem_relinquish<2>();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool aborted = (*abort_slot != 0);

    if (warp < kAttXfWarp0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
        if (aborted) {
        } else if (warp == 0) {
            // ---------------- TMA producer ----------------
            // Two lanes, one stream each: lane 0 fetches the row operand of dQ / dK and the Y tiles, lane 1 the Z tiles.  A
            // Z slot is freed late in a block's life (after its second product); in one thread that wait held back the
            // next Y tile, the one the issuer needs first.
            if (lane < 2) {
                const bool do_y = lane == 0, do_z = lane == 1;
                bool ok = true;
                uint32_t it = 0, ul = 0;
                ATT_PROF_T0
                for (int k = 0, u; (u = unit_of(k)) >= 0 && ok; k++, ul++) {
                    const AttnUnit d = attn_unit<MODE>(p, u);
                    // planes: both halves (values, whose low mantissa bits the tensor core ignores, and precomputed
                    // remainders) come by TMA, and the bytes of both CTAs are counted by the leader's "conv" barrier,
                    // the one the MMA issuer waits on: no converter, no proxy fence, one hop less per tile
                    const bool pl = p.planes != 0;
                    if (NX == 2 && do_y) {
                        // the shared-memory row operand of this unit, once the previous unit's first products no longer read it
                        if (!ATT_PROF_WAIT(13, mbar_wait_bounded(x_empty, (ul & 1) ^ 1, p.wait_limit))) { ok = false; break; }
                        const int xrow = d.row0 + cta_rank * kRowsPerCta;
                        if (pl) {
                            const uint32_t fb = mapa_shared(x_conv, 0);
                            if (leader) mbar_arrive_expect_tx(x_conv, (uint32_t)(4 * kbh * 16384));
                            for (int kb = 0; kb < kbh; kb++) {
                                if (p.t_first) {
                                    tma_load_4d_pair(x_base + kb * 16384, &mx2, fb, 32 * kb, xrow, d.h, d.b);
                                    tma_load_4d_pair(x_base + Cfg::kXTile + kb * 16384, &mx2l, fb, 32 * kb, xrow, d.h, d.b);
                                } else {
                                    tma_load_4d_pair(x_base + kb * 16384, &mx2, fb, 32 * kb, d.h, xrow, d.b);
                                    tma_load_4d_pair(x_base + Cfg::kXTile + kb * 16384, &mx2l, fb, 32 * kb, d.h, xrow, d.b);
                                }
                            }
                        } else {
                            mbar_arrive_expect_tx(x_full, (uint32_t)(kbh * 16384));
                            for (int kb = 0; kb < kbh; kb++) {
                                if (p.t_first) tma_load_4d(x_base + kb * 16384, &mx2, x_full, 32 * kb, xrow, d.h, d.b);
                                else tma_load_4d(x_base + kb * 16384, &mx2, x_full, 32 * kb, d.h, xrow, d.b);
                            }
                        }
                    }
                    for (int c = 0; c < d.nb && ok; c++, it++) {
                        const int col0 = (d.cb0 + c) * kColBlock;
                        if (do_y) {   // Y: this CTA's 32 of the block's 64 columns, K-major
                            const int s = it % NYS;
                            if (!ATT_PROF_WAIT(13, mbar_wait_bounded(y_empty0 + 8u * s, ((it / NYS) & 1) ^ 1, p.wait_limit))) { ok = false; break; }
#ifdef ZNN_ATTN_PROFILE
                            if (prof_on && s == 0 && it >= (uint32_t)NYS) { prof_acc[5] += clock64() - tstamp[8]; prof_acc[11] += 1; }
#endif
                            const uint32_t st = y_base + s * Cfg::kYStage;
                            const int yrow = col0 + cta_rank * 32;
                            if (pl) {
                                const uint32_t fb = mapa_shared(y_conv0 + 8u * s, 0);
                                if (leader) mbar_arrive_expect_tx(y_conv0 + 8u * s, (uint32_t)(4 * NX * kbh * 4096));
                                for (int kb = 0; kb < kbh; kb++) {
                                    if (p.t_first) {
                                        tma_load_4d_pair(st + kb * 4096, &my1, fb, 32 * kb, yrow, d.h, d.b);
                                        tma_load_4d_pair(st + Cfg::kYTile + kb * 4096, &my1l, fb, 32 * kb, yrow, d.h, d.b);
                                    } else {
                                        tma_load_4d_pair(st + kb * 4096, &my1, fb, 32 * kb, d.h, yrow, d.b);
                                        tma_load_4d_pair(st + Cfg::kYTile + kb * 4096, &my1l, fb, 32 * kb, d.h, yrow, d.b);
                                    }
                                    if (NX == 2) {
                                        if (p.t_first) {
                                            tma_load_4d_pair(st + 2 * Cfg::kYTile + kb * 4096, &my2, fb, 32 * kb, yrow, d.h, d.b);
                                            tma_load_4d_pair(st + 3 * Cfg::kYTile + kb * 4096, &my2l, fb, 32 * kb, yrow, d.h, d.b);
                                        } else {
                                            tma_load_4d_pair(st + 2 * Cfg::kYTile + kb * 4096, &my2, fb, 32 * kb, d.h, yrow, d.b);
                                            tma_load_4d_pair(st + 3 * Cfg::kYTile + kb * 4096, &my2l, fb, 32 * kb, d.h, yrow, d.b);
                                        }
                                    }
                                }
                            } else {
                                const uint32_t fb = y_full0 + 8u * s;
                                mbar_arrive_expect_tx(fb, (uint32_t)(NX * kbh * 4096));
                                for (int kb = 0; kb < kbh; kb++) {
                                    if (p.t_first) tma_load_4d(st + kb * 4096, &my1, fb, 32 * kb, yrow, d.h, d.b);
                                    else tma_load_4d(st + kb * 4096, &my1, fb, 32 * kb, d.h, yrow, d.b);
                                    if (NX == 2) {
                                        if (p.t_first) tma_load_4d(st + 2 * Cfg::kYTile + kb * 4096, &my2, fb, 32 * kb, yrow, d.h, d.b);
                                        else tma_load_4d(st + 2 * Cfg::kYTile + kb * 4096, &my2, fb, 32 * kb, d.h, yrow, d.b);
                                    }
                                }
                            }
#ifdef ZNN_ATTN_PROFILE
                            if (prof_on && s == 0) tstamp[9] = clock64();
#endif
                        }
                        if (do_z) {   // Z: the block's 64 contraction rows x this CTA's 32 output columns, MN-major
                            const int s = it % NZS;
                            if (!ATT_PROF_WAIT(13, mbar_wait_bounded(z_empty0 + 8u * s, ((it / NZS) & 1) ^ 1, p.wait_limit))) { ok = false; break; }
                            const uint32_t st = z_base + s * Cfg::kZStage;
                            const int d0 = cta_rank * 32;     // beyond hs (hs = 32, second CTA): the box is zero-filled
                            if (pl) {
                                const uint32_t fb = mapa_shared(z_conv0 + 8u * s, 0);
                                if (leader) mbar_arrive_expect_tx(z_conv0 + 8u * s, 4u * 8192u);
                                for (int kk = 0; kk < 2; kk++) {
                                    if (p.t_first) {
                                        tma_load_4d_pair(st + kk * 4096, &mz, fb, d0, col0 + 32 * kk, d.h, d.b);
                                        tma_load_4d_pair(st + Cfg::kZTile + kk * 4096, &mzl, fb, d0, col0 + 32 * kk, d.h, d.b);
                                    } else {
                                        tma_load_4d_pair(st + kk * 4096, &mz, fb, d0, d.h, col0 + 32 * kk, d.b);
                                        tma_load_4d_pair(st + Cfg::kZTile + kk * 4096, &mzl, fb, d0, d.h, col0 + 32 * kk, d.b);
                                    }
                                }
                            } else {
                                const uint32_t fb = z_full0 + 8u * s;
                                mbar_arrive_expect_tx(fb, 8192u);
                                for (int kk = 0; kk < 2; kk++) {
                                    if (p.t_first) tma_load_4d(st + kk * 4096, &mz, fb, d0, col0 + 32 * kk, d.h, d.b);
                                    else tma_load_4d(st + kk * 4096, &mz, fb, d0, d.h, col0 + 32 * kk, d.b);
                                }
                            }
                        }
                    }
                }
                if (!ok) atomicOr(p.status, ZNN_DEV_TMA_WAIT_EXPIRED);
                ATT_PROF_END(12)
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer (leader CTA only) ----------------
            // All 32 lanes run the loop, poll the barriers and compute the (warp-uniform) descriptors; one elected lane
            // issues the instructions.  Descriptors computed by a single diverged thread instead gave wrong
            // products once the instructions followed each other closely (measured: correct again with a pause
            // between them), and cost about twice the issue time.
            if (leader) {
                const bool elected = elect_one();
                // every lane polls (one warp-wide instruction per poll, no broadcast of the answer); the vote keeps the
                // warp's decision uniform should the limit run out for some lanes only
                auto warp_wait = [&](uint32_t bar, uint32_t parity) -> bool {
                    return __all_sync(0xffffffffu, mbar_wait_bounded_tight(bar, parity, p.wait_limit));
                };
                constexpr uint32_t idesc1 = make_tf32_idesc_major(256, 64, false, false);
                constexpr uint32_t idesc2 = make_tf32_idesc_major(256, 64, false, true);
                bool ok = true;
                uint32_t it = 0, ul = 0, g = 0;               // it: blocks whose first products were issued; g: the same, named for the buffers
                const int ksteps1 = p.hs >> 3;                // K = 8 per instruction
                const uint64_t dx0 = make_kmajor_sw128_desc(x_base), dy0 = make_kmajor_sw128_desc(y_base);
                const uint64_t dz0 = make_mnmajor_sw128_desc(z_base);
                uint32_t itz = 0;
                ATT_PROF_T0
                // second product of block gb (program order: P1(c), P2(c-1), P1(c+1), P2(c), ...)
                auto second = [&](uint32_t gb) -> bool {
                    const uint32_t sbuf = gb & 1, wbuf = gb % NWB;
                    if (!ATT_PROF_WAIT(3, warp_wait(w_ready0 + 8u * sbuf, (gb >> 1) & 1))) return false;
#ifdef ZNN_ATTN_PROFILE
                    if (prof_on) { prof_acc[27] += clock64() - tstamp[4 + (gb & 3)]; prof_acc[29] += 1; }
#endif
                    const int s = itz % NZS;
                    if (!ATT_PROF_WAIT(4, warp_wait(z_conv0 + 8u * s, (itz / NZS) & 1))) return false;
                    tc_fence_after();
                    const uint64_t z_hi = dz0 + (uint64_t)((s * Cfg::kZStage) >> 4), z_lo = z_hi + (Cfg::kZTile >> 4);
                    const uint32_t a_hi = tmem_base + kColS + 64u * sbuf, a_lo = tmem_base + kColWlo + 64u * wbuf;
                    const uint32_t d_acc = tmem_base + kColAcc + 64u * wbuf;
                    constexpr uint32_t zstep = 1024 >> 4;
                    ATT_PROF_MARK2(pm)
                    if (elected) {
#pragma unroll
                        for (int k = 0; k < 8; k++) umma_tf32_ts_pair(d_acc, a_lo + 8u * k, z_hi + zstep * k, idesc2, k == 0 ? 0u : 1u);
#pragma unroll
                        for (int k = 0; k < 8; k++) umma_tf32_ts_pair(d_acc, a_hi + 8u * k, z_lo + zstep * k, idesc2, 1);
#pragma unroll
                        for (int k = 0; k < 8; k++) umma_tf32_ts_pair(d_acc, a_hi + 8u * k, z_hi + zstep * k, idesc2, 1);
                        umma_commit_pair(acc_full0 + 8u * wbuf);
                        umma_commit_pair(z_empty0 + 8u * s);
                    }
                    __syncwarp();
                    ATT_PROF_ADD2(7, pm)
                    itz++;
                    return true;
                };
                // Waits for `bar`; while it is not there, the second product of the oldest block that still lacks it
                // (block h, h < g: its first product has been issued) is issued as soon as its own inputs are, so that a
                // late tile of block g does not hold back work that is ready.  The two products of different blocks use
                // different score buffers, so their order is free; P1(g) only needs P2(g - 2) issued before it.
                uint32_t h = 0;                               // second products issued so far
                auto wait_or_second = [&](uint32_t bar, uint32_t parity) -> bool {
                    if (__all_sync(0xffffffffu, mbar_test(bar, parity))) return true;
                    if (p.issue_in_order) return warp_wait(bar, parity);
                    const uint64_t t0 = wait_clock();
                    for (uint32_t polls = 0;; polls++) {
                        // (every lane looks and the warp votes: no broadcast of one lane's answer)
                        if (__all_sync(0xffffffffu, mbar_test(bar, parity))) return true;
                        bool ready2 = false;
                        if (h < g) {
                            const uint32_t zs = itz % NZS;
                            ready2 = __all_sync(0xffffffffu, mbar_test(w_ready0 + 8u * (h & 1), (h >> 1) & 1) &&
                                                                 mbar_test(z_conv0 + 8u * zs, (itz / NZS) & 1));
                        }
                        if (ready2) {
                            if (!second(h)) return false;
                            h++;
                        } else if ((polls & 255u) == 255u && wait_clock() - t0 > p.wait_limit) return false;
                    }
                };
                for (int k = 0, u; (u = unit_of(k)) >= 0 && ok; k++, ul++) {
                    const AttnUnit d = attn_unit<MODE>(p, u);
                    if (!ATT_PROF_WAIT(1, wait_or_second(x1_ready, ul & 1))) { ok = false; break; }
                    if (NX == 2 && !ATT_PROF_WAIT(1, wait_or_second(x_conv, ul & 1))) { ok = false; break; }
                    tc_fence_after();
                    for (int c = 0; c < d.nb && ok; c++, g++, it++) {
                        const uint32_t buf = g & 1;
                        const int s = it % NYS;
                        if (!ATT_PROF_WAIT(2, wait_or_second(y_conv0 + 8u * s, (it / NYS) & 1))) { ok = false; break; }
                        tc_fence_after();
#ifdef ZNN_ATTN_PROFILE
                        if (prof_on && s == 0) prof_acc[30] += clock64() - tstamp[10];
#endif
                        ATT_PROF_MARK2(pm)
                        if (elected) {
                            // descriptors differ from the base ones by constant offsets (in 16-byte units): k-step k lies in
                            // k-block k / 4 (4 KB apart in Y, 16 KB in the shared-memory X), 32 bytes per step
                            const uint64_t yb_hi = dy0 + (uint64_t)((s * Cfg::kYStage) >> 4), yb_lo = yb_hi + (Cfg::kYTile >> 4);
                            const uint32_t x_hi = tmem_base + Cfg::kColXhi, x_lo = tmem_base + Cfg::kColXlo;
                            const uint32_t d_s = tmem_base + kColS + 64u * buf;
                            // S = X1.Y1^T with X1 in tensor memory: lo*hi, hi*lo, hi*hi
#pragma unroll
                            for (int k = 0; k < 8; k++)
                                if (k < ksteps1) umma_tf32_ts_pair(d_s, x_lo + 8u * k, yb_hi + (uint64_t)((k >> 2) * 256 + (k & 3) * 2), idesc1, k == 0 ? 0u : 1u);
#pragma unroll
                            for (int k = 0; k < 8; k++)
                                if (k < ksteps1) umma_tf32_ts_pair(d_s, x_hi + 8u * k, yb_lo + (uint64_t)((k >> 2) * 256 + (k & 3) * 2), idesc1, 1);
#pragma unroll
                            for (int k = 0; k < 8; k++)
                                if (k < ksteps1) umma_tf32_ts_pair(d_s, x_hi + 8u * k, yb_hi + (uint64_t)((k >> 2) * 256 + (k & 3) * 2), idesc1, 1);
                            if (NX == 2) {
                                // dP = X2.Y2^T with X2 in shared memory
                                const uint64_t xa_hi = dx0, xa_lo = dx0 + (Cfg::kXTile >> 4);
                                const uint64_t y2_hi = yb_hi + (uint64_t)((2 * Cfg::kYTile) >> 4), y2_lo = y2_hi + (Cfg::kYTile >> 4);
                                const uint32_t d_dp = tmem_base + kColDp + 64u * buf;
#pragma unroll
                                for (int k = 0; k < 8; k++)
                                    if (k < ksteps1)
                                        umma_tf32<2>(d_dp, xa_lo + (uint64_t)((k >> 2) * 1024 + (k & 3) * 2), y2_hi + (uint64_t)((k >> 2) * 256 + (k & 3) * 2), idesc1, k == 0 ? 0u : 1u);
#pragma unroll
                                for (int k = 0; k < 8; k++)
                                    if (k < ksteps1)
                                        umma_tf32<2>(d_dp, xa_hi + (uint64_t)((k >> 2) * 1024 + (k & 3) * 2), y2_lo + (uint64_t)((k >> 2) * 256 + (k & 3) * 2), idesc1, 1);
#pragma unroll
                                for (int k = 0; k < 8; k++)
                                    if (k < ksteps1)
                                        umma_tf32<2>(d_dp, xa_hi + (uint64_t)((k >> 2) * 1024 + (k & 3) * 2), y2_hi + (uint64_t)((k >> 2) * 256 + (k & 3) * 2), idesc1, 1);
                            }
                            umma_commit_pair(s_full0 + 8u * buf);
                            umma_commit_pair(y_empty0 + 8u * s);
#ifdef ZNN_ATTN_PROFILE
                            tstamp[g & 3] = clock64();
                            if (s == 0) tstamp[8] = clock64();
#endif
                            if (NX == 2 && c == d.nb - 1) umma_commit_pair(x_empty);   // the shared-memory row operand is free after these
                        }
                        __syncwarp();
                        ATT_PROF_ADD2(6, pm)
                        // the previous block's second product (of this unit or of the one before): program order
                        // P1(g), P2(g-1), P1(g+1), P2(g), ... runs on across units
                        if (h < g) {
                            if (!second(h)) { ok = false; break; }
                            h++;
                        }
                    }
                }
                if (ok && h < g && !second(h)) ok = false;
                if (!ok && lane == 0) atomicOr(p.status, ZNN_DEV_MMA_WAIT_EXPIRED);
                ATT_PROF_END(0)
            }
        } else {
            // ---------------- converters: lo = x - (x with the 13 low mantissa bits cleared), next to each landed tile ----------------
            // The conversion of a landed tile and its hand-off sit in the middle of the supply chain (producer -> TMA ->
            // converter -> MMA issuer), so the six warps work apart, each on a small piece with its own hand-off:
            // forward and dV (tiles Y, Z per block) warps 0, 2, 4 take the Y tiles of blocks 0, 1, 2 (mod 3) and warps
            // 1, 3, 5 the Z tiles; dQ and dK (tiles Y1, Y2, Z per block) two warps take half a tile each of every block.
            // Either way a warp meets every ring slot it works on in turn (three stages, three groups; or every block), so
            // when it waits for a slot's tile it has itself seen the slot's previous tile land: the parity wait cannot
            // mistake an older phase for the new one.  The shared-memory row operand (dQ, dK) is converted by all six.
            const int cw = warp - kAttConvWarp0;                               // 0 .. 5
            constexpr int kJobs = NX + 1;                                      // tiles per block
            constexpr int kSplit = NX;                                         // warps per tile
            constexpr int kGroups = kAttConvWarps / (kJobs * kSplit);          // groups of warps taking blocks in turn: 3 or 1
            static_assert(NYS % kGroups == 0 && NZS % kGroups == 0, "a converter warp always meets the same ring slots");
            const int job = cw % kJobs, sub = (cw / kJobs) % kSplit, turn = cw / (kJobs * kSplit);
            const int kind = job == NX ? 1 : 0;                                // Y (job = which of the NX tiles) or Z
            const int ct = threadIdx.x - 32 * kAttConvWarp0;                   // 0 .. 191 over all converter warps
            const uint32_t x_conv_l = mapa_shared(x_conv, 0), y_conv_l0 = mapa_shared(y_conv0, 0), z_conv_l0 = mapa_shared(z_conv0, 0);
            auto convert = [&](uint8_t* base, int nvec, int lo_off, int tid, int nthr) {
#pragma unroll 1
                for (int i0 = tid; i0 < nvec; i0 += 4 * nthr) {
                    uint4 x[4];
#pragma unroll
                    for (int v = 0; v < 4; v++)
                        if (i0 + v * nthr < nvec) x[v] = *reinterpret_cast<const uint4*>(base + 16 * (i0 + v * nthr));
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        if (i0 + v * nthr >= nvec) continue;
                        float4 l;
                        l.x = __uint_as_float(x[v].x) - __uint_as_float(x[v].x & 0xFFFFE000u);
                        l.y = __uint_as_float(x[v].y) - __uint_as_float(x[v].y & 0xFFFFE000u);
                        l.z = __uint_as_float(x[v].z) - __uint_as_float(x[v].z & 0xFFFFE000u);
                        l.w = __uint_as_float(x[v].w) - __uint_as_float(x[v].w & 0xFFFFE000u);
                        *reinterpret_cast<float4*>(base + 16 * (i0 + v * nthr) + lo_off) = l;
                    }
                }
            };
            // Every lane polls and the warp votes.  With one polling lane and a broadcast of its answer a wait that passes at
            // once cost 240 cycles against 90, and the warp stayed split through the conversion loop that follows (lane 0
            // and the other 31 ran it one after the other: twice the time, both measured).
            auto wait_full = [&](uint32_t bar, uint32_t ph) -> bool {
                const bool ok = ATT_PROF_WAIT(15 + pslot, mbar_wait_bounded_tight(bar, ph, p.wait_limit));
                return __all_sync(0xffffffffu, ok);
            };
            auto done = [&](uint32_t leader_bar) {
                asm volatile("" ::: "memory");
                ATT_PROF_MARK2(pf)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(leader_bar);
                ATT_PROF_ADD2(17 + pslot, pf)
            };
            bool got = true;
            uint32_t it = 0, ul = 0;       // it: blocks seen so far (the ring counter of both streams)
            ATT_PROF_T0
            for (int k = 0, u; !p.planes && (u = unit_of(k)) >= 0 && got; k++, ul++) {   // (planes: nothing to convert)
                const AttnUnit d = attn_unit<MODE>(p, u);
                if (NX == 2) {
                    if (!(got = wait_full(x_full, ul & 1))) break;
                    convert(smem_gen, kbh * 1024, Cfg::kXTile, ct, 32 * kAttConvWarps);
                    done(x_conv_l);
                }
                for (int c = 0; c < d.nb; c++, it++) {
                    if ((int)(it % kGroups) != turn) continue;
                    if (kind == 0) {
                        const int s = it % NYS;
                        if (!(got = wait_full(y_full0 + 8u * s, (it / NYS) & 1))) break;
#ifdef ZNN_ATTN_PROFILE
                        const long long tc0 = clock64();
                        if (prof_on && s == 0) prof_acc[16] += tc0 - tstamp[9];
#endif
                        uint8_t* st = smem_gen + Cfg::kXBytes + s * Cfg::kYStage;
                        convert(st + job * 2 * Cfg::kYTile + sub * (kbh * 4096 / kSplit), kbh * 256 / kSplit, Cfg::kYTile, lane, 32);
#ifdef ZNN_ATTN_PROFILE
                        if (prof_on && s == 0) prof_acc[24] += clock64() - tc0;
#endif
                        done(y_conv_l0 + 8u * s);
#ifdef ZNN_ATTN_PROFILE
                        if (prof_on && s == 0) tstamp[10] = clock64();
#endif
                    } else {
                        const int s = it % NZS;
                        if (!(got = wait_full(z_full0 + 8u * s, (it / NZS) & 1))) break;
                        uint8_t* st = smem_gen + Cfg::kXBytes + NYS * Cfg::kYStage + s * Cfg::kZStage;
                        convert(st + sub * (8192 / kSplit), 512 / kSplit, Cfg::kZTile, lane, 32);
                        done(z_conv_l0 + 8u * s);
                    }
                }
            }
            if (!got && lane == 0) atomicOr(p.status, ZNN_DEV_TMA_WAIT_EXPIRED);
            ATT_PROF_END(14 + pslot)
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
        if (!aborted) {
            // ---------------- transform warps: two threads per row of this CTA's 128, 32 columns each ----------------
            // Warp w works on tensor-memory lanes 32 * (w & 3) .. + 31 (the quarter a warp may access) and on columns
            // 32 * half .. + 31 of every 64-wide block (X1, S, dP, W and the accumulator alike), half = (w - 8) / 4.
            const int q = warp & 3, half = (warp - kAttXfWarp0) >> 2;
            const int rloc = q * 32 + lane;
            const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
            const uint32_t col_sel = 32u * (uint32_t)half;
            const uint32_t w_ready_l0 = mapa_shared(w_ready0, 0);
            const uint32_t x1_ready_l = mapa_shared(x1_ready, 0);
            const int hs = p.hs;
            // forward: the two threads of a row exchange their block maxima (and, at the end, their sums) here
            float* const exch = reinterpret_cast<float*>(smem_gen + Cfg::kBarOff + 512);   // [2 parities][2 halves][128 rows]
            bool got = true;
            uint32_t g = 0, ul = 0;
            // every lane polls (one warp-wide instruction per poll; no broadcast afterwards); the vote keeps the warp's
            // decision uniform should the limit run out for some lanes only
            auto wait_bar = [&](uint32_t bar, uint32_t ph, int slot) -> bool {
                const bool ok = ATT_PROF_WAIT(slot, mbar_wait_bounded_tight(bar, ph, p.wait_limit));
                return __all_sync(0xffffffffu, ok);
            };
            auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory"); };   // the two warps of a lane quarter
            ATT_PROF_T0
            // This thread's 32 columns of its row of X1 for unit `un`: global memory -> registers ...
            // (coalesced: lane l fetches float4 l % 8 of rows l / 8, l / 8 + 4, ..., i.e. four whole 128-byte rows per
            // instruction; the rows change hands in shared memory inside store_x1)
            float4* const stage = reinterpret_cast<float4*>(smem_gen + Cfg::kStageOff + (warp - kAttXfWarp0) * Cfg::kStageWarpBytes);
            float* const colstat = reinterpret_cast<float*>(smem_gen + Cfg::kColStatOff + (warp - kAttXfWarp0) * 256);
            constexpr int CH = Cfg::kStageRows;
            const int lr = lane >> 3, lc = lane & 7;
            auto load_x1 = [&](int un, float4 (&xr)[8]) {
                const AttnUnit dn = attn_unit<MODE>(p, un);
                const int row_w = dn.row0 + cta_rank * kRowsPerCta + q * 32;      // the warp's first row
                const float* src = p.x1 + (size_t)dn.b * p.stride_b + (size_t)dn.h * p.stride_h + (size_t)row_w * p.ld + 32 * half + 4 * lc;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = 4 * i + lr;
                    const bool have = row_w + r < p.T && 32 * half < hs;
                    xr[i] = have ? *reinterpret_cast<const float4*>(src + (size_t)r * p.ld) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            };
            // ... -> hi / lo -> tensor memory, and the MMA issuer is told.  Called once the first products of the previous
            // unit have completed (they read the old rows).
            auto store_x1 = [&](const float4 (&xf)[8]) {
                // rows change hands: written as fetched, read back by the thread that owns the row
                float4 xr[8];
#pragma unroll
                for (int ps = 0; ps < 32 / CH; ps++) {
#pragma unroll
                    for (int i = ps * (CH / 4); i < (ps + 1) * (CH / 4); i++) stage[(4 * i + lr - ps * CH) * 9 + lc] = xf[i];
                    __syncwarp();
                    if (lane / CH == ps) {
#pragma unroll
                        for (int j = 0; j < 8; j++) xr[j] = stage[(lane - ps * CH) * 9 + j];
                    }
                    __syncwarp();
                }
                uint32_t hi[32], lo[32];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    split_hi_lo(xr[i].x, hi[4 * i], lo[4 * i]);
                    split_hi_lo(xr[i].y, hi[4 * i + 1], lo[4 * i + 1]);
                    split_hi_lo(xr[i].z, hi[4 * i + 2], lo[4 * i + 2]);
                    split_hi_lo(xr[i].w, hi[4 * i + 3], lo[4 * i + 3]);
                }
                tmem_st_32x32(tmem_base + lane_sel + Cfg::kColXhi + col_sel, hi);
                tmem_st_32x32(tmem_base + lane_sel + Cfg::kColXlo + col_sel, lo);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(x1_ready_l);
            };
            if (unit_of(0) >= 0) {
                float4 xr[8];
                load_x1(unit_of(0), xr);
                store_x1(xr);
            }
            // After an expired wait (got = false) a warp keeps walking its blocks without touching barriers or tensor
            // memory, so that the pair_sync calls of the forward stay matched with its partner warp's.
            for (int k = 0, u; (u = unit_of(k)) >= 0; k++, ul++) {
                const AttnUnit d = attn_unit<MODE>(p, u);
                const int row = d.row0 + cta_rank * kRowsPerCta + rloc;       // absolute row inside the slice
                const bool row_ok = row < p.T;
                const size_t stat_off = (size_t)d.slice * p.T;
                float acc[32];
#pragma unroll
                for (int i = 0; i < 32; i++) acc[i] = 0.0f;
                float m_run = -CUDART_INF_F, l_run = 0.0f, corr_prev = 1.0f;   // forward
                float lse_r = 0.0f, d_r = 0.0f;                               // dQ: this row's statistics
                if (MODE == ATT_BWD_Q && row_ok) {
                    lse_r = p.lse[stat_off + row];
                    d_r = p.dvec[stat_off + row];
                }
                // adds this thread's 32 columns of block gb's accumulator into the registers
                auto drain = [&](uint32_t gb, float factor) -> bool {
                    const uint32_t wbuf = gb % NWB;
                    if (!wait_bar(acc_full0 + 8u * wbuf, (gb / NWB) & 1, 10)) return false;
                    ATT_PROF_MARK2(pd)
                    tc_fence_after();
                    float v[32];
                    tmem_ld_32x32(tmem_base + lane_sel + kColAcc + 64u * wbuf + col_sel, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        if (MODE == ATT_FWD) acc[i] = acc[i] * factor + v[i];
                        else acc[i] += v[i];
                    }
                    tc_fence_before();
                    __syncwarp();
                    ATT_PROF_ADD2(20, pd)
                    return true;
                };
                for (int c = 0; c < d.nb; c++, g++) {
                    const uint32_t buf = g & 1, wbuf = g % NWB;
                    const int col0 = (d.cb0 + c) * kColBlock + 32 * half;     // this thread's first column of the block
                    // last block of the unit: the next unit's X1 rows are fetched now and go to tensor memory as soon as this
                    // block's first products (the last readers of the old rows) are done, so that the MMA issuer can run on
                    const bool next_x1 = got && c == d.nb - 1 && unit_of(k + 1) >= 0;
                    float4 xn[8];
                    if (next_x1) load_x1(unit_of(k + 1), xn);
                    // dK, dV: this lane's column of the block's statistics, asked for before the wait so that the answer is
                    // there when the scores are
                    float st_l = 0.0f, st_d = 0.0f;
                    if ((MODE == ATT_BWD_K || MODE == ATT_BWD_V) && col0 + lane < p.T) {
                        st_l = p.lse[stat_off + col0 + lane];
                        if (MODE == ATT_BWD_K) st_d = p.dvec[stat_off + col0 + lane];
                    }
                    if (got) got = wait_bar(s_full0 + 8u * buf, (g >> 1) & 1, 9);
                    if (!got) {
                        if (MODE == ATT_FWD) pair_sync();
                        continue;
                    }
                    ATT_PROF_MARK2(pt)
#ifdef ZNN_ATTN_PROFILE
                    if (prof_on) { prof_acc[26] += clock64() - tstamp[g & 3]; prof_acc[28] += 1; }
#endif
                    tc_fence_after();
                    const uint32_t ts = tmem_base + lane_sel + kColS + 64u * buf + col_sel;
                    const uint32_t tl = tmem_base + lane_sel + kColWlo + 64u * wbuf + col_sel;
                    const uint32_t tdp = tmem_base + lane_sel + kColDp + 64u * buf + col_sel;
                    float corr = 1.0f;
                    float s[32], dp[32];
                    if (NX == 2) {
                        // both loads in flight, one wait
                        uint32_t rs[32], rd[32];
                        tmem_ld_32x32_issue(ts, rs);
                        tmem_ld_32x32_issue(tdp, rd);
                        tmem_ld_wait2(rs, rd);
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            s[j] = __uint_as_float(rs[j]);
                            dp[j] = __uint_as_float(rd[j]);
                        }
                    } else {
                        tmem_ld_32x32(ts, s);
                    }
                    ATT_PROF_ADD2(18, pt)
                    uint32_t hi[32], lo[32];
                    if (MODE == ATT_FWD) {
                        // m_run is kept in the scaled (base-2 exponent) domain; c2 > 0, so the maximum commutes with the scaling
                        const bool diag = col0 + 31 > d.row0 + cta_rank * kRowsPerCta + q * 32;   // warp-uniform: some element may be masked
                        if (diag) {
#pragma unroll
                            for (int j = 0; j < 32; j++) s[j] = (col0 + j <= row) ? s[j] : -CUDART_INF_F;
                        }
                        float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
                        for (int j = 4; j < 32; j++) m4[j & 3] = fmaxf(m4[j & 3], s[j]);
                        float mx = fmaxf(m_run, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.c2);
                        // the row's maximum over both halves of the block
                        float* const ex = exch + (g & 1) * 256;
                        ex[half * 128 + rloc] = mx;
                        pair_sync();
                        mx = fmaxf(mx, ex[(half ^ 1) * 128 + rloc]);
                        corr = fast_exp2(m_run - mx);
                        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float pv = fast_exp2(fmaf(s[j], p.c2, -mx));
                            s4[j & 3] += pv;
                            split_hi_lo(pv, hi[j], lo[j]);
                        }
                        l_run = l_run * corr + ((s4[0] + s4[1]) + (s4[2] + s4[3]));     // this thread's columns only; the halves are added at the end
                        m_run = mx;
                    } else if (MODE == ATT_BWD_V) {
                        // W = P^T: rows are keys, columns queries; statistics per column
                        colstat[lane] = st_l;
                        __syncwarp();
#pragma unroll
                        for (int j4 = 0; j4 < 8; j4++) {
                            const int qc = col0 + 4 * j4;
                            const float4 l4 = *reinterpret_cast<const float4*>(colstat + 4 * j4);
                            const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const int j = 4 * j4 + e;
                                const bool vis = (row <= qc + e) && (qc + e < p.T);
                                const float pv = vis ? fast_exp2(fmaf(s[j], p.c2, -ls[e])) : 0.0f;
                                split_hi_lo(pv, hi[j], lo[j]);
                            }
                        }
                    } else {
                        if (MODE == ATT_BWD_Q) {
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const bool vis = (col0 + j <= row);
                                const float pv = vis ? fast_exp2(fmaf(s[j], p.c2, -lse_r)) : 0.0f;
                                split_hi_lo((pv * (dp[j] - d_r)) * p.scale, hi[j], lo[j]);
                            }
                        } else {   // ATT_BWD_K
                            colstat[lane] = st_l;
                            colstat[32 + lane] = st_d;
                            __syncwarp();
#pragma unroll
                            for (int j4 = 0; j4 < 8; j4++) {
                                const int qc = col0 + 4 * j4;
                                const float4 l4 = *reinterpret_cast<const float4*>(colstat + 4 * j4);
                                const float4 d4 = *reinterpret_cast<const float4*>(colstat + 32 + 4 * j4);
                                const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                                for (int e = 0; e < 4; e++) {
                                    const int j = 4 * j4 + e;
                                    const bool vis = (row <= qc + e) && (qc + e < p.T);
                                    const float pv = vis ? fast_exp2(fmaf(s[j], p.c2, -ls[e])) : 0.0f;
                                    split_hi_lo((pv * (dp[j] - dd[e])) * p.scale, hi[j], lo[j]);
                                }
                            }
                        }
                    }
                    ATT_PROF_MARK2(ps)
                    tmem_st_32x32(ts, hi);
                    if (NWB == 1 && c >= 1) {
                        // one W_lo / accumulator buffer (dQ, dK): the previous block's second product must have finished reading
                        // W_lo before it is overwritten; its accumulator is drained at the same time
                        got = drain(g - 1, corr_prev);
                        if (!got) continue;
                    }
                    tmem_st_32x32(tl, lo);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
#ifdef ZNN_ATTN_PROFILE
                    if (prof_on) tstamp[4 + (g & 3)] = clock64();
#endif
                    if (lane == 0) mbar_arrive_remote(w_ready_l0 + 8u * buf);
                    ATT_PROF_ADD2(19, ps)
                    ATT_PROF_ADD2(21, pt)
                    // the next unit's rows go to tensor memory after this block's hand-off: the issuer needs the hand-off first
                    // (the last second product of this unit, whose result the unit's epilogue below waits for)
                    if (next_x1) store_x1(xn);
                    // two buffers: the previous block's second product has had this block's transform time to finish
                    if (NWB == 2 && c >= 1) got = drain(g - 1, corr_prev);
                    corr_prev = corr;
                }
                if (got) got = drain(g - 1, corr_prev);
                // ---- the rows leave: O = acc / l and the row's log-sum-exp, or the gradient rows ----
                float inv = 1.0f;
                if (MODE == ATT_FWD) {
                    float* const ex = exch + (g & 1) * 256;
                    ex[half * 128 + rloc] = l_run;
                    pair_sync();
                    const float l_all = l_run + ex[(half ^ 1) * 128 + rloc];
                    inv = 1.0f / l_all;
                    if (row_ok && got && half == 0) p.lse[stat_off + row] = m_run + log2f(l_all);
                    pair_sync();      // the slot may be rewritten by the next unit's first block (same parity)
                }
                // the rows leave through shared memory, four whole 128-byte rows per store instruction (a thread storing
                // its own row touches 32 different lines per instruction)
                if (32 * half < hs && __all_sync(0xffffffffu, got)) {
                    const int row_w = d.row0 + cta_rank * kRowsPerCta + q * 32;
                    float* const dst_w = p.out + (size_t)d.b * p.stride_b + (size_t)d.h * p.stride_h + (size_t)row_w * p.ld + 32 * half + 4 * lc;
#pragma unroll
                    for (int ps = 0; ps < 32 / CH; ps++) {
                        if (lane / CH == ps) {
#pragma unroll
                            for (int j = 0; j < 8; j++)
                                stage[(lane - ps * CH) * 9 + j] = make_float4(acc[4 * j] * inv, acc[4 * j + 1] * inv, acc[4 * j + 2] * inv, acc[4 * j + 3] * inv);
                        }
                        __syncwarp();
#pragma unroll
                        for (int i = ps * (CH / 4); i < (ps + 1) * (CH / 4); i++) {
                            const int r = 4 * i + lr;
                            if (row_w + r >= p.T) continue;
                            float4 o = stage[(r - ps * CH) * 9 + lc];
                            float* const dst = dst_w + (size_t)r * p.ld;
                            if (MODE != ATT_FWD && p.accumulate) {
                                const float4 old = *reinterpret_cast<const float4*>(dst);
                                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                            }
                            *reinterpret_cast<float4*>(dst) = o;
                        }
                        __syncwarp();
                    }
                }
            }
            if (!got && lane == 0) atomicOr(p.status, ZNN_DEV_EPI_WAIT_EXPIRED);
            ATT_PROF_END(8)
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<2>(tmem_base, 512);
    }
}

// D[s, t] = sum_d dO[s, t, d] * O[s, t, d]  (= rowsum(dP o P) of the softmax backward): hs / 4 lanes per row
__global__ void attn_rowdot_kernel(const float* __restrict__ dO, const float* __restrict__ O, float* __restrict__ D, int nslices,
                                   int nh, int T, int hs, long long ld, long long stride_h, long long stride_b)
{
    const int lpr = hs >> 2;                            // lanes per row (8 or 16)
    const int rows_per_warp = 32 / lpr;
    const size_t warp_id = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const size_t r = warp_id * rows_per_warp + lane / lpr;
    const bool ok = r < (size_t)nslices * T;
    float s = 0.0f;
    if (ok) {
        const int slice = (int)(r / T), t = (int)(r - (size_t)slice * T);
        const int b = slice / nh, h = slice - b * nh;
        const size_t off = (size_t)b * stride_b + (size_t)h * stride_h + (size_t)t * ld + 4 * (lane % lpr);
        const float4 a = *reinterpret_cast<const float4*>(dO + off), o = *reinterpret_cast<const float4*>(O + off);
        s = (a.x * o.x + a.y * o.y) + (a.z * o.z + a.w * o.w);
    }
    for (int o = lpr >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (ok && (lane % lpr) == 0) D[r] = s;
}

// Remainder planes: dst_i[j] = src_i[j] - (src_i[j] with the 13 low mantissa bits cleared), over the whole extent of up to
// four tensors (blockIdx.y picks one).  The tensor core takes the values themselves as the TF32 heads (it ignores the low
// bits), so a 3xTF32 operand that comes straight from TMA needs only this second plane.
struct AttnLoArgs {
    const float4* src[4];
    float4* dst[4];
};
__global__ void attn_lo_kernel(const AttnLoArgs a, size_t n4)
{
    const float4* __restrict__ src = a.src[blockIdx.y];
    float4* __restrict__ dst = a.dst[blockIdx.y];
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 x = src[i];
        float4 l;
        l.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
        l.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
        l.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
        l.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
        dst[i] = l;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn4)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn4 attn_encode_fn()
{
    static EncodeTiledFn4 fn = nullptr;
    if (!fn) {
        void* q = nullptr;
        cudaDriverEntryPointQueryResult r;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess && r == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn4)q;
    }
    return fn;
}

struct AttnLayout {
    int B, nh, T, hs;
    long long ld, stride_h, stride_b;
    bool t_first;
};

// box_rows > 0: K-major tile of box_rows rows x 32 floats (128-byte swizzle); box_rows == 0: MN-major 32 x 32 box
static int make_attn_map(CUtensorMap* tm, const float* X, const AttnLayout& L, int box_rows)
{
    EncodeTiledFn4 enc = attn_encode_fn();
    if (!enc) return fail(ZNN_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    const cuuint32_t rows = box_rows > 0 ? (cuuint32_t)box_rows : 32u;
    cuuint64_t dims[4], strides[3];
    cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
    dims[0] = (cuuint64_t)L.hs;
    box[0] = 32;
    if (L.t_first) {
        dims[1] = (cuuint64_t)L.T; dims[2] = (cuuint64_t)L.nh;
        strides[0] = (cuuint64_t)L.ld * 4; strides[1] = (cuuint64_t)L.stride_h * 4;
        box[1] = rows; box[2] = 1;
    } else {
        dims[1] = (cuuint64_t)L.nh; dims[2] = (cuuint64_t)L.T;
        strides[0] = (cuuint64_t)L.stride_h * 4; strides[1] = (cuuint64_t)L.ld * 4;
        box[1] = 1; box[2] = rows;
    }
    dims[3] = (cuuint64_t)L.B;
    strides[2] = (cuuint64_t)L.stride_b * 4;
    box[3] = 1;
    const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(X), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE,
                           box_rows > 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ZNN_ERR_CUDA, "cuTensorMapEncodeTiled (attention operand) failed with %d", (int)r);
    return ZNN_OK;
}

static thread_local int t_attn_in_order = 0;
static thread_local int t_attn_sched = 1;     // 0: no schedule tables (units dealt to the pairs by arithmetic)
unsigned long long tc_wait_limit();

int attn_profile_read(long long* out32)
{
    ZNN_CUDA_OK(cudaMemcpyFromSymbol(out32, g_attn_prof, 32 * sizeof(long long)));
    long long zero[32] = {0};
    ZNN_CUDA_OK(cudaMemcpyToSymbol(g_attn_prof, zero, sizeof(zero)));
    return ZNN_OK;
}

// X2l, Y1l, Y2l, Zl: the remainder planes of X2, Y1, Y2, Z (same layout), or all NULL: the kernel then converts in place
// Schedule table of one problem shape on one device: units (numbered dearest first, as attn_unit counts them) dealt to the
// CTA pairs by "longest job to the least loaded pair"; a unit costs its blocks plus about two blocks' worth of time for
// the change of unit.  Tables are made once per shape and stay on the device (a few hundred bytes each); a shape first
// met while the stream is being captured runs without one (the allocation and the copy are not stream operations).
struct AttnSchedKey {
    int dev, rows_first, nslices, nrb, ncb, T, pairs;
    bool operator<(const AttnSchedKey& o) const
    {
        return std::tie(dev, rows_first, nslices, nrb, ncb, T, pairs) < std::tie(o.dev, o.rows_first, o.nslices, o.nrb, o.ncb, o.T, o.pairs);
    }
};
struct AttnSched { const int* table; int k; };

// blocks of unit u (units numbered dearest first, as attn_unit counts them)
static int attn_unit_blocks(bool rows_first, int nslices, int nrb, int ncb, int T, long u)
{
    const int rbi = (int)(u / nslices);
    if (rows_first) {            // forward, dQ: rows are queries, the blocks run up to the diagonal
        const int rb = nrb - 1 - rbi;
        const int last = std::min(T, rb * 256 + 256);
        return (last + kColBlock - 1) / kColBlock;
    }
    return ncb - rbi * 256 / kColBlock;     // dK, dV: rows are keys, the blocks run from the diagonal to the end
}

// The units of every pair, in the order the pair takes them (host arithmetic only).
static std::vector<std::vector<int>> attn_plan(bool rows_first, int nslices, int nrb, int ncb, int T, int pairs)
{
    const long total = (long)nslices * nrb;
    std::vector<std::vector<int>> rows(pairs);
    std::vector<double> load(pairs, 0.0);
    for (long u = 0; u < total; u++) {
        int best = 0;
        for (int i = 1; i < pairs; i++)
            if (load[i] < load[best]) best = i;
        load[best] += attn_unit_blocks(rows_first, nslices, nrb, ncb, T, u) + 2.0;
        rows[best].push_back((int)u);
    }
    return rows;
}

static AttnSched attn_schedule(int dev, bool rows_first, const AttnParams& p, int pairs)
{
    static std::mutex mu;
    static std::map<AttnSchedKey, AttnSched> cache;
    const AttnSchedKey key = {dev, rows_first ? 1 : 0, p.nslices, p.nrb, p.ncb, p.T, pairs};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    AttnSched none = {nullptr, 0};
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream(), &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return none;
    }
    const std::vector<std::vector<int>> rows = attn_plan(rows_first, p.nslices, p.nrb, p.ncb, p.T, pairs);
    size_t k = 0;
    for (const auto& r : rows) k = std::max(k, r.size());
    if (k > (size_t)kAttSchedMax) { cache[key] = none; return none; }
    std::vector<int> flat((size_t)pairs * k, -1);
    for (int i = 0; i < pairs; i++) std::copy(rows[i].begin(), rows[i].end(), flat.begin() + (size_t)i * k);
    int* d = nullptr;
    if (cudaMalloc(&d, flat.size() * sizeof(int)) != cudaSuccess ||
        cudaMemcpy(d, flat.data(), flat.size() * sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        if (d) cudaFree(d);
        return none;       // not cached: the next call tries again
    }
    const AttnSched made = {d, (int)k};
    cache[key] = made;
    return made;
}

template <int MODE>
static int launch_attn(const float* X1, const float* X2, const float* Y1, const float* Y2, const float* Z, const AttnLayout& L,
                       AttnParams p, const float* X2l = nullptr, const float* Y1l = nullptr, const float* Y2l = nullptr,
                       const float* Zl = nullptr)
{
    using Cfg = AttnCfg<MODE>;
    auto kern = attn_kernel<MODE>;
    static bool attr_set[64] = {false};
    static int pairs_by_device[64] = {0};
    int dev = 0;
    ZNN_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(ZNN_ERR_INVALID, "device index %d out of range", dev);
    if (!attr_set[dev]) {
        ZNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[dev] = true;
    }
    CUtensorMap mx2, my1, my2, mz;
    int rc;
    p.x1 = X1;
    if ((rc = make_attn_map(&mx2, X2 ? X2 : X1, L, kRowsPerCta))) return rc;
    if ((rc = make_attn_map(&my1, Y1, L, 32))) return rc;
    if ((rc = make_attn_map(&my2, Y2 ? Y2 : Y1, L, 32))) return rc;
    if ((rc = make_attn_map(&mz, Z, L, 0))) return rc;
    CUtensorMap mx2l = mx2, my1l = my1, my2l = my2, mzl = mz;
    p.planes = (Y1l && Zl) ? 1 : 0;
    if (p.planes) {
        if ((rc = make_attn_map(&mx2l, X2l ? X2l : Y1l, L, kRowsPerCta))) return rc;
        if ((rc = make_attn_map(&my1l, Y1l, L, 32))) return rc;
        if ((rc = make_attn_map(&my2l, Y2l ? Y2l : Y1l, L, 32))) return rc;
        if ((rc = make_attn_map(&mzl, Zl, L, 0))) return rc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kAttThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (pairs_by_device[dev] == 0) {
        cfg.gridDim = dim3((unsigned)sm_count(), 1, 1);
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters < 1) {
            cudaGetLastError();
            clusters = sm_count() / 2;
        }
        pairs_by_device[dev] = clusters;
    }
    const long units = (long)p.nslices * p.nrb;
    const long pairs = units < pairs_by_device[dev] ? units : pairs_by_device[dev];
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    if (units > pairs && t_attn_sched) {       // (with a pair per unit there is nothing to deal)
        const AttnSched sc = attn_schedule(dev, MODE == ATT_FWD || MODE == ATT_BWD_Q, p, (int)pairs);
        p.sched = sc.table;
        p.sched_k = sc.k;
    }
    ZNN_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, mx2, my1, my2, mz, mx2l, my1l, my2l, mzl, p));
    count_launch();
    if (inject_launch_failure()) return fail(ZNN_ERR_CUDA, "launch of the attention kernel failed: injected failure (znn_debug_fail_after)");
    return ZNN_OK;
}

static int attn_check(const void* const* ptrs, int nptr, int B, int nh, int T, int hs, long long ld, long long stride_h,
                      long long stride_b, AttnLayout* L)
{
    ZNN_REQUIRE(B > 0 && nh > 0 && T > 0, "empty attention problem");
    if (!(hs == 32 || hs == 64)) return fail(ZNN_ERR_UNSUPPORTED, "fused attention: head size %d (32 or 64 supported)", hs);
    if (T % 4 != 0) return fail(ZNN_ERR_UNSUPPORTED, "fused attention: T = %d is not a multiple of 4", T);
    if ((ld & 3) || (stride_h & 3) || (stride_b & 3) || ld < hs)
        return fail(ZNN_ERR_UNSUPPORTED, "fused attention: row pitch and strides must be multiples of 4 floats");
    for (int i = 0; i < nptr; i++) {
        ZNN_REQUIRE(ptrs[i], "NULL pointer");
        if (reinterpret_cast<uintptr_t>(ptrs[i]) & 15) return fail(ZNN_ERR_UNSUPPORTED, "fused attention: pointers must be 16-byte aligned");
    }
    if ((long long)B * nh > 0x3fffffLL) return fail(ZNN_ERR_INVALID, "too many (batch, head) slices");
    L->B = B; L->nh = nh; L->T = T; L->hs = hs;
    L->ld = ld; L->stride_h = stride_h; L->stride_b = stride_b;
    L->t_first = (ld <= stride_h);   // tensor-map dimensions in order of ascending stride
    return ZNN_OK;
}

static AttnParams attn_params(const AttnLayout& L, float scale)
{
    AttnParams p;
    p.T = L.T; p.hs = L.hs; p.nh = L.nh; p.nslices = L.B * L.nh;
    p.nrb = (L.T + 255) / 256;
    p.ncb = (L.T + kColBlock - 1) / kColBlock;
    p.t_first = L.t_first ? 1 : 0;
    p.scale = scale;
    p.c2 = scale * 1.4426950408889634f;
    p.ld = L.ld; p.stride_h = L.stride_h; p.stride_b = L.stride_b;
    p.x1 = nullptr; p.out = nullptr; p.lse = nullptr; p.dvec = nullptr;
    p.accumulate = 0;
    p.planes = 0;
    p.issue_in_order = t_attn_in_order;
    p.sched = nullptr;
    p.sched_k = 0;
    p.status = device_status_word();
    p.wait_limit = tc_wait_limit();
    return p;
}

void attn_set_issue_order(int in_order) { t_attn_in_order = in_order ? 1 : 0; }
static thread_local int t_attn_planes = 0;   // measured: no faster than the converter warps, and the pre-pass costs 16-32 us per call
void attn_set_planes(int on) { t_attn_planes = on ? 1 : 0; }

// Remainder planes of n (<= 4) tensors of layout L in scratch slot 1; dst[i] receives the plane of src[i].
static int attn_make_lo_planes(const AttnLayout& L, int n, const float* const* src, const float** dst)
{
    const size_t span = (size_t)(L.B - 1) * L.stride_b + (size_t)(L.nh - 1) * L.stride_h + (size_t)(L.T - 1) * L.ld + L.hs;
    const size_t span4 = (span + 3) / 4;            // (strides and hs are multiples of 4, so span is)
    float* base = (float*)workspace_slot(1, (size_t)n * span4 * 4 * sizeof(float));
    if (!base) return fail(ZNN_ERR_NOMEM, "scratch for the attention operands' remainder planes");
    AttnLoArgs a{};
    for (int i = 0; i < n; i++) {
        a.src[i] = reinterpret_cast<const float4*>(src[i]);
        a.dst[i] = reinterpret_cast<float4*>(base + (size_t)i * span4 * 4);
        dst[i] = base + (size_t)i * span4 * 4;
    }
    size_t blocks = (span4 + 255) / 256;
    const size_t cap = (size_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    attn_lo_kernel<<<dim3((unsigned)blocks, (unsigned)n), 256, 0, stream()>>>(a, span4);
    ZNN_LAUNCH_OK("attn_lo_kernel");
    return ZNN_OK;
}

}  // namespace znn

using namespace znn;

extern "C" {

int znn_debug_set_attn_planes(int enable)
{
    attn_set_planes(enable);
    return ZNN_OK;
}

int znn_debug_attn_plan(int rows_first, int nslices, int T, int pairs, int table_form, int* units_per_pair, int* blocks_per_pair)
{
    ZNN_REQUIRE(nslices > 0 && T > 0 && pairs > 0 && units_per_pair && blocks_per_pair, "bad argument");
    const int nrb = (T + 255) / 256, ncb = (T + kColBlock - 1) / kColBlock;
    const long total = (long)nslices * nrb;
    for (int i = 0; i < pairs; i++) units_per_pair[i] = blocks_per_pair[i] = 0;
    if (table_form) {
        const std::vector<std::vector<int>> rows = attn_plan(rows_first != 0, nslices, nrb, ncb, T, pairs);
        std::vector<char> seen((size_t)total, 0);
        for (int i = 0; i < pairs; i++)
            for (int u : rows[i]) {
                if (u < 0 || u >= total || seen[u]) return fail(ZNN_ERR_INVALID, "the plan names unit %d twice or out of range", u);
                seen[u] = 1;
                units_per_pair[i]++;
                blocks_per_pair[i] += attn_unit_blocks(rows_first != 0, nslices, nrb, ncb, T, u);
            }
        for (long u = 0; u < total; u++)
            if (!seen[u]) return fail(ZNN_ERR_INVALID, "the plan leaves out unit %ld", u);
    } else {
        // the kernel's own dealing: round k gives units k * pairs .. to the pairs in alternating direction
        for (int i = 0; i < pairs; i++)
            for (long k = 0;; k++) {
                const long u = k * pairs + ((k & 1) ? pairs - 1 - i : i);
                if (u >= total) break;
                units_per_pair[i]++;
                blocks_per_pair[i] += attn_unit_blocks(rows_first != 0, nslices, nrb, ncb, T, u);
            }
    }
    return ZNN_OK;
}

int znn_debug_set_attn_schedule(int enable)
{
    t_attn_sched = enable ? 1 : 0;
    return ZNN_OK;
}

int znn_debug_set_attn_issue_order(int in_order)
{
    attn_set_issue_order(in_order);
    return ZNN_OK;
}

int znn_debug_attn_profile(long long* out32)
{
    ZNN_REQUIRE(out32, "out32 is NULL");
    return attn_profile_read(out32);
}

int znn_attn_fwd(const float* Q, const float* K, const float* V, float* O, float* LSE, int B, int nh, int T, int hs,
                 long long ld, long long stride_h, long long stride_b, float scale)
{
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (this library has no CPU fallback)");
    AttnLayout L;
    const void* ptrs[5] = {Q, K, V, O, LSE};
    int rc = attn_check(ptrs, 5, B, nh, T, hs, ld, stride_h, stride_b, &L);
    if (rc) return rc;
    AttnParams p = attn_params(L, scale);
    if (!p.status) return fail(ZNN_ERR_CUDA, "no device state (call znn_init first)");
    p.out = O;
    p.lse = LSE;
    if (t_attn_planes) {
        const float* src[2] = {K, V};
        const float* lo[2] = {nullptr, nullptr};
        if ((rc = attn_make_lo_planes(L, 2, src, lo))) return rc;
        return launch_attn<ATT_FWD>(Q, nullptr, K, nullptr, V, L, p, nullptr, lo[0], nullptr, lo[1]);
    }
    return launch_attn<ATT_FWD>(Q, nullptr, K, nullptr, V, L, p);
}

int znn_attn_bwd(const float* Q, const float* K, const float* V, const float* O, const float* dO, const float* LSE, float* dQ,
                 float* dK, float* dV, int B, int nh, int T, int hs, long long ld, long long stride_h, long long stride_b,
                 float scale, int accumulate)
{
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (this library has no CPU fallback)");
    AttnLayout L;
    const void* ptrs[6] = {Q, K, V, O, dO, LSE};
    int rc = attn_check(ptrs, 6, B, nh, T, hs, ld, stride_h, stride_b, &L);
    if (rc) return rc;
    const void* grads[3] = {dQ, dK, dV};
    for (const void* g : grads)
        if (g && (reinterpret_cast<uintptr_t>(g) & 15)) return fail(ZNN_ERR_UNSUPPORTED, "fused attention: pointers must be 16-byte aligned");
    AttnParams p = attn_params(L, scale);
    if (!p.status) return fail(ZNN_ERR_CUDA, "no device state (call znn_init first)");
    p.accumulate = accumulate ? 1 : 0;
    p.lse = const_cast<float*>(LSE);
    if (dQ || dK) {
        const size_t rows = (size_t)p.nslices * T;
        float* D = (float*)workspace(rows * sizeof(float));
        if (!D) return fail(ZNN_ERR_NOMEM, "scratch for the attention row sums");
        const int rows_per_block = 256 / (hs / 4);
        attn_rowdot_kernel<<<(unsigned)((rows + rows_per_block - 1) / rows_per_block), 256, 0, stream()>>>(
            dO, O, D, p.nslices, nh, T, hs, ld, stride_h, stride_b);
        ZNN_LAUNCH_OK("attn_rowdot_kernel");
        p.dvec = D;
    }
    const float* lo[4] = {nullptr, nullptr, nullptr, nullptr};   // remainder planes of Q, K, V, dO
    if (t_attn_planes) {
        const float* src[4] = {Q, K, V, dO};
        if ((rc = attn_make_lo_planes(L, 4, src, lo))) return rc;
    }
    const float *Ql = lo[0], *Kl = lo[1], *Vl = lo[2], *dOl = lo[3];
    if (dQ) {
        p.out = dQ;
        if ((rc = launch_attn<ATT_BWD_Q>(Q, dO, K, V, K, L, p, dOl, Kl, Vl, Kl))) return rc;
    }
    if (dK) {
        p.out = dK;
        if ((rc = launch_attn<ATT_BWD_K>(K, V, Q, dO, Q, L, p, Vl, Ql, dOl, Ql))) return rc;
    }
    if (dV) {
        p.out = dV;
        if ((rc = launch_attn<ATT_BWD_V>(K, nullptr, Q, nullptr, dO, L, p, nullptr, Ql, nullptr, dOl))) return rc;
    }
    return ZNN_OK;
}

}  // extern "C"
