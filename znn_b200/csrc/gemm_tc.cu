// fp32-accurate GEMM on the 5th-generation tensor cores (sm_100a).
//
//   C[M,N] = alpha * op(A) * op(B) + beta * C        (row-major, fp32)
//
// Each product is three tcgen05.mma.kind::tf32 passes over a hi/lo split of the operands (lo*hi, hi*lo, hi*hi;
// lo*lo is below fp32 resolution), accumulated in fp32 in tensor memory in chunks of 256 contraction elements that
// the epilogue warps add up in registers (the tensor core's accumulator truncates).  Two kernels:
//
//  * gemm3x_direct_kernel (the default): TMA reads the caller's matrices in place, K-major or MN-major; converter
//    warps write the lo plane next to each landed tile; CTA pairs (cta_group::2) on 256 x BN tiles; persistent (one
//    pair per SM pair walks the tiles, the epilogue of one tile overlaps the main loop of the next); optional
//    split-K, tail split of a thin last round, triangular-structure hints, fused bias and softmax-backward epilogues.
//  * gemm3x_tf32_kernel (operands the TMA cannot read in place: unaligned bases or leading dimensions): a split
//    pre-pass rewrites op(A) and op(B) as K-major hi/lo planes in scratch, then one CTA or a CTA pair per tile.
//
// No TMA multicast anywhere (each CTA loads its own half of A and B).  Every mbarrier wait is bounded: on expiry the
// role sets a bit in the device status word and leaves; later CTAs and kernels see the word and return at once.
#include <cuda.h>

#include <stdlib.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace znn {

// ---------------------------------------------------------------------------
// the GEMM kernel
// ---------------------------------------------------------------------------
struct GemmTcParams {
    int M, N;            // output extent
    int k_blocks;        // padded K / 32
    int k_real;          // the caller's K (for flop accounting only)
    int chunk_kblocks;   // k-blocks accumulated inside tensor memory before promotion
    int kblocks_per_split;  // split-K: k-blocks handled by one blockIdx.y slice (== k_blocks when not split)
    float* partial;      // split-K: [splits][batch][M][N] partial sums, nullptr when not split
    int conv_mode;       // direct kernel: 0 = store the masked hi tile, 1 = leave the raw tile as hi
    const float* bias;   // optional [N] vector added to every output row (fused AddBias), may be nullptr
    int tiles_m, tiles_n;
    int splits, batch;   // in-place kernel: work units = tiles_m * tiles_n * splits * batch
    int tri;             // in-place kernel: triangular structure hint (ZNN_TRI_*), 0 = none; never combined with split-K
    // in-place kernel, tail split: work units from tail_first on are the tiles of the last, partly filled round of the
    // persistent walk, each cut into tail_slices K-slices of tail_kbps k-blocks whose raw 256 x BN partial tiles go to
    // tail_partial[unit - tail_first]; a small kernel adds the slices in order.  tail_first = number of units when off.
    int tail_first, tail_slices, tail_kbps;
    float* tail_partial;
    // in-place kernel, softmax-backward epilogue: C = alpha * P o (A.B - d[row]) with P laid out like C (ldc, stride_c)
    // and d one float per row and batch slice; nullptr = the ordinary epilogue
    const float* ep_p;
    const float* ep_d;
    // in-place kernel, activation / residual epilogue (batch 1, 16-byte form; all laid out like C):
    //   ep_act 1 = ReLU, 2 = GELU: C = act(h) with h = alpha * A.B + bias (+ ep_res); ep_out2 (optional) receives h;
    //   ep_act 3 = ReLU', 4 = GELU': C = (alpha * A.B) o act'(ep_dpre) + beta * C  (the gradient of the layer below);
    //   ep_act 0 with ep_res: C = alpha * A.B + bias + ep_res (residual connection).
    int ep_act;
    float* ep_out2;
    const float* ep_res;
    const float* ep_dpre;
    // in-place kernel, grouped products: an operand shared by all slices (batch stride 0: its tensor map has one slice),
    // a bias row per slice, and K-concatenation: kcat_segs > 1 makes the `kcat_segs` slices of A and B one product whose
    // contraction runs through the slices one after the other (k-block kb lies in slice kb / kcat_kb), into one C.
    int a_bcast, b_bcast;
    long long stride_bias;
    int kcat_segs, kcat_kb;
    // in-place kernel, triangular hint: the tiles of one slice that have work, dearest first (tile_m << 8 | tile_n);
    // units are then (table entry, slice) with the slice running fastest, so that the walk deals every CTA pair the
    // same mix of dear and cheap tiles.  tri_n = 0: no table (more than 64 tiles per slice), plain order.
    int tri_n;
    unsigned short tri_tab[64], tri_kf[64], tri_kc[64];   // tile code, first k-block, k-block count per entry
    float alpha, beta;
    float* C;
    long long ldc, stride_c;
    int* status;
    unsigned long long wait_limit;   // SM cycles a role waits on an mbarrier before it gives up (znn_debug_set_wait_limit)
};

constexpr int kBK = 32;          // fp32 elements per k-block = one 128-byte swizzle row
constexpr int kTileM = 128;      // rows of A per CTA
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;  // warp 0 TMA, warp 1 MMA + TMEM, warps 2..9 epilogue

template <int BN, int CTAS>
struct TcCfg {
    static constexpr int kBRows = BN / CTAS;                   // rows of B this CTA loads
    static constexpr int kABytes = kTileM * kBK * 4;           // one A plane tile
    static constexpr int kBBytes = kBRows * kBK * 4;           // one B plane tile
    static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
    static constexpr int kStages = (200 * 1024) / kStageBytes > 6 ? 6 : (200 * 1024) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulator buffers
    static constexpr int kColsPerThread = BN / 2;                // each epilogue warp owns a lane quarter x column half
};



// Final store of one epilogue warp's 32 x CPT sub-tile.  Each thread holds one row in registers; a store straight
// from there would write 16 bytes per row per instruction.  The sub-tile is turned through shared memory (the
// operand ring is idle by now) so that every instruction moves one contiguous run of a row: 512 bytes for CPT = 128.
template <int CPT>
__device__ __forceinline__ void epilogue_store_warp(const float (&acc)[CPT], float* stage, int lane, int row_base, int cbase,
                                                    int M, int N, float* out, long long out_ld, float alpha, float beta,
                                                    const float* bias, bool vec_ok)
{
    constexpr int PITCH = CPT + 4;  // floats; keeps the 16-byte row writes of a quarter warp in distinct banks
#pragma unroll
    for (int c = 0; c < CPT; c += 4)
        *reinterpret_cast<float4*>(stage + lane * PITCH + c) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
    __syncwarp();
    const int rows = min(32, M - row_base);
    constexpr int RB = 8;  // rows in flight: the loads of old C (beta != 0) are issued together
    for (int r0 = 0; r0 < rows; r0 += RB) {
        for (int c4 = lane; c4 < CPT / 4; c4 += 32) {
            const int col = cbase + 4 * c4;
            if (col >= N) continue;
            const bool full = vec_ok && (col + 3 < N);
            float4 old[RB];
            if (beta != 0.0f && full) {
#pragma unroll
                for (int u = 0; u < RB; u++)
                    if (r0 + u < rows) old[u] = *reinterpret_cast<const float4*>(out + (size_t)(row_base + r0 + u) * out_ld + col);
            }
            float4 b4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (bias && full) b4 = *reinterpret_cast<const float4*>(bias + col);
#pragma unroll
            for (int u = 0; u < RB; u++) {
                if (r0 + u >= rows) continue;
                float* crow = out + (size_t)(row_base + r0 + u) * out_ld;
                const float4 v = *reinterpret_cast<const float4*>(stage + (r0 + u) * PITCH + 4 * c4);
                float o[4] = {alpha * v.x, alpha * v.y, alpha * v.z, alpha * v.w};
                if (full) {
                    o[0] += b4.x; o[1] += b4.y; o[2] += b4.z; o[3] += b4.w;
                    if (beta != 0.0f) {
                        o[0] += beta * old[u].x; o[1] += beta * old[u].y; o[2] += beta * old[u].z; o[3] += beta * old[u].w;
                    }
                    *reinterpret_cast<float4*>(crow + col) = make_float4(o[0], o[1], o[2], o[3]);
                } else {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if (col + e < N) {
                            float t = o[e];
                            if (bias) t += bias[col + e];
                            if (beta != 0.0f) t += beta * crow[col + e];
                            crow[col + e] = t;
                        }
                    }
                }
            }
        }
    }
}

// The tensor core adds into its fp32 accumulator with truncation, so the error of
// a long accumulation grows linearly with K (measured: 7e-6 relative at K = 1024,
// 5.7e-5 at K = 8192).  The k-loop is therefore cut into chunks of
// `chunk_kblocks` k-blocks: each chunk accumulates in one of two tensor-memory
// buffers, and the epilogue warps add finished chunks into fp32 registers with
// round-to-nearest while the next chunk is being multiplied.
template <int BN, int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
gemm3x_tf32_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
                   const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
                   const GemmTcParams p)
{
    using Cfg = TcCfg<BN, CTAS>;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment is required by the 128-byte swizzle atoms.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + Cfg::kStages * Cfg::kStageBytes;
    // barrier block: full[kStages], empty[kStages], acc_full[2], acc_empty[2], then two words
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + 2 + b); };
    constexpr int kWordOff = 8 * (2 * Cfg::kStages + 4);
    volatile uint32_t* tmem_slot =
        reinterpret_cast<volatile uint32_t*>(smem_gen + Cfg::kStages * Cfg::kStageBytes + kWordOff);
    const uint32_t tmem_slot_addr = bar_base + kWordOff;
    volatile uint32_t* abort_slot = tmem_slot + 1;
    const uint32_t abort_slot_addr = tmem_slot_addr + 4;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
    const bool leader = (cta_rank == 0);

    // tile coordinates: groups of 8 tile-rows are walked column by column so
    // that CTAs running together share A row panels and B column panels in L2
    const int unit = (CTAS == 2) ? (blockIdx.x >> 1) : blockIdx.x;
    int tile_m, tile_n;
    {
        constexpr int G = 8;
        const int per_group = G * p.tiles_n;
        const int g = unit / per_group;
        const int first_m = g * G;
        const int rows_in_group = min(G, p.tiles_m - first_m);
        const int r = unit - g * per_group;
        tile_m = first_m + r % rows_in_group;
        tile_n = r / rows_in_group;
    }
    const int batch = blockIdx.z;
    const int row0 = (tile_m * CTAS + (int)cta_rank) * kTileM;  // first C / A row of this CTA
    const int col0 = tile_n * BN;
    const int chunk = p.chunk_kblocks;
    // split-K: this CTA (pair) contracts k-blocks [kb_first, kb_first + kb_count)
    const int kb_first = (int)blockIdx.y * p.kblocks_per_split;
    const int kb_count = min(p.k_blocks - kb_first, p.kblocks_per_split);
    const int nchunks = (kb_count + chunk - 1) / chunk;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), kEpiWarps * CTAS);  // every epilogue warp of the tile's CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // A failure recorded by an earlier CTA or kernel makes this one do nothing.
        // One thread decides for the whole CTA (pair), so the decision is uniform.
        if (leader) {
            const uint32_t prior = (uint32_t)(*reinterpret_cast<volatile int*>(p.status));
            *abort_slot = prior;
            if (CTAS == 2)
                asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(mapa_shared(abort_slot_addr, 1)), "r"(prior) : "memory");
        }
    }
    if (warp == 1) {
        tmem_alloc<CTAS>(tmem_slot_addr, Cfg::kTmemCols);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();  // the peer's barriers must exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool aborted = (*abort_slot != 0);

    bool ok = true;
    if (aborted) {
        // nothing to do: fall through to the teardown
    } else if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const uint32_t full_leader0 = (CTAS == 2) ? mapa_shared(full_bar(0), 0) : full_bar(0);
            for (int kb = 0; kb < kb_count; kb++) {
                const int s = kb % Cfg::kStages;
                const uint32_t ph = (kb / Cfg::kStages) & 1;
                if (!mbar_wait_bounded(empty_bar(s), ph ^ 1, p.wait_limit)) { ok = false; break; }
                const uint32_t st = smem_base + s * Cfg::kStageBytes;
                const int k0 = (kb_first + kb) * kBK;
                if (CTAS == 1) {
                    mbar_arrive_expect_tx(full_bar(s), Cfg::kStageBytes);
                    tma_load_3d(st, &tm_a_hi, full_bar(s), k0, row0, batch);
                    tma_load_3d(st + Cfg::kABytes, &tm_a_lo, full_bar(s), k0, row0, batch);
                    tma_load_3d(st + 2 * Cfg::kABytes, &tm_b_hi, full_bar(s), k0, col0, batch);
                    tma_load_3d(st + 2 * Cfg::kABytes + Cfg::kBBytes, &tm_b_lo, full_bar(s), k0, col0, batch);
                } else {
                    // the leader's barrier collects the bytes of both CTAs
                    if (leader) mbar_arrive_expect_tx(full_bar(s), 2 * Cfg::kStageBytes);
                    const uint32_t fb = full_leader0 + 8u * s;
                    const int brow0 = col0 + (int)cta_rank * Cfg::kBRows;
                    tma_load_3d_pair(st, &tm_a_hi, fb, k0, row0, batch);
                    tma_load_3d_pair(st + Cfg::kABytes, &tm_a_lo, fb, k0, row0, batch);
                    tma_load_3d_pair(st + 2 * Cfg::kABytes, &tm_b_hi, fb, k0, brow0, batch);
                    tma_load_3d_pair(st + 2 * Cfg::kABytes + Cfg::kBBytes, &tm_b_lo, fb, k0, brow0, batch);
                }
            }
            if (!ok) atomicOr(p.status, ZNN_DEV_TMA_WAIT_EXPIRED);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only in pair mode) ----------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_tf32_idesc(kTileM * CTAS, BN);
            int kb = 0;
            for (int c = 0; c < nchunks && ok; c++) {
                const int buf = c & 1;
                // the epilogue warps must have drained this buffer (two chunks ago)
                if (!mbar_wait_bounded(acc_empty_bar(buf), ((c >> 1) & 1) ^ 1, p.wait_limit)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                const int kb_end = min(kb_count, kb + chunk);
                for (bool first = true; kb < kb_end; kb++) {
                    const int s = kb % Cfg::kStages;
                    const uint32_t ph = (kb / Cfg::kStages) & 1;
                    if (!mbar_wait_bounded(full_bar(s), ph, p.wait_limit)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t st = smem_base + s * Cfg::kStageBytes;
                    const uint64_t a_hi = make_kmajor_sw128_desc(st);
                    const uint64_t a_lo = make_kmajor_sw128_desc(st + Cfg::kABytes);
                    const uint64_t b_hi = make_kmajor_sw128_desc(st + 2 * Cfg::kABytes);
                    const uint64_t b_lo = make_kmajor_sw128_desc(st + 2 * Cfg::kABytes + Cfg::kBBytes);
                    // small terms first, then the leading term; 8 tf32 = 32 bytes = 2 sixteen-byte units per k step
#pragma unroll
                    for (int k = 0; k < kBK / 8; k++)
                        umma_tf32<CTAS>(d_tmem, a_lo + 2 * k, b_hi + 2 * k, idesc, (first && k == 0) ? 0u : 1u);
#pragma unroll
                    for (int k = 0; k < kBK / 8; k++) umma_tf32<CTAS>(d_tmem, a_hi + 2 * k, b_lo + 2 * k, idesc, 1);
#pragma unroll
                    for (int k = 0; k < kBK / 8; k++) umma_tf32<CTAS>(d_tmem, a_hi + 2 * k, b_hi + 2 * k, idesc, 1);
                    if (CTAS == 1) umma_commit_1cta(empty_bar(s)); else umma_commit_pair(empty_bar(s));
                    first = false;
                }
                if (ok) {
                    if (CTAS == 1) umma_commit_1cta(acc_full_bar(buf)); else umma_commit_pair(acc_full_bar(buf));
                }
            }
            if (!ok) atomicOr(p.status, ZNN_DEV_MMA_WAIT_EXPIRED);
        }
    } else {
        // ---------------- epilogue: tensor memory -> fp32 registers (per chunk) -> C ----------------
        const int q = warp & 3;              // the TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;    // which half of the tile's columns
        constexpr int CPT = Cfg::kColsPerThread;
        float acc[CPT];
#pragma unroll
        for (int i = 0; i < CPT; i++) acc[i] = 0.0f;
        const uint32_t acc_empty_leader0 = (CTAS == 2) ? mapa_shared(acc_empty_bar(0), 0) : acc_empty_bar(0);
        bool got = true;
        for (int c = 0; c < nchunks; c++) {
            const int buf = c & 1;
            got = __all_sync(0xffffffffu, mbar_wait_bounded_tight(acc_full_bar(buf), (c >> 1) & 1, p.wait_limit));   // every lane polls, the warp votes
            if (!got) break;
            tc_fence_after();
            const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * CPT);
#pragma unroll
            for (int j = 0; j < CPT / 32; j++) {
                float v[32];
                tmem_ld_32x32(t0 + 32u * j, v);
#pragma unroll
                for (int i = 0; i < 32; i++) acc[32 * j + i] += v[i];
            }
            // hand the buffer back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 1) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty_bar(buf)) : "memory");
                else mbar_arrive_remote(acc_empty_leader0 + 8u * buf);
            }
        }
        if (!got) {
            if (lane == 0) atomicOr(p.status, ZNN_DEV_EPI_WAIT_EXPIRED);
        } else {
            const int cbase = col0 + half * CPT;
            // split-K slices store their raw partial sums; a reduce kernel applies alpha/beta afterwards
            const bool to_partial = (p.partial != nullptr);
            float* const out = to_partial ? p.partial + ((size_t)blockIdx.y * gridDim.z + batch) * (size_t)p.M * p.N
                                          : p.C + (size_t)batch * p.stride_c;
            const long long out_ld = to_partial ? (long long)p.N : p.ldc;
            const float* const bias = to_partial ? nullptr : p.bias;
            const bool vec_ok = ((out_ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                                ((reinterpret_cast<uintptr_t>(p.bias) & 15) == 0);
            const float alpha = to_partial ? 1.0f : p.alpha, beta = to_partial ? 0.0f : p.beta;
            float* stage = reinterpret_cast<float*>(smem_gen) + (size_t)(warp - 2) * 32 * (CPT + 4);
            epilogue_store_warp<CPT>(acc, stage, lane, row0 + q * 32, cbase, p.M, p.N, out, out_ld, alpha, beta, bias, vec_ok);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();  // the peer may still signal this CTA's barriers / read its tiles
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// split pre-pass
// ---------------------------------------------------------------------------
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo)
{
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    h &= 0xFFFFE000u;
    float hf = __uint_as_float(h);
    if (!isfinite(hf)) hf = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);  // rounding overflowed (or x is inf/nan)
    float r = isfinite(x) ? (x - hf) : 0.0f;
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(r));
    l &= 0xFFFFE000u;
    hi = hf;
    lo = __uint_as_float(l);
}

// X is [rows, cols] with leading dimension ld (no transpose needed):
// plane[b][r][k] = split(X[b*stride + r*ld + k]), zero for k >= cols.
__global__ void split_rows_kernel(const float* __restrict__ X, long long ld, long long stride_x, int rows, int cols,
                                  int kpad, float* __restrict__ hi, float* __restrict__ lo)
{
    const int b = blockIdx.z;
    const float* xb = X + (size_t)b * stride_x;
    const size_t plane_off = (size_t)b * rows * kpad;
    const int kq = kpad >> 2;  // float4 groups per row
    const bool vec_in = ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(xb) & 15) == 0);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < (size_t)rows * kq;
         i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / kq);
        const int k = (int)(i % kq) * 4;
        float x[4];
        if (vec_in && k + 3 < cols) {
            const float4 t = *reinterpret_cast<const float4*>(xb + (size_t)r * ld + k);
            x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) x[j] = (k + j < cols) ? xb[(size_t)r * ld + k + j] : 0.0f;
        }
        float4 h, l;
        split_tf32(x[0], h.x, l.x); split_tf32(x[1], h.y, l.y);
        split_tf32(x[2], h.z, l.z); split_tf32(x[3], h.w, l.w);
        *reinterpret_cast<float4*>(hi + plane_off + (size_t)r * kpad + k) = h;
        *reinterpret_cast<float4*>(lo + plane_off + (size_t)r * kpad + k) = l;
    }
}

// X is stored [cols(k), rows] with leading dimension ld: plane[b][r][k] = split(X[b*stride + k*ld + r]).
// 32x32 tiles through shared memory so that both the read and the write are coalesced.
__global__ void split_transpose_kernel(const float* __restrict__ X, long long ld, long long stride_x, int rows,
                                       int cols, int kpad, float* __restrict__ hi, float* __restrict__ lo)
{
    __shared__ float tile[32][33];
    const int b = blockIdx.z;
    const float* xb = X + (size_t)b * stride_x;
    const size_t plane_off = (size_t)b * rows * kpad;
    const int r0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    // threads: (32, 8)
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int k = k0 + j, r = r0 + threadIdx.x;
        tile[j][threadIdx.x] = (k < cols && r < rows) ? xb[(size_t)k * ld + r] : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int r = r0 + j, k = k0 + threadIdx.x;
        if (r < rows && k < kpad) {
            float h, l;
            split_tf32(tile[threadIdx.x][j], h, l);
            hi[plane_off + (size_t)r * kpad + k] = h;
            lo[plane_off + (size_t)r * kpad + k] = l;
        }
    }
}

// ---------------------------------------------------------------------------
// the direct GEMM kernel: no pre-pass, the hi/lo split happens in shared memory
// ---------------------------------------------------------------------------
// Operands are read by TMA straight from the caller's fp32 matrices, K-major (the contraction index contiguous) or
// MN-major (the row/column index contiguous), whatever the transpose flags give, so nothing is transposed or copied
// in HBM.  Converter warps store lo = x - (x with the 13 low mantissa bits cleared) next to each landed tile; the raw
// tile itself serves as hi (the tensor core ignores those 13 bits); the conversion is elementwise, so it is blind to
// the 128-byte swizzle.  CTA pairs only.
//   16 warps: 0 TMA, 1 MMA + TMEM, 2-7 converters, 8-15 epilogue.  The converters work as two groups of
//   three warps that take alternate pipeline stages, so that one group's proxy fence and barrier arrival
//   overlap the other group's conversion.  The epilogue warps hold 128 accumulators per thread, so registers
//   are moved to them with setmaxnreg (warpgroups 0-1 shrink to 56, warpgroups 2-3 grow to 200); the code of the
//   56-register roles has to stay lean: spills there cost 6 % of the 8192^3 product when they crept in once (`-Xptxas -v`
//   shows them; the few bytes the 200-register epilogue role spills today cost nothing measurable).
constexpr int kDirectThreads = 512;
constexpr int kConvWarps = 3;     // warps per converter group
constexpr int kConvGroups = 2;
constexpr int kConvWarp0 = 2, kEpiWarp0 = 8;


// Epilogue staging: each epilogue warp turns 32 rows x 32 columns at a time through its own block of shared
// memory (pitch 33 floats: conflict-free both ways), so that every store instruction writes one contiguous
// 128-byte run of a row of C.  The blocks are separate from the operand ring, which is busy with the next tile.
constexpr int kEpiStagePitch = 33;
constexpr int kEpiStageBytes = kEpiWarps * 32 * kEpiStagePitch * 4;   // 33792

// Where the first bounded wait of the in-place kernel expired (diagnostic; read and cleared by znn_gemm_wait_record):
// [0] claimed, [1] role (0 TMA, 1 MMA, 2 converter, 3 epilogue), [2] barrier (0 empty, 1 full, 2 conv, 3 acc_empty,
// 4 acc_full), [3] work unit, [4] stage counter or chunk counter, [5..7] M N K, [8] split-K slices, [9] BN, [10] CTA rank,
// [11] CTA pair, [12] units in the launch, [13] pairs in the launch.
__device__ int g_wait_record[16];

__device__ __forceinline__ void record_expiry(int role, int barrier, int unit, unsigned counter, int cta_rank, int pair)
{
    if (atomicCAS(&g_wait_record[0], 0, 1) != 0) return;
    g_wait_record[1] = role; g_wait_record[2] = barrier; g_wait_record[3] = unit; g_wait_record[4] = (int)counter;
    g_wait_record[10] = cta_rank; g_wait_record[11] = pair;
}

// filled by thread 0 of the CTA that recorded the expiry, at the end of the kernel (keeps the hot loops lean)
__device__ __forceinline__ void record_shape(const GemmTcParams& p, int bn, int npairs)
{
    g_wait_record[5] = p.M; g_wait_record[6] = p.N; g_wait_record[7] = p.k_real; g_wait_record[8] = p.splits;
    g_wait_record[9] = bn; g_wait_record[12] = p.tiles_m * p.tiles_n * p.splits * p.batch; g_wait_record[13] = npairs;
    g_wait_record[14] = (int)(p.beta * 1000.0f); g_wait_record[15] = p.batch;
}

// Optional role profile (compile with -DZNN_ROLE_PROFILE; off in the product build): CTA pair 0's leader adds up, per
// role, the cycles spent inside waits and the cycles of the whole role loop, and leaves them in g_wait_record[1..8]
// ([0] = 2) for znn_gemm_wait_record to read: which role is the one that never waits is the pipeline's bottleneck.
#ifdef ZNN_ROLE_PROFILE
#define ZNN_PROF_DECL long long prof_wait = 0; const long long prof_t0 = clock64();
#define ZNN_PROF_WAIT(expr) [&]() { const long long t_ = clock64(); const bool r_ = (expr); prof_wait += clock64() - t_; return r_; }()
#define ZNN_PROF_END(role, cond)                                                       \
    if (cond) {                                                                        \
        g_wait_record[1 + 2 * (role)] = (int)(prof_wait >> 4);                         \
        g_wait_record[2 + 2 * (role)] = (int)((clock64() - prof_t0) >> 4);             \
        g_wait_record[0] = 2;                                                          \
    }
#else
#define ZNN_PROF_DECL
#define ZNN_PROF_WAIT(expr) (expr)
#define ZNN_PROF_END(role, cond)
#endif

template <int BN>
struct DirectCfg {
    static constexpr int kBRows = BN / 2;
    static constexpr int kABytes = kTileM * kBK * 4;
    static constexpr int kBBytes = kBRows * kBK * 4;
    static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;  // A raw/hi, A lo, B raw/hi, B lo
    static constexpr int kRingBudget = 232448 - 1024 - 512 - kEpiStageBytes;
    static constexpr int kStages = kRingBudget / kStageBytes > 6 ? 6 : kRingBudget / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 512 + kEpiStageBytes;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int kColsPerThread = BN / 2;
    static_assert(kStageBytes % 1024 == 0, "stages must keep the 1 KB alignment of what follows");
};

// One work unit = one 256 x BN output tile of one batch slice and one split-K slice.
struct DirectUnit {
    int row0, col0, batch, split, kb_first, kb_count, nchunks;
};

__device__ __forceinline__ DirectUnit direct_unit(const GemmTcParams& p, int u, int cta_rank, int bn)
{
    DirectUnit d;
    if (p.tri_n > 0) {
        // triangular hint with a tile table: unit = (table entry, slice), slices fastest (no split-K, no tail split)
        const int e = u / p.batch;
        const unsigned tt = p.tri_tab[e];
        d.split = 0;
        d.batch = u - e * p.batch;
        d.row0 = ((int)(tt >> 8) * 2 + cta_rank) * kTileM;
        d.col0 = (int)(tt & 255u) * bn;
        d.kb_first = p.tri_kf[e];
        d.kb_count = p.tri_kc[e];
        d.nchunks = (d.kb_count + p.chunk_kblocks - 1) / p.chunk_kblocks;
        return d;
    }
    int slice = -1;
    int uu = u;
    if (u >= p.tail_first) {   // a K-slice of one of the last round's tiles
        const int sub = u - p.tail_first;
        uu = p.tail_first + sub / p.tail_slices;
        slice = sub - (uu - p.tail_first) * p.tail_slices;
    }
    const int units_per = p.tiles_m * p.tiles_n;
    const int t = uu % units_per;
    const int sb = uu / units_per;
    d.split = sb % p.splits;
    d.batch = sb / p.splits;
    // groups of 8 tile-rows are walked column by column so that CTA pairs running together share
    // A row panels and B column panels in L2
    constexpr int G = 8;
    const int per_group = G * p.tiles_n;
    const int g = t / per_group;
    const int first_m = g * G;
    const int rows_in_group = min(G, p.tiles_m - first_m);
    const int r = t - g * per_group;
    const int tile_m = first_m + r % rows_in_group;
    const int tile_n = r / rows_in_group;
    d.row0 = (tile_m * 2 + cta_rank) * kTileM;
    d.col0 = tile_n * bn;
    d.kb_first = d.split * p.kblocks_per_split;
    d.kb_count = min(p.k_blocks - d.kb_first, p.kblocks_per_split);
    if (slice >= 0) {
        d.kb_first = slice * p.tail_kbps;
        d.kb_count = min(p.k_blocks - d.kb_first, p.tail_kbps);
    }
    d.nchunks = (d.kb_count + p.chunk_kblocks - 1) / p.chunk_kblocks;
    return d;
}

// k-blocks of work unit u (all the converter warps need to know about it)
__device__ __forceinline__ int direct_unit_kb_count(const GemmTcParams& p, int u, int bn)
{
    if (p.tri_n > 0) return p.tri_kc[u / p.batch];
    if (u >= p.tail_first) {
        const int slice = (u - p.tail_first) % p.tail_slices;
        return min(p.k_blocks - slice * p.tail_kbps, p.tail_kbps);
    }
    if (p.splits == 1) return p.k_blocks;
    const int split = (u / (p.tiles_m * p.tiles_n)) % p.splits;
    return min(p.k_blocks - split * p.kblocks_per_split, p.kblocks_per_split);
}

// Activation / residual extension of the epilogue (see GemmTcParams::ep_act); pointers are laid out like C.
struct EpiExt {
    int act;
    float* out2;
    const float* res;
    const float* dpre;
};

__device__ __forceinline__ float gelu_exact(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float gelu_exact_grad(float x)
{
    const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
    const float pdf = 0.3989422804014327f * expf(-0.5f * x * x);
    return cdf + x * pdf;
}
// h = alpha * acc + bias so far.  Forward forms: + residual, keep h, activate.  Gradient forms: multiply by act'(pre).
__device__ __forceinline__ float4 epi_ext_apply(float4 o, const EpiExt& x, size_t off)
{
    if (x.act >= 3) {
        const float4 pre = *reinterpret_cast<const float4*>(x.dpre + off);
        if (x.act == 3) {
            o.x = pre.x > 0.0f ? o.x : 0.0f; o.y = pre.y > 0.0f ? o.y : 0.0f;
            o.z = pre.z > 0.0f ? o.z : 0.0f; o.w = pre.w > 0.0f ? o.w : 0.0f;
        } else {
            o.x *= gelu_exact_grad(pre.x); o.y *= gelu_exact_grad(pre.y);
            o.z *= gelu_exact_grad(pre.z); o.w *= gelu_exact_grad(pre.w);
        }
        return o;
    }
    if (x.res) {
        const float4 r = *reinterpret_cast<const float4*>(x.res + off);
        o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
    }
    if (x.out2) *reinterpret_cast<float4*>(x.out2 + off) = o;
    if (x.act == 1) {
        o.x = fmaxf(o.x, 0.0f); o.y = fmaxf(o.y, 0.0f); o.z = fmaxf(o.z, 0.0f); o.w = fmaxf(o.w, 0.0f);
    } else if (x.act == 2) {
        o.x = gelu_exact(o.x); o.y = gelu_exact(o.y); o.z = gelu_exact(o.z); o.w = gelu_exact(o.w);
    }
    return o;
}

// Final store of one epilogue warp's 32 x CPT sub-tile (each thread holds one row in registers).
template <int CPT>
__device__ __forceinline__ void epilogue_store_rows(const float (&acc)[CPT], float* stage, int lane, int row_base, int cbase,
                                                    int M, int N, float* out, long long out_ld, float alpha, float beta,
                                                    const float* bias)
{
    const int rows = min(32, M - row_base);
    constexpr int RB = 8;  // rows in flight: the loads of old C (beta != 0) are issued together
#pragma unroll
    for (int j = 0; j < CPT / 32; j++) {
#pragma unroll
        for (int c = 0; c < 32; c++) stage[lane * kEpiStagePitch + c] = acc[32 * j + c];
        __syncwarp();
        const int col = cbase + 32 * j + lane;
        if (col < N) {
            const float bv = bias ? bias[col] : 0.0f;
            for (int r0 = 0; r0 < rows; r0 += RB) {
                float old[RB];
                if (beta != 0.0f) {
#pragma unroll
                    for (int u = 0; u < RB; u++)
                        if (r0 + u < rows) old[u] = out[(size_t)(row_base + r0 + u) * out_ld + col];
                }
#pragma unroll
                for (int u = 0; u < RB; u++) {
                    if (r0 + u >= rows) continue;
                    float o = alpha * stage[(r0 + u) * kEpiStagePitch + lane];
                    if (bias) o += bv;
                    if (beta != 0.0f) o += beta * old[u];
                    out[(size_t)(row_base + r0 + u) * out_ld + col] = o;
                }
            }
        }
        __syncwarp();
    }
}

// The same store with 16-byte accesses, for a 16-byte aligned C whose leading dimension is a multiple of 4: the warp's
// 4 KB block holds 1024 / CPT whole rows of the sub-tile at a time (8 rows of 128 columns), written by the lanes that
// own those rows and read back row by row, so that one instruction stores up to 512 contiguous bytes of C.  The float4
// index is XOR-ed with the row so that neither direction has bank conflicts.  A third of the instructions of the
// scalar form, which matters because the epilogue warps share the SM with the next tile's main loop.
// Full 32-row blocks with all columns inside C take one of two leaner forms first (beta = 0 without bias; the
// softmax-backward form): 32-column blocks staged by all 32 lanes and read back as 4 rows x 128 bytes per instruction,
// without edge tests.  The epilogue warps are instruction-latency bound (two per scheduler), so instructions per
// stored byte are what counts: the causal score product went from 152 to 72 us with these forms.
template <int CPT>
__device__ __forceinline__ void epilogue_store_vec(const float (&acc)[CPT], float* stage, int lane, int row_base, int cbase,
                                                   int M, int N, float* out, long long out_ld, float alpha, float beta,
                                                   const float* bias, int rot, const float* ep_p = nullptr,
                                                   const float* ep_d = nullptr, const EpiExt ex = EpiExt{0, nullptr, nullptr, nullptr})
{
    const bool has_ex = ex.act != 0 || ex.res != nullptr;
    // ep_p != nullptr: softmax-backward form, out = alpha * P o (acc - d[row]) with P laid out like out and d one
    // value per row of this slice (beta and bias unused, N a multiple of 4)
    constexpr int LPR = CPT / 4;          // lanes (float4) per row
    constexpr int RPP = 1024 / CPT;       // rows per pass (block = 1024 floats)
    constexpr int RPI = 32 / LPR;         // rows per read instruction
    constexpr int NI = RPP / RPI;         // read instructions per pass
    const int rows = min(32, M - row_base);
    if (rows <= 0) return;
    float4* const st4 = reinterpret_cast<float4*>(stage);
    const int my_f = lane % LPR;           // float4 index inside the row this lane reads
    const int col = cbase + 4 * my_f;
    const bool col_full = col + 3 < N;
    float4 b4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (bias && col_full) b4 = *reinterpret_cast<const float4*>(bias + col);
    const bool fast = !ep_p && !has_ex && beta == 0.0f && bias == nullptr && rows == 32 && cbase + CPT <= N;
    const bool fast_p = ep_p && rows == 32 && cbase + CPT <= N;
    // The order in which the row groups (and the rows inside a group) leave is rotated by `rot` (warp and CTA pair):
    // when every warp of every SM writes rows 0, 1, 2, ... of a power-of-two-pitched C at the same time the stores
    // pile up on the same memory channels (measured with a stand-alone store kernel: 3.7 vs 6.0 TB/s).
    if (fast) {
        // full block, beta = 0, no bias: 32-column blocks staged by all 32 lanes (8 staging stores per block instead of
        // 32 by a quarter of the lanes), read back as 4 rows x 128 bytes per instruction
        static_assert(CPT % 32 == 0, "the column blocks are 32 wide");
        constexpr int NB = CPT / 32;
        float* const cp = out + (size_t)(row_base + lane / 8) * out_ld + cbase + 4 * (lane % 8);
#pragma unroll
        for (int b0 = 0; b0 < NB; b0++) {
#pragma unroll
            for (int f = 0; f < 8; f++)
                st4[lane * 8 + (f ^ (lane & 7))] =
                    make_float4(acc[32 * b0 + 4 * f], acc[32 * b0 + 4 * f + 1], acc[32 * b0 + 4 * f + 2], acc[32 * b0 + 4 * f + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int ri = (i + rot) % 8;
                const int r = 4 * ri + lane / 8;
                const float4 v = st4[r * 8 + ((lane % 8) ^ (r & 7))];
                *reinterpret_cast<float4*>(cp + (size_t)(4 * ri) * out_ld + 32 * b0) =
                    make_float4(alpha * v.x, alpha * v.y, alpha * v.z, alpha * v.w);
            }
            __syncwarp();
        }
        return;
    }
    if (!ep_p && rows == 32 && cbase + CPT <= N) {
        // full block with a bias row and / or beta != 0 (every Linear forward, every accumulating gradient product):
        // staged like the form above; the old values of C for four row groups are loaded together, then four
        // combine-and-store chains.  Same arithmetic order as the general form below: alpha * acc, + bias, + beta * old.
        constexpr int NB = CPT / 32;
        const size_t off = (size_t)(row_base + lane / 8) * out_ld + cbase + 4 * (lane % 8);
#pragma unroll
        for (int b0 = 0; b0 < NB; b0++) {
#pragma unroll
            for (int f = 0; f < 8; f++)
                st4[lane * 8 + (f ^ (lane & 7))] =
                    make_float4(acc[32 * b0 + 4 * f], acc[32 * b0 + 4 * f + 1], acc[32 * b0 + 4 * f + 2], acc[32 * b0 + 4 * f + 3]);
            __syncwarp();
            float4 bb = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (bias) bb = *reinterpret_cast<const float4*>(bias + cbase + 32 * b0 + 4 * (lane % 8));
#pragma unroll
            for (int i0 = 0; i0 < 8; i0 += 4) {
                float4 old[4];
                if (beta != 0.0f) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int ri = (i0 + i + rot) % 8;
                        old[i] = *reinterpret_cast<const float4*>(out + off + (size_t)(4 * ri) * out_ld + 32 * b0);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int ri = (i0 + i + rot) % 8;
                    const int r = 4 * ri + lane / 8;
                    const float4 v = st4[r * 8 + ((lane % 8) ^ (r & 7))];
                    float4 o = make_float4(alpha * v.x, alpha * v.y, alpha * v.z, alpha * v.w);
                    if (bias) { o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w; }
                    if (has_ex) o = epi_ext_apply(o, ex, off + (size_t)(4 * ri) * out_ld + 32 * b0);
                    if (beta != 0.0f) { o.x += beta * old[i].x; o.y += beta * old[i].y; o.z += beta * old[i].z; o.w += beta * old[i].w; }
                    *reinterpret_cast<float4*>(out + off + (size_t)(4 * ri) * out_ld + 32 * b0) = o;
                }
            }
            __syncwarp();
        }
        return;
    }
    if (fast_p) {
        // the softmax-backward form on full blocks, staged the same way: P for four row groups in flight, then four
        // load-combine-store chains
        constexpr int NB = CPT / 32;
        const size_t off = (size_t)(row_base + lane / 8) * out_ld + cbase + 4 * (lane % 8);
        const float* const dp = ep_d + row_base + lane / 8;
#pragma unroll
        for (int b0 = 0; b0 < NB; b0++) {
#pragma unroll
            for (int f = 0; f < 8; f++)
                st4[lane * 8 + (f ^ (lane & 7))] =
                    make_float4(acc[32 * b0 + 4 * f], acc[32 * b0 + 4 * f + 1], acc[32 * b0 + 4 * f + 2], acc[32 * b0 + 4 * f + 3]);
            __syncwarp();
#pragma unroll
            for (int i0 = 0; i0 < 8; i0 += 4) {
                float4 pv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int ri = (i0 + i + rot) % 8;
                    pv[i] = *reinterpret_cast<const float4*>(ep_p + off + (size_t)(4 * ri) * out_ld + 32 * b0);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int ri = (i0 + i + rot) % 8;
                    const int r = 4 * ri + lane / 8;
                    const float4 v = st4[r * 8 + ((lane % 8) ^ (r & 7))];
                    const float dr = dp[4 * ri];
                    *reinterpret_cast<float4*>(out + off + (size_t)(4 * ri) * out_ld + 32 * b0) =
                        make_float4((pv[i].x * (v.x - dr)) * alpha, (pv[i].y * (v.y - dr)) * alpha,
                                    (pv[i].z * (v.z - dr)) * alpha, (pv[i].w * (v.w - dr)) * alpha);
                }
            }
            __syncwarp();
        }
        return;
    }
    for (int g0 = 0; g0 < 32 / RPP; g0++) {
        const int g = (g0 + rot) % (32 / RPP);
        if (g * RPP >= rows) continue;
        // lanes g*RPP .. g*RPP+RPP-1 own the rows of this pass
        if (lane / RPP == g) {
            const int rl = lane % RPP;
#pragma unroll
            for (int f = 0; f < LPR; f++)
                st4[rl * LPR + (f ^ (rl & 7) & (LPR - 1))] = make_float4(acc[4 * f], acc[4 * f + 1], acc[4 * f + 2], acc[4 * f + 3]);
        }
        __syncwarp();
        constexpr int IB = NI < 4 ? NI : 4;   // old-C loads in flight per lane
#pragma unroll
        for (int i0 = 0; i0 < NI; i0 += IB) {
            float4 old[IB];
            if ((beta != 0.0f || ep_p) && col_full) {
                const float* src = ep_p ? ep_p : out;
#pragma unroll
                for (int i = 0; i < IB; i++) {
                    const int r = g * RPP + ((i0 + i + rot) % NI) * RPI + lane / LPR;
                    if (r < rows) {
                        old[i] = *reinterpret_cast<const float4*>(src + (size_t)(row_base + r) * out_ld + col);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < IB; i++) {
                const int rl = ((i0 + i + rot) % NI) * RPI + lane / LPR;
                const int r = g * RPP + rl;
                if (r >= rows || col >= N) continue;
                const float4 v = st4[rl * LPR + (my_f ^ (rl & 7) & (LPR - 1))];
                float* crow = out + (size_t)(row_base + r) * out_ld;
                if (ep_p) {
                    if (col_full) {
                        const float dr = ep_d[row_base + r];
                        *reinterpret_cast<float4*>(crow + col) =
                            make_float4((old[i].x * (v.x - dr)) * alpha, (old[i].y * (v.y - dr)) * alpha,
                                        (old[i].z * (v.z - dr)) * alpha, (old[i].w * (v.w - dr)) * alpha);
                    }
                    continue;
                }
                float o[4] = {alpha * v.x, alpha * v.y, alpha * v.z, alpha * v.w};
                if (col_full) {
                    o[0] += b4.x; o[1] += b4.y; o[2] += b4.z; o[3] += b4.w;
                    if (has_ex) {   // (the extension exists in the 16-byte form only: N is a multiple of 4 then)
                        const float4 t4 = epi_ext_apply(make_float4(o[0], o[1], o[2], o[3]), ex, (size_t)(row_base + r) * out_ld + col);
                        o[0] = t4.x; o[1] = t4.y; o[2] = t4.z; o[3] = t4.w;
                    }
                    if (beta != 0.0f) {
                        o[0] += beta * old[i].x; o[1] += beta * old[i].y; o[2] += beta * old[i].z; o[3] += beta * old[i].w;
                    }
                    *reinterpret_cast<float4*>(crow + col) = make_float4(o[0], o[1], o[2], o[3]);
                } else {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if (col + e < N) {
                            float t = o[e];
                            if (bias) t += bias[col + e];
                            if (beta != 0.0f) t += beta * crow[col + e];
                            crow[col + e] = t;
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
}

// Persistent: each CTA pair walks the work units pair, pair + npairs, ...  Pipeline-stage and accumulator-buffer
// counters run on across units, so the TMA/convert/MMA side starts the next unit while the epilogue warps still
// store the previous one (the two tensor-memory buffers that serve chunked promotion also decouple the units).
template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kDirectThreads, 1)
gemm3x_direct_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const GemmTcParams p)
{
    using Cfg = DirectCfg<BN>;
    constexpr int CTAS = 2;
    constexpr int S = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // layout: operand ring | epilogue staging | barrier block
    const uint32_t epi_stage_addr = smem_base + S * Cfg::kStageBytes;
    const uint32_t bar_base = epi_stage_addr + kEpiStageBytes;
    // barriers: full[S] (TMA -> converters, per CTA), conv[S] (converters of both CTAs -> MMA, in the leader),
    // empty[S] (MMA -> TMA, both CTAs), acc_full[2], acc_empty[2]
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto conv_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * S + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (3 * S + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (3 * S + 2 + b); };
    constexpr int kWordOff = 8 * (3 * S + 4);
    static_assert(kWordOff + 8 <= 512, "barrier block overflows");
    volatile uint32_t* tmem_slot =
        reinterpret_cast<volatile uint32_t*>(smem_gen + S * Cfg::kStageBytes + kEpiStageBytes + kWordOff);
    const uint32_t tmem_slot_addr = bar_base + kWordOff;
    volatile uint32_t* abort_slot = tmem_slot + 1;
    const uint32_t abort_slot_addr = tmem_slot_addr + 4;
    float* const epi_stage_all = reinterpret_cast<float*>(smem_gen + S * Cfg::kStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta_rank = (int)cluster_ctarank();
    const bool leader = (cta_rank == 0);
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int base_units = (p.tri_n > 0 ? p.tri_n : p.tiles_m * p.tiles_n * p.splits) * p.batch;
    const int total_units = p.tail_first + (base_units - p.tail_first) * p.tail_slices;
    const int chunk = p.chunk_kblocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(conv_bar(s), kConvWarps * CTAS);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), kEpiWarps * CTAS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (leader) {
            const uint32_t prior = (uint32_t)(*reinterpret_cast<volatile int*>(p.status));
            *abort_slot = prior;
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(mapa_shared(abort_slot_addr, 1)), "r"(prior) : "memory");
        }
    }
    if (warp == 1) {
        tmem_alloc<CTAS>(tmem_slot_addr, Cfg::kTmemCols);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool aborted = (*abort_slot != 0);

    bool ok = true;
    if (warp < kEpiWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (aborted) {
    } else if (warp == 0) {
        // ---------------- TMA producer: raw fp32 tiles of this CTA's rows of A and of B ----------------
        if (lane == 0) {
            ZNN_PROF_DECL
            uint32_t it = 0;
            for (int u = pair; u < total_units && ok; u += npairs) {
                const DirectUnit d = direct_unit(p, u, cta_rank, BN);
                for (int kb = 0; kb < d.kb_count; kb++, it++) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (!ZNN_PROF_WAIT(mbar_wait_bounded(empty_bar(s), ph ^ 1, p.wait_limit))) { record_expiry(0, 0, u, it, cta_rank, pair); ok = false; break; }
                    const uint32_t st = smem_base + s * Cfg::kStageBytes;
                    int kbl = d.kb_first + kb, slice = d.batch;
                    if (p.kcat_segs > 1) {   // K-concatenated slices: which slice this k-block lies in
                        slice = kbl / p.kcat_kb;
                        kbl -= slice * p.kcat_kb;
                    }
                    const int k0 = kbl * kBK;
                    const int sa = p.a_bcast ? 0 : slice, sbt = p.b_bcast ? 0 : slice;
                    mbar_arrive_expect_tx(full_bar(s), Cfg::kABytes + Cfg::kBBytes);
                    if (A_MN) {
#pragma unroll
                        for (int j = 0; j < kTileM / 32; j++)
                            tma_load_3d(st + j * 4096, &tm_a, full_bar(s), d.row0 + 32 * j, k0, sa);
                    } else {
                        tma_load_3d(st, &tm_a, full_bar(s), k0, d.row0, sa);
                    }
                    const uint32_t sb = st + 2 * Cfg::kABytes;
                    const int brow0 = d.col0 + cta_rank * Cfg::kBRows;
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < Cfg::kBRows / 32; j++)
                            tma_load_3d(sb + j * 4096, &tm_b, full_bar(s), brow0 + 32 * j, k0, sbt);
                    } else {
                        tma_load_3d(sb, &tm_b, full_bar(s), k0, brow0, sbt);
                    }
                }
            }
            if (!ok) atomicOr(p.status, ZNN_DEV_TMA_WAIT_EXPIRED);
            ZNN_PROF_END(0, pair == 0 && cta_rank == 0)
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_tf32_idesc_major(kTileM * CTAS, BN, A_MN, B_MN);
            // descriptor start-address step per K=8 MMA, in 16-byte units
            constexpr uint32_t a_step = A_MN ? (1024 >> 4) : (32 >> 4);
            constexpr uint32_t b_step = B_MN ? (1024 >> 4) : (32 >> 4);
            ZNN_PROF_DECL
            uint32_t it = 0, cc = 0;
            for (int u = pair; u < total_units && ok; u += npairs) {
                const DirectUnit d = direct_unit(p, u, cta_rank, BN);
                int kb = 0;
                for (int c = 0; c < d.nchunks && ok; c++, cc++) {
                    const int buf = cc & 1;
                    // the epilogue warps must have drained this buffer (two chunks ago, possibly of the previous unit)
                    if (!ZNN_PROF_WAIT(mbar_wait_bounded_cluster(acc_empty_bar(buf), ((cc >> 1) & 1) ^ 1, p.wait_limit))) { record_expiry(1, 3, u, cc, cta_rank, pair); ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                    const int kb_end = min(d.kb_count, kb + chunk);
                    for (bool first = true; kb < kb_end; kb++, it++) {
                        const int s = it % S;
                        const uint32_t ph = (it / S) & 1;
                        if (!ZNN_PROF_WAIT(mbar_wait_bounded_cluster(conv_bar(s), ph, p.wait_limit))) { record_expiry(1, 2, u, it, cta_rank, pair); ok = false; break; }
                        tc_fence_after();
                        const uint32_t st = smem_base + s * Cfg::kStageBytes;
                        const uint64_t a_hi = A_MN ? make_mnmajor_sw128_desc(st) : make_kmajor_sw128_desc(st);
                        const uint64_t a_lo = A_MN ? make_mnmajor_sw128_desc(st + Cfg::kABytes) : make_kmajor_sw128_desc(st + Cfg::kABytes);
                        const uint32_t sb = st + 2 * Cfg::kABytes;
                        const uint64_t b_hi = B_MN ? make_mnmajor_sw128_desc(sb) : make_kmajor_sw128_desc(sb);
                        const uint64_t b_lo = B_MN ? make_mnmajor_sw128_desc(sb + Cfg::kBBytes) : make_kmajor_sw128_desc(sb + Cfg::kBBytes);
#pragma unroll
                        for (int k = 0; k < kBK / 8; k++)
                            umma_tf32<CTAS>(d_tmem, a_lo + a_step * k, b_hi + b_step * k, idesc, (first && k == 0) ? 0u : 1u);
#pragma unroll
                        for (int k = 0; k < kBK / 8; k++) umma_tf32<CTAS>(d_tmem, a_hi + a_step * k, b_lo + b_step * k, idesc, 1);
#pragma unroll
                        for (int k = 0; k < kBK / 8; k++) umma_tf32<CTAS>(d_tmem, a_hi + a_step * k, b_hi + b_step * k, idesc, 1);
                        umma_commit_pair(empty_bar(s));
                        first = false;
                    }
                    if (ok) umma_commit_pair(acc_full_bar(buf));
                }
            }
            if (!ok) atomicOr(p.status, ZNN_DEV_MMA_WAIT_EXPIRED);
            ZNN_PROF_END(1, pair == 0)
        }
    } else {
        // ---------------- converters: raw tile -> hi (in place) and lo ----------------
        const int group = (warp - kConvWarp0) / kConvWarps;                      // which alternate stages
        const int ct = threadIdx.x - 32 * (kConvWarp0 + group * kConvWarps);    // 0..95 inside the group
        const uint32_t conv_leader0 = mapa_shared(conv_bar(0), 0);
        constexpr int kAVec = Cfg::kABytes / 16, kBVec = Cfg::kBBytes / 16;
        const bool store_hi = (p.conv_mode == 0);
        bool got = true;
        uint32_t it = 0;
        ZNN_PROF_DECL
        for (int u = pair; u < total_units && got; u += npairs) {
            const int kb_count = direct_unit_kb_count(p, u, BN);
            for (int kb = 0; kb < kb_count; kb++, it++) {
                if ((int)(it % kConvGroups) != group) continue;
                const int s = it % S;
                const uint32_t ph = (it / S) & 1;
                // A parity wait cannot tell a phase from the one two uses earlier.  Where the groups do not divide the
                // stages (three stages, two groups) the slot's previous tile was the other group's and this group has not
                // seen it land; it therefore first waits until that tile has been consumed (the wait the producer makes
                // before it refills the slot: no extra latency), after which the slot's "full" barrier can only be one
                // phase away from the one waited for.
                if (S % kConvGroups != 0) {
                    got = __all_sync(0xffffffffu, mbar_wait_bounded_tight(empty_bar(s), ph ^ 1, p.wait_limit));
                    if (!got) {
                        if (lane == 0) record_expiry(2, 0, u, it, cta_rank, pair);
                        break;
                    }
                }
                // every lane polls and the warp votes: a wait that passes at once costs 90 cycles this way, 240 with one
                // polling lane and a broadcast of its answer (measured), and the hand-off of a tile is this role's latency
                got = ZNN_PROF_WAIT(mbar_wait_bounded_tight(full_bar(s), ph, p.wait_limit));
                got = __all_sync(0xffffffffu, got);
                if (!got) {
                    if (lane == 0) record_expiry(2, 1, u, it, cta_rank, pair);
                    break;
                }
                uint8_t* st = smem_gen + s * Cfg::kStageBytes;
                // hi = x with the 13 low mantissa bits cleared (exactly a TF32 value); lo = x - hi is exact in
                // fp32 and at most 2^-10 |x|; the tensor core drops lo's own low bits, a 2^-21 relative effect
                auto convert = [&](uint8_t* base, int nvec, int lo_off) {
                    constexpr int kT = 32 * kConvWarps;
                    constexpr int kLd = 4;   // 16-byte loads in flight per thread
#pragma unroll 1
                    for (int i0 = ct; i0 < nvec; i0 += kLd * kT) {
                        uint4 x[kLd];
#pragma unroll
                        for (int v = 0; v < kLd; v++)
                            if (i0 + v * kT < nvec) x[v] = *reinterpret_cast<const uint4*>(base + 16 * (i0 + v * kT));
#pragma unroll
                        for (int v = 0; v < kLd; v++) {
                            if (i0 + v * kT >= nvec) continue;
                            uint4 h;
                            h.x = x[v].x & 0xFFFFE000u; h.y = x[v].y & 0xFFFFE000u;
                            h.z = x[v].z & 0xFFFFE000u; h.w = x[v].w & 0xFFFFE000u;
                            float4 l;
                            l.x = __uint_as_float(x[v].x) - __uint_as_float(h.x);
                            l.y = __uint_as_float(x[v].y) - __uint_as_float(h.y);
                            l.z = __uint_as_float(x[v].z) - __uint_as_float(h.z);
                            l.w = __uint_as_float(x[v].w) - __uint_as_float(h.w);
                            uint8_t* src = base + 16 * (i0 + v * kT);
                            if (store_hi) *reinterpret_cast<uint4*>(src) = h;
                            *reinterpret_cast<float4*>(src + lo_off) = l;
                        }
                    }
                };
                convert(st, kAVec, Cfg::kABytes);
                convert(st + 2 * Cfg::kABytes, kBVec, Cfg::kBBytes);
                // make the generic-proxy writes visible to the tensor core (async proxy), then signal the leader
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(conv_leader0 + 8u * s);
            }
        }
        if (!got && lane == 0) atomicOr(p.status, ZNN_DEV_TMA_WAIT_EXPIRED);
        ZNN_PROF_END(2, pair == 0 && cta_rank == 0 && ct == 0 && group == 0)
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
        if (!aborted) {
        // ---------------- epilogue: tensor memory -> fp32 registers (per chunk) -> C ----------------
        const int q = warp & 3;
        const int half = (warp - kEpiWarp0) >> 2;
        constexpr int CPT = Cfg::kColsPerThread;
        const uint32_t acc_empty_leader0 = mapa_shared(acc_empty_bar(0), 0);
        float* const stage = epi_stage_all + (size_t)(warp - kEpiWarp0) * 32 * kEpiStagePitch;
        const bool to_partial = (p.partial != nullptr);
        const long long out_ld = to_partial ? (long long)p.N : p.ldc;
        const float* const bias = to_partial ? nullptr : p.bias;
        const float alpha = to_partial ? 1.0f : p.alpha, beta = to_partial ? 0.0f : p.beta;
        bool got = true;
        uint32_t cc = 0;
        ZNN_PROF_DECL
        for (int u = pair; u < total_units && got; u += npairs) {
            const DirectUnit d = direct_unit(p, u, cta_rank, BN);
            float acc[CPT];
#pragma unroll
            for (int i = 0; i < CPT; i++) acc[i] = 0.0f;
            for (int c = 0; c < d.nchunks; c++, cc++) {
                const int buf = cc & 1;
                got = ZNN_PROF_WAIT(mbar_wait_bounded_tight(acc_full_bar(buf), (cc >> 1) & 1, p.wait_limit));
                got = __all_sync(0xffffffffu, got);
                if (!got) {
                    if (lane == 0) record_expiry(3, 4, u, cc, cta_rank, pair);
                    break;
                }
                tc_fence_after();
                const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * CPT);
#pragma unroll
                for (int j = 0; j < CPT / 32; j++) {
                    float v[32];
                    tmem_ld_32x32(t0 + 32u * j, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) acc[32 * j + i] += v[i];
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(acc_empty_leader0 + 8u * buf);
            }
            if (!got) break;
            // split-K slices store their raw partial sums; a reduce kernel applies alpha/beta afterwards
            if (u >= p.tail_first) {
                // a K-slice of a last-round tile: the raw 256 x BN partial tile, packed, to its own slot
                float* const slot = p.tail_partial + (size_t)(u - p.tail_first) * (size_t)(2 * kTileM * BN);
                epilogue_store_vec<CPT>(acc, stage, lane, cta_rank * kTileM + q * 32, half * CPT, 2 * kTileM, BN, slot, BN, 1.0f,
                                        0.0f, nullptr, warp + pair);
                continue;
            }
            float* const out = to_partial ? p.partial + ((size_t)d.split * p.batch + d.batch) * (size_t)p.M * p.N
                                          : p.C + (size_t)d.batch * p.stride_c;
            const float* const bias_s = bias ? bias + (size_t)d.batch * p.stride_bias : nullptr;
            const bool vec_ok = ((out_ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                                ((reinterpret_cast<uintptr_t>(bias_s) & 15) == 0);
            if (vec_ok)
                epilogue_store_vec<CPT>(acc, stage, lane, d.row0 + q * 32, d.col0 + half * CPT, p.M, p.N, out, out_ld, alpha, beta, bias_s,
                                        warp + pair, p.ep_p ? p.ep_p + (size_t)d.batch * p.stride_c : nullptr,
                                        p.ep_d ? p.ep_d + (size_t)d.batch * p.M : nullptr,
                                        EpiExt{p.ep_act, p.ep_out2, p.ep_res, p.ep_dpre});
            else
                epilogue_store_rows<CPT>(acc, stage, lane, d.row0 + q * 32, d.col0 + half * CPT, p.M, p.N, out, out_ld, alpha, beta, bias_s);
        }
        if (!got && lane == 0) atomicOr(p.status, ZNN_DEV_EPI_WAIT_EXPIRED);
        ZNN_PROF_END(3, pair == 0 && cta_rank == 0 && warp == kEpiWarp0 && lane == 0)
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, Cfg::kTmemCols);
    }
    if (threadIdx.x == 0 && !aborted && g_wait_record[0] == 1 && g_wait_record[11] == pair && g_wait_record[5] == 0)
        record_shape(p, BN, npairs);
}

// C = alpha * sum_s partial[s] + beta * C, slices added in order (deterministic)
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int M, int N, int batch, float alpha,
                                     float beta, float* __restrict__ C, long long ldc, long long stride_c,
                                     const float* __restrict__ bias)
{
    const size_t per = (size_t)M * N;
    const size_t total = per * batch;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (int k = 0; k < splits; k++) s += partial[(size_t)k * total + i];
        const size_t b = i / per, r = (i % per) / N, c = i % N;
        float* dst = C + b * stride_c + r * ldc + c;
        float o = alpha * s;
        if (bias) o += bias[c];
        if (beta != 0.0f) o += beta * (*dst);
        *dst = o;
    }
}

// The same with 16-byte accesses (N, ldc, stride_c multiples of 4; C, bias 16-byte aligned); the slices are still
// added in index order, eight loads in flight per thread.
__global__ void splitk_reduce_vec_kernel(const float4* __restrict__ partial, int splits, int M, int N4, int batch, float alpha,
                                         float beta, float* __restrict__ C, long long ldc, long long stride_c,
                                         const float* __restrict__ bias)
{
    const size_t per4 = (size_t)M * N4;
    const size_t total4 = per4 * batch;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
        float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int k0 = 0; k0 < splits; k0 += 8) {
            float4 v[8];
#pragma unroll
            for (int k = 0; k < 8; k++)
                if (k0 + k < splits) v[k] = partial[(size_t)(k0 + k) * total4 + i];
#pragma unroll
            for (int k = 0; k < 8; k++)
                if (k0 + k < splits) { s.x += v[k].x; s.y += v[k].y; s.z += v[k].z; s.w += v[k].w; }
        }
        const size_t b = i / per4;
        const unsigned rem = (unsigned)(i - b * per4);
        const unsigned r = rem / (unsigned)N4, c = (rem - r * (unsigned)N4) * 4u;
        float4* dst = reinterpret_cast<float4*>(C + b * stride_c + (size_t)r * ldc + c);
        float4 o = make_float4(alpha * s.x, alpha * s.y, alpha * s.z, alpha * s.w);
        if (bias) {
            const float4 b4 = *reinterpret_cast<const float4*>(bias + c);
            o.x += b4.x; o.y += b4.y; o.z += b4.z; o.w += b4.w;
        }
        if (beta != 0.0f) {
            const float4 old = *dst;
            o.x += beta * old.x; o.y += beta * old.y; o.z += beta * old.z; o.w += beta * old.w;
        }
        *dst = o;
    }
}

// Adds the K-slices of the last-round tiles (tail split of the in-place kernel) in slice order and applies
// alpha / beta / bias: C[tile] = alpha * sum_s partial[tile][s] + bias + beta * C[tile].  One block row per tile.
template <int BN>
__global__ void tail_reduce_kernel(const GemmTcParams p)
{
    const int j = blockIdx.y;                      // which tail tile
    __shared__ DirectUnit sd;
    if (threadIdx.x == 0) sd = direct_unit(p, p.tail_first + j * p.tail_slices, 0, BN);   // slice 0: the tile's coordinates
    __syncthreads();
    const DirectUnit d = sd;
    constexpr int kElems = 2 * kTileM * BN;
    const float4* base = reinterpret_cast<const float4*>(p.tail_partial + (size_t)j * p.tail_slices * (size_t)kElems);
    float* const Cb = p.C + (size_t)d.batch * p.stride_c;
    const float* const bias_s = p.bias ? p.bias + (size_t)d.batch * p.stride_bias : nullptr;
    const bool vec = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(Cb) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(bias_s) & 15) == 0);
    const int e4 = blockIdx.x * blockDim.x + threadIdx.x;     // one float4 of the tile per thread
    if (e4 >= kElems / 4) return;
    const int r = e4 / (BN / 4), c = (e4 - r * (BN / 4)) * 4;
    const int row = d.row0 + r, col = d.col0 + c;
    if (row >= p.M || col >= p.N) return;
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 v[8];
#pragma unroll
    for (int sl = 0; sl < 8; sl++)
        if (sl < p.tail_slices) v[sl] = base[(size_t)sl * (kElems / 4) + e4];
#pragma unroll
    for (int sl = 0; sl < 8; sl++)
        if (sl < p.tail_slices) { sum.x += v[sl].x; sum.y += v[sl].y; sum.z += v[sl].z; sum.w += v[sl].w; }
    float o[4] = {p.alpha * sum.x, p.alpha * sum.y, p.alpha * sum.z, p.alpha * sum.w};
    float* dst = Cb + (size_t)row * p.ldc + col;
    if (vec && col + 3 < p.N) {
        if (bias_s) {
            const float4 b4 = *reinterpret_cast<const float4*>(bias_s + col);
            o[0] += b4.x; o[1] += b4.y; o[2] += b4.z; o[3] += b4.w;
        }
        if (p.ep_act != 0 || p.ep_res) {
            const float4 t4 = epi_ext_apply(make_float4(o[0], o[1], o[2], o[3]), EpiExt{p.ep_act, p.ep_out2, p.ep_res, p.ep_dpre},
                                            (size_t)row * p.ldc + col);
            o[0] = t4.x; o[1] = t4.y; o[2] = t4.z; o[3] = t4.w;
        }
        if (p.beta != 0.0f) {
            const float4 old = *reinterpret_cast<const float4*>(dst);
            o[0] += p.beta * old.x; o[1] += p.beta * old.y; o[2] += p.beta * old.z; o[3] += p.beta * old.w;
        }
        *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (col + e >= p.N) break;
            float t = o[e];
            if (bias_s) t += bias_s[col + e];
            if (p.beta != 0.0f) t += p.beta * dst[e];
            dst[e] = t;
        }
    }
}

// Test aid for the bounded-wait recovery path: one thread waits, with the same wait routine as the GEMM roles, on an
// mbarrier that nothing ever arrives at; when the limit runs out it records the expiry in the device status word, as
// a GEMM role would, and returns.  No trap, no fault: the context stays usable.
__global__ void wait_probe_kernel(int* status, unsigned long long limit)
{
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        const uint32_t b = smem_u32(&bar);
        mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait_bounded(b, 0, limit)) atomicOr(status, ZNN_DEV_TMA_WAIT_EXPIRED);
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
int tc_wait_probe(unsigned long long limit_cycles)
{
    int* status = device_status_word();
    if (!status) return fail(ZNN_ERR_CUDA, "no device state (call znn_init first)");
    if (limit_cycles == 0 || limit_cycles > 2000000000ull) return fail(ZNN_ERR_INVALID, "limit must be 1 .. 2e9 cycles");
    wait_probe_kernel<<<1, 32, 0, stream()>>>(status, limit_cycles);
    ZNN_LAUNCH_OK("wait_probe_kernel");
    return ZNN_OK;
}

int launch_splitk_reduce(const float* partial, int splits, int M, int N, int batch, float alpha, float beta, float* C,
                         long long ldc, long long stride_c, const float* bias)
{
    const size_t total = (size_t)batch * M * N;
    const bool vec = (N & 3) == 0 && (ldc & 3) == 0 && (batch == 1 || (stride_c & 3) == 0) &&
                     (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (reinterpret_cast<uintptr_t>(bias) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(partial) & 15) == 0 && (size_t)M * (N / 4) < 0xffffffffull;
    const size_t items = vec ? total / 4 : total;
    int blocks = (int)((items + 255) / 256);
    const int cap = sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (vec)
        splitk_reduce_vec_kernel<<<blocks, 256, 0, stream()>>>(reinterpret_cast<const float4*>(partial), splits, M, N / 4, batch,
                                                               alpha, beta, C, ldc, stride_c, bias);
    else
        splitk_reduce_kernel<<<blocks, 256, 0, stream()>>>(partial, splits, M, N, batch, alpha, beta, C, ldc, stride_c, bias);
    ZNN_LAUNCH_OK("splitk_reduce_kernel");
    return ZNN_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// plane: [batch][rows][kpad] fp32; box = 32 (k) x box_rows x 1
static int make_plane_map(CUtensorMap* tm, float* plane, int rows, int kpad, int batch, int box_rows)
{
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(ZNN_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[3] = {(cuuint64_t)kpad, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)kpad * 4, (cuuint64_t)kpad * 4 * (cuuint64_t)rows};
    cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, plane, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ZNN_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return ZNN_OK;
}

// ---- optional event bracketing of the tensor-core kernel (measurement aid) ----
struct TcProfile {
    bool on = false;
    static constexpr int kMaxEvents = 4096;
    cudaEvent_t ev[kMaxEvents][2];
    int created = 0;
    int used = 0;
    double flops = 0.0;
};
static thread_local TcProfile t_prof;

static cudaEvent_t* prof_begin(double flops)
{
    TcProfile& pr = t_prof;
    if (!pr.on || pr.used >= TcProfile::kMaxEvents) return nullptr;
    if (pr.used >= pr.created) {
        if (cudaEventCreate(&pr.ev[pr.created][0]) != cudaSuccess) return nullptr;
        if (cudaEventCreate(&pr.ev[pr.created][1]) != cudaSuccess) return nullptr;
        pr.created++;
    }
    cudaEvent_t* e = pr.ev[pr.used++];
    pr.flops += flops;
    cudaEventRecord(e[0], stream());
    return e;
}

static void prof_end(cudaEvent_t* e)
{
    if (e) cudaEventRecord(e[1], stream());
}

int tc_wait_record(int* out16)
{
    ZNN_CUDA_OK(cudaMemcpyFromSymbol(out16, g_wait_record, 16 * sizeof(int)));
    int zero[16] = {0};
    ZNN_CUDA_OK(cudaMemcpyToSymbol(g_wait_record, zero, sizeof(zero)));
    return ZNN_OK;
}

int tc_profile_enable(int enable)
{
    t_prof.on = (enable != 0);
    t_prof.used = 0;
    t_prof.flops = 0.0;
    return ZNN_OK;
}

int tc_profile_read(double* kernel_ms, long long* launches, double* flops)
{
    TcProfile& pr = t_prof;
    double total = 0.0;
    for (int i = 0; i < pr.used; i++) {
        ZNN_CUDA_OK(cudaEventSynchronize(pr.ev[i][1]));
        float ms = 0.0f;
        ZNN_CUDA_OK(cudaEventElapsedTime(&ms, pr.ev[i][0], pr.ev[i][1]));
        total += ms;
    }
    if (kernel_ms) *kernel_ms = total;
    if (launches) *launches = pr.used;
    if (flops) *flops = pr.flops;
    pr.used = 0;
    pr.flops = 0.0;
    return ZNN_OK;
}

template <int BN, int CTAS>
static int launch_tc(const CUtensorMap* maps, const GemmTcParams& p, int batch)
{
    using Cfg = TcCfg<BN, CTAS>;
    // the attribute is per device: a process that drives several GPUs sets it once on each
    static bool attr_set[64] = {false};
    auto kern = gemm3x_tf32_kernel<BN, CTAS>;
    int adev = 0;
    ZNN_CUDA_OK(cudaGetDevice(&adev));
    if (adev < 0 || adev >= 64) return fail(ZNN_ERR_INVALID, "device index %d out of range", adev);
    if (!attr_set[adev]) {
        ZNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[adev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    const int splits = (p.k_blocks + p.kblocks_per_split - 1) / p.kblocks_per_split;
    cfg.gridDim = dim3((unsigned)(p.tiles_m * p.tiles_n * CTAS), (unsigned)splits, (unsigned)batch);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaEvent_t* ev = prof_begin(2.0 * p.M * (double)p.N * p.k_real * batch);
    ZNN_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, maps[0], maps[1], maps[2], maps[3], p));
    prof_end(ev);
    count_launch();
    if (inject_launch_failure()) return fail(ZNN_ERR_CUDA, "launch of the tensor-core GEMM failed: injected failure (znn_debug_fail_after)");
    return ZNN_OK;
}

static unsigned long long g_wait_limit = kWaitLimitCycles;
void tc_set_wait_limit(unsigned long long cycles) { g_wait_limit = cycles ? cycles : kWaitLimitCycles; }
unsigned long long tc_wait_limit() { return g_wait_limit; }
static thread_local int t_conv_mode = 1;
void tc_set_conv_mode(int m) { t_conv_mode = m; }
static thread_local bool t_tail_split = true;
void tc_set_tail_split(int on) { t_tail_split = (on != 0); }
static thread_local bool t_persistent = true;
void tc_set_persistent(int on) { t_persistent = (on != 0); }
static thread_local bool t_splitk_enabled = true;
void tc_set_splitk(int on) { t_splitk_enabled = (on != 0); }
static thread_local int t_chunk_kblocks = 8;  // 256 contraction elements per tensor-memory accumulation
int tc_chunk_kblocks() { return t_chunk_kblocks; }
void tc_set_chunk_kblocks(int v) { t_chunk_kblocks = v < 1 ? 1 : v; }

struct TcPlan {
    int bn, tiles_m, tiles_n, k_blocks, chunk, splits, kbps;
};

// Tail split of the persistent walk: `units` tiles on `slots` CTA pairs; when the last round would be less than 70 %
// full its tiles are cut into K-slices (whole chunks, at most 8) so that the round costs 1/slices.  Returns the number
// of slices (1 = no split) and the k-blocks per slice.
static int tail_slices_for(long units, long slots, int k_blocks, int chunk, int* kbps_out)
{
    *kbps_out = k_blocks;
    const long rounds = units / slots, tail = units % slots;
    if (rounds < 1 || tail == 0 || tail * 10 >= slots * 7) return 1;
    long s = slots / tail;
    const long by_k = k_blocks / chunk;
    if (s > by_k) s = by_k;
    if (s > 8) s = 8;
    if (s < 2) return 1;
    int kbps = (int)((k_blocks + s - 1) / s);
    kbps = ((kbps + chunk - 1) / chunk) * chunk;
    const int eff = (k_blocks + kbps - 1) / kbps;
    if (eff < 2) return 1;
    *kbps_out = kbps;
    return eff;
}

// rounds of the walk in units of one tile's time (the tail round costs 1/slices plus the small reduce pass)
static double plan_rounds(long units, long slots, int k_blocks, int chunk, bool tail_ok)
{
    const long rounds = units / slots, tail = units % slots;
    if (tail == 0) return (double)rounds;
    int kbps;
    const int s = tail_ok ? tail_slices_for(units, slots, k_blocks, chunk, &kbps) : 1;
    // a slice pays the pipeline fill again (~6 k-blocks' worth) and the reduce pass another ~4
    return (double)rounds + (s > 1 ? ((double)kbps + 10.0) / ((double)k_blocks + 6.0) : 1.0);
}

static TcPlan make_plan(int M, int N, int K, int batch, int ctas, bool tail_ok = false)
{
    TcPlan pl;
    pl.bn = 256;
    if (N <= 64) pl.bn = 64;
    else if (N <= 128) pl.bn = 128;
    else if (ctas == 2) {
        // Few tiles: with 256-wide tiles the last round of the persistent walk may be mostly empty (96 tiles on 74
        // CTA pairs take two rounds).  128-wide tiles cost ~0.6 of a 256-wide one each (measured; shared-memory
        // bound) and fill the rounds better; the in-place kernel can also cut the tiles of a thin last round into
        // K-slices (tail split).  Take the width whose rounds x cost comes out lower.
        const long slots = sm_count() / 2;
        const long tm = (M + 2 * kTileM - 1) / (2 * kTileM);
        const long u256 = tm * ((N + 255) / 256) * batch, u128 = tm * ((N + 127) / 128) * batch;
        const int kb = (K + kBK - 1) / kBK, ch = tc_chunk_kblocks();
        const double c256 = plan_rounds(u256, slots, kb, ch, tail_ok), c128 = 0.6 * plan_rounds(u128, slots, kb, ch, tail_ok);
        if (u256 >= slots && u256 < 4 * slots && c128 < c256) pl.bn = 128;
    }
    const int tile_rows = kTileM * ctas;
    pl.tiles_m = (M + tile_rows - 1) / tile_rows;
    pl.tiles_n = (N + pl.bn - 1) / pl.bn;
    pl.k_blocks = (K + kBK - 1) / kBK;
    pl.chunk = tc_chunk_kblocks();
    // Few output tiles and a long contraction (parameter gradients: dW = X^T dY): cut K over
    // blockIdx.y so that every CTA pair slot of the GPU has work; slices are whole chunks.
    int splits = 1;
    const long units = (long)pl.tiles_m * pl.tiles_n * batch;
    const int slots = sm_count() / ctas;
    const int max_by_k = pl.k_blocks / (pl.chunk > 8 ? pl.chunk : 8);
    if (t_splitk_enabled && units * 2 <= slots && max_by_k >= 2) {
        splits = (int)(slots / units);
        if (splits > max_by_k) splits = max_by_k;
        if (splits > 32) splits = 32;
        if (splits < 1) splits = 1;
    }
    int kbps = (pl.k_blocks + splits - 1) / splits;
    kbps = ((kbps + pl.chunk - 1) / pl.chunk) * pl.chunk;  // whole chunks per slice
    pl.kbps = kbps;
    pl.splits = (pl.k_blocks + kbps - 1) / kbps;
    return pl;
}

// op(A) is M x K, op(B) is K x N.  ctas = 1 or 2.
// True when the plan for this product cuts the contraction over several CTA pairs (few output tiles, long K): the
// epilogue forms that finish the result in the GEMM kernel itself do not exist for such products.
bool tc_plan_splits_k(int M, int N, int K) { return make_plan(M, N, K, 1, 2).splits > 1; }

int gemm_tc(int ta, int tb, int M, int N, int K, float alpha, const float* A, long long lda, long long stride_a,
            const float* B, long long ldb, long long stride_b, float beta, float* C, long long ldc,
            long long stride_c, int batch, int ctas, const float* bias)
{
    int* status = device_status_word();
    if (!status) return fail(ZNN_ERR_CUDA, "no device state (call znn_init first)");
    const int kpad = ((K + kBK - 1) / kBK) * kBK;
    const size_t a_plane = (size_t)batch * M * kpad, b_plane = (size_t)batch * N * kpad;
    const TcPlan pl = make_plan(M, N, K, batch, ctas);
    const int bn = pl.bn, tiles_m = pl.tiles_m, tiles_n = pl.tiles_n, k_blocks = pl.k_blocks, chunk = pl.chunk;
    const int splits = pl.splits, kbps = pl.kbps;
    const size_t partial_floats = splits > 1 ? (size_t)splits * batch * M * N : 0;
    const size_t need = (2 * a_plane + 2 * b_plane + partial_floats) * sizeof(float);
    float* ws = (float*)workspace(need);
    if (!ws) return fail(ZNN_ERR_NOMEM, "GEMM scratch of %zu bytes could not be allocated", need);
    float* a_hi = ws;
    float* a_lo = a_hi + a_plane;
    float* b_hi = a_lo + a_plane;
    float* b_lo = b_hi + b_plane;
    cudaStream_t st = stream();

    // ---- split pre-pass: both operands become K-major planes ----
    auto split = [&](const float* X, long long ld, long long stride_x, int rows, bool k_contiguous, float* hi,
                     float* lo) -> int {
        if (k_contiguous) {
            const size_t work = (size_t)rows * (kpad / 4);
            int blocks = (int)((work + 255) / 256);
            const int cap = sm_count() * 16;
            if (blocks > cap) blocks = cap;
            if (blocks < 1) blocks = 1;
            split_rows_kernel<<<dim3(blocks, 1, batch), 256, 0, st>>>(X, ld, stride_x, rows, K, kpad, hi, lo);
        } else {
            dim3 grid((rows + 31) / 32, kpad / 32, batch);
            split_transpose_kernel<<<grid, dim3(32, 8), 0, st>>>(X, ld, stride_x, rows, K, kpad, hi, lo);
        }
        ZNN_LAUNCH_OK("split pre-pass");
        return ZNN_OK;
    };
    // op(A)[i,p]: NoTrans -> A[i*lda+p] (k contiguous); Trans -> A[p*lda+i]
    int rc = split(A, lda, stride_a, M, ta == ZNN_NO_TRANS, a_hi, a_lo);
    if (rc) return rc;
    // op(B)[p,j] as plane[j][p]: Trans -> B[j*ldb+p] (k contiguous); NoTrans -> B[p*ldb+j]
    rc = split(B, ldb, stride_b, N, tb == ZNN_TRANS, b_hi, b_lo);
    if (rc) return rc;

    GemmTcParams p;
    p.M = M; p.N = N; p.k_blocks = k_blocks; p.k_real = K; p.chunk_kblocks = chunk;
    p.kblocks_per_split = kbps;
    p.partial = splits > 1 ? (b_lo + b_plane) : nullptr;
    p.ep_p = nullptr;
    p.ep_d = nullptr;
    p.ep_act = 0; p.ep_out2 = nullptr; p.ep_res = nullptr; p.ep_dpre = nullptr;
    p.a_bcast = 0; p.b_bcast = 0; p.stride_bias = 0; p.kcat_segs = 0; p.kcat_kb = 0;
    p.conv_mode = 0;
    p.bias = bias;
    p.tiles_m = tiles_m;
    p.tiles_n = tiles_n;
    p.alpha = alpha; p.beta = beta; p.C = C; p.ldc = ldc; p.stride_c = stride_c; p.status = status;
    p.wait_limit = g_wait_limit;

    CUtensorMap maps[4];
    if ((rc = make_plane_map(&maps[0], a_hi, M, kpad, batch, kTileM))) return rc;
    if ((rc = make_plane_map(&maps[1], a_lo, M, kpad, batch, kTileM))) return rc;
    if ((rc = make_plane_map(&maps[2], b_hi, N, kpad, batch, bn / ctas))) return rc;
    if ((rc = make_plane_map(&maps[3], b_lo, N, kpad, batch, bn / ctas))) return rc;

    if (ctas == 1) {
        if (bn == 256) rc = launch_tc<256, 1>(maps, p, batch);
        else if (bn == 128) rc = launch_tc<128, 1>(maps, p, batch);
        else rc = launch_tc<64, 1>(maps, p, batch);
    } else {
        if (bn == 256) rc = launch_tc<256, 2>(maps, p, batch);
        else if (bn == 128) rc = launch_tc<128, 2>(maps, p, batch);
        else rc = launch_tc<64, 2>(maps, p, batch);
    }
    if (rc) return rc;
    if (splits > 1) return launch_splitk_reduce(p.partial, splits, M, N, batch, alpha, beta, C, ldc, stride_c, bias);
    return ZNN_OK;
}


// ---- direct path host side ----
// X is the caller's matrix.  K-major: X[row*ld + k]; MN-major: X[k*ld + row].
static int make_operand_map(CUtensorMap* tm, const float* X, bool mn_major, int rows, int K, long long ld,
                            long long stride, int batch, int box_rows)
{
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(ZNN_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    const cuuint64_t inner = mn_major ? (cuuint64_t)rows : (cuuint64_t)K;
    const cuuint64_t outer = mn_major ? (cuuint64_t)K : (cuuint64_t)rows;
    cuuint64_t dims[3] = {inner, outer, (cuuint64_t)batch};
    const cuuint64_t bstride = (batch > 1) ? (cuuint64_t)stride * 4 : (cuuint64_t)ld * 4 * outer;
    cuuint64_t strides[2] = {(cuuint64_t)ld * 4, bstride};
    cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)(mn_major ? kBK : box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(X), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ZNN_ERR_CUDA, "cuTensorMapEncodeTiled (operand) failed with %d", (int)r);
    return ZNN_OK;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_direct(const CUtensorMap& ma, const CUtensorMap& mb, const GemmTcParams& p_in, int batch)
{
    using Cfg = DirectCfg<BN>;
    // the attribute is per device: a process that drives several GPUs sets it once on each
    static bool attr_set[64] = {false};
    auto kern = gemm3x_direct_kernel<BN, A_MN, B_MN>;
    int dev = 0;
    ZNN_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(ZNN_ERR_INVALID, "device index %d out of range", dev);
    if (!attr_set[dev]) {
        ZNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[dev] = true;
    }
    GemmTcParams p = p_in;
    p.splits = (p.k_blocks + p.kblocks_per_split - 1) / p.kblocks_per_split;
    p.batch = batch;
    const long base_units = (p.tri_n > 0 ? (long)p.tri_n : (long)p.tiles_m * p.tiles_n * p.splits) * batch;
    if (base_units > 0x3fffffffL) return fail(ZNN_ERR_INVALID, "too many output tiles (%ld)", base_units);
    if (p.tail_slices < 1) {   // no tail split
        p.tail_first = (int)base_units;
        p.tail_slices = 1;
    }
    const long total_units = p.tail_first + (base_units - p.tail_first) * p.tail_slices;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kDirectThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // persistent: one CTA pair per pair of SMs that can hold one (asked of the driver once per device)
    static int pairs_by_device[64] = {0};
    if (pairs_by_device[dev] == 0) {
        cfg.gridDim = dim3((unsigned)sm_count(), 1, 1);
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters < 1) {
            cudaGetLastError();
            clusters = sm_count() / 2;
        }
        pairs_by_device[dev] = clusters;
    }
    const long pairs = (!t_persistent || total_units < pairs_by_device[dev]) ? total_units : pairs_by_device[dev];
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cudaEvent_t* ev = prof_begin(2.0 * p.M * (double)p.N * p.k_real * batch);
    ZNN_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ma, mb, p));
    prof_end(ev);
    count_launch();
    if (inject_launch_failure()) return fail(ZNN_ERR_CUDA, "launch of the tensor-core GEMM failed: injected failure (znn_debug_fail_after)");
    return ZNN_OK;
}

template <int BN>
static int launch_direct_major(bool a_mn, bool b_mn, const CUtensorMap& ma, const CUtensorMap& mb, const GemmTcParams& p,
                               int batch)
{
    if (a_mn) return b_mn ? launch_direct<BN, true, true>(ma, mb, p, batch) : launch_direct<BN, true, false>(ma, mb, p, batch);
    return b_mn ? launch_direct<BN, false, true>(ma, mb, p, batch) : launch_direct<BN, false, false>(ma, mb, p, batch);
}

// True when TMA can read both operands where they lie: 16-byte aligned bases, leading dimensions and batch strides.
bool gemm_tc_direct_eligible(const float* A, long long lda, long long stride_a, const float* B, long long ldb,
                             long long stride_b, int batch)
{
    auto ok = [&](const float* X, long long ld, long long stride) {
        return (reinterpret_cast<uintptr_t>(X) & 15) == 0 && (ld & 3) == 0 && (batch == 1 || (stride & 3) == 0);
    };
    return ok(A, lda, stride_a) && ok(B, ldb, stride_b);
}

int gemm_tc_direct(int ta, int tb, int M, int N, int K, float alpha, const float* A, long long lda, long long stride_a,
                   const float* B, long long ldb, long long stride_b, float beta, float* C, long long ldc,
                   long long stride_c, int batch, const float* bias, int tri, const float* ep_p, const float* ep_d,
                   int ep_act, float* ep_out2, const float* ep_res, const float* ep_dpre, long long stride_bias, int kcat)
{
    // kcat != 0: the `batch` slices are one product, concatenated along K (C is a single matrix); K a multiple of 32
    const int segs = kcat ? batch : 0;
    const int seg_kb = (K + kBK - 1) / kBK;
    if (kcat) {
        if ((K % kBK) != 0 || bias || tri != 0 || ep_p || ep_act != 0 || ep_res)
            return fail(ZNN_ERR_UNSUPPORTED, "K-concatenated product: K must be a multiple of 32, no epilogue forms");
        K = K * batch;      // the plan, the k-block walk and the flop count see the whole contraction
        batch = 1;
    }
    int* status = device_status_word();
    if (!status) return fail(ZNN_ERR_CUDA, "no device state (call znn_init first)");
    const bool has_ex = ep_act != 0 || ep_res != nullptr;
    if (has_ex) {
        // 16-byte form only, one slice, whole-K tiles (slices of a tail split are finished by the reduce kernel, which
        // knows the extension; split-K is switched off below)
        auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
        if ((N & 3) || (ldc & 3) || !al(C) || !al(bias) || !al(ep_out2) || !al(ep_res) || !al(ep_dpre) || batch != 1 || ep_p ||
            tri != 0 || (ep_act >= 3 && !ep_dpre) || (ep_act < 3 && beta != 0.0f) || ep_act < 0 || ep_act > 4)
            return fail(ZNN_ERR_UNSUPPORTED, "activation / residual epilogue: unaligned output or unsupported arguments");
    }
    if (ep_p) {
        // the softmax-backward epilogue exists in the 16-byte form only, and never meets partial tiles
        if ((N & 3) || (ldc & 3) || (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(ep_p) & 15) ||
            (batch > 1 && (stride_c & 3)) || !ep_d || bias || beta != 0.0f)
            return fail(ZNN_ERR_UNSUPPORTED, "softmax-backward epilogue: unaligned output or unsupported arguments");
    }
    const bool tail_ok = t_tail_split && t_persistent && tri == 0 && !ep_p;
    TcPlan pl = make_plan(M, N, K, batch, 2, tail_ok);
    // (the split-K reduce kernel knows neither the epilogue forms nor a bias row per slice)
    if ((tri != 0 || ep_p || has_ex || (bias && stride_bias != 0 && batch > 1)) && pl.splits > 1) {   // the triangular k-ranges are per tile; no split-K on top of them
        pl.splits = 1;
        pl.kbps = ((pl.k_blocks + pl.chunk - 1) / pl.chunk) * pl.chunk;
    }
    // tail split (only without split-K): the tiles of a thin last round are cut into K-slices
    int tail_slices = 1, tail_kbps = pl.k_blocks;
    long tail_tiles = 0;
    const long units = (long)pl.tiles_m * pl.tiles_n * batch, slots = sm_count() / 2;
    if (tail_ok && pl.splits == 1) {
        tail_slices = tail_slices_for(units, slots, pl.k_blocks, pl.chunk, &tail_kbps);
        if (tail_slices > 1) tail_tiles = units % slots;
    }
    float* partial = nullptr;
    if (pl.splits > 1) {
        partial = (float*)workspace((size_t)pl.splits * batch * M * N * sizeof(float));
        if (!partial) return fail(ZNN_ERR_NOMEM, "split-K scratch could not be allocated");
    }
    float* tail_partial = nullptr;
    if (tail_tiles > 0) {
        tail_partial = (float*)workspace((size_t)tail_tiles * tail_slices * 2 * kTileM * pl.bn * sizeof(float));
        if (!tail_partial) return fail(ZNN_ERR_NOMEM, "tail-split scratch could not be allocated");
    }
    const bool a_mn = (ta == ZNN_TRANS), b_mn = (tb == ZNN_NO_TRANS);
    CUtensorMap ma, mb;
    int rc;
    // an operand with batch stride 0 is one matrix shared by all slices: its map has one slice, always read at 0
    const int map_slices = kcat ? segs : batch;
    const int map_k = kcat ? K / segs : K;
    const bool a_bc = map_slices > 1 && stride_a == 0, b_bc = map_slices > 1 && stride_b == 0;
    if ((rc = make_operand_map(&ma, A, a_mn, M, map_k, lda, stride_a, a_bc ? 1 : map_slices, kTileM))) return rc;
    if ((rc = make_operand_map(&mb, B, b_mn, N, map_k, ldb, stride_b, b_bc ? 1 : map_slices, pl.bn / 2))) return rc;
    GemmTcParams p;
    p.M = M; p.N = N; p.k_blocks = pl.k_blocks; p.k_real = K; p.chunk_kblocks = pl.chunk;
    p.kblocks_per_split = pl.kbps;
    p.partial = partial;
    p.conv_mode = t_conv_mode;
    p.bias = bias;
    p.tiles_m = pl.tiles_m;
    p.tiles_n = pl.tiles_n;
    p.splits = pl.splits;
    p.batch = batch;
    p.tail_first = (int)(units * pl.splits - tail_tiles);
    p.tail_slices = tail_tiles > 0 ? tail_slices : 0;   // 0 = off (launch_direct normalises it)
    p.tail_kbps = tail_kbps;
    p.tail_partial = tail_partial;
    p.ep_p = ep_p;
    p.ep_d = ep_d;
    p.ep_act = ep_act; p.ep_out2 = ep_out2; p.ep_res = ep_res; p.ep_dpre = ep_dpre;
    p.a_bcast = a_bc ? 1 : 0; p.b_bcast = b_bc ? 1 : 0;
    p.stride_bias = stride_bias;
    p.kcat_segs = segs; p.kcat_kb = seg_kb;
    // The hint works through a table of the slice's tiles (which have work, and which k-blocks); a slice of more than
    // 64 tiles is computed in full instead (the hint never changes values that may be read).
    p.tri_n = 0;
    p.tri = 0;
    if (tri != 0 && pl.splits == 1 && pl.tiles_m * pl.tiles_n <= 64 && pl.k_blocks < 65536) {
        p.tri = tri;
        // k-blocks every tile of a slice needs under the hint; the table lists the tiles with work, dearest first
        struct Ent { int cost; unsigned short code, kf; };
        Ent ent[64];
        int n = 0;
        for (int tm = 0; tm < pl.tiles_m; tm++)
            for (int tn = 0; tn < pl.tiles_n; tn++) {
                const int row0 = tm * 2 * kTileM, col0 = tn * pl.bn;
                int lo = 0, hi = pl.k_blocks;
                if (tri == ZNN_TRI_C_LOWER) { if (col0 > row0 + 2 * kTileM - 1) hi = 0; }
                else if (tri == ZNN_TRI_A_LOWER) { const int h2 = (row0 + 2 * kTileM + kBK - 1) / kBK; if (h2 < hi) hi = h2; }
                else if (tri == ZNN_TRI_A_UPPER) { lo = row0 / kBK < hi ? row0 / kBK : hi; }
                else if (tri == ZNN_TRI_B_LOWER) { lo = col0 / kBK < hi ? col0 / kBK : hi; }
                // a tile without k-blocks still has to be stored (zeros, or beta * C) unless it lies above the diagonal
                if (hi - lo <= 0 && tri == ZNN_TRI_C_LOWER) continue;
                ent[n].cost = hi - lo > 0 ? hi - lo : 0;
                ent[n].kf = (unsigned short)lo;
                ent[n].code = (unsigned short)((tm << 8) | tn);
                n++;
            }
        for (int i = 1; i < n; i++) {   // insertion sort, dearest first (stable)
            const Ent x = ent[i];
            int j = i - 1;
            while (j >= 0 && ent[j].cost < x.cost) { ent[j + 1] = ent[j]; j--; }
            ent[j + 1] = x;
        }
        for (int i = 0; i < n; i++) {
            p.tri_tab[i] = ent[i].code;
            p.tri_kf[i] = ent[i].kf;
            p.tri_kc[i] = (unsigned short)ent[i].cost;
        }
        p.tri_n = n;
    }
    p.alpha = alpha; p.beta = beta; p.C = C; p.ldc = ldc; p.stride_c = stride_c; p.status = status;
    p.wait_limit = g_wait_limit;
    if (pl.bn == 256) rc = launch_direct_major<256>(a_mn, b_mn, ma, mb, p, batch);
    else if (pl.bn == 128) rc = launch_direct_major<128>(a_mn, b_mn, ma, mb, p, batch);
    else rc = launch_direct_major<64>(a_mn, b_mn, ma, mb, p, batch);
    if (rc) return rc;
    if (tail_tiles > 0) {
        p.tail_slices = tail_slices;
        const dim3 grid((unsigned)(2 * kTileM * pl.bn / 4 / 256), (unsigned)tail_tiles, 1);   // one float4 per thread
        if (pl.bn == 256) tail_reduce_kernel<256><<<grid, 256, 0, stream()>>>(p);
        else if (pl.bn == 128) tail_reduce_kernel<128><<<grid, 256, 0, stream()>>>(p);
        else tail_reduce_kernel<64><<<grid, 256, 0, stream()>>>(p);
        ZNN_LAUNCH_OK("tail_reduce_kernel");
    }
    if (pl.splits > 1) return launch_splitk_reduce(partial, pl.splits, M, N, batch, alpha, beta, C, ldc, stride_c, bias);
    return ZNN_OK;
}

}  // namespace znn
