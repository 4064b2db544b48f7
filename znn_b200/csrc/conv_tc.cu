// Conv2D (NCHW, stride 1) as an implicit-im2col GEMM on the tensor cores (tcgen05, kind::tf32, 3xTF32 split).
//
// The im2col matrix col[p][k] (p = output pixel (n, h, w), k = (ci, kh, kw)) is never written to memory: producer
// warps gather its tiles from the input tensor straight into the swizzled shared-memory stages the tensor core reads,
// splitting every value into its TF32 head and the fp32 remainder on the way (rows of K = Ci*KH*KW taps are not
// boxes a TMA copy could fetch).
//
//   forward        Y[p, co]   = bias[co] + sum_k col(X)[p, k] * W[co, k]           rows = pixels, contraction = taps
//   data gradient  dX[q, ci] += sum_k' col(dY)[q, k'] * Wt[ci, k']                  the same kernel on dY with the
//                                                                                   flipped, channel-swapped weights
//   weight grad.   dW[co, k] += sum_p dY[p, co] * col(X)[p, k]                      rows = taps, contraction = pixels,
//                  dbias[co] += sum_p dY[p, co]                                     (an extra row of ones in col^T)
//
// One persistent CTA per SM (cta_group::1) walks 128-row output tiles: 8 producer warps fill a four-stage ring of
// [128 x 32] A and [NT x 32] B tiles (head and remainder planes), fetching the next k-block into registers while they
// split and store the current one; one warp issues the MMAs (remainder*head + head*remainder + head*head into one
// fp32 accumulator in tensor memory, two accumulators in turn); four epilogue warps add each finished chunk of 256
// contraction elements to fp32 registers (the tensor core's own accumulator truncates) and store the tile while the
// main loop of the next tile runs.
// Every wait is bounded; an expired wait sets a bit in the device status word and the CTA winds down.
//
// Reference arms: src/tensor.zig:523-585 (conv2d), src/autodiff.zig:929-995 (Conv2D backward).
#include "tc_ptx.cuh"

namespace znn {

unsigned long long tc_wait_limit();

namespace {

constexpr int kCvEpiWarps = 4;        // warps 0-3: tensor-memory lane quarter = warp index
constexpr int kCvMmaWarp = 4;
constexpr int kCvProducerWarp0 = 5;
constexpr int kCvProducerWarps = 8;
constexpr int kCvThreads = 32 * (kCvProducerWarp0 + kCvProducerWarps);
#ifndef ZNN_CV_STAGES
#define ZNN_CV_STAGES 4
#endif
constexpr int kCvStages = ZNN_CV_STAGES;
constexpr int kCvChunk = 8;          // k-blocks (of 32 contraction elements) per tensor-memory accumulation
constexpr int kCvSplitPixels = 512;  // pixels per unit of the weight-gradient product (two chunks)
constexpr int kCvABytes = 128 * 128; // one plane of the A tile: 128 rows of 32 floats

enum { CV_FWD = 0, CV_WGRAD = 1 };

// Optional role profile (compile with -DZNN_CONV_PROFILE; off in the product build): CTA 0 adds the cycles one lane of
// each role spends in its loop and in each part of it to g_conv_prof, read by znn_debug_conv_profile:
// [0] producer loop, [1] gather issue, [2] wait for a free stage, [3] split + store, [4] proxy fence, [5] hand-off;
// [6] MMA loop, [7] wait for a full stage, [8] wait for a drained accumulator, [9] issue;
// [10] epilogue loop, [11] wait for a finished chunk, [12] drain, [13] store.
__device__ long long g_conv_prof[16];
#ifdef ZNN_CONV_PROFILE
#define CV_PROF_DECL long long pa[16]; for (int i_ = 0; i_ < 16; i_++) pa[i_] = 0; long long pt = clock64(); const long long pt0 = pt;
#define CV_PROF(slot) { const long long n_ = clock64(); pa[slot] += n_ - pt; pt = n_; }
#define CV_PROF_END(total, on) if (on) { pa[total] = clock64() - pt0; for (int i_ = 0; i_ < 16; i_++) if (pa[i_]) atomicAdd((unsigned long long*)&g_conv_prof[i_], (unsigned long long)pa[i_]); }
#else
#define CV_PROF_DECL
#define CV_PROF(slot)
#define CV_PROF_END(total, on)
#endif

struct ConvTcParams {
    const float* src;    // the gathered tensor [N][C][H][W]: X (forward, weight gradient) or dY (data gradient)
    const float* bmat;   // forward: weight matrix [Co][K]; weight gradient: dY [N][Co][Ho][Wo]
    const float* bias;   // forward only (may be NULL)
    float* out;          // forward: [N][Co][Ho][Wo]; weight gradient: partial sums [split][rows][NT]
    int C, H, W;         // dimensions of src
    int KH, KW, pad_h, pad_w;
    int Ho, Wo;          // pixel grid the rows (forward) or the contraction (weight gradient) runs over
    int Co;              // columns of the product
    int K;               // C*KH*KW
    int kblocks;         // forward: ceil(K / 32)
    int rows;            // weight gradient: rows of the partial-sum matrix (a multiple of 128, > K)
    int nunits;          // forward: row tiles; weight gradient: splits * (rows / 128)
    long long P;         // N*Ho*Wo
    int accumulate;      // forward: out += product (no bias)
    int relu;            // forward, storing form: out = max(0, product + bias)
    int* status;
    unsigned long long wait_limit;
};

// One unit of work: a 128-row output tile (forward) or a (pixel split, 128 tap rows) pair (weight gradient).
struct ConvUnit {
    long long first;   // forward: first pixel row of the tile; weight gradient: first pixel of the split
    long long end;     // weight gradient: one past the split's last pixel
    int mt;            // weight gradient: which 128 tap rows
    int split;
    int nkb;
};

template <int MODE>
__device__ __forceinline__ ConvUnit conv_unit(const ConvTcParams& p, int u)
{
    ConvUnit d;
    if (MODE == CV_FWD) {
        d.first = (long long)u * 128;
        d.end = 0; d.mt = 0; d.split = 0;
        d.nkb = p.kblocks;
    } else {
        const int mts = p.rows / 128;
        d.split = u / mts;
        d.mt = u - d.split * mts;
        d.first = (long long)d.split * kCvSplitPixels;
        d.end = d.first + kCvSplitPixels < p.P ? d.first + kCvSplitPixels : p.P;
        d.nkb = (int)((d.end - d.first + 31) / 32);
    }
    return d;
}

__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo)
{
    hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);   // exactly a TF32 value
    lo = x - hi;                                              // exact in fp32
}

template <int MODE, int NT>
__global__ void __launch_bounds__(kCvThreads, 1) conv_tc_kernel(const ConvTcParams p)
{
    constexpr int kBBytes = NT * 128;
    constexpr int kStageBytes = 2 * kCvABytes + 2 * kBBytes;
    constexpr int kTmemCols = 2 * NT < 32 ? 32 : 2 * NT;
    constexpr int S = kCvStages;
    static_assert(NT == 32 || NT == 64, "column tile");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // layout: ring | barriers, words | tap table
    const uint32_t bar_base = smem_base + S * kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * S + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * S + 2 + b); };
    static_assert(8 * (2 * S + 4) <= 96, "barrier block");
    volatile uint32_t* const words = reinterpret_cast<volatile uint32_t*>(smem_gen + S * kStageBytes + 96);
    const uint32_t tmem_slot_addr = bar_base + 96;
    float* const sbias = reinterpret_cast<float*>(smem_gen + S * kStageBytes + 128);   // [NT], zero past Co
    int2* const tab = reinterpret_cast<int2*>(smem_gen + S * kStageBytes + 128 + NT * 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int HW = p.H * p.W, HoWo = p.Ho * p.Wo;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full_bar(s), kCvProducerWarps);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), kCvEpiWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        words[1] = (uint32_t)(*reinterpret_cast<volatile int*>(p.status));
    }
    if (warp == kCvMmaWarp) {
        tmem_alloc<1>(tmem_slot_addr, kTmemCols);
        tmem_relinquish<1>();
    }
    if (threadIdx.x < NT)
        sbias[threadIdx.x] = (MODE == CV_FWD && p.bias && (int)threadIdx.x < p.Co) ? p.bias[threadIdx.x] : 0.0f;
    // Table entry k = (ci, kh, kw): x = offset of the element from the row's own pixel, y = tap = kh * KW + kw, the bit
    // of the row's border mask that says whether the element lies inside the input (31 = beyond K: never valid).
    // Channel-major order keeps the taps of one channel together: they touch the same few cache lines.
    const int T = p.KH * p.KW;
    {
        const int nent = (MODE == CV_FWD) ? p.kblocks * 32 : p.rows;
        for (int k = threadIdx.x; k < nent; k += kCvThreads) {
            int2 e;
            if (k < p.K) {
                const int ci = k / T, tap = k - ci * T;
                const int kh = tap / p.KW, kw = tap - kh * p.KW;
                e.x = ci * HW + (kh - p.pad_h) * p.W + (kw - p.pad_w);
                e.y = tap;
            } else {
                e.x = 0;
                e.y = 31;
            }
            tab[k] = e;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = words[0];
    const bool aborted = (words[1] != 0);

    if (aborted) {
    } else if (warp >= kCvProducerWarp0) {
        // ---------------- producers: gather the next k-block into registers while the current one is stored ----------------
        const int t = threadIdx.x - 32 * kCvProducerWarp0;   // 0..255
        const int pw = warp - kCvProducerWarp0;
        float xa[16], xb[8];
        // load cursor
        int lu = blockIdx.x, lkb = 0;
        ConvUnit un = conv_unit<MODE>(p, lu < p.nunits ? lu : 0);
        // forward: this thread's row of the current tile
        const int r = t & 127, half = t >> 7;
        uint32_t rmask = 0;   // which taps of this row's pixel fall inside the input (bit = tap)
        long long rbase = 0;
        // bit tap = (h + kh - pad_h, w + kw - pad_w) lies inside the input
        auto tap_mask = [&](int h, int w) {
            uint32_t m = 0;
            for (int kh = 0, tap = 0; kh < p.KH; kh++) {
                const bool hin = (unsigned)(h + kh - p.pad_h) < (unsigned)p.H;
                for (int kw = 0; kw < p.KW; kw++, tap++)
                    if (hin && (unsigned)(w + kw - p.pad_w) < (unsigned)p.W) m |= 1u << tap;
            }
            return m;
        };
        auto load = [&]() {
            if (MODE == CV_FWD) {
                if (lkb == 0) {
                    const long long pp = un.first + r;
                    rmask = 0; rbase = 0;
                    if (pp < p.P) {
                        const int n = (int)(pp / HoWo), hw = (int)(pp - (long long)n * HoWo);
                        const int rh = hw / p.Wo, rw = hw - rh * p.Wo;
                        rbase = (long long)n * p.C * HW + (long long)rh * p.W + rw;
                        rmask = tap_mask(rh, rw);
                    }
                }
                // A: thread = row (consecutive pixels across the warp: coalesced), sixteen consecutive k'
                const float* const srow = p.src + rbase;
                const int kq0 = lkb * 32 + 16 * half;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int2 te = tab[kq0 + i];
                    xa[i] = ((rmask >> te.y) & 1u) ? __ldg(srow + te.x) : 0.0f;
                }
                // B: a row of the weight matrix, eight consecutive taps
                const int row = t >> 2, k0 = lkb * 32 + 8 * (t & 3);
                const float* const wrow = p.bmat + (long long)row * p.K + k0;
                const int nvalid = row < p.Co ? p.K - k0 : 0;
#pragma unroll
                for (int e = 0; e < 8; e++) xb[e] = e < nvalid ? __ldg(wrow + e) : 0.0f;
            } else {
                // lane = pixel of the k-block (consecutive pixels: coalesced), the warp walks the rows
                const long long pp = un.first + (long long)lkb * 32 + lane;
                const bool pvalid = pp < un.end;
                int n = 0, h = 0, w = 0, hw = 0;
                if (pvalid) {
                    n = (int)(pp / HoWo); hw = (int)(pp - (long long)n * HoWo);
                    h = hw / p.Wo; w = hw - h * p.Wo;
                }
                const float* const srow = p.src + (long long)n * p.C * HW + (long long)h * p.W + w;
                const uint32_t pmask = pvalid ? tap_mask(h, w) : 0u;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int kg = un.mt * 128 + 16 * pw + i;   // consecutive taps: the same few cache lines
                    const int2 te = tab[kg];
                    float x = ((pmask >> te.y) & 1u) ? __ldg(srow + te.x) : 0.0f;
                    if (kg == p.K) x = pvalid ? 1.0f : 0.0f;   // the bias row: sums dY over the pixels
                    xa[i] = x;
                }
                const float* const drow = p.bmat + (long long)n * p.Co * HoWo + hw;
#pragma unroll
                for (int i = 0; i < NT / kCvProducerWarps; i++) {
                    const int row = (NT / kCvProducerWarps) * pw + i;
                    xb[i] = (pvalid && row < p.Co) ? __ldg(drow + (long long)row * HoWo) : 0.0f;
                }
            }
        };
        bool have = lu < p.nunits, ok = true;
        if (have) load();
        uint32_t it = 0;
        CV_PROF_DECL
        while (have && ok) {
            CV_PROF(5)
            float ya[16], yb[8];
#pragma unroll
            for (int i = 0; i < 16; i++) ya[i] = xa[i];
#pragma unroll
            for (int i = 0; i < 8; i++) yb[i] = xb[i];
            if (++lkb == un.nkb) {
                lkb = 0;
                lu += gridDim.x;
                if (lu < p.nunits) un = conv_unit<MODE>(p, lu);
            }
            const bool have_next = lu < p.nunits;
            if (have_next) load();
            CV_PROF(1)
            const int s = it % S;
            bool got = true;
            got = __all_sync(0xffffffffu, mbar_wait_bounded_tight(empty_bar(s), (uint32_t)(((it / S) & 1) ^ 1), p.wait_limit));   // every lane polls, the warp votes
            if (!got) { ok = false; break; }
            CV_PROF(2)
            uint8_t* const st = smem_gen + s * kStageBytes;
            uint8_t* const sb = st + 2 * kCvABytes;
            if (MODE == CV_FWD) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float4 h4, l4;
                    split_tf32(ya[4 * j], h4.x, l4.x); split_tf32(ya[4 * j + 1], h4.y, l4.y);
                    split_tf32(ya[4 * j + 2], h4.z, l4.z); split_tf32(ya[4 * j + 3], h4.w, l4.w);
                    const int c = 4 * half + j;
                    const int off = r * 128 + ((c ^ (r & 7)) << 4);
                    *reinterpret_cast<float4*>(st + off) = h4;
                    *reinterpret_cast<float4*>(st + kCvABytes + off) = l4;
                }
                const int row = t >> 2;
                if (row < NT) {
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        float4 h4, l4;
                        split_tf32(yb[4 * j], h4.x, l4.x); split_tf32(yb[4 * j + 1], h4.y, l4.y);
                        split_tf32(yb[4 * j + 2], h4.z, l4.z); split_tf32(yb[4 * j + 3], h4.w, l4.w);
                        const int c = 2 * (t & 3) + j;
                        const int off = row * 128 + ((c ^ (row & 7)) << 4);
                        *reinterpret_cast<float4*>(sb + off) = h4;
                        *reinterpret_cast<float4*>(sb + kBBytes + off) = l4;
                    }
                }
            } else {
                const int soff = ((lane >> 2) << 4), sw = (lane & 3) * 4;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int row = 16 * pw + i;
                    float hi, lo;
                    split_tf32(ya[i], hi, lo);
                    const int off = row * 128 + (soff ^ ((row & 7) << 4)) + sw;
                    *reinterpret_cast<float*>(st + off) = hi;
                    *reinterpret_cast<float*>(st + kCvABytes + off) = lo;
                }
#pragma unroll
                for (int i = 0; i < NT / kCvProducerWarps; i++) {
                    const int row = (NT / kCvProducerWarps) * pw + i;
                    float hi, lo;
                    split_tf32(yb[i], hi, lo);
                    const int off = row * 128 + (soff ^ ((row & 7) << 4)) + sw;
                    *reinterpret_cast<float*>(sb + off) = hi;
                    *reinterpret_cast<float*>(sb + kBBytes + off) = lo;
                }
            }
            CV_PROF(3)
            // make the generic-proxy stores visible to the tensor core, then hand the stage over
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            CV_PROF(4)
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full_bar(s)) : "memory");
            it++;
            have = have_next;
        }
        CV_PROF_END(0, blockIdx.x == 0 && pw == 0 && lane == 0)
        if (!ok && lane == 0) atomicOr(p.status, ZNN_DEV_TMA_WAIT_EXPIRED);
    } else if (warp == kCvMmaWarp) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
        constexpr uint32_t idesc = make_tf32_idesc(128, NT);
        bool ok = true;
        uint32_t it = 0, cc = 0;
        CV_PROF_DECL
        for (int u = blockIdx.x; u < p.nunits && ok; u += gridDim.x) {
            const ConvUnit un = conv_unit<MODE>(p, u);
            for (int kb = 0; kb < un.nkb && ok; kb++, it++) {
                const int s = it % S;
                const int buf = cc & 1;
                bool got = true;
                CV_PROF(9)
                if (kb % kCvChunk == 0) {
                    // the drain of the chunk that used this accumulator two chunks ago
                    got = __all_sync(0xffffffffu, mbar_wait_bounded_tight(acc_empty_bar(buf), (uint32_t)(((cc >> 1) & 1) ^ 1), p.wait_limit));   // every lane polls, the warp votes
                    if (!got) { ok = false; break; }
                }
                CV_PROF(8)
                got = __all_sync(0xffffffffu, mbar_wait_bounded_tight(full_bar(s), (uint32_t)((it / S) & 1), p.wait_limit));   // every lane polls, the warp votes
                if (!got) { ok = false; break; }
                CV_PROF(7)
                tc_fence_after();
                const uint32_t st = smem_base + s * kStageBytes;
                const uint64_t a_hi = make_kmajor_sw128_desc(st), a_lo = make_kmajor_sw128_desc(st + kCvABytes);
                const uint64_t b_hi = make_kmajor_sw128_desc(st + 2 * kCvABytes);
                const uint64_t b_lo = make_kmajor_sw128_desc(st + 2 * kCvABytes + kBBytes);
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * NT);
                const bool fresh = (kb % kCvChunk == 0);
                const bool last = (kb % kCvChunk == kCvChunk - 1) || kb == un.nkb - 1;
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < 4; k++) umma_tf32<1>(d_tmem, a_lo + 2 * k, b_hi + 2 * k, idesc, (fresh && k == 0) ? 0u : 1u);
#pragma unroll
                    for (int k = 0; k < 4; k++) umma_tf32<1>(d_tmem, a_hi + 2 * k, b_lo + 2 * k, idesc, 1u);
#pragma unroll
                    for (int k = 0; k < 4; k++) umma_tf32<1>(d_tmem, a_hi + 2 * k, b_hi + 2 * k, idesc, 1u);
                    umma_commit_1cta(empty_bar(s));
                    if (last) umma_commit_1cta(acc_full_bar(buf));
                }
                __syncwarp();
                if (last) cc++;
            }
        }
        CV_PROF_END(6, blockIdx.x == 0 && lane == 0)
        if (!ok && lane == 0) atomicOr(p.status, ZNN_DEV_MMA_WAIT_EXPIRED);
    } else {
        // ---------------- epilogue: every finished chunk is added to fp32 registers, then the tile is stored ----------------
        const int q = warp;
        bool ok = true;
        uint32_t cc = 0;
        CV_PROF_DECL
        for (int u = blockIdx.x; u < p.nunits && ok; u += gridDim.x) {
            const ConvUnit un = conv_unit<MODE>(p, u);
            const int nchunks = (un.nkb + kCvChunk - 1) / kCvChunk;
            float acc[NT];
#pragma unroll
            for (int c = 0; c < NT; c++) acc[c] = 0.0f;
            for (int c = 0; c < nchunks && ok; c++, cc++) {
                const int buf = cc & 1;
                bool got = true;
                CV_PROF(13)
                got = __all_sync(0xffffffffu, mbar_wait_bounded_tight(acc_full_bar(buf), (uint32_t)((cc >> 1) & 1), p.wait_limit));   // every lane polls, the warp votes
                if (!got) { ok = false; break; }
                CV_PROF(11)
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < NT / 32; j++) {
                    float v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * NT + 32 * j), v);
#pragma unroll
                    for (int c2 = 0; c2 < 32; c2++) acc[32 * j + c2] += v[c2];
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty_bar(buf)) : "memory");
                CV_PROF(12)
            }
            if (!ok) break;
            if (MODE == CV_FWD) {
                const long long pp = un.first + 32 * q + lane;
                if (pp < p.P) {
                    const int n = (int)(pp / HoWo), hw = (int)(pp - (long long)n * HoWo);
                    float* const o = p.out + (long long)n * p.Co * HoWo + hw;
                    // sixteen channels at a time, the loads of the old values (accumulating form) issued together:
                    // one store per channel, each a run of consecutive pixels across the warp
#pragma unroll
                    for (int c0 = 0; c0 < NT; c0 += 16) {
                        float add[16];
                        if (p.accumulate) {
#pragma unroll
                            for (int j = 0; j < 16; j++) add[j] = (c0 + j < p.Co) ? o[(long long)(c0 + j) * HoWo] : 0.0f;
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j++) add[j] = sbias[c0 + j];
                        }
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (c0 + j < p.Co) {
                                const float v = acc[c0 + j] + add[j];
                                o[(long long)(c0 + j) * HoWo] = p.relu ? fmaxf(v, 0.0f) : v;
                            }
                    }
                }
            } else {
                const int kg = un.mt * 128 + 32 * q + lane;
                float4* const o = reinterpret_cast<float4*>(p.out + ((long long)un.split * p.rows + kg) * NT);
#pragma unroll
                for (int c = 0; c < NT / 4; c++) o[c] = make_float4(acc[4 * c], acc[4 * c + 1], acc[4 * c + 2], acc[4 * c + 3]);
            }
        }
        CV_PROF(13)
        CV_PROF_END(10, blockIdx.x == 0 && q == 0 && lane == 0)
        if (!ok && lane == 0) atomicOr(p.status, ZNN_DEV_EPI_WAIT_EXPIRED);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kCvMmaWarp) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

// dW[co][k] += sum over the splits of partial[split][k][co]; dbias[co] += the same of row K
__global__ void conv_wgrad_reduce_kernel(const float* __restrict__ partial, int splits, int rows, int nt, int K, int Co,
                                         float* __restrict__ dW, float* __restrict__ dbias)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;   // (k, co), co fastest
    if (i >= (K + 1) * Co) return;
    const int k = i / Co, co = i - k * Co;
    if (k == K && !dbias) return;
    if (k < K && !dW) return;
    const float* src = partial + (size_t)k * nt + co;
    const size_t pitch = (size_t)rows * nt;
    float s = 0.0f;
    int sp = 0;
    for (; sp + 8 <= splits; sp += 8) {   // eight loads in flight, added in split order
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = src[(size_t)(sp + u) * pitch];
#pragma unroll
        for (int u = 0; u < 8; u++) s += v[u];
    }
    for (; sp < splits; sp++) s += src[(size_t)sp * pitch];
    if (k == K) dbias[co] += s;
    else dW[(size_t)co * K + k] += s;
}

// Wt[ci][(co, kh, kw)] = W[co][ci][KH-1-kh][KW-1-kw]: the data gradient is a convolution of dY with these
__global__ void conv_flip_weights_kernel(const float* __restrict__ W, float* __restrict__ Wt, int Co, int Ci, int KH, int KW)
{
    const int total = Co * Ci * KH * KW;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int kw = i % KW, kh = (i / KW) % KH, co = (i / (KW * KH)) % Co, ci = i / (KW * KH * Co);
    Wt[i] = W[(((size_t)co * Ci + ci) * KH + (KH - 1 - kh)) * KW + (KW - 1 - kw)];
}

template <int MODE, int NT>
int launch_conv_tc(const ConvTcParams& p)
{
    static bool attr_set[64] = {};
    int dev = 0;
    ZNN_CUDA_OK(cudaGetDevice(&dev));
    const int tab = (MODE == CV_FWD) ? p.kblocks * 32 : p.rows;
    const size_t smem = (size_t)kCvStages * (2 * kCvABytes + 2 * NT * 128) + 1024 + 128 + NT * 4 + (size_t)tab * sizeof(int2);
    if (smem > 227 * 1024) return fail(ZNN_ERR_UNSUPPORTED, "conv tensor path: tap table beyond shared memory");
    if (dev < 64 && !attr_set[dev]) {
        ZNN_CUDA_OK(cudaFuncSetAttribute(conv_tc_kernel<MODE, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev] = true;
    }
    const int grid = p.nunits < sm_count() ? p.nunits : sm_count();
    conv_tc_kernel<MODE, NT><<<grid, kCvThreads, smem, stream()>>>(p);
    ZNN_LAUNCH_OK("conv_tc_kernel");
    return ZNN_OK;
}

}  // namespace

int conv_profile_read(long long* out16)
{
    ZNN_CUDA_OK(cudaStreamSynchronize(stream()));
    ZNN_CUDA_OK(cudaMemcpyFromSymbol(out16, g_conv_prof, sizeof(long long) * 16));
    long long zero[16] = {};
    ZNN_CUDA_OK(cudaMemcpyToSymbol(g_conv_prof, zero, sizeof(zero)));
    return ZNN_OK;
}

static thread_local int t_conv_path = 0;   // 0 = automatic, 1 = never the tensor path
void conv_set_path(int mode) { t_conv_path = mode; }

// Which layers take the tensor path: enough taps to fill k-blocks (K >= 64), at most 64 output channels per tile,
// enough pixels to fill the machine, at most 31 kernel positions (one bit each in the border mask), 32-bit offsets.
bool conv_tc_applicable(long long n, int C, int H, int W, int Co, int KH, int KW, int Ho, int Wo)
{
    if (t_conv_path == 1) return false;
    const long long K = (long long)C * KH * KW, P = n * Ho * Wo;
    if (K < 64 || K > 1536 || Co > 64 || P < 4096 || KH * KW > 31) return false;
    if (n * C * H * W >= (1ll << 31) || P * Co >= (1ll << 31)) return false;
    if (H >= 16384 || W >= 16384) return false;
    return true;
}

// out[N][Co][Ho][Wo] (= bias +) or (+=) conv(src[N][C][H][W], wm[Co][C*KH*KW]) with zero padding (pad_h, pad_w)
int conv_tc_forward(const float* src, const float* wm, const float* bias, float* out, int N, int C, int H, int W, int Co,
                    int KH, int KW, int pad_h, int pad_w, int accumulate)
{
    ConvTcParams p{};
    // accumulate: 0 = store product + bias, 1 = add the product to out (no bias), 2 = store max(0, product + bias)
    p.relu = (accumulate == 2);
    if (accumulate == 2) accumulate = 0;
    p.src = src; p.bmat = wm; p.bias = accumulate ? nullptr : bias; p.out = out;
    p.C = C; p.H = H; p.W = W; p.KH = KH; p.KW = KW; p.pad_h = pad_h; p.pad_w = pad_w;
    p.Ho = H + 2 * pad_h - KH + 1; p.Wo = W + 2 * pad_w - KW + 1;
    p.Co = Co; p.K = C * KH * KW; p.kblocks = (p.K + 31) / 32;
    p.P = (long long)N * p.Ho * p.Wo;
    p.accumulate = accumulate;
    p.status = device_status_word();
    p.wait_limit = tc_wait_limit();
    if (!p.status) return fail(ZNN_ERR_CUDA, "no device state (call znn_init first)");
    p.nunits = (int)((p.P + 127) / 128);
    return Co <= 32 ? launch_conv_tc<CV_FWD, 32>(p) : launch_conv_tc<CV_FWD, 64>(p);
}

// dW[Co][K] += dY^T . col(X), dbias[Co] += column sums of dY; `scratch` holds splits * rows * NT floats
size_t conv_tc_wgrad_scratch(long long P, int K, int Co)
{
    const long long splits = (P + kCvSplitPixels - 1) / kCvSplitPixels;
    const int rows = (K + 1 + 127) / 128 * 128;
    return (size_t)splits * rows * (Co <= 32 ? 32 : 64);
}

int conv_tc_wgrad(const float* X, const float* dY, float* dW, float* dbias, float* scratch, int N, int Ci, int H, int W,
                  int Co, int KH, int KW, int pad, int Ho, int Wo)
{
    ConvTcParams p{};
    p.src = X; p.bmat = dY; p.out = scratch;
    p.C = Ci; p.H = H; p.W = W; p.KH = KH; p.KW = KW; p.pad_h = pad; p.pad_w = pad;
    p.Ho = Ho; p.Wo = Wo; p.Co = Co; p.K = Ci * KH * KW;
    p.rows = (p.K + 1 + 127) / 128 * 128;
    p.P = (long long)N * Ho * Wo;
    p.status = device_status_word();
    p.wait_limit = tc_wait_limit();
    if (!p.status) return fail(ZNN_ERR_CUDA, "no device state (call znn_init first)");
    const int splits = (int)((p.P + kCvSplitPixels - 1) / kCvSplitPixels);
    p.nunits = splits * (p.rows / 128);
    const int nt = Co <= 32 ? 32 : 64;
    int rc = Co <= 32 ? launch_conv_tc<CV_WGRAD, 32>(p) : launch_conv_tc<CV_WGRAD, 64>(p);
    if (rc) return rc;
    const int total = (p.K + 1) * Co;
    conv_wgrad_reduce_kernel<<<(total + 63) / 64, 64, 0, stream()>>>(scratch, splits, p.rows, nt, p.K, Co, dW, dbias);
    ZNN_LAUNCH_OK("conv_wgrad_reduce_kernel");
    return ZNN_OK;
}

// dX[N][Ci][H][W] += conv(dY[N][Co][Ho][Wo], flipped weights) ; `wt` holds Ci * Co*KH*KW floats
int conv_tc_dgrad(const float* dY, const float* Wgt, float* dX, float* wt, int N, int Ci, int H, int W, int Co, int KH, int KW,
                  int pad, int Ho, int Wo)
{
    const int total = Co * Ci * KH * KW;
    conv_flip_weights_kernel<<<(total + 255) / 256, 256, 0, stream()>>>(Wgt, wt, Co, Ci, KH, KW);
    ZNN_LAUNCH_OK("conv_flip_weights_kernel");
    return conv_tc_forward(dY, wt, nullptr, dX, N, Co, Ho, Wo, Ci, KH, KW, KH - 1 - pad, KW - 1 - pad, 1);
}

}  // namespace znn
