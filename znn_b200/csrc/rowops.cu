// Row-wise and elementwise operators of the znn hot path (HBM-bound kernels).
// Compiled with -fmad=false: the reference rounds every product before the add
// (Zig does not contract), and these kernels are bandwidth-bound, so keeping the
// same rounding points costs nothing and keeps results close to bit-identical.
#include <math_constants.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace znn {

constexpr int kEwThreads = 256;

static inline int ew_blocks(size_t n, int per_thread = 4)
{
    size_t b = (n + (size_t)kEwThreads * per_thread - 1) / ((size_t)kEwThreads * per_thread);
    const size_t cap = (size_t)sm_count() * 32;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// block-wide reductions for up to 1024 threads; result valid in every thread
__device__ __forceinline__ float block_sum(float v, float* sh)
{
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float t = (lane < nw) ? sh[lane] : 0.0f;
    return warp_sum(t);
}

__device__ __forceinline__ float block_max(float v, float* sh)
{
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float t = (lane < nw) ? sh[lane] : -CUDART_INF_F;
    return warp_max(t);
}

// ---------------------------------------------------------------------------
// elementwise: 128-bit accesses when both pointers are 16-byte aligned
// ---------------------------------------------------------------------------
template <class F>
__global__ void ew1_kernel(const float* __restrict__ a, float* __restrict__ out, size_t n, F f)
{
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const bool vec = (((uintptr_t)a | (uintptr_t)out) & 15) == 0;
    const size_t n4 = vec ? n / 4 : 0;
    for (size_t i = tid; i < n4; i += nth) {
        const float4 x = reinterpret_cast<const float4*>(a)[i];
        float4 o = reinterpret_cast<float4*>(out)[i];
        o.x = f(x.x, o.x); o.y = f(x.y, o.y); o.z = f(x.z, o.z); o.w = f(x.w, o.w);
        reinterpret_cast<float4*>(out)[i] = o;
    }
    for (size_t i = n4 * 4 + tid; i < n; i += nth) out[i] = f(a[i], out[i]);
}

template <class F>
__global__ void ew2_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, size_t n, F f)
{
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const bool vec = (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0;
    const size_t n4 = vec ? n / 4 : 0;
    for (size_t i = tid; i < n4; i += nth) {
        const float4 x = reinterpret_cast<const float4*>(a)[i];
        const float4 y = reinterpret_cast<const float4*>(b)[i];
        float4 o = reinterpret_cast<float4*>(out)[i];
        o.x = f(x.x, y.x, o.x); o.y = f(x.y, y.y, o.y); o.z = f(x.z, y.z, o.z); o.w = f(x.w, y.w, o.w);
        reinterpret_cast<float4*>(out)[i] = o;
    }
    for (size_t i = n4 * 4 + tid; i < n; i += nth) out[i] = f(a[i], b[i], out[i]);
}

// write-only variants (the old value of out is not read)
template <class F>
__global__ void ew1w_kernel(const float* __restrict__ a, float* __restrict__ out, size_t n, F f)
{
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const bool vec = (((uintptr_t)a | (uintptr_t)out) & 15) == 0;
    const size_t n4 = vec ? n / 4 : 0;
    for (size_t i = tid; i < n4; i += nth) {
        const float4 x = reinterpret_cast<const float4*>(a)[i];
        float4 o;
        o.x = f(x.x); o.y = f(x.y); o.z = f(x.z); o.w = f(x.w);
        reinterpret_cast<float4*>(out)[i] = o;
    }
    for (size_t i = n4 * 4 + tid; i < n; i += nth) out[i] = f(a[i]);
}

template <class F>
__global__ void ew2w_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, size_t n, F f)
{
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const bool vec = (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0;
    const size_t n4 = vec ? n / 4 : 0;
    for (size_t i = tid; i < n4; i += nth) {
        const float4 x = reinterpret_cast<const float4*>(a)[i];
        const float4 y = reinterpret_cast<const float4*>(b)[i];
        float4 o;
        o.x = f(x.x, y.x); o.y = f(x.y, y.y); o.z = f(x.z, y.z); o.w = f(x.w, y.w);
        reinterpret_cast<float4*>(out)[i] = o;
    }
    for (size_t i = n4 * 4 + tid; i < n; i += nth) out[i] = f(a[i], b[i]);
}

struct ReluF { __device__ float operator()(float x) const { return x > 0.0f ? x : 0.0f; } };
struct GeluF {
    __device__ float operator()(float x) const
    {
        const float sqrt_2 = 1.41421356237309504880f;
        return 0.5f * x * (1.0f + erff(x / sqrt_2));
    }
};
struct ReluBwdF { __device__ float operator()(float a, float dc, float da) const { return da + (a > 0.0f ? dc : 0.0f); } };
struct GeluBwdF {
    __device__ float operator()(float x, float dc, float da) const
    {
        const float sqrt_2 = 1.41421356237309504880f;
        const float inv_sqrt_2pi = 0.3989422804014327f;
        const float cdf = 0.5f * (1.0f + erff(x / sqrt_2));
        const float pdf = inv_sqrt_2pi * expf(-0.5f * x * x);
        return da + dc * (cdf + x * pdf);
    }
};
struct GeluBwdSetF {   // the same derivative, stored instead of added
    __device__ float operator()(float x, float dc) const
    {
        const float sqrt_2 = 1.41421356237309504880f;
        const float inv_sqrt_2pi = 0.3989422804014327f;
        const float cdf = 0.5f * (1.0f + erff(x / sqrt_2));
        const float pdf = inv_sqrt_2pi * expf(-0.5f * x * x);
        return dc * (cdf + x * pdf);
    }
};
struct AddF { __device__ float operator()(float a, float b) const { return a + b; } };
struct AccF { __device__ float operator()(float s, float d) const { return d + s; } };
struct MulF { float v; __device__ float operator()(float a) const { return a * v; } };
struct MulAccF { float v; __device__ float operator()(float dc, float da) const { return da + dc * v; } };

// dst[i] = i mod period: the position ids of a [batch, T] window (src/nn.zig:1183-1196 builds them on the host)
__global__ void iota_mod_kernel(float* dst, size_t n, int period)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = (float)(i % (size_t)period);
}

__global__ void fill_kernel(float* dst, float v, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = v;
}

// ---------------------------------------------------------------------------
// AddBias
// ---------------------------------------------------------------------------
__global__ void add_bias_fwd_kernel(const float* __restrict__ A, const float* __restrict__ bias, float* __restrict__ C,
                                    size_t total, int N)
{
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const bool vec = ((N & 3) == 0) && ((((uintptr_t)A | (uintptr_t)C | (uintptr_t)bias) & 15) == 0);
    if (vec) {
        const size_t t4 = total / 4;
        const int n4 = N / 4;
        for (size_t i = tid; i < t4; i += nth) {
            const float4 a = reinterpret_cast<const float4*>(A)[i];
            const float4 b = reinterpret_cast<const float4*>(bias)[i % n4];
            float4 o;
            o.x = a.x + b.x; o.y = a.y + b.y; o.z = a.z + b.z; o.w = a.w + b.w;
            reinterpret_cast<float4*>(C)[i] = o;
        }
    } else {
        for (size_t i = tid; i < total; i += nth) C[i] = A[i] + bias[i % N];
    }
}

// Column sums in two deterministic stages.  Stage 1: block (32 columns x 8 row
// lanes) walks a chunk of rows; the 8 row lanes are summed in fixed order and the
// chunk's partial goes to scratch[chunk][n].  Stage 2 adds the chunk partials in
// order into out[n].  `PassThrough` also does dA += dC on the way (AddBias backward).
template <bool PassThrough>
__global__ void colsum_stage1_kernel(const float* __restrict__ dC, float* __restrict__ dA, float* __restrict__ partial,
                                     int M, int N, int rows_per_chunk, unsigned* __restrict__ counters, float* __restrict__ out)
{
    __shared__ float sh[8][33];
    __shared__ bool last;
    const int n = blockIdx.x * 32 + threadIdx.x;
    const int m0 = blockIdx.y * rows_per_chunk;
    const int m1 = min(M, m0 + rows_per_chunk);
    float s = 0.0f;
    if (n < N) {
        for (int m = m0 + threadIdx.y; m < m1; m += 8) {
            const float g = dC[(size_t)m * N + n];
            if (PassThrough) dA[(size_t)m * N + n] += g;
            s += g;
        }
    }
    sh[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && n < N) {
        float t = 0.0f;
#pragma unroll
        for (int y = 0; y < 8; y++) t += sh[y][threadIdx.x];
        partial[(size_t)blockIdx.y * N + n] = t;
    }
    if (!counters) return;   // the caller runs the second stage as its own kernel
    // The chunk that finishes last for these 32 columns adds all chunk partials in chunk order (the same order whichever
    // chunk that is: the result does not depend on the scheduling) and leaves the counter at zero for the next launch.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0) last = (atomicAdd(&counters[blockIdx.x], 1u) == gridDim.y - 1);
    __syncthreads();
    if (!last) return;
    __threadfence();
    float t = 0.0f;
    if (n < N)
        for (int c = threadIdx.y; c < (int)gridDim.y; c += 8) t += __ldcg(partial + (size_t)c * N + n);
    __syncthreads();
    sh[threadIdx.y][threadIdx.x] = t;
    __syncthreads();
    if (threadIdx.y == 0 && n < N) {
        float u = 0.0f;
#pragma unroll
        for (int y = 0; y < 8; y++) u += sh[y][threadIdx.x];
        out[n] += u;
    }
    if (threadIdx.x == 0 && threadIdx.y == 0) counters[blockIdx.x] = 0u;
}

// The same with 16-byte accesses: a block covers 128 columns (each lane four), its eight warps walk the chunk's rows
// eight apart (512 contiguous bytes per warp and row instead of 128).  N a multiple of 4, 16-byte aligned pointers.
template <bool PassThrough>
__global__ void __launch_bounds__(256)
colsum_vec_kernel(const float* __restrict__ dC, float* __restrict__ dA, float* __restrict__ partial, int M, int N,
                  int rows_per_chunk, unsigned* __restrict__ counters, float* __restrict__ out)
{
    __shared__ float4 sh[8][33];
    __shared__ bool last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * 128 + 4 * lane;
    const int m0 = blockIdx.y * rows_per_chunk;
    const int m1 = min(M, m0 + rows_per_chunk);
    float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (n < N) {
        int m = m0 + warp;
        for (; m + 24 < m1; m += 32) {   // four rows in flight per lane
            float4 g[4];
#pragma unroll
            for (int u = 0; u < 4; u++) g[u] = *reinterpret_cast<const float4*>(dC + (size_t)(m + 8 * u) * N + n);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (PassThrough) {
                    float4* a = reinterpret_cast<float4*>(dA + (size_t)(m + 8 * u) * N + n);
                    float4 o = *a;
                    o.x += g[u].x; o.y += g[u].y; o.z += g[u].z; o.w += g[u].w;
                    *a = o;
                }
                s.x += g[u].x; s.y += g[u].y; s.z += g[u].z; s.w += g[u].w;
            }
        }
        for (; m < m1; m += 8) {
            const float4 g = *reinterpret_cast<const float4*>(dC + (size_t)m * N + n);
            if (PassThrough) {
                float4* a = reinterpret_cast<float4*>(dA + (size_t)m * N + n);
                float4 o = *a;
                o.x += g.x; o.y += g.y; o.z += g.z; o.w += g.w;
                *a = o;
            }
            s.x += g.x; s.y += g.y; s.z += g.z; s.w += g.w;
        }
    }
    sh[warp][lane] = s;
    __syncthreads();
    if (warp == 0 && n < N) {
        float4 t = sh[0][lane];
#pragma unroll
        for (int y = 1; y < 8; y++) { const float4 v = sh[y][lane]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
        *reinterpret_cast<float4*>(partial + (size_t)blockIdx.y * N + n) = t;
    }
    if (!counters) return;   // the caller runs the second stage as its own kernel
    // the chunk that finishes last for these columns adds all chunk partials in chunk order and resets the counter
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = (atomicAdd(&counters[blockIdx.x], 1u) == gridDim.y - 1);
    __syncthreads();
    if (!last) return;
    __threadfence();
    float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (n < N)
        for (int c = warp; c < (int)gridDim.y; c += 8) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + (size_t)c * N + n));
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
    __syncthreads();
    sh[warp][lane] = t;
    __syncthreads();
    if (warp == 0 && n < N) {
        float4 u = sh[0][lane];
#pragma unroll
        for (int y = 1; y < 8; y++) { const float4 v = sh[y][lane]; u.x += v.x; u.y += v.y; u.z += v.z; u.w += v.w; }
        float4* o = reinterpret_cast<float4*>(out + n);
        float4 w = *o;
        w.x += u.x; w.y += u.y; w.z += u.z; w.w += u.w;
        *o = w;
    }
    if (threadIdx.x == 0) counters[blockIdx.x] = 0u;
}

// block = 32 columns x 8 lanes; lane y adds chunks y, y+8, ... in order, then the 8 lane sums are added in order
__global__ void colsum_stage2_kernel(const float* __restrict__ partial, float* __restrict__ out, int chunks, int N)
{
    __shared__ float sh[8][33];
    const int n = blockIdx.x * 32 + threadIdx.x;
    float t = 0.0f;
    if (n < N)
        for (int c = threadIdx.y; c < chunks; c += 8) t += partial[(size_t)c * N + n];
    sh[threadIdx.y][threadIdx.x] = t;
    __syncthreads();
    if (threadIdx.y == 0 && n < N) {
        float u = 0.0f;
#pragma unroll
        for (int y = 0; y < 8; y++) u += sh[y][threadIdx.x];
        out[n] += u;
    }
}

// same, for sum over rows of a[m,n] * b[m,n] * rowscale[m]  (RmsNorm / LayerNorm parameter gradients)
template <int Mode>  // 0: dy*x*scale (rms dG), 1: dy*(x-mean)*rstd (ln dG), 2: dy (ln dB)
__global__ void colsum_norm_stage1_kernel(const float* __restrict__ dY, const float* __restrict__ X,
                                          const float* __restrict__ rowstat, float* __restrict__ partial, int M, int N,
                                          int rows_per_chunk)
{
    __shared__ float sh[8][33];
    const int n = blockIdx.x * 32 + threadIdx.x;
    const int m0 = blockIdx.y * rows_per_chunk;
    const int m1 = min(M, m0 + rows_per_chunk);
    float s = 0.0f;
    if (n < N) {
        for (int m = m0 + threadIdx.y; m < m1; m += 8) {
            const float dy = dY[(size_t)m * N + n];
            if (Mode == 0) s += dy * X[(size_t)m * N + n] * rowstat[m];
            else if (Mode == 1) s += dy * ((X[(size_t)m * N + n] - rowstat[2 * m]) * rowstat[2 * m + 1]);
            else s += dy;
        }
    }
    sh[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && n < N) {
        float t = 0.0f;
#pragma unroll
        for (int y = 0; y < 8; y++) t += sh[y][threadIdx.x];
        partial[(size_t)blockIdx.y * N + n] = t;
    }
}

static void colsum_plan(int M, int& chunks, int& rows_per_chunk)
{
    chunks = (M + 63) / 64;
    if (chunks > 256) chunks = 256;
    if (chunks < 1) chunks = 1;
    rows_per_chunk = (M + chunks - 1) / chunks;
    chunks = (M + rows_per_chunk - 1) / rows_per_chunk;
    if (chunks < 1) chunks = 1;
}

// ---------------------------------------------------------------------------
// SoftmaxCrossEntropy
// ---------------------------------------------------------------------------
template <class TargetT>
__global__ void softmax_xent_fwd_kernel(const float* __restrict__ logits, const TargetT* __restrict__ targets,
                                        float* __restrict__ probs, float* __restrict__ rowloss, int N,
                                        int* __restrict__ status)
{
    __shared__ float sh[32];
    const size_t row = blockIdx.x;
    const float* x = logits + row * N;
    float* p = probs + row * N;
    float mx = -CUDART_INF_F;
    for (int j = threadIdx.x; j < N; j += blockDim.x) mx = fmaxf(mx, x[j]);
    mx = block_max(mx, sh);
    float sum = 0.0f;
    for (int j = threadIdx.x; j < N; j += blockDim.x) sum += expf(x[j] - mx);
    sum = block_sum(sum, sh);
    for (int j = threadIdx.x; j < N; j += blockDim.x) p[j] = expf(x[j] - mx) / sum;
    if (threadIdx.x == 0) {
        const int t = (int)targets[row];
        if (t < 0 || t >= N) {
            // a label outside [0, N): nothing is read through it; the row's loss (and so the mean) becomes NaN and the
            // device status word says why (the reference asserts on the same condition)
            rowloss[row] = CUDART_NAN_F;
            if (status) atomicOr(status, ZNN_DEV_BAD_INDEX);
        } else {
            const float pt = expf(x[t] - mx) / sum;
            rowloss[row] = -logf(fmaxf(pt, 1e-15f));
        }
    }
}

// Rows of at most 1024*V4 logits with N % 4 == 0: one 128-bit read of the row into registers, one write of
// the probabilities.
template <class TargetT, int V4>
__global__ void __launch_bounds__(256)
softmax_xent_fwd_reg_kernel(const float* __restrict__ logits, const TargetT* __restrict__ targets,
                            float* __restrict__ probs, float* __restrict__ rowloss, int N, int* __restrict__ status)
{
    __shared__ float sh[32];
    const size_t row = blockIdx.x;
    const float4* x = reinterpret_cast<const float4*>(logits + row * N);
    float4* p = reinterpret_cast<float4*>(probs + row * N);
    const int n4 = N >> 2;
    float4 v[V4];
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int j4 = threadIdx.x + 256 * k;
        if (j4 < n4) {
            v[k] = x[j4];
            mx = fmaxf(mx, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
        }
    }
    mx = block_max(mx, sh);
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int j4 = threadIdx.x + 256 * k;
        if (j4 < n4) {
            v[k].x = expf(v[k].x - mx); v[k].y = expf(v[k].y - mx);
            v[k].z = expf(v[k].z - mx); v[k].w = expf(v[k].w - mx);
            sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
    }
    sum = block_sum(sum, sh);
    const int t = (int)targets[row];
    if ((t < 0 || t >= N) && threadIdx.x == 0) {   // see softmax_xent_fwd_kernel
        rowloss[row] = CUDART_NAN_F;
        if (status) atomicOr(status, ZNN_DEV_BAD_INDEX);
    }
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int j4 = threadIdx.x + 256 * k;
        if (j4 < n4) {
            float4 o;
            o.x = v[k].x / sum; o.y = v[k].y / sum; o.z = v[k].z / sum; o.w = v[k].w / sum;
            p[j4] = o;
            if ((t >> 2) == j4) {
                const float pt = (t & 3) == 0 ? o.x : (t & 3) == 1 ? o.y : (t & 3) == 2 ? o.z : o.w;
                rowloss[row] = -logf(fmaxf(pt, 1e-15f));
            }
        }
    }
}

// mean of M per-row losses, summed in a fixed order
__global__ void mean_rows_kernel(const float* __restrict__ rowloss, float* __restrict__ loss, int M)
{
    __shared__ float sh[32];
    float s = 0.0f;
    for (int i = threadIdx.x; i < M; i += blockDim.x) s += rowloss[i];
    s = block_sum(s, sh);
    if (threadIdx.x == 0) loss[0] = s / (float)M;
}

template <class TargetT>
__global__ void softmax_xent_bwd_kernel(const float* __restrict__ probs, const TargetT* __restrict__ targets,
                                        float* __restrict__ dlogits, int M, int N)
{
    const float scale = 1.0f / (float)M;
    const size_t total = (size_t)M * N;
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    if ((N & 3) == 0 && ((((uintptr_t)probs | (uintptr_t)dlogits) & 15) == 0)) {
        const size_t n4 = (size_t)(N >> 2);
        for (size_t i = tid; i < total / 4; i += nth) {
            const size_t r = i / n4;
            const int j = (int)(i - r * n4) * 4;
            const int t = (int)targets[r];
            const float4 p = reinterpret_cast<const float4*>(probs)[i];
            float4 d = reinterpret_cast<float4*>(dlogits)[i];
            d.x += scale * (p.x - (j == t ? 1.0f : 0.0f));
            d.y += scale * (p.y - (j + 1 == t ? 1.0f : 0.0f));
            d.z += scale * (p.z - (j + 2 == t ? 1.0f : 0.0f));
            d.w += scale * (p.w - (j + 3 == t ? 1.0f : 0.0f));
            reinterpret_cast<float4*>(dlogits)[i] = d;
        }
        return;
    }
    for (size_t i = tid; i < total; i += nth) {
        const size_t r = i / N;
        const int j = (int)(i - r * N);
        const float ind = (j == (int)targets[r]) ? 1.0f : 0.0f;
        dlogits[i] += scale * (probs[i] - ind);
    }
}

// ---------------------------------------------------------------------------
// Softmax rows (one warp per row)
// ---------------------------------------------------------------------------
// Causal = true: row i of each T x T slice sees columns j <= i of scale*S; the
// reference adds -1e9 to the others, whose exp underflows to exactly 0.
template <bool Causal>
__global__ void softmax_rows_fwd_kernel(const float* __restrict__ S, float scale, float* __restrict__ P, size_t rows, int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = S + row * D;
    float* p = P + row * D;
    const int lim = Causal ? (int)(row % D) + 1 : D;  // number of visible columns
    float mx = -CUDART_INF_F;
    for (int j = lane; j < lim; j += 32) mx = fmaxf(mx, Causal ? x[j] * scale : x[j]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int j = lane; j < lim; j += 32) sum += expf((Causal ? x[j] * scale : x[j]) - mx);
    sum = warp_sum(sum);
    for (int j = lane; j < D; j += 32) p[j] = (j < lim) ? expf((Causal ? x[j] * scale : x[j]) - mx) / sum : 0.0f;
}

// Same, for rows of at most 128*V4 elements with D % 4 == 0: the row is read once with 128-bit loads,
// kept in registers, and written once.
template <bool Causal, int V4>
__global__ void softmax_rows_reg_kernel(const float* __restrict__ S, float scale, float* __restrict__ P, size_t rows, int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float4* x = reinterpret_cast<const float4*>(S + row * D);
    float4* p = reinterpret_cast<float4*>(P + row * D);
    const int lim = Causal ? (int)(row % D) + 1 : D;
    float4 v[V4];
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int j = 4 * (lane + 32 * k);
        if (j < lim) {
            float4 t = x[lane + 32 * k];
            if (Causal) { t.x *= scale; t.y *= scale; t.z *= scale; t.w *= scale; }
            if (j + 1 >= lim) t.y = -CUDART_INF_F;
            if (j + 2 >= lim) t.z = -CUDART_INF_F;
            if (j + 3 >= lim) t.w = -CUDART_INF_F;
            v[k] = t;
            mx = fmaxf(mx, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
        } else {
            v[k] = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        }
    }
    mx = warp_max(mx);
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int j = 4 * (lane + 32 * k);
        if (j < lim) {
            float4 e;
            e.x = expf(v[k].x - mx);
            e.y = (j + 1 < lim) ? expf(v[k].y - mx) : 0.0f;
            e.z = (j + 2 < lim) ? expf(v[k].z - mx) : 0.0f;
            e.w = (j + 3 < lim) ? expf(v[k].w - mx) : 0.0f;
            v[k] = e;
            sum += (e.x + e.y) + (e.z + e.w);
        }
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int j = 4 * (lane + 32 * k);
        if (j < D) {
            float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (j < lim) { o.x = v[k].x / sum; o.y = v[k].y / sum; o.z = v[k].z / sum; o.w = v[k].w / sum; }
            p[lane + 32 * k] = o;
        }
    }
}

// dA += scale * Y * (dY - sum(dY*Y))   (scale = 1 for the plain Softmax op)
// set = 1 stores the gradient (zeros beyond the causal limit) instead of adding it
__global__ void softmax_rows_bwd_kernel(const float* __restrict__ Y, const float* __restrict__ dY, float scale,
                                        float* __restrict__ dA, size_t rows, int D, int causal, int set = 0)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* y = Y + row * D;
    const float* dy = dY + row * D;
    float* da = dA + row * D;
    const int lim = causal ? (int)(row % D) + 1 : D;  // Y is exactly 0 beyond lim
    float s = 0.0f;
    for (int j = lane; j < lim; j += 32) s += dy[j] * y[j];
    s = warp_sum(s);
    if (!set) {
        for (int j = lane; j < lim; j += 32) da[j] += (y[j] * (dy[j] - s)) * scale;
    } else {
        for (int j = lane; j < D; j += 32) da[j] = (j < lim) ? (y[j] * (dy[j] - s)) * scale : 0.0f;
    }
}

// out[row] = sum_j a[row,j] * b[row,j], one warp per row
__global__ void rowdot_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ out, size_t rows,
                              int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* a = A + row * D;
    const float* b = B + row * D;
    float s = 0.0f;
    for (int j = lane; j < D; j += 32) s += a[j] * b[j];
    s = warp_sum(s);
    if (lane == 0) out[row] = s;
}

// ---------------------------------------------------------------------------
// RmsNorm / LayerNorm (one warp per row)
// ---------------------------------------------------------------------------
__global__ void rmsnorm_fwd_kernel(const float* __restrict__ X, const float* __restrict__ G, float eps,
                                   float* __restrict__ Y, size_t rows, int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = X + row * D;
    float* y = Y + row * D;
    float s = 0.0f;
    for (int j = lane; j < D; j += 32) s += x[j] * x[j];
    s = warp_sum(s);
    const float rms = sqrtf(s / (float)D + eps);
    for (int j = lane; j < D; j += 32) y[j] = x[j] / rms * G[j];
}

// dX (optional) and the per-row 1/rms needed by the dG column sums
__global__ void rmsnorm_bwd_rows_kernel(const float* __restrict__ X, const float* __restrict__ G,
                                        const float* __restrict__ dY, float eps, float* __restrict__ dX,
                                        float* __restrict__ rowscale, size_t rows, int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = X + row * D;
    const float* dy = dY + row * D;
    float s = 0.0f;
    for (int j = lane; j < D; j += 32) s += x[j] * x[j];
    s = warp_sum(s);
    const float scale = 1.0f / sqrtf(s / (float)D + eps);
    if (rowscale && lane == 0) rowscale[row] = scale;
    if (dX) {
        float t = 0.0f;
        for (int j = lane; j < D; j += 32) t += dy[j] * G[j] * x[j];
        t = warp_sum(t);
        float* dx = dX + row * D;
        for (int j = lane; j < D; j += 32) {
            const float term1 = G[j] * dy[j];
            const float term2 = x[j] * scale * scale * t / (float)D;
            dx[j] += scale * (term1 - term2);
        }
    }
}

// Register-cached forms for rows of at most 128*V4 elements with D % 4 == 0 and 16-byte aligned pointers: every
// operand is read once with 128-bit loads (the loops above read x three times with 32-bit loads).  Same expressions
// per element; only the order of the row sums differs.
template <int V4>
__global__ void rmsnorm_fwd_reg_kernel(const float* __restrict__ X, const float* __restrict__ G, float eps,
                                       float* __restrict__ Y, size_t rows, int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31, nv = D >> 2;
    const float4* x = reinterpret_cast<const float4*>(X + row * D);
    const float4* g = reinterpret_cast<const float4*>(G);
    float4* y = reinterpret_cast<float4*>(Y + row * D);
    float4 v[V4];
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int i = lane + 32 * k;
        if (i < nv) {
            v[k] = x[i];
            s += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
        }
    }
    s = warp_sum(s);
    const float rms = sqrtf(s / (float)D + eps);
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int i = lane + 32 * k;
        if (i < nv) {
            const float4 gg = g[i];
            y[i] = make_float4(v[k].x / rms * gg.x, v[k].y / rms * gg.y, v[k].z / rms * gg.z, v[k].w / rms * gg.w);
        }
    }
}

template <int V4>
__global__ void rmsnorm_bwd_rows_reg_kernel(const float* __restrict__ X, const float* __restrict__ G,
                                            const float* __restrict__ dY, float eps, float* __restrict__ dX,
                                            float* __restrict__ rowscale, size_t rows, int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31, nv = D >> 2;
    const float4* x = reinterpret_cast<const float4*>(X + row * D);
    const float4* dy = reinterpret_cast<const float4*>(dY + row * D);
    const float4* g = reinterpret_cast<const float4*>(G);
    float4 xv[V4], gy[V4];   // x and G o dY
    float s = 0.0f, t = 0.0f;
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int i = lane + 32 * k;
        if (i < nv) {
            xv[k] = x[i];
            s += (xv[k].x * xv[k].x + xv[k].y * xv[k].y) + (xv[k].z * xv[k].z + xv[k].w * xv[k].w);
            if (dX) {
                const float4 d = dy[i], gg = g[i];
                gy[k] = make_float4(d.x * gg.x, d.y * gg.y, d.z * gg.z, d.w * gg.w);
                t += (gy[k].x * xv[k].x + gy[k].y * xv[k].y) + (gy[k].z * xv[k].z + gy[k].w * xv[k].w);
            }
        }
    }
    s = warp_sum(s);
    const float scale = 1.0f / sqrtf(s / (float)D + eps);
    if (rowscale && lane == 0) rowscale[row] = scale;
    if (!dX) return;
    t = warp_sum(t);
    float4* dx = reinterpret_cast<float4*>(dX + row * D);
    const float fd = (float)D;
#pragma unroll
    for (int k = 0; k < V4; k++) {
        const int i = lane + 32 * k;
        if (i < nv) {
            float4 o = dx[i];
            o.x += scale * (gy[k].x - xv[k].x * scale * scale * t / fd);
            o.y += scale * (gy[k].y - xv[k].y * scale * scale * t / fd);
            o.z += scale * (gy[k].z - xv[k].z * scale * scale * t / fd);
            o.w += scale * (gy[k].w - xv[k].w * scale * scale * t / fd);
            dx[i] = o;
        }
    }
}

// The same with the gain gradient in the same pass: a warp walks rows gw, gw + nw, ... and keeps its share of
// dG[c] = sum_r dY[r,c] * x[r,c] * scale_r in registers; the block's eight warps are added in warp order and the
// block's partial row goes to partial[blockIdx.x][D] (a second kernel adds the blocks in order: deterministic for a
// given grid).  X and dY are read once: 16 bytes per element with the accumulating dX.
template <int V4>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dg_reg_kernel(const float* __restrict__ X, const float* __restrict__ G, const float* __restrict__ dY, float eps,
                          float* __restrict__ dX, float* __restrict__ partial, size_t rows, int D)
{
    __shared__ float4 red[8][32 * V4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nv = D >> 2;
    const size_t gw = blockIdx.x * (size_t)8 + warp, nw = (size_t)gridDim.x * 8;
    const float4* g = reinterpret_cast<const float4*>(G);
    float4 dg[V4];
#pragma unroll
    for (int k = 0; k < V4; k++) dg[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float fd = (float)D;
    for (size_t row = gw; row < rows; row += nw) {
        const float4* x = reinterpret_cast<const float4*>(X + row * D);
        const float4* dy = reinterpret_cast<const float4*>(dY + row * D);
        float4 xv[V4], dv[V4], ov[V4];   // the old dX is fetched with X and dY: one memory latency per row
        float4* dx = dX ? reinterpret_cast<float4*>(dX + row * D) : nullptr;
        float s = 0.0f, t = 0.0f;
#pragma unroll
        for (int k = 0; k < V4; k++) {
            const int i = lane + 32 * k;
            if (i < nv) {
                xv[k] = x[i];
                dv[k] = dy[i];
                if (dx) ov[k] = dx[i];
            }
        }
#pragma unroll
        for (int k = 0; k < V4; k++) {
            const int i = lane + 32 * k;
            if (i < nv) {
                const float4 gg = g[i];
                s += (xv[k].x * xv[k].x + xv[k].y * xv[k].y) + (xv[k].z * xv[k].z + xv[k].w * xv[k].w);
                t += ((dv[k].x * gg.x) * xv[k].x + (dv[k].y * gg.y) * xv[k].y) + ((dv[k].z * gg.z) * xv[k].z + (dv[k].w * gg.w) * xv[k].w);
            }
        }
        s = warp_sum(s);
        t = warp_sum(t);
        const float scale = 1.0f / sqrtf(s / fd + eps);
#pragma unroll
        for (int k = 0; k < V4; k++) {
            const int i = lane + 32 * k;
            if (i < nv) {
                dg[k].x += dv[k].x * xv[k].x * scale; dg[k].y += dv[k].y * xv[k].y * scale;
                dg[k].z += dv[k].z * xv[k].z * scale; dg[k].w += dv[k].w * xv[k].w * scale;
                if (dx) {
                    const float4 gg = g[i];
                    float4 o = ov[k];
                    o.x += scale * (dv[k].x * gg.x - xv[k].x * scale * scale * t / fd);
                    o.y += scale * (dv[k].y * gg.y - xv[k].y * scale * scale * t / fd);
                    o.z += scale * (dv[k].z * gg.z - xv[k].z * scale * scale * t / fd);
                    o.w += scale * (dv[k].w * gg.w - xv[k].w * scale * scale * t / fd);
                    dx[i] = o;
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < V4; k++) red[warp][lane + 32 * k] = dg[k];
    __syncthreads();
    float4* out = reinterpret_cast<float4*>(partial + (size_t)blockIdx.x * D);
    for (int i = threadIdx.x; i < nv; i += 256) {
        float4 u = red[0][i];
#pragma unroll
        for (int w = 1; w < 8; w++) { const float4 v = red[w][i]; u.x += v.x; u.y += v.y; u.z += v.z; u.w += v.w; }
        out[i] = u;
    }
}

__global__ void layernorm_fwd_kernel(const float* __restrict__ X, const float* __restrict__ G,
                                     const float* __restrict__ Bt, float eps, float* __restrict__ Y, size_t rows, int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = X + row * D;
    float* y = Y + row * D;
    float s = 0.0f;
    for (int j = lane; j < D; j += 32) s += x[j];
    const float mean = warp_sum(s) / (float)D;
    float v = 0.0f;
    for (int j = lane; j < D; j += 32) { const float d = x[j] - mean; v += d * d; }
    const float rstd = 1.0f / sqrtf(warp_sum(v) / (float)D + eps);
    for (int j = lane; j < D; j += 32) y[j] = (x[j] - mean) * rstd * G[j] + Bt[j];
}

__global__ void layernorm_bwd_rows_kernel(const float* __restrict__ X, const float* __restrict__ G,
                                          const float* __restrict__ dY, float eps, float* __restrict__ dX,
                                          float* __restrict__ rowstat, size_t rows, int D)
{
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = X + row * D;
    const float* dy = dY + row * D;
    float s = 0.0f;
    for (int j = lane; j < D; j += 32) s += x[j];
    const float mean = warp_sum(s) / (float)D;
    float v = 0.0f;
    for (int j = lane; j < D; j += 32) { const float d = x[j] - mean; v += d * d; }
    const float rstd = 1.0f / sqrtf(warp_sum(v) / (float)D + eps);
    if (rowstat && lane == 0) { rowstat[2 * row] = mean; rowstat[2 * row + 1] = rstd; }
    if (dX) {
        float s1 = 0.0f, s2 = 0.0f;
        for (int j = lane; j < D; j += 32) {
            const float gdy = G[j] * dy[j];
            s1 += gdy;
            s2 += gdy * ((x[j] - mean) * rstd);
        }
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        float* dx = dX + row * D;
        for (int j = lane; j < D; j += 32) {
            const float xh = (x[j] - mean) * rstd;
            dx[j] += rstd * (G[j] * dy[j] - s1 / (float)D - xh * s2 / (float)D);
        }
    }
}

// ---------------------------------------------------------------------------
// Embedding
// ---------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const float* __restrict__ W, const float* __restrict__ ids, float* __restrict__ Y,
                                     size_t n, int D, int vocab, int* __restrict__ status)
{
    for (size_t i = blockIdx.x; i < n; i += gridDim.x) {
        const float idf = ids[i];
        float* y = Y + i * D;
        if (!(idf >= 0.0f && idf < (float)vocab)) {
            // an id outside [0, vocab) (the reference asserts idx < VocabSize): no table row is read, the output row is
            // zero and the device status word says why
            for (int j = threadIdx.x; j < D; j += blockDim.x) y[j] = 0.0f;
            if (threadIdx.x == 0) atomicOr(status, ZNN_DEV_BAD_INDEX);
            continue;
        }
        const float* w = W + (size_t)idf * D;
        for (int j = threadIdx.x; j < D; j += blockDim.x) y[j] = w[j];
    }
}

// One warp per output row, 16-byte copies (D a multiple of 4, 16-byte aligned table and output).
__global__ void embedding_fwd_vec_kernel(const float4* __restrict__ W, const float* __restrict__ ids, float4* __restrict__ Y,
                                         size_t n, int D4, int vocab, int* __restrict__ status)
{
    const int lane = threadIdx.x & 31;
    const size_t nw = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t i = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5); i < n; i += nw) {
        const float idf = ids[i];
        float4* y = Y + i * D4;
        if (!(idf >= 0.0f && idf < (float)vocab)) {
            for (int j = lane; j < D4; j += 32) y[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (lane == 0) atomicOr(status, ZNN_DEV_BAD_INDEX);
            continue;
        }
        const float4* w = W + (size_t)idf * D4;
        for (int j = lane; j < D4; j += 32) y[j] = w[j];
    }
}

// One block per vocabulary row: finds the positions that use this row (kept in
// (b,t) order) and adds their dY rows one after the other, as the reference's
// sequential scatter-add does for that row.  The ids are scanned 2048 at a time: warp w scans the w-th run of
// 256 ids with ballots and lists its hits in its own part of `matches`, so a round needs two block barriers
// and the lists, read warp after warp, are in ascending position order.
__global__ void embedding_bwd_kernel(const float* __restrict__ ids, const float* __restrict__ dY,
                                     float* __restrict__ dW, int n, int D)
{
    constexpr int kPerWarp = 256, kRound = 8 * kPerWarp;
    __shared__ int matches[kRound];
    __shared__ int warp_counts[8];
    const int v = blockIdx.x;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    // each thread owns columns threadIdx.x, +256, ... (D <= 256*8)
    float acc[8];
#pragma unroll
    for (int c = 0; c < 8; c++) acc[c] = 0.0f;
    bool any = false;
    for (int base = 0; base < n; base += kRound) {
        int cw = 0;
#pragma unroll
        for (int s = 0; s < kPerWarp / 32; s++) {
            const int i = base + w * kPerWarp + s * 32 + lane;
            const bool hit = (i < n) && ((int)ids[i] == v);
            const unsigned bal = __ballot_sync(0xffffffffu, hit);
            if (hit) matches[w * kPerWarp + cw + __popc(bal & ((1u << lane) - 1))] = i;
            cw += __popc(bal);
        }
        if (lane == 0) warp_counts[w] = cw;
        __syncthreads();
        for (int ww = 0; ww < 8; ww++) {
            const int nm = warp_counts[ww];
            for (int k = 0; k < nm; k++) {
                const float* g = dY + (size_t)matches[ww * kPerWarp + k] * D;
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const int j = threadIdx.x + c * 256;
                    if (j < D) acc[c] += g[j];
                }
                any = true;
            }
        }
        __syncthreads();
    }
    if (any) {
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const int j = threadIdx.x + c * 256;
            if (j < D) dW[(size_t)v * D + j] += acc[c];
        }
    }
}

// general (D > 2048) fallback: thread per (vocab row, column), scanning ids in order
__global__ void embedding_bwd_wide_kernel(const float* __restrict__ ids, const float* __restrict__ dY,
                                          float* __restrict__ dW, int n, int D)
{
    const int v = blockIdx.x;
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        float acc = 0.0f;
        bool any = false;
        for (int i = 0; i < n; i++)
            if ((int)ids[i] == v) { acc += dY[(size_t)i * D + j]; any = true; }
        if (any) dW[(size_t)v * D + j] += acc;
    }
}

// ---------------------------------------------------------------------------
// Transpose of two dims (rank <= 8)
// ---------------------------------------------------------------------------
struct TransposeDesc {
    int rank;
    long long out_dims[8];
    long long src_strides[8];
};

template <bool Backward>
__global__ void transpose_generic_kernel(const float* __restrict__ in, float* __restrict__ out, TransposeDesc d, size_t total)
{
    for (size_t f = blockIdx.x * (size_t)blockDim.x + threadIdx.x; f < total; f += (size_t)gridDim.x * blockDim.x) {
        size_t rem = f;
        long long src = 0;
#pragma unroll 1
        for (int k = d.rank - 1; k >= 0; k--) {
            const long long idx = (long long)(rem % (size_t)d.out_dims[k]);
            rem /= (size_t)d.out_dims[k];
            src += idx * d.src_strides[k];
        }
        if (Backward) out[src] += in[f];   // dA[src] += dC[f]  (a permutation: no two f share a src)
        else out[f] = in[src];             // C[f] = A[src]
    }
}

// Swapped dims both before the last one: the tensor is [o][a][m][b][inner] -> [o][b][m][a][inner] with runs of
// `inner` contiguous floats moved as float4 (head split / merge of attention: inner = head size).
template <bool Backward>
__global__ void transpose_runs_kernel(const float4* __restrict__ in, float4* __restrict__ out, unsigned O, unsigned Ad,
                                      unsigned Mm, unsigned Bd, unsigned I4, unsigned total4)
{
    for (unsigned f = blockIdx.x * blockDim.x + threadIdx.x; f < total4; f += gridDim.x * blockDim.x) {
        unsigned t = f;
        const unsigned i4 = t % I4; t /= I4;
        const unsigned a = t % Ad; t /= Ad;
        const unsigned mm = t % Mm; t /= Mm;
        const unsigned b = t % Bd;
        const unsigned o = t / Bd;
        const unsigned src = (((o * Ad + a) * Mm + mm) * Bd + b) * I4 + i4;
        if (Backward) {
            float4 d = out[src];
            const float4 g = in[f];
            d.x += g.x; d.y += g.y; d.z += g.z; d.w += g.w;
            out[src] = d;
        } else {
            out[f] = in[src];
        }
    }
}

// last two dims swapped: per-slice R x Cc -> Cc x R through a shared-memory tile
template <bool Backward>
__global__ void transpose_last2_kernel(const float* __restrict__ in, float* __restrict__ out, int R, int Cc)
{
    __shared__ float tile[32][33];
    const size_t slice = blockIdx.z;
    // forward: in is [R, Cc], out is [Cc, R].  backward: in (dC) is [Cc, R], out (dA) is [R, Cc], accumulated.
    const int in_rows = Backward ? Cc : R, in_cols = Backward ? R : Cc;
    const float* src = in + slice * (size_t)R * Cc;
    float* dst = out + slice * (size_t)R * Cc;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;  // tile origin in the input
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        tile[j][threadIdx.x] = (r < in_rows && c < in_cols) ? src[(size_t)r * in_cols + c] : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int orow = c0 + j, ocol = r0 + threadIdx.x;  // output is [in_cols, in_rows]
        if (orow < in_cols && ocol < in_rows) {
            float* p = dst + (size_t)orow * in_rows + ocol;
            if (Backward) *p += tile[threadIdx.x][j]; else *p = tile[threadIdx.x][j];
        }
    }
}

// The same through a 64 x 64 tile with 16-byte global accesses in both directions (R and Cc multiples of 4, 16-byte
// aligned tensors): 16 KB per block instead of 4 KB and a quarter of the memory instructions.
template <bool Backward>
__global__ void __launch_bounds__(256) transpose_last2_vec_kernel(const float* __restrict__ in, float* __restrict__ out, int R, int Cc)
{
    __shared__ float tile[64][65];
    const size_t slice = blockIdx.z;
    const int in_rows = Backward ? Cc : R, in_cols = Backward ? R : Cc;
    const float* src = in + slice * (size_t)R * Cc;
    float* dst = out + slice * (size_t)R * Cc;
    const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int idx = threadIdx.x + 256 * k, r = idx >> 4, c4 = idx & 15;
        const int gr = r0 + r, gc = c0 + 4 * c4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (gr < in_rows && gc < in_cols) v = *reinterpret_cast<const float4*>(src + (size_t)gr * in_cols + gc);
        tile[r][4 * c4] = v.x; tile[r][4 * c4 + 1] = v.y; tile[r][4 * c4 + 2] = v.z; tile[r][4 * c4 + 3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int idx = threadIdx.x + 256 * k, orow = idx >> 4, oc4 = idx & 15;   // output is [in_cols, in_rows]
        const int go = c0 + orow, gc = r0 + 4 * oc4;
        if (go < in_cols && gc < in_rows) {
            float4 v = make_float4(tile[4 * oc4][orow], tile[4 * oc4 + 1][orow], tile[4 * oc4 + 2][orow], tile[4 * oc4 + 3][orow]);
            float4* p = reinterpret_cast<float4*>(dst + (size_t)go * in_rows + gc);
            if (Backward) { const float4 o = *p; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
            *p = v;
        }
    }
}

// ---------------------------------------------------------------------------
// argmax, SGD
// ---------------------------------------------------------------------------
// first maximum wins: strict > while scanning, lower index on equal values when merging
__global__ void argmax_rows_kernel(const float* __restrict__ A, float* __restrict__ out, int M, int N)
{
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= M) return;
    const int lane = threadIdx.x & 31;
    const float* a = A + (size_t)row * N;
    float mv = -CUDART_INF_F;
    int mi = 0x7fffffff;
    for (int j = lane; j < N; j += 32) {
        const float v = a[j];
        if (mi == 0x7fffffff || v > mv) { mv = v; mi = j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, mv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
        if (oi != 0x7fffffff && (mi == 0x7fffffff || ov > mv || (ov == mv && oi < mi))) { mv = ov; mi = oi; }
    }
    if (lane == 0) out[row] = (float)mi;
}

__global__ void argmax_cols_kernel(const float* __restrict__ A, float* __restrict__ out, int M, int N)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= N) return;
    float mv = A[j];
    int mi = 0;
    for (int i = 1; i < M; i++) {
        const float v = A[(size_t)i * N + j];
        if (v > mv) { mv = v; mi = i; }
    }
    out[j] = (float)mi;
}

// src/optim.zig:141-149 per element; lr_t is computed once on the host as the reference does
__global__ void adam_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                            float lr_t, float beta1, float beta2, float eps, float grad_scale, size_t n)
{
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const float ob1 = 1.0f - beta1, ob2 = 1.0f - beta2;
    for (size_t i = tid; i < n; i += nth) {
        float gi = g[i];
        if (grad_scale != 1.0f) gi *= grad_scale;
        const float mi = beta1 * m[i] + ob1 * gi;
        const float vi = beta2 * v[i] + ob2 * gi * gi;
        m[i] = mi;
        v[i] = vi;
        w[i] -= lr_t * mi / (sqrtf(vi) + eps);
    }
}

__global__ void sgd_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ v, float lr,
                           float momentum, float grad_scale, size_t n)
{
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const bool scaled = (grad_scale != 1.0f);
    const bool vec = ((((uintptr_t)w | (uintptr_t)g | (uintptr_t)v) & 15) == 0);
    const size_t n4 = vec ? n / 4 : 0;
    auto upd = [&](float& wi, float gi, float* vi) {
        if (scaled) gi *= grad_scale;
        if (vi) {
            const float vel = momentum * (*vi) + lr * gi;
            *vi = vel;
            wi -= vel;
        } else {
            wi -= lr * gi;
        }
    };
    for (size_t i = tid; i < n4; i += nth) {
        float4 wv = reinterpret_cast<float4*>(w)[i];
        const float4 gv = reinterpret_cast<const float4*>(g)[i];
        if (v) {
            float4 vv = reinterpret_cast<float4*>(v)[i];
            upd(wv.x, gv.x, &vv.x); upd(wv.y, gv.y, &vv.y); upd(wv.z, gv.z, &vv.z); upd(wv.w, gv.w, &vv.w);
            reinterpret_cast<float4*>(v)[i] = vv;
        } else {
            upd(wv.x, gv.x, nullptr); upd(wv.y, gv.y, nullptr); upd(wv.z, gv.z, nullptr); upd(wv.w, gv.w, nullptr);
        }
        reinterpret_cast<float4*>(w)[i] = wv;
    }
    for (size_t i = n4 * 4 + tid; i < n; i += nth) upd(w[i], g[i], v ? v + i : nullptr);
}

// pixel bytes -> fp32 in [0, 1]: IEEE division by 255 as the reference's loader does per pixel
__global__ void pixels_to_unit_kernel(const uint8_t* __restrict__ px, float* __restrict__ out, size_t n)
{
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const size_t n4 = ((reinterpret_cast<uintptr_t>(px) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) ? n / 4 : 0;
    for (size_t i = tid; i < n4; i += nth) {
        const uchar4 b = reinterpret_cast<const uchar4*>(px)[i];
        reinterpret_cast<float4*>(out)[i] =
            make_float4(__fdiv_rn((float)b.x, 255.0f), __fdiv_rn((float)b.y, 255.0f), __fdiv_rn((float)b.z, 255.0f),
                        __fdiv_rn((float)b.w, 255.0f));
    }
    for (size_t i = n4 * 4 + tid; i < n; i += nth) out[i] = __fdiv_rn((float)px[i], 255.0f);
}

// one batch of sample rows and labels picked by index; blockIdx.y = slot in the batch
__global__ void batch_gather_kernel(const float* __restrict__ images, const uint8_t* __restrict__ labels,
                                    const int32_t* __restrict__ indices, float* __restrict__ x_dest,
                                    uint8_t* __restrict__ y_dest, int input_dim, int vec_ok, size_t num_samples,
                                    int* __restrict__ status)
{
    const int j = blockIdx.y;
    const int32_t raw = indices[j];
    float* dst = x_dest + (size_t)j * input_dim;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
    if (raw < 0 || (size_t)raw >= num_samples) {
        // a sample index outside the dataset: nothing is read through it; the slot is zero-filled and flagged
        for (int i = tid; i < input_dim; i += nth) dst[i] = 0.0f;
        if (tid == 0) {
            if (y_dest) y_dest[j] = 0;
            atomicOr(status, ZNN_DEV_BAD_INDEX);
        }
        return;
    }
    const size_t idx = (size_t)raw;
    const float* src = images + idx * (size_t)input_dim;
    if (vec_ok) {
        for (int i = tid; i < input_dim / 4; i += nth) reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
    } else {
        for (int i = tid; i < input_dim; i += nth) dst[i] = src[i];
    }
    if (tid == 0 && labels && y_dest) y_dest[j] = labels[idx];
}

// ---------------------------------------------------------------------------
// Random fills (weight initialisation)
// ---------------------------------------------------------------------------
// Counter-based generator: element i of a fill with seed s draws from hash(s, i, draw), so the result does not depend
// on the launch geometry.  The reference draws from Zig's DefaultPrng stream, which cannot be reproduced here; the
// distribution and the fan-in rule are the reference's, the stream is not.
__device__ __forceinline__ uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// uniform in [0, 1) with 24 random bits, the granularity of a float drawn as in std.Random.float(f32)
__device__ __forceinline__ float uniform24(uint64_t seed, uint64_t index, uint32_t draw)
{
    const uint64_t h = mix64(mix64(seed ^ (index * 0xD1342543DE82EF95ull)) + draw);
    return (float)(uint32_t)(h >> 40) * (1.0f / 16777216.0f);
}

// Box-Muller pair for element pair `pair` (src/nn.zig:1343-1350, src/tensor.zig:354-373): u1 is redrawn while it is 0
__device__ __forceinline__ void box_muller(uint64_t seed, uint64_t pair, float& radius, float& angle)
{
    float u1 = 0.0f;
    uint32_t draw = 0;
    while (u1 == 0.0f && draw < 64) u1 = uniform24(seed, pair, draw++);
    if (u1 == 0.0f) u1 = 1.0f / 16777216.0f;
    const float u2 = uniform24(seed, pair, 64);
    radius = sqrtf(-2.0f * logf(u1));
    angle = 6.283185307179586f * u2;
}

// mode 0: every element its own draw, cosine branch only (initializeWeights / normalRandom of src/nn.zig:1336-1350);
// mode 1: elements 2k and 2k+1 share one draw, cosine then sine (Tensor.fillNormal, src/tensor.zig:354-373)
__global__ void fill_normal_kernel(float* __restrict__ w, size_t n, float mean, float stddev, uint64_t seed, int mode)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float r, a;
        box_muller(seed, mode == 0 ? i : (i >> 1), r, a);
        const float z = (mode == 1 && (i & 1)) ? r * sinf(a) : r * cosf(a);
        w[i] = mean + z * stddev;
    }
}

// Tensor.fillUniform (src/tensor.zig:375-379)
__global__ void fill_uniform_kernel(float* __restrict__ w, size_t n, float lo, float range, uint64_t seed)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        w[i] = lo + uniform24(seed, i, 0) * range;
}

// fraction of rows whose predicted class (fp32 index, as argmax writes it) equals the byte label; one block,
// integer count, so the result does not depend on the order of the rows
__global__ void accuracy_u8_kernel(const float* __restrict__ preds, const uint8_t* __restrict__ labels, int n,
                                   float* __restrict__ acc)
{
    __shared__ int warp_hits[32];
    int hits = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) hits += ((int)preds[i] == (int)labels[i]) ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hits += __shfl_xor_sync(0xffffffffu, hits, o);
    if ((threadIdx.x & 31) == 0) warp_hits[threadIdx.x >> 5] = hits;
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) total += warp_hits[w];
        *acc = (float)total / (float)n;
    }
}

}  // namespace znn

using namespace znn;

#define ZNN_NEED_DEVICE()                                                                                  \
    do {                                                                                                   \
        if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (no CPU fallback)"); \
    } while (0)

extern "C" {

int znn_pixels_to_unit(const uint8_t* pixels, float* out, size_t n)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(pixels && out, "pixels/out is NULL");
    pixels_to_unit_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(pixels, out, n);
    ZNN_LAUNCH_OK("pixels_to_unit_kernel");
    return ZNN_OK;
}

int znn_batch_gather(const float* images, const uint8_t* labels, const int32_t* indices, float* x_dest, uint8_t* y_dest,
                     int batch, int input_dim, size_t num_samples)
{
    if (batch <= 0 || input_dim <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(images && indices && x_dest, "images/indices/x_dest is NULL");
    ZNN_REQUIRE((labels == nullptr) == (y_dest == nullptr), "labels and y_dest go together");
    ZNN_REQUIRE(batch <= 65535, "batch exceeds 65535 rows per call");
    const int vec_ok = input_dim % 4 == 0 && (reinterpret_cast<uintptr_t>(images) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(x_dest) & 15) == 0;
    const int per_row = vec_ok ? input_dim / 4 : input_dim;
    const dim3 grid((unsigned)std::min(64, (per_row + kEwThreads - 1) / kEwThreads), (unsigned)batch);
    batch_gather_kernel<<<grid, kEwThreads, 0, stream()>>>(images, labels, indices, x_dest, y_dest, input_dim, vec_ok,
                                                           num_samples, device_status_word());
    ZNN_LAUNCH_OK("batch_gather_kernel");
    return ZNN_OK;
}

int znn_init_he_normal(float* w, size_t n, size_t fan_in, unsigned long long seed)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(w, "w is NULL");
    ZNN_REQUIRE(fan_in > 0, "fan_in must be positive");
    const float std_dev = sqrtf(2.0f / (float)fan_in);
    fill_normal_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(w, n, 0.0f, std_dev, seed, 0);
    ZNN_LAUNCH_OK("fill_normal_kernel");
    return ZNN_OK;
}

int znn_fill_normal(float* w, size_t n, float mean, float stddev, unsigned long long seed)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(w, "w is NULL");
    fill_normal_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(w, n, mean, stddev, seed, 1);
    ZNN_LAUNCH_OK("fill_normal_kernel");
    return ZNN_OK;
}

int znn_fill_uniform(float* w, size_t n, float min_val, float max_val, unsigned long long seed)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(w, "w is NULL");
    fill_uniform_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(w, n, min_val, max_val - min_val, seed);
    ZNN_LAUNCH_OK("fill_uniform_kernel");
    return ZNN_OK;
}

int znn_fill(float* dst, float value, size_t n)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(dst, "dst is NULL");
    fill_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(dst, value, n);
    ZNN_LAUNCH_OK("fill_kernel");
    return ZNN_OK;
}

int znn_iota_mod(float* dst, size_t n, int period)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(dst && period > 0, "dst is NULL or period <= 0");
    iota_mod_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(dst, n, period);
    ZNN_LAUNCH_OK("iota_mod_kernel");
    return ZNN_OK;
}

int znn_add_bias_fwd(const float* A, const float* bias, float* C, int M, int N)
{
    if (M <= 0 || N <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(A && bias && C, "NULL pointer");
    const size_t total = (size_t)M * N;
    add_bias_fwd_kernel<<<ew_blocks(total), kEwThreads, 0, stream()>>>(A, bias, C, total, N);
    ZNN_LAUNCH_OK("add_bias_fwd_kernel");
    return ZNN_OK;
}

int znn_add_bias_bwd(const float* dC, float* dA, float* dbias, int M, int N)
{
    if (M <= 0 || N <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(dC, "dC is NULL");
    if (!dbias) {
        if (dA) return znn_accumulate(dC, dA, (size_t)M * N);
        return ZNN_OK;
    }
    int chunks, rpc;
    colsum_plan(M, chunks, rpc);
    float* partial = (float*)workspace((size_t)chunks * N * sizeof(float));
    if (!partial) return fail(ZNN_ERR_NOMEM, "scratch for bias gradient");
    const bool vec = (N & 3) == 0 && ((((uintptr_t)dC | (uintptr_t)dA | (uintptr_t)dbias | (uintptr_t)partial)) & 15) == 0;
    if (vec) {
        dim3 vgrid(ceil_div(N, 128), chunks);
        unsigned* vcounters = (int)vgrid.x <= kScratchCounters ? scratch_counters() : nullptr;
        if (dA) colsum_vec_kernel<true><<<vgrid, 256, 0, stream()>>>(dC, dA, partial, M, N, rpc, vcounters, dbias);
        else colsum_vec_kernel<false><<<vgrid, 256, 0, stream()>>>(dC, nullptr, partial, M, N, rpc, vcounters, dbias);
        ZNN_LAUNCH_OK("colsum_vec_kernel");
        if (!vcounters) {
            colsum_stage2_kernel<<<ceil_div(N, 32), dim3(32, 8), 0, stream()>>>(partial, dbias, chunks, N);
            ZNN_LAUNCH_OK("colsum_stage2_kernel");
        }
        return ZNN_OK;
    }
    dim3 grid(ceil_div(N, 32), chunks), block(32, 8);
    // one launch when the block counters are at hand (the last chunk of a column block finishes its sum), else two
    unsigned* counters = (int)grid.x <= kScratchCounters ? scratch_counters() : nullptr;
    if (dA) colsum_stage1_kernel<true><<<grid, block, 0, stream()>>>(dC, dA, partial, M, N, rpc, counters, dbias);
    else colsum_stage1_kernel<false><<<grid, block, 0, stream()>>>(dC, nullptr, partial, M, N, rpc, counters, dbias);
    ZNN_LAUNCH_OK("colsum_stage1_kernel");
    if (!counters) {
        colsum_stage2_kernel<<<ceil_div(N, 32), dim3(32, 8), 0, stream()>>>(partial, dbias, chunks, N);
        ZNN_LAUNCH_OK("colsum_stage2_kernel");
    }
    return ZNN_OK;
}

int znn_relu_fwd(const float* A, float* C, size_t n)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ew1w_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(A, C, n, ReluF());
    ZNN_LAUNCH_OK("relu_fwd");
    return ZNN_OK;
}

int znn_relu_bwd(const float* A, const float* dC, float* dA, size_t n)
{
    if (n == 0 || !dA) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ew2_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(A, dC, dA, n, ReluBwdF());
    ZNN_LAUNCH_OK("relu_bwd");
    return ZNN_OK;
}

int znn_gelu_fwd(const float* A, float* C, size_t n)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ew1w_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(A, C, n, GeluF());
    ZNN_LAUNCH_OK("gelu_fwd");
    return ZNN_OK;
}

int znn_gelu_bwd(const float* A, const float* dC, float* dA, size_t n)
{
    if (n == 0 || !dA) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ew2_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(A, dC, dA, n, GeluBwdF());
    ZNN_LAUNCH_OK("gelu_bwd");
    return ZNN_OK;
}

int znn_gelu_bwd_set(const float* A, const float* dC, float* dA, size_t n)
{
    if (n == 0 || !dA) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ew2w_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(A, dC, dA, n, GeluBwdSetF());
    ZNN_LAUNCH_OK("gelu_bwd_set");
    return ZNN_OK;
}

}  // extern "C"

template <class T>
static int xent_fwd(const float* logits, const T* targets, float* probs, float* loss, int M, int N)
{
    ZNN_REQUIRE(M > 0 && N > 0, "empty logits");
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(logits && targets && probs && loss, "NULL pointer");
    float* rowloss = (float*)workspace((size_t)M * sizeof(float));
    if (!rowloss) return fail(ZNN_ERR_NOMEM, "scratch for per-row losses");
    int* status = device_status_word();
    const bool v4 = (N % 4 == 0) && ((((uintptr_t)logits | (uintptr_t)probs) & 15) == 0);
    if (v4 && N > 2048 && N <= 1024 * 8) {
        if (N <= 1024 * 4) softmax_xent_fwd_reg_kernel<T, 4><<<M, 256, 0, stream()>>>(logits, targets, probs, rowloss, N, status);
        else softmax_xent_fwd_reg_kernel<T, 8><<<M, 256, 0, stream()>>>(logits, targets, probs, rowloss, N, status);
    } else {
        const int threads = N >= 1024 ? 256 : (N >= 128 ? 128 : 32);
        softmax_xent_fwd_kernel<T><<<M, threads, 0, stream()>>>(logits, targets, probs, rowloss, N, status);
    }
    ZNN_LAUNCH_OK("softmax_xent_fwd_kernel");
    mean_rows_kernel<<<1, 1024, 0, stream()>>>(rowloss, loss, M);
    ZNN_LAUNCH_OK("mean_rows_kernel");
    return ZNN_OK;
}

template <class T>
static int xent_bwd(const float* probs, const T* targets, float* dlogits, int M, int N)
{
    if (M <= 0 || N <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(probs && targets && dlogits, "NULL pointer");
    softmax_xent_bwd_kernel<T><<<ew_blocks((size_t)M * N, 2), kEwThreads, 0, stream()>>>(probs, targets, dlogits, M, N);
    ZNN_LAUNCH_OK("softmax_xent_bwd_kernel");
    return ZNN_OK;
}

extern "C" {

int znn_softmax_xent_fwd(const float* logits, const int32_t* targets, float* probs, float* loss, int M, int N)
{
    return xent_fwd<int32_t>(logits, targets, probs, loss, M, N);
}

int znn_softmax_xent_fwd_u8(const float* logits, const uint8_t* targets, float* probs, float* loss, int M, int N)
{
    return xent_fwd<uint8_t>(logits, targets, probs, loss, M, N);
}

int znn_softmax_xent_bwd(const float* probs, const int32_t* targets, float* dlogits, int M, int N)
{
    return xent_bwd<int32_t>(probs, targets, dlogits, M, N);
}

int znn_softmax_xent_bwd_u8(const float* probs, const uint8_t* targets, float* dlogits, int M, int N)
{
    return xent_bwd<uint8_t>(probs, targets, dlogits, M, N);
}

static inline unsigned row_blocks(size_t rows, int warps_per_block) { return (unsigned)((rows + warps_per_block - 1) / warps_per_block); }

int znn_softmax_fwd(const float* A, float* C, size_t rows, int D)
{
    if (rows == 0 || D <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    const bool v4 = (D % 4 == 0) && ((((uintptr_t)A | (uintptr_t)C) & 15) == 0);
    if (v4 && D <= 256) softmax_rows_reg_kernel<false, 2><<<row_blocks(rows, 8), 256, 0, stream()>>>(A, 1.0f, C, rows, D);
    else if (v4 && D <= 1024) softmax_rows_reg_kernel<false, 8><<<row_blocks(rows, 8), 256, 0, stream()>>>(A, 1.0f, C, rows, D);
    else softmax_rows_fwd_kernel<false><<<row_blocks(rows, 8), 256, 0, stream()>>>(A, 1.0f, C, rows, D);
    ZNN_LAUNCH_OK("softmax_rows_fwd_kernel");
    return ZNN_OK;
}

int znn_softmax_bwd(const float* Y, const float* dY, float* dA, size_t rows, int D)
{
    if (rows == 0 || D <= 0 || !dA) return ZNN_OK;
    ZNN_NEED_DEVICE();
    softmax_rows_bwd_kernel<<<row_blocks(rows, 8), 256, 0, stream()>>>(Y, dY, 1.0f, dA, rows, D, 0);
    ZNN_LAUNCH_OK("softmax_rows_bwd_kernel");
    return ZNN_OK;
}

int znn_causal_softmax_fwd(const float* S, float scale, float* P, int nslices, int T)
{
    if (nslices <= 0 || T <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    const size_t rows = (size_t)nslices * T;
    const bool v4 = (T % 4 == 0) && ((((uintptr_t)S | (uintptr_t)P) & 15) == 0);
    if (v4 && T <= 256) softmax_rows_reg_kernel<true, 2><<<row_blocks(rows, 8), 256, 0, stream()>>>(S, scale, P, rows, T);
    else if (v4 && T <= 1024) softmax_rows_reg_kernel<true, 8><<<row_blocks(rows, 8), 256, 0, stream()>>>(S, scale, P, rows, T);
    else softmax_rows_fwd_kernel<true><<<row_blocks(rows, 8), 256, 0, stream()>>>(S, scale, P, rows, T);
    ZNN_LAUNCH_OK("causal softmax fwd");
    return ZNN_OK;
}

int znn_causal_softmax_bwd(const float* P, const float* dP, float scale, float* dS, int nslices, int T)
{
    if (nslices <= 0 || T <= 0 || !dS) return ZNN_OK;
    ZNN_NEED_DEVICE();
    const size_t rows = (size_t)nslices * T;
    softmax_rows_bwd_kernel<<<row_blocks(rows, 8), 256, 0, stream()>>>(P, dP, scale, dS, rows, T, 1);
    ZNN_LAUNCH_OK("causal softmax bwd");
    return ZNN_OK;
}

int znn_causal_softmax_bwd_set(const float* P, const float* dP, float scale, float* dS, int nslices, int T)
{
    if (nslices <= 0 || T <= 0 || !dS) return ZNN_OK;
    ZNN_NEED_DEVICE();
    const size_t rows = (size_t)nslices * T;
    softmax_rows_bwd_kernel<<<row_blocks(rows, 8), 256, 0, stream()>>>(P, dP, scale, dS, rows, T, 1, 1);
    ZNN_LAUNCH_OK("causal softmax bwd (set)");
    return ZNN_OK;
}

int znn_rowdot(const float* A, const float* B, float* out, size_t rows, int D)
{
    if (rows == 0 || D <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(A && B && out, "NULL pointer");
    rowdot_kernel<<<row_blocks(rows, 8), 256, 0, stream()>>>(A, B, out, rows, D);
    ZNN_LAUNCH_OK("rowdot_kernel");
    return ZNN_OK;
}

int znn_rmsnorm_fwd(const float* X, const float* G, float eps, float* Y, size_t rows, int D)
{
    if (rows == 0 || D <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    const bool v4 = (D % 4 == 0) && ((((uintptr_t)X | (uintptr_t)G | (uintptr_t)Y) & 15) == 0);
    const dim3 grid = row_blocks(rows, 8);
    if (v4 && D <= 256) rmsnorm_fwd_reg_kernel<2><<<grid, 256, 0, stream()>>>(X, G, eps, Y, rows, D);
    else if (v4 && D <= 768) rmsnorm_fwd_reg_kernel<6><<<grid, 256, 0, stream()>>>(X, G, eps, Y, rows, D);
    else if (v4 && D <= 1024) rmsnorm_fwd_reg_kernel<8><<<grid, 256, 0, stream()>>>(X, G, eps, Y, rows, D);
    else rmsnorm_fwd_kernel<<<grid, 256, 0, stream()>>>(X, G, eps, Y, rows, D);
    ZNN_LAUNCH_OK("rmsnorm_fwd_kernel");
    return ZNN_OK;
}

int znn_rmsnorm_bwd(const float* X, const float* G, const float* dY, float eps, float* dX, float* dG, size_t rows, int D)
{
    if (rows == 0 || D <= 0 || (!dX && !dG)) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(rows <= 0x7fffffff, "too many rows");
    const bool v4 = (D % 4 == 0) && ((((uintptr_t)X | (uintptr_t)G | (uintptr_t)dY | (uintptr_t)dX) & 15) == 0);
    if (dG && v4 && D <= 1024) {
        // one pass: dX and per-block partial rows of dG, then the blocks are added in order
        size_t blocks = (rows + 7) / 8;
        const size_t cap = (size_t)sm_count() * 4;
        if (blocks > cap) blocks = cap;
        float* partial = (float*)workspace(blocks * (size_t)D * sizeof(float));
        if (!partial) return fail(ZNN_ERR_NOMEM, "scratch for RmsNorm backward");
        if (D <= 256) rmsnorm_bwd_dg_reg_kernel<2><<<(unsigned)blocks, 256, 0, stream()>>>(X, G, dY, eps, dX, partial, rows, D);
        else if (D <= 768) rmsnorm_bwd_dg_reg_kernel<6><<<(unsigned)blocks, 256, 0, stream()>>>(X, G, dY, eps, dX, partial, rows, D);
        else rmsnorm_bwd_dg_reg_kernel<8><<<(unsigned)blocks, 256, 0, stream()>>>(X, G, dY, eps, dX, partial, rows, D);
        ZNN_LAUNCH_OK("rmsnorm_bwd_dg_reg_kernel");
        colsum_stage2_kernel<<<ceil_div(D, 32), dim3(32, 8), 0, stream()>>>(partial, dG, (int)blocks, D);
        ZNN_LAUNCH_OK("colsum_stage2_kernel");
        return ZNN_OK;
    }
    int chunks = 0, rpc = 0;
    float* rowscale = nullptr;
    float* partial = nullptr;
    if (dG) {
        colsum_plan((int)rows, chunks, rpc);
        float* ws = (float*)workspace((rows + (size_t)chunks * D) * sizeof(float));
        if (!ws) return fail(ZNN_ERR_NOMEM, "scratch for RmsNorm backward");
        rowscale = ws;
        partial = ws + rows;
    }
    const dim3 rgrid = row_blocks(rows, 8);
    if (v4 && D <= 256) rmsnorm_bwd_rows_reg_kernel<2><<<rgrid, 256, 0, stream()>>>(X, G, dY, eps, dX, rowscale, rows, D);
    else if (v4 && D <= 768) rmsnorm_bwd_rows_reg_kernel<6><<<rgrid, 256, 0, stream()>>>(X, G, dY, eps, dX, rowscale, rows, D);
    else if (v4 && D <= 1024) rmsnorm_bwd_rows_reg_kernel<8><<<rgrid, 256, 0, stream()>>>(X, G, dY, eps, dX, rowscale, rows, D);
    else rmsnorm_bwd_rows_kernel<<<rgrid, 256, 0, stream()>>>(X, G, dY, eps, dX, rowscale, rows, D);
    ZNN_LAUNCH_OK("rmsnorm_bwd_rows_kernel");
    if (dG) {
        dim3 grid(ceil_div(D, 32), chunks), block(32, 8);
        colsum_norm_stage1_kernel<0><<<grid, block, 0, stream()>>>(dY, X, rowscale, partial, (int)rows, D, rpc);
        ZNN_LAUNCH_OK("colsum_norm_stage1_kernel");
        colsum_stage2_kernel<<<ceil_div(D, 32), dim3(32, 8), 0, stream()>>>(partial, dG, chunks, D);
        ZNN_LAUNCH_OK("colsum_stage2_kernel");
    }
    return ZNN_OK;
}

int znn_layernorm_fwd(const float* X, const float* G, const float* B, float eps, float* Y, size_t rows, int D)
{
    if (rows == 0 || D <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    layernorm_fwd_kernel<<<row_blocks(rows, 8), 256, 0, stream()>>>(X, G, B, eps, Y, rows, D);
    ZNN_LAUNCH_OK("layernorm_fwd_kernel");
    return ZNN_OK;
}

int znn_layernorm_bwd(const float* X, const float* G, const float* dY, float eps, float* dX, float* dG, float* dB,
                      size_t rows, int D)
{
    if (rows == 0 || D <= 0 || (!dX && !dG && !dB)) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(rows <= 0x7fffffff, "too many rows");
    int chunks = 0, rpc = 0;
    float* rowstat = nullptr;
    float* partial = nullptr;
    if (dG || dB) {
        colsum_plan((int)rows, chunks, rpc);
        float* ws = (float*)workspace((2 * rows + (size_t)chunks * D) * sizeof(float));
        if (!ws) return fail(ZNN_ERR_NOMEM, "scratch for LayerNorm backward");
        rowstat = ws;
        partial = ws + 2 * rows;
    }
    layernorm_bwd_rows_kernel<<<row_blocks(rows, 8), 256, 0, stream()>>>(X, G, dY, eps, dX, rowstat, rows, D);
    ZNN_LAUNCH_OK("layernorm_bwd_rows_kernel");
    dim3 grid(ceil_div(D, 32), chunks), block(32, 8);
    if (dG) {
        colsum_norm_stage1_kernel<1><<<grid, block, 0, stream()>>>(dY, X, rowstat, partial, (int)rows, D, rpc);
        ZNN_LAUNCH_OK("colsum_norm_stage1_kernel");
        colsum_stage2_kernel<<<ceil_div(D, 32), dim3(32, 8), 0, stream()>>>(partial, dG, chunks, D);
        ZNN_LAUNCH_OK("colsum_stage2_kernel");
    }
    if (dB) {
        colsum_norm_stage1_kernel<2><<<grid, block, 0, stream()>>>(dY, X, rowstat, partial, (int)rows, D, rpc);
        ZNN_LAUNCH_OK("colsum_norm_stage1_kernel");
        colsum_stage2_kernel<<<ceil_div(D, 32), dim3(32, 8), 0, stream()>>>(partial, dB, chunks, D);
        ZNN_LAUNCH_OK("colsum_stage2_kernel");
    }
    return ZNN_OK;
}

int znn_embedding_fwd(const float* W, const float* ids, float* Y, size_t n, int D, int vocab)
{
    if (n == 0 || D <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(vocab > 0, "vocab must be positive");
    if ((D & 3) == 0 && (((uintptr_t)W | (uintptr_t)Y) & 15) == 0) {
        size_t vblocks = (n + 7) / 8;
        const size_t cap = (size_t)sm_count() * 32;
        if (vblocks > cap) vblocks = cap;
        embedding_fwd_vec_kernel<<<(unsigned)vblocks, 256, 0, stream()>>>((const float4*)W, ids, (float4*)Y, n, D / 4, vocab,
                                                                          device_status_word());
        ZNN_LAUNCH_OK("embedding_fwd_vec_kernel");
        return ZNN_OK;
    }
    const unsigned blocks = (unsigned)(n < 65535u * 16u ? n : 65535u * 16u);
    embedding_fwd_kernel<<<blocks, D >= 256 ? 256 : 64, 0, stream()>>>(W, ids, Y, n, D, vocab, device_status_word());
    ZNN_LAUNCH_OK("embedding_fwd_kernel");
    return ZNN_OK;
}

int znn_embedding_bwd(const float* ids, const float* dY, float* dW, size_t n, int D, int vocab)
{
    if (n == 0 || D <= 0 || !dW) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(vocab > 0, "vocab must be given for the backward pass");
    ZNN_REQUIRE(n <= 0x7fffffff, "too many ids");
    if (D <= 2048) embedding_bwd_kernel<<<vocab, 256, 0, stream()>>>(ids, dY, dW, (int)n, D);
    else embedding_bwd_wide_kernel<<<vocab, 256, 0, stream()>>>(ids, dY, dW, (int)n, D);
    ZNN_LAUNCH_OK("embedding_bwd_kernel");
    return ZNN_OK;
}

static int transpose_impl(const float* in, float* out, const int64_t* dims, int rank, int d0, int d1, bool backward)
{
    ZNN_REQUIRE(rank >= 1 && rank <= 8, "rank must be 1..8");
    ZNN_REQUIRE(d0 >= 0 && d0 < rank && d1 >= 0 && d1 < rank, "dims out of range");
    ZNN_NEED_DEVICE();
    size_t total = 1;
    for (int k = 0; k < rank; k++) total *= (size_t)dims[k];
    if (total == 0) return ZNN_OK;
    if (d0 > d1) { int t = d0; d0 = d1; d1 = t; }
    if (d0 != d1 && d0 == rank - 2 && d1 == rank - 1) {
        size_t slices = 1;
        for (int k = 0; k < rank - 2; k++) slices *= (size_t)dims[k];
        const int R = (int)dims[rank - 2], Cc = (int)dims[rank - 1];
        if (slices <= 65535 && (R & 3) == 0 && (Cc & 3) == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
            const int in_rows = backward ? Cc : R, in_cols = backward ? R : Cc;
            dim3 grid(ceil_div(in_cols, 64), ceil_div(in_rows, 64), (unsigned)slices);
            if (backward) transpose_last2_vec_kernel<true><<<grid, 256, 0, stream()>>>(in, out, R, Cc);
            else transpose_last2_vec_kernel<false><<<grid, 256, 0, stream()>>>(in, out, R, Cc);
            ZNN_LAUNCH_OK("transpose_last2_vec_kernel");
            return ZNN_OK;
        }
        if (slices <= 65535) {
            const int in_rows = backward ? Cc : R, in_cols = backward ? R : Cc;
            dim3 grid(ceil_div(in_cols, 32), ceil_div(in_rows, 32), (unsigned)slices), block(32, 8);
            if (backward) transpose_last2_kernel<true><<<grid, block, 0, stream()>>>(in, out, R, Cc);
            else transpose_last2_kernel<false><<<grid, block, 0, stream()>>>(in, out, R, Cc);
            ZNN_LAUNCH_OK("transpose_last2_kernel");
            return ZNN_OK;
        }
    }
    if (d0 != d1 && d1 < rank - 1) {
        size_t inner = 1, mid = 1, outer = 1;
        for (int k = d1 + 1; k < rank; k++) inner *= (size_t)dims[k];
        for (int k = d0 + 1; k < d1; k++) mid *= (size_t)dims[k];
        for (int k = 0; k < d0; k++) outer *= (size_t)dims[k];
        if ((inner & 3) == 0 && total / 4 < 0x7fffffffu && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
            const unsigned total4 = (unsigned)(total / 4);
            const unsigned blocks = (unsigned)ew_blocks(total4, 2);
            if (backward)
                transpose_runs_kernel<true><<<blocks, kEwThreads, 0, stream()>>>(
                    (const float4*)in, (float4*)out, (unsigned)outer, (unsigned)dims[d0], (unsigned)mid, (unsigned)dims[d1],
                    (unsigned)(inner / 4), total4);
            else
                transpose_runs_kernel<false><<<blocks, kEwThreads, 0, stream()>>>(
                    (const float4*)in, (float4*)out, (unsigned)outer, (unsigned)dims[d0], (unsigned)mid, (unsigned)dims[d1],
                    (unsigned)(inner / 4), total4);
            ZNN_LAUNCH_OK("transpose_runs_kernel");
            return ZNN_OK;
        }
    }
    TransposeDesc d;
    d.rank = rank;
    long long strides[8];
    long long s = 1;
    for (int k = rank - 1; k >= 0; k--) { strides[k] = s; s *= dims[k]; }
    for (int k = 0; k < rank; k++) { d.out_dims[k] = dims[k]; d.src_strides[k] = strides[k]; }
    d.out_dims[d0] = dims[d1]; d.out_dims[d1] = dims[d0];
    d.src_strides[d0] = strides[d1]; d.src_strides[d1] = strides[d0];
    if (backward) transpose_generic_kernel<true><<<ew_blocks(total, 2), kEwThreads, 0, stream()>>>(in, out, d, total);
    else transpose_generic_kernel<false><<<ew_blocks(total, 2), kEwThreads, 0, stream()>>>(in, out, d, total);
    ZNN_LAUNCH_OK("transpose_generic_kernel");
    return ZNN_OK;
}

int znn_transpose_fwd(const float* A, float* C, const int64_t* dims, int rank, int d0, int d1)
{
    return transpose_impl(A, C, dims, rank, d0, d1, false);
}

int znn_transpose_bwd(const float* dC, float* dA, const int64_t* dims, int rank, int d0, int d1)
{
    if (!dA) return ZNN_OK;
    return transpose_impl(dC, dA, dims, rank, d0, d1, true);
}

int znn_add_fwd(const float* A, const float* B, float* C, size_t n)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ew2w_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(A, B, C, n, AddF());
    ZNN_LAUNCH_OK("add_fwd");
    return ZNN_OK;
}

int znn_accumulate(const float* src, float* dst, size_t n)
{
    if (n == 0 || !dst) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ew1_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(src, dst, n, AccF());
    ZNN_LAUNCH_OK("accumulate");
    return ZNN_OK;
}

int znn_mul_scalar_fwd(const float* A, float v, float* C, size_t n)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    MulF f; f.v = v;
    ew1w_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(A, C, n, f);
    ZNN_LAUNCH_OK("mul_scalar_fwd");
    return ZNN_OK;
}

int znn_mul_scalar_bwd(const float* dC, float v, float* dA, size_t n)
{
    if (n == 0 || !dA) return ZNN_OK;
    ZNN_NEED_DEVICE();
    MulAccF f; f.v = v;
    ew1_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(dC, dA, n, f);
    ZNN_LAUNCH_OK("mul_scalar_bwd");
    return ZNN_OK;
}

int znn_argmax(const float* A, float* out, int M, int N, int dim)
{
    ZNN_REQUIRE(dim == 0 || dim == 1, "dim must be 0 or 1");
    if (M <= 0 || N <= 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    if (dim == 1) argmax_rows_kernel<<<ceil_div(M, 8), 256, 0, stream()>>>(A, out, M, N);
    else argmax_cols_kernel<<<ceil_div(N, 128), 128, 0, stream()>>>(A, out, M, N);
    ZNN_LAUNCH_OK("argmax kernel");
    return ZNN_OK;
}

int znn_accuracy_u8(const float* logits, const uint8_t* labels, int M, int N, float* acc)
{
    ZNN_REQUIRE(M > 0 && N > 0, "M and N must be positive");
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(logits && labels && acc, "NULL pointer");
    float* preds = (float*)workspace((size_t)M * sizeof(float));
    if (!preds) return fail(ZNN_ERR_NOMEM, "scratch for the predictions");
    argmax_rows_kernel<<<ceil_div(M, 8), 256, 0, stream()>>>(logits, preds, M, N);
    ZNN_LAUNCH_OK("argmax kernel");
    accuracy_u8_kernel<<<1, 1024, 0, stream()>>>(preds, labels, M, acc);
    ZNN_LAUNCH_OK("accuracy_u8_kernel");
    return ZNN_OK;
}

int znn_adam_step(float* w, const float* g, float* m, float* v, float lr, float beta1, float beta2, float eps, float t,
                  float grad_scale, size_t n)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(w && g && m && v, "NULL pointer");
    ZNN_REQUIRE(t >= 1.0f, "t is the step count after the increment (>= 1)");
    const float correction1 = 1.0f - powf(beta1, t);
    const float correction2 = 1.0f - powf(beta2, t);
    const float lr_t = lr * sqrtf(correction2) / correction1;
    adam_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(w, g, m, v, lr_t, beta1, beta2, eps, grad_scale, n);
    ZNN_LAUNCH_OK("adam_kernel");
    return ZNN_OK;
}

int znn_sgd_step(float* w, const float* g, float* v, float lr, float momentum, float grad_scale, size_t n)
{
    if (n == 0) return ZNN_OK;
    ZNN_NEED_DEVICE();
    ZNN_REQUIRE(w && g, "NULL pointer");
    ZNN_REQUIRE(v || momentum == 0.0f, "momentum needs a velocity buffer");
    sgd_kernel<<<ew_blocks(n), kEwThreads, 0, stream()>>>(w, g, (momentum > 0.0f) ? v : nullptr, lr, momentum, grad_scale, n);
    ZNN_LAUNCH_OK("sgd_kernel");
    return ZNN_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// SoftmaxCrossEntropy forward for callers that may not allocate
// ---------------------------------------------------------------------------
// znn_softmax_xent_fwd keeps its per-row losses in the shim's scratch block,
// which is grown with cudaMalloc when a call needs more than it holds.  Some
// callers cannot tolerate that: a serving loop whose memory budget was fixed at
// start-up and must not grow, or a latency-critical host thread that must never
// block on the allocator (cudaMalloc synchronises the whole device).  For them the per-row losses live in the fixed array below, which
// is part of the library image: every GPU that loads libznn_cuda.so holds these
// 256 KiB until the process exits, whether or not the entry point is used.
constexpr int kStaticXentMaxRows = 65536;
static __device__ __align__(256) float g_static_xent_rowloss[kStaticXentMaxRows];

// In host code the array's name is only a handle for the runtime, not an address
// a kernel can use; the device address is looked up once per device, with that
// device current, and cached here.
static float* g_static_xent_ptr[16] = {nullptr};
static std::mutex g_static_xent_mu;

static int static_xent_scratch(float** out)
{
    int dev = -1;
    ZNN_CUDA_OK(cudaGetDevice(&dev));
    ZNN_REQUIRE(dev >= 0 && dev < 16, "device index %d is outside the supported range", dev);
    std::lock_guard<std::mutex> lk(g_static_xent_mu);
    if (!g_static_xent_ptr[dev]) {
        float* p = nullptr;
        ZNN_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_static_xent_rowloss));
        ZNN_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a null device address");
        g_static_xent_ptr[dev] = p;
    }
    *out = g_static_xent_ptr[dev];
    return ZNN_OK;
}

extern "C" int znn_softmax_xent_fwd_static(const float* logits, const int32_t* targets, float* probs, float* loss,
                                           int M, int N, void* cuda_stream)
{
    ZNN_REQUIRE(M > 0 && N > 0, "empty logits");
    ZNN_REQUIRE(M <= kStaticXentMaxRows,
                "M = %d rows exceeds the %d rows the fixed scratch array holds; use znn_softmax_xent_fwd", M,
                kStaticXentMaxRows);
    ZNN_REQUIRE(logits && targets && probs && loss, "NULL pointer");
    float* rowloss = nullptr;
    const int rc = static_xent_scratch(&rowloss);
    if (rc != ZNN_OK) return rc;
    cudaStream_t st = (cudaStream_t)cuda_stream;
    const int threads = N >= 1024 ? 256 : (N >= 128 ? 128 : 32);
    // Rows 0..M-1 of the array are overwritten before they are read, so nothing has
    // to be cleared; rows beyond M keep whatever an earlier call left there.
    // no status word here (this entry point does not touch the shim's state): a label outside [0, N) makes the loss NaN
    softmax_xent_fwd_kernel<int32_t><<<M, threads, 0, st>>>(logits, targets, probs, rowloss, N, nullptr);
    ZNN_LAUNCH_OK("softmax_xent_fwd_kernel (fixed scratch)");
    mean_rows_kernel<<<1, 1024, 0, st>>>(rowloss, loss, M);
    ZNN_LAUNCH_OK("mean_rows_kernel (fixed scratch)");
    return ZNN_OK;
}
