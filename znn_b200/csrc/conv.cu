// Conv2D (NCHW, stride 1, optional zero padding) and MaxPool2D.
//
// Backward of all but tiny layers is lowered to GEMMs over an explicit im2col matrix:
//   dW[Co,K] += dYt^T . col,  dcol = dYt . W  followed by a col2im gather,  dbias = column sums of dYt,
// with col[p][k] the input taps under output pixel p and dYt the gradient in pixel-major order.
//
// The reference's convolutions have K = Ci*KH*KW between 9 and 288 and at most
// 64 output channels: far below a tensor-core tile, and a few GFLOP per step at
// most.  They run as direct CUDA-core kernels that keep the reference's
// summation order (bias, then ci -> kh -> kw) and, being compiled with
// -fmad=false, its rounding points: the forward pass is bit-identical to the
// reference loops, which is what keeps MaxPool argmax indices bit-exact.
#include "common.cuh"
#include "../../include/znn_debug.h"

namespace znn {

constexpr int kCoTile = 8;  // output channels per thread

// One thread: one output pixel (n, h, w) for kCoTile consecutive output channels.
// The weights of the channel tile sit in shared memory.
template <bool Relu>
__global__ void conv2d_fwd_kernel(const float* __restrict__ X, const float* __restrict__ W, const float* __restrict__ bias,
                                  float* __restrict__ Y, int N, int Ci, int H, int Wd, int Co, int KH, int KW, int pad,
                                  int Ho, int Wo)
{
    extern __shared__ float wsh[];  // [kCoTile][Ci*KH*KW]
    const int kk = Ci * KH * KW;
    const int co0 = blockIdx.y * kCoTile;
    for (int i = threadIdx.x; i < kCoTile * kk; i += blockDim.x) {
        const int c = i / kk;
        wsh[i] = (co0 + c < Co) ? W[(size_t)(co0 + c) * kk + (i - c * kk)] : 0.0f;
    }
    __syncthreads();
    const size_t pix = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const size_t npix = (size_t)N * Ho * Wo;
    if (pix >= npix) return;
    const int w = (int)(pix % Wo);
    const int h = (int)((pix / Wo) % Ho);
    const int n = (int)(pix / ((size_t)Wo * Ho));
    float acc[kCoTile];
#pragma unroll
    for (int c = 0; c < kCoTile; c++) acc[c] = (bias && co0 + c < Co) ? bias[co0 + c] : 0.0f;
    const float* xn = X + (size_t)n * Ci * H * Wd;
    int widx = 0;
    for (int ci = 0; ci < Ci; ci++)
        for (int kh = 0; kh < KH; kh++) {
            const int ih = h + kh - pad;
            for (int kw = 0; kw < KW; kw++, widx++) {
                const int iw = w + kw - pad;
                if (ih < 0 || ih >= H || iw < 0 || iw >= Wd) continue;
                const float xv = xn[((size_t)ci * H + ih) * Wd + iw];
#pragma unroll
                for (int c = 0; c < kCoTile; c++) acc[c] += xv * wsh[c * kk + widx];
            }
        }
#pragma unroll
    for (int c = 0; c < kCoTile; c++)
        if (co0 + c < Co) Y[(((size_t)n * Co + co0 + c) * Ho + h) * Wo + w] = Relu ? fmaxf(acc[c], 0.0f) : acc[c];
}

// dX[n,ci,ih,iw] += sum_{co,kh,kw} dY[n,co,ih-kh+pad,iw-kw+pad] * W[co,ci,kh,kw]  (gather form)
__global__ void conv2d_bwd_data_kernel(const float* __restrict__ dY, const float* __restrict__ W, float* __restrict__ dX,
                                       int N, int Ci, int H, int Wd, int Co, int KH, int KW, int pad, int Ho, int Wo)
{
    extern __shared__ float wsh[];  // all weights [Co][Ci][KH][KW]
    const int wtotal = Co * Ci * KH * KW;
    for (int i = threadIdx.x; i < wtotal; i += blockDim.x) wsh[i] = W[i];
    __syncthreads();
    const size_t total = (size_t)N * Ci * H * Wd;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const int iw = (int)(e % Wd);
        const int ih = (int)((e / Wd) % H);
        const int ci = (int)((e / ((size_t)Wd * H)) % Ci);
        const int n = (int)(e / ((size_t)Wd * H * Ci));
        float acc = 0.0f;
        for (int co = 0; co < Co; co++) {
            const float* dy = dY + ((size_t)n * Co + co) * Ho * Wo;
            const float* wk = wsh + ((size_t)co * Ci + ci) * KH * KW;
            for (int kh = 0; kh < KH; kh++) {
                const int h = ih - kh + pad;
                if (h < 0 || h >= Ho) continue;
                for (int kw = 0; kw < KW; kw++) {
                    const int w = iw - kw + pad;
                    if (w < 0 || w >= Wo) continue;
                    acc += dy[(size_t)h * Wo + w] * wk[kh * KW + kw];
                }
            }
        }
        dX[e] += acc;
    }
}

// One block per (co, ci): the KH*KW weight gradients of that pair, reduced over
// all (n, h, w) in a fixed order (thread-strided partial sums, then a tree).
__global__ void conv2d_bwd_weight_kernel(const float* __restrict__ X, const float* __restrict__ dY, float* __restrict__ dW,
                                         int N, int Ci, int H, int Wd, int Co, int KH, int KW, int pad, int Ho, int Wo)
{
    extern __shared__ float red[];  // [blockDim.x]
    const int co = blockIdx.x / Ci, ci = blockIdx.x % Ci;
    const size_t npix = (size_t)N * Ho * Wo;
    for (int kh = 0; kh < KH; kh++)
        for (int kw = 0; kw < KW; kw++) {
            float s = 0.0f;
            for (size_t pix = threadIdx.x; pix < npix; pix += blockDim.x) {
                const int w = (int)(pix % Wo);
                const int h = (int)((pix / Wo) % Ho);
                const int n = (int)(pix / ((size_t)Wo * Ho));
                const int ih = h + kh - pad, iw = w + kw - pad;
                if (ih < 0 || ih >= H || iw < 0 || iw >= Wd) continue;
                const float g = dY[(((size_t)n * Co + co) * Ho + h) * Wo + w];
                s += g * X[(((size_t)n * Ci + ci) * H + ih) * Wd + iw];
            }
            red[threadIdx.x] = s;
            __syncthreads();
            for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
                if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
                __syncthreads();
            }
            if (threadIdx.x == 0) dW[(((size_t)co * Ci + ci) * KH + kh) * KW + kw] += red[0];
            __syncthreads();
        }
}

__global__ void conv2d_bwd_bias_kernel(const float* __restrict__ dY, float* __restrict__ dbias, int N, int Co, int HoWo)
{
    extern __shared__ float red[];
    const int co = blockIdx.x;
    float s = 0.0f;
    const size_t total = (size_t)N * HoWo;
    for (size_t i = threadIdx.x; i < total; i += blockDim.x) {
        const size_t n = i / HoWo, r = i % HoWo;
        s += dY[(n * Co + co) * HoWo + r];
    }
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) dbias[co] += red[0];
}

// window origin (h*stride, w*stride); first maximum in (ph, pw) order wins (strict >)
__device__ __forceinline__ int pool_argmax(const float* __restrict__ x, int H, int W, int h, int w, int pool, int stride,
                                           float& best)
{
    int bi = (h * stride) * W + (w * stride);
    best = x[bi];
    for (int ph = 0; ph < pool; ph++)
        for (int pw = 0; pw < pool; pw++) {
            const int ih = h * stride + ph, iw = w * stride + pw;
            if (ih < H && iw < W) {
                const float v = x[ih * W + iw];
                if (v > best) { best = v; bi = ih * W + iw; }
            }
        }
    return bi;
}

__global__ void maxpool2d_fwd_kernel(const float* __restrict__ X, float* __restrict__ Y, int32_t* __restrict__ idx,
                                     size_t planes, int H, int W, int Ho, int Wo, int pool, int stride)
{
    const size_t total = planes * Ho * Wo;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const int w = (int)(e % Wo), h = (int)((e / Wo) % Ho);
        const size_t pl = e / ((size_t)Wo * Ho);
        float best;
        const int bi = pool_argmax(X + pl * H * W, H, W, h, w, pool, stride, best);
        Y[e] = best;
        if (idx) idx[e] = bi;
    }
}

// ReluMask: X is the output of a ReLU and dX the gradient of the ReLU's input: the winner receives g only where X > 0
// (MaxPool2D backward and Relu backward, src/autodiff.zig:996-1053 and :673-683, in one pass).
template <bool Overlap, bool ReluMask>
__global__ void maxpool2d_bwd_kernel(const float* __restrict__ X, const float* __restrict__ dY, float* __restrict__ dX,
                                     size_t planes, int H, int W, int Ho, int Wo, int pool, int stride)
{
    const size_t total = planes * Ho * Wo;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const float g = dY[e];
        if (g == 0.0f) continue;
        const int w = (int)(e % Wo), h = (int)((e / Wo) % Ho);
        const size_t pl = e / ((size_t)Wo * Ho);
        float best;
        const int bi = pool_argmax(X + pl * H * W, H, W, h, w, pool, stride, best);
        if (ReluMask && !(best > 0.0f)) continue;
        // windows are disjoint when stride >= pool: a plain add is race-free
        if (Overlap) atomicAdd(dX + pl * H * W + bi, g); else dX[pl * H * W + bi] += g;
    }
}


// ---- backward through GEMMs: im2col, pixel-major gradient, col2im ----
// col[p][k], p = (n, h, w) output pixel, k = (ci, kh, kw): the row of input taps under output pixel p
// (zero where the tap falls into the padding).  K contiguous.
__global__ void im2col_kernel(const float* __restrict__ X, float* __restrict__ col, int N, int Ci, int H, int Wd, int KH,
                              int KW, int pad, int Ho, int Wo)
{
    const int K = Ci * KH * KW;
    const size_t total = (size_t)N * Ho * Wo * K;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(e % K);
        const size_t p = e / K;
        const int w = (int)(p % Wo), h = (int)((p / Wo) % Ho), n = (int)(p / ((size_t)Wo * Ho));
        const int kw = k % KW, kh = (k / KW) % KH, ci = k / (KW * KH);
        const int ih = h + kh - pad, iw = w + kw - pad;
        col[e] = (ih >= 0 && ih < H && iw >= 0 && iw < Wd) ? X[(((size_t)n * Ci + ci) * H + ih) * Wd + iw] : 0.0f;
    }
}

// dY [N][Co][HW] -> dYt [N*HW][Co] (per-sample transpose through a shared tile)
__global__ void nchw_to_pixel_major_kernel(const float* __restrict__ dY, float* __restrict__ dYt, int Co, int HW)
{
    __shared__ float tile[32][33];
    const size_t n = blockIdx.z;
    const float* src = dY + n * (size_t)Co * HW;
    float* dst = dYt + n * (size_t)HW * Co;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int c = c0 + j, p = p0 + threadIdx.x;
        tile[j][threadIdx.x] = (c < Co && p < HW) ? src[(size_t)c * HW + p] : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int p = p0 + j, c = c0 + threadIdx.x;
        if (p < HW && c < Co) dst[(size_t)p * Co + c] = tile[threadIdx.x][j];
    }
}

// dX[n,ci,ih,iw] += sum_{kh,kw} dcol[p(n, ih-kh+pad, iw-kw+pad)][ci,kh,kw]   (gather: no atomics)
__global__ void col2im_add_kernel(const float* __restrict__ dcol, float* __restrict__ dX, int N, int Ci, int H, int Wd,
                                  int KH, int KW, int pad, int Ho, int Wo)
{
    const int K = Ci * KH * KW;
    const size_t total = (size_t)N * Ci * H * Wd;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const int iw = (int)(e % Wd), ih = (int)((e / Wd) % H);
        const int ci = (int)((e / ((size_t)Wd * H)) % Ci), n = (int)(e / ((size_t)Wd * H * Ci));
        float acc = 0.0f;
        for (int kh = 0; kh < KH; kh++) {
            const int h = ih - kh + pad;
            if (h < 0 || h >= Ho) continue;
            for (int kw = 0; kw < KW; kw++) {
                const int w = iw - kw + pad;
                if (w < 0 || w >= Wo) continue;
                acc += dcol[(((size_t)n * Ho + h) * Wo + w) * K + (ci * KH + kh) * KW + kw];
            }
        }
        dX[e] += acc;
    }
}

// ---- weight and bias gradients of a layer with few taps (K = Ci*KH*KW <= 40): no im2col matrix, no GEMM ----
// A block walks its share of the output pixels in tiles of 128: the taps under the tile's pixels and the tile of dY go
// to shared memory (coalesced along the pixels), then thread (co, k) adds the tile's 128 products to its sum; k = K is
// the bias column (a tap that is always 1).  Blocks write partial sums; a second kernel adds them in block order.
constexpr int kSkTile = 128;
constexpr int kSkThreads = 384;
__global__ void __launch_bounds__(kSkThreads)
conv2d_bwd_weight_smallk_kernel(const float* __restrict__ X, const float* __restrict__ dY, float* __restrict__ partial,
                                int Ci, int H, int Wd, int Co, int KH, int KW, int pad, int Ho, int Wo, int P,
                                int pix_per_block)
{
    extern __shared__ float sh[];
    const int K = Ci * KH * KW, K1 = K + 1;
    constexpr int pitch = kSkTile + 1;
    float* const cols = sh;                 // [K1][pitch]
    float* const dys = sh + K1 * pitch;     // [Co][pitch]
    const int pairs = Co * K1;
    const int i0 = threadIdx.x, i1 = threadIdx.x + kSkThreads;
    const int co0 = i0 / K1, k0 = i0 - co0 * K1, co1 = i1 / K1, k1 = i1 - co1 * K1;
    float acc0 = 0.0f, acc1 = 0.0f;
    const int HoWo = Ho * Wo, HW = H * Wd;
    const int p_begin = blockIdx.x * pix_per_block;
    const int p_end = min(P, p_begin + pix_per_block);
    // loading: thread = (pixel j of the tile, one of three row groups); the pixel is decoded once per tile
    const int j = threadIdx.x & (kSkTile - 1), grp = threadIdx.x / kSkTile;
    for (int t0 = p_begin; t0 < p_end; t0 += kSkTile) {
        const int pix = t0 + j;
        const bool pv = pix < p_end;
        int n = 0, h = 0, w = 0, hw = 0;
        if (pv) {
            n = pix / HoWo; hw = pix - n * HoWo;
            h = hw / Wo; w = hw - h * Wo;
        }
        const float* const xn = X + (size_t)n * Ci * HW;
        const float* const dyn = dY + (size_t)n * Co * HoWo + hw;
#pragma unroll 4
        for (int row = grp; row < K1 + Co; row += kSkThreads / kSkTile) {
            if (row < K1) {
                float v = 0.0f;
                if (pv) {
                    if (row == K) {
                        v = 1.0f;
                    } else {
                        const int kw = row % KW, kh = (row / KW) % KH, ci = row / (KW * KH);
                        const int ih = h + kh - pad, iw = w + kw - pad;
                        if (ih >= 0 && ih < H && iw >= 0 && iw < Wd) v = xn[(size_t)ci * HW + ih * Wd + iw];
                    }
                }
                cols[row * pitch + j] = v;
            } else {
                const int co = row - K1;
                dys[co * pitch + j] = pv ? dyn[(size_t)co * HoWo] : 0.0f;
            }
        }
        __syncthreads();
        if (i0 < pairs) {
            const float* a = dys + co0 * pitch;
            const float* b = cols + k0 * pitch;
#pragma unroll 8
            for (int jj = 0; jj < kSkTile; jj++) acc0 += a[jj] * b[jj];
        }
        if (i1 < pairs) {
            const float* a = dys + co1 * pitch;
            const float* b = cols + k1 * pitch;
#pragma unroll 8
            for (int jj = 0; jj < kSkTile; jj++) acc1 += a[jj] * b[jj];
        }
        __syncthreads();
    }
    if (i0 < pairs) partial[(size_t)blockIdx.x * pairs + i0] = acc0;
    if (i1 < pairs) partial[(size_t)blockIdx.x * pairs + i1] = acc1;
}

// One warp per (co, k) pair: lane l adds blocks l, l + 32, ... in order, then the 32 lane sums are added in lane order
// (a fixed order, whatever the scheduling).
__global__ void conv2d_bwd_weight_smallk_reduce_kernel(const float* __restrict__ partial, int blocks, int Co, int K,
                                                       float* __restrict__ dW, float* __restrict__ dbias)
{
    const int K1 = K + 1, pairs = Co * K1;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= pairs) return;
    const int co = i / K1, k = i - co * K1;
    if ((k == K) ? !dbias : !dW) return;
    float s = 0.0f;
    for (int b = lane; b < blocks; b += 32) s += partial[(size_t)b * pairs + i];
    float t = 0.0f;
    for (int l = 0; l < 32; l++) t += __shfl_sync(0xffffffffu, s, l);
    if (lane == 0) {
        if (k == K) dbias[co] += t;
        else dW[(size_t)co * K + k] += t;
    }
}

// the tensor-core path (conv_tc.cu)
bool conv_tc_applicable(long long n, int C, int H, int W, int Co, int KH, int KW, int Ho, int Wo);
int conv_tc_forward(const float* src, const float* wm, const float* bias, float* out, int N, int C, int H, int W, int Co,
                    int KH, int KW, int pad_h, int pad_w, int accumulate);
void conv_set_path(int mode);
int conv_profile_read(long long* out16);
size_t conv_tc_wgrad_scratch(long long P, int K, int Co);
int conv_tc_wgrad(const float* X, const float* dY, float* dW, float* dbias, float* scratch, int N, int Ci, int H, int W,
                  int Co, int KH, int KW, int pad, int Ho, int Wo);
int conv_tc_dgrad(const float* dY, const float* Wgt, float* dX, float* wt, int N, int Ci, int H, int W, int Co, int KH, int KW,
                  int pad, int Ho, int Wo);

}  // namespace znn

using namespace znn;

extern "C" {

int znn_debug_set_conv_path(int mode)
{
    ZNN_REQUIRE(mode == 0 || mode == 1, "mode is 0 or 1");
    conv_set_path(mode);
    return ZNN_OK;
}

int znn_debug_conv_profile(long long* out16)
{
    ZNN_REQUIRE(out16, "out16 is NULL");
    return conv_profile_read(out16);
}

int znn_conv2d_fwd_act(const float* X, const float* W, const float* bias, float* Y, int N, int Ci, int H, int Wd, int Co,
                       int KH, int KW, int pad, int act)
{
    ZNN_REQUIRE(N >= 0 && Ci > 0 && Co > 0 && KH > 0 && KW > 0 && pad >= 0, "bad conv shape");
    ZNN_REQUIRE(act == 0 || act == 1, "act is 0 (none) or 1 (ReLU)");
    const int Ho = H + 2 * pad - KH + 1, Wo = Wd + 2 * pad - KW + 1;
    ZNN_REQUIRE(Ho > 0 && Wo > 0, "kernel larger than padded input");
    if (N == 0) return ZNN_OK;
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (no CPU fallback)");
    ZNN_REQUIRE(X && W && Y, "NULL pointer");
    if (conv_tc_applicable(N, Ci, H, Wd, Co, KH, KW, Ho, Wo))   // implicit-im2col GEMM on the tensor cores
        return conv_tc_forward(X, W, bias, Y, N, Ci, H, Wd, Co, KH, KW, pad, pad, act ? 2 : 0);
    const size_t smem = (size_t)kCoTile * Ci * KH * KW * sizeof(float);
    ZNN_REQUIRE(smem <= 96 * 1024, "Ci*KH*KW = %d is beyond what the direct kernel keeps in shared memory", Ci * KH * KW);
    if (smem > 48 * 1024) {
        ZNN_CUDA_OK(cudaFuncSetAttribute(conv2d_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        ZNN_CUDA_OK(cudaFuncSetAttribute(conv2d_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    const size_t npix = (size_t)N * Ho * Wo;
    dim3 grid((unsigned)((npix + 127) / 128), ceil_div(Co, kCoTile));
    if (act) conv2d_fwd_kernel<true><<<grid, 128, smem, stream()>>>(X, W, bias, Y, N, Ci, H, Wd, Co, KH, KW, pad, Ho, Wo);
    else conv2d_fwd_kernel<false><<<grid, 128, smem, stream()>>>(X, W, bias, Y, N, Ci, H, Wd, Co, KH, KW, pad, Ho, Wo);
    ZNN_LAUNCH_OK("conv2d_fwd_kernel");
    return ZNN_OK;
}

int znn_conv2d_fwd(const float* X, const float* W, const float* bias, float* Y, int N, int Ci, int H, int Wd, int Co,
                   int KH, int KW, int pad)
{
    return znn_conv2d_fwd_act(X, W, bias, Y, N, Ci, H, Wd, Co, KH, KW, pad, 0);
}

int znn_conv2d_bwd(const float* X, const float* W, const float* dY, float* dX, float* dW, float* dbias, int N, int Ci,
                   int H, int Wd, int Co, int KH, int KW, int pad)
{
    ZNN_REQUIRE(N >= 0 && Ci > 0 && Co > 0 && KH > 0 && KW > 0 && pad >= 0, "bad conv shape");
    const int Ho = H + 2 * pad - KH + 1, Wo = Wd + 2 * pad - KW + 1;
    ZNN_REQUIRE(Ho > 0 && Wo > 0, "kernel larger than padded input");
    if (N == 0) return ZNN_OK;
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (no CPU fallback)");
    ZNN_REQUIRE(X && W && dY, "NULL pointer");
    const size_t P = (size_t)N * Ho * Wo;   // output pixels
    const int K = Ci * KH * KW;
    {
        // Tensor-core path: weight (and bias) gradient with the pixels as the contraction, data gradient as a
        // convolution of dY with the flipped weights; neither writes an im2col matrix.  What it does not take
        // falls through to the paths below.
        const bool tc_w = (dW || dbias) && conv_tc_applicable(N, Ci, H, Wd, Co, KH, KW, Ho, Wo);
        const bool tc_x = dX && pad <= KH - 1 && pad <= KW - 1 && conv_tc_applicable(N, Co, Ho, Wo, Ci, KH, KW, H, Wd);
        if (tc_w || tc_x) {
            const size_t wg_f = tc_w ? conv_tc_wgrad_scratch((long long)P, K, Co) : 0;
            const size_t wt_f = tc_x ? (size_t)Co * K : 0;
            float* ws = (float*)workspace_slot(1, (wg_f + wt_f) * sizeof(float));
            if (!ws) return fail(ZNN_ERR_NOMEM, "conv backward scratch (%zu bytes)", (wg_f + wt_f) * sizeof(float));
            int rc;
            if (tc_w) {
                if ((rc = conv_tc_wgrad(X, dY, dW, dbias, ws, N, Ci, H, Wd, Co, KH, KW, pad, Ho, Wo))) return rc;
                dW = nullptr;
                dbias = nullptr;
            }
            if (tc_x) {
                if ((rc = conv_tc_dgrad(dY, W, dX, ws + wg_f, N, Ci, H, Wd, Co, KH, KW, pad, Ho, Wo))) return rc;
                dX = nullptr;
            }
            if (!dW && !dbias && !dX) return ZNN_OK;
        }
    }
    if ((dW || dbias) && P >= 4096 && P < ((size_t)1 << 30) && K <= 40 && Co <= 64 && Co * (K + 1) <= 2 * kSkThreads) {
        // few taps: per-block partial sums over the pixels, added in block order (no im2col matrix, no GEMM)
        const int blocks = sm_count() * 2;
        long long per = ((long long)P + blocks - 1) / blocks;
        per = (per + kSkTile - 1) / kSkTile * kSkTile;
        const int used = (int)(((long long)P + per - 1) / per);
        const int pairs = Co * (K + 1);
        float* part = (float*)workspace_slot(1, (size_t)used * pairs * sizeof(float));
        if (!part) return fail(ZNN_ERR_NOMEM, "conv backward scratch");
        const size_t smem = (size_t)(K + 1 + Co) * (kSkTile + 1) * sizeof(float);
        if (smem > 48 * 1024)
            ZNN_CUDA_OK(cudaFuncSetAttribute(conv2d_bwd_weight_smallk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        conv2d_bwd_weight_smallk_kernel<<<used, kSkThreads, smem, stream()>>>(X, dY, part, Ci, H, Wd, Co, KH, KW, pad, Ho, Wo,
                                                                              (int)P, (int)per);
        ZNN_LAUNCH_OK("conv2d_bwd_weight_smallk_kernel");
        conv2d_bwd_weight_smallk_reduce_kernel<<<(pairs + 7) / 8, 256, 0, stream()>>>(part, used, Co, K, dW, dbias);
        ZNN_LAUNCH_OK("conv2d_bwd_weight_smallk_reduce_kernel");
        dW = nullptr;
        dbias = nullptr;
        if (!dX) return ZNN_OK;
    }
    // Large layers: lower the backward pass to GEMMs over an explicit im2col matrix (the contraction runs
    // on the tensor cores / the split-K FMA kernel).  Tiny layers keep the direct kernels below.
    if (P >= 4096 && P * (size_t)K <= ((size_t)1 << 31) && P <= 0x7fffffff / 2) {
        const size_t col_f = (dW || dX) ? P * K : 0;
        const size_t dyt_f = P * (size_t)Co;
        float* ws = (float*)workspace_slot(1, (col_f + dyt_f) * sizeof(float));
        if (!ws) return fail(ZNN_ERR_NOMEM, "conv backward scratch (%zu bytes)", (col_f + dyt_f) * sizeof(float));
        float* col = ws;              // im2col(X) for dW, then reused as dcol for dX
        float* dyt = ws + col_f;
        const int cap = sm_count() * 16;
        {
            dim3 grid(ceil_div(Ho * Wo, 32), ceil_div(Co, 32), N), block(32, 8);
            nchw_to_pixel_major_kernel<<<grid, block, 0, stream()>>>(dY, dyt, Co, Ho * Wo);
            ZNN_LAUNCH_OK("nchw_to_pixel_major_kernel");
        }
        int rc;
        if (dbias && (rc = znn_add_bias_bwd(dyt, nullptr, dbias, (int)P, Co))) return rc;   // column sums over pixels
        if (dW) {
            size_t blocks = (P * K + 255) / 256;
            if (blocks > (size_t)cap) blocks = cap;
            im2col_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(X, col, N, Ci, H, Wd, KH, KW, pad, Ho, Wo);
            ZNN_LAUNCH_OK("im2col_kernel");
            // dW[Co,K] += dYt^T[Co,P] . col[P,K]
            if ((rc = znn_sgemm(ZNN_ROW_MAJOR, ZNN_TRANS, ZNN_NO_TRANS, Co, K, (int)P, 1.0f, dyt, Co, col, K, 1.0f, dW, K)))
                return rc;
        }
        if (dX) {
            // dcol[P,K] = dYt[P,Co] . W[Co,K], then gather back onto the input
            if ((rc = znn_sgemm(ZNN_ROW_MAJOR, ZNN_NO_TRANS, ZNN_NO_TRANS, (int)P, K, Co, 1.0f, dyt, Co, W, K, 0.0f, col, K)))
                return rc;
            const size_t total = (size_t)N * Ci * H * Wd;
            size_t blocks = (total + 255) / 256;
            if (blocks > (size_t)cap) blocks = cap;
            col2im_add_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(col, dX, N, Ci, H, Wd, KH, KW, pad, Ho, Wo);
            ZNN_LAUNCH_OK("col2im_add_kernel");
        }
        return ZNN_OK;
    }
    if (dbias) {
        conv2d_bwd_bias_kernel<<<Co, 256, 256 * sizeof(float), stream()>>>(dY, dbias, N, Co, Ho * Wo);
        ZNN_LAUNCH_OK("conv2d_bwd_bias_kernel");
    }
    if (dW) {
        conv2d_bwd_weight_kernel<<<Co * Ci, 256, 256 * sizeof(float), stream()>>>(X, dY, dW, N, Ci, H, Wd, Co, KH, KW, pad,
                                                                                  Ho, Wo);
        ZNN_LAUNCH_OK("conv2d_bwd_weight_kernel");
    }
    if (dX) {
        const size_t smem = (size_t)Co * Ci * KH * KW * sizeof(float);
        ZNN_REQUIRE(smem <= 200 * 1024, "weights (%zu bytes) beyond the shared memory of the data-gradient kernel", smem);
        if (smem > 48 * 1024)
            ZNN_CUDA_OK(cudaFuncSetAttribute(conv2d_bwd_data_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const size_t total = (size_t)N * Ci * H * Wd;
        size_t blocks = (total + 255) / 256;
        const size_t cap = (size_t)sm_count() * 8;
        if (blocks > cap) blocks = cap;
        conv2d_bwd_data_kernel<<<(unsigned)blocks, 256, smem, stream()>>>(dY, W, dX, N, Ci, H, Wd, Co, KH, KW, pad, Ho, Wo);
        ZNN_LAUNCH_OK("conv2d_bwd_data_kernel");
    }
    return ZNN_OK;
}

int znn_maxpool2d_fwd(const float* X, float* Y, int32_t* idx, int N, int C, int H, int W, int pool, int stride)
{
    ZNN_REQUIRE(pool > 0 && stride > 0, "bad pooling parameters");
    const int Ho = H / stride, Wo = W / stride;
    const size_t planes = (size_t)N * C;
    if (planes == 0 || Ho == 0 || Wo == 0) return ZNN_OK;
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (no CPU fallback)");
    const size_t total = planes * Ho * Wo;
    size_t blocks = (total + 255) / 256;
    const size_t cap = (size_t)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    maxpool2d_fwd_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(X, Y, idx, planes, H, W, Ho, Wo, pool, stride);
    ZNN_LAUNCH_OK("maxpool2d_fwd_kernel");
    return ZNN_OK;
}

static int maxpool2d_bwd_impl(const float* X, const float* dY, float* dX, int N, int C, int H, int W, int pool, int stride,
                              bool relu_mask)
{
    ZNN_REQUIRE(pool > 0 && stride > 0, "bad pooling parameters");
    const int Ho = H / stride, Wo = W / stride;
    const size_t planes = (size_t)N * C;
    if (planes == 0 || Ho == 0 || Wo == 0 || !dX) return ZNN_OK;
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (no CPU fallback)");
    const size_t total = planes * Ho * Wo;
    size_t blocks = (total + 255) / 256;
    const size_t cap = (size_t)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    const unsigned nb = (unsigned)blocks;
    if (stride < pool) {
        if (relu_mask) maxpool2d_bwd_kernel<true, true><<<nb, 256, 0, stream()>>>(X, dY, dX, planes, H, W, Ho, Wo, pool, stride);
        else maxpool2d_bwd_kernel<true, false><<<nb, 256, 0, stream()>>>(X, dY, dX, planes, H, W, Ho, Wo, pool, stride);
    } else {
        if (relu_mask) maxpool2d_bwd_kernel<false, true><<<nb, 256, 0, stream()>>>(X, dY, dX, planes, H, W, Ho, Wo, pool, stride);
        else maxpool2d_bwd_kernel<false, false><<<nb, 256, 0, stream()>>>(X, dY, dX, planes, H, W, Ho, Wo, pool, stride);
    }
    ZNN_LAUNCH_OK("maxpool2d_bwd_kernel");
    return ZNN_OK;
}

int znn_maxpool2d_bwd(const float* X, const float* dY, float* dX, int N, int C, int H, int W, int pool, int stride)
{
    return maxpool2d_bwd_impl(X, dY, dX, N, C, H, W, pool, stride, false);
}

int znn_maxpool2d_bwd_relu(const float* X, const float* dY, float* dX, int N, int C, int H, int W, int pool, int stride)
{
    return maxpool2d_bwd_impl(X, dY, dX, N, C, H, W, pool, stride, true);
}

}  // extern "C"
