// znn_sgemm / znn_sgemm_batched_strided: the cblas_sgemm boundary of the
// reference (src/cblas.zig:17-34) on device pointers.  Large problems go to the
// tcgen05 3xTF32 kernel (gemm_tc.cu); small or launch-bound ones to the fp32 FMA
// kernel below, which takes any transposes, leading dimensions and alignment.
#include <stdlib.h>

#include "common.cuh"
#include "../../include/znn_debug.h"

namespace znn {

int gemm_tc(int ta, int tb, int M, int N, int K, float alpha, const float* A, long long lda, long long stride_a,
            const float* B, long long ldb, long long stride_b, float beta, float* C, long long ldc,
            long long stride_c, int batch, int ctas, const float* bias);
bool gemm_tc_direct_eligible(const float* A, long long lda, long long stride_a, const float* B, long long ldb,
                             long long stride_b, int batch);
int gemm_tc_direct(int ta, int tb, int M, int N, int K, float alpha, const float* A, long long lda, long long stride_a,
                   const float* B, long long ldb, long long stride_b, float beta, float* C, long long ldc,
                   long long stride_c, int batch, const float* bias, int tri, const float* ep_p, const float* ep_d,
                   int ep_act, float* ep_out2, const float* ep_res, const float* ep_dpre, long long stride_bias, int kcat);
int launch_splitk_reduce(const float* partial, int splits, int M, int N, int batch, float alpha, float beta, float* C,
                         long long ldc, long long stride_c, const float* bias);
bool tc_plan_splits_k(int M, int N, int K);
int tc_profile_enable(int enable);
void tc_set_chunk_kblocks(int v);
void tc_set_splitk(int on);
void tc_set_persistent(int on);
void tc_set_tail_split(int on);
int tc_wait_record(int* out16);
void tc_set_conv_mode(int m);
int tc_profile_read(double* kernel_ms, long long* launches, double* flops);
void tc_set_wait_limit(unsigned long long cycles);
int tc_wait_probe(unsigned long long limit_cycles);

// C = alpha * op(A) * op(B) + beta * C with fp32 FMAs, k ascending.
// 64x64 output tile, 16-deep k slices, 256 threads, 4x4 outputs per thread.
__global__ void __launch_bounds__(256)
sgemm_fma_kernel(int M, int N, int K, float alpha, const float* __restrict__ A, long long sa_i, long long sa_p,
                 long long stride_a, const float* __restrict__ B, long long sb_p, long long sb_j, long long stride_b,
                 float beta, float* __restrict__ C, long long ldc, long long stride_c, int splits, int k_per_split,
                 const float* __restrict__ bias)
{
    __shared__ float As[16][64 + 4];
    __shared__ float Bs[16][64 + 4];
    // blockIdx.z = slice * batch + b; with split-K (splits > 1) C is the [splits][batch][M][N] partial buffer
    const int nbatch = gridDim.z / splits;
    const int b = blockIdx.z % nbatch, slice = blockIdx.z / nbatch;
    const int k_begin = slice * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    A += (size_t)b * stride_a;
    B += (size_t)b * stride_b;
    C += (size_t)b * stride_c + (size_t)slice * nbatch * stride_c;
    const int i0 = blockIdx.y * 64, j0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[r][c] = 0.0f;

    // loader mapping: pick the index that is contiguous in memory as the fast one
    const bool a_p_fast = (sa_p == 1);
    const bool b_j_fast = (sb_j == 1);
    for (int p0 = k_begin; p0 < k_end; p0 += 16) {
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const int e = threadIdx.x + t * 256;  // 0..1023
            int li, lp;
            if (a_p_fast) { lp = e & 15; li = e >> 4; } else { li = e & 63; lp = e >> 6; }
            const int gi = i0 + li, gp = p0 + lp;
            As[lp][li] = (gi < M && gp < k_end) ? A[(size_t)gi * sa_i + (size_t)gp * sa_p] : 0.0f;
            int lj, lq;
            if (b_j_fast) { lj = e & 63; lq = e >> 6; } else { lq = e & 15; lj = e >> 4; }
            const int gj = j0 + lj, gq = p0 + lq;
            Bs[lq][lj] = (gj < N && gq < k_end) ? B[(size_t)gq * sb_p + (size_t)gj * sb_j] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int p = 0; p < 16; p++) {
            float a[4], bb[4];
#pragma unroll
            for (int r = 0; r < 4; r++) a[r] = As[p][ty * 4 + r];
#pragma unroll
            for (int c = 0; c < 4; c++) bb[c] = Bs[p][tx * 4 + c];
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) acc[r][c] = fmaf(a[r], bb[c], acc[r][c]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int gi = i0 + ty * 4 + r;
        if (gi >= M) continue;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int gj = j0 + tx * 4 + c;
            if (gj >= N) continue;
            float* dst = C + (size_t)gi * ldc + gj;
            float o = alpha * acc[r][c];
            if (bias) o += bias[gj];
            if (beta != 0.0f) o += beta * (*dst);
            *dst = o;
        }
    }
}

// C[m][n] = T[n][m] + bias[n] + beta * C[m][n]: the last step of a skinny product that was computed transposed
__global__ void transpose_finish_kernel(const float* __restrict__ T, int M, int N, const float* __restrict__ bias, float beta,
                                        float* __restrict__ C, long long ldc)
{
    __shared__ float tile[32][33];
    const int n0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int n = n0 + j, m = m0 + threadIdx.x;
        tile[j][threadIdx.x] = (n < N && m < M) ? T[(size_t)n * M + m] : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int m = m0 + j, n = n0 + threadIdx.x;
        if (m < M && n < N) {
            float o = tile[threadIdx.x][j];
            if (bias) o += bias[n];
            float* dst = C + (size_t)m * ldc + n;
            if (beta != 0.0f) o += beta * (*dst);
            *dst = o;
        }
    }
}

// beta pass for the degenerate cases (K == 0 or alpha == 0), cblas.zig:56-70.
__global__ void scale_c_kernel(float* C, long long ldc, long long stride_c, int M, int N, float beta)
{
    float* c = C + (size_t)blockIdx.z * stride_c;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < (size_t)M * N;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / N, col = i % N;
        float* d = c + r * ldc + col;
        *d = (beta == 0.0f) ? 0.0f : beta * (*d);
    }
}

static thread_local bool t_skinny = true;  // products of at most 64 rows are computed transposed (znn_gemm_set_skinny)
static thread_local int t_path = 0;       // requested
static thread_local int t_last_path = 0;  // taken by the last call

// bias (optional, [N]) is added to every row of the result: the fused form of MatMul + AddBias
static int gemm_dispatch(int ta, int tb, int M, int N, int K, float alpha, const float* A, long long lda,
                         long long stride_a, const float* B, long long ldb, long long stride_b, float beta, float* C,
                         long long ldc, long long stride_c, int batch, const float* bias = nullptr, int tri = 0,
                         const float* ep_p = nullptr, const float* ep_d = nullptr, int ep_act = 0, float* ep_out2 = nullptr,
                         const float* ep_res = nullptr, const float* ep_dpre = nullptr, long long stride_bias = 0, int kcat = 0,
                         bool grouped = false)
{
    ZNN_REQUIRE(ta == ZNN_NO_TRANS || ta == ZNN_TRANS, "trans_a must be 111 or 112");
    ZNN_REQUIRE(tb == ZNN_NO_TRANS || tb == ZNN_TRANS, "trans_b must be 111 or 112");
    ZNN_REQUIRE(M >= 0 && N >= 0 && K >= 0 && batch >= 0, "negative dimension");
    if (M == 0 || N == 0 || batch == 0) return ZNN_OK;
    ZNN_REQUIRE(C, "C is NULL");
    ZNN_REQUIRE(ldc >= N, "ldc (%lld) < N (%d)", ldc, N);
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (this library has no CPU fallback)");
    if (K == 0 || alpha == 0.0f) {
        ZNN_REQUIRE(!bias, "bias with an empty contraction is not supported");
        if (beta != 1.0f) {
            const int blocks = ceil_div((long)M * N, 256) > 4096 ? 4096 : ceil_div((long)M * N, 256);
            scale_c_kernel<<<dim3(blocks, 1, batch), 256, 0, stream()>>>(C, ldc, stride_c, M, N, beta);
            ZNN_LAUNCH_OK("scale_c_kernel");
        }
        t_last_path = 1;
        return ZNN_OK;
    }
    ZNN_REQUIRE(A && B, "A or B is NULL");
    ZNN_REQUIRE(lda >= (ta == ZNN_NO_TRANS ? K : M), "lda too small");
    ZNN_REQUIRE(ldb >= (tb == ZNN_NO_TRANS ? N : K), "ldb too small");

    int path = t_path;
    const bool direct_ok = gemm_tc_direct_eligible(A, lda, stride_a, B, ldb, stride_b, batch);
    if (ep_p || ep_act != 0 || ep_res || grouped) {   // the fused epilogues and the grouped forms exist on the in-place tensor-core path only
        if (!direct_ok) return fail(ZNN_ERR_UNSUPPORTED, "fused epilogue / grouped product: operands not readable in place");
        path = 4;
    }
    if (path == 0 && t_skinny && batch == 1 && tri == 0 && !grouped && M >= 8 && M <= 64 && (M & 3) == 0 && N >= 512 && K >= 512 &&
        2.0 * M * N * (double)K >= 1.3e8 && gemm_tc_direct_eligible(B, ldb, 0, A, lda, 0, 1)) {
        // A few rows against a wide matrix (a 64-row batch against a weight matrix: decode, the sweep's skinny shapes):
        // as it stands the product would fill a quarter of one 256-row tile per column block and leave most SMs idle.
        // The transposed product C^T = op(B)^T . op(A)^T has N rows (many tiles, split over K as well) and M <= 64
        // columns; a small kernel writes it back transposed, adding bias and beta * C on the way.
        float* T = (float*)workspace_slot(1, (size_t)N * M * sizeof(float));
        if (T) {
            const int ta2 = (tb == ZNN_NO_TRANS) ? ZNN_TRANS : ZNN_NO_TRANS, tb2 = (ta == ZNN_NO_TRANS) ? ZNN_TRANS : ZNN_NO_TRANS;
            int rc = gemm_tc_direct(ta2, tb2, N, M, K, alpha, B, ldb, 0, A, lda, 0, 0.0f, T, M, 0, 1, nullptr, 0, nullptr, nullptr,
                                    0, nullptr, nullptr, nullptr, 0, 0);
            if (rc) return rc;
            transpose_finish_kernel<<<dim3(ceil_div(N, 32), ceil_div(M, 32)), dim3(32, 8), 0, stream()>>>(T, M, N, bias, beta, C, ldc);
            ZNN_LAUNCH_OK("transpose_finish_kernel");
            t_last_path = 5;
            return ZNN_OK;
        }
    }
    if (path == 0) {
        // The tensor-core paths cost extra launches; below ~0.13 GFLOP per call the FMA kernel finishes sooner.
        const double flops = 2.0 * M * N * (double)K * batch;
        if (!(flops >= 1.3e8 && M >= 64 && N >= 32 && K >= 32)) {
            path = 1;
        } else {
            // In place whenever TMA can read the operands where they lie: the in-place kernel runs as fast as the
            // planes kernel (measured on B200: 270 TFLOP/s at 8192^3 for both) and has no split pre-pass.
            path = direct_ok ? 4 : 3;
        }
    }
    // the in-place path needs TMA-readable operands; otherwise the pre-split planes path takes any layout
    if (path == 4 && !direct_ok) path = 3;
    t_last_path = path;
    if (path >= 2) {
        int rc = (path == 4) ? gemm_tc_direct(ta, tb, M, N, K, alpha, A, lda, stride_a, B, ldb, stride_b, beta, C, ldc,
                                              stride_c, batch, bias, tri, ep_p, ep_d, ep_act, ep_out2, ep_res, ep_dpre, stride_bias, kcat)
                             : gemm_tc(ta, tb, M, N, K, alpha, A, lda, stride_a, B, ldb, stride_b, beta, C, ldc, stride_c,
                                       batch, path == 2 ? 1 : 2, bias);
        // Debug aid (environment ZNN_GEMM_CHECK=1): wait for every tensor-core product and name the first one
        // whose kernel reported an expired device-side wait.
        static const bool check = [] { const char* e = getenv("ZNN_GEMM_CHECK"); return e && e[0] == '1'; }();
        if (rc == ZNN_OK && check) {
            int st = 0;
            ZNN_CUDA_OK(cudaStreamSynchronize(stream()));
            ZNN_CUDA_OK(cudaMemcpy(&st, device_status_word(), sizeof(int), cudaMemcpyDeviceToHost));
            if (st != 0)
                return fail(ZNN_ERR_CUDA,
                            "device status %d after GEMM path %d ta %d tb %d M %d N %d K %d batch %d lda %lld ldb %lld ldc %lld "
                            "beta %g bias %d A %p B %p C %p",
                            st, path, ta, tb, M, N, K, batch, lda, ldb, ldc, (double)beta, bias != nullptr, (const void*)A,
                            (const void*)B, (void*)C);
        }
        return rc;
    }

    const long long sa_i = (ta == ZNN_NO_TRANS) ? lda : 1, sa_p = (ta == ZNN_NO_TRANS) ? 1 : lda;
    const long long sb_p = (tb == ZNN_NO_TRANS) ? ldb : 1, sb_j = (tb == ZNN_NO_TRANS) ? 1 : ldb;
    // few output tiles and a long contraction (small-channel conv weight gradients): split K over blocks,
    // partial tiles to scratch, fixed-order reduction
    const long tiles = (long)ceil_div(N, 64) * ceil_div(M, 64) * batch;
    int splits = 1;
    if (tiles * 2 <= sm_count() && K >= 256) {
        // slices of at least 64 contraction elements (128 once K is long): a 64-row product against a wide weight matrix
        // (decode, the MLP layers) is a stream over the weights and needs every SM on it
        const int min_slice = K >= 2048 ? 128 : 64;
        splits = (int)((2L * sm_count()) / tiles);
        if (splits > K / min_slice) splits = K / min_slice;
        if (splits > 128) splits = 128;
        if ((long)splits * batch > 65535) splits = 65535 / batch;
        if (splits < 1) splits = 1;
    }
    if (splits > 1) {
        int kps = (K + splits - 1) / splits;
        kps = ((kps + 15) / 16) * 16;
        splits = (K + kps - 1) / kps;
        float* partial = (float*)workspace((size_t)splits * batch * M * N * sizeof(float));
        if (!partial) return fail(ZNN_ERR_NOMEM, "split-K scratch could not be allocated");
        dim3 grid(ceil_div(N, 64), ceil_div(M, 64), batch * splits);
        sgemm_fma_kernel<<<grid, 256, 0, stream()>>>(M, N, K, 1.0f, A, sa_i, sa_p, stride_a, B, sb_p, sb_j, stride_b, 0.0f,
                                                     partial, N, (long long)M * N, splits, kps, nullptr);
        ZNN_LAUNCH_OK("sgemm_fma_kernel (split-K)");
        return launch_splitk_reduce(partial, splits, M, N, batch, alpha, beta, C, ldc, stride_c, bias);
    }
    dim3 grid(ceil_div(N, 64), ceil_div(M, 64), batch);
    sgemm_fma_kernel<<<grid, 256, 0, stream()>>>(M, N, K, alpha, A, sa_i, sa_p, stride_a, B, sb_p, sb_j, stride_b,
                                                 beta, C, ldc, stride_c, 1, K, bias);
    ZNN_LAUNCH_OK("sgemm_fma_kernel");
    return ZNN_OK;
}

}  // namespace znn

using namespace znn;

extern "C" {

int znn_sgemm(int order, int trans_a, int trans_b, int M, int N, int K, float alpha, const float* A, int lda,
              const float* B, int ldb, float beta, float* C, int ldc)
{
    ZNN_REQUIRE(order == ZNN_ROW_MAJOR, "only row-major (101) is supported, as in the reference");
    return gemm_dispatch(trans_a, trans_b, M, N, K, alpha, A, lda, 0, B, ldb, 0, beta, C, ldc, 0, 1);
}

int znn_sgemm_batched_strided(int trans_a, int trans_b, int M, int N, int K, float alpha, const float* A, int lda,
                              long long stride_a, const float* B, int ldb, long long stride_b, float beta, float* C,
                              int ldc, long long stride_c, int batch)
{
    ZNN_REQUIRE(batch <= 65535, "batch %d exceeds 65535", batch);
    return gemm_dispatch(trans_a, trans_b, M, N, K, alpha, A, lda, stride_a, B, ldb, stride_b, beta, C, ldc, stride_c,
                         batch);
}

int znn_sgemm_batched_strided_tri(int trans_a, int trans_b, int M, int N, int K, float alpha, const float* A, int lda,
                                  long long stride_a, const float* B, int ldb, long long stride_b, float beta, float* C,
                                  int ldc, long long stride_c, int batch, int tri)
{
    ZNN_REQUIRE(batch <= 65535, "batch %d exceeds 65535", batch);
    ZNN_REQUIRE(tri >= ZNN_TRI_NONE && tri <= ZNN_TRI_B_LOWER, "tri must be one of ZNN_TRI_*");
    return gemm_dispatch(trans_a, trans_b, M, N, K, alpha, A, lda, stride_a, B, ldb, stride_b, beta, C, ldc, stride_c,
                         batch, nullptr, tri);
}

int znn_attn_dscores(const float* dO, const float* V, const float* P, const float* D, float scale, float* dS, int T, int hs,
                     int nslices)
{
    ZNN_REQUIRE(dO && V && P && D && dS, "NULL pointer");
    ZNN_REQUIRE(T > 0 && hs > 0 && nslices > 0 && nslices <= 65535, "bad dimensions");
    return gemm_dispatch(ZNN_NO_TRANS, ZNN_TRANS, T, T, hs, scale, dO, hs, (long long)T * hs, V, hs, (long long)T * hs, 0.0f, dS, T,
                         (long long)T * T, nslices, nullptr, ZNN_TRI_C_LOWER, P, D);
}

int znn_linear_fwd(const float* X, const float* W, const float* bias, float* Y, int M, int K, int N)
{
    ZNN_REQUIRE(bias, "bias is NULL");
    return gemm_dispatch(ZNN_NO_TRANS, ZNN_NO_TRANS, M, N, K, 1.0f, X, K, 0, W, N, 0, 0.0f, Y, N, 0, 1, bias);
}

int znn_linear_bwd(const float* X, const float* W, const float* dY, float* dX, float* dW, float* dbias, int M, int K, int N)
{
    int rc;
    if (dbias && (rc = znn_add_bias_bwd(dY, nullptr, dbias, M, N))) return rc;
    if (dX && (rc = gemm_dispatch(ZNN_NO_TRANS, ZNN_TRANS, M, K, N, 1.0f, dY, N, 0, W, N, 0, 1.0f, dX, K, 0, 1))) return rc;
    if (dW && (rc = gemm_dispatch(ZNN_TRANS, ZNN_NO_TRANS, K, N, M, 1.0f, X, K, 0, dY, N, 0, 1.0f, dW, N, 0, 1))) return rc;
    return ZNN_OK;
}

int znn_linear_fwd_ex(const float* X, const float* W, const float* bias, float* Y, float* pre, const float* residual, int M,
                      int K, int N, int act)
{
    ZNN_REQUIRE(bias, "bias is NULL");
    ZNN_REQUIRE(act >= 0 && act <= 2, "act is 0 (none), 1 (ReLU) or 2 (GELU)");
    if (act == 0 && !residual) return znn_linear_fwd(X, W, bias, Y, M, K, N);
    // the epilogue forms live on the tensor-core path: shapes the dispatcher sends to the FMA kernel keep the two-op form
    if (!(2.0 * M * N * (double)K >= 1.3e8 && M >= 64 && N >= 32 && K >= 32))
        return fail(ZNN_ERR_UNSUPPORTED, "fused epilogue: product too small for the tensor-core path");
    if (tc_plan_splits_k(M, N, K))   // few tiles, long contraction: the split-K form (partials + reduce kernel) is faster
        return fail(ZNN_ERR_UNSUPPORTED, "fused epilogue: this product is split over K");
    return gemm_dispatch(ZNN_NO_TRANS, ZNN_NO_TRANS, M, N, K, 1.0f, X, K, 0, W, N, 0, 0.0f, Y, N, 0, 1, bias, 0, nullptr, nullptr,
                         act, pre, residual, nullptr);
}

int znn_linear_bwd_ex(const float* X, const float* W, const float* dY, float* dX, float* dW, float* dbias, int M, int K, int N,
                      const float* x_pre, int x_act, int dx_fresh)
{
    ZNN_REQUIRE(x_act >= 0 && x_act <= 2, "x_act is 0 (none), 1 (ReLU) or 2 (GELU)");
    if (x_act == 0 || !dX) return znn_linear_bwd(X, W, dY, dX, dW, dbias, M, K, N);
    ZNN_REQUIRE(x_pre, "x_pre is NULL");
    if (!(2.0 * M * N * (double)K >= 1.3e8 && M >= 64 && K >= 32 && N >= 32))
        return fail(ZNN_ERR_UNSUPPORTED, "fused epilogue: product too small for the tensor-core path");
    if (tc_plan_splits_k(M, K, N)) return fail(ZNN_ERR_UNSUPPORTED, "fused epilogue: this product is split over K");
    int rc;
    // dX (+)= (dY . W^T) o act'(x_pre): the gradient with respect to the pre-activation of the layer below
    if ((rc = gemm_dispatch(ZNN_NO_TRANS, ZNN_TRANS, M, K, N, 1.0f, dY, N, 0, W, N, 0, dx_fresh ? 0.0f : 1.0f, dX, K, 0, 1, nullptr,
                            0, nullptr, nullptr, 2 + x_act, nullptr, nullptr, x_pre)))
        return rc;
    if (dbias && (rc = znn_add_bias_bwd(dY, nullptr, dbias, M, N))) return rc;
    if (dW && (rc = gemm_dispatch(ZNN_TRANS, ZNN_NO_TRANS, K, N, M, 1.0f, X, K, 0, dY, N, 0, 1.0f, dW, N, 0, 1))) return rc;
    return ZNN_OK;
}

int znn_sgemm_grouped(int trans_a, int trans_b, int M, int N, int K, float alpha, const float* A, int lda, long long stride_a,
                      const float* B, int ldb, long long stride_b, float beta, float* C, int ldc, long long stride_c, int batch,
                      const float* bias, long long stride_bias, int kcat)
{
    ZNN_REQUIRE(batch >= 1 && batch <= 64, "batch must be 1..64");
    ZNN_REQUIRE(stride_a >= 0 && stride_b >= 0 && stride_c >= 0 && stride_bias >= 0, "negative stride");
    ZNN_REQUIRE(kcat == 0 || kcat == 1, "kcat is 0 or 1");
    if (!(2.0 * M * N * (double)K * batch >= 1.3e8 && M >= 64 && N >= 32 && K >= 32))
        return fail(ZNN_ERR_UNSUPPORTED, "grouped product: too small for the tensor-core path");
    if (kcat == 0 && batch > 1 && stride_c < (long long)M * ldc && stride_c != 0)
        return fail(ZNN_ERR_INVALID, "grouped product: the slices of C overlap");
    if (kcat == 0 && batch > 1 && stride_c == 0) return fail(ZNN_ERR_INVALID, "grouped product: every slice needs its own C");
    return gemm_dispatch(trans_a, trans_b, M, N, K, alpha, A, lda, stride_a, B, ldb, stride_b, beta, C, ldc, stride_c, batch, bias, 0,
                         nullptr, nullptr, 0, nullptr, nullptr, nullptr, stride_bias, kcat, true);
}

int znn_gemm_set_path(int path)
{
    ZNN_REQUIRE(path >= 0 && path <= 4, "path must be 0..4");
    t_path = path;
    return ZNN_OK;
}

int znn_gemm_last_path(void) { return t_last_path; }

int znn_gemm_set_skinny(int enable)
{
    t_skinny = (enable != 0);
    return ZNN_OK;
}

int znn_gemm_set_chunk(int k_elements)
{
    ZNN_REQUIRE(k_elements >= 32 && k_elements % 32 == 0, "chunk must be a positive multiple of 32");
    tc_set_chunk_kblocks(k_elements / 32);
    return ZNN_OK;
}

int znn_gemm_set_splitk(int enable)
{
    tc_set_splitk(enable);
    return ZNN_OK;
}

int znn_gemm_wait_record(int* out16)
{
    ZNN_REQUIRE(out16, "out16 is NULL");
    return tc_wait_record(out16);
}

int znn_gemm_set_persistent(int enable)
{
    tc_set_persistent(enable);
    return ZNN_OK;
}

int znn_gemm_set_tail_split(int enable)
{
    tc_set_tail_split(enable);
    return ZNN_OK;
}

int znn_gemm_set_conv_mode(int mode)
{
    ZNN_REQUIRE(mode == 0 || mode == 1, "mode must be 0 or 1");
    tc_set_conv_mode(mode);
    return ZNN_OK;
}

int znn_debug_set_wait_limit(unsigned long long sm_cycles)
{
    tc_set_wait_limit(sm_cycles);
    return ZNN_OK;
}

int znn_debug_wait_probe(unsigned long long limit_cycles) { return tc_wait_probe(limit_cycles); }

int znn_gemm_profile(int enable) { return tc_profile_enable(enable); }

int znn_gemm_profile_read(double* kernel_ms, long long* launches, double* flops)
{
    return tc_profile_read(kernel_ms, launches, flops);
}

}  // extern "C"
