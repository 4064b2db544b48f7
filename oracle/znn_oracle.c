/*
 * znn_oracle.c -- CPU restatement of the znn hot path (see znn_oracle.h).
 * TEST INFRASTRUCTURE ONLY: the checker, never the product.
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -shared -fPIC (see Makefile).
 */
#include "znn_oracle.h"
#include <math.h>
#include <string.h>

static zo_sgemm_fn g_bound_sgemm = 0;

void zo_bind_sgemm(zo_sgemm_fn fn) { g_bound_sgemm = fn; }

/* src/cblas.zig:37-96 */
void zo_sgemm_naive(int order, int ta, int tb, int M, int N, int K, float alpha,
                    const float *A, int lda, const float *B, int ldb,
                    float beta, float *C, int ldc)
{
    (void)order; /* the reference asserts row-major (cblas.zig:53) */
    size_t m = (size_t)M, n = (size_t)N, k = (size_t)K;
    size_t lda_u = (size_t)lda, ldb_u = (size_t)ldb, ldc_u = (size_t)ldc;
    if (beta == 0.0f) {
        for (size_t i = 0; i < m; i++) memset(C + i * ldc_u, 0, n * sizeof(float));
    } else if (beta != 1.0f) {
        for (size_t i = 0; i < m; i++)
            for (size_t j = 0; j < n; j++) C[i * ldc_u + j] *= beta;
    }
    if (alpha == 0.0f) return;
    const int tA = (ta == ZO_TRANS), tB = (tb == ZO_TRANS);
    for (size_t i = 0; i < m; i++) {
        for (size_t p = 0; p < k; p++) {
            const float a_val = alpha * (tA ? A[p * lda_u + i] : A[i * lda_u + p]);
            if (a_val == 0.0f) continue;
            float *c_row = C + i * ldc_u;
            if (tB) {
                for (size_t j = 0; j < n; j++) c_row[j] += a_val * B[j * ldb_u + p];
            } else {
                const float *b_row = B + p * ldb_u;
                for (size_t j = 0; j < n; j++) c_row[j] += a_val * b_row[j];
            }
        }
    }
}

void zo_sgemm_f64(int ta, int tb, int M, int N, int K, const float *A, int lda,
                  const float *B, int ldb, double *C, int ldc)
{
    const int tA = (ta == ZO_TRANS), tB = (tb == ZO_TRANS);
    for (size_t i = 0; i < (size_t)M; i++) {
        double *c_row = C + i * (size_t)ldc;
        for (size_t j = 0; j < (size_t)N; j++) c_row[j] = 0.0;
        for (size_t p = 0; p < (size_t)K; p++) {
            const double a = tA ? A[p * (size_t)lda + i] : A[i * (size_t)lda + p];
            if (tB) {
                for (size_t j = 0; j < (size_t)N; j++) c_row[j] += a * (double)B[j * (size_t)ldb + p];
            } else {
                const float *b_row = B + p * (size_t)ldb;
                for (size_t j = 0; j < (size_t)N; j++) c_row[j] += a * (double)b_row[j];
            }
        }
    }
}

void zo_sgemm(int order, int ta, int tb, int M, int N, int K, float alpha,
              const float *A, int lda, const float *B, int ldb, float beta,
              float *C, int ldc)
{
    if (g_bound_sgemm) g_bound_sgemm(order, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
    else zo_sgemm_naive(order, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

/* src/autodiff.zig:110-133 */
void zo_matmul_fwd(const float *A, const float *B, float *C, int M, int K, int N)
{
    zo_sgemm(ZO_ROW_MAJOR, ZO_NO_TRANS, ZO_NO_TRANS, M, N, K, 1.0f, A, K, B, N, 0.0f, C, N);
}

/* src/autodiff.zig:593-641 */
void zo_matmul_bwd(const float *A, const float *B, const float *dC, float *dA,
                   float *dB, int M, int K, int N)
{
    if (dA) zo_sgemm(ZO_ROW_MAJOR, ZO_NO_TRANS, ZO_TRANS, M, K, N, 1.0f, dC, N, B, N, 1.0f, dA, K);
    if (dB) zo_sgemm(ZO_ROW_MAJOR, ZO_TRANS, ZO_NO_TRANS, K, N, M, 1.0f, A, K, dC, N, 1.0f, dB, N);
}

/* src/autodiff.zig:485-531 */
void zo_batch_matmul_fwd(const float *A, const float *B, float *C, int nb, int M, int K, int N)
{
    for (size_t s = 0; s < (size_t)nb; s++)
        zo_sgemm(ZO_ROW_MAJOR, ZO_NO_TRANS, ZO_NO_TRANS, M, N, K, 1.0f,
                 A + s * (size_t)M * K, K, B + s * (size_t)K * N, N, 0.0f,
                 C + s * (size_t)M * N, N);
}

/* src/autodiff.zig:1117-1182 */
void zo_batch_matmul_bwd(const float *A, const float *B, const float *dC,
                         float *dA, float *dB, int nb, int M, int K, int N)
{
    for (size_t s = 0; s < (size_t)nb; s++) {
        const float *a = A + s * (size_t)M * K, *b = B + s * (size_t)K * N;
        const float *dc = dC + s * (size_t)M * N;
        if (dA) zo_sgemm(ZO_ROW_MAJOR, ZO_NO_TRANS, ZO_TRANS, M, K, N, 1.0f, dc, N, b, N, 1.0f, dA + s * (size_t)M * K, K);
        if (dB) zo_sgemm(ZO_ROW_MAJOR, ZO_TRANS, ZO_NO_TRANS, K, N, M, 1.0f, a, K, dc, N, 1.0f, dB + s * (size_t)K * N, N);
    }
}

/* src/autodiff.zig:134-147 */
void zo_add_bias_fwd(const float *A, const float *bias, float *C, int M, int N)
{
    for (size_t i = 0; i < (size_t)M; i++)
        for (size_t j = 0; j < (size_t)N; j++) C[i * N + j] = A[i * N + j] + bias[j];
}

/* src/autodiff.zig:652-672: column-major walk, bias sum sequential in m */
void zo_add_bias_bwd(const float *dC, float *dA, float *dbias, int M, int N)
{
    for (size_t n = 0; n < (size_t)N; n++) {
        float bias_sum = 0.0f;
        for (size_t m = 0; m < (size_t)M; m++) {
            const float g = dC[m * N + n];
            if (dA) dA[m * N + n] += g;
            bias_sum += g;
        }
        if (dbias) dbias[n] += bias_sum;
    }
}

/* src/autodiff.zig:148-154 */
void zo_relu_fwd(const float *A, float *C, size_t n)
{
    for (size_t i = 0; i < n; i++) C[i] = (A[i] > 0.0f) ? A[i] : 0.0f;
}

/* src/autodiff.zig:681-691 */
void zo_relu_bwd(const float *A, const float *dC, float *dA, size_t n)
{
    for (size_t i = 0; i < n; i++) dA[i] += (A[i] > 0.0f) ? dC[i] : 0.0f;
}

/* src/autodiff.zig:156-165 */
void zo_gelu_fwd(const float *A, float *C, size_t n)
{
    const float sqrt_2 = sqrtf(2.0f);
    for (size_t i = 0; i < n; i++) {
        const float e = erff(A[i] / sqrt_2);
        C[i] = 0.5f * A[i] * (1.0f + e);
    }
}

/* src/autodiff.zig:699-716 */
void zo_gelu_bwd(const float *A, const float *dC, float *dA, size_t n)
{
    const float sqrt_2 = sqrtf(2.0f);
    const float inv_sqrt_2pi = 1.0f / sqrtf((float)(2.0 * 3.14159265358979323846));
    for (size_t i = 0; i < n; i++) {
        const float x = A[i];
        const float e = erff(x / sqrt_2);
        const float cdf = 0.5f * (1.0f + e);
        const float pdf = inv_sqrt_2pi * expf(-0.5f * x * x);
        const float deriv = cdf + x * pdf;
        dA[i] += dC[i] * deriv;
    }
}

/* src/autodiff.zig:196-238 */
void zo_softmax_xent_fwd(const float *logits, const int32_t *targets,
                         float *probs, float *loss, int M, int N)
{
    float loss_sum = 0.0f;
    for (size_t i = 0; i < (size_t)M; i++) {
        const float *row = logits + i * N;
        float *p = probs + i * N;
        float max_val = row[0];
        for (int j = 0; j < N; j++) if (row[j] > max_val) max_val = row[j];
        float sum = 0.0f;
        for (int j = 0; j < N; j++) {
            const float e = expf(row[j] - max_val);
            p[j] = e;
            sum += e;
        }
        for (int j = 0; j < N; j++) p[j] /= sum;
        const float prob = p[targets[i]];
        const float clipped = (prob > 1e-15f) ? prob : 1e-15f;
        loss_sum += -logf(clipped);
    }
    loss[0] = loss_sum / (float)M;
}

/* src/autodiff.zig:758-774 (ignores the upstream loss gradient) */
void zo_softmax_xent_bwd(const float *probs, const int32_t *targets,
                         float *dlogits, int M, int N)
{
    const float scale = 1.0f / (float)M;
    for (size_t i = 0; i < (size_t)M; i++) {
        const int32_t label = targets[i];
        for (int j = 0; j < N; j++)
            dlogits[i * N + j] += scale * (probs[i * N + j] - ((j == label) ? 1.0f : 0.0f));
    }
}

/* src/autodiff.zig:435-461 */
void zo_softmax_fwd(const float *A, float *C, size_t M, int D)
{
    for (size_t i = 0; i < M; i++) {
        const float *in = A + i * D;
        float *out = C + i * D;
        float max_val = in[0];
        for (int j = 1; j < D; j++) if (in[j] > max_val) max_val = in[j];
        float sum = 0.0f;
        for (int j = 0; j < D; j++) {
            const float e = expf(in[j] - max_val);
            out[j] = e;
            sum += e;
        }
        for (int j = 0; j < D; j++) out[j] /= sum;
    }
}

/* src/autodiff.zig:1054-1076 */
void zo_softmax_bwd(const float *Y, const float *dY, float *dA, size_t M, int D)
{
    for (size_t i = 0; i < M; i++) {
        const float *y = Y + i * D, *dy = dY + i * D;
        float *da = dA + i * D;
        float sum_dy_y = 0.0f;
        for (int j = 0; j < D; j++) sum_dy_y += dy[j] * y[j];
        for (int j = 0; j < D; j++) da[j] += y[j] * (dy[j] - sum_dy_y);
    }
}

/* src/nn.zig:835-886: mulScalar, + mask(-1e9 above the diagonal), softmax */
void zo_causal_softmax_fwd(const float *S, float scale, float *P, int nslices, int T)
{
    for (size_t s = 0; s < (size_t)nslices; s++) {
        for (int i = 0; i < T; i++) {
            const float *in = S + (s * T + i) * (size_t)T;
            float *out = P + (s * T + i) * (size_t)T;
            /* att_scaled = att*scale ; att_masked = att_scaled + mask */
            for (int j = 0; j < T; j++) {
                const float scaled = in[j] * scale;
                const float mask = (j > i) ? -1e9f : 0.0f;
                out[j] = scaled + mask;
            }
            float max_val = out[0];
            for (int j = 1; j < T; j++) if (out[j] > max_val) max_val = out[j];
            float sum = 0.0f;
            for (int j = 0; j < T; j++) {
                const float e = expf(out[j] - max_val);
                out[j] = e;
                sum += e;
            }
            for (int j = 0; j < T; j++) out[j] /= sum;
        }
    }
}

void zo_causal_softmax_bwd(const float *P, const float *dP, float scale,
                           float *dS, int nslices, int T)
{
    const size_t rows = (size_t)nslices * T;
    for (size_t r = 0; r < rows; r++) {
        const float *y = P + r * T, *dy = dP + r * T;
        float *ds = dS + r * T;
        float sum_dy_y = 0.0f;
        for (int j = 0; j < T; j++) sum_dy_y += dy[j] * y[j];
        for (int j = 0; j < T; j++) {
            /* softmax bwd into a zeroed grad, Add bwd copies it on, MulScalar
             * bwd multiplies by the scalar and accumulates */
            const float g = 0.0f + y[j] * (dy[j] - sum_dy_y);
            ds[j] += g * scale;
        }
    }
}

/* src/autodiff.zig:462-484 */
void zo_rmsnorm_fwd(const float *X, const float *G, float eps, float *Y, size_t M, int D)
{
    for (size_t i = 0; i < M; i++) {
        const float *x = X + i * D;
        float *y = Y + i * D;
        float sum_x2 = 0.0f;
        for (int j = 0; j < D; j++) sum_x2 += x[j] * x[j];
        const float rms = sqrtf(sum_x2 / (float)D + eps);
        for (int j = 0; j < D; j++) y[j] = x[j] / rms * G[j];
    }
}

/* src/autodiff.zig:1077-1116 */
void zo_rmsnorm_bwd(const float *X, const float *G, const float *dY, float eps,
                    float *dX, float *dG, size_t M, int D)
{
    for (size_t i = 0; i < M; i++) {
        const float *x = X + i * D, *dy = dY + i * D;
        float sum_x2 = 0.0f;
        for (int j = 0; j < D; j++) sum_x2 += x[j] * x[j];
        const float scale = 1.0f / sqrtf(sum_x2 / (float)D + eps);
        if (dG) for (int j = 0; j < D; j++) dG[j] += dy[j] * x[j] * scale;
        if (dX) {
            float *dx = dX + i * D;
            float sum_dy_g_x = 0.0f;
            for (int j = 0; j < D; j++) sum_dy_g_x += dy[j] * G[j] * x[j];
            for (int j = 0; j < D; j++) {
                const float term1 = G[j] * dy[j];
                const float term2 = x[j] * scale * scale * sum_dy_g_x / (float)D;
                dx[j] += scale * (term1 - term2);
            }
        }
    }
}

/* Extension with no reference counterpart. */
void zo_layernorm_fwd(const float *X, const float *G, const float *Bt, float eps,
                      float *Y, size_t M, int D)
{
    for (size_t i = 0; i < M; i++) {
        const float *x = X + i * D;
        float *y = Y + i * D;
        float sum = 0.0f;
        for (int j = 0; j < D; j++) sum += x[j];
        const float mean = sum / (float)D;
        float var = 0.0f;
        for (int j = 0; j < D; j++) { const float d = x[j] - mean; var += d * d; }
        const float rstd = 1.0f / sqrtf(var / (float)D + eps);
        for (int j = 0; j < D; j++) y[j] = (x[j] - mean) * rstd * G[j] + Bt[j];
    }
}

void zo_layernorm_bwd(const float *X, const float *G, const float *dY, float eps,
                      float *dX, float *dG, float *dB, size_t M, int D)
{
    for (size_t i = 0; i < M; i++) {
        const float *x = X + i * D, *dy = dY + i * D;
        float sum = 0.0f;
        for (int j = 0; j < D; j++) sum += x[j];
        const float mean = sum / (float)D;
        float var = 0.0f;
        for (int j = 0; j < D; j++) { const float d = x[j] - mean; var += d * d; }
        const float rstd = 1.0f / sqrtf(var / (float)D + eps);
        float s1 = 0.0f, s2 = 0.0f;
        for (int j = 0; j < D; j++) {
            const float xh = (x[j] - mean) * rstd;
            const float gdy = G[j] * dy[j];
            s1 += gdy;
            s2 += gdy * xh;
            if (dG) dG[j] += dy[j] * xh;
            if (dB) dB[j] += dy[j];
        }
        if (dX) {
            float *dx = dX + i * D;
            for (int j = 0; j < D; j++) {
                const float xh = (x[j] - mean) * rstd;
                dx[j] += rstd * (G[j] * dy[j] - s1 / (float)D - xh * s2 / (float)D);
            }
        }
    }
}

/* src/tensor.zig:523-585 / src/autodiff.zig:339-388; pad is an extension:
 * out-of-range taps contribute x=0 (they are skipped, which adds nothing). */
void zo_conv2d_fwd(const float *X, const float *W, const float *bias, float *Y,
                   int N, int Ci, int H, int Wd, int Co, int KH, int KW, int pad)
{
    const int Ho = H + 2 * pad - KH + 1, Wo = Wd + 2 * pad - KW + 1;
    for (int n = 0; n < N; n++)
        for (int co = 0; co < Co; co++) {
            const float b_val = bias ? bias[co] : 0.0f;
            for (int h = 0; h < Ho; h++)
                for (int w = 0; w < Wo; w++) {
                    float sum = b_val;
                    for (int ci = 0; ci < Ci; ci++)
                        for (int kh = 0; kh < KH; kh++)
                            for (int kw = 0; kw < KW; kw++) {
                                const int ih = h + kh - pad, iw = w + kw - pad;
                                if (ih < 0 || ih >= H || iw < 0 || iw >= Wd) continue;
                                const float xv = X[(((size_t)n * Ci + ci) * H + ih) * Wd + iw];
                                const float wv = W[(((size_t)co * Ci + ci) * KH + kh) * KW + kw];
                                sum += xv * wv;
                            }
                    Y[(((size_t)n * Co + co) * Ho + h) * Wo + w] = sum;
                }
        }
}

/* src/autodiff.zig:929-995 */
void zo_conv2d_bwd(const float *X, const float *W, const float *dY, float *dX,
                   float *dW, float *dbias, int N, int Ci, int H, int Wd, int Co,
                   int KH, int KW, int pad)
{
    const int Ho = H + 2 * pad - KH + 1, Wo = Wd + 2 * pad - KW + 1;
    for (int n = 0; n < N; n++)
        for (int co = 0; co < Co; co++)
            for (int h = 0; h < Ho; h++)
                for (int w = 0; w < Wo; w++) {
                    const float g = dY[(((size_t)n * Co + co) * Ho + h) * Wo + w];
                    if (g == 0.0f) continue;
                    if (dbias) dbias[co] += g;
                    for (int ci = 0; ci < Ci; ci++)
                        for (int kh = 0; kh < KH; kh++)
                            for (int kw = 0; kw < KW; kw++) {
                                const int ih = h + kh - pad, iw = w + kw - pad;
                                if (ih < 0 || ih >= H || iw < 0 || iw >= Wd) continue;
                                const size_t xi = (((size_t)n * Ci + ci) * H + ih) * Wd + iw;
                                const size_t wi = (((size_t)co * Ci + ci) * KH + kh) * KW + kw;
                                if (dW) dW[wi] += g * X[xi];
                                if (dX) dX[xi] += g * W[wi];
                            }
                }
}

/* src/autodiff.zig:389-434 */
void zo_maxpool2d_fwd(const float *X, float *Y, int32_t *idx, int N, int C,
                      int H, int W, int pool, int stride)
{
    const int Ho = H / stride, Wo = W / stride;
    for (size_t nc = 0; nc < (size_t)N * C; nc++) {
        const float *x = X + nc * H * W;
        for (int h = 0; h < Ho; h++)
            for (int w = 0; w < Wo; w++) {
                float max_val = x[(h * stride) * W + (w * stride)];
                int max_i = (h * stride) * W + (w * stride);
                for (int ph = 0; ph < pool; ph++)
                    for (int pw = 0; pw < pool; pw++) {
                        const int ih = h * stride + ph, iw = w * stride + pw;
                        if (ih < H && iw < W) {
                            const float v = x[ih * W + iw];
                            if (v > max_val) { max_val = v; max_i = ih * W + iw; }
                        }
                    }
                Y[nc * Ho * Wo + h * Wo + w] = max_val;
                if (idx) idx[nc * Ho * Wo + h * Wo + w] = max_i;
            }
    }
}

/* src/autodiff.zig:996-1053: recomputes the argmax, skips zero gradients */
void zo_maxpool2d_bwd(const float *X, const float *dY, float *dX, int N, int C,
                      int H, int W, int pool, int stride)
{
    const int Ho = H / stride, Wo = W / stride;
    for (size_t nc = 0; nc < (size_t)N * C; nc++) {
        const float *x = X + nc * H * W;
        for (int h = 0; h < Ho; h++)
            for (int w = 0; w < Wo; w++) {
                const float g = dY[nc * Ho * Wo + h * Wo + w];
                if (g == 0.0f) continue;
                float max_val = x[(h * stride) * W + (w * stride)];
                int max_i = (h * stride) * W + (w * stride);
                for (int ph = 0; ph < pool; ph++)
                    for (int pw = 0; pw < pool; pw++) {
                        const int ih = h * stride + ph, iw = w * stride + pw;
                        if (ih < H && iw < W) {
                            const float v = x[ih * W + iw];
                            if (v > max_val) { max_val = v; max_i = ih * W + iw; }
                        }
                    }
                dX[nc * H * W + max_i] += g;
            }
    }
}

/* src/autodiff.zig:532-553 */
void zo_embedding_fwd(const float *W, const float *ids, float *Y, size_t n, int D)
{
    for (size_t i = 0; i < n; i++) {
        const size_t idx = (size_t)ids[i];
        memcpy(Y + i * D, W + idx * D, (size_t)D * sizeof(float));
    }
}

/* src/autodiff.zig:1183-1207: sequential scatter-add in (b,t) order */
void zo_embedding_bwd(const float *ids, const float *dY, float *dW, size_t n, int D)
{
    for (size_t i = 0; i < n; i++) {
        const size_t idx = (size_t)ids[i];
        for (int j = 0; j < D; j++) dW[idx * D + j] += dY[i * D + j];
    }
}

static void zo_transposed_strides(const int64_t *dims, int rank, int d0, int d1,
                                  int64_t *out_dims, int64_t *src_strides)
{
    int64_t strides[8];
    int64_t s = 1;
    for (int d = rank - 1; d >= 0; d--) { strides[d] = s; s *= dims[d]; }
    for (int d = 0; d < rank; d++) { out_dims[d] = dims[d]; src_strides[d] = strides[d]; }
    out_dims[d0] = dims[d1]; out_dims[d1] = dims[d0];
    src_strides[d0] = strides[d1]; src_strides[d1] = strides[d0];
}

/* src/autodiff.zig:276-302 */
void zo_transpose_fwd(const float *A, float *C, const int64_t *dims, int rank, int d0, int d1)
{
    int64_t od[8], ss[8], idx[8] = {0};
    zo_transposed_strides(dims, rank, d0, d1, od, ss);
    size_t total = 1;
    for (int d = 0; d < rank; d++) total *= (size_t)dims[d];
    for (size_t f = 0; f < total; f++) {
        int64_t src = 0;
        for (int d = 0; d < rank; d++) src += idx[d] * ss[d];
        C[f] = A[src];
        for (int d = rank; d > 0;) { d--; if (++idx[d] < od[d]) break; idx[d] = 0; }
    }
}

/* src/autodiff.zig:848-876 */
void zo_transpose_bwd(const float *dC, float *dA, const int64_t *dims, int rank, int d0, int d1)
{
    int64_t od[8], ss[8], idx[8] = {0};
    zo_transposed_strides(dims, rank, d0, d1, od, ss);
    size_t total = 1;
    for (int d = 0; d < rank; d++) total *= (size_t)dims[d];
    for (size_t f = 0; f < total; f++) {
        int64_t src = 0;
        for (int d = 0; d < rank; d++) src += idx[d] * ss[d];
        dA[src] += dC[f];
        for (int d = rank; d > 0;) { d--; if (++idx[d] < od[d]) break; idx[d] = 0; }
    }
}

/* src/autodiff.zig:331-338 */
void zo_add_fwd(const float *A, const float *B, float *C, size_t n)
{
    for (size_t i = 0; i < n; i++) C[i] = A[i] + B[i];
}

/* src/autodiff.zig:831-839, :914-928: grad pass-through accumulate */
void zo_accumulate(const float *src, float *dst, size_t n)
{
    for (size_t i = 0; i < n; i++) dst[i] += src[i];
}

/* src/autodiff.zig:315-322 */
void zo_mul_scalar_fwd(const float *A, float v, float *C, size_t n)
{
    for (size_t i = 0; i < n; i++) C[i] = A[i] * v;
}

/* src/autodiff.zig:895-904 */
void zo_mul_scalar_bwd(const float *dC, float v, float *dA, size_t n)
{
    for (size_t i = 0; i < n; i++) dA[i] += dC[i] * v;
}

/* src/tensor.zig:813-851 */
void zo_argmax(const float *A, float *out, int M, int N, int dim)
{
    if (dim == 1) {
        for (int i = 0; i < M; i++) {
            float mv = A[(size_t)i * N];
            int mi = 0;
            for (int j = 1; j < N; j++) {
                const float v = A[(size_t)i * N + j];
                if (v > mv) { mv = v; mi = j; }
            }
            out[i] = (float)mi;
        }
    } else {
        for (int j = 0; j < N; j++) {
            float mv = A[j];
            int mi = 0;
            for (int i = 1; i < M; i++) {
                const float v = A[(size_t)i * N + j];
                if (v > mv) { mv = v; mi = i; }
            }
            out[j] = (float)mi;
        }
    }
}

/* src/optim.zig:133-151 (AdamOptimizer.step): t is the step count AFTER the increment; lr_t as the reference computes it */
void zo_adam_step(float *w, const float *g, float *m, float *v, float lr, float beta1, float beta2, float eps, float t,
                  size_t n)
{
    const float correction1 = 1.0f - powf(beta1, t);
    const float correction2 = 1.0f - powf(beta2, t);
    const float lr_t = lr * sqrtf(correction2) / correction1;
    for (size_t i = 0; i < n; i++) {
        m[i] = beta1 * m[i] + (1.0f - beta1) * g[i];
        v[i] = beta2 * v[i] + (1.0f - beta2) * g[i] * g[i];
        w[i] -= lr_t * m[i] / (sqrtf(v[i]) + eps);
    }
}

/* src/optim.zig:50-66 */
void zo_sgd_step(float *w, const float *g, float *v, float lr, float momentum, size_t n)
{
    if (v) {
        for (size_t i = 0; i < n; i++) {
            v[i] = momentum * v[i] + lr * g[i];
            w[i] -= v[i];
        }
    } else {
        for (size_t i = 0; i < n; i++) w[i] -= lr * g[i];
    }
}
