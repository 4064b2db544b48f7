/*
 * znn_oracle.h -- CPU restatement of the znn dense-contraction hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is the checker the CUDA path is compared
 * against; nothing shipped may call it.  Each function restates one loop of
 * the reference (chen-gz/znn) in plain C11 with the same iteration order and
 * the same fp32 rounding points (build with -ffp-contract=off).  Citations are
 * to the reference's files by their path inside that project.
 *
 * Parity pin: the reference is Zig 0.16 and cannot be built where this code is
 * developed, so the oracle is pinned against the known-answer constants that
 * the reference's own inline tests assert (tests/golden/ref_kats.json holds
 * them, transcribed from the test blocks cited there).  Ops with no
 * value-pinning reference test (SoftmaxCrossEntropy values and gradient, the
 * causal mask path, multi-channel conv, pooling ties) are "parity unpinned":
 * for them this restatement is the only authority.
 *
 * All tensors are contiguous row-major fp32.
 */
#ifndef ZNN_ORACLE_H
#define ZNN_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define ZO_ROW_MAJOR 101
#define ZO_NO_TRANS 111
#define ZO_TRANS 112

typedef void (*zo_sgemm_fn)(int order, int ta, int tb, int M, int N, int K,
                            float alpha, const float *A, int lda,
                            const float *B, int ldb, float beta, float *C,
                            int ldc);

/* src/cblas.zig:37-96 (cblas_sgemm_fallback): beta pass, then i-p-j loops with
 * the a_val==0 skip, product rounded to fp32 before the add. */
void zo_sgemm_naive(int order, int ta, int tb, int M, int N, int K, float alpha,
                    const float *A, int lda, const float *B, int ldb,
                    float beta, float *C, int ldc);
/* Same contraction accumulated in fp64 and written as fp64: the arbiter used
 * to classify near-ties and to report error against exact arithmetic. */
void zo_sgemm_f64(int ta, int tb, int M, int N, int K, const float *A, int lda,
                  const float *B, int ldb, double *C, int ldc);
/* src/cblas.zig:11-14 chooses between an external cblas_sgemm (Apple) and the
 * fallback.  zo_bind_sgemm(fn) plays that switch: NULL = fallback (Linux
 * behaviour), otherwise every matmul below goes to fn (a host CBLAS). */
void zo_bind_sgemm(zo_sgemm_fn fn);
void zo_sgemm(int order, int ta, int tb, int M, int N, int K, float alpha,
              const float *A, int lda, const float *B, int ldb, float beta,
              float *C, int ldc);

/* MatMul: src/autodiff.zig:110-133 (fwd), :593-641 (bwd; dA/dB may be NULL =
 * requires_grad false; both accumulate). */
void zo_matmul_fwd(const float *A, const float *B, float *C, int M, int K, int N);
void zo_matmul_bwd(const float *A, const float *B, const float *dC, float *dA,
                   float *dB, int M, int K, int N);
/* BatchMatMul: src/autodiff.zig:485-531, :1117-1182.  nb = batch*heads
 * contiguous slices. */
void zo_batch_matmul_fwd(const float *A, const float *B, float *C, int nb, int M, int K, int N);
void zo_batch_matmul_bwd(const float *A, const float *B, const float *dC,
                         float *dA, float *dB, int nb, int M, int K, int N);
/* AddBias: src/autodiff.zig:134-147, :652-672 */
void zo_add_bias_fwd(const float *A, const float *bias, float *C, int M, int N);
void zo_add_bias_bwd(const float *dC, float *dA, float *dbias, int M, int N);
/* Relu: src/autodiff.zig:148-154, :681-691 */
void zo_relu_fwd(const float *A, float *C, size_t n);
void zo_relu_bwd(const float *A, const float *dC, float *dA, size_t n);
/* Gelu: src/autodiff.zig:156-165, :699-716 */
void zo_gelu_fwd(const float *A, float *C, size_t n);
void zo_gelu_bwd(const float *A, const float *dC, float *dA, size_t n);
/* SoftmaxCrossEntropy: src/autodiff.zig:196-238 (fwd), :758-774 (bwd).
 * Targets are int32 here (the reference carries u8). */
void zo_softmax_xent_fwd(const float *logits, const int32_t *targets,
                         float *probs, float *loss, int M, int N);
void zo_softmax_xent_bwd(const float *probs, const int32_t *targets,
                         float *dlogits, int M, int N);
/* Softmax over the last dim: src/autodiff.zig:435-461, :1054-1076 */
void zo_softmax_fwd(const float *A, float *C, size_t M, int D);
void zo_softmax_bwd(const float *Y, const float *dY, float *dA, size_t M, int D);
/* The attention score path of src/nn.zig:835-886 as the reference runs it:
 * mulScalar (autodiff.zig:315-322), add of the -1e9 mask (nn.zig:847-866,
 * autodiff.zig:331-338), softmax.  rows = B*nh*T rows of length T. */
void zo_causal_softmax_fwd(const float *S, float scale, float *P, int nslices, int T);
/* backward through softmax, add and mulScalar (autodiff.zig:1054-1076,
 * :914-928, :895-904): dS += scale * P*(dP - sum(dP*P)) */
void zo_causal_softmax_bwd(const float *P, const float *dP, float scale,
                           float *dS, int nslices, int T);
/* RmsNorm: src/autodiff.zig:462-484, :1077-1116 (dG/dX may be NULL) */
void zo_rmsnorm_fwd(const float *X, const float *G, float eps, float *Y, size_t M, int D);
void zo_rmsnorm_bwd(const float *X, const float *G, const float *dY, float eps,
                    float *dX, float *dG, size_t M, int D);
/* LayerNorm: NOT in the reference (extension asked for by the workload
 * definition).  Own definition: biased variance, eps inside the sqrt. */
void zo_layernorm_fwd(const float *X, const float *G, const float *Bt, float eps,
                      float *Y, size_t M, int D);
void zo_layernorm_bwd(const float *X, const float *G, const float *dY, float eps,
                      float *dX, float *dG, float *dB, size_t M, int D);
/* Conv2D: src/tensor.zig:523-585, src/autodiff.zig:339-388 (fwd), :929-995
 * (bwd).  pad is an extension (0 = reference). stride is 1. bias may be NULL. */
void zo_conv2d_fwd(const float *X, const float *W, const float *bias, float *Y,
                   int N, int Ci, int H, int Wd, int Co, int KH, int KW, int pad);
void zo_conv2d_bwd(const float *X, const float *W, const float *dY, float *dX,
                   float *dW, float *dbias, int N, int Ci, int H, int Wd, int Co,
                   int KH, int KW, int pad);
/* MaxPool2D: src/autodiff.zig:389-434, :996-1053.  idx (optional) receives the
 * flat input offset (within the n,c plane) of the first maximum. */
void zo_maxpool2d_fwd(const float *X, float *Y, int32_t *idx, int N, int C,
                      int H, int W, int pool, int stride);
void zo_maxpool2d_bwd(const float *X, const float *dY, float *dX, int N, int C,
                      int H, int W, int pool, int stride);
/* Embedding: src/autodiff.zig:532-553, :1183-1207 (ids are fp32) */
void zo_embedding_fwd(const float *W, const float *ids, float *Y, size_t n, int D);
void zo_embedding_bwd(const float *ids, const float *dY, float *dW, size_t n, int D);
/* Transpose: src/autodiff.zig:276-302, :848-876 (odometer over <=8 dims) */
void zo_transpose_fwd(const float *A, float *C, const int64_t *dims, int rank, int d0, int d1);
void zo_transpose_bwd(const float *dC, float *dA, const int64_t *dims, int rank, int d0, int d1);
/* Add / MulScalar / Reshape-bwd: src/autodiff.zig:315-338, :831-839, :895-928 */
void zo_add_fwd(const float *A, const float *B, float *C, size_t n);
void zo_accumulate(const float *src, float *dst, size_t n);
void zo_mul_scalar_fwd(const float *A, float v, float *C, size_t n);
void zo_mul_scalar_bwd(const float *dC, float v, float *dA, size_t n);
/* argmax: src/tensor.zig:813-851 (first maximum wins, result as fp32) */
void zo_argmax(const float *A, float *out, int M, int N, int dim);
/* SGD: src/optim.zig:50-66 (v may be NULL when momentum == 0) */
void zo_sgd_step(float *w, const float *g, float *v, float lr, float momentum, size_t n);
void zo_adam_step(float *w, const float *g, float *m, float *v, float lr, float beta1, float beta2, float eps, float t,
                  size_t n);

#ifdef __cplusplus
}
#endif
#endif
