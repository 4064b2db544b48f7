/*
 * znn_cuda.h -- C ABI of libznn_cuda.so: the B200 (sm_100a) implementation of
 * the dense-contraction hot path of chen-gz/znn.
 *
 * Every entry point is what the reference's host code would bind for one loop
 * of its hot path; the comment on each names the reference code it replaces
 * (paths are inside the reference project).  Conventions:
 *   - all tensor pointers are DEVICE pointers to contiguous row-major fp32
 *     unless a comment says otherwise; the caller owns every buffer;
 *   - every call returns 0 on success or a negative ZNN_ERR_* code, never
 *     aborts; znn_last_error() gives the text for the calling host thread;
 *   - calls enqueue work on the calling thread's stream (znn_set_stream) and
 *     return without waiting; znn_sync() waits;
 *   - "accumulate" arguments follow the reference's backward arms, which add
 *     into the input gradients (+=): a NULL gradient pointer means the input
 *     has requires_grad == false and that arm is skipped.
 * There is no CPU fallback: without a CUDA device every compute call fails.
 */
#ifndef ZNN_CUDA_H
#define ZNN_CUDA_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define ZNN_OK 0
#define ZNN_ERR_INVALID (-1)  /* bad argument */
#define ZNN_ERR_CUDA (-2)     /* a CUDA runtime/driver call failed */
#define ZNN_ERR_NOMEM (-3)
#define ZNN_ERR_DEVICE_WAIT (-4) /* a bounded device-side wait expired */
#define ZNN_ERR_NCCL (-5)
#define ZNN_ERR_UNSUPPORTED (-6)

/* bits of the device status word (znn_device_status) */
#define ZNN_DEV_TMA_WAIT_EXPIRED 1
#define ZNN_DEV_MMA_WAIT_EXPIRED 2
#define ZNN_DEV_EPI_WAIT_EXPIRED 4
#define ZNN_DEV_BAD_INDEX 8        /* a token id, class label or sample index was outside its range */

/* same constants as src/cblas.zig:5-8 */
#define ZNN_ROW_MAJOR 101
#define ZNN_COL_MAJOR 102
#define ZNN_NO_TRANS 111
#define ZNN_TRANS 112

/* ---- runtime (the reference allocates with Zig allocators: src/autodiff.zig:1301-1326,
 *      src/nn.zig:1352-1377; these are the device equivalents) ---- */
int znn_init(int device);                 /* select device, create per-device state */
/* Makes `device` the calling host thread's current device (cudaSetDevice) and creates its state on first use.  One host
 * thread may drive several devices by switching between calls; streams, scratch blocks, the status word and kernel
 * attributes are all kept per device. */
int znn_set_device(int device);
int znn_device_count(int* count);
int znn_set_stream(void* cuda_stream);    /* cudaStream_t to launch on (NULL = shim-owned stream) */
int znn_get_stream(void** cuda_stream);
int znn_sync(void);
int znn_malloc(void** ptr, size_t bytes);
int znn_free(void* ptr);
int znn_memset(void* ptr, int value, size_t bytes);
int znn_memcpy_h2d(void* dst, const void* src, size_t bytes);   /* async on the stream */
int znn_memcpy_d2h(void* dst, const void* src, size_t bytes);   /* waits for completion */
int znn_memcpy_d2h_async(void* dst, const void* src, size_t bytes); /* async on the stream (pinned dst); znn_sync() completes it */
int znn_memcpy_d2d(void* dst, const void* src, size_t bytes);
/* rows x width_bytes between pitched device arrays (async on the stream); used to append K/V rows to a decode cache */
int znn_memcpy2d_d2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows);
/* Per-step bump allocator over one device block: the analogue of Graph.arena (std.heap.ArenaAllocator,
 * src/autodiff.zig:1237-1258: every intermediate of a batch is freed at once by graph.deinit).  alloc returns
 * 256-byte aligned device memory or ZNN_ERR_NOMEM when the block is exhausted; reset makes everything reusable. */
typedef struct znn_arena znn_arena;
int znn_arena_create(size_t bytes, znn_arena** out);
int znn_arena_alloc(znn_arena* a, size_t bytes, void** ptr);
int znn_arena_reset(znn_arena* a);
int znn_arena_usage(znn_arena* a, size_t* used, size_t* high_water, size_t* capacity);
int znn_arena_destroy(znn_arena* a);
/* Persistent parameters (createPersistentTensor, src/nn.zig:1352-1369) as three contiguous device slabs -- values,
 * gradients, SGD velocities, all zero at creation -- holding n tensors of counts[i] floats in the caller's
 * collectParameters order (src/nn.zig:142-171), each starting 16-byte aligned.  One memset is model.zeroGrad()
 * (:121-140), one kernel the optimizer step (src/optim.zig:50-66), one call the data-parallel gradient sum. */
typedef struct znn_param_slab znn_param_slab;
int znn_param_slab_create(const size_t* counts, int n, znn_param_slab** out);
int znn_param_slab_total(znn_param_slab* s, size_t* total_floats);
int znn_param_slab_tensor(znn_param_slab* s, int i, float** value, float** grad, float** velocity, size_t* offset);
int znn_param_slab_zero_grad(znn_param_slab* s);
int znn_param_slab_sgd_step(znn_param_slab* s, float lr, float momentum, float grad_scale);
int znn_param_slab_allreduce_grads(znn_param_slab* s);   /* in-place sum over the data-parallel ranks */
int znn_param_slab_destroy(znn_param_slab* s);
int znn_last_error(char* buf, size_t buflen);
int znn_device_status(int* status, int clear); /* syncs, reads (and clears) the device status word */
int znn_gemm_workspace_reserve(size_t bytes);  /* pre-size the GEMM scratch (avoids cudaMalloc later) */
int znn_launch_count(long long* count, int reset); /* kernels launched by this host thread so far */
/* Scratch blocks are kept per (device, stream) and grow on demand; growing frees the old block after synchronising the
 * stream and is refused during stream capture.  The counter increases whenever a block of the current device moved:
 * whoever keeps raw scratch addresses alive across calls (a captured CUDA graph) compares it before reuse. */
int znn_workspace_generation(unsigned long long* generation);

/* ---- GEMM: replaces cblas_sgemm (src/cblas.zig:11-96; prototype :17-34) at its 8 call
 *      sites (src/tensor.zig:181,721; src/autodiff.zig:117,513,604,624,1143,1163).
 *      Row-major only, like the reference (cblas.zig:53).  Results carry fp32 accuracy:
 *      large shapes run 3xTF32 split-precision tcgen05 MMAs, small/ragged ones fp32 FMAs. */
int znn_sgemm(int order, int trans_a, int trans_b, int M, int N, int K, float alpha,
              const float* A, int lda, const float* B, int ldb, float beta, float* C, int ldc);
/* The per-(batch,head) sgemm loops of BatchMatMul (src/autodiff.zig:485-531, :1117-1182)
 * as one call; strides are in elements between consecutive slices. */
int znn_sgemm_batched_strided(int trans_a, int trans_b, int M, int N, int K, float alpha,
                              const float* A, int lda, long long stride_a,
                              const float* B, int ldb, long long stride_b, float beta,
                              float* C, int ldc, long long stride_c, int batch);
/* cblas_sgemm with HOST operands, the exact shape of the reference's binding (src/cblas.zig:17-34 is
 * called with host slices at all 8 call sites): A, B and C are host pointers; C is final in host memory
 * when the call returns.  The product is pipelined by row panels of C: panel i's rows of op(A) (and of C
 * when beta != 0) travel host->device while panel i-1 is multiplied and panel i-2's result travels
 * device->host.  Pinned (page-locked) host memory makes the copies asynchronous; pageable memory works
 * but serialises them.  panels: number of row panels, 0 = automatic (one per ~1024 rows, at most 16). */
int znn_sgemm_host(int order, int trans_a, int trans_b, int M, int N, int K, float alpha,
                   const float* A, int lda, const float* B, int ldb, float beta, float* C, int ldc, int panels);
/* The MatMul operator's forward and backward arms (src/autodiff.zig:107-133 and :593-641) over HOST
 * tensors in one pipelined call: C = A.B, dA (+)= dC.B^T, dB (+)= A^T.dC with A[M,K], B[K,N], dC[M,N],
 * all compact row-major host arrays.  Each operand crosses the link once; C and dA leave by row panels
 * while later operand rows still arrive, dB by column panels once dC is complete.  NULL outputs are
 * skipped (dC may be NULL when both gradients are).  accumulate = 1 adds to the gradients already in
 * dA/dB (the reference's +=, which costs their upload); 0 overwrites them (the same result after
 * zeroGrad).  panels as for znn_sgemm_host. */
int znn_matmul_host_fwd_bwd(const float* A, const float* B, const float* dC, float* C, float* dA, float* dB,
                            int M, int K, int N, int accumulate, int panels);
/* The same call with a hint about triangular structure, for the products around a causal softmax
 * (src/nn.zig:835-906: S = Q.K^T -> mask -> softmax -> P.V).  The hint never changes a value the caller may read:
 *   ZNN_TRI_C_LOWER  only the lower triangle of C (col <= row) will be read (S and dP feed the causal softmax, which
 *                    never reads above the diagonal): output tiles entirely above it are neither computed nor written;
 *   ZNN_TRI_A_LOWER  op(A)[m,k] is exactly 0 for k > m (P, dS as left operand): the contraction stops at the tile's last row;
 *   ZNN_TRI_A_UPPER  op(A)[m,k] is exactly 0 for k < m (P^T, dS^T as left operand): it starts at the tile's first row;
 *   ZNN_TRI_B_LOWER  op(B)[k,n] is exactly 0 for n > k (dS as right operand): it starts at the tile's first column.
 * Skipped terms are products with exact zeros, so results equal the unhinted call (for finite operands).  Only the
 * in-place tensor-core path uses the hint (whole 256-row / BN-column tiles); the other paths compute everything. */
#define ZNN_TRI_NONE 0
#define ZNN_TRI_C_LOWER 1
#define ZNN_TRI_A_LOWER 2
#define ZNN_TRI_A_UPPER 3
#define ZNN_TRI_B_LOWER 4
int znn_sgemm_batched_strided_tri(int trans_a, int trans_b, int M, int N, int K, float alpha,
                                  const float* A, int lda, long long stride_a,
                                  const float* B, int ldb, long long stride_b, float beta,
                                  float* C, int ldc, long long stride_c, int batch, int tri);
/* Backward of the attention probabilities fused into the product that feeds it (an addition; src/autodiff.zig:1117-1182
 * BatchMatMul backward dA followed by :1054-1076 Softmax backward and the mulScalar backward of src/nn.zig:836):
 *   dS[s] = scale * P[s] o (dO[s].V[s]^T - D[s][:, None]),   D[s][i] = sum_j dP[s][i,j] P[s][i,j] = dO[s][i,:].O[s][i,:]
 * for nslices slices of T x T scores, dO, V of T x hs; dP is never written.  Only tiles that touch the lower triangle
 * are computed and stored (P is zero above the diagonal, so dS is zero there inside those tiles; tiles entirely above
 * it are left untouched).  dS is overwritten.  Needs the in-place tensor-core path (16-byte aligned pointers, T and hs
 * multiples of 4); returns ZNN_ERR_UNSUPPORTED otherwise and the caller uses the separate ops. */
int znn_attn_dscores(const float* dO, const float* V, const float* P, const float* D, float scale, float* dS, int T, int hs,
                     int nslices);
/* Causal self-attention as one fused operation (an addition; it replaces the chain of src/nn.zig:796-906 --
 * transposeND x4, batchMatMul, mulScalar, mask, add, softmax, batchMatMul, transposeND -- whose operator arms are
 * src/autodiff.zig:485-531, :1054-1076, :1117-1182):
 *     O[b,h] = softmax_rows(scale * Q[b,h].K[b,h]^T + causal mask) . V[b,h]
 * The T x T score and probability matrices are never written to memory: a CTA pair holds 256 rows of one (batch, head)
 * slice, walks the 64-wide blocks of the other sequence dimension up to (or from) the diagonal, and keeps scores,
 * probabilities and partial outputs in tensor memory; all products are 3xTF32 tcgen05 MMAs with fp32 promotion per block.
 * Element (b, h, t, d) of Q, K, V, O, dO and the gradients lies at  b * stride_b + h * stride_h + t * ld + d  (floats):
 *   [B, T, nh, hs] as the projections produce it:   ld = nh * hs, stride_h = hs,     stride_b = T * nh * hs
 *   [B, nh, T, hs] as the reference's transposeND:   ld = hs,      stride_h = T * hs, stride_b = nh * T * hs
 * so neither the head split nor the merge needs a copy.  LSE ([B * nh, T] floats) receives, per row, the base-2
 * log-sum-exp of the scaled visible scores; the backward recomputes the probabilities from it.
 * znn_attn_bwd: dQ, dK, dV (any may be NULL = requires_grad false) from dO, by three launches of the same kernel
 * (dQ by query rows; dK and dV by key rows), deterministic (no atomics); accumulate = 1 adds into the gradients (the
 * reference's +=), 0 stores them.
 * Limits: hs = 32 or 64; T, ld and the strides multiples of 4; 16-byte aligned pointers; otherwise
 * ZNN_ERR_UNSUPPORTED and the caller runs the separate operators. */
int znn_attn_fwd(const float* Q, const float* K, const float* V, float* O, float* LSE, int B, int nh, int T, int hs,
                 long long ld, long long stride_h, long long stride_b, float scale);
int znn_attn_bwd(const float* Q, const float* K, const float* V, const float* O, const float* dO, const float* LSE, float* dQ,
                 float* dK, float* dV, int B, int nh, int T, int hs, long long ld, long long stride_h, long long stride_b,
                 float scale, int accumulate);
/* out[r] = sum_j A[r,j] * B[r,j] for `rows` rows of D floats (the D vector above from dO and O) */
int znn_rowdot(const float* A, const float* B, float* out, size_t rows, int D);
/* Fused form of Linear.forward = addBias(matmul(x, W), b) (src/nn.zig:44-51): Y[M,N] = X[M,K].W[K,N] + bias[N]
 * in one pass (the bias is added in the GEMM epilogue); an addition, the two separate ops remain.
 * Backward of the pair (src/autodiff.zig:593-641 and :652-672 chained): dX += dY.W^T, dW += X^T.dY,
 * dbias += column sums of dY; NULL gradient pointers are skipped. */
int znn_linear_fwd(const float* X, const float* W, const float* bias, float* Y, int M, int K, int N);
int znn_linear_bwd(const float* X, const float* W, const float* dY, float* dX, float* dW, float* dbias, int M, int K, int N);
/* Grouped products on the in-place tensor-core path (the three projections of CausalSelfAttention.forward share their
 * input: src/nn.zig:776-793), `batch` slices at uniform strides (in floats); a stride of 0 means one matrix shared by all slices.
 *   kcat = 0: C_s = alpha * op(A_s).op(B_s) + bias_s + beta * C_s for every slice (bias may be NULL; bias_s = bias + s*stride_bias).
 *   kcat = 1: ONE product whose contraction runs through the slices one after the other,
 *             C = alpha * sum_s op(A_s).op(B_s) + beta * C  (stride_c ignored, no bias, K a multiple of 32): the sum of the
 *             slices' data gradients in one launch instead of `batch` accumulating ones.
 * ZNN_ERR_UNSUPPORTED when the operands cannot be read in place (16-byte alignment) or the product is too small: the caller
 * then makes `batch` znn_sgemm calls. */
int znn_sgemm_grouped(int trans_a, int trans_b, int M, int N, int K, float alpha, const float* A, int lda, long long stride_a,
                      const float* B, int ldb, long long stride_b, float beta, float* C, int ldc, long long stride_c, int batch,
                      const float* bias, long long stride_bias, int kcat);
/* Linear with the next elementwise step folded into the GEMM epilogue (src/nn.zig:660-668: gelu(c_fc(x)); :996-1021:
 * x + c_proj(...)):  h = X.W + bias (+ residual);  Y = act(h),  act = 0 none, 1 ReLU, 2 GELU (erf form, autodiff.zig:156-165).
 * pre (may be NULL) receives h, which the activation's backward needs; residual (may be NULL) has Y's shape.
 * Values equal the separate ops to fp32 rounding of the same sum.  ZNN_ERR_UNSUPPORTED when the product is too small for
 * the tensor-core path or a pointer is not 16-byte aligned / N not a multiple of 4: the caller keeps the separate ops. */
int znn_linear_fwd_ex(const float* X, const float* W, const float* bias, float* Y, float* pre, const float* residual, int M,
                      int K, int N, int act);
/* Backward of Linear whose input X is act(x_pre) of the layer below: dX receives the gradient with respect to x_pre,
 * dX (+)= (dY.W^T) o act'(x_pre) (dx_fresh = 1 stores, 0 accumulates); dW, dbias as znn_linear_bwd.  x_act = 0: plain
 * znn_linear_bwd.  Same ZNN_ERR_UNSUPPORTED rule. */
int znn_linear_bwd_ex(const float* X, const float* W, const float* dY, float* dX, float* dW, float* dbias, int M, int K, int N,
                      const float* x_pre, int x_act, int dx_fresh);
/* path: 0 = automatic, 1 = fp32 FMA kernel, 2 = tcgen05 one CTA per tile over pre-split operand
 * planes, 3 = tcgen05 CTA pairs over pre-split planes, 4 = tcgen05 CTA pairs reading the operands
 * in place (hi/lo split in shared memory; needs 16-byte aligned bases and leading dimensions that
 * are multiples of 4, otherwise path 3 is taken) */
int znn_gemm_set_path(int path);
int znn_gemm_last_path(void);
/* Number of contraction elements the tensor-core paths accumulate inside tensor memory before
 * the partial sum is promoted to an fp32 register sum (multiple of 32; default 256).  The
 * tensor core's accumulator truncates, so longer chunks trade accuracy for fewer promotions. */
int znn_gemm_set_chunk(int k_elements);
/* Split-K (default on): when a product has too few output tiles to fill the GPU and a long
 * contraction (parameter gradients dW = X^T dY), K is cut into slices run by different CTAs and
 * the partial sums are added in a fixed order by a second kernel.  0 switches it off. */
int znn_gemm_set_splitk(int enable);
/* ---- row-wise operators: the arms of Op.forward (src/autodiff.zig:107-575) and
 *      Op.backward (:579-1231) ---- */
/* AddBias: src/autodiff.zig:134-147 / :652-672 */
int znn_add_bias_fwd(const float* A, const float* bias, float* C, int M, int N);
int znn_add_bias_bwd(const float* dC, float* dA, float* dbias, int M, int N);
/* Relu: :148-154 / :681-691 */
int znn_relu_fwd(const float* A, float* C, size_t n);
int znn_relu_bwd(const float* A, const float* dC, float* dA, size_t n);
/* Gelu (exact erf form): :156-165 / :699-716 */
int znn_gelu_fwd(const float* A, float* C, size_t n);
int znn_gelu_bwd(const float* A, const float* dC, float* dA, size_t n);
/* the same gradient STORED into dA (an addition: for a gradient buffer nothing has been added to yet, it saves the
 * zero fill and the read of the zeros) */
int znn_gelu_bwd_set(const float* A, const float* dC, float* dA, size_t n);
/* SoftmaxCrossEntropy: :196-238 / :758-774; probs is the M x N buffer the reference keeps in
 * OpContext; loss is one device float.  Targets are int32 (the reference's []const u8 cannot
 * hold a vocabulary above 255); the _u8 form takes the reference's type.  A target outside [0, N) is never used as
 * an index: that row's loss (and the mean) becomes NaN and ZNN_DEV_BAD_INDEX is set in the device status word; the
 * backward treats such a row as having no target column. */
int znn_softmax_xent_fwd(const float* logits, const int32_t* targets, float* probs, float* loss, int M, int N);
int znn_softmax_xent_fwd_u8(const float* logits, const uint8_t* targets, float* probs, float* loss, int M, int N);
int znn_softmax_xent_bwd(const float* probs, const int32_t* targets, float* dlogits, int M, int N);
int znn_softmax_xent_bwd_u8(const float* probs, const uint8_t* targets, float* dlogits, int M, int N);
/* No counterpart in the reference.  Same result as znn_softmax_xent_fwd for callers that must
 * not allocate (a service whose memory budget was fixed at start-up, or a latency-critical
 * thread that cannot afford cudaMalloc, which synchronises the whole device): the per-row losses go to a fixed 256 KiB device array inside
 * the library instead of the growable scratch block, so this call never reaches cudaMalloc,
 * cudaFree or any allocating routine.  Limits and rules:
 *   - M <= 65536 rows; larger M is rejected with ZNN_ERR_INVALID (N is not limited);
 *   - work is enqueued on cuda_stream (a cudaStream_t; NULL = the legacy default stream), the
 *     shim's own stream and state are not touched, znn_init is not required;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, which may load the module): make that first call before any
 *     stream capture starts;
 *   - all calls on a device share the one array and it keeps the last call's contents
 *     (rows < M are rewritten before use, nothing needs clearing): two calls whose kernels can
 *     overlap on the GPU (different streams, no dependency) race on it; serialise them. */
int znn_softmax_xent_fwd_static(const float* logits, const int32_t* targets, float* probs, float* loss,
                                int M, int N, void* cuda_stream);
/* Softmax over the last dimension: :435-461 / :1054-1076 */
int znn_softmax_fwd(const float* A, float* C, size_t rows, int D);
int znn_softmax_bwd(const float* Y, const float* dY, float* dA, size_t rows, int D);
/* Fused form of mulScalar + causal -1e9 mask add + softmax as CausalSelfAttention runs them
 * (src/nn.zig:835-886); the mask is applied by index and never materialised.
 * S and P are nslices x T x T. Backward is the chain softmax -> add -> mulScalar
 * (src/autodiff.zig:1054-1076, :914-928, :895-904): dS += scale * P * (dP - sum(dP*P)). */
int znn_causal_softmax_fwd(const float* S, float scale, float* P, int nslices, int T);
int znn_causal_softmax_bwd(const float* P, const float* dP, float scale, float* dS, int nslices, int T);
/* the same gradient STORED into dS, with zeros above the diagonal (an addition, as znn_gelu_bwd_set) */
int znn_causal_softmax_bwd_set(const float* P, const float* dP, float scale, float* dS, int nslices, int T);
/* RmsNorm: :462-484 / :1077-1116 */
int znn_rmsnorm_fwd(const float* X, const float* G, float eps, float* Y, size_t rows, int D);
int znn_rmsnorm_bwd(const float* X, const float* G, const float* dY, float eps, float* dX, float* dG, size_t rows, int D);
/* LayerNorm: no counterpart in the reference (it only has RmsNorm); biased variance,
 * eps inside the square root. */
int znn_layernorm_fwd(const float* X, const float* G, const float* B, float eps, float* Y, size_t rows, int D);
int znn_layernorm_bwd(const float* X, const float* G, const float* dY, float eps, float* dX, float* dG, float* dB, size_t rows, int D);
/* Conv2D, NCHW, stride 1: src/tensor.zig:523-585, src/autodiff.zig:339-388 / :929-995.
 * pad = 0 is the reference; pad > 0 (zero padding) is an extension. bias may be NULL. */
int znn_conv2d_fwd(const float* X, const float* W, const float* bias, float* Y,
                   int N, int Ci, int H, int Wd, int Co, int KH, int KW, int pad);
/* The same with the following Relu (examples/cnn.zig:35-56: relu(conv(x))) applied as the result is stored: act = 1.
 * Y = max(0, conv(X) + bias); the pre-activation is not kept (Relu backward only needs the sign, which Y has). */
int znn_conv2d_fwd_act(const float* X, const float* W, const float* bias, float* Y, int N, int Ci, int H, int Wd, int Co,
                       int KH, int KW, int pad, int act);
int znn_conv2d_bwd(const float* X, const float* W, const float* dY, float* dX, float* dW, float* dbias,
                   int N, int Ci, int H, int Wd, int Co, int KH, int KW, int pad);
/* MaxPool2D: :389-434 / :996-1053. idx (may be NULL) receives, per output, the offset inside
 * the (n,c) input plane of the first maximum in (ph,pw) order. */
int znn_maxpool2d_fwd(const float* X, float* Y, int32_t* idx, int N, int C, int H, int W, int pool, int stride);
int znn_maxpool2d_bwd(const float* X, const float* dY, float* dX, int N, int C, int H, int W, int pool, int stride);
/* MaxPool2D backward followed by the backward of the Relu that produced the pool's input X (src/autodiff.zig:996-1053,
 * :673-683) in one pass: dX is the gradient of the Relu's INPUT; the window's winner receives g where X > 0. */
int znn_maxpool2d_bwd_relu(const float* X, const float* dY, float* dX, int N, int C, int H, int W, int pool, int stride);
/* Embedding (ids carried as fp32, as in the reference): :532-553 / :1183-1207.
 * The backward scatter-add is deterministic: rows with the same id are summed in (b,t) order.
 * The reference asserts id < vocab (:547); here an id outside [0, vocab) is never dereferenced: the forward writes a zero
 * row and sets ZNN_DEV_BAD_INDEX in the device status word, the backward ignores the position. */
int znn_embedding_fwd(const float* W, const float* ids, float* Y, size_t n, int D, int vocab);
int znn_embedding_bwd(const float* ids, const float* dY, float* dW, size_t n, int D, int vocab);
/* Transpose of two dims of a rank<=8 tensor: :276-302 / :848-876 (bwd accumulates) */
int znn_transpose_fwd(const float* A, float* C, const int64_t* dims, int rank, int d0, int d1);
int znn_transpose_bwd(const float* dC, float* dA, const int64_t* dims, int rank, int d0, int d1);
/* Add :331-338, gradient pass-through accumulate (Reshape/Add/AddScalar backward :831-839,
 * :905-928), MulScalar :315-322 / :895-904 */
int znn_add_fwd(const float* A, const float* B, float* C, size_t n);
int znn_accumulate(const float* src, float* dst, size_t n);
int znn_mul_scalar_fwd(const float* A, float v, float* C, size_t n);
int znn_mul_scalar_bwd(const float* dC, float v, float* dA, size_t n);
/* argmax over dim 0 or 1 of an M x N tensor, first maximum wins, result as fp32:
 * src/tensor.zig:813-851 (and the greedy pick of examples/transformer_gpt.zig:135-142) */
int znn_argmax(const float* A, float* out, int M, int N, int dim);
/* computeAccuracy of the example programs (examples/cnn.zig:193-205): argmax over each row of the M x N logits, compared
 * with the byte labels; *acc (device memory) = correct / M. */
int znn_accuracy_u8(const float* logits, const uint8_t* labels, int M, int N, float* acc);
/* SGD with optional momentum: src/optim.zig:50-66. v may be NULL when momentum == 0.
 * grad_scale multiplies the gradient first (1.0 = reference; 1/world for data parallel). */
int znn_sgd_step(float* w, const float* g, float* v, float lr, float momentum, float grad_scale, size_t n);
/* Adam: src/optim.zig:133-151.  t = step count after the increment (1 for the first step); the bias-corrected step size
 * lr*sqrt(1-beta2^t)/(1-beta1^t) is computed on the host in fp32 as the reference does; m, v are the moment buffers. */
int znn_adam_step(float* w, const float* g, float* m, float* v, float lr, float beta1, float beta2, float eps, float t,
                  float grad_scale, size_t n);
/* Input pipeline on the device.
 * znn_pixels_to_unit: IDX pixel bytes -> fp32 pixel / 255.0, the conversion of loadImages (src/dataset.zig:53-63).
 * znn_batch_gather: the copy loop of DataLoader.nextInto (src/dataset.zig:211-220): for j < batch,
 *   x_dest[j, :] = images[indices[j], :] (input_dim floats) and y_dest[j] = labels[indices[j]].
 *   images, labels, indices and both destinations are device memory; labels and y_dest may both be NULL.
 *   num_samples is the number of rows of images: an index outside [0, num_samples) is never dereferenced; its slot is
 *   zero-filled and ZNN_DEV_BAD_INDEX is set in the device status word. */
int znn_pixels_to_unit(const uint8_t* pixels, float* out, size_t n);
int znn_batch_gather(const float* images, const uint8_t* labels, const int32_t* indices, float* x_dest, uint8_t* y_dest,
                     int batch, int input_dim, size_t num_samples);
/* fill helpers (src/tensor.zig:354-379 fills; used for dC = 1 seeds and zeroGrad) */
int znn_fill(float* dst, float value, size_t n);
/* dst[i] = i mod period as floats: the position ids of a [batch, T] window (GPT.forward, src/nn.zig:1183-1196), made on the
 * device so that a training step uploads nothing */
int znn_iota_mod(float* dst, size_t n, int period);
/* Weight initialisation on the device.
 * znn_init_he_normal: initializeWeights (src/nn.zig:1336-1350): w[i] = N(0,1) * sqrt(2 / fan_in), one Box-Muller draw per
 *   element, cosine branch, u1 redrawn while it is 0.
 * znn_fill_normal / znn_fill_uniform: Tensor.fillNormal (src/tensor.zig:354-373: elements 2k, 2k+1 share one draw, cosine
 *   then sine) and Tensor.fillUniform (:375-379).
 * The distributions and the fan-in rule are the reference's.  The random STREAM is not: the reference draws from Zig's
 * std.Random.DefaultPrng, these draw from a counter-based hash of (seed, element index), so the same seed gives different
 * numbers than the reference would (parity of the stream is unpinned; parity tests share explicit weights instead). */
int znn_init_he_normal(float* w, size_t n, size_t fan_in, unsigned long long seed);
int znn_fill_normal(float* w, size_t n, float mean, float stddev, unsigned long long seed);
int znn_fill_uniform(float* w, size_t n, float min_val, float max_val, unsigned long long seed);

/* ---- data parallelism (new: the reference is single-process).  One process per GPU; the
 *      training step's only exchange is the sum of parameter gradients over ranks.
 *      znn_dp_unique_id is called on rank 0 and its 128 bytes are handed to every rank out of
 *      band (torch.distributed, a file, MPI ...).  All-reduces run on a communication stream
 *      ordered after the work already queued on the compute stream; znn_dp_join makes the
 *      compute stream wait for them. ---- */
int znn_dp_unique_id(char* out128);
int znn_dp_init(int world, int rank, const char* id128);     /* one process per GPU: this process is `rank` of `world` */
/* One process that drives devices 0 .. ndev-1 itself (ncclCommInitAll): device d becomes rank d.  The calling thread
 * selects the rank it speaks for with znn_set_device; collective calls issued for several devices by ONE thread must be
 * bracketed by znn_dp_group_begin / znn_dp_group_end (ncclGroupStart / ncclGroupEnd), or each device needs its own thread. */
int znn_dp_init_all(int ndev);
int znn_dp_group_begin(void);
int znn_dp_group_end(void);
int znn_dp_world(int* world, int* rank);
int znn_dp_allreduce_async(float* buf, size_t count);   /* in-place fp32 sum */
int znn_dp_join(void);
int znn_dp_allreduce(float* buf, size_t count);
int znn_dp_broadcast(float* buf, size_t count, int root);
/* Failure detection.  znn_dp_set_timeout_ms(ms > 0), called before znn_dp_init, creates the communicator non-blocking:
 * every NCCL call is then polled (ncclCommGetAsyncError) until NCCL has accepted it, at most ms milliseconds.
 * znn_dp_wait(timeout_ms) blocks the HOST until the reductions queued so far have finished, polling the communicator's
 * asynchronous error state meanwhile.  On an NCCL error or an expired deadline the communicator is aborted
 * (ncclCommAbort) so that this rank does not stay blocked on a peer that is gone, and ZNN_ERR_NCCL is returned;
 * later collective calls fail at once until znn_dp_finalize + znn_dp_init.  znn_dp_abort does the same on request. */
int znn_dp_set_timeout_ms(long long ms);
int znn_dp_wait(long long timeout_ms);
int znn_dp_abort(void);
int znn_dp_finalize(void);

#ifdef __cplusplus
}
#endif
#endif
