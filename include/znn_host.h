/*
 * znn_host.h -- C entry points of the host-side mirror of the reference's
 * Tensor / Graph / Op / nn / optim layer (znn_b200/csrc/host/), for callers that
 * cannot use the C++ classes directly (the Python tests and benchmarks).
 *
 * Two levels:
 *  - znn_graph_*: a Graph (src/autodiff.zig:1237-2264) with integer tensor
 *    handles; `znn_graph_op` appends one op by its reference builder name
 *    ("matmul", "addBias", "relu", "gelu", "softmaxCrossEntropy", "reshape",
 *    "transposeND", "mulScalar", "add", "conv2d", "maxpool2d", "softmax",
 *    "rmsNorm", "batchMatMul", "embedding", plus the additions "causalSoftmax", "layerNorm", "linear", "causalAttention"
 *    (args: B, T, heads, scale)).
 *  - znn_model_*: the example programs' models (examples/fashion_mnist.zig,
 *    examples/cnn.zig, examples/transformer_block.zig, examples/transformer_gpt.zig)
 *    with their training step: new graph -> forward -> SoftmaxCrossEntropy ->
 *    zeroGrad -> backward -> [gradient all-reduce] -> SGD step.
 * All functions return 0 or a negative ZNN_ERR_* code (text: znn_last_error).
 */
#ifndef ZNN_HOST_H
#define ZNN_HOST_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct znn_graph znn_graph;
typedef struct znn_model znn_model;

int znn_graph_create(size_t arena_bytes, znn_graph** out);
int znn_graph_destroy(znn_graph* g);
/* Graph.array / Graph.tensorND (host_data may be NULL = zeros) */
int znn_graph_array(znn_graph* g, const long long* dims, int rank, const float* host_data, int requires_grad, int* id);
/* args: reshape -> new dims; transposeND -> dim0, dim1; mulScalar -> value; maxpool2d -> pool, stride;
 * rmsNorm/layerNorm -> eps; conv2d -> pad (optional); causalSoftmax -> scale;
 * softmaxCrossEntropy -> the M integer class labels */
int znn_graph_op(znn_graph* g, const char* name, const int* inputs, int n_inputs, const double* args, int n_args, int* id);
int znn_graph_backward(znn_graph* g, int id, int seed_one);  /* seed_one=1: Graph.backward, 0: backwardWithGrad */
int znn_graph_forward(znn_graph* g);                         /* Graph.forward: re-execute the tape */
int znn_graph_zero_grad(znn_graph* g);
int znn_graph_shape(znn_graph* g, int id, long long* dims8, int* rank, int* requires_grad);
int znn_graph_read(znn_graph* g, int id, int which, float* host, size_t count);        /* which: 0 data, 1 grad */
int znn_graph_write(znn_graph* g, int id, int which, const float* host, size_t count);
int znn_graph_num_ops(znn_graph* g, int* n);

#define ZNN_MODEL_MLP 1         /* dims: in, h1, h2, out            (examples/fashion_mnist.zig:25-27) */
#define ZNN_MODEL_CNN_REF 2     /* no dims                          (examples/cnn.zig:24-27)           */
#define ZNN_MODEL_CNN_PADDED 3  /* no dims: 1->32->64 pad 1, 3136->128->10 (workload definition)      */
#define ZNN_MODEL_BLOCK 4       /* dims: n_embd, n_head             (src/nn.zig:950-1022)              */
#define ZNN_MODEL_GPT 5         /* dims: vocab, block_size, n_embd, n_head, n_layer (src/nn.zig:1125) */

int znn_model_create(int kind, const long long* dims, int ndims, size_t arena_bytes, znn_model** out);
int znn_model_destroy(znn_model* m);
int znn_model_param_count(znn_model* m, int* n);
int znn_model_param_info(znn_model* m, int i, char* name, size_t name_len, long long* dims8, int* rank,
                         long long* offset, long long* fan_in);
int znn_model_total_floats(znn_model* m, long long* total);   /* slab length incl. alignment padding */
/* Checkpoint files byte-compatible with the reference's saveModel / loadModel (src/nn.zig:268-382): 8-byte little-endian
 * header length, a safetensors-style JSON header (entries in parameter order, no spaces, padded with spaces to a multiple
 * of 8), then the fp32 data in the same order.  Loading checks names, dtype, shapes, sizes and that offsets do not go
 * backwards, as the reference does. */
int znn_model_save(znn_model* m, const char* path);
int znn_model_load(znn_model* m, const char* path);
/* Optimizer state for resuming (an extension: the reference's file holds parameters only): the SGD velocities in a
 * second file of the same layout, one entry per parameter under the parameter's name, so the reference's reader and
 * writer handle it too.  With the Adam optimizer the file holds the first moments and a second file, path + ".v2",
 * the second moments; the step count is the "adam_t" option. */
int znn_model_save_optimizer(znn_model* m, const char* path);
int znn_model_load_optimizer(znn_model* m, const char* path);
/* The modules' own initialisation (src/nn.zig:22-23, :71-72, :520, :565): weights He-normal with the module's fan-in
 * (znn_init_he_normal), biases 0, norm gains 1.  Parameter i draws with seed + i; the random stream is not the
 * reference's (see znn_init_he_normal). */
int znn_model_init_weights(znn_model* m, unsigned long long seed);
int znn_model_set_params(znn_model* m, const float* host_slab);
int znn_model_get_params(znn_model* m, float* host_slab);
int znn_model_get_grads(znn_model* m, float* host_slab);
int znn_model_get_velocities(znn_model* m, float* host_slab);
/* keys: "lr", "momentum", "fused_softmax" (1/0), "fused_linear" (1/0, process-wide), "causal_skip" (1/0, process-wide: attention products
 * skip the tiles above the causal diagonal; needs fused_softmax), "fused_softmax_bwd" (1/0, process-wide: the gradient of the attention scores comes out of
 * the dO.V^T product's epilogue, no dP buffer and no separate softmax backward), "fused_attention" (1/0, process-wide, default 1: the whole attention chain
 * as the one fused op znn_attn_fwd / znn_attn_bwd on the [B*T, C] projections when the head size is 32 or 64 and T a multiple
 * of 4; needs fused_softmax; 0 = the separate products and softmax below), "fused_epilogue" (bit mask, process-wide, default 2: 1 = the residual add
 * after an output projection, 2 = ReLU after a Linear and its derivative in backward, 4 = GELU forward, 8 = GELU derivative
 * backward run in the epilogue of the neighbouring GEMM, znn_linear_fwd_ex / znn_linear_bwd_ex; the tape keeps the separate
 * ops; only the ReLU form is on by default: the others measured slower than the separate kernels on the GPT step), "group_linear" (1/0, process-wide, default 1: the three attention projections, which share
 * their input, run as grouped launches, znn_sgemm_grouped: one forward, one for the three weight gradients, one K-concatenated
 * product for the sum of the three data gradients), "fused_qkt" (1/0, process-wide: attention scores as one
 * Q.K^T op instead of a transposed copy of K and a product), "alias_reshape_grad" (1/0, process-wide: Reshape views
 * share the gradient buffer of their input instead of adding into it in backward), "lazy_zero_grad" (1/0, process-wide:
 * gradient buffers of intermediates are zero-filled only when first added to; GEMM arms overwrite them with beta = 0), "dp_bucket_floats",
 * "dp_overlap" (1/0), "cuda_graph" (1/0: capture the training step once per (input buffers, batch) and replay it;
 * MLP / CNN models with device-resident inputs on one GPU; the capture is redone when lr, momentum or
 * a fused_* option changes, or when one of the shim's scratch blocks has moved since),
 * "optimizer" (0 = SGD with "lr" / "momentum" as the example programs use, 1 = Adam, src/optim.zig:69-152, with "lr",
 * "beta1", "beta2", "eps" and the step count "adam_t"; no CUDA-graph replay with Adam: the step size changes per step),
 * "targets_u8" (1/0: the targets pointer of znn_model_train_step holds byte labels, the reference's label type,
 * e.g. the y_dest of znn_loader_next_into; default 0 = int32) */
int znn_model_set_option(znn_model* m, const char* key, double value);
/* One training step.  x: [batch, features] pixels (MLP/CNN) or [batch, seq] fp32 token ids (GPT); targets: batch
 * (or batch*seq) int32 labels.  on_device = 1: both pointers are device memory and are used in place.
 * loss_host may be NULL (no read-back, no synchronisation). */
int znn_model_train_step(znn_model* m, const float* x, const int32_t* targets, int batch, int seq, int on_device,
                         float* loss_host);
/* One evaluation batch as the example programs' evaluateModel runs it (examples/cnn.zig:212-256): forward, mean
 * cross-entropy loss, and computeAccuracy (:193-205) = fraction of rows whose argmax equals the byte label.  MLP / CNN
 * models; x and labels are host memory, or device memory used in place when on_device = 1 (e.g. a loader's batch). */
int znn_model_evaluate(znn_model* m, const float* x, const uint8_t* labels, int batch, int on_device, float* loss_host,
                       float* acc_host);
/* forward only; logits_host receives batch x classes (MLP/CNN) or batch*seq x vocab (GPT); may be NULL */
int znn_model_forward(znn_model* m, const float* x, int batch, int seq, int on_device, float* logits_host);
/* transformer block: y = block(x); backward from dy; x,dy,y host arrays of B*T*n_embd; dx may be NULL */
int znn_model_block_fwd_bwd(znn_model* m, const float* x, const float* dy, int B, int T, float* y, float* dx);
/* the same with DEVICE arrays; asynchronous on the thread's stream */
int znn_model_block_fwd_bwd_device(znn_model* m, const float* x, const float* dy, int B, int T, float* y, float* dx);
/* greedy decode as examples/transformer_gpt.zig:116-146 (full re-forward per token over the last block_size ids,
 * first-maximum argmax), for `batch` prompts of prompt_len ids at once; out_ids: batch x n_new */
int znn_model_greedy_decode(znn_model* m, const float* prompt_ids, int batch, int prompt_len, int n_new, float* out_ids);
/* The same tokens with a key/value cache (an addition: the reference re-runs the whole window per token): every position
 * passes through the layers once.  Needs prompt_len + n_new - 1 <= block_size (no sliding window).  Logits agree with the
 * full re-forward to GEMM rounding, so the greedy tokens are the same unless two logits tie within that rounding. */
int znn_model_greedy_decode_kv(znn_model* m, const float* prompt_ids, int batch, int prompt_len, int n_new, float* out_ids);
int znn_model_arena_high_water(znn_model* m, long long* bytes);
int znn_model_last_step_ops(znn_model* m, int* n_ops);
int znn_model_graph_replays(znn_model* m, long long* n);

/* ---- input pipeline: src/dataset.zig ------------------------------------------------------------------------------
 * The dataset stays resident in device memory; a batch is produced by one gather launch, no host data moves.
 * znn_dataset_load_idx: loadDataset's two readers (src/dataset.zig:23-106): big-endian IDX headers, magic 0x803 /
 *   0x801 (else an error naming InvalidMagicNumber), pixels as fp32 pixel/255.  Returns device pointers the caller
 *   frees with znn_free.  The counts are returned as read; the reference does not compare them either.
 * znn_loader_*: DataLoader (src/dataset.zig:132-223).  seed < 0 = the reference's default 1337.  shuffle permutes
 *   the order at create and at every reset with the reference's generator and draw (std.Random.DefaultPrng,
 *   intRangeLessThan).  next_into writes x_dest (n x input_dim fp32) and y_dest (n bytes), both device memory, and
 *   sets *n = 0 where the reference returns null (epoch finished, or a short tail with drop_last). */
typedef struct znn_loader znn_loader;
int znn_dataset_load_idx(const char* images_path, const char* labels_path, float** images, uint8_t** labels,
                         unsigned* num_images, unsigned* rows, unsigned* cols, unsigned* num_labels);
int znn_loader_create(const float* images, const uint8_t* labels, size_t num_samples, int input_dim, size_t batch_size,
                      int shuffle, int drop_last, long long seed, znn_loader** out);
int znn_loader_destroy(znn_loader* l);
int znn_loader_reset(znn_loader* l);
int znn_loader_set_drop_last(znn_loader* l, int drop_last);
int znn_loader_peek_next_batch_size(znn_loader* l, size_t* n);
int znn_loader_next_into(znn_loader* l, float* x_dest, uint8_t* y_dest, size_t* n);
int znn_loader_indices(znn_loader* l, int32_t* host_out, size_t count);   /* the current sample order */

#ifdef __cplusplus
}
#endif
#endif
