// Host-side mirror of the reference's Tensor / Op / Graph (src/tensor.zig:14-88,
// src/autodiff.zig:14-105, :1237-2264) over device memory.
//
// Same names and semantics as the reference: every Graph builder runs the eager
// forward, sets requires_grad to the OR of its inputs, allocates a zeroed grad,
// and appends an Op to the tape; backward() sorts topologically from the loss
// (DFS post-order over creator.inputs), seeds loss.grad[0] = 1 and sweeps in
// reverse calling each creator's backward arm, which ACCUMULATES into its
// inputs' grads.  All arithmetic is done by the C ABI of include/znn_cuda.h;
// this layer is bookkeeping only.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <functional>
#include <initializer_list>
#include <stdexcept>
#include <string>
#include <vector>

namespace znn {
namespace host {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& what) : std::runtime_error(what), code(c) {}
};
// throws Error when rc != 0 (text from znn_last_error)
void check(int rc, const char* what);

// src/tensor.zig:14-39
struct Shape {
    size_t dims[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t len = 0;
    Shape() = default;
    Shape(std::initializer_list<size_t> d);
    Shape(const size_t* d, size_t n);
    size_t numel() const;
    bool operator==(const Shape& o) const;
};
Shape contiguous_strides(const Shape& s);  // src/tensor.zig:49-65

struct Op;

// src/tensor.zig:81-88: data / grad are DEVICE pointers here
struct Tensor {
    float* data = nullptr;
    float* grad = nullptr;  // nullptr when !requires_grad (the reference's empty slice)
    Shape shape, strides;
    bool requires_grad = false;
    Op* creator = nullptr;
    // Gradient buffers of graph intermediates are zero-filled lazily: grad_valid is false until the first backward
    // arm touches the buffer; an arm that overwrites the whole buffer (a GEMM with beta = 0) then needs no fill at all.
    // A Reshape view that shares its input's buffer points at the owner, whose flag counts.
    bool grad_valid = true;
    Tensor* grad_owner = nullptr;
    int consumers = 0;   // ops that read this tensor (counted while the tape is built)
    Op* last_consumer = nullptr;   // the latest of them
    size_t numel() const { return shape.numel(); }
};

// Zero-fills t's gradient buffer if nothing has written it yet (call before reading it or adding into it).
void ensure_grad(Tensor* t);
// For an arm that can overwrite the whole buffer: true = do so (the buffer then counts as written), false = add.
bool claim_grad_overwrite(Tensor* t);
// True when nothing has been written or added to t's gradient buffer yet.
bool grad_is_fresh(Tensor* t);
// After the caller stored a complete gradient into the buffer.
void mark_grad_written(Tensor* t);
// Lazy zero-fill of intermediate gradients (default on; off = every gradient buffer is zero-filled when created).
// BatchMatMul role 2 backward produces the gradient of the SCORES directly (znn_attn_dscores), skipping dP and the
// separate softmax backward; default on.
void set_fused_softmax_bwd(bool on);
bool fused_softmax_bwd();
void set_lazy_zero_grad(bool on);
bool lazy_zero_grad();
// The elementwise step after (or before, in the backward) a Linear runs in the GEMM's epilogue where the shapes allow
// (znn_linear_fwd_ex / znn_linear_bwd_ex).  The tape keeps the separate ops; only which kernels fill their tensors changes.
// Bit mask: 1 = residual add after an output projection, 2 = ReLU forward and its derivative backward, 4 = GELU forward,
// 8 = GELU derivative backward.  Default 2.  The epilogue warps of the GEMM kernel are its latency-bound role: measured on
// the GPT step (18.79 ms with mask 0), the residual form costs +0.08 ms net (one more 16-byte load per stored float4
// against two 25 MB add kernels saved per layer), GELU forward +0.5 ms and its derivative +0.95 ms (erf and exp per
// element in the epilogue against bandwidth-bound stand-alone kernels).  ReLU is free (one max per element).
void set_fused_epilogue(int mask);
int fused_epilogue();
// Linear layers that share their input run as grouped launches (Graph::linearGroup); default on.
void set_group_linear(bool on);
bool group_linear();

// hot-path subset of src/autodiff.zig:14-40, plus two additions
enum class OpType {
    MatMul, AddBias, Relu, Gelu, SoftmaxCrossEntropy, Reshape, Transpose, MulScalar, Add, Conv2D, MaxPool2D,
    Softmax, RmsNorm, BatchMatMul, Embedding,
    CausalSoftmax,  // fused mulScalar + mask add + softmax of src/nn.zig:835-886 (an addition)
    LayerNorm,      // extension, no reference counterpart
    LinearBias,     // fused matmul + addBias of Linear.forward (src/nn.zig:44-51), an addition
    BatchMatMulNT,  // C = A.B^T per (batch, head) slice: transposeND(K) + batchMatMul of src/nn.zig:796-835 in one op, an addition
    CausalAttention // the whole chain of src/nn.zig:796-906 (head split, Q.K^T, scale, mask, softmax, P.V, head merge) as one
                    // fused op on the [B*T, C] projections (znn_attn_fwd / znn_attn_bwd), an addition
};

// src/autodiff.zig:100-105 (OpContext flattened)
struct Op {
    OpType type;
    std::vector<Tensor*> inputs, outputs;
    float scalar = 0.0f;        // MulScalar value / RmsNorm eps / CausalSoftmax scale
    int dim0 = 0, dim1 = 0;     // Transpose
    int pool = 0, stride = 0;   // MaxPool2D
    int pad = 0;                // Conv2D (0 = reference)
    int att_B = 0, att_T = 0, att_nh = 0;   // CausalAttention: batch, sequence length, heads (scratch = the rows' log-sum-exp)
    int tri_role = 0;           // BatchMatMul next to a causal softmax: 1 = C are the scores, 2 = A are the probabilities
    float* scratch = nullptr;   // BatchMatMul role 2: one float per probability row (the D vector of the fused backward)
    bool skip_backward = false; // CausalSoftmax: its input gradient was already produced by the consumer's fused backward
    std::vector<Op*> group;     // LinearBias, last of a group on one input (Graph::linearGroup): all members, in creation order
    float* probs = nullptr;     // SoftmaxCrossEntropy: device M x N
    int32_t* targets = nullptr; // SoftmaxCrossEntropy: device int32 labels (device bytes when targets_u8)
    bool targets_u8 = false;
    void forward();             // src/autodiff.zig:107-575
    void backward();            // src/autodiff.zig:579-1231
};

// Reshape views share their input's gradient buffer (default on; off = a separate, zeroed gradient and an adding
// backward arm as in src/autodiff.zig:1346-1347, :831-839).  The sums are the same; only their order differs.
void set_alias_reshape_grad(bool on);
bool alias_reshape_grad();

// Device bump allocator: the analogue of Graph.arena (std.heap.ArenaAllocator).
// reset() makes every allocation of the previous step reusable at once.
class Arena {
public:
    explicit Arena(size_t bytes);
    ~Arena();
    Arena(const Arena&) = delete;
    Arena& operator=(const Arena&) = delete;
    void* alloc(size_t bytes);  // 256-byte aligned; throws Error(ZNN_ERR_NOMEM) when exhausted
    void reset() { used_ = 0; }
    size_t used() const { return used_; }
    size_t high_water() const { return high_; }
    size_t capacity() const { return cap_; }

private:
    char* base_ = nullptr;
    size_t cap_ = 0, used_ = 0, high_ = 0;
};

// src/autodiff.zig:1237-2264
class Graph {
public:
    explicit Graph(Arena* arena) : arena_(arena) {}
    ~Graph();
    Graph(const Graph&) = delete;
    Graph& operator=(const Graph&) = delete;

    // creators (:1260-1326)
    Tensor* tensorND(const Shape& shape, bool requires_grad);
    Tensor* array(const Shape& shape, const float* host_data, bool requires_grad);      // uploads
    Tensor* arrayFromDevice(const Shape& shape, const float* dev_data, bool requires_grad);

    // builders
    Tensor* matmul(Tensor* A, Tensor* B);                                   // :1414
    Tensor* addBias(Tensor* A, Tensor* bias);                               // :1446
    Tensor* relu(Tensor* A);                                                // :1478
    Tensor* gelu(Tensor* A);                                                // :1508
    Tensor* softmaxCrossEntropy(Tensor* logits, const int32_t* dev_targets); // :1630 (int32 labels on device)
    Tensor* softmaxCrossEntropyU8(Tensor* logits, const uint8_t* dev_targets); // the reference's own label type (u8)
    Tensor* reshape(Tensor* A, const Shape& new_shape);                     // :1329 (aliases data, own grad)
    Tensor* transposeND(Tensor* A, int dim0, int dim1);                     // :1378
    Tensor* mulScalar(Tensor* A, float v);                                  // :1910
    Tensor* add(Tensor* A, Tensor* B);                                      // :1972
    Tensor* conv2d(Tensor* A, Tensor* W, Tensor* bias, int pad = 0);        // :2003
    Tensor* maxpool2d(Tensor* A, int pool, int stride);                     // :2038
    Tensor* softmax(Tensor* A);                                             // :2068
    Tensor* rmsNorm(Tensor* X, Tensor* G, float eps);                       // :2098
    // tri_role (an addition): 1 = C = Q.K^T feeds a causal softmax (only its lower triangle is ever read, and its
    // gradient is lower-triangular), 2 = A holds causal-softmax probabilities (lower-triangular); the products then
    // skip the tiles the mask makes irrelevant (znn_sgemm_batched_strided_tri).  0 = the reference's full products.
    Tensor* batchMatMul(Tensor* A, Tensor* B, int tri_role = 0);            // :2129
    // C[b,h] = A[b,h] . B[b,h]^T for A [b,h,M,K], B [b,h,N,K] (an addition: no transposed copy of B is made and the
    // gradient of B comes out as dC^T.A, a product with a tall output instead of a 64-row one); tri_role as above
    Tensor* batchMatMulNT(Tensor* A, Tensor* B, int tri_role = 0);
    Tensor* embedding(Tensor* W, Tensor* X);                                // :2160
    Tensor* causalSoftmax(Tensor* S, float scale);                          // fused addition
    // y[B*T, C] = merge_heads(softmax(scale * Q_h.K_h^T + causal mask).V_h) for q, k, v of shape [B*T, C] with nh heads
    // of C / nh columns each (src/nn.zig:796-906 in one op; no score matrix, no head split / merge copies)
    Tensor* causalAttention(Tensor* q, Tensor* k, Tensor* v, size_t B, size_t T, size_t nh, float scale);
    Tensor* layerNorm(Tensor* X, Tensor* G, Tensor* B, float eps);          // extension
    Tensor* linear(Tensor* X, Tensor* W, Tensor* bias);                     // fused addBias(matmul(X, W), bias)
    // act(linear(X, W, bias)) with act = Relu or Gelu: the tape gets the Linear and the activation op, one GEMM fills both
    // outputs (pre-activation and activation) when the epilogue form applies
    Tensor* linearAct(Tensor* X, Tensor* W, Tensor* bias, OpType act);
    // add(R, linear(X, W, bias)): the residual is added in the GEMM's epilogue when the form applies
    Tensor* linearResidual(Tensor* X, Tensor* W, Tensor* bias, Tensor* R);
    // relu(conv2d(A, W, bias)): the tape gets the Conv2D and the Relu op, one kernel stores max(0, .) (the pre-activation is
    // not kept: no backward arm reads it)
    Tensor* conv2dRelu(Tensor* A, Tensor* W, Tensor* bias, int pad);
    // n Linear layers of the same shape on one input (the q, k, v projections): n LinearBias ops on the tape; when their
    // parameters and outputs lie at uniform strides the forward is one grouped launch, and the backward of the last one
    // runs all members' weight gradients as one grouped launch and their data gradients as one K-concatenated product
    void linearGroup(Tensor* X, int n, Tensor* const* W, Tensor* const* bias, Tensor** out);

    // `after_op(op)` is called after a tape op has run its
    // backward arm; data-parallel training uses it to start gradient all-reduces.
    void backward(Tensor* loss, const std::function<void(Op*)>* after_op = nullptr);   // :2192
    void backwardWithGrad(Tensor* out, const std::function<void(Op*)>* after_op = nullptr); // :2217
    void forward();    // :2252 re-executes the tape in creation order
    void zeroGrad();   // :2259

    const std::vector<Op*>& ops() const { return ops_; }
    const std::vector<Tensor*>& tensors() const { return tensors_; }
    Arena* arena() { return arena_; }
    // index of `op` in the tape (creation order)
    size_t op_index(const Op* op) const;

private:
    Tensor* new_tensor(const Shape& shape, bool requires_grad, bool zero_data);
    Op* new_op(OpType type, std::initializer_list<Tensor*> inputs, Tensor* out);
    void sweep(Tensor* root, const std::function<void(Op*)>* after_op);
    Arena* arena_;
    std::vector<Tensor*> tensors_;
    std::vector<Op*> ops_;
};

}  // namespace host
}  // namespace znn
