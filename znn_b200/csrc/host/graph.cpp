// Host-side Tensor / Op / Graph mirror: see graph.hpp.  Bookkeeping only; every
// arm forwards to the C ABI.
#include "graph.hpp"

#include <algorithm>
#include <unordered_set>

#include "../../../include/znn_cuda.h"

namespace znn {
namespace host {

void check(int rc, const char* what)
{
    if (rc == 0) return;
    char buf[512];
    znn_last_error(buf, sizeof(buf));
    throw Error(rc, std::string(what) + ": " + buf);
}

Shape::Shape(std::initializer_list<size_t> d)
{
    if (d.size() > 8) throw Error(ZNN_ERR_INVALID, "rank above 8");
    for (size_t v : d) dims[len++] = v;
}

Shape::Shape(const size_t* d, size_t n)
{
    if (n > 8) throw Error(ZNN_ERR_INVALID, "rank above 8");
    for (size_t i = 0; i < n; i++) dims[i] = d[i];
    len = n;
}

size_t Shape::numel() const
{
    size_t t = 1;
    for (size_t i = 0; i < len; i++) t *= dims[i];
    return t;
}

bool Shape::operator==(const Shape& o) const
{
    if (len != o.len) return false;
    for (size_t i = 0; i < len; i++)
        if (dims[i] != o.dims[i]) return false;
    return true;
}

Shape contiguous_strides(const Shape& s)
{
    Shape st;
    st.len = s.len;
    size_t acc = 1;
    for (size_t i = s.len; i > 0;) {
        i--;
        st.dims[i] = acc;
        acc *= s.dims[i];
    }
    return st;
}

// ---------------------------------------------------------------- Arena
Arena::Arena(size_t bytes) : cap_(bytes)
{
    void* p = nullptr;
    check(znn_malloc(&p, bytes), "Arena: znn_malloc");
    base_ = (char*)p;
}

Arena::~Arena()
{
    if (base_) znn_free(base_);
}

void* Arena::alloc(size_t bytes)
{
    const size_t need = (bytes + 255) & ~(size_t)255;
    if (used_ + need > cap_)
        throw Error(ZNN_ERR_NOMEM, "graph arena exhausted: need " + std::to_string(used_ + need) + " of " +
                                       std::to_string(cap_) + " bytes");
    void* p = base_ + used_;
    used_ += need;
    if (used_ > high_) high_ = used_;
    return p;
}

// ---------------------------------------------------------------- Graph
Graph::~Graph()
{
    for (Tensor* t : tensors_) delete t;
    for (Op* o : ops_) delete o;
}

static bool g_lazy_zero_grad = true;
void set_lazy_zero_grad(bool on) { g_lazy_zero_grad = on; }
bool lazy_zero_grad() { return g_lazy_zero_grad; }

static Tensor* grad_root(Tensor* t)
{
    while (t->grad_owner) t = t->grad_owner;
    return t;
}

void ensure_grad(Tensor* t)
{
    if (!t->grad) return;
    Tensor* r = grad_root(t);
    if (r->grad_valid) return;
    check(znn_memset(r->grad, 0, r->numel() * sizeof(float)), "znn_memset");
    r->grad_valid = true;
}

bool claim_grad_overwrite(Tensor* t)
{
    Tensor* r = grad_root(t);
    if (r->grad_valid) return false;
    r->grad_valid = true;
    return true;
}

void mark_grad_written(Tensor* t) { grad_root(t)->grad_valid = true; }

bool grad_is_fresh(Tensor* t) { return t->grad && !grad_root(t)->grad_valid; }

static int g_fused_epilogue = 2;
void set_fused_epilogue(int mask) { g_fused_epilogue = mask; }
int fused_epilogue() { return g_fused_epilogue; }

static bool g_group_linear = true;
void set_group_linear(bool on) { g_group_linear = on; }
bool group_linear() { return g_group_linear; }

static bool g_fused_softmax_bwd = true;
void set_fused_softmax_bwd(bool on) { g_fused_softmax_bwd = on; }
bool fused_softmax_bwd() { return g_fused_softmax_bwd; }

Tensor* Graph::new_tensor(const Shape& shape, bool requires_grad, bool zero_data)
{
    Tensor* t = new Tensor();
    t->shape = shape;
    t->strides = contiguous_strides(shape);
    t->requires_grad = requires_grad;
    const size_t bytes = shape.numel() * sizeof(float);
    t->data = (float*)arena_->alloc(bytes);
    if (zero_data) check(znn_memset(t->data, 0, bytes), "znn_memset");
    if (requires_grad) {
        t->grad = (float*)arena_->alloc(bytes);
        if (g_lazy_zero_grad) t->grad_valid = false;
        else check(znn_memset(t->grad, 0, bytes), "znn_memset");
    }
    tensors_.push_back(t);
    return t;
}

Op* Graph::new_op(OpType type, std::initializer_list<Tensor*> inputs, Tensor* out)
{
    Op* o = new Op();
    o->type = type;
    o->inputs.assign(inputs.begin(), inputs.end());
    o->outputs.push_back(out);
    out->creator = o;
    for (Tensor* in : o->inputs) {
        in->consumers++;
        in->last_consumer = o;
    }
    ops_.push_back(o);
    return o;
}

Tensor* Graph::tensorND(const Shape& shape, bool requires_grad) { return new_tensor(shape, requires_grad, true); }

Tensor* Graph::array(const Shape& shape, const float* host_data, bool requires_grad)
{
    Tensor* t = new_tensor(shape, requires_grad, false);
    check(znn_memcpy_h2d(t->data, host_data, shape.numel() * sizeof(float)), "znn_memcpy_h2d");
    check(znn_sync(), "znn_sync");  // the host buffer may be a temporary
    return t;
}

Tensor* Graph::arrayFromDevice(const Shape& shape, const float* dev_data, bool requires_grad)
{
    Tensor* t = new_tensor(shape, requires_grad, false);
    check(znn_memcpy_d2d(t->data, dev_data, shape.numel() * sizeof(float)), "znn_memcpy_d2d");
    return t;
}

static bool any_grad(std::initializer_list<Tensor*> ts)
{
    for (Tensor* t : ts)
        if (t && t->requires_grad) return true;
    return false;
}

Tensor* Graph::matmul(Tensor* A, Tensor* B)
{
    if (A->shape.len < 2 || B->shape.len < 2 || A->shape.dims[1] != B->shape.dims[0])
        throw Error(ZNN_ERR_INVALID, "matmul: inner dimensions differ");
    Tensor* C = new_tensor(Shape{A->shape.dims[0], B->shape.dims[1]}, any_grad({A, B}), false);
    Op* o = new_op(OpType::MatMul, {A, B}, C);
    o->forward();
    return C;
}

Tensor* Graph::addBias(Tensor* A, Tensor* bias)
{
    Tensor* C = new_tensor(A->shape, any_grad({A, bias}), false);
    new_op(OpType::AddBias, {A, bias}, C)->forward();
    return C;
}

Tensor* Graph::relu(Tensor* A)
{
    Tensor* C = new_tensor(A->shape, A->requires_grad, false);
    new_op(OpType::Relu, {A}, C)->forward();
    return C;
}

Tensor* Graph::gelu(Tensor* A)
{
    Tensor* C = new_tensor(A->shape, A->requires_grad, false);
    new_op(OpType::Gelu, {A}, C)->forward();
    return C;
}

Tensor* Graph::softmaxCrossEntropy(Tensor* logits, const int32_t* dev_targets)
{
    if (logits->shape.len != 2) throw Error(ZNN_ERR_INVALID, "softmaxCrossEntropy needs 2-D logits");
    Tensor* loss = new_tensor(Shape{1, 1}, logits->requires_grad, false);
    Op* o = new_op(OpType::SoftmaxCrossEntropy, {logits}, loss);
    o->probs = (float*)arena_->alloc(logits->numel() * sizeof(float));
    o->targets = const_cast<int32_t*>(dev_targets);
    o->forward();
    return loss;
}

Tensor* Graph::softmaxCrossEntropyU8(Tensor* logits, const uint8_t* dev_targets)
{
    if (logits->shape.len != 2) throw Error(ZNN_ERR_INVALID, "softmaxCrossEntropy needs 2-D logits");
    Tensor* loss = new_tensor(Shape{1, 1}, logits->requires_grad, false);
    Op* o = new_op(OpType::SoftmaxCrossEntropy, {logits}, loss);
    o->probs = (float*)arena_->alloc(logits->numel() * sizeof(float));
    o->targets = reinterpret_cast<int32_t*>(const_cast<uint8_t*>(dev_targets));
    o->targets_u8 = true;
    o->forward();
    return loss;
}

static bool g_alias_reshape_grad = true;
void set_alias_reshape_grad(bool on) { g_alias_reshape_grad = on; }
bool alias_reshape_grad() { return g_alias_reshape_grad; }

Tensor* Graph::reshape(Tensor* A, const Shape& new_shape)
{
    if (new_shape.numel() != A->numel()) throw Error(ZNN_ERR_INVALID, "reshape: element counts differ");
    Tensor* C = new Tensor();
    C->shape = new_shape;
    C->strides = contiguous_strides(new_shape);
    C->requires_grad = A->requires_grad;
    C->data = A->data;  // shares the forward data (autodiff.zig:1346)
    if (A->requires_grad) {
        if (alias_reshape_grad()) {
            // The view shares the gradient buffer too: every backward arm accumulates (+=), so consumers of the
            // view add straight into the input's gradient and Reshape.backward has nothing left to add.
            C->grad = A->grad;
            C->grad_owner = A;
        } else {
            C->grad = (float*)arena_->alloc(A->numel() * sizeof(float));   // own grad, as autodiff.zig:1347
            if (g_lazy_zero_grad) C->grad_valid = false;
            else check(znn_memset(C->grad, 0, A->numel() * sizeof(float)), "znn_memset");
        }
    }
    tensors_.push_back(C);
    new_op(OpType::Reshape, {A}, C);
    return C;
}

Tensor* Graph::transposeND(Tensor* A, int dim0, int dim1)
{
    if (dim0 < 0 || dim1 < 0 || (size_t)dim0 >= A->shape.len || (size_t)dim1 >= A->shape.len)
        throw Error(ZNN_ERR_INVALID, "transposeND: dimension out of range");
    Shape s = A->shape;
    std::swap(s.dims[dim0], s.dims[dim1]);
    Tensor* C = new_tensor(s, A->requires_grad, false);
    Op* o = new_op(OpType::Transpose, {A}, C);
    o->dim0 = dim0;
    o->dim1 = dim1;
    o->forward();
    return C;
}

Tensor* Graph::mulScalar(Tensor* A, float v)
{
    Tensor* C = new_tensor(A->shape, A->requires_grad, false);
    Op* o = new_op(OpType::MulScalar, {A}, C);
    o->scalar = v;
    o->forward();
    return C;
}

Tensor* Graph::add(Tensor* A, Tensor* B)
{
    if (A->numel() != B->numel()) throw Error(ZNN_ERR_INVALID, "add: sizes differ");
    Tensor* C = new_tensor(A->shape, any_grad({A, B}), false);
    new_op(OpType::Add, {A, B}, C)->forward();
    return C;
}

Tensor* Graph::conv2d(Tensor* A, Tensor* W, Tensor* bias, int pad)
{
    if (A->shape.len != 4 || W->shape.len != 4 || A->shape.dims[1] != W->shape.dims[1])
        throw Error(ZNN_ERR_INVALID, "conv2d: need NCHW input and [Co,Ci,KH,KW] weights with matching Ci");
    const size_t Ho = A->shape.dims[2] + 2 * pad - W->shape.dims[2] + 1;
    const size_t Wo = A->shape.dims[3] + 2 * pad - W->shape.dims[3] + 1;
    Tensor* C = new_tensor(Shape{A->shape.dims[0], W->shape.dims[0], Ho, Wo}, any_grad({A, W, bias}), false);
    Op* o = bias ? new_op(OpType::Conv2D, {A, W, bias}, C) : new_op(OpType::Conv2D, {A, W}, C);
    o->pad = pad;
    o->forward();
    return C;
}

Tensor* Graph::conv2dRelu(Tensor* A, Tensor* W, Tensor* bias, int pad)
{
    if (A->shape.len != 4 || W->shape.len != 4 || A->shape.dims[1] != W->shape.dims[1])
        throw Error(ZNN_ERR_INVALID, "conv2d: need NCHW input and [Co,Ci,KH,KW] weights with matching Ci");
    const size_t Ho = A->shape.dims[2] + 2 * pad - W->shape.dims[2] + 1;
    const size_t Wo = A->shape.dims[3] + 2 * pad - W->shape.dims[3] + 1;
    Tensor* P = new_tensor(Shape{A->shape.dims[0], W->shape.dims[0], Ho, Wo}, any_grad({A, W, bias}), false);
    Op* o = bias ? new_op(OpType::Conv2D, {A, W, bias}, P) : new_op(OpType::Conv2D, {A, W}, P);
    o->pad = pad;
    Tensor* R = new_tensor(P->shape, P->requires_grad, false);
    new_op(OpType::Relu, {P}, R);
    check(znn_conv2d_fwd_act(A->data, W->data, bias ? bias->data : nullptr, R->data, (int)A->shape.dims[0], (int)A->shape.dims[1],
                             (int)A->shape.dims[2], (int)A->shape.dims[3], (int)W->shape.dims[0], (int)W->shape.dims[2],
                             (int)W->shape.dims[3], pad, 1),
          "Conv2D + Relu forward");
    return R;
}

Tensor* Graph::maxpool2d(Tensor* A, int pool, int stride)
{
    if (A->shape.len != 4 || pool <= 0 || stride <= 0) throw Error(ZNN_ERR_INVALID, "maxpool2d: bad arguments");
    Tensor* C = new_tensor(Shape{A->shape.dims[0], A->shape.dims[1], A->shape.dims[2] / stride, A->shape.dims[3] / stride},
                           A->requires_grad, false);
    Op* o = new_op(OpType::MaxPool2D, {A}, C);
    o->pool = pool;
    o->stride = stride;
    o->forward();
    return C;
}

Tensor* Graph::softmax(Tensor* A)
{
    Tensor* C = new_tensor(A->shape, A->requires_grad, false);
    new_op(OpType::Softmax, {A}, C)->forward();
    return C;
}

Tensor* Graph::causalSoftmax(Tensor* S, float scale)
{
    if (S->shape.len < 2 || S->shape.dims[S->shape.len - 1] != S->shape.dims[S->shape.len - 2])
        throw Error(ZNN_ERR_INVALID, "causalSoftmax: the last two dimensions must be equal");
    Tensor* C = new_tensor(S->shape, S->requires_grad, false);
    Op* o = new_op(OpType::CausalSoftmax, {S}, C);
    o->scalar = scale;
    o->forward();
    return C;
}

Tensor* Graph::causalAttention(Tensor* q, Tensor* k, Tensor* v, size_t B, size_t T, size_t nh, float scale)
{
    if (q->shape.len != 2 || !(q->shape == k->shape) || !(q->shape == v->shape) || q->shape.dims[0] != B * T || nh == 0 ||
        q->shape.dims[1] % nh != 0)
        throw Error(ZNN_ERR_INVALID, "causalAttention: need q, k, v of shape [B*T, C] with C a multiple of the head count");
    Tensor* y = new_tensor(q->shape, any_grad({q, k, v}), false);
    Op* o = new_op(OpType::CausalAttention, {q, k, v}, y);
    o->scalar = scale;
    o->att_B = (int)B;
    o->att_T = (int)T;
    o->att_nh = (int)nh;
    o->scratch = (float*)arena_->alloc(B * nh * T * sizeof(float));
    o->forward();
    return y;
}

Tensor* Graph::rmsNorm(Tensor* X, Tensor* G, float eps)
{
    Tensor* Y = new_tensor(X->shape, any_grad({X, G}), false);
    Op* o = new_op(OpType::RmsNorm, {X, G}, Y);
    o->scalar = eps;
    o->forward();
    return Y;
}

Tensor* Graph::layerNorm(Tensor* X, Tensor* G, Tensor* B, float eps)
{
    Tensor* Y = new_tensor(X->shape, any_grad({X, G, B}), false);
    Op* o = new_op(OpType::LayerNorm, {X, G, B}, Y);
    o->scalar = eps;
    o->forward();
    return Y;
}

Tensor* Graph::linear(Tensor* X, Tensor* W, Tensor* bias)
{
    if (X->shape.len < 2 || W->shape.len < 2 || X->shape.dims[1] != W->shape.dims[0] || bias->numel() != W->shape.dims[1])
        throw Error(ZNN_ERR_INVALID, "linear: need X [M,K], W [K,N], bias [N]");
    Tensor* Y = new_tensor(Shape{X->shape.dims[0], W->shape.dims[1]}, any_grad({X, W, bias}), false);
    new_op(OpType::LinearBias, {X, W, bias}, Y)->forward();
    return Y;
}

// distance in floats between consecutive pointers when it is the same, positive and a multiple of 4; else 0
static long long uniform_stride(int n, const float* const* p)
{
    if (n < 2) return 0;
    const long long d = p[1] - p[0];
    if (d <= 0 || (d & 3)) return 0;
    for (int i = 2; i < n; i++)
        if (p[i] - p[i - 1] != d) return 0;
    return d;
}

void Graph::linearGroup(Tensor* X, int n, Tensor* const* W, Tensor* const* bias, Tensor** out)
{
    if (n < 1 || n > 8) throw Error(ZNN_ERR_INVALID, "linearGroup: 1..8 members");
    for (int i = 0; i < n; i++)
        if (X->shape.len < 2 || W[i]->shape.len < 2 || X->shape.dims[1] != W[i]->shape.dims[0] ||
            bias[i]->numel() != W[i]->shape.dims[1] || W[i]->shape.dims[1] != W[0]->shape.dims[1])
            throw Error(ZNN_ERR_INVALID, "linearGroup: need X [M,K] and n times W [K,N], bias [N]");
    const int M = (int)X->shape.dims[0], K = (int)X->shape.dims[1], N = (int)W[0]->shape.dims[1];
    std::vector<Op*> ops;
    for (int i = 0; i < n; i++) {
        out[i] = new_tensor(Shape{X->shape.dims[0], W[i]->shape.dims[1]}, any_grad({X, W[i], bias[i]}), false);
        ops.push_back(new_op(OpType::LinearBias, {X, W[i], bias[i]}, out[i]));
    }
    ops.back()->group = ops;
    int rc = ZNN_ERR_UNSUPPORTED;
    if (g_group_linear && n > 1) {
        const float* w[8]; const float* b[8]; const float* y[8];
        for (int i = 0; i < n; i++) { w[i] = W[i]->data; b[i] = bias[i]->data; y[i] = out[i]->data; }
        const long long sw = uniform_stride(n, w), sb = uniform_stride(n, b), sy = uniform_stride(n, y);
        if (sw && sb && sy)
            rc = znn_sgemm_grouped(ZNN_NO_TRANS, ZNN_NO_TRANS, M, N, K, 1.0f, X->data, K, 0, W[0]->data, N, sw, 0.0f, out[0]->data, N,
                                   sy, n, bias[0]->data, sb, 0);
    }
    if (rc == ZNN_ERR_UNSUPPORTED) {
        for (Op* o : ops) o->forward();
    } else {
        check(rc, "grouped Linear forward");
    }
}

Tensor* Graph::linearAct(Tensor* X, Tensor* W, Tensor* bias, OpType act)
{
    if (act != OpType::Relu && act != OpType::Gelu) throw Error(ZNN_ERR_INVALID, "linearAct: the activation is Relu or Gelu");
    if (X->shape.len < 2 || W->shape.len < 2 || X->shape.dims[1] != W->shape.dims[0] || bias->numel() != W->shape.dims[1])
        throw Error(ZNN_ERR_INVALID, "linear: need X [M,K], W [K,N], bias [N]");
    Tensor* H = new_tensor(Shape{X->shape.dims[0], W->shape.dims[1]}, any_grad({X, W, bias}), false);
    Op* lin = new_op(OpType::LinearBias, {X, W, bias}, H);
    Tensor* A = new_tensor(H->shape, H->requires_grad, false);
    Op* a = new_op(act, {H}, A);
    int rc = ZNN_ERR_UNSUPPORTED;
    if (g_fused_epilogue & (act == OpType::Relu ? 2 : 4))
        rc = znn_linear_fwd_ex(X->data, W->data, bias->data, A->data, H->data, nullptr, (int)X->shape.dims[0],
                               (int)X->shape.dims[1], (int)W->shape.dims[1], act == OpType::Relu ? 1 : 2);
    if (rc == ZNN_ERR_UNSUPPORTED) {   // small or unaligned: the two kernels
        lin->forward();
        a->forward();
    } else {
        check(rc, "Linear + activation forward");
    }
    return A;
}

Tensor* Graph::linearResidual(Tensor* X, Tensor* W, Tensor* bias, Tensor* R)
{
    if (X->shape.len < 2 || W->shape.len < 2 || X->shape.dims[1] != W->shape.dims[0] || bias->numel() != W->shape.dims[1])
        throw Error(ZNN_ERR_INVALID, "linear: need X [M,K], W [K,N], bias [N]");
    if (R->numel() != X->shape.dims[0] * W->shape.dims[1]) throw Error(ZNN_ERR_INVALID, "linearResidual: residual size");
    Tensor* L = new_tensor(Shape{X->shape.dims[0], W->shape.dims[1]}, any_grad({X, W, bias}), false);
    Op* lin = new_op(OpType::LinearBias, {X, W, bias}, L);
    Tensor* S = new_tensor(L->shape, any_grad({R, L}), false);
    Op* add = new_op(OpType::Add, {R, L}, S);
    int rc = ZNN_ERR_UNSUPPORTED;
    if (g_fused_epilogue & 1)   // S = X.W + bias + R in one kernel; L's values are never needed (no backward arm reads them)
        rc = znn_linear_fwd_ex(X->data, W->data, bias->data, S->data, nullptr, R->data, (int)X->shape.dims[0],
                               (int)X->shape.dims[1], (int)W->shape.dims[1], 0);
    if (rc == ZNN_ERR_UNSUPPORTED) {
        lin->forward();
        add->forward();
    } else {
        check(rc, "Linear + residual forward");
    }
    return S;
}

Tensor* Graph::batchMatMul(Tensor* A, Tensor* B, int tri_role)
{
    if (A->shape.len != 4 || B->shape.len != 4 || A->shape.dims[3] != B->shape.dims[2] ||
        A->shape.dims[0] != B->shape.dims[0] || A->shape.dims[1] != B->shape.dims[1])
        throw Error(ZNN_ERR_INVALID, "batchMatMul: need [b,h,M,K] x [b,h,K,N]");
    Tensor* C = new_tensor(Shape{A->shape.dims[0], A->shape.dims[1], A->shape.dims[2], B->shape.dims[3]},
                           any_grad({A, B}), false);
    if (tri_role != 0 && (tri_role < 0 || tri_role > 2 || A->shape.dims[2] != (tri_role == 1 ? B->shape.dims[3] : A->shape.dims[3])))
        throw Error(ZNN_ERR_INVALID, "batchMatMul: a causal role needs square scores");
    Op* op = new_op(OpType::BatchMatMul, {A, B}, C);
    op->tri_role = tri_role;
    if (tri_role == 2 && A->requires_grad)
        op->scratch = (float*)arena_->alloc(A->shape.dims[0] * A->shape.dims[1] * A->shape.dims[2] * sizeof(float));
    op->forward();
    return C;
}

Tensor* Graph::batchMatMulNT(Tensor* A, Tensor* B, int tri_role)
{
    if (A->shape.len != 4 || B->shape.len != 4 || A->shape.dims[3] != B->shape.dims[3] ||
        A->shape.dims[0] != B->shape.dims[0] || A->shape.dims[1] != B->shape.dims[1])
        throw Error(ZNN_ERR_INVALID, "batchMatMulNT: need [b,h,M,K] x [b,h,N,K]");
    if (tri_role != 0 && (tri_role != 1 || A->shape.dims[2] != B->shape.dims[2]))
        throw Error(ZNN_ERR_INVALID, "batchMatMulNT: the causal role needs square scores");
    Tensor* C = new_tensor(Shape{A->shape.dims[0], A->shape.dims[1], A->shape.dims[2], B->shape.dims[2]},
                           any_grad({A, B}), false);
    Op* op = new_op(OpType::BatchMatMulNT, {A, B}, C);
    op->tri_role = tri_role;
    op->forward();
    return C;
}

Tensor* Graph::embedding(Tensor* W, Tensor* X)
{
    if (W->shape.len != 2 || X->shape.len != 2) throw Error(ZNN_ERR_INVALID, "embedding: W [V,D], ids [B,T]");
    Tensor* Y = new_tensor(Shape{X->shape.dims[0], X->shape.dims[1], W->shape.dims[1]}, W->requires_grad, false);
    new_op(OpType::Embedding, {W, X}, Y)->forward();
    return Y;
}

// ---------------------------------------------------------------- Op arms
static int64_t* dims64(const Shape& s, int64_t* buf)
{
    for (size_t i = 0; i < s.len; i++) buf[i] = (int64_t)s.dims[i];
    return buf;
}

void Op::forward()
{
    Tensor* A = inputs[0];
    Tensor* C = outputs[0];
    switch (type) {
    case OpType::MatMul: {
        Tensor* B = inputs[1];
        const int M = (int)A->shape.dims[0], K = (int)A->shape.dims[1], N = (int)B->shape.dims[1];
        check(znn_sgemm(ZNN_ROW_MAJOR, ZNN_NO_TRANS, ZNN_NO_TRANS, M, N, K, 1.0f, A->data, K, B->data, N, 0.0f, C->data, N),
              "MatMul forward");
        break;
    }
    case OpType::AddBias:
        check(znn_add_bias_fwd(A->data, inputs[1]->data, C->data, (int)A->shape.dims[0], (int)A->shape.dims[1]), "AddBias forward");
        break;
    case OpType::Relu: check(znn_relu_fwd(A->data, C->data, A->numel()), "Relu forward"); break;
    case OpType::Gelu: check(znn_gelu_fwd(A->data, C->data, A->numel()), "Gelu forward"); break;
    case OpType::SoftmaxCrossEntropy:
        check(targets_u8 ? znn_softmax_xent_fwd_u8(A->data, reinterpret_cast<const uint8_t*>(targets), probs, C->data,
                                                   (int)A->shape.dims[0], (int)A->shape.dims[1])
                         : znn_softmax_xent_fwd(A->data, targets, probs, C->data, (int)A->shape.dims[0], (int)A->shape.dims[1]),
              "SoftmaxCrossEntropy forward");
        break;
    case OpType::Reshape: break;  // aliased data (autodiff.zig:272-275)
    case OpType::Transpose: {
        int64_t d[8];
        check(znn_transpose_fwd(A->data, C->data, dims64(A->shape, d), (int)A->shape.len, dim0, dim1), "Transpose forward");
        break;
    }
    case OpType::MulScalar: check(znn_mul_scalar_fwd(A->data, scalar, C->data, A->numel()), "MulScalar forward"); break;
    case OpType::Add: check(znn_add_fwd(A->data, inputs[1]->data, C->data, A->numel()), "Add forward"); break;
    case OpType::Conv2D: {
        Tensor* W = inputs[1];
        const float* b = inputs.size() > 2 ? inputs[2]->data : nullptr;
        check(znn_conv2d_fwd(A->data, W->data, b, C->data, (int)A->shape.dims[0], (int)A->shape.dims[1], (int)A->shape.dims[2],
                             (int)A->shape.dims[3], (int)W->shape.dims[0], (int)W->shape.dims[2], (int)W->shape.dims[3], pad),
              "Conv2D forward");
        break;
    }
    case OpType::MaxPool2D:
        check(znn_maxpool2d_fwd(A->data, C->data, nullptr, (int)A->shape.dims[0], (int)A->shape.dims[1], (int)A->shape.dims[2],
                                (int)A->shape.dims[3], pool, stride),
              "MaxPool2D forward");
        break;
    case OpType::Softmax: {
        const int D = (int)A->shape.dims[A->shape.len - 1];
        check(znn_softmax_fwd(A->data, C->data, A->numel() / D, D), "Softmax forward");
        break;
    }
    case OpType::CausalSoftmax: {
        const int T = (int)A->shape.dims[A->shape.len - 1];
        check(znn_causal_softmax_fwd(A->data, scalar, C->data, (int)(A->numel() / ((size_t)T * T)), T), "CausalSoftmax forward");
        break;
    }
    case OpType::RmsNorm: {
        const int D = (int)A->shape.dims[A->shape.len - 1];
        check(znn_rmsnorm_fwd(A->data, inputs[1]->data, scalar, C->data, A->numel() / D, D), "RmsNorm forward");
        break;
    }
    case OpType::LayerNorm: {
        const int D = (int)A->shape.dims[A->shape.len - 1];
        check(znn_layernorm_fwd(A->data, inputs[1]->data, inputs[2]->data, scalar, C->data, A->numel() / D, D), "LayerNorm forward");
        break;
    }
    case OpType::LinearBias: {
        Tensor* W = inputs[1];
        check(znn_linear_fwd(A->data, W->data, inputs[2]->data, C->data, (int)A->shape.dims[0], (int)A->shape.dims[1],
                             (int)W->shape.dims[1]),
              "Linear forward");
        break;
    }
    case OpType::BatchMatMul: {
        Tensor* B = inputs[1];
        const int nb = (int)(A->shape.dims[0] * A->shape.dims[1]);
        const int M = (int)A->shape.dims[2], K = (int)A->shape.dims[3], N = (int)B->shape.dims[3];
        const int tri = tri_role == 1 ? ZNN_TRI_C_LOWER : tri_role == 2 ? ZNN_TRI_A_LOWER : ZNN_TRI_NONE;
        check(znn_sgemm_batched_strided_tri(ZNN_NO_TRANS, ZNN_NO_TRANS, M, N, K, 1.0f, A->data, K, (long long)M * K, B->data,
                                            N, (long long)K * N, 0.0f, C->data, N, (long long)M * N, nb, tri),
              "BatchMatMul forward");
        break;
    }
    case OpType::BatchMatMulNT: {
        Tensor* B = inputs[1];
        const int nb = (int)(A->shape.dims[0] * A->shape.dims[1]);
        const int M = (int)A->shape.dims[2], K = (int)A->shape.dims[3], N = (int)B->shape.dims[2];
        check(znn_sgemm_batched_strided_tri(ZNN_NO_TRANS, ZNN_TRANS, M, N, K, 1.0f, A->data, K, (long long)M * K, B->data, K,
                                            (long long)N * K, 0.0f, C->data, N, (long long)M * N, nb,
                                            tri_role == 1 ? ZNN_TRI_C_LOWER : ZNN_TRI_NONE),
              "BatchMatMulNT forward");
        break;
    }
    case OpType::Embedding: {
        Tensor* W = inputs[0];
        Tensor* X = inputs[1];
        check(znn_embedding_fwd(W->data, X->data, C->data, X->numel(), (int)W->shape.dims[1], (int)W->shape.dims[0]),
              "Embedding forward");
        break;
    }
    case OpType::CausalAttention: {
        const long long Cw = (long long)A->shape.dims[1], hs = Cw / att_nh;
        check(znn_attn_fwd(A->data, inputs[1]->data, inputs[2]->data, C->data, scratch, att_B, att_nh, att_T, (int)hs, Cw, hs,
                           (long long)att_T * Cw, scalar),
              "CausalAttention forward");
        break;
    }
    }
}

void Op::backward()
{
    Tensor* A = inputs[0];
    Tensor* C = outputs[0];
    if (skip_backward) {   // the consumer's fused backward already produced this op's input gradient
        skip_backward = false;
        return;
    }
    // the upstream gradient is read: zero if no consumer wrote it
    ensure_grad(C);
    // arms that only add need a defined buffer; the GEMM arms below overwrite a fresh one instead (beta = 0)
    // (so do Gelu, CausalSoftmax, Add, MulScalar, Reshape and Transpose, with a storing kernel or a plain copy)
    const bool can_store = type == OpType::MatMul || type == OpType::BatchMatMul || type == OpType::BatchMatMulNT ||
                           type == OpType::LinearBias || type == OpType::CausalAttention ||
                           type == OpType::Gelu || type == OpType::CausalSoftmax || type == OpType::Add ||
                           type == OpType::MulScalar || type == OpType::Reshape || type == OpType::Transpose;
    if (!can_store)
        for (Tensor* in : inputs) ensure_grad(in);
    switch (type) {
    case OpType::MatMul: {
        Tensor* B = inputs[1];
        const int M = (int)A->shape.dims[0], K = (int)A->shape.dims[1], N = (int)B->shape.dims[1];
        if (A->requires_grad) {  // dA += dC . B^T (autodiff.zig:602-620)
            const float beta = claim_grad_overwrite(A) ? 0.0f : 1.0f;
            check(znn_sgemm(ZNN_ROW_MAJOR, ZNN_NO_TRANS, ZNN_TRANS, M, K, N, 1.0f, C->grad, N, B->data, N, beta, A->grad, K),
                  "MatMul backward dA");
        }
        if (B->requires_grad) {  // dB += A^T . dC (:623-640)
            const float beta = claim_grad_overwrite(B) ? 0.0f : 1.0f;
            check(znn_sgemm(ZNN_ROW_MAJOR, ZNN_TRANS, ZNN_NO_TRANS, K, N, M, 1.0f, A->data, K, C->grad, N, beta, B->grad, N),
                  "MatMul backward dB");
        }
        break;
    }
    case OpType::AddBias:
        check(znn_add_bias_bwd(C->grad, A->requires_grad ? A->grad : nullptr, inputs[1]->requires_grad ? inputs[1]->grad : nullptr,
                               (int)A->shape.dims[0], (int)A->shape.dims[1]),
              "AddBias backward");
        break;
    case OpType::Relu:
        // the mask is read from the output (max(0, a) > 0 exactly where a > 0): a fused producer need not keep a
        if (A->requires_grad) check(znn_relu_bwd(C->data, C->grad, A->grad, A->numel()), "Relu backward");
        break;
    case OpType::Gelu:
        if (A->requires_grad) {
            if (claim_grad_overwrite(A)) check(znn_gelu_bwd_set(A->data, C->grad, A->grad, A->numel()), "Gelu backward");
            else check(znn_gelu_bwd(A->data, C->grad, A->grad, A->numel()), "Gelu backward");
        }
        break;
    case OpType::SoftmaxCrossEntropy:
        // ignores loss.grad and has no requires_grad gate, as the reference (:758-774); a logits
        // tensor without a grad buffer simply has nothing to receive it
        if (A->grad)
            check(targets_u8 ? znn_softmax_xent_bwd_u8(probs, reinterpret_cast<const uint8_t*>(targets), A->grad,
                                                       (int)A->shape.dims[0], (int)A->shape.dims[1])
                             : znn_softmax_xent_bwd(probs, targets, A->grad, (int)A->shape.dims[0], (int)A->shape.dims[1]),
                  "SoftmaxCrossEntropy backward");
        break;
    case OpType::Reshape:
        if (A->requires_grad && C->grad != A->grad) {
            if (claim_grad_overwrite(A)) check(znn_memcpy_d2d(A->grad, C->grad, A->numel() * sizeof(float)), "Reshape backward");
            else check(znn_accumulate(C->grad, A->grad, A->numel()), "Reshape backward");
        }
        break;
    case OpType::Transpose:
        if (A->requires_grad) {
            int64_t d[8];
            if (claim_grad_overwrite(A))   // a fresh gradient: the transpose of dC back, stored
                check(znn_transpose_fwd(C->grad, A->grad, dims64(C->shape, d), (int)C->shape.len, dim0, dim1), "Transpose backward");
            else
                check(znn_transpose_bwd(C->grad, A->grad, dims64(A->shape, d), (int)A->shape.len, dim0, dim1), "Transpose backward");
        }
        break;
    case OpType::MulScalar:
        if (A->requires_grad) {
            if (claim_grad_overwrite(A)) check(znn_mul_scalar_fwd(C->grad, scalar, A->grad, A->numel()), "MulScalar backward");
            else check(znn_mul_scalar_bwd(C->grad, scalar, A->grad, A->numel()), "MulScalar backward");
        }
        break;
    case OpType::Add:
        for (Tensor* in : {A, inputs[1]}) {
            if (!in->requires_grad) continue;
            if (claim_grad_overwrite(in)) check(znn_memcpy_d2d(in->grad, C->grad, A->numel() * sizeof(float)), "Add backward");
            else check(znn_accumulate(C->grad, in->grad, A->numel()), "Add backward");
        }
        break;
    case OpType::Conv2D: {
        Tensor* W = inputs[1];
        Tensor* b = inputs.size() > 2 ? inputs[2] : nullptr;
        check(znn_conv2d_bwd(A->data, W->data, C->grad, A->requires_grad ? A->grad : nullptr, W->requires_grad ? W->grad : nullptr,
                             (b && b->requires_grad) ? b->grad : nullptr, (int)A->shape.dims[0], (int)A->shape.dims[1],
                             (int)A->shape.dims[2], (int)A->shape.dims[3], (int)W->shape.dims[0], (int)W->shape.dims[2],
                             (int)W->shape.dims[3], pad),
              "Conv2D backward");
        break;
    }
    case OpType::MaxPool2D:
        if (A->requires_grad) {
            // the pool's input is a Relu output nobody else reads: the winner's gradient goes straight to the Relu's
            // input, masked by the sign, and the Relu's own backward is skipped
            Op* prod = A->creator;
            if ((g_fused_epilogue & 2) && prod && prod->type == OpType::Relu && A->consumers == 1 && prod->inputs[0]->requires_grad &&
                prod->inputs[0]->grad && grad_is_fresh(A)) {
                Tensor* P = prod->inputs[0];
                ensure_grad(P);
                check(znn_maxpool2d_bwd_relu(A->data, C->grad, P->grad, (int)A->shape.dims[0], (int)A->shape.dims[1],
                                             (int)A->shape.dims[2], (int)A->shape.dims[3], pool, stride),
                      "MaxPool2D + Relu backward");
                prod->skip_backward = true;
                break;
            }
            check(znn_maxpool2d_bwd(A->data, C->grad, A->grad, (int)A->shape.dims[0], (int)A->shape.dims[1], (int)A->shape.dims[2],
                                    (int)A->shape.dims[3], pool, stride),
                  "MaxPool2D backward");
        }
        break;
    case OpType::Softmax:
        if (A->requires_grad) {
            const int D = (int)A->shape.dims[A->shape.len - 1];
            check(znn_softmax_bwd(C->data, C->grad, A->grad, A->numel() / D, D), "Softmax backward");
        }
        break;
    case OpType::CausalSoftmax:
        if (A->requires_grad) {
            const int T = (int)A->shape.dims[A->shape.len - 1];
            if (claim_grad_overwrite(A))
                check(znn_causal_softmax_bwd_set(C->data, C->grad, scalar, A->grad, (int)(A->numel() / ((size_t)T * T)), T),
                      "CausalSoftmax backward");
            else
                check(znn_causal_softmax_bwd(C->data, C->grad, scalar, A->grad, (int)(A->numel() / ((size_t)T * T)), T),
                      "CausalSoftmax backward");
        }
        break;
    case OpType::RmsNorm: {
        Tensor* G = inputs[1];
        const int D = (int)A->shape.dims[A->shape.len - 1];
        check(znn_rmsnorm_bwd(A->data, G->data, C->grad, scalar, A->requires_grad ? A->grad : nullptr,
                              G->requires_grad ? G->grad : nullptr, A->numel() / D, D),
              "RmsNorm backward");
        break;
    }
    case OpType::LayerNorm: {
        Tensor* G = inputs[1];
        Tensor* B = inputs[2];
        const int D = (int)A->shape.dims[A->shape.len - 1];
        check(znn_layernorm_bwd(A->data, G->data, C->grad, scalar, A->requires_grad ? A->grad : nullptr,
                                G->requires_grad ? G->grad : nullptr, B->requires_grad ? B->grad : nullptr, A->numel() / D, D),
              "LayerNorm backward");
        break;
    }
    case OpType::LinearBias: {
        Tensor* W = inputs[1];
        Tensor* b = inputs[2];
        const int M = (int)A->shape.dims[0], K = (int)A->shape.dims[1], N = (int)W->shape.dims[1];
        if (g_group_linear && group.size() > 1) {
            // Last member of a group on one input (the tape runs it first): every member's output gradient is complete
            // by now, so all weight gradients run as one grouped launch and the data gradients as one product whose
            // contraction runs through the members; the other members' own backward is then skipped.
            const int n = (int)group.size();
            const float* w[8]; const float* wg[8]; const float* yg[8];
            bool ok = n <= 8 && A->requires_grad;
            // "complete" holds when one op reads all the outputs and nothing else does: it ran before any member
            // (with separate consumers the tape may still owe a member's output gradient when the last member runs)
            for (int i = 0; i < n && ok; i++)
                ok = group[i]->outputs[0]->consumers == 1 && group[i]->outputs[0]->last_consumer == group[0]->outputs[0]->last_consumer;
            for (int i = 0; i < n && ok; i++) {
                Op* o = group[i];
                ensure_grad(o->outputs[0]);
                ok = o->inputs[1]->requires_grad && o->inputs[2]->requires_grad && !grad_is_fresh(o->inputs[1]);
                w[i] = o->inputs[1]->data; wg[i] = o->inputs[1]->grad; yg[i] = o->outputs[0]->grad;
            }
            const long long sw = ok ? uniform_stride(n, w) : 0, swg = ok ? uniform_stride(n, wg) : 0, syg = ok ? uniform_stride(n, yg) : 0;
            if (ok && sw && swg && syg) {
                const bool fresh = grad_is_fresh(A);
                int rc = znn_sgemm_grouped(ZNN_NO_TRANS, ZNN_TRANS, M, K, N, 1.0f, yg[0], N, syg, w[0], N, sw, fresh ? 0.0f : 1.0f,
                                           A->grad, K, 0, n, nullptr, 0, 1);
                if (rc == ZNN_OK) {
                    mark_grad_written(A);
                    rc = znn_sgemm_grouped(ZNN_TRANS, ZNN_NO_TRANS, K, N, M, 1.0f, A->data, K, 0, yg[0], N, syg, 1.0f,
                                           const_cast<float*>(wg[0]), N, swg, n, nullptr, 0, 0);
                    for (int i = 0; i < n; i++) {
                        Op* o = group[i];
                        ensure_grad(o->inputs[2]);
                        check(znn_add_bias_bwd(yg[i], nullptr, o->inputs[2]->grad, M, N), "Linear backward dbias");
                        if (rc == ZNN_ERR_UNSUPPORTED)
                            check(znn_sgemm(ZNN_ROW_MAJOR, ZNN_TRANS, ZNN_NO_TRANS, K, N, M, 1.0f, A->data, K, yg[i], N, 1.0f,
                                            o->inputs[1]->grad, N),
                                  "Linear backward dW");
                        if (o != this) o->skip_backward = true;
                    }
                    if (rc != ZNN_ERR_UNSUPPORTED) check(rc, "grouped Linear backward dW");
                    break;
                }
                if (rc != ZNN_ERR_UNSUPPORTED) check(rc, "grouped Linear backward dX");
            }
        }
        // znn_linear_bwd in pieces, so that a fresh dX is overwritten (beta = 0) instead of zero-filled and added to
        if (b->requires_grad) {
            ensure_grad(b);
            check(znn_add_bias_bwd(C->grad, nullptr, b->grad, M, N), "Linear backward dbias");
        }
        if (A->requires_grad) {
            // X = act(H) read by this op alone: the activation's derivative rides in the epilogue of dY.W^T, the result
            // is the gradient of H and the activation op's own backward is skipped
            Op* prod = A->creator;
            bool fused = false;
            if (prod && (prod->type == OpType::Relu ? (g_fused_epilogue & 2) : prod->type == OpType::Gelu ? (g_fused_epilogue & 8) : 0) &&
                A->consumers == 1 &&
                prod->inputs[0]->requires_grad && prod->inputs[0]->grad && grad_is_fresh(A)) {
                Tensor* H = prod->inputs[0];
                const int rc = znn_linear_bwd_ex(A->data, W->data, C->grad, H->grad, nullptr, nullptr, M, K, N, H->data,
                                                 prod->type == OpType::Relu ? 1 : 2, grad_is_fresh(H) ? 1 : 0);
                if (rc == ZNN_OK) {
                    mark_grad_written(H);
                    prod->skip_backward = true;
                    fused = true;
                } else if (rc != ZNN_ERR_UNSUPPORTED) {
                    check(rc, "Linear backward dX with the activation gradient");
                }
            }
            if (!fused) {
                const float beta = claim_grad_overwrite(A) ? 0.0f : 1.0f;
                check(znn_sgemm(ZNN_ROW_MAJOR, ZNN_NO_TRANS, ZNN_TRANS, M, K, N, 1.0f, C->grad, N, W->data, N, beta, A->grad, K),
                      "Linear backward dX");
            }
        }
        if (W->requires_grad) {
            const float beta = claim_grad_overwrite(W) ? 0.0f : 1.0f;
            check(znn_sgemm(ZNN_ROW_MAJOR, ZNN_TRANS, ZNN_NO_TRANS, K, N, M, 1.0f, A->data, K, C->grad, N, beta, W->grad, N),
                  "Linear backward dW");
        }
        break;
    }
    case OpType::BatchMatMul: {
        Tensor* B = inputs[1];
        const int nb = (int)(A->shape.dims[0] * A->shape.dims[1]);
        const int M = (int)A->shape.dims[2], K = (int)A->shape.dims[3], N = (int)B->shape.dims[3];
        // role 1: C->grad = dS is lower-triangular (left operand of dA, right operand of dB);
        // role 2: A->grad = dP is read below the diagonal only, and A^T = P^T is upper-triangular
        const int tri_da = tri_role == 1 ? ZNN_TRI_A_LOWER : tri_role == 2 ? ZNN_TRI_C_LOWER : ZNN_TRI_NONE;
        const int tri_db = tri_role == 1 ? ZNN_TRI_B_LOWER : tri_role == 2 ? ZNN_TRI_A_UPPER : ZNN_TRI_NONE;
        // Role 2 with the probabilities coming straight from a CausalSoftmax whose input gradient is still fresh: produce
        // the gradient of the scores in the epilogue of dO.V^T (znn_attn_dscores); dP is never written and the softmax's
        // own backward is skipped.  (Role 2 asserts that the probabilities have no other consumer.)
        bool fused_done = false;
        if (tri_role == 2 && g_fused_softmax_bwd && scratch && A->requires_grad && A->creator &&
            A->creator->type == OpType::CausalSoftmax && grad_is_fresh(A)) {
            Op* sm = A->creator;
            Tensor* S = sm->inputs[0];
            if (S->requires_grad && grad_is_fresh(S)) {
                check(znn_rowdot(C->grad, C->data, scratch, (size_t)nb * M, N), "attention D vector");
                const int rc = znn_attn_dscores(C->grad, B->data, A->data, scratch, sm->scalar, S->grad, M, N, nb);
                if (rc == ZNN_OK) {
                    claim_grad_overwrite(S);
                    sm->skip_backward = true;
                    fused_done = true;
                } else if (rc != ZNN_ERR_UNSUPPORTED) {
                    check(rc, "fused attention score gradient");
                }
            }
        }
        if (A->requires_grad && !fused_done) {
            // (with ZNN_TRI_C_LOWER a fresh dP keeps undefined values above the diagonal, where nobody reads)
            const float beta = claim_grad_overwrite(A) ? 0.0f : 1.0f;
            check(znn_sgemm_batched_strided_tri(ZNN_NO_TRANS, ZNN_TRANS, M, K, N, 1.0f, C->grad, N, (long long)M * N, B->data,
                                                N, (long long)K * N, beta, A->grad, K, (long long)M * K, nb, tri_da),
                  "BatchMatMul backward dA");
        }
        if (B->requires_grad) {
            const float beta = claim_grad_overwrite(B) ? 0.0f : 1.0f;
            check(znn_sgemm_batched_strided_tri(ZNN_TRANS, ZNN_NO_TRANS, K, N, M, 1.0f, A->data, K, (long long)M * K, C->grad,
                                                N, (long long)M * N, beta, B->grad, N, (long long)K * N, nb, tri_db),
                  "BatchMatMul backward dB");
        }
        break;
    }
    case OpType::BatchMatMulNT: {
        // C = A.B^T  =>  dA += dC.B (left operand dC lower-triangular when C are causal scores),
        //                dB += dC^T.A (left operand dC^T upper-triangular)
        Tensor* B = inputs[1];
        const int nb = (int)(A->shape.dims[0] * A->shape.dims[1]);
        const int M = (int)A->shape.dims[2], K = (int)A->shape.dims[3], N = (int)B->shape.dims[2];
        if (A->requires_grad) {
            const float beta = claim_grad_overwrite(A) ? 0.0f : 1.0f;
            check(znn_sgemm_batched_strided_tri(ZNN_NO_TRANS, ZNN_NO_TRANS, M, K, N, 1.0f, C->grad, N, (long long)M * N, B->data,
                                                K, (long long)N * K, beta, A->grad, K, (long long)M * K, nb,
                                                tri_role == 1 ? ZNN_TRI_A_LOWER : ZNN_TRI_NONE),
                  "BatchMatMulNT backward dA");
        }
        if (B->requires_grad) {
            const float beta = claim_grad_overwrite(B) ? 0.0f : 1.0f;
            check(znn_sgemm_batched_strided_tri(ZNN_TRANS, ZNN_NO_TRANS, N, K, M, 1.0f, C->grad, N, (long long)M * N, A->data,
                                                K, (long long)M * K, beta, B->grad, K, (long long)N * K, nb,
                                                tri_role == 1 ? ZNN_TRI_A_UPPER : ZNN_TRI_NONE),
                  "BatchMatMulNT backward dB");
        }
        break;
    }
    case OpType::Embedding: {
        Tensor* W = inputs[0];
        Tensor* X = inputs[1];
        if (W->requires_grad)
            check(znn_embedding_bwd(X->data, C->grad, W->grad, X->numel(), (int)W->shape.dims[1], (int)W->shape.dims[0]),
                  "Embedding backward");
        break;
    }
    case OpType::CausalAttention: {
        Tensor* Kt = inputs[1];
        Tensor* Vt = inputs[2];
        const long long Cw = (long long)A->shape.dims[1], hs = Cw / att_nh;
        // one store/add switch for the three gradients: store when every wanted buffer is still untouched
        bool fresh = true;
        for (Tensor* t : inputs)
            if (t->requires_grad && !grad_is_fresh(t)) fresh = false;
        for (Tensor* t : inputs) {
            if (!t->requires_grad) continue;
            if (fresh) mark_grad_written(t);
            else ensure_grad(t);
        }
        check(znn_attn_bwd(A->data, Kt->data, Vt->data, C->data, C->grad, scratch, A->requires_grad ? A->grad : nullptr,
                           Kt->requires_grad ? Kt->grad : nullptr, Vt->requires_grad ? Vt->grad : nullptr, att_B, att_nh, att_T,
                           (int)hs, Cw, hs, (long long)att_T * Cw, scalar, fresh ? 0 : 1),
              "CausalAttention backward");
        break;
    }
    }
}

// ---------------------------------------------------------------- sweeps
static void topo(Tensor* node, std::unordered_set<Tensor*>& seen, std::vector<Tensor*>& out)
{
    // iterative DFS post-order, inputs visited in order (autodiff.zig:2239-2249)
    struct Frame { Tensor* t; size_t next; };
    std::vector<Frame> stack;
    if (!seen.insert(node).second) return;
    stack.push_back({node, 0});
    while (!stack.empty()) {
        Frame& f = stack.back();
        Op* op = f.t->creator;
        if (op && f.next < op->inputs.size()) {
            Tensor* in = op->inputs[f.next++];
            if (seen.insert(in).second) stack.push_back({in, 0});
        } else {
            out.push_back(f.t);
            stack.pop_back();
        }
    }
}

void Graph::sweep(Tensor* root, const std::function<void(Op*)>* after_op)
{
    std::unordered_set<Tensor*> seen;
    std::vector<Tensor*> order;
    topo(root, seen, order);
    for (size_t i = order.size(); i > 0;) {
        i--;
        Op* op = order[i]->creator;
        if (op) {
            op->backward();
            if (after_op) (*after_op)(op);
        }
    }
}

void Graph::backward(Tensor* loss, const std::function<void(Op*)>* after_op)
{
    if (!loss->grad) throw Error(ZNN_ERR_INVALID, "backward: the loss tensor has no gradient buffer");
    ensure_grad(loss);
    check(znn_fill(loss->grad, 1.0f, 1), "seed loss gradient");  // loss.grad[0] = 1 (autodiff.zig:2203)
    sweep(loss, after_op);
}

void Graph::backwardWithGrad(Tensor* out, const std::function<void(Op*)>* after_op) { sweep(out, after_op); }

void Graph::forward()
{
    for (Op* o : ops_) o->forward();
}

void Graph::zeroGrad()
{
    for (Tensor* t : tensors_)
        if (t->grad) {
            check(znn_memset(t->grad, 0, t->numel() * sizeof(float)), "znn_memset");
            mark_grad_written(t);
        }
}

size_t Graph::op_index(const Op* op) const
{
    for (size_t i = 0; i < ops_.size(); i++)
        if (ops_[i] == op) return i;
    return (size_t)-1;
}

}  // namespace host
}  // namespace znn
