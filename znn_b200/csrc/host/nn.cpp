// Modules, models and optimizer of the host mirror: see nn.hpp.
#include "nn.hpp"

#include <math.h>

#include "../../../include/znn_cuda.h"

namespace znn {
namespace host {

// ---------------------------------------------------------------- ParamStore
ParamStore::~ParamStore()
{
    for (ParamInfo& p : params_) delete p.tensor;
    if (w_) znn_free(w_);
    if (g_) znn_free(g_);
    if (v_) znn_free(v_);
    if (v2_) znn_free(v2_);
}

Tensor* ParamStore::add(const std::string& name, const Shape& shape, size_t fan_in)
{
    if (w_) throw Error(ZNN_ERR_INVALID, "ParamStore::add after finalize");
    Tensor* t = new Tensor();
    t->shape = shape;
    t->strides = contiguous_strides(shape);
    t->requires_grad = true;
    params_.push_back(ParamInfo{name, t, total_, fan_in});
    // keep every parameter 16-byte aligned inside the slabs (vector loads, TMA rules)
    total_ += (shape.numel() + 3) & ~(size_t)3;
    return t;
}

void ParamStore::finalize()
{
    if (w_) return;
    const size_t bytes = total_ * sizeof(float);
    void* p = nullptr;
    check(znn_malloc(&p, bytes), "ParamStore values");
    w_ = (float*)p;
    check(znn_malloc(&p, bytes), "ParamStore grads");
    g_ = (float*)p;
    check(znn_malloc(&p, bytes), "ParamStore velocities");
    v_ = (float*)p;
    check(znn_memset(w_, 0, bytes), "znn_memset");
    check(znn_memset(g_, 0, bytes), "znn_memset");
    check(znn_memset(v_, 0, bytes), "znn_memset");
    for (ParamInfo& pi : params_) {
        pi.tensor->data = w_ + pi.offset;
        pi.tensor->grad = g_ + pi.offset;
    }
}

float* ParamStore::second_moments()
{
    if (!v2_ && w_) {
        void* p = nullptr;
        check(znn_malloc(&p, total_ * sizeof(float)), "ParamStore second moments");
        v2_ = (float*)p;
        check(znn_memset(v2_, 0, total_ * sizeof(float)), "znn_memset");
    }
    return v2_;
}

void ParamStore::zeroGrad()
{
    if (g_) check(znn_memset(g_, 0, total_ * sizeof(float)), "zeroGrad");
}

// ---------------------------------------------------------------- modules
Linear::Linear(ParamStore& ps, const std::string& name, size_t in_features, size_t out_features)
{
    weight = ps.add(name + ".weight", Shape{in_features, out_features}, in_features);
    bias = ps.add(name + ".bias", Shape{1, out_features}, 0);
}

static bool g_fused_qkt = true;
void set_fused_qkt(bool on) { g_fused_qkt = on; }
bool fused_qkt() { return g_fused_qkt; }

static bool g_causal_skip = true;
void set_causal_skip(bool on) { g_causal_skip = on; }
bool causal_skip() { return g_causal_skip; }

static bool g_fused_attention = true;
void set_fused_attention(bool on) { g_fused_attention = on; }
bool fused_attention() { return g_fused_attention; }

static bool g_fused_linear = true;
void set_fused_linear(bool on) { g_fused_linear = on; }
bool fused_linear() { return g_fused_linear; }

Tensor* Linear::forward(Graph& g, Tensor* x) const
{
    if (g_fused_linear) return g.linear(x, weight, bias);
    return g.addBias(g.matmul(x, weight), bias);
}

Tensor* Linear::forward_act(Graph& g, Tensor* x, OpType act) const
{
    if (g_fused_linear && (fused_epilogue() & (act == OpType::Relu ? 2 : 4))) return g.linearAct(x, weight, bias, act);
    Tensor* h = forward(g, x);
    return act == OpType::Relu ? g.relu(h) : g.gelu(h);
}

Tensor* Linear::forward_residual(Graph& g, Tensor* x, Tensor* r) const
{
    if (g_fused_linear && (fused_epilogue() & 1)) return g.linearResidual(x, weight, bias, r);
    return g.add(r, forward(g, x));
}

Conv2D::Conv2D(ParamStore& ps, const std::string& name, size_t in_ch, size_t out_ch, size_t k, int pad_) : pad(pad_)
{
    weight = ps.add(name + ".weight", Shape{out_ch, in_ch, k, k}, in_ch * k * k);
    bias = ps.add(name + ".bias", Shape{out_ch}, 0);
}

Tensor* Conv2D::forward(Graph& g, Tensor* x) const { return g.conv2d(x, weight, bias, pad); }

Tensor* Conv2D::forward_relu(Graph& g, Tensor* x) const
{
    if (fused_epilogue() & 2) return g.conv2dRelu(x, weight, bias, pad);
    return g.relu(g.conv2d(x, weight, bias, pad));
}

Embedding::Embedding(ParamStore& ps, const std::string& name, size_t vocab, size_t dim)
{
    weight = ps.add(name + ".weight", Shape{vocab, dim}, dim);  // fan_in = n_embd (nn.zig:520)
}

Tensor* Embedding::forward(Graph& g, Tensor* ids) const { return g.embedding(weight, ids); }

RMSNorm::RMSNorm(ParamStore& ps, const std::string& name, size_t dim, float eps_) : eps(eps_)
{
    weight = ps.add(name + ".weight", Shape{dim}, 0);
}

Tensor* RMSNorm::forward(Graph& g, Tensor* x) const { return g.rmsNorm(x, weight, eps); }

MLP::MLP(ParamStore& ps, const std::string& name, size_t dim, size_t hidden)
    : c_fc(ps, name + ".c_fc", dim, hidden), c_proj(ps, name + ".c_proj", hidden, dim)
{
}

Tensor* MLP::forward(Graph& g, Tensor* x, Tensor* residual) const
{
    // src/nn.zig:638-685 (and the residual add of :1016-1020 when the caller hands it in)
    const bool is_3d = (x->shape.len == 3);
    Tensor* x_2d = x;
    if (is_3d) x_2d = g.reshape(x, Shape{x->shape.dims[0] * x->shape.dims[1], x->shape.dims[2]});
    Tensor* a1 = c_fc.forward_act(g, x_2d, OpType::Gelu);
    Tensor* h2;
    if (residual) {
        Tensor* r_2d = residual->shape.len == 2 ? residual : g.reshape(residual, x_2d->shape);
        h2 = c_proj.forward_residual(g, a1, r_2d);
    } else {
        h2 = c_proj.forward(g, a1);
    }
    if (is_3d) return g.reshape(h2, x->shape);
    return h2;
}

CausalSelfAttention::CausalSelfAttention(ParamStore& ps, const std::string& name, size_t n_embd_, size_t n_head_)
    : q_attn(ps, name + ".q_attn", n_embd_, n_embd_), k_attn(ps, name + ".k_attn", n_embd_, n_embd_),
      v_attn(ps, name + ".v_attn", n_embd_, n_embd_), c_proj(ps, name + ".c_proj", n_embd_, n_embd_),
      n_head(n_head_), n_embd(n_embd_)
{
}

Tensor* CausalSelfAttention::forward(Graph& g, Tensor* x, Tensor* residual) const
{
    // src/nn.zig:752-937, same op sequence
    const size_t B = x->shape.dims[0], T = x->shape.dims[1], C = x->shape.dims[2];
    const size_t nh = n_head, hs = C / nh;
    Tensor* x_2d = g.reshape(x, Shape{B * T, C});
    Tensor *q_2d, *k_2d, *v_2d;
    if (g_fused_linear && group_linear()) {   // the three projections share their input: grouped launches
        Tensor* const W3[3] = {q_attn.weight, k_attn.weight, v_attn.weight};
        Tensor* const b3[3] = {q_attn.bias, k_attn.bias, v_attn.bias};
        Tensor* o3[3];
        g.linearGroup(x_2d, 3, W3, b3, o3);
        q_2d = o3[0]; k_2d = o3[1]; v_2d = o3[2];
    } else {
        q_2d = q_attn.forward(g, x_2d);
        k_2d = k_attn.forward(g, x_2d);
        v_2d = v_attn.forward(g, x_2d);
    }
    // (short sequences keep the separate products: a 256-row unit of the fused kernel is mostly empty below T = 128)
    if (fused_softmax && g_fused_attention && (hs == 32 || hs == 64) && T % 4 == 0 && T >= 128) {
        // one op on the projections where they lie: the heads are read and written through strides
        Tensor* y_2d = g.causalAttention(q_2d, k_2d, v_2d, B, T, nh, 1.0f / sqrtf((float)hs));
        Tensor* out_2d = residual ? c_proj.forward_residual(g, y_2d, g.reshape(residual, Shape{B * T, C})) : c_proj.forward(g, y_2d);
        return g.reshape(out_2d, Shape{B, T, C});
    }
    Tensor* q_4d = g.reshape(q_2d, Shape{B, T, nh, hs});
    Tensor* k_4d = g.reshape(k_2d, Shape{B, T, nh, hs});
    Tensor* v_4d = g.reshape(v_2d, Shape{B, T, nh, hs});
    Tensor* q = g.transposeND(q_4d, 1, 2);
    Tensor* k = g.transposeND(k_4d, 1, 2);
    Tensor* v = g.transposeND(v_4d, 1, 2);
    // with the fused causal softmax nobody reads the scores above the diagonal, and the probabilities there are
    // exact zeros: the two products and their four gradient products skip those tiles
    const bool skip = fused_softmax && g_causal_skip;
    Tensor* att;
    if (g_fused_qkt) {
        att = g.batchMatMulNT(q, k, skip ? 1 : 0);          // Q.K^T without the transposed copy of K
    } else {
        Tensor* k_t = g.transposeND(k, 2, 3);               // nn.zig:796-835 literally
        att = g.batchMatMul(q, k_t, skip ? 1 : 0);
    }
    const float scale = 1.0f / sqrtf((float)hs);
    Tensor* att_sm;
    if (fused_softmax) {
        att_sm = g.causalSoftmax(att, scale);
    } else {
        Tensor* att_scaled = g.mulScalar(att, scale);
        std::vector<float> mask(B * nh * T * T, 0.0f);  // nn.zig:847-860
        for (size_t s = 0; s < B * nh; s++)
            for (size_t i = 0; i < T; i++)
                for (size_t j = i + 1; j < T; j++) mask[(s * T + i) * T + j] = -1e9f;
        Tensor* mask_node = g.array(Shape{B, nh, T, T}, mask.data(), false);
        Tensor* att_masked = g.add(att_scaled, mask_node);
        att_sm = g.softmax(att_masked);
    }
    Tensor* y_4d = g.batchMatMul(att_sm, v, skip ? 2 : 0);
    Tensor* y_trans = g.transposeND(y_4d, 1, 2);
    Tensor* y_3d = g.reshape(y_trans, Shape{B, T, C});
    Tensor* y_2d = g.reshape(y_3d, Shape{B * T, C});
    Tensor* out_2d = residual ? c_proj.forward_residual(g, y_2d, g.reshape(residual, Shape{B * T, C})) : c_proj.forward(g, y_2d);
    return g.reshape(out_2d, Shape{B, T, C});
}

TransformerBlock::TransformerBlock(ParamStore& ps, const std::string& name, size_t n_embd, size_t n_head)
    : ln_1(ps, name + ".ln_1", n_embd, 1e-5f), attn(ps, name + ".attn", n_embd, n_head),
      ln_2(ps, name + ".ln_2", n_embd, 1e-5f), mlp(ps, name + ".mlp", n_embd, 4 * n_embd)
{
}

Tensor* TransformerBlock::forward(Graph& g, Tensor* x) const
{
    // src/nn.zig:996-1021
    Tensor* x_norm1 = ln_1.forward(g, x);
    if (fused_epilogue() & 1) {   // the two residual adds ride in the epilogues of the output projections
        Tensor* x1 = attn.forward(g, x_norm1, x);
        Tensor* x_norm2 = ln_2.forward(g, x1);
        return mlp.forward(g, x_norm2, x1);
    }
    Tensor* x_attn = attn.forward(g, x_norm1);
    Tensor* x1 = g.add(x, x_attn);
    Tensor* x_norm2 = ln_2.forward(g, x1);
    Tensor* x_mlp = mlp.forward(g, x_norm2);
    return g.add(x1, x_mlp);
}

GPT::GPT(ParamStore& ps, const GPTConfig& c)
    : cfg(c), token_embedding(ps, "token_embedding", c.vocab_size, c.n_embd),
      position_embedding(ps, "position_embedding", c.block_size, c.n_embd)
{
    for (size_t i = 0; i < c.n_layer; i++)
        h.emplace_back(ps, "decoder.h." + std::to_string(i), c.n_embd, c.n_head);
    ln_f = RMSNorm(ps, "decoder.ln_f", c.n_embd, 1e-5f);
    lm_head = Linear(ps, "lm_head", c.n_embd, c.vocab_size);
}

void GPT::set_fused_softmax(bool on)
{
    for (TransformerBlock& b : h) b.attn.fused_softmax = on;
}

Tensor* GPT::forward(Graph& g, Tensor* ids) const
{
    // src/nn.zig:1172-1233
    const size_t B = ids->shape.dims[0], T = ids->shape.dims[1];
    if (T > cfg.block_size) throw Error(ZNN_ERR_INVALID, "GPT.forward: sequence longer than block_size");
    Tensor* tok_emb = token_embedding.forward(g, ids);
    // the position ids 0..T-1 of every row, written on the device (the reference fills them on the host): the step
    // then uploads nothing and can be captured into a CUDA graph
    Tensor* pos_node = g.tensorND(Shape{B, T}, false);
    check(znn_iota_mod(pos_node->data, B * T, (int)T), "position ids");
    Tensor* pos_emb = position_embedding.forward(g, pos_node);
    Tensor* cur = g.add(tok_emb, pos_emb);
    for (const TransformerBlock& blk : h) cur = blk.forward(g, cur);
    Tensor* out = ln_f.forward(g, cur);
    Tensor* ln_x_2d = g.reshape(out, Shape{B * T, cfg.n_embd});
    Tensor* logits_2d = lm_head.forward(g, ln_x_2d);
    return g.reshape(logits_2d, Shape{B, T, cfg.vocab_size});
}

MlpNet::MlpNet(ParamStore& ps, size_t in, size_t h1, size_t h2, size_t out)
    : fc1(ps, "fc1", in, h1), fc2(ps, "fc2", h1, h2), fc3(ps, "fc3", h2, out)
{
}

Tensor* MlpNet::forward(Graph& g, Tensor* x) const
{
    Tensor* a1 = fc1.forward_act(g, x, OpType::Relu);
    Tensor* a2 = fc2.forward_act(g, a1, OpType::Relu);
    return fc3.forward(g, a2);
}

CnnNet::CnnNet(ParamStore& ps, bool ref) : reference_shape(ref)
{
    if (ref) {
        conv1 = Conv2D(ps, "conv1", 1, 4, 3);
        conv2 = Conv2D(ps, "conv2", 4, 8, 3);
        conv3 = Conv2D(ps, "conv3", 8, 16, 3);
        fc1 = Linear(ps, "fc1", 144, 10);
    } else {
        conv1 = Conv2D(ps, "conv1", 1, 32, 3, 1);
        conv2 = Conv2D(ps, "conv2", 32, 64, 3, 1);
        fc1 = Linear(ps, "fc1", 3136, 128);
        fc2 = Linear(ps, "fc2", 128, 10);
    }
}

Tensor* CnnNet::forward(Graph& g, Tensor* x) const
{
    const size_t B = x->shape.dims[0];
    Tensor* xr = g.reshape(x, Shape{B, 1, 28, 28});
    if (reference_shape) {
        // examples/cnn.zig:35-56
        Tensor* p1 = g.maxpool2d(conv1.forward_relu(g, xr), 2, 2);
        Tensor* p2 = g.maxpool2d(conv2.forward_relu(g, p1), 2, 2);
        Tensor* a3 = conv3.forward_relu(g, p2);
        Tensor* flat = g.reshape(a3, Shape{B, 144});
        return fc1.forward(g, flat);
    }
    Tensor* p1 = g.maxpool2d(conv1.forward_relu(g, xr), 2, 2);   // 32 @ 14x14
    Tensor* p2 = g.maxpool2d(conv2.forward_relu(g, p1), 2, 2);   // 64 @ 7x7
    Tensor* flat = g.reshape(p2, Shape{B, 3136});
    Tensor* a = fc1.forward_act(g, flat, OpType::Relu);
    return fc2.forward(g, a);
}

void SGDOptimizer::step(float grad_scale) const
{
    check(znn_sgd_step(ps->values(), ps->grads(), momentum > 0.0f ? ps->velocities() : nullptr, lr, momentum, grad_scale,
                       ps->total()),
          "SGD step");
}

void AdamOptimizer::step(float grad_scale)
{
    t += 1.0f;
    check(znn_adam_step(ps->values(), ps->grads(), ps->velocities(), ps->second_moments(), lr, beta1, beta2, eps, t,
                        grad_scale, ps->total()),
          "Adam step");
}

}  // namespace host
}  // namespace znn
