// Host-side mirror of the reference's modules (src/nn.zig) and optimizer
// (src/optim.zig:6-67), composed from Graph builders exactly as the reference
// composes them.  Parameters live in one ParamStore: three contiguous device
// slabs (values, gradients, SGD velocities) laid out in the reference's
// collectParameters order (struct-field order, src/nn.zig:142-171), so that
// zeroGrad is one memset, the optimizer one kernel and the data-parallel
// gradient exchange a few large all-reduces.
#pragma once
#include <string>
#include <vector>

#include "graph.hpp"

namespace znn {
namespace host {

struct ParamInfo {
    std::string name;   // dotted path as in the reference's save format, e.g. decoder.h.0.attn.q_attn.weight
    Tensor* tensor;
    size_t offset;      // in floats, into the slabs
    size_t fan_in;      // for initialisation by the caller
};

class ParamStore {
public:
    ParamStore() = default;
    ~ParamStore();
    ParamStore(const ParamStore&) = delete;
    ParamStore& operator=(const ParamStore&) = delete;
    // Registration phase: returns a persistent tensor (requires_grad = true) whose
    // pointers are assigned by finalize().  nn.zig:1352-1377 (createPersistentTensor).
    Tensor* add(const std::string& name, const Shape& shape, size_t fan_in);
    void finalize();                 // allocates the slabs, zero-fills them, assigns pointers
    void zeroGrad();                 // model.zeroGrad(): nn.zig:121-140
    size_t total() const { return total_; }
    float* values() { return w_; }
    float* grads() { return g_; }
    float* velocities() { return v_; }
    float* second_moments();         // Adam's v slab, allocated and zeroed on first use
    const std::vector<ParamInfo>& params() const { return params_; }

private:
    std::vector<ParamInfo> params_;
    size_t total_ = 0;
    float *w_ = nullptr, *g_ = nullptr, *v_ = nullptr, *v2_ = nullptr;
};

// Linear.forward runs the fused matmul+addBias op by default; false = the reference's two ops.
// The attention products skip the tiles the causal mask makes irrelevant (only with fused_softmax); default on.
void set_causal_skip(bool on);
bool causal_skip();
// Attention scores as one Q.K^T op instead of transposeND(K) + batchMatMul; default on.
void set_fused_qkt(bool on);
bool fused_qkt();
void set_fused_linear(bool on);
bool fused_linear();
// The attention chain (head split, Q.K^T, scale + mask + softmax, P.V, head merge) as the one fused op whenever the
// fused kernel takes the shape (head size 32 or 64, T a multiple of 4); default on, needs fused_softmax.
void set_fused_attention(bool on);
bool fused_attention();

// src/nn.zig:10-52.  W is [in, out], b is [1, out]; forward = addBias(matmul(x, W), b)
struct Linear {
    Tensor* weight = nullptr;
    Tensor* bias = nullptr;
    Linear() = default;
    Linear(ParamStore& ps, const std::string& name, size_t in_features, size_t out_features);
    Tensor* forward(Graph& g, Tensor* x) const;
    Tensor* forward_act(Graph& g, Tensor* x, OpType act) const;        // act(forward(x)), act = Relu or Gelu
    Tensor* forward_residual(Graph& g, Tensor* x, Tensor* r) const;    // r + forward(x)
};

// src/nn.zig:54-96.  weight [Co, Ci, k, k], bias [Co]; pad is an extension (0 = reference)
struct Conv2D {
    Tensor* weight = nullptr;
    Tensor* bias = nullptr;
    int pad = 0;
    Conv2D() = default;
    Conv2D(ParamStore& ps, const std::string& name, size_t in_ch, size_t out_ch, size_t k, int pad = 0);
    Tensor* forward(Graph& g, Tensor* x) const;
    Tensor* forward_relu(Graph& g, Tensor* x) const;   // relu(forward(x))
};

// src/nn.zig:509-542
struct Embedding {
    Tensor* weight = nullptr;
    Embedding() = default;
    Embedding(ParamStore& ps, const std::string& name, size_t vocab, size_t dim);
    Tensor* forward(Graph& g, Tensor* ids) const;
};

// src/nn.zig:553-592 (gamma initialised to 1 by the caller's parameter upload)
struct RMSNorm {
    Tensor* weight = nullptr;
    float eps = 1e-5f;
    RMSNorm() = default;
    RMSNorm(ParamStore& ps, const std::string& name, size_t dim, float eps);
    Tensor* forward(Graph& g, Tensor* x) const;
};

// src/nn.zig:603-686: Linear -> GELU -> Linear on [B*T, D]
struct MLP {
    Linear c_fc, c_proj;
    MLP() = default;
    MLP(ParamStore& ps, const std::string& name, size_t dim, size_t hidden);
    Tensor* forward(Graph& g, Tensor* x, Tensor* residual = nullptr) const;   // residual: returns residual + mlp(x)
};

// src/nn.zig:700-938.  fused_softmax = true replaces the reference's
// mulScalar -> mask build -> add -> softmax chain (:835-886) by the one fused op
// with identical values; false runs the reference's op sequence literally
// (including the materialised -1e9 mask).
struct CausalSelfAttention {
    Linear q_attn, k_attn, v_attn, c_proj;
    size_t n_head = 1, n_embd = 0;
    bool fused_softmax = true;
    CausalSelfAttention() = default;
    CausalSelfAttention(ParamStore& ps, const std::string& name, size_t n_embd, size_t n_head);
    Tensor* forward(Graph& g, Tensor* x, Tensor* residual = nullptr) const;   // residual: returns residual + attn(x)
};

// src/nn.zig:950-1022: x1 = x + attn(rms1(x)); out = x1 + mlp(rms2(x1))
struct TransformerBlock {
    RMSNorm ln_1;
    CausalSelfAttention attn;
    RMSNorm ln_2;
    MLP mlp;
    TransformerBlock() = default;
    TransformerBlock(ParamStore& ps, const std::string& name, size_t n_embd, size_t n_head);
    Tensor* forward(Graph& g, Tensor* x) const;
};

// src/nn.zig:1106-1235
struct GPTConfig {
    size_t vocab_size = 0, block_size = 0, n_embd = 0, n_head = 0, n_layer = 0;
};

struct GPT {
    GPTConfig cfg;
    Embedding token_embedding, position_embedding;
    std::vector<TransformerBlock> h;   // decoder.h
    RMSNorm ln_f;                      // decoder.ln_f
    Linear lm_head;
    GPT() = default;
    GPT(ParamStore& ps, const GPTConfig& cfg);
    // ids: [B, T] fp32 token ids; returns logits [B, T, vocab] (src/nn.zig:1172-1233)
    Tensor* forward(Graph& g, Tensor* ids) const;
    void set_fused_softmax(bool on);
};

// examples/fashion_mnist.zig:25-42: Linear -> ReLU -> Linear -> ReLU -> Linear
struct MlpNet {
    Linear fc1, fc2, fc3;
    MlpNet() = default;
    MlpNet(ParamStore& ps, size_t in, size_t h1, size_t h2, size_t out);
    Tensor* forward(Graph& g, Tensor* x) const;
};

// examples/cnn.zig:24-56 (reference shape: 1->4->8->16 valid convs, fc 144->10) and the
// padded 1->32->64 / 3136->128->10 shape of the workload definition.
struct CnnNet {
    bool reference_shape = true;
    Conv2D conv1, conv2, conv3;
    Linear fc1, fc2;
    CnnNet() = default;
    CnnNet(ParamStore& ps, bool reference_shape);
    Tensor* forward(Graph& g, Tensor* x) const;   // x: [B, 784] or [B,1,28,28]
};

// src/optim.zig:6-67 over the flat slabs: v = mu*v + lr*g ; w -= v
struct SGDOptimizer {
    ParamStore* ps = nullptr;
    float lr = 0.01f, momentum = 0.0f;
    void step(float grad_scale = 1.0f) const;
};

// src/optim.zig:69-152 over the flat slabs (first moments in the velocity slab, second moments in their own):
// t += 1; lr_t = lr * sqrt(1 - beta2^t) / (1 - beta1^t) in fp32 on the host, then one kernel for all parameters
struct AdamOptimizer {
    ParamStore* ps = nullptr;
    float lr = 0.001f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f;
    float t = 0.0f;
    void step(float grad_scale = 1.0f);
};

}  // namespace host
}  // namespace znn
