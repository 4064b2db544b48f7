// C entry points of the host mirror (include/znn_host.h).
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <memory>
#include <unordered_map>

#include "../../../include/znn_cuda.h"
#include "../../../include/znn_host.h"
#include "../../../include/znn_debug.h"
#include "bucket_schedule.hpp"
#include "nn.hpp"

namespace znn {
int fail(int code, const char* fmt, ...);  // runtime.cu: sets the thread's error text
}

using namespace znn::host;

#define ZNN_HOST_TRY try {
#define ZNN_HOST_CATCH                                              \
    }                                                               \
    catch (const Error& e) { return znn::fail(e.code, "%s", e.what()); } \
    catch (const std::exception& e) { return znn::fail(ZNN_ERR_INVALID, "%s", e.what()); } \
    return ZNN_OK;

struct znn_graph {
    std::unique_ptr<Arena> arena;
    std::unique_ptr<Graph> g;
    std::vector<Tensor*> handles;
};

static Tensor* handle(znn_graph* g, int id)
{
    if (id < 0 || (size_t)id >= g->handles.size()) throw Error(ZNN_ERR_INVALID, "unknown tensor handle " + std::to_string(id));
    return g->handles[id];
}

static Shape shape_from(const long long* dims, int rank)
{
    if (rank < 0 || rank > 8) throw Error(ZNN_ERR_INVALID, "rank must be 0..8");
    size_t d[8];
    for (int i = 0; i < rank; i++) {
        if (dims[i] < 0) throw Error(ZNN_ERR_INVALID, "negative dimension");
        d[i] = (size_t)dims[i];
    }
    return Shape(d, (size_t)rank);
}

extern "C" {

int znn_graph_create(size_t arena_bytes, znn_graph** out)
{
    ZNN_HOST_TRY
    if (!out) throw Error(ZNN_ERR_INVALID, "out is NULL");
    std::unique_ptr<znn_graph> zg(new znn_graph());
    zg->arena.reset(new Arena(arena_bytes));
    zg->g.reset(new Graph(zg->arena.get()));
    *out = zg.release();
    ZNN_HOST_CATCH
}

int znn_graph_destroy(znn_graph* g)
{
    ZNN_HOST_TRY
    if (g) {
        znn_sync();
        delete g;
    }
    ZNN_HOST_CATCH
}

int znn_graph_array(znn_graph* g, const long long* dims, int rank, const float* host_data, int requires_grad, int* id)
{
    ZNN_HOST_TRY
    const Shape s = shape_from(dims, rank);
    Tensor* t = host_data ? g->g->array(s, host_data, requires_grad != 0) : g->g->tensorND(s, requires_grad != 0);
    g->handles.push_back(t);
    if (id) *id = (int)g->handles.size() - 1;
    ZNN_HOST_CATCH
}

int znn_graph_op(znn_graph* zg, const char* name, const int* inputs, int n_inputs, const double* args, int n_args, int* id)
{
    ZNN_HOST_TRY
    Graph& g = *zg->g;
    const std::string op(name ? name : "");
    auto in = [&](int i) -> Tensor* {
        if (i >= n_inputs) throw Error(ZNN_ERR_INVALID, op + ": too few inputs");
        return handle(zg, inputs[i]);
    };
    auto arg = [&](int i) -> double {
        if (i >= n_args) throw Error(ZNN_ERR_INVALID, op + ": too few arguments");
        return args[i];
    };
    Tensor* out = nullptr;
    if (op == "matmul") out = g.matmul(in(0), in(1));
    else if (op == "addBias") out = g.addBias(in(0), in(1));
    else if (op == "relu") out = g.relu(in(0));
    else if (op == "gelu") out = g.gelu(in(0));
    else if (op == "softmaxCrossEntropy") {
        Tensor* logits = in(0);
        const size_t M = logits->shape.dims[0];
        if ((size_t)n_args != M) throw Error(ZNN_ERR_INVALID, "softmaxCrossEntropy: one label per row expected");
        std::vector<int32_t> t(M);
        for (size_t i = 0; i < M; i++) t[i] = (int32_t)args[i];
        int32_t* dev = (int32_t*)zg->arena->alloc(M * sizeof(int32_t));
        check(znn_memcpy_h2d(dev, t.data(), M * sizeof(int32_t)), "upload labels");
        check(znn_sync(), "znn_sync");
        out = g.softmaxCrossEntropy(logits, dev);
    } else if (op == "reshape") {
        size_t d[8];
        if (n_args > 8) throw Error(ZNN_ERR_INVALID, "reshape: rank above 8");
        for (int i = 0; i < n_args; i++) d[i] = (size_t)args[i];
        out = g.reshape(in(0), Shape(d, (size_t)n_args));
    } else if (op == "transposeND" || op == "transpose") out = g.transposeND(in(0), (int)arg(0), (int)arg(1));
    else if (op == "mulScalar") out = g.mulScalar(in(0), (float)arg(0));
    else if (op == "add") out = g.add(in(0), in(1));
    else if (op == "conv2d") out = g.conv2d(in(0), in(1), n_inputs > 2 ? in(2) : nullptr, n_args > 0 ? (int)args[0] : 0);
    else if (op == "maxpool2d") out = g.maxpool2d(in(0), (int)arg(0), (int)arg(1));
    else if (op == "softmax") out = g.softmax(in(0));
    else if (op == "causalSoftmax") out = g.causalSoftmax(in(0), (float)arg(0));
    else if (op == "rmsNorm") out = g.rmsNorm(in(0), in(1), (float)arg(0));
    else if (op == "layerNorm") out = g.layerNorm(in(0), in(1), in(2), (float)arg(0));
    else if (op == "batchMatMul") out = g.batchMatMul(in(0), in(1));
    else if (op == "batchMatMulNT") out = g.batchMatMulNT(in(0), in(1));
    else if (op == "linear") out = g.linear(in(0), in(1), in(2));
    else if (op == "causalAttention")
        out = g.causalAttention(in(0), in(1), in(2), (size_t)arg(0), (size_t)arg(1), (size_t)arg(2), (float)arg(3));
    else if (op == "embedding") out = g.embedding(in(0), in(1));
    else throw Error(ZNN_ERR_INVALID, "unknown op '" + op + "'");
    zg->handles.push_back(out);
    if (id) *id = (int)zg->handles.size() - 1;
    ZNN_HOST_CATCH
}

int znn_graph_backward(znn_graph* g, int id, int seed_one)
{
    ZNN_HOST_TRY
    if (seed_one) g->g->backward(handle(g, id));
    else g->g->backwardWithGrad(handle(g, id));
    ZNN_HOST_CATCH
}

int znn_graph_forward(znn_graph* g)
{
    ZNN_HOST_TRY
    g->g->forward();
    ZNN_HOST_CATCH
}

int znn_graph_zero_grad(znn_graph* g)
{
    ZNN_HOST_TRY
    g->g->zeroGrad();
    ZNN_HOST_CATCH
}

int znn_graph_shape(znn_graph* g, int id, long long* dims8, int* rank, int* requires_grad)
{
    ZNN_HOST_TRY
    Tensor* t = handle(g, id);
    if (dims8)
        for (size_t i = 0; i < t->shape.len; i++) dims8[i] = (long long)t->shape.dims[i];
    if (rank) *rank = (int)t->shape.len;
    if (requires_grad) *requires_grad = t->requires_grad ? 1 : 0;
    ZNN_HOST_CATCH
}

int znn_graph_read(znn_graph* g, int id, int which, float* host, size_t count)
{
    ZNN_HOST_TRY
    Tensor* t = handle(g, id);
    const float* src = which ? t->grad : t->data;
    if (!src) throw Error(ZNN_ERR_INVALID, "tensor has no gradient buffer (requires_grad is false)");
    if (count > t->numel()) throw Error(ZNN_ERR_INVALID, "read beyond the tensor");
    if (which) ensure_grad(t);
    check(znn_memcpy_d2h(host, src, count * sizeof(float)), "znn_memcpy_d2h");
    ZNN_HOST_CATCH
}

int znn_graph_write(znn_graph* g, int id, int which, const float* host, size_t count)
{
    ZNN_HOST_TRY
    Tensor* t = handle(g, id);
    float* dst = which ? t->grad : t->data;
    if (!dst) throw Error(ZNN_ERR_INVALID, "tensor has no gradient buffer (requires_grad is false)");
    if (count > t->numel()) throw Error(ZNN_ERR_INVALID, "write beyond the tensor");
    if (which) ensure_grad(t);
    check(znn_memcpy_h2d(dst, host, count * sizeof(float)), "znn_memcpy_h2d");
    check(znn_sync(), "znn_sync");
    ZNN_HOST_CATCH
}

int znn_graph_num_ops(znn_graph* g, int* n)
{
    ZNN_HOST_TRY
    if (n) *n = (int)g->g->ops().size();
    ZNN_HOST_CATCH
}

}  // extern "C"

// ------------------------------------------------------------------ models
struct znn_model {
    int kind = 0;
    ParamStore ps;
    std::unique_ptr<Arena> arena;
    MlpNet mlp;
    CnnNet cnn;
    TransformerBlock block;
    GPT gpt;
    SGDOptimizer opt;
    AdamOptimizer adam;
    bool use_adam = false;            // "optimizer" option: 0 = SGD (the example programs), 1 = Adam
    size_t in_features = 0, classes = 0;
    size_t dp_bucket_floats = 8u << 20;  // 32 MB buckets
    bool dp_overlap = true;
    bool targets_u8 = false;          // targets are bytes, the reference's label type (src/dataset.zig:14-16)
    int last_ops = 0;
    std::unordered_map<const Tensor*, int> param_index;
    // CUDA-graph replay of the training step (option "cuda_graph"): the step's launch sequence is captured once
    // per (input pointers, batch) and replayed; the per-step arena hands out the same addresses every step, so the
    // captured kernels stay valid.
    bool use_graph = false;
    cudaGraphExec_t graph_exec = nullptr;
    const void* graph_x = nullptr;
    const void* graph_t = nullptr;
    int graph_batch = 0, graph_seq = 0, graph_seen = 0;
    float* graph_loss = nullptr;
    long long graph_replays = 0;
    // the captured kernels hold raw addresses of the shim's scratch blocks: the graph is only valid while none of
    // them has moved since the capture (znn_workspace_generation)
    unsigned long long graph_generation = 0;
};

static void drop_graph(znn_model* m)
{
    if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
    m->graph_exec = nullptr;
    m->graph_seen = 0;
}

namespace {

// Starts the all-reduce of a gradient bucket as soon as the backward sweep has run every op that writes into it
// (the bookkeeping is BucketSchedule; this class maps tape ops to parameters and fires NCCL).
class DpSchedule {
public:
    DpSchedule(znn_model& m, const Graph& g) : m_(m), sched_(make(m, g)) {}

    void after(Op* op)
    {
        for (const Tensor* in : op->inputs) {
            auto it = m_.param_index.find(in);
            if (it == m_.param_index.end()) continue;
            check(sched_.after(it->second), "gradient all-reduce");
        }
    }

    void finish()
    {
        check(sched_.finish(), "gradient all-reduce");
        check(znn_dp_join(), "znn_dp_join");
    }

    size_t buckets() const { return sched_.buckets(); }

private:
    static BucketSchedule make(znn_model& m, const Graph& g)
    {
        const auto& ps = m.ps.params();
        std::vector<size_t> offsets(ps.size());
        std::vector<int> uses(ps.size(), 0);
        for (size_t i = 0; i < ps.size(); i++) offsets[i] = ps[i].offset;
        for (const Op* op : g.ops())
            for (const Tensor* in : op->inputs) {
                auto it = m.param_index.find(in);
                if (it != m.param_index.end()) uses[it->second]++;
            }
        float* grads = m.ps.grads();
        return BucketSchedule(offsets, m.ps.total(), m.dp_bucket_floats, uses,
                              [grads](size_t begin, size_t count) { return znn_dp_allreduce_async(grads + begin, count); });
    }
    znn_model& m_;
    BucketSchedule sched_;
};

Tensor* wrap_device(Graph& g, const Shape& s, const float* dev)
{
    // a graph input that lives in caller-owned device memory: no copy, no gradient
    Tensor* t = g.tensorND(Shape{1}, false);
    t->shape = s;
    t->strides = contiguous_strides(s);
    t->data = const_cast<float*>(dev);
    return t;
}

Tensor* model_forward(znn_model& m, Graph& g, const float* x, int batch, int seq, bool on_device)
{
    Tensor* xt = nullptr;
    switch (m.kind) {
    case ZNN_MODEL_MLP:
    case ZNN_MODEL_CNN_REF:
    case ZNN_MODEL_CNN_PADDED: {
        const Shape s{(size_t)batch, m.in_features};
        xt = on_device ? wrap_device(g, s, x) : g.array(s, x, false);
        return m.kind == ZNN_MODEL_MLP ? m.mlp.forward(g, xt) : m.cnn.forward(g, xt);
    }
    case ZNN_MODEL_GPT: {
        const Shape s{(size_t)batch, (size_t)seq};
        xt = on_device ? wrap_device(g, s, x) : g.array(s, x, false);
        Tensor* logits = m.gpt.forward(g, xt);
        return g.reshape(logits, Shape{(size_t)batch * seq, m.gpt.cfg.vocab_size});  // transformer_gpt.zig:90-92
    }
    default: throw Error(ZNN_ERR_INVALID, "this model kind has no classification forward");
    }
}

}  // namespace

extern "C" {

int znn_model_create(int kind, const long long* dims, int ndims, size_t arena_bytes, znn_model** out)
{
    ZNN_HOST_TRY
    if (!out) throw Error(ZNN_ERR_INVALID, "out is NULL");
    auto need = [&](int n) {
        if (ndims < n) throw Error(ZNN_ERR_INVALID, "too few dims for this model kind");
    };
    std::unique_ptr<znn_model> m(new znn_model());
    m->kind = kind;
    switch (kind) {
    case ZNN_MODEL_MLP:
        need(4);
        m->mlp = MlpNet(m->ps, (size_t)dims[0], (size_t)dims[1], (size_t)dims[2], (size_t)dims[3]);
        m->in_features = (size_t)dims[0];
        m->classes = (size_t)dims[3];
        break;
    case ZNN_MODEL_CNN_REF:
    case ZNN_MODEL_CNN_PADDED:
        m->cnn = CnnNet(m->ps, kind == ZNN_MODEL_CNN_REF);
        m->in_features = 784;
        m->classes = 10;
        break;
    case ZNN_MODEL_BLOCK:
        need(2);
        m->block = TransformerBlock(m->ps, "block", (size_t)dims[0], (size_t)dims[1]);
        m->in_features = (size_t)dims[0];
        break;
    case ZNN_MODEL_GPT: {
        need(5);
        GPTConfig c;
        c.vocab_size = (size_t)dims[0];
        c.block_size = (size_t)dims[1];
        c.n_embd = (size_t)dims[2];
        c.n_head = (size_t)dims[3];
        c.n_layer = (size_t)dims[4];
        if (c.n_head == 0 || c.n_embd % c.n_head != 0) throw Error(ZNN_ERR_INVALID, "n_embd must be a multiple of n_head");
        m->gpt = GPT(m->ps, c);
        m->classes = c.vocab_size;
        break;
    }
    default: throw Error(ZNN_ERR_INVALID, "unknown model kind");
    }
    m->ps.finalize();
    for (size_t i = 0; i < m->ps.params().size(); i++) m->param_index[m->ps.params()[i].tensor] = (int)i;
    m->arena.reset(new Arena(arena_bytes));
    m->opt.ps = &m->ps;
    m->adam.ps = &m->ps;
    *out = m.release();
    ZNN_HOST_CATCH
}

int znn_model_destroy(znn_model* m)
{
    ZNN_HOST_TRY
    if (m) {
        znn_sync();
        drop_graph(m);
        delete m;
    }
    ZNN_HOST_CATCH
}

int znn_model_param_count(znn_model* m, int* n)
{
    ZNN_HOST_TRY
    if (n) *n = (int)m->ps.params().size();
    ZNN_HOST_CATCH
}

int znn_model_param_info(znn_model* m, int i, char* name, size_t name_len, long long* dims8, int* rank, long long* offset,
                         long long* fan_in)
{
    ZNN_HOST_TRY
    if (i < 0 || (size_t)i >= m->ps.params().size()) throw Error(ZNN_ERR_INVALID, "parameter index out of range");
    const ParamInfo& p = m->ps.params()[i];
    if (name && name_len) {
        strncpy(name, p.name.c_str(), name_len - 1);
        name[name_len - 1] = 0;
    }
    if (dims8)
        for (size_t k = 0; k < p.tensor->shape.len; k++) dims8[k] = (long long)p.tensor->shape.dims[k];
    if (rank) *rank = (int)p.tensor->shape.len;
    if (offset) *offset = (long long)p.offset;
    if (fan_in) *fan_in = (long long)p.fan_in;
    ZNN_HOST_CATCH
}

int znn_model_total_floats(znn_model* m, long long* total)
{
    ZNN_HOST_TRY
    if (total) *total = (long long)m->ps.total();
    ZNN_HOST_CATCH
}

int znn_model_set_params(znn_model* m, const float* host_slab)
{
    ZNN_HOST_TRY
    check(znn_memcpy_h2d(m->ps.values(), host_slab, m->ps.total() * sizeof(float)), "upload parameters");
    check(znn_sync(), "znn_sync");
    ZNN_HOST_CATCH
}

int znn_model_get_params(znn_model* m, float* host_slab)
{
    ZNN_HOST_TRY
    check(znn_memcpy_d2h(host_slab, m->ps.values(), m->ps.total() * sizeof(float)), "download parameters");
    ZNN_HOST_CATCH
}

int znn_model_get_grads(znn_model* m, float* host_slab)
{
    ZNN_HOST_TRY
    check(znn_memcpy_d2h(host_slab, m->ps.grads(), m->ps.total() * sizeof(float)), "download gradients");
    ZNN_HOST_CATCH
}

int znn_model_get_velocities(znn_model* m, float* host_slab)
{
    ZNN_HOST_TRY
    check(znn_memcpy_d2h(host_slab, m->ps.velocities(), m->ps.total() * sizeof(float)), "download velocities");
    ZNN_HOST_CATCH
}

int znn_model_set_option(znn_model* m, const char* key, double value)
{
    ZNN_HOST_TRY
    const std::string k(key ? key : "");
    // every option that changes a baked-in kernel argument or the launch sequence invalidates a captured step
    if (k == "lr" || k == "momentum" || k.rfind("fused_", 0) == 0 || k == "causal_skip" || k == "alias_reshape_grad" ||
        k == "lazy_zero_grad" || k == "fused_attention" || k == "group_linear")
        drop_graph(m);
    if (k == "lr") m->opt.lr = m->adam.lr = (float)value;
    else if (k == "optimizer") {
        if (value != 0.0 && value != 1.0) throw Error(ZNN_ERR_INVALID, "optimizer: 0 = SGD, 1 = Adam");
        m->use_adam = (value == 1.0);
        drop_graph(m);
    }
    else if (k == "beta1") m->adam.beta1 = (float)value;
    else if (k == "beta2") m->adam.beta2 = (float)value;
    else if (k == "eps") m->adam.eps = (float)value;
    else if (k == "adam_t") m->adam.t = (float)value;
    else if (k == "momentum") m->opt.momentum = (float)value;
    else if (k == "fused_softmax") {
        m->gpt.set_fused_softmax(value != 0.0);
        m->block.attn.fused_softmax = (value != 0.0);
    } else if (k == "fused_linear") set_fused_linear(value != 0.0);
    else if (k == "causal_skip") set_causal_skip(value != 0.0);
    else if (k == "fused_qkt") set_fused_qkt(value != 0.0);
    else if (k == "fused_attention") set_fused_attention(value != 0.0);
    else if (k == "fused_epilogue") set_fused_epilogue((int)value);
    else if (k == "group_linear") set_group_linear(value != 0.0);
    else if (k == "fused_softmax_bwd") set_fused_softmax_bwd(value != 0.0);
    else if (k == "alias_reshape_grad") set_alias_reshape_grad(value != 0.0);
    else if (k == "lazy_zero_grad") set_lazy_zero_grad(value != 0.0);
    else if (k == "cuda_graph") {
        m->use_graph = (value != 0.0);
        if (!m->use_graph) drop_graph(m);
    }
    else if (k == "dp_bucket_floats") m->dp_bucket_floats = (size_t)value;
    else if (k == "dp_overlap") m->dp_overlap = (value != 0.0);
    else if (k == "targets_u8") {
        m->targets_u8 = (value != 0.0);
        drop_graph(m);
    }
    else throw Error(ZNN_ERR_INVALID, "unknown option '" + k + "'");
    ZNN_HOST_CATCH
}

// One training step as the example programs run it (examples/fashion_mnist.zig:131-167); returns the device
// address of the loss scalar.
static float* run_train_step(znn_model* m, const float* x, const int32_t* targets, int batch, int seq, bool on_device)
{
    m->arena->reset();                       // Graph.init / graph.deinit of the previous batch
    Graph g(m->arena.get());
    const size_t rows = (m->kind == ZNN_MODEL_GPT) ? (size_t)batch * seq : (size_t)batch;
    const int32_t* dev_targets = targets;
    if (!on_device) {
        const size_t bytes = rows * (m->targets_u8 ? 1 : sizeof(int32_t));
        int32_t* t = (int32_t*)m->arena->alloc(bytes);
        check(znn_memcpy_h2d(t, targets, bytes), "upload targets");
        dev_targets = t;  // the stream synchronisation of the input upload below covers this copy
    }
    Tensor* logits = model_forward(*m, g, x, batch, seq, on_device);
    Tensor* loss = m->targets_u8 ? g.softmaxCrossEntropyU8(logits, reinterpret_cast<const uint8_t*>(dev_targets))
                                 : g.softmaxCrossEntropy(logits, dev_targets);
    m->ps.zeroGrad();                        // model.zeroGrad() (fashion_mnist.zig:155)
    int world = 1;
    znn_dp_world(&world, nullptr);
    if (world > 1) {
        DpSchedule sched(*m, g);
        if (m->dp_overlap) {
            std::function<void(Op*)> hook = [&](Op* op) { sched.after(op); };
            g.backward(loss, &hook);
        } else {
            g.backward(loss);
        }
        sched.finish();
    } else {
        g.backward(loss);
    }
    // optimizer.step(); 1/world turns the rank sum into the global mean
    if (m->use_adam) m->adam.step(1.0f / (float)world);
    else m->opt.step(1.0f / (float)world);
    m->last_ops = (int)g.ops().size();
    return loss->data;
}

int znn_model_train_step(znn_model* m, const float* x, const int32_t* targets, int batch, int seq, int on_device,
                         float* loss_host)
{
    ZNN_HOST_TRY
    if (batch <= 0) throw Error(ZNN_ERR_INVALID, "batch must be positive");
    if (m->kind == ZNN_MODEL_GPT && seq <= 0) throw Error(ZNN_ERR_INVALID, "seq must be positive");
    int world = 1;
    znn_dp_world(&world, nullptr);
    // Replay is possible when nothing in the step touches the host: device-resident inputs and one GPU (the gradient
    // exchange polls its communicator from the host).
    const bool can_replay = m->use_graph && !m->use_adam && on_device && world == 1 && m->kind != ZNN_MODEL_BLOCK;
    float* loss_dev = nullptr;
    if (!can_replay) {
        loss_dev = run_train_step(m, x, targets, batch, seq, on_device != 0);
    } else {
        unsigned long long gen = 0;
        check(znn_workspace_generation(&gen), "znn_workspace_generation");
        if (m->graph_x != x || m->graph_t != targets || m->graph_batch != batch || m->graph_seq != seq ||
            (m->graph_exec && gen != m->graph_generation)) {
            drop_graph(m);
            m->graph_x = x;
            m->graph_t = targets;
            m->graph_batch = batch;
            m->graph_seq = seq;
        }
        if (m->graph_exec) {
            void* st = nullptr;
            check(znn_get_stream(&st), "znn_get_stream");
            if (cudaGraphLaunch(m->graph_exec, (cudaStream_t)st) != cudaSuccess)
                throw Error(ZNN_ERR_CUDA, std::string("cudaGraphLaunch: ") + cudaGetErrorString(cudaGetLastError()));
            m->graph_replays++;
            loss_dev = m->graph_loss;
        } else if (m->graph_seen == 0) {
            // first step with these buffers: run eagerly so that scratch blocks reach their final size
            loss_dev = run_train_step(m, x, targets, batch, seq, true);
            m->graph_seen = 1;
        } else {
            void* stv = nullptr;
            check(znn_get_stream(&stv), "znn_get_stream");
            cudaStream_t st = (cudaStream_t)stv;
            if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
                throw Error(ZNN_ERR_CUDA, std::string("cudaStreamBeginCapture: ") + cudaGetErrorString(cudaGetLastError()));
            cudaGraph_t graph = nullptr;
            try {
                m->graph_loss = run_train_step(m, x, targets, batch, seq, true);
            } catch (...) {
                cudaStreamEndCapture(st, &graph);
                if (graph) cudaGraphDestroy(graph);
                cudaGetLastError();
                m->use_graph = false;
                throw;
            }
            if (cudaStreamEndCapture(st, &graph) != cudaSuccess || !graph)
                throw Error(ZNN_ERR_CUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(cudaGetLastError()));
            const cudaError_t e = cudaGraphInstantiate(&m->graph_exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) {
                m->graph_exec = nullptr;
                throw Error(ZNN_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
            }
            check(znn_workspace_generation(&m->graph_generation), "znn_workspace_generation");
            if (cudaGraphLaunch(m->graph_exec, st) != cudaSuccess)
                throw Error(ZNN_ERR_CUDA, std::string("cudaGraphLaunch: ") + cudaGetErrorString(cudaGetLastError()));
            m->graph_replays++;
            loss_dev = m->graph_loss;
        }
    }
    if (loss_host) check(znn_memcpy_d2h(loss_host, loss_dev, sizeof(float)), "read loss");
    ZNN_HOST_CATCH
}

int znn_model_forward(znn_model* m, const float* x, int batch, int seq, int on_device, float* logits_host)
{
    ZNN_HOST_TRY
    m->arena->reset();
    Graph g(m->arena.get());
    Tensor* logits = model_forward(*m, g, x, batch, seq, on_device != 0);
    if (logits_host) check(znn_memcpy_d2h(logits_host, logits->data, logits->numel() * sizeof(float)), "read logits");
    ZNN_HOST_CATCH
}

// One batch of the example programs' evaluateModel (examples/cnn.zig:212-256): forward, the mean cross-entropy
// loss and computeAccuracy (:193-205) on the device; only the two scalars come back.
int znn_model_evaluate(znn_model* m, const float* x, const uint8_t* labels, int batch, int on_device, float* loss_host,
                       float* acc_host)
{
    ZNN_HOST_TRY
    if (m->kind == ZNN_MODEL_GPT || m->kind == ZNN_MODEL_BLOCK) throw Error(ZNN_ERR_INVALID, "evaluate: classifier models only");
    if (!x || !labels || batch <= 0) throw Error(ZNN_ERR_INVALID, "evaluate: x/labels is NULL or batch <= 0");
    m->arena->reset();
    Graph g(m->arena.get());
    const uint8_t* dev_labels = labels;
    if (!on_device) {
        uint8_t* t = (uint8_t*)m->arena->alloc((size_t)batch);
        check(znn_memcpy_h2d(t, labels, (size_t)batch), "upload labels");
        dev_labels = t;
    }
    Tensor* logits = model_forward(*m, g, x, batch, 0, on_device != 0);
    Tensor* loss = g.softmaxCrossEntropyU8(logits, dev_labels);
    float* acc = (float*)m->arena->alloc(sizeof(float));
    check(znn_accuracy_u8(logits->data, dev_labels, (int)logits->shape.dims[0], (int)logits->shape.dims[1], acc), "accuracy");
    if (loss_host) check(znn_memcpy_d2h(loss_host, loss->data, sizeof(float)), "read loss");
    if (acc_host) check(znn_memcpy_d2h(acc_host, acc, sizeof(float)), "read accuracy");
    ZNN_HOST_CATCH
}

int znn_model_block_fwd_bwd(znn_model* m, const float* x, const float* dy, int B, int T, float* y, float* dx)
{
    ZNN_HOST_TRY
    if (m->kind != ZNN_MODEL_BLOCK) throw Error(ZNN_ERR_INVALID, "not a transformer block model");
    m->arena->reset();
    Graph g(m->arena.get());
    const Shape s{(size_t)B, (size_t)T, m->in_features};
    Tensor* xt = g.array(s, x, dx != nullptr);
    Tensor* out = m->block.forward(g, xt);
    if (y) check(znn_memcpy_d2h(y, out->data, out->numel() * sizeof(float)), "read y");
    if (dy) {
        m->ps.zeroGrad();
        check(znn_memcpy_h2d(out->grad, dy, out->numel() * sizeof(float)), "upload dy");
        mark_grad_written(out);
        check(znn_sync(), "znn_sync");
        g.backwardWithGrad(out);
        if (dx) {
            ensure_grad(xt);
            check(znn_memcpy_d2h(dx, xt->grad, xt->numel() * sizeof(float)), "read dx");
        }
    }
    m->last_ops = (int)g.ops().size();
    ZNN_HOST_CATCH
}

int znn_model_block_fwd_bwd_device(znn_model* m, const float* x, const float* dy, int B, int T, float* y, float* dx)
{
    ZNN_HOST_TRY
    if (m->kind != ZNN_MODEL_BLOCK) throw Error(ZNN_ERR_INVALID, "not a transformer block model");
    m->arena->reset();
    Graph g(m->arena.get());
    const Shape s{(size_t)B, (size_t)T, m->in_features};
    Tensor* xt = g.arrayFromDevice(s, x, dx != nullptr);
    Tensor* out = m->block.forward(g, xt);
    if (y) check(znn_memcpy_d2d(y, out->data, out->numel() * sizeof(float)), "copy y");
    if (dy) {
        m->ps.zeroGrad();
        check(znn_memcpy_d2d(out->grad, dy, out->numel() * sizeof(float)), "copy dy");
        mark_grad_written(out);
        g.backwardWithGrad(out);
        if (dx) {
            ensure_grad(xt);
            check(znn_memcpy_d2d(dx, xt->grad, xt->numel() * sizeof(float)), "copy dx");
        }
    }
    m->last_ops = (int)g.ops().size();
    ZNN_HOST_CATCH
}

int znn_model_greedy_decode(znn_model* m, const float* prompt_ids, int batch, int prompt_len, int n_new, float* out_ids)
{
    ZNN_HOST_TRY
    if (m->kind != ZNN_MODEL_GPT) throw Error(ZNN_ERR_INVALID, "not a GPT model");
    const size_t block = m->gpt.cfg.block_size, V = m->gpt.cfg.vocab_size;
    std::vector<std::vector<float>> seqs(batch);
    for (int b = 0; b < batch; b++) seqs[b].assign(prompt_ids + (size_t)b * prompt_len, prompt_ids + (size_t)(b + 1) * prompt_len);
    void* p = nullptr;
    check(znn_malloc(&p, (size_t)batch * sizeof(float)), "decode scratch");
    float* next_dev = (float*)p;
    std::vector<float> next(batch), window;
    for (int step = 0; step < n_new; step++) {
        const size_t len = seqs[0].size();
        const size_t T = len < block ? len : block;  // last min(len, block_size) ids (transformer_gpt.zig:121-128)
        window.resize((size_t)batch * T);
        for (int b = 0; b < batch; b++)
            memcpy(&window[(size_t)b * T], &seqs[b][len - T], T * sizeof(float));
        m->arena->reset();
        Graph g(m->arena.get());
        Tensor* ids = g.array(Shape{(size_t)batch, T}, window.data(), false);
        Tensor* logits = m->gpt.forward(g, ids);  // [batch, T, V]
        for (int b = 0; b < batch; b++)           // first-maximum pick over the last position (:135-142)
            check(znn_argmax(logits->data + ((size_t)b * T + (T - 1)) * V, next_dev + b, 1, (int)V, 1), "argmax");
        check(znn_memcpy_d2h(next.data(), next_dev, (size_t)batch * sizeof(float)), "read tokens");
        for (int b = 0; b < batch; b++) {
            seqs[b].push_back(next[b]);
            out_ids[(size_t)b * n_new + step] = next[b];
        }
    }
    znn_free(next_dev);
    ZNN_HOST_CATCH
}

// Greedy decode with a key/value cache: position p of every sequence goes through the layers once; its key and value
// rows are appended to per-layer caches [batch, head, Tmax, hs] and its query attends to rows 0..p.  The arithmetic per
// element is that of the full re-forward (same operators: Embedding, Add, RmsNorm, Linear, scaled dot products, row
// softmax over the visible positions, GELU), so the logits agree to GEMM rounding and the greedy tokens are the same
// unless two logits tie within that rounding.  No host synchronisation inside the loop: the picked ids stay on the device.
int znn_model_greedy_decode_kv(znn_model* m, const float* prompt_ids, int batch, int prompt_len, int n_new, float* out_ids)
{
    ZNN_HOST_TRY
    if (m->kind != ZNN_MODEL_GPT) throw Error(ZNN_ERR_INVALID, "not a GPT model");
    const GPTConfig& cfg = m->gpt.cfg;
    const size_t C = cfg.n_embd, nh = cfg.n_head, hs = C / nh, V = cfg.vocab_size, L = cfg.n_layer;
    const size_t Tmax = (size_t)prompt_len + (size_t)n_new;
    if (prompt_len < 1 || n_new < 1 || batch < 1) throw Error(ZNN_ERR_INVALID, "empty prompt, batch or request");
    if (Tmax - 1 > cfg.block_size)
        throw Error(ZNN_ERR_INVALID, "the key/value cache decode needs prompt_len + n_new - 1 <= block_size (the window must not slide)");
    const size_t B = (size_t)batch;
    m->arena->reset();
    auto dev = [&](size_t n) { return (float*)m->arena->alloc(n * sizeof(float)); };
    float* ids_all = dev(B * Tmax);           // [Tmax][B]: prompt ids, then the picked ids
    float* posv = dev(B);
    float *x = dev(B * C), *x1 = dev(B * C), *tmp = dev(B * C), *xn = dev(B * C);
    float *q = dev(B * C), *k = dev(B * C), *v = dev(B * C), *y = dev(B * C);
    float *att = dev(B * nh * Tmax), *prob = dev(B * nh * Tmax);
    float *hid = dev(B * 4 * C), *act = dev(B * 4 * C), *logits = dev(B * V);
    std::vector<float*> Kc(L), Vc(L);
    for (size_t l = 0; l < L; l++) {
        Kc[l] = dev(B * nh * Tmax * hs);
        Vc[l] = dev(B * nh * Tmax * hs);
    }
    {   // prompt, transposed to [position][sequence]
        std::vector<float> pt((size_t)prompt_len * B);
        for (size_t b = 0; b < B; b++)
            for (int t = 0; t < prompt_len; t++) pt[(size_t)t * B + b] = prompt_ids[b * prompt_len + t];
        check(znn_memcpy_h2d(ids_all, pt.data(), pt.size() * sizeof(float)), "upload prompt");
        check(znn_sync(), "znn_sync");
    }
    const float scale = 1.0f / sqrtf((float)hs);
    auto linear = [&](const Linear& lin, const float* in, float* out, size_t K, size_t N) {
        check(znn_linear_fwd(in, lin.weight->data, lin.bias->data, out, (int)B, (int)K, (int)N), "Linear");
    };
    for (size_t pos = 0; pos + 1 < Tmax; pos++) {
        const float* ids = ids_all + pos * B;
        check(znn_fill(posv, (float)pos, B), "positions");
        check(znn_embedding_fwd(m->gpt.token_embedding.weight->data, ids, x, B, (int)C, (int)V), "token embedding");
        check(znn_embedding_fwd(m->gpt.position_embedding.weight->data, posv, tmp, B, (int)C, (int)cfg.block_size), "position embedding");
        check(znn_add_fwd(x, tmp, x1, B * C), "embedding sum");
        std::swap(x, x1);
        const int len = (int)pos + 1;
        for (size_t l = 0; l < L; l++) {
            const TransformerBlock& blk = m->gpt.h[l];
            check(znn_rmsnorm_fwd(x, blk.ln_1.weight->data, blk.ln_1.eps, xn, B, (int)C), "ln_1");
            linear(blk.attn.q_attn, xn, q, C, C);
            linear(blk.attn.k_attn, xn, k, C, C);
            linear(blk.attn.v_attn, xn, v, C, C);
            // rows [b, h, pos, :] of the caches
            check(znn_memcpy2d_d2d(Kc[l] + pos * hs, Tmax * hs * sizeof(float), k, hs * sizeof(float), hs * sizeof(float), B * nh), "K cache");
            check(znn_memcpy2d_d2d(Vc[l] + pos * hs, Tmax * hs * sizeof(float), v, hs * sizeof(float), hs * sizeof(float), B * nh), "V cache");
            // scores[b,h,0:len] = scale * q[b,h,:] . K[b,h,0:len,:]^T   (rows of `len` floats, packed)
            check(znn_sgemm_batched_strided(ZNN_NO_TRANS, ZNN_TRANS, 1, len, (int)hs, scale, q, (int)hs, (long long)hs, Kc[l], (int)hs,
                                            (long long)(Tmax * hs), 0.0f, att, len, (long long)len, (int)(B * nh)),
                  "scores");
            // softmax over the visible positions (the causal mask of the full forward leaves exactly these)
            check(znn_softmax_fwd(att, prob, B * nh, len), "softmax");
            check(znn_sgemm_batched_strided(ZNN_NO_TRANS, ZNN_NO_TRANS, 1, (int)hs, len, 1.0f, prob, len, (long long)len, Vc[l], (int)hs,
                                            (long long)(Tmax * hs), 0.0f, y, (int)hs, (long long)hs, (int)(B * nh)),
                  "P.V");
            linear(blk.attn.c_proj, y, tmp, C, C);
            check(znn_add_fwd(x, tmp, x1, B * C), "residual 1");
            check(znn_rmsnorm_fwd(x1, blk.ln_2.weight->data, blk.ln_2.eps, xn, B, (int)C), "ln_2");
            linear(blk.mlp.c_fc, xn, hid, C, 4 * C);
            check(znn_gelu_fwd(hid, act, B * 4 * C), "gelu");
            linear(blk.mlp.c_proj, act, tmp, 4 * C, C);
            check(znn_add_fwd(x1, tmp, x, B * C), "residual 2");
        }
        if (pos + 1 >= (size_t)prompt_len) {   // the next position is a new token: pick it
            check(znn_rmsnorm_fwd(x, m->gpt.ln_f.weight->data, m->gpt.ln_f.eps, xn, B, (int)C), "ln_f");
            linear(m->gpt.lm_head, xn, logits, C, V);
            check(znn_argmax(logits, ids_all + (pos + 1) * B, (int)B, (int)V, 1), "argmax");   // first maximum per row
        }
    }
    std::vector<float> picked((size_t)n_new * B);
    check(znn_memcpy_d2h(picked.data(), ids_all + (size_t)prompt_len * B, picked.size() * sizeof(float)), "read tokens");
    for (size_t b = 0; b < B; b++)
        for (int t = 0; t < n_new; t++) out_ids[b * n_new + t] = picked[(size_t)t * B + b];
    ZNN_HOST_CATCH
}

// ---- checkpoint files in the reference's layout (src/nn.zig:173-455): 8-byte little-endian header length, a JSON
// header {"name":{"dtype":"F32","shape":[..],"data_offsets":[start,end]},...} without spaces, entries in parameter
// (struct-field) order, padded with spaces to a multiple of 8, then the fp32 data back to back in the same order ----
static std::string checkpoint_header(const ParamStore& ps)
{
    std::string h = "{";
    size_t off = 0;
    bool first = true;
    for (const ParamInfo& pi : ps.params()) {
        if (!first) h += ",";
        first = false;
        h += "\"" + pi.name + "\":{\"dtype\":\"F32\",\"shape\":[";
        for (size_t i = 0; i < pi.tensor->shape.len; i++) {
            if (i) h += ",";
            h += std::to_string(pi.tensor->shape.dims[i]);
        }
        const size_t bytes = pi.tensor->numel() * 4;
        h += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + bytes) + "]}";
        off += bytes;
    }
    h += "}";
    h.append((8 - h.size() % 8) % 8, ' ');
    return h;
}

// slab = the values slab (the model file) or the velocity slab (the optimizer-state file): same layout, same offsets
static void save_slab(znn_model* m, const char* path, float* slab)
{
    if (!path) throw Error(ZNN_ERR_INVALID, "path is NULL");
    const std::string header = checkpoint_header(m->ps);
    FILE* f = fopen(path, "wb");
    if (!f) throw Error(ZNN_ERR_INVALID, std::string("cannot create ") + path);
    const uint64_t hl = header.size();
    unsigned char le[8];
    for (int i = 0; i < 8; i++) le[i] = (unsigned char)(hl >> (8 * i));
    bool ok = fwrite(le, 1, 8, f) == 8 && fwrite(header.data(), 1, header.size(), f) == header.size();
    std::vector<float> host;
    for (const ParamInfo& pi : m->ps.params()) {
        if (!ok) break;
        host.resize(pi.tensor->numel());
        check(znn_memcpy_d2h(host.data(), slab + pi.offset, host.size() * sizeof(float)), "read parameter");
        ok = fwrite(host.data(), sizeof(float), host.size(), f) == host.size();
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) throw Error(ZNN_ERR_INVALID, std::string("write to ") + path + " failed");
}

int znn_model_save(znn_model* m, const char* path)
{
    ZNN_HOST_TRY
    save_slab(m, path, m->ps.values());
    ZNN_HOST_CATCH
}

int znn_model_save_optimizer(znn_model* m, const char* path)
{
    ZNN_HOST_TRY
    save_slab(m, path, m->ps.velocities());
    if (m->use_adam) save_slab(m, (std::string(path) + ".v2").c_str(), m->ps.second_moments());
    ZNN_HOST_CATCH
}

// value of `"key":` inside the JSON object that starts at obj (a '{'); returns the position after the colon or npos
static size_t json_member(const std::string& h, size_t obj, size_t obj_end, const char* key)
{
    const std::string pat = std::string("\"") + key + "\"";
    size_t p = h.find(pat, obj);
    if (p == std::string::npos || p >= obj_end) return std::string::npos;
    p = h.find(':', p + pat.size());
    return (p == std::string::npos || p >= obj_end) ? std::string::npos : p + 1;
}

static std::vector<long long> json_int_array(const std::string& h, size_t p, size_t obj_end)
{
    std::vector<long long> v;
    p = h.find('[', p);
    if (p == std::string::npos || p >= obj_end) throw Error(ZNN_ERR_INVALID, "checkpoint header: array expected");
    const size_t e = h.find(']', p);
    if (e == std::string::npos || e > obj_end) throw Error(ZNN_ERR_INVALID, "checkpoint header: unterminated array");
    size_t i = p + 1;
    while (i < e) {
        while (i < e && (h[i] == ' ' || h[i] == ',')) i++;
        if (i >= e) break;
        size_t used = 0;
        v.push_back(std::stoll(h.substr(i, e - i), &used));
        i += used;
    }
    return v;
}

static void load_slab(znn_model* m, const char* path, float* slab)
{
    if (!path) throw Error(ZNN_ERR_INVALID, "path is NULL");
    FILE* f = fopen(path, "rb");
    if (!f) throw Error(ZNN_ERR_INVALID, std::string("cannot open ") + path);
    struct Closer { FILE* f; ~Closer() { if (f) fclose(f); } } closer{f};
    unsigned char le[8];
    if (fread(le, 1, 8, f) != 8) throw Error(ZNN_ERR_INVALID, "checkpoint: no header length");
    uint64_t hl = 0;
    for (int i = 0; i < 8; i++) hl |= (uint64_t)le[i] << (8 * i);
    if (hl == 0 || hl > (1ull << 30)) throw Error(ZNN_ERR_INVALID, "checkpoint: implausible header length");
    std::string h(hl, ' ');
    if (fread(&h[0], 1, hl, f) != hl) throw Error(ZNN_ERR_INVALID, "checkpoint: truncated header");
    size_t current = 0;   // the reference reads sequentially and refuses offsets that go backwards (nn.zig:431-434)
    std::vector<float> host;
    for (const ParamInfo& pi : m->ps.params()) {
        const std::string key = "\"" + pi.name + "\"";
        size_t k = h.find(key + ":");
        if (k == std::string::npos) k = h.find(key + " :");
        if (k == std::string::npos) throw Error(ZNN_ERR_INVALID, "checkpoint: tensor '" + pi.name + "' not found in the header");
        const size_t obj = h.find('{', k + key.size());
        const size_t obj_end = obj == std::string::npos ? obj : h.find('}', obj);
        if (obj_end == std::string::npos) throw Error(ZNN_ERR_INVALID, "checkpoint header: malformed entry for " + pi.name);
        const size_t dt = json_member(h, obj, obj_end, "dtype");
        if (dt == std::string::npos || h.find("\"F32\"", dt) == std::string::npos || h.find("\"F32\"", dt) > obj_end)
            throw Error(ZNN_ERR_INVALID, "checkpoint: '" + pi.name + "' is not F32");
        const size_t sh = json_member(h, obj, obj_end, "shape");
        const size_t of = json_member(h, obj, obj_end, "data_offsets");
        if (sh == std::string::npos || of == std::string::npos)
            throw Error(ZNN_ERR_INVALID, "checkpoint header: shape or data_offsets missing for " + pi.name);
        const std::vector<long long> shape = json_int_array(h, sh, obj_end), offs = json_int_array(h, of, obj_end);
        if (shape.size() != pi.tensor->shape.len) throw Error(ZNN_ERR_INVALID, "checkpoint: rank mismatch for " + pi.name);
        for (size_t i = 0; i < shape.size(); i++)
            if ((size_t)shape[i] != pi.tensor->shape.dims[i]) throw Error(ZNN_ERR_INVALID, "checkpoint: shape mismatch for " + pi.name);
        const size_t bytes = pi.tensor->numel() * 4;
        if (offs.size() != 2 || (size_t)(offs[1] - offs[0]) != bytes) throw Error(ZNN_ERR_INVALID, "checkpoint: size mismatch for " + pi.name);
        if ((size_t)offs[0] < current) throw Error(ZNN_ERR_INVALID, "checkpoint: offsets of '" + pi.name + "' go backwards");
        if (fseek(f, (long)(8 + hl + (uint64_t)offs[0]), SEEK_SET) != 0) throw Error(ZNN_ERR_INVALID, "checkpoint: seek failed");
        host.resize(pi.tensor->numel());
        if (fread(host.data(), 1, bytes, f) != bytes) throw Error(ZNN_ERR_INVALID, "checkpoint: truncated data for " + pi.name);
        check(znn_memcpy_h2d(slab + pi.offset, host.data(), bytes), "write parameter");
        check(znn_sync(), "znn_sync");
        current = (size_t)offs[1];
    }
}

int znn_model_load(znn_model* m, const char* path)
{
    ZNN_HOST_TRY
    load_slab(m, path, m->ps.values());
    ZNN_HOST_CATCH
}

int znn_model_load_optimizer(znn_model* m, const char* path)
{
    ZNN_HOST_TRY
    load_slab(m, path, m->ps.velocities());
    if (m->use_adam) load_slab(m, (std::string(path) + ".v2").c_str(), m->ps.second_moments());
    ZNN_HOST_CATCH
}

int znn_model_arena_high_water(znn_model* m, long long* bytes)
{
    ZNN_HOST_TRY
    if (bytes) *bytes = (long long)m->arena->high_water();
    ZNN_HOST_CATCH
}

int znn_model_graph_replays(znn_model* m, long long* n)
{
    ZNN_HOST_TRY
    if (n) *n = m->graph_replays;
    ZNN_HOST_CATCH
}

int znn_model_last_step_ops(znn_model* m, int* n_ops)
{
    ZNN_HOST_TRY
    if (n_ops) *n_ops = m->last_ops;
    ZNN_HOST_CATCH
}

}  // extern "C"

// ------------------------------------------------------------------ arena, parameter slabs, initialisation
struct znn_arena {
    std::unique_ptr<Arena> a;
};

struct znn_param_slab {
    size_t total = 0;
    std::vector<size_t> offsets;
    float *w = nullptr, *g = nullptr, *v = nullptr;
};

extern "C" {

int znn_arena_create(size_t bytes, znn_arena** out)
{
    ZNN_HOST_TRY
    if (!out) throw Error(ZNN_ERR_INVALID, "out is NULL");
    std::unique_ptr<znn_arena> a(new znn_arena());
    a->a.reset(new Arena(bytes));
    *out = a.release();
    ZNN_HOST_CATCH
}

int znn_arena_alloc(znn_arena* a, size_t bytes, void** ptr)
{
    ZNN_HOST_TRY
    if (!a || !ptr) throw Error(ZNN_ERR_INVALID, "arena/ptr is NULL");
    *ptr = a->a->alloc(bytes);
    ZNN_HOST_CATCH
}

int znn_arena_reset(znn_arena* a)
{
    ZNN_HOST_TRY
    if (!a) throw Error(ZNN_ERR_INVALID, "arena is NULL");
    a->a->reset();
    ZNN_HOST_CATCH
}

int znn_arena_usage(znn_arena* a, size_t* used, size_t* high_water, size_t* capacity)
{
    ZNN_HOST_TRY
    if (!a) throw Error(ZNN_ERR_INVALID, "arena is NULL");
    if (used) *used = a->a->used();
    if (high_water) *high_water = a->a->high_water();
    if (capacity) *capacity = a->a->capacity();
    ZNN_HOST_CATCH
}

int znn_arena_destroy(znn_arena* a)
{
    ZNN_HOST_TRY
    if (a) {
        znn_sync();
        delete a;
    }
    ZNN_HOST_CATCH
}

int znn_param_slab_create(const size_t* counts, int n, znn_param_slab** out)
{
    ZNN_HOST_TRY
    if (!counts || n <= 0 || !out) throw Error(ZNN_ERR_INVALID, "counts/out is NULL or n <= 0");
    std::unique_ptr<znn_param_slab> s(new znn_param_slab());
    for (int i = 0; i < n; i++) {
        s->offsets.push_back(s->total);
        s->total += (counts[i] + 3) & ~(size_t)3;   // every parameter starts 16-byte aligned
    }
    const size_t bytes = s->total * sizeof(float);
    void* p = nullptr;
    float** slabs[3] = {&s->w, &s->g, &s->v};
    for (float** slab : slabs) {
        const int rc = znn_malloc(&p, bytes);
        if (rc != ZNN_OK) {
            znn_free(s->w);
            znn_free(s->g);
            znn_free(s->v);
            check(rc, "znn_param_slab_create");
        }
        *slab = (float*)p;
        check(znn_memset(p, 0, bytes), "znn_memset");
    }
    *out = s.release();
    ZNN_HOST_CATCH
}

int znn_param_slab_total(znn_param_slab* s, size_t* total_floats)
{
    ZNN_HOST_TRY
    if (!s || !total_floats) throw Error(ZNN_ERR_INVALID, "slab/total_floats is NULL");
    *total_floats = s->total;
    ZNN_HOST_CATCH
}

int znn_param_slab_tensor(znn_param_slab* s, int i, float** value, float** grad, float** velocity, size_t* offset)
{
    ZNN_HOST_TRY
    if (!s || i < 0 || (size_t)i >= s->offsets.size()) throw Error(ZNN_ERR_INVALID, "slab is NULL or index out of range");
    const size_t off = s->offsets[i];
    if (value) *value = s->w + off;
    if (grad) *grad = s->g + off;
    if (velocity) *velocity = s->v + off;
    if (offset) *offset = off;
    ZNN_HOST_CATCH
}

int znn_param_slab_zero_grad(znn_param_slab* s)
{
    ZNN_HOST_TRY
    if (!s) throw Error(ZNN_ERR_INVALID, "slab is NULL");
    check(znn_memset(s->g, 0, s->total * sizeof(float)), "zeroGrad");
    ZNN_HOST_CATCH
}

int znn_param_slab_sgd_step(znn_param_slab* s, float lr, float momentum, float grad_scale)
{
    ZNN_HOST_TRY
    if (!s) throw Error(ZNN_ERR_INVALID, "slab is NULL");
    check(znn_sgd_step(s->w, s->g, momentum > 0.0f ? s->v : nullptr, lr, momentum, grad_scale, s->total), "SGD step");
    ZNN_HOST_CATCH
}

int znn_param_slab_allreduce_grads(znn_param_slab* s)
{
    ZNN_HOST_TRY
    if (!s) throw Error(ZNN_ERR_INVALID, "slab is NULL");
    check(znn_dp_allreduce(s->g, s->total), "gradient all-reduce");
    ZNN_HOST_CATCH
}

int znn_param_slab_destroy(znn_param_slab* s)
{
    ZNN_HOST_TRY
    if (s) {
        znn_sync();
        znn_free(s->w);
        znn_free(s->g);
        znn_free(s->v);
        delete s;
    }
    ZNN_HOST_CATCH
}

// The modules' init rule (src/nn.zig:22-23, :71-72, :520, :565): weights He-normal with the module's fan-in, biases 0,
// norm gains 1.  Parameter i draws with seed + i.
int znn_model_init_weights(znn_model* m, unsigned long long seed)
{
    ZNN_HOST_TRY
    if (!m) throw Error(ZNN_ERR_INVALID, "model is NULL");
    unsigned long long k = 0;
    for (const ParamInfo& pi : m->ps.params()) {
        const size_t n = pi.tensor->numel();
        const bool is_bias = pi.name.size() >= 5 && pi.name.compare(pi.name.size() - 5, 5, ".bias") == 0;
        if (pi.fan_in > 0) check(znn_init_he_normal(pi.tensor->data, n, pi.fan_in, seed + k), "znn_init_he_normal");
        else check(znn_fill(pi.tensor->data, is_bias ? 0.0f : 1.0f, n), "znn_fill");
        k++;
    }
    drop_graph(m);
    ZNN_HOST_CATCH
}

int znn_debug_bucket_schedule_run(const size_t* offsets, int n_params, size_t total, size_t bucket_floats, const int* uses,
                                  const int* completion_order, int n_events, znn_debug_allreduce_fn fn, void* ctx,
                                  int* n_buckets)
{
    ZNN_HOST_TRY
    if (!offsets || !uses || n_params <= 0 || !fn) throw Error(ZNN_ERR_INVALID, "offsets/uses/fn is NULL or n_params <= 0");
    BucketSchedule sched(std::vector<size_t>(offsets, offsets + n_params), total, bucket_floats,
                         std::vector<int>(uses, uses + n_params),
                         [fn, ctx](size_t begin, size_t count) { return fn(ctx, begin, count); });
    if (n_buckets) *n_buckets = (int)sched.buckets();
    int rc = 0;
    for (int e = 0; e < n_events && rc == 0; e++) rc = sched.after(completion_order[e]);
    if (rc == 0) rc = sched.finish();
    if (rc != 0) return znn::fail(rc, "bucket schedule: the reduction callback returned %d", rc);
    ZNN_HOST_CATCH
}

}  // extern "C"
