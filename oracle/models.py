"""The reference's modules and example models (src/nn.zig, examples/*.zig) written
once against a graph interface with the reference's builder names.  TEST
INFRASTRUCTURE: run on oracle.ograph.OGraph they give the CPU result the CUDA
path is compared with; the same functions also run on znn_b200.graph.Graph.

Parameters are passed as a dict name -> graph tensor, with the dotted names the
reference's save format uses (decoder.h.0.attn.q_attn.weight ...).
"""
import math

import numpy as np


def linear(g, P, name, x):                     # src/nn.zig:44-51
    return g.addBias(g.matmul(x, P[name + ".weight"]), P[name + ".bias"])


def mlp_net(g, P, x):                          # examples/fashion_mnist.zig:36-42
    a1 = g.relu(linear(g, P, "fc1", x))
    a2 = g.relu(linear(g, P, "fc2", a1))
    return linear(g, P, "fc3", a2)


def cnn_net(g, P, x, reference_shape=True):    # examples/cnn.zig:35-56
    B = x.shape[0]
    xr = g.reshape(x, (B, 1, 28, 28))
    if reference_shape:
        p1 = g.maxpool2d(g.relu(g.conv2d(xr, P["conv1.weight"], P["conv1.bias"])), 2, 2)
        p2 = g.maxpool2d(g.relu(g.conv2d(p1, P["conv2.weight"], P["conv2.bias"])), 2, 2)
        a3 = g.relu(g.conv2d(p2, P["conv3.weight"], P["conv3.bias"]))
        return linear(g, P, "fc1", g.reshape(a3, (B, 144)))
    p1 = g.maxpool2d(g.relu(g.conv2d(xr, P["conv1.weight"], P["conv1.bias"], 1)), 2, 2)
    p2 = g.maxpool2d(g.relu(g.conv2d(p1, P["conv2.weight"], P["conv2.bias"], 1)), 2, 2)
    a = g.relu(linear(g, P, "fc1", g.reshape(p2, (B, 3136))))
    return linear(g, P, "fc2", a)


def mlp_block(g, P, name, x):                  # src/nn.zig:638-685
    shp = x.shape
    x2 = g.reshape(x, (shp[0] * shp[1], shp[2])) if len(shp) == 3 else x
    h2 = linear(g, P, name + ".c_proj", g.gelu(linear(g, P, name + ".c_fc", x2)))
    return g.reshape(h2, shp) if len(shp) == 3 else h2


def causal_self_attention(g, P, name, x, n_head):   # src/nn.zig:752-937, the literal op sequence
    B, T, C = x.shape
    hs = C // n_head
    x2 = g.reshape(x, (B * T, C))
    q2, k2, v2 = (linear(g, P, f"{name}.{w}", x2) for w in ("q_attn", "k_attn", "v_attn"))
    q, k, v = (g.transposeND(g.reshape(t, (B, T, n_head, hs)), 1, 2) for t in (q2, k2, v2))
    att = g.batchMatMul(q, g.transposeND(k, 2, 3))
    scale = np.float32(1.0) / np.sqrt(np.float32(hs))
    att_scaled = g.mulScalar(att, float(scale))
    mask = np.zeros((B, n_head, T, T), np.float32)
    iu = np.triu_indices(T, 1)
    mask[:, :, iu[0], iu[1]] = -1e9            # nn.zig:847-860
    att_sm = g.softmax(g.add(att_scaled, g.array(mask, False)))
    y = g.transposeND(g.batchMatMul(att_sm, v), 1, 2)
    y2 = g.reshape(g.reshape(y, (B, T, C)), (B * T, C))
    return g.reshape(linear(g, P, name + ".c_proj", y2), (B, T, C))


def transformer_block(g, P, name, x, n_head, eps=1e-5):   # src/nn.zig:996-1021
    x_attn = causal_self_attention(g, P, name + ".attn", g.rmsNorm(x, P[name + ".ln_1.weight"], eps), n_head)
    x1 = g.add(x, x_attn)
    x_mlp = mlp_block(g, P, name + ".mlp", g.rmsNorm(x1, P[name + ".ln_2.weight"], eps))
    return g.add(x1, x_mlp)


def gpt(g, P, ids, cfg):                       # src/nn.zig:1172-1233; ids: graph tensor [B, T] of fp32 token ids
    B, T = ids.shape
    tok = g.embedding(P["token_embedding.weight"], ids)
    pos = g.array(np.tile(np.arange(T, dtype=np.float32), (B, 1)), False)
    h = g.add(tok, g.embedding(P["position_embedding.weight"], pos))
    for i in range(cfg["n_layer"]):
        h = transformer_block(g, P, f"decoder.h.{i}", h, cfg["n_head"])
    out = g.rmsNorm(h, P["decoder.ln_f.weight"], 1e-5)
    logits2 = linear(g, P, "lm_head", g.reshape(out, (B * T, cfg["n_embd"])))
    return g.reshape(logits2, (B, T, cfg["vocab_size"]))


def param_shapes(kind, cfg=None):
    """name -> (shape, fan_in) in the reference's collectParameters order (src/nn.zig:142-171)."""
    out = []

    def lin(n, i, o):
        out.append((n + ".weight", (i, o), i))
        out.append((n + ".bias", (1, o), 0))

    def conv(n, ci, co, k):
        out.append((n + ".weight", (co, ci, k, k), ci * k * k))
        out.append((n + ".bias", (co,), 0))

    def block(n, d):
        out.append((n + ".ln_1.weight", (d,), 0))
        for w in ("q_attn", "k_attn", "v_attn", "c_proj"):
            lin(f"{n}.attn.{w}", d, d)
        out.append((n + ".ln_2.weight", (d,), 0))
        lin(n + ".mlp.c_fc", d, 4 * d)
        lin(n + ".mlp.c_proj", 4 * d, d)

    if kind == "mlp":
        i, h1, h2, o = cfg
        lin("fc1", i, h1), lin("fc2", h1, h2), lin("fc3", h2, o)
    elif kind == "cnn_ref":
        conv("conv1", 1, 4, 3), conv("conv2", 4, 8, 3), conv("conv3", 8, 16, 3), lin("fc1", 144, 10)
    elif kind == "cnn_padded":
        conv("conv1", 1, 32, 3), conv("conv2", 32, 64, 3), lin("fc1", 3136, 128), lin("fc2", 128, 10)
    elif kind == "block":
        block("block", cfg["n_embd"])
    elif kind == "gpt":
        d = cfg["n_embd"]
        out.append(("token_embedding.weight", (cfg["vocab_size"], d), d))
        out.append(("position_embedding.weight", (cfg["block_size"], d), d))
        for i in range(cfg["n_layer"]):
            block(f"decoder.h.{i}", d)
        out.append(("decoder.ln_f.weight", (d,), 0))
        lin("lm_head", d, cfg["vocab_size"])
    else:
        raise ValueError(kind)
    return out


def init_params(kind, cfg=None, seed=0, scheme="he"):
    """Seeded synthetic parameters (the reference's Zig PRNG stream cannot be reproduced):
    'he' = N(0, sqrt(2/fan_in)) as src/nn.zig:1336-1341, 'n002' = N(0, 0.02), 'uniform' = U(+-1/sqrt(fan_in));
    biases 0, norm gains 1."""
    r = np.random.default_rng(seed)
    P = {}
    for name, shape, fan_in in param_shapes(kind, cfg):
        if fan_in == 0:
            P[name] = np.ones(shape, np.float32) if name.endswith(("ln_1.weight", "ln_2.weight", "ln_f.weight")) \
                else np.zeros(shape, np.float32)
        elif scheme == "he":
            P[name] = (r.standard_normal(shape) * math.sqrt(2.0 / fan_in)).astype(np.float32)
        elif scheme == "n002":
            P[name] = (r.standard_normal(shape) * 0.02).astype(np.float32)
        else:
            b = 1.0 / math.sqrt(fan_in)
            P[name] = r.uniform(-b, b, shape).astype(np.float32)
    return P


class OracleTrainer:
    """The example programs' training step on the CPU oracle: new graph -> forward -> SoftmaxCrossEntropy ->
    zeroGrad -> backward -> SGD (examples/fashion_mnist.zig:131-167, src/optim.zig:50-66)."""

    def __init__(self, kind, params, cfg=None, lr=0.01, momentum=0.9, adam=None):
        """adam = (beta1, beta2, eps): AdamOptimizer (src/optim.zig:69-152) instead of SGD."""
        from . import ograph, zo
        self.og, self.zo = ograph, zo
        self.kind, self.cfg, self.lr, self.momentum = kind, cfg, lr, momentum
        self.P = {k: v.copy() for k, v in params.items()}
        self.V = {k: np.zeros_like(v) for k, v in params.items()} if (momentum > 0 or adam) else None
        self.adam, self.t = adam, 0.0
        self.V2 = {k: np.zeros_like(v) for k, v in params.items()} if adam else None
        self.grads = None

    def forward_logits(self, g, P, x):
        if self.kind == "mlp":
            return mlp_net(g, P, g.array(x, False))
        if self.kind in ("cnn_ref", "cnn_padded"):
            return cnn_net(g, P, g.array(x, False), self.kind == "cnn_ref")
        if self.kind == "gpt":
            lg = gpt(g, P, g.array(x, False), self.cfg)
            return g.reshape(lg, (lg.shape[0] * lg.shape[1], lg.shape[2]))
        raise ValueError(self.kind)

    def loss_and_grads(self, x, targets):
        g = self.og.OGraph()
        P = {k: g.array(v, True) for k, v in self.P.items()}
        logits = self.forward_logits(g, P, x)
        loss = g.softmaxCrossEntropy(logits, np.asarray(targets, np.int32).reshape(-1))
        g.backward(loss)
        self.grads = {k: t.grad.reshape(self.P[k].shape) for k, t in P.items()}
        return float(loss.data.reshape(-1)[0]), logits.data

    def step(self, x, targets, grad_scale=1.0):
        loss, logits = self.loss_and_grads(x, targets)
        self.apply(self.grads, grad_scale)
        return loss, logits

    def apply(self, grads, grad_scale=1.0):
        if self.adam:
            self.t += 1.0
        for k in self.P:
            gk = np.ascontiguousarray(grads[k], np.float32)
            if grad_scale != 1.0:
                gk = (gk * np.float32(grad_scale)).astype(np.float32)
            if self.adam:
                self.zo.adam_step(self.P[k].reshape(-1), gk.reshape(-1), self.V[k].reshape(-1), self.V2[k].reshape(-1),
                                  self.lr, self.adam[0], self.adam[1], self.adam[2], self.t)
                continue
            self.zo.sgd_step(self.P[k].reshape(-1), gk.reshape(-1), self.V[k].reshape(-1) if self.V else None,
                             self.lr, self.momentum)
