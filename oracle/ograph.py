"""CPU restatement of the reference's autodiff Graph (src/autodiff.zig:1237-2264)
over the C oracle's operator loops.  TEST INFRASTRUCTURE ONLY.

Bookkeeping follows the reference: every builder runs the eager forward, sets
requires_grad to the OR of its inputs, allocates a zeroed grad, appends an Op to
the tape; backward() sorts topologically by DFS post-order over creator.inputs
(:2239-2249), seeds loss.grad[0] = 1 (:2203) and sweeps in reverse calling each
creator's backward arm, which accumulates into its inputs' grads.
"""
import numpy as np

from . import zo


class OTensor:
    def __init__(self, data, requires_grad=False):
        self.data = np.ascontiguousarray(data, dtype=np.float32)
        self.requires_grad = bool(requires_grad)
        self.grad = np.zeros_like(self.data) if requires_grad else None
        self.creator = None

    @property
    def shape(self):
        return self.data.shape


class OOp:
    def __init__(self, kind, inputs, output, **ctx):
        self.kind, self.inputs, self.output, self.ctx = kind, inputs, output, ctx


class OGraph:
    def __init__(self):
        self.tensors, self.ops = [], []

    # ---- creators (:1260-1326)
    def array(self, data, requires_grad=False):
        t = OTensor(np.array(data, dtype=np.float32, copy=True), requires_grad)
        self.tensors.append(t)
        return t

    def _out(self, data, kind, inputs, **ctx):
        rg = any(i is not None and i.requires_grad for i in inputs)
        t = OTensor(data, rg)
        self.tensors.append(t)
        op = OOp(kind, [i for i in inputs if i is not None], t, **ctx)
        t.creator = op
        self.ops.append(op)
        return t

    # ---- builders
    def matmul(self, A, B):                       # :1414
        return self._out(zo.matmul_fwd(A.data, B.data), "MatMul", [A, B])

    def addBias(self, A, bias):                   # :1446
        return self._out(zo.add_bias_fwd(A.data, bias.data.reshape(-1)), "AddBias", [A, bias])

    def relu(self, A):                            # :1478
        return self._out(zo.relu_fwd(A.data), "Relu", [A])

    def gelu(self, A):                            # :1508
        return self._out(zo.gelu_fwd(A.data), "Gelu", [A])

    def softmaxCrossEntropy(self, logits, targets):   # :1630
        loss, probs = zo.softmax_xent_fwd(logits.data, targets)
        t = OTensor(loss.reshape(1, 1), logits.requires_grad)
        self.tensors.append(t)
        op = OOp("SoftmaxCrossEntropy", [logits], t, probs=probs, targets=np.asarray(targets, np.int32))
        t.creator = op
        self.ops.append(op)
        return t

    def reshape(self, A, new_shape):              # :1329: shares data, own grad
        t = OTensor.__new__(OTensor)
        t.data = A.data.reshape(new_shape)        # a view: aliases A.data
        t.requires_grad = A.requires_grad
        t.grad = np.zeros(new_shape, np.float32) if A.requires_grad else None
        t.creator = None
        self.tensors.append(t)
        op = OOp("Reshape", [A], t)
        t.creator = op
        self.ops.append(op)
        return t

    def transposeND(self, A, d0, d1):             # :1378
        return self._out(zo.transpose_fwd(A.data, d0, d1), "Transpose", [A], d0=d0, d1=d1)

    def mulScalar(self, A, v):                    # :1910
        return self._out(zo.mul_scalar_fwd(A.data, v), "MulScalar", [A], v=float(v))

    def add(self, A, B):                          # :1972
        return self._out(zo.add_fwd(A.data, B.data).reshape(A.shape), "Add", [A, B])

    def conv2d(self, A, W, bias=None, pad=0):     # :2003
        b = bias.data.reshape(-1) if bias is not None else None
        return self._out(zo.conv2d_fwd(A.data, W.data, b, pad), "Conv2D", [A, W, bias], pad=pad)

    def maxpool2d(self, A, pool, stride):         # :2038
        return self._out(zo.maxpool2d_fwd(A.data, pool, stride), "MaxPool2D", [A], pool=pool, stride=stride)

    def softmax(self, A):                         # :2068
        return self._out(zo.softmax_fwd(A.data), "Softmax", [A])

    def rmsNorm(self, X, G, eps):                 # :2098
        return self._out(zo.rmsnorm_fwd(X.data, G.data.reshape(-1), eps), "RmsNorm", [X, G], eps=float(eps))

    def batchMatMul(self, A, B):                  # :2129
        return self._out(zo.batch_matmul_fwd(A.data, B.data), "BatchMatMul", [A, B])

    def embedding(self, W, X):                    # :2160: requires_grad follows W only
        t = OTensor(zo.embedding_fwd(W.data, X.data), W.requires_grad)
        self.tensors.append(t)
        op = OOp("Embedding", [W, X], t)
        t.creator = op
        self.ops.append(op)
        return t

    # ---- sweeps
    def _topo(self, root):
        order, seen = [], set()
        stack = [(root, 0)]
        seen.add(id(root))
        while stack:
            node, nxt = stack.pop()
            ins = node.creator.inputs if node.creator is not None else []
            if nxt < len(ins):
                stack.append((node, nxt + 1))
                child = ins[nxt]
                if id(child) not in seen:
                    seen.add(id(child))
                    stack.append((child, 0))
            else:
                order.append(node)
        return order

    def backward(self, loss):                     # :2192
        loss.grad.reshape(-1)[0] = 1.0
        self.backwardWithGrad(loss)

    def backwardWithGrad(self, out):              # :2217
        for node in reversed(self._topo(out)):
            if node.creator is not None:
                self._bwd(node.creator)

    def zeroGrad(self):                           # :2259
        for t in self.tensors:
            if t.grad is not None:
                t.grad[...] = 0.0

    def _bwd(self, op):                           # Op.backward, :579-1231
        C = op.output
        k = op.kind
        ins = op.inputs
        g = lambda t: t.grad if t.requires_grad else None
        if k == "MatMul":
            zo.matmul_bwd(ins[0].data, ins[1].data, C.grad, g(ins[0]), g(ins[1]))
        elif k == "AddBias":
            zo.add_bias_bwd(C.grad, g(ins[0]), g(ins[1]).reshape(-1) if ins[1].requires_grad else None)
        elif k == "Relu":
            if ins[0].requires_grad:
                zo.relu_bwd(ins[0].data, C.grad, ins[0].grad)
        elif k == "Gelu":
            if ins[0].requires_grad:
                zo.gelu_bwd(ins[0].data, C.grad, ins[0].grad)
        elif k == "SoftmaxCrossEntropy":
            if ins[0].grad is not None:
                zo.softmax_xent_bwd(op.ctx["probs"], op.ctx["targets"], ins[0].grad)
        elif k in ("Reshape",):
            if ins[0].requires_grad:
                zo.accumulate(np.ascontiguousarray(C.grad), ins[0].grad)
        elif k == "Transpose":
            if ins[0].requires_grad:
                zo.transpose_bwd(C.grad, ins[0].grad, op.ctx["d0"], op.ctx["d1"])
        elif k == "MulScalar":
            if ins[0].requires_grad:
                zo.mul_scalar_bwd(C.grad, op.ctx["v"], ins[0].grad)
        elif k == "Add":
            for t in ins:
                if t.requires_grad:
                    zo.accumulate(C.grad, t.grad)
        elif k == "Conv2D":
            A, W = ins[0], ins[1]
            b = ins[2] if len(ins) > 2 else None
            zo.conv2d_bwd(A.data, W.data, C.grad, g(A), g(W),
                          b.grad.reshape(-1) if (b is not None and b.requires_grad) else None, op.ctx["pad"])
        elif k == "MaxPool2D":
            if ins[0].requires_grad:
                zo.maxpool2d_bwd(ins[0].data, C.grad, ins[0].grad, op.ctx["pool"], op.ctx["stride"])
        elif k == "Softmax":
            if ins[0].requires_grad:
                zo.softmax_bwd(C.data, C.grad, ins[0].grad)
        elif k == "RmsNorm":
            X, G = ins
            zo.rmsnorm_bwd(X.data, G.data.reshape(-1), C.grad, op.ctx["eps"], g(X),
                           G.grad.reshape(-1) if G.requires_grad else None)
        elif k == "BatchMatMul":
            zo.batch_matmul_bwd(ins[0].data, ins[1].data, C.grad, g(ins[0]), g(ins[1]))
        elif k == "Embedding":
            W, X = ins
            if W.requires_grad:
                zo.embedding_bwd(X.data, C.grad, W.grad)
        else:
            raise ValueError(k)
