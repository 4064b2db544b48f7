"""Python view of the host mirror's Graph (include/znn_host.h, znn_graph_*): the
reference's Graph builders by name, over device memory.  Tensors are integer
handles; `.data` / `.grad` copy to the host."""
import ctypes as C

import numpy as np

from ._lib import lib


class GTensor:
    def __init__(self, graph, tid):
        self.graph, self.id = graph, tid
        dims = (C.c_longlong * 8)()
        rank, rg = C.c_int(), C.c_int()
        lib().call("znn_graph_shape", graph.h, tid, dims, C.byref(rank), C.byref(rg))
        self.shape = tuple(int(dims[i]) for i in range(rank.value))
        self.requires_grad = bool(rg.value)

    def _read(self, which):
        out = np.empty(self.shape, np.float32)
        lib().call("znn_graph_read", self.graph.h, self.id, which, out.ctypes.data, out.size)
        return out

    @property
    def data(self):
        return self._read(0)

    @property
    def grad(self):
        return self._read(1) if self.requires_grad else None

    def set_data(self, arr):
        a = np.ascontiguousarray(arr, np.float32)
        lib().call("znn_graph_write", self.graph.h, self.id, 0, a.ctypes.data, a.size)

    def set_grad(self, arr):
        a = np.ascontiguousarray(arr, np.float32)
        lib().call("znn_graph_write", self.graph.h, self.id, 1, a.ctypes.data, a.size)


class Graph:
    """src/autodiff.zig:1237-2264 (Graph) by way of znn_b200/csrc/host/graph.cpp."""

    def __init__(self, arena_bytes=256 << 20):
        h = C.c_void_p()
        lib().call("znn_graph_create", arena_bytes, C.byref(h))
        self.h = h

    def close(self):
        if self.h:
            lib().call("znn_graph_destroy", self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def array(self, data, requires_grad=False):
        a = np.ascontiguousarray(data, np.float32)
        dims = (C.c_longlong * max(1, a.ndim))(*a.shape)
        tid = C.c_int()
        lib().call("znn_graph_array", self.h, dims, a.ndim, a.ctypes.data, int(requires_grad), C.byref(tid))
        return GTensor(self, tid.value)

    def _op(self, name, inputs, args=()):
        ins = (C.c_int * max(1, len(inputs)))(*[t.id for t in inputs])
        av = (C.c_double * max(1, len(args)))(*[float(a) for a in args])
        tid = C.c_int()
        lib().call("znn_graph_op", self.h, name.encode(), ins, len(inputs), av, len(args), C.byref(tid))
        return GTensor(self, tid.value)

    def matmul(self, A, B): return self._op("matmul", [A, B])
    def addBias(self, A, b): return self._op("addBias", [A, b])
    def relu(self, A): return self._op("relu", [A])
    def gelu(self, A): return self._op("gelu", [A])
    def softmaxCrossEntropy(self, logits, targets): return self._op("softmaxCrossEntropy", [logits], list(np.asarray(targets).reshape(-1)))
    def reshape(self, A, shape): return self._op("reshape", [A], list(shape))
    def transposeND(self, A, d0, d1): return self._op("transposeND", [A], [d0, d1])
    def mulScalar(self, A, v): return self._op("mulScalar", [A], [v])
    def add(self, A, B): return self._op("add", [A, B])
    def conv2d(self, A, W, bias=None, pad=0): return self._op("conv2d", [A, W] + ([bias] if bias is not None else []), [pad])
    def maxpool2d(self, A, pool, stride): return self._op("maxpool2d", [A], [pool, stride])
    def softmax(self, A): return self._op("softmax", [A])
    def causalSoftmax(self, A, scale): return self._op("causalSoftmax", [A], [scale])
    def rmsNorm(self, X, G, eps): return self._op("rmsNorm", [X, G], [eps])
    def layerNorm(self, X, G, B, eps): return self._op("layerNorm", [X, G, B], [eps])
    def batchMatMul(self, A, B): return self._op("batchMatMul", [A, B])
    def batchMatMulNT(self, A, B): return self._op("batchMatMulNT", [A, B])
    def embedding(self, W, X): return self._op("embedding", [W, X])
    def linear(self, X, W, b): return self._op("linear", [X, W, b])

    def backward(self, t): lib().call("znn_graph_backward", self.h, t.id, 1)
    def backwardWithGrad(self, t): lib().call("znn_graph_backward", self.h, t.id, 0)
    def forward(self): lib().call("znn_graph_forward", self.h)
    def zeroGrad(self): lib().call("znn_graph_zero_grad", self.h)

    def num_ops(self):
        n = C.c_int()
        lib().call("znn_graph_num_ops", self.h, C.byref(n))
        return n.value
