"""The host mirror's Graph (C++ over the CUDA kernels) against the reference's own graph-level
tests and against the CPU restatement of the Graph on seeded inputs."""
import numpy as np
import pytest

import kat_runner
from oracle import models, ograph

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    from znn_b200 import ops
    from znn_b200.graph import Graph
    ops.init(0)
    return Graph


def close(a, b, rtol=1e-5, what="", floor=0.0):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    scale = max(1e-30, float(np.abs(b).max()), floor)
    err = float(np.abs(a - b).max())
    assert err <= rtol * scale + 1e-12, f"{what}: {err:.3e} vs scale {scale:.3e}"


def test_matmul_addbias_autograd(G):                          # src/root.zig:185-245
    k = kat_runner.KATS["matmul_addbias_autograd"]
    g = G()
    A = g.array(np.array(k["A"], np.float32).reshape(2, 3), True)
    B = g.array(np.array(k["B"], np.float32).reshape(3, 2), True)
    bias = g.array(np.array(k["bias"], np.float32).reshape(1, 2), True)
    Cm = g.matmul(A, B)
    assert Cm.shape == (2, 2)
    kat_runner.check(Cm.data, k["expect_C"], "C")
    D = g.addBias(Cm, bias)
    kat_runner.check(D.data, k["expect_D"], "D")
    D.set_grad(np.ones((2, 2), np.float32))
    g.backward(D)
    kat_runner.check(bias.grad, k["expect_dbias"], "bias.grad")
    kat_runner.check(B.grad, k["expect_dB"], "B.grad")
    kat_runner.check(A.grad, k["expect_dA"], "A.grad")


def test_conv_and_pool_autograd(G):                           # src/root.zig:247-323
    k = kat_runner.KATS["conv2d_autograd"]
    g = G()
    A = g.array(np.array(k["X"], np.float32).reshape(k["X_shape"]), True)
    W = g.array(np.array(k["W"], np.float32).reshape(k["W_shape"]), True)
    b = g.array(np.array(k["bias"], np.float32), True)
    Cm = g.conv2d(A, W, b)
    assert Cm.shape == (1, 1, 2, 2)
    kat_runner.check(Cm.data, k["expect_Y"], "C")
    Cm.set_grad(np.ones(Cm.shape, np.float32))
    g.backward(Cm)
    kat_runner.check(b.grad, k["expect_dbias"], "bias.grad")
    kat_runner.check(W.grad, k["expect_dW"], "W.grad")
    kat_runner.check(A.grad, k["expect_dX"], "A.grad")
    k = kat_runner.KATS["maxpool2d_autograd"]
    g = G()
    A = g.array(np.array(k["X"], np.float32).reshape(k["X_shape"]), True)
    Cm = g.maxpool2d(A, 2, 2)
    kat_runner.check(Cm.data, k["expect_Y"], "C")
    Cm.set_grad(np.ones(Cm.shape, np.float32))
    g.backward(Cm)
    kat_runner.check(A.grad, k["expect_dX"], "A.grad")


def test_transpose_reshape_autograd(G):                       # src/root.zig:126-183
    k = kat_runner.KATS["transpose_reshape"]
    g = G()
    A = g.array(np.array(k["A"], np.float32).reshape(2, 3), True)
    B = g.transposeND(A, 0, 1)
    assert B.shape == (3, 2)
    kat_runner.check(B.data, k["expect_B"], "B")
    Cc = g.reshape(B, (1, 6))
    assert Cc.shape == (1, 6)
    Cc.set_grad(np.array(k["dC"], np.float32))
    g.backwardWithGrad(Cc)
    kat_runner.check(A.grad, k["expect_dA"], "A.grad")


def test_static_graph_forward_and_backward(G):                # src/tensor.zig:1406-1453
    k = kat_runner.KATS["static_graph_mulscalar_add"]
    g = G()
    A = g.array(np.zeros((2, 2), np.float32), True)
    B = g.array(np.zeros((2, 2), np.float32), True)
    D = g.add(g.mulScalar(A, k["scalar"]), B)
    for run in k["runs"]:
        A.set_data(np.array(run["A"], np.float32))
        B.set_data(np.array(run["B"], np.float32))
        g.forward()
        kat_runner.check(D.data, run["expect_D"], "D")
        g.zeroGrad()
        D.set_grad(np.ones((2, 2), np.float32))
        g.backward(D)
        kat_runner.check(B.grad, k["expect_dB"], "B.grad")
        kat_runner.check(A.grad, k["expect_dA"], "A.grad")


def test_requires_grad_gating_and_errors(G):
    from znn_b200._lib import ZnnError
    g = G()
    x = g.array(np.ones((4, 3), np.float32), False)            # an input: no gradient (fashion_mnist.zig:141)
    W = g.array(np.ones((3, 2), np.float32), True)
    y = g.matmul(x, W)
    assert y.requires_grad and not x.requires_grad and x.grad is None
    y.set_grad(np.ones((4, 2), np.float32))
    g.backwardWithGrad(y)
    np.testing.assert_array_equal(W.grad, np.full((3, 2), 4.0, np.float32))
    with pytest.raises(ZnnError):
        g.matmul(W, W)                                         # inner dimensions differ
    with pytest.raises(ZnnError):
        g.reshape(W, (5,))


def test_transformer_block_matches_cpu_graph(G):
    """The reference's literal attention op sequence, op by op on both graphs (examples/transformer_block.zig)."""
    r = np.random.default_rng(5)
    cfg = {"n_embd": 16}
    P0 = models.init_params("block", cfg, seed=3)
    x = r.standard_normal((2, 5, 16), np.float32)
    dy = r.standard_normal((2, 5, 16), np.float32)
    outs = []
    for graph in (ograph.OGraph(), G()):
        P = {k: graph.array(v, True) for k, v in P0.items()}
        xt = graph.array(x, True)
        y = models.transformer_block(graph, P, "block", xt, n_head=2)
        if isinstance(graph, ograph.OGraph):
            y.grad[...] = dy
        else:
            y.set_grad(dy)
        graph.backwardWithGrad(y)
        outs.append((np.array(y.data), np.array(xt.grad), {k: np.array(t.grad).reshape(P0[k].shape) for k, t in P.items()}))
    (y0, dx0, g0), (y1, dx1, g1) = outs
    close(y1, y0, what="block output")
    close(dx1, dx0, rtol=3e-5, what="block dx")
    # the key-bias gradient is zero in exact arithmetic (softmax cancels a per-row shift): compare
    # such tensors on the scale of their neighbours
    floor = 1e-2 * max(float(np.abs(v).max()) for v in g0.values())
    for k in g0:
        close(g1[k], g0[k], rtol=3e-5, what=k, floor=floor)


def test_batch_matmul_nt_equals_transpose_then_batch_matmul(G):
    """batchMatMulNT(A, B) = batchMatMul(A, transposeND(B, 2, 3)) in values and in both gradients."""
    r = np.random.default_rng(12)
    a = r.standard_normal((2, 3, 20, 8), np.float32)
    b = r.standard_normal((2, 3, 12, 8), np.float32)
    dc = r.standard_normal((2, 3, 20, 12), np.float32)
    outs = []
    for fused in (True, False):
        g = G()
        A, B = g.array(a, True), g.array(b, True)
        Cn = g.batchMatMulNT(A, B) if fused else g.batchMatMul(A, g.transposeND(B, 2, 3))
        Cn.set_grad(dc)
        g.backwardWithGrad(Cn)
        outs.append((np.array(Cn.data), np.array(A.grad), np.array(B.grad)))
    for x, y in zip(outs[0], outs[1]):
        np.testing.assert_allclose(x, y, rtol=1e-5, atol=1e-6)
