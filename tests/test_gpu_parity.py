"""Row-wise / conv / pooling operators: CUDA (through the C ABI) against the CPU
oracle on the same seeded inputs, including ragged and unaligned sizes.

Tolerances: integer/index results (argmax, MaxPool indices) bit-exact; Conv2D
forward bit-exact (same summation order and rounding points as the reference
loops); everything else relative 1e-5 of the result's scale.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL = 1e-5


@pytest.fixture(scope="module")
def ops():
    from znn_b200 import ops as _ops
    _ops.init(0)
    return _ops


def close(got, want, rtol=RTOL, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = max(1e-30, float(np.abs(want).max())) if want.size else 1.0
    err = float(np.abs(got - want).max()) if want.size else 0.0
    assert err <= rtol * scale + 1e-12, f"{what}: max abs err {err:.3e} vs scale {scale:.3e} (rel {err / scale:.3e})"


def rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("M,N", [(1, 1), (2, 3), (64, 10), (100, 128), (257, 769), (8, 4096)])
def test_add_bias(ops, zo, M, N):
    r = rng(M * 1000 + N)
    A, b = r.standard_normal((M, N), np.float32), r.standard_normal(N, np.float32)
    np.testing.assert_array_equal(ops.add_bias_fwd(A, b), zo.add_bias_fwd(A, b))
    dC = r.standard_normal((M, N), np.float32)
    dA0, db0 = r.standard_normal((M, N), np.float32), r.standard_normal(N, np.float32)
    dA1, db1, dA2, db2 = dA0.copy(), db0.copy(), dA0.copy(), db0.copy()
    ops.add_bias_bwd(dC, dA1, db1)
    zo.add_bias_bwd(dC, dA2, db2)
    np.testing.assert_array_equal(dA1, dA2)
    close(db1, db2, what="dbias")
    db3, db4 = db0.copy(), db0.copy()
    ops.add_bias_bwd(dC, None, db3)   # input without requires_grad
    zo.add_bias_bwd(dC, None, db4)
    close(db3, db4, what="dbias (no dA)")


@pytest.mark.parametrize("n", [1, 5, 1024, 4099, 1 << 20])
def test_relu_gelu(ops, zo, n):
    r = rng(n)
    A = (r.standard_normal(n, np.float32) * 2.0).astype(np.float32)
    A[::7] = 0.0
    np.testing.assert_array_equal(ops.relu_fwd(A), zo.relu_fwd(A))
    close(ops.gelu_fwd(A), zo.gelu_fwd(A), what="gelu")
    dC = r.standard_normal(n, np.float32)
    base = r.standard_normal(n, np.float32)
    g1, g2 = base.copy(), base.copy()
    ops.relu_bwd(A, dC, g1)
    zo.relu_bwd(A, dC, g2)
    np.testing.assert_array_equal(g1, g2)
    g1, g2 = base.copy(), base.copy()
    ops.gelu_bwd(A, dC, g1)
    zo.gelu_bwd(A, dC, g2)
    close(g1, g2, what="gelu bwd")
    g3, g4 = np.full(n, np.nan, np.float32), np.zeros(n, np.float32)   # the storing form ignores what the buffer held
    ops.gelu_bwd_set(A, dC, g3)
    zo.gelu_bwd(A, dC, g4)
    close(g3, g4, what="gelu bwd (set)")


@pytest.mark.parametrize("M,N", [(1, 2), (64, 10), (256, 10), (33, 255), (16, 8192), (5, 1000)])
def test_softmax_xent(ops, zo, M, N):
    r = rng(M * 7 + N)
    X = (r.standard_normal((M, N), np.float32) * 3.0).astype(np.float32)
    t = r.integers(0, N, M).astype(np.int32)
    l1, p1 = ops.softmax_xent_fwd(X, t)
    l2, p2 = zo.softmax_xent_fwd(X, t)
    close(p1, p2, what="probs")
    close(l1, l2, what="loss")
    d0 = r.standard_normal((M, N), np.float32)
    d1, d2 = d0.copy(), d0.copy()
    ops.softmax_xent_bwd(p2, t, d1)
    zo.softmax_xent_bwd(p2, t, d2)
    close(d1, d2, what="dlogits")
    if N <= 256:  # the reference's u8 targets
        l3, p3 = ops.softmax_xent_fwd(X, t.astype(np.uint8), u8=True)
        np.testing.assert_array_equal(p3, p1)
        np.testing.assert_array_equal(l3, l1)


def test_softmax_xent_clip(ops, zo):
    """The target's probability underflows: the loss clips at -log(1e-15)."""
    X = np.array([[200.0, -200.0], [0.0, 1.0]], np.float32)
    t = np.array([1, 1], np.int32)
    l1, _ = ops.softmax_xent_fwd(X, t)
    l2, _ = zo.softmax_xent_fwd(X, t)
    close(l1, l2, what="clipped loss")


@pytest.mark.parametrize("rows,D", [(1, 1), (6, 3), (64, 256), (40, 1000), (3, 5000)])
def test_softmax_rows(ops, zo, rows, D):
    r = rng(rows + D)
    X = (r.standard_normal((rows, D), np.float32) * 4.0).astype(np.float32)
    Y1, Y2 = ops.softmax_fwd(X), zo.softmax_fwd(X)
    close(Y1, Y2, what="softmax")
    dY = r.standard_normal((rows, D), np.float32)
    d0 = r.standard_normal((rows, D), np.float32)
    d1, d2 = d0.copy(), d0.copy()
    ops.softmax_bwd(Y2, dY, d1)
    zo.softmax_bwd(Y2, dY, d2)
    close(d1, d2, what="softmax bwd")


@pytest.mark.parametrize("ns,T", [(1, 1), (3, 5), (4, 64), (2, 256), (1, 1024), (2, 100)])
def test_causal_softmax(ops, zo, ns, T):
    """Fused scale + causal mask + softmax against the reference's three separate ops."""
    r = rng(ns * 31 + T)
    S = (r.standard_normal((ns, T, T), np.float32) * 5.0).astype(np.float32)
    scale = 1.0 / np.sqrt(64.0).astype(np.float32)
    P1, P2 = ops.causal_softmax_fwd(S, float(scale)), zo.causal_softmax_fwd(S, float(scale))
    close(P1, P2, what="causal softmax")
    iu = np.triu_indices(T, 1)
    assert np.all(P1[:, iu[0], iu[1]] == 0.0)
    dP = r.standard_normal((ns, T, T), np.float32)
    d0 = r.standard_normal((ns, T, T), np.float32)
    d1, d2 = d0.copy(), d0.copy()
    ops.causal_softmax_bwd(P2, dP, float(scale), d1)
    zo.causal_softmax_bwd(P2, dP, float(scale), d2)
    close(d1, d2, what="causal softmax bwd")
    # the storing form: same gradient as adding into zeros, whatever the buffer held, zeros above the diagonal
    d3 = np.full((ns, T, T), np.nan, np.float32)
    ops.causal_softmax_bwd_set(P2, dP, float(scale), d3)
    d4 = np.zeros((ns, T, T), np.float32)
    zo.causal_softmax_bwd(P2, dP, float(scale), d4)
    close(d3, d4, what="causal softmax bwd (set)")
    assert np.all(d3[:, iu[0], iu[1]] == 0.0)


@pytest.mark.parametrize("rows,D", [(1, 1), (2, 3), (64, 512), (100, 768), (7, 1001), (33, 4), (9, 256), (5, 260), (10, 772),
                                    (3, 1024), (3, 1028), (5000, 768), (9000, 256)])
def test_rmsnorm_layernorm(ops, zo, rows, D):
    r = rng(rows * 3 + D)
    X = r.standard_normal((rows, D), np.float32)
    G = (1.0 + 0.1 * r.standard_normal(D)).astype(np.float32)
    Bt = (0.1 * r.standard_normal(D)).astype(np.float32)
    dY = r.standard_normal((rows, D), np.float32)
    close(ops.rmsnorm_fwd(X, G, 1e-5), zo.rmsnorm_fwd(X, G, 1e-5), what="rmsnorm")
    dx0, dg0 = r.standard_normal((rows, D), np.float32), r.standard_normal(D, np.float32)
    a, b, c, d = dx0.copy(), dg0.copy(), dx0.copy(), dg0.copy()
    ops.rmsnorm_bwd(X, G, dY, 1e-5, a, b)
    zo.rmsnorm_bwd(X, G, dY, 1e-5, c, d)
    close(a, c, what="rmsnorm dX")
    close(b, d, rtol=3e-5, what="rmsnorm dG")
    close(ops.layernorm_fwd(X, G, Bt, 1e-5), zo.layernorm_fwd(X, G, Bt, 1e-5), what="layernorm")
    a, b, e = dx0.copy(), dg0.copy(), dg0.copy()
    c, d, f = dx0.copy(), dg0.copy(), dg0.copy()
    ops.layernorm_bwd(X, G, dY, 1e-5, a, b, e)
    zo.layernorm_bwd(X, G, dY, 1e-5, c, d, f)
    close(a, c, rtol=3e-5, what="layernorm dX")
    close(b, d, rtol=3e-5, what="layernorm dG")
    close(e, f, rtol=3e-5, what="layernorm dB")


CONV_CASES = [
    # N, Ci, H, W, Co, K, pad
    (1, 1, 3, 3, 1, 2, 0),
    (64, 1, 28, 28, 4, 3, 0),     # reference CNN layer 1 (examples/cnn.zig)
    (64, 4, 13, 13, 8, 3, 0),     # layer 2
    (64, 8, 5, 5, 16, 3, 0),      # layer 3
    (16, 1, 28, 28, 32, 3, 1),    # workload-definition shapes (padded), reduced batch
    (8, 32, 14, 14, 64, 3, 1),
    (3, 5, 9, 7, 11, 3, 1),       # ragged everything
    (2, 3, 6, 6, 2, 5, 2),
]


@pytest.mark.parametrize("N,Ci,H,W,Co,K,pad", CONV_CASES)
def test_conv2d(ops, zo, N, Ci, H, W, Co, K, pad):
    r = rng(N + Ci * 10 + H * 100 + Co * 1000 + pad)
    X = r.random((N, Ci, H, W), np.float32)
    Wt = (r.standard_normal((Co, Ci, K, K)) * 0.3).astype(np.float32)
    b = (r.standard_normal(Co) * 0.1).astype(np.float32)
    Y1, Y2 = ops.conv2d_fwd(X, Wt, b, pad), zo.conv2d_fwd(X, Wt, b, pad)
    np.testing.assert_array_equal(Y1, Y2)   # same order, same rounding: bit-exact
    np.testing.assert_array_equal(ops.conv2d_fwd(X, Wt, None, pad), zo.conv2d_fwd(X, Wt, None, pad))
    dY = r.standard_normal(Y2.shape, np.float32)
    dY[r.random(Y2.shape) < 0.3] = 0.0      # ReLU-like zeros: the reference skips them
    g = [np.zeros_like(X), np.zeros_like(Wt), np.zeros_like(b)]
    h = [np.zeros_like(X), np.zeros_like(Wt), np.zeros_like(b)]
    ops.conv2d_bwd(X, Wt, dY, g[0], g[1], g[2], pad)
    zo.conv2d_bwd(X, Wt, dY, h[0], h[1], h[2], pad)
    close(g[0], h[0], what="conv dX")
    close(g[1], h[1], rtol=3e-5, what="conv dW")
    close(g[2], h[2], rtol=3e-5, what="conv dbias")
    # first layer: the input has no gradient
    g1, h1 = np.zeros_like(Wt), np.zeros_like(Wt)
    ops.conv2d_bwd(X, Wt, dY, None, g1, None, pad)
    zo.conv2d_bwd(X, Wt, dY, None, h1, None, pad)
    close(g1, h1, rtol=3e-5, what="conv dW only")


TC_CONV_CASES = [
    # N, Ci, H, W, Co, KH, KW, pad: layers the tensor-core path takes (>= 64 taps, <= 64 channels, >= 4096 pixels)
    (256, 32, 14, 14, 64, 3, 3, 1),   # second layer of the padded CNN at its stated batch
    (64, 8, 16, 16, 16, 3, 3, 1),     # 32-wide column tile
    (48, 12, 11, 13, 20, 3, 3, 0),    # ragged, no padding
    (32, 7, 12, 12, 33, 5, 5, 2),     # 825 taps in the data gradient: several accumulation chunks
    (40, 9, 10, 14, 24, 3, 5, 1),     # KH != KW
]


@pytest.mark.parametrize("N,Ci,H,W,Co,KH,KW,pad", TC_CONV_CASES)
def test_conv2d_tensor_path(ops, zo, N, Ci, H, W, Co, KH, KW, pad):
    """Implicit-im2col GEMM path against the reference loops (src/tensor.zig:523-585, src/autodiff.zig:929-995):
    forward and dX within 1e-5 of scale, dW and dbias within 3e-5; and against the direct/im2col path of the library."""
    from znn_b200 import _lib
    L = _lib.lib()
    r = rng(N + Ci * 10 + H * 100 + Co * 1000 + pad + KW)
    X = r.random((N, Ci, H, W), np.float32)
    Wt = (r.standard_normal((Co, Ci, KH, KW)) * 0.3).astype(np.float32)
    b = (r.standard_normal(Co) * 0.1).astype(np.float32)
    Y1, Y2 = ops.conv2d_fwd(X, Wt, b, pad), zo.conv2d_fwd(X, Wt, b, pad)
    close(Y1, Y2, what="conv fwd (tensor path)")
    close(ops.conv2d_fwd(X, Wt, None, pad), zo.conv2d_fwd(X, Wt, None, pad), what="conv fwd without bias")
    dY = r.standard_normal(Y2.shape, np.float32)
    dY[r.random(Y2.shape) < 0.3] = 0.0
    # the backward arms accumulate: start from non-zero gradients
    g0 = [r.standard_normal(X.shape, np.float32), r.standard_normal(Wt.shape, np.float32), r.standard_normal(Co).astype(np.float32)]
    g = [a.copy() for a in g0]
    h = [a.copy() for a in g0]
    ops.conv2d_bwd(X, Wt, dY, g[0], g[1], g[2], pad)
    zo.conv2d_bwd(X, Wt, dY, h[0], h[1], h[2], pad)
    close(g[0], h[0], what="conv dX")
    close(g[1], h[1], rtol=3e-5, what="conv dW")
    close(g[2], h[2], rtol=3e-5, what="conv dbias")
    L.call("znn_debug_set_conv_path", 1)
    try:
        Yd = ops.conv2d_fwd(X, Wt, b, pad)
        d = [a.copy() for a in g0]
        ops.conv2d_bwd(X, Wt, dY, d[0], d[1], d[2], pad)
    finally:
        L.call("znn_debug_set_conv_path", 0)
    np.testing.assert_array_equal(Yd, Y2)      # the direct kernel keeps the reference's order: bit-exact
    close(g[0], d[0], what="dX, tensor path vs im2col path")
    close(g[1], d[1], rtol=3e-5, what="dW, tensor path vs im2col path")
    # weight gradient alone (first layer of a network), data gradient alone
    g1, h1 = np.zeros_like(Wt), np.zeros_like(Wt)
    ops.conv2d_bwd(X, Wt, dY, None, g1, None, pad)
    zo.conv2d_bwd(X, Wt, dY, None, h1, None, pad)
    close(g1, h1, rtol=3e-5, what="conv dW only")
    g2, h2 = np.zeros_like(X), np.zeros_like(X)
    ops.conv2d_bwd(X, Wt, dY, g2, None, None, pad)
    zo.conv2d_bwd(X, Wt, dY, h2, None, None, pad)
    close(g2, h2, what="conv dX only")
    ops.check_device_status()


@pytest.mark.parametrize("N,C,H,W,pool,stride", [(1, 1, 4, 4, 2, 2), (64, 4, 26, 26, 2, 2), (64, 8, 11, 11, 2, 2),
                                                (8, 32, 28, 28, 2, 2), (3, 2, 7, 9, 3, 2), (2, 2, 8, 8, 3, 1)])
def test_maxpool2d(ops, zo, N, C, H, W, pool, stride):
    r = rng(N + C + H + W + pool)
    X = r.standard_normal((N, C, H, W), np.float32)
    Y1, i1 = ops.maxpool2d_fwd(X, pool, stride, want_idx=True)
    Y2, i2 = zo.maxpool2d_fwd(X, pool, stride, want_idx=True)
    np.testing.assert_array_equal(i1, i2)
    np.testing.assert_array_equal(Y1, Y2)
    dY = r.standard_normal(Y2.shape, np.float32)
    dY[r.random(Y2.shape) < 0.2] = 0.0
    d0 = r.standard_normal(X.shape, np.float32)
    d1, d2 = d0.copy(), d0.copy()
    ops.maxpool2d_bwd(X, dY, d1, pool, stride)
    zo.maxpool2d_bwd(X, dY, d2, pool, stride)
    if stride >= pool:
        np.testing.assert_array_equal(d1, d2)
    else:
        close(d1, d2, what="overlapping pool bwd")


def test_maxpool2d_ties(ops, zo):
    """Constructed ties: the first maximum in (ph, pw) order must win."""
    X = np.zeros((2, 3, 6, 6), np.float32)
    X[0, 0] = 1.0                       # every window all-equal
    X[0, 1, ::2, 1::2] = 5.0            # ties between (0,1) of neighbouring windows only
    X[0, 2, 1::2, :] = 2.0              # ties along the bottom row of each window
    X[1] = np.tile(np.array([[3, 3], [3, 3]], np.float32), (3, 3))
    Y1, i1 = ops.maxpool2d_fwd(X, 2, 2, want_idx=True)
    Y2, i2 = zo.maxpool2d_fwd(X, 2, 2, want_idx=True)
    np.testing.assert_array_equal(i1, i2)
    assert i2[0, 0, 0, 0] == 0 and i2[0, 2, 0, 0] == 6
    d1, d2 = np.zeros_like(X), np.zeros_like(X)
    ops.maxpool2d_bwd(X, np.ones_like(Y2), d1, 2, 2)
    zo.maxpool2d_bwd(X, np.ones_like(Y2), d2, 2, 2)
    np.testing.assert_array_equal(d1, d2)


@pytest.mark.parametrize("V,D,shape", [(3, 4, (2, 2)), (50, 33, (4, 7)), (1000, 768, (2, 300)), (16, 2500, (3, 9)),
                                       (5, 64, (3, 1500)), (700, 40, (1, 2049)), (1, 8, (2, 2300))])
def test_embedding(ops, zo, V, D, shape):
    r = rng(V + D)
    W = r.standard_normal((V, D), np.float32)
    ids = r.integers(0, V, shape).astype(np.float32)
    np.testing.assert_array_equal(ops.embedding_fwd(W, ids), zo.embedding_fwd(W, ids))
    dY = r.standard_normal(shape + (D,), np.float32)
    g0 = r.standard_normal((V, D), np.float32)
    g1, g2 = g0.copy(), g0.copy()
    ops.embedding_bwd(ids, dY, g1)
    zo.embedding_bwd(ids, dY, g2)
    close(g1, g2, what="embedding dW")


@pytest.mark.parametrize("shape,d0,d1", [((2, 3), 0, 1), ((4, 16, 12, 64), 1, 2), ((2, 3, 5, 7), 2, 3),
                                          ((2, 12, 100, 64), 2, 3), ((3, 4, 5), 0, 2), ((33, 65), 0, 1), ((3, 132, 72), 1, 2),
                                          ((5, 200, 68), 1, 2)])
def test_transpose(ops, zo, shape, d0, d1):
    r = rng(sum(shape))
    A = r.standard_normal(shape, np.float32)
    np.testing.assert_array_equal(ops.transpose_fwd(A, d0, d1), zo.transpose_fwd(A, d0, d1))
    oshape = list(shape)
    oshape[d0], oshape[d1] = oshape[d1], oshape[d0]
    dC = r.standard_normal(oshape, np.float32)
    g0 = r.standard_normal(shape, np.float32)
    g1, g2 = g0.copy(), g0.copy()
    ops.transpose_bwd(dC, g1, d0, d1)
    zo.transpose_bwd(dC, g2, d0, d1)
    np.testing.assert_array_equal(g1, g2)


@pytest.mark.parametrize("n", [1, 7, 4096, 100003])
def test_add_mul_accumulate(ops, zo, n):
    r = rng(n)
    A, B = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
    np.testing.assert_array_equal(ops.add_fwd(A, B), zo.add_fwd(A, B))
    np.testing.assert_array_equal(ops.mul_scalar_fwd(A, 0.125), zo.mul_scalar_fwd(A, 0.125))
    np.testing.assert_array_equal(ops.mul_scalar_fwd(A, 0.3), zo.mul_scalar_fwd(A, 0.3))
    d1, d2 = B.copy(), B.copy()
    ops.accumulate(A, d1)
    zo.accumulate(A, d2)
    np.testing.assert_array_equal(d1, d2)
    d1, d2 = B.copy(), B.copy()
    ops.mul_scalar_bwd(A, 0.3, d1)
    zo.mul_scalar_bwd(A, 0.3, d2)
    np.testing.assert_array_equal(d1, d2)


@pytest.mark.parametrize("M,N", [(2, 3), (64, 10), (100, 1), (1, 100), (64, 8192), (7, 33)])
def test_argmax_bit_exact(ops, zo, M, N):
    r = rng(M * 13 + N)
    A = r.integers(-3, 4, (M, N)).astype(np.float32)   # many exact ties
    for dim in (0, 1):
        np.testing.assert_array_equal(ops.argmax(A, dim), zo.argmax(A, dim))
    A = r.standard_normal((M, N), np.float32)
    for dim in (0, 1):
        np.testing.assert_array_equal(ops.argmax(A, dim), zo.argmax(A, dim))


@pytest.mark.parametrize("n", [1, 1000, 1 << 18])
def test_sgd_step(ops, zo, n):
    r = rng(n)
    w0, g = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
    w1, w2 = w0.copy(), w0.copy()
    ops.sgd_step(w1, g, None, 0.05, 0.0)
    zo.sgd_step(w2, g, None, 0.05, 0.0)
    np.testing.assert_array_equal(w1, w2)
    w1, w2, v1, v2 = w0.copy(), w0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for _ in range(3):
        ops.sgd_step(w1, g, v1, 0.01, 0.9)
        zo.sgd_step(w2, g, v2, 0.01, 0.9)
    np.testing.assert_array_equal(w1, w2)
    np.testing.assert_array_equal(v1, v2)


@pytest.mark.parametrize("M,K,N", [(64, 784, 128), (5, 7, 3), (512, 768, 3072), (300, 100, 10)])
def test_fused_linear(ops, zo, M, K, N):
    """znn_linear_fwd / znn_linear_bwd (one GEMM with the bias in its epilogue) against the reference's
    two ops, matmul then addBias (src/nn.zig:44-51), and their backward arms chained."""
    import ctypes as C
    from znn_b200._lib import lib
    r = rng(M + K + N)
    X, W, b = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32), r.standard_normal(N, np.float32)
    dY = r.standard_normal((M, N), np.float32)
    L = lib()
    dX_, dW_, db_ = (ops.DevBuf.from_host(np.zeros(s, np.float32)) for s in ((M, K), (K, N), (N,)))
    x_, w_, b_, dy_ = (ops.DevBuf.from_host(a) for a in (X, W, b, dY))
    y_ = ops.DevBuf(M * N * 4)
    L.call("znn_linear_fwd", x_.ptr, w_.ptr, b_.ptr, y_.ptr, M, K, N)
    L.call("znn_linear_bwd", x_.ptr, w_.ptr, dy_.ptr, dX_.ptr, dW_.ptr, db_.ptr, M, K, N)
    ops.check_device_status()
    want_y = zo.add_bias_fwd(zo.matmul_fwd(X, W), b)
    dC, dbr = np.zeros((M, N), np.float32), np.zeros(N, np.float32)
    zo.add_bias_bwd(dY, dC, dbr)
    dXr, dWr = np.zeros_like(X), np.zeros_like(W)
    zo.matmul_bwd(X, W, dC, dXr, dWr)
    close(y_.to_host((M, N)), want_y, what="linear fwd")
    close(dX_.to_host((M, K)), dXr, what="linear dX")
    close(dW_.to_host((K, N)), dWr, what="linear dW")
    close(db_.to_host((N,)), dbr, what="linear dbias")


@pytest.mark.parametrize("ns,T,hs", [(3, 520, 64), (2, 1024, 64), (4, 96, 32)])
def test_fused_attention_score_gradient(ops, zo, ns, T, hs):
    """znn_attn_dscores = BatchMatMul backward dA (dP = dO.V^T), Softmax backward and the scale of the reference's
    attention, in one product: against the oracle's separate steps on the lower triangle (what is ever read)."""
    r = rng(ns * 7 + T)
    S = (r.standard_normal((ns, T, T), np.float32) * 3.0).astype(np.float32)
    scale = float(1.0 / np.sqrt(np.float32(hs)))
    P = zo.causal_softmax_fwd(S, scale)
    dO = r.standard_normal((ns, T, hs), np.float32)
    V = r.standard_normal((ns, T, hs), np.float32)
    dP = np.zeros((ns, T, T), np.float32)
    for s in range(ns):
        zo.sgemm(111, 112, T, T, hs, 1.0, dO[s], hs, V[s], hs, 0.0, dP[s], T, naive=True)
    want = np.zeros((ns, T, T), np.float32)
    zo.causal_softmax_bwd(P, dP, scale, want)
    got = ops.attn_dscores(dO, V, P, scale)
    close(np.tril(got), np.tril(want), what="fused attention score gradient")
    a, b = r.standard_normal((50, 64), np.float32), r.standard_normal((50, 64), np.float32)
    close(ops.rowdot(a, b), (a.astype(np.float64) * b).sum(1).astype(np.float32), what="rowdot")


@pytest.mark.parametrize("n", [1, 7, 1000, 65537])
def test_adam_step(ops, zo, n):
    """AdamOptimizer.step (src/optim.zig:133-151): three consecutive steps, bit for bit (no fused multiply-adds)."""
    r = rng(n)
    w1 = r.standard_normal(n, np.float32)
    w2 = w1.copy()
    m1, v1 = np.zeros(n, np.float32), np.zeros(n, np.float32)
    m2, v2 = m1.copy(), v1.copy()
    for t in (1.0, 2.0, 3.0):
        g = r.standard_normal(n, np.float32)
        ops.adam_step(w1, g, m1, v1, 1e-3, 0.9, 0.999, 1e-8, t)
        zo.adam_step(w2, g, m2, v2, 1e-3, 0.9, 0.999, 1e-8, t)
        np.testing.assert_array_equal(m1, m2)
        np.testing.assert_array_equal(v1, v2)
        close(w1, w2, rtol=1e-6, what="adam weights")


@pytest.mark.parametrize("N,Ci,H,W,Co,K,pad", [(64, 1, 28, 28, 4, 3, 0), (256, 32, 14, 14, 64, 3, 1), (3, 5, 9, 7, 11, 3, 1)])
def test_conv2d_with_relu_and_pool_backward_with_relu(ops, zo, N, Ci, H, W, Co, K, pad):
    """znn_conv2d_fwd_act(act = 1) equals Relu of znn_conv2d_fwd bit for bit (direct and tensor-core path), and
    znn_maxpool2d_bwd_relu equals MaxPool2D backward followed by Relu backward (src/autodiff.zig:996-1053, :673-683)."""
    import ctypes as C
    from znn_b200 import _lib
    L = _lib.lib()
    r = rng(N + Ci + H + Co)
    X = r.standard_normal((N, Ci, H, W), np.float32)
    Wt = (r.standard_normal((Co, Ci, K, K)) * 0.3).astype(np.float32)
    b = (r.standard_normal(Co) * 0.1).astype(np.float32)
    Y = ops.conv2d_fwd(X, Wt, b, pad)
    Ho, Wo = Y.shape[2], Y.shape[3]
    x, w, bb = ops._up(X), ops._up(Wt), ops._up(b)
    yr = ops.DevBuf(Y.size * 4)
    L.call("znn_conv2d_fwd_act", x.ptr, w.ptr, bb.ptr, yr.ptr, N, Ci, H, W, Co, K, K, pad, 1)
    R = yr.to_host(Y.shape)
    np.testing.assert_array_equal(R, np.maximum(Y, 0.0))
    # pool backward with the Relu mask, against the two reference arms run one after the other
    dYp = r.standard_normal((N, Co, Ho // 2, Wo // 2), np.float32)
    dA = np.zeros_like(R)
    zo.maxpool2d_bwd(R, dYp, dA, 2, 2)
    want = r.standard_normal(R.shape, np.float32)
    got0 = want.copy()
    zo.relu_bwd(Y, dA, want)
    g = ops._up(got0)
    dy = ops._up(dYp)
    L.call("znn_maxpool2d_bwd_relu", yr.ptr, dy.ptr, g.ptr, N, Co, Ho, Wo, 2, 2)
    g.into(got0)
    np.testing.assert_array_equal(got0, want)
