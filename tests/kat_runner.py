"""Runs the reference's known-answer tests (tests/golden/ref_kats.json) against
any backend exposing the op-level numpy interface (the CPU oracle's `zo`
module, or `znn_b200.ops`, which goes through the C-ABI to the CUDA kernels)."""
import json
import os

import numpy as np

_GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kats.json")

with open(_GOLD) as fh:
    KATS = json.load(fh)

CASES = [k for k in KATS if not k.startswith("_")]


def f32(v, shape=None):
    a = np.array(v, dtype=np.float32)
    return a.reshape(shape) if shape is not None else a


def check(arr, expect, what):
    flat = np.asarray(arr).reshape(-1)
    for idx, val, tol in expect:
        got = float(flat[idx])
        assert abs(got - val) <= tol, f"{what}[{idx}] = {got!r}, reference test expects {val} (abs tol {tol})"


def run_case(be, name):
    k = KATS[name]
    globals()["_case_" + name](be, k)


def _case_sgemm_2x3_3x2(be, k):
    A, B = f32(k["A"], (2, 3)), f32(k["B"], (3, 2))
    C = np.zeros((2, 2), np.float32)
    be.sgemm(111, 111, 2, 2, 3, 1.0, A, 3, B, 2, 0.0, C, 2)
    check(C, k["expect_C"], "C")


def _case_matmul_addbias_autograd(be, k):
    A, B, bias = f32(k["A"], (2, 3)), f32(k["B"], (3, 2)), f32(k["bias"])
    Cm = be.matmul_fwd(A, B)
    check(Cm, k["expect_C"], "C")
    D = be.add_bias_fwd(Cm, bias)
    check(D, k["expect_D"], "D")
    dD = np.full((2, 2), k["dD_fill"], np.float32)
    dC, dbias = np.zeros((2, 2), np.float32), np.zeros(2, np.float32)
    be.add_bias_bwd(dD, dC, dbias)
    dA, dB = np.zeros_like(A), np.zeros_like(B)
    be.matmul_bwd(A, B, dC, dA, dB)
    check(dbias, k["expect_dbias"], "bias.grad")
    check(dB, k["expect_dB"], "B.grad")
    check(dA, k["expect_dA"], "A.grad")


def _case_eager_chain(be, k):
    A, B, bias = f32(k["A"], (2, 3)), f32(k["B"], (3, 2)), f32(k["bias"])
    Cm = be.matmul_fwd(A, B)
    check(Cm, k["expect_C"], "C")
    D = be.add_bias_fwd(Cm, bias)
    check(D, k["expect_D"], "D")
    E = be.relu_fwd(D)
    check(E, k["expect_E"], "E")
    loss, _ = be.softmax_xent_fwd(E, np.array(k["targets"], np.int32))
    assert float(loss[0]) > 0.0


def _case_conv2d_autograd(be, k):
    X, W, b = f32(k["X"], k["X_shape"]), f32(k["W"], k["W_shape"]), f32(k["bias"])
    Y = be.conv2d_fwd(X, W, b)
    assert Y.shape == (1, 1, 2, 2)
    check(Y, k["expect_Y"], "Y")
    dY = np.full_like(Y, k["dY_fill"])
    dX, dW, db = np.zeros_like(X), np.zeros_like(W), np.zeros_like(b)
    be.conv2d_bwd(X, W, dY, dX, dW, db)
    check(db, k["expect_dbias"], "bias.grad")
    check(dW, k["expect_dW"], "W.grad")
    check(dX, k["expect_dX"], "A.grad")


def _case_maxpool2d_autograd(be, k):
    X = f32(k["X"], k["X_shape"])
    Y = be.maxpool2d_fwd(X, k["pool"], k["stride"])
    assert Y.shape == (1, 1, 2, 2)
    check(Y, k["expect_Y"], "Y")
    dY = np.full_like(Y, k["dY_fill"])
    dX = np.zeros_like(X)
    be.maxpool2d_bwd(X, dY, dX, k["pool"], k["stride"])
    check(dX, k["expect_dX"], "A.grad")


def _case_softmax(be, k):
    X = f32(k["X"], k["X_shape"])
    Y = be.softmax_fwd(X)
    check(Y, k["expect_Y"], "Y")
    dX = np.zeros_like(X)
    be.softmax_bwd(Y, np.ones_like(Y), dX)
    check(dX, k["bwd_ones_expect_dX"], "X.grad")
    dX = np.zeros_like(X)
    be.softmax_bwd(Y, f32(k["bwd_onehot_dY"], k["X_shape"]), dX)
    y0, y1 = float(Y.reshape(-1)[0]), float(Y.reshape(-1)[1])
    assert abs(float(dX.reshape(-1)[0]) - y0 * (1.0 - y0)) <= 1e-5
    assert abs(float(dX.reshape(-1)[1]) - (-y1 * y0)) <= 1e-5


def _case_rmsnorm(be, k):
    X, G = f32(k["X"], k["X_shape"]), f32(k["G"])
    Y = be.rmsnorm_fwd(X, G, k["eps"])
    check(Y, k["expect_Y"], "Y")
    dX, dG = np.zeros_like(X), np.zeros_like(G)
    be.rmsnorm_bwd(X, G, np.full_like(X, k["dY_fill"]), k["eps"], dX, dG)
    check(dG, k["expect_dG"], "G.grad")


def _case_embedding(be, k):
    W, ids = f32(k["W"], k["W_shape"]), f32(k["ids"], k["ids_shape"])
    Y = be.embedding_fwd(W, ids)
    assert Y.shape == (2, 2, 4)
    check(Y, k["expect_Y"], "Y")
    dW = np.zeros_like(W)
    be.embedding_bwd(ids, np.full_like(Y, k["dY_fill"]), dW)
    check(dW, k["expect_dW"], "W.grad")


def _case_batch_matmul(be, k):
    A, B = f32(k["A"], k["A_shape"]), f32(k["B"], k["B_shape"])
    Cm = be.batch_matmul_fwd(A, B)
    check(Cm, k["expect_C"], "C")
    dA, dB = np.zeros_like(A), np.zeros_like(B)
    be.batch_matmul_bwd(A, B, np.full_like(Cm, k["dC_fill"]), dA, dB)
    check(dA, k["expect_dA"], "A.grad")


def _case_gelu(be, k):
    X = f32(k["X"], (2, 2))
    Y = be.gelu_fwd(X)
    check(Y, k["expect_Y"], "Y")
    dX = np.zeros_like(X)
    be.gelu_bwd(X, np.full_like(X, k["dY_fill"]), dX)
    check(dX, k["expect_dX"], "A.grad")


def _case_argmax(be, k):
    A = f32(k["A"], k["A_shape"])
    assert be.argmax(A, 1).tolist() == [float(v) for v in k["expect_dim1"]]
    assert be.argmax(A, 0).tolist() == [float(v) for v in k["expect_dim0"]]


def _case_sgd(be, k):
    w, g = f32([k["w0"], 3.0]), f32([k["g"], 0.0])
    be.sgd_step(w, g, None, k["lr"], 0.0)
    assert abs(float(w[0]) - k["plain_expect"][0]) <= k["tol"]
    w, v = f32([k["w0"], 3.0]), np.zeros(2, np.float32)
    for want in k["momentum_expect"]:
        be.sgd_step(w, g, v, k["lr"], k["momentum"])
        assert abs(float(w[0]) - want) <= k["tol"]


def _case_transpose_reshape(be, k):
    A = f32(k["A"], k["A_shape"])
    B = be.transpose_fwd(A, 0, 1)
    assert B.shape == (3, 2)
    check(B, k["expect_B"], "B")
    # reshape aliases the data; its backward adds the flat gradient (autodiff.zig:831-839)
    dB = np.zeros((3, 2), np.float32)
    be.accumulate(f32(k["dC"]), dB)
    dA = np.zeros_like(A)
    be.transpose_bwd(dB, dA, 0, 1)
    check(dA, k["expect_dA"], "A.grad")


def _case_static_graph_mulscalar_add(be, k):
    for run in k["runs"]:
        A, B = f32(run["A"], (2, 2)), f32(run["B"], (2, 2))
        Cm = be.mul_scalar_fwd(A, k["scalar"])
        D = be.add_fwd(Cm, B)
        check(D, run["expect_D"], "D")
        dD = np.full_like(D, k["dD_fill"])
        dC, dB, dA = np.zeros_like(D), np.zeros_like(D), np.zeros_like(D)
        be.accumulate(dD, dC)
        be.accumulate(dD, dB)
        be.mul_scalar_bwd(dC, k["scalar"], dA)
        check(dB, k["expect_dB"], "B.grad")
        check(dA, k["expect_dA"], "A.grad")
