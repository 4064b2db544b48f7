"""Pins the Python restatement of the reference's Graph (oracle/ograph.py) and module
compositions (oracle/models.py) with the reference's own graph-level tests, on the CPU."""
import numpy as np

import kat_runner
from oracle import models, ograph


def test_matmul_addbias_autograd_through_graph_backward():   # src/root.zig:185-245
    k = kat_runner.KATS["matmul_addbias_autograd"]
    g = ograph.OGraph()
    A = g.array(np.array(k["A"], np.float32).reshape(2, 3), True)
    B = g.array(np.array(k["B"], np.float32).reshape(3, 2), True)
    bias = g.array(np.array(k["bias"], np.float32).reshape(1, 2), True)
    D = g.addBias(g.matmul(A, B), bias)
    kat_runner.check(D.data, k["expect_D"], "D")
    D.grad[...] = 1.0
    g.backward(D)
    kat_runner.check(bias.grad, k["expect_dbias"], "bias.grad")
    kat_runner.check(B.grad, k["expect_dB"], "B.grad")
    kat_runner.check(A.grad, k["expect_dA"], "A.grad")


def test_transpose_reshape_aliasing_and_backward():           # src/root.zig:126-183
    k = kat_runner.KATS["transpose_reshape"]
    g = ograph.OGraph()
    A = g.array(np.array(k["A"], np.float32).reshape(2, 3), True)
    B = g.transposeND(A, 0, 1)
    Cc = g.reshape(B, (1, 6))
    assert np.shares_memory(Cc.data, B.data)
    Cc.grad[...] = np.array(k["dC"], np.float32).reshape(1, 6)
    g.backwardWithGrad(Cc)
    kat_runner.check(A.grad, k["expect_dA"], "A.grad")


def test_module_shapes_and_nonzero_grads():                   # the reference's module smoke tests, src/nn.zig:1379-1611
    cfg = {"vocab_size": 11, "block_size": 6, "n_embd": 8, "n_head": 2, "n_layer": 2}
    P0 = models.init_params("gpt", cfg, seed=1)
    tr = models.OracleTrainer("gpt", P0, cfg, lr=0.1, momentum=0.9)
    r = np.random.default_rng(0)
    ids = r.integers(0, 11, (2, 5)).astype(np.float32)
    tg = r.integers(0, 11, (2, 5))
    l0, logits = tr.step(ids, tg)
    assert logits.shape == (10, 11) and l0 > 0
    assert all(float(np.abs(v).sum()) > 0 for k, v in tr.grads.items() if "bias" not in k or True)
    losses = [tr.step(ids, tg)[0] for _ in range(20)]
    assert losses[-1] < l0   # the same batch is being fitted
