"""Runtime behaviour of the shim beyond arithmetic: bounded-wait recovery, host-side fault injection, index range
checks, device-side weight initialisation, the arena and parameter-slab entry points, CUDA-graph invalidation, and
per-thread / per-device state."""
import ctypes as C
import threading

import numpy as np
import pytest

from oracle import models

pytestmark = pytest.mark.gpu

ZNN_ERR_CUDA = -2
DEV_TMA_WAIT_EXPIRED, DEV_BAD_INDEX = 1, 8


@pytest.fixture(scope="module")
def ops():
    from znn_b200 import ops as _ops
    _ops.init(0)
    return _ops


@pytest.fixture(scope="module")
def L(ops):
    from znn_b200._lib import lib
    return lib()


def status(L, clear=1):
    st = C.c_int(0)
    L.call("znn_device_status", C.byref(st), clear)
    return st.value


def test_bounded_wait_expiry_and_recovery(ops, L):
    """A wait that nothing ever satisfies runs out after its limit (1e6 cycles, well under a millisecond), the kernel
    returns normally and the status word carries the bit; while the bit is set every tensor-core GEMM returns without
    doing work; clearing the word restores service."""
    r = np.random.default_rng(1)
    A, B = r.standard_normal((256, 256), np.float32), r.standard_normal((256, 256), np.float32)
    assert status(L) == 0
    L.call("znn_debug_wait_probe", 1000000)
    assert status(L, clear=0) == DEV_TMA_WAIT_EXPIRED
    dA, dB = ops.DevBuf.from_host(A), ops.DevBuf.from_host(B)
    sentinel = np.full((256, 256), 7.0, np.float32)
    dC = ops.DevBuf.from_host(sentinel)
    ops.set_gemm_path(4)
    try:
        L.call("znn_sgemm", 101, 111, 111, 256, 256, 256, C.c_float(1.0), dA.ptr, 256, dB.ptr, 256, C.c_float(0.0), dC.ptr, 256)
        np.testing.assert_array_equal(dC.to_host((256, 256)), sentinel)      # a no-op: C untouched
        assert status(L, clear=1) == DEV_TMA_WAIT_EXPIRED                    # reported, then cleared
        assert status(L) == 0
        L.call("znn_sgemm", 101, 111, 111, 256, 256, 256, C.c_float(1.0), dA.ptr, 256, dB.ptr, 256, C.c_float(0.0), dC.ptr, 256)
        got = dC.to_host((256, 256))
    finally:
        ops.set_gemm_path(0)
    exact = A.astype(np.float64) @ B.astype(np.float64)
    assert np.linalg.norm(got - exact) / np.linalg.norm(exact) <= 1e-5
    assert status(L) == 0


def test_injected_launch_failure_unwinds_cleanly(ops, L):
    """znn_debug_fail_after(n): the n-th launch of a training step is reported as failed; the step returns an error,
    and the model trains on afterwards exactly like a model that never saw the failure (parameters are only written
    by the optimizer step, which the failed step never reached)."""
    from znn_b200.models import Model
    dims = (784, 128, 64, 10)
    r = np.random.default_rng(3)
    P0 = models.init_params("mlp", dims, seed=4)
    x = (r.integers(0, 256, (64, 784)) / 255.0).astype(np.float32)
    t = r.integers(0, 10, 64).astype(np.int32)
    ref = Model("mlp", dims, arena_bytes=64 << 20)
    ref.set_params(P0)
    want_loss = ref.train_step(x, t)
    want = ref.get_params()
    m = Model("mlp", dims, arena_bytes=64 << 20)
    m.set_params(P0)
    for n in (0, 5, 11):
        L.call("znn_debug_fail_after", n)
        with pytest.raises(RuntimeError, match="injected failure"):
            m.train_step(x, t)
        L.call("znn_sync")
        got = m.get_params()
        assert all(np.array_equal(got[k], P0[k].reshape(got[k].shape)) for k in got), f"parameters changed by a failed step (n={n})"
    L.call("znn_debug_fail_after", -1)
    assert m.train_step(x, t) == want_loss
    got = m.get_params()
    assert all(np.array_equal(got[k], want[k]) for k in want)


def test_out_of_range_indices_are_flagged_not_dereferenced(ops, L):
    """A token id, class label or sample index outside its range is never used as an address: the op writes a
    defined value and ZNN_DEV_BAD_INDEX appears in the device status word."""
    r = np.random.default_rng(5)
    assert status(L) == 0
    # Embedding
    W = r.standard_normal((11, 8), np.float32)
    ids = np.array([0, 10, 11, 3, -1, 2.0e9], np.float32)
    dW_, dI = ops.DevBuf.from_host(W), ops.DevBuf.from_host(ids)
    dY = ops.DevBuf(ids.size * 8 * 4)
    L.call("znn_embedding_fwd", dW_.ptr, dI.ptr, dY.ptr, ids.size, 8, 11)
    assert status(L) == DEV_BAD_INDEX
    Y = dY.to_host((ids.size, 8))
    np.testing.assert_array_equal(Y[[0, 1, 3]], W[[0, 10, 3]])
    np.testing.assert_array_equal(Y[[2, 4, 5]], np.zeros((3, 8), np.float32))
    # the backward ignores such positions
    dYg = r.standard_normal((ids.size, 8)).astype(np.float32)
    dWg = np.zeros_like(W)
    d1, d2 = ops.DevBuf.from_host(dYg), ops.DevBuf.from_host(dWg)
    L.call("znn_embedding_bwd", dI.ptr, d1.ptr, d2.ptr, ids.size, 8, 11)
    got = d2.to_host((11, 8))
    want = np.zeros_like(W)
    for i in (0, 1, 3):
        want[int(ids[i])] += dYg[i]
    np.testing.assert_array_equal(got, want)
    assert status(L) == 0
    # SoftmaxCrossEntropy, both kernels (rows of 10 and rows of 4096)
    for N in (10, 4096):
        x = r.standard_normal((6, N), np.float32)
        t = np.array([1, N - 1, N, 0, -3, 2], np.int32)
        dx, dt = ops.DevBuf.from_host(x), ops.DevBuf.from_host(t)
        dp, dl = ops.DevBuf(x.nbytes), ops.DevBuf(4)
        L.call("znn_softmax_xent_fwd", dx.ptr, dt.ptr, dp.ptr, dl.ptr, 6, N)
        assert status(L) == DEV_BAD_INDEX
        assert np.isnan(dl.to_host((1,))[0])
        t_ok = np.array([1, N - 1, 0, 0, 5, 2], np.int32)
        dt2 = ops.DevBuf.from_host(t_ok)
        L.call("znn_softmax_xent_fwd", dx.ptr, dt2.ptr, dp.ptr, dl.ptr, 6, N)
        assert status(L) == 0 and np.isfinite(dl.to_host((1,))[0])
    # batch gather
    images = r.standard_normal((20, 12), np.float32)
    labels = r.integers(0, 10, 20).astype(np.uint8)
    idx = np.array([3, 19, 20, -1, 0], np.int32)
    di, dl_, dx_ = ops.DevBuf.from_host(images), ops.DevBuf.from_host(labels), ops.DevBuf.from_host(idx)
    dxo, dyo = ops.DevBuf(5 * 12 * 4), ops.DevBuf(8)
    L.call("znn_batch_gather", di.ptr, dl_.ptr, dx_.ptr, dxo.ptr, dyo.ptr, 5, 12, 20)
    assert status(L) == DEV_BAD_INDEX
    X = dxo.to_host((5, 12))
    np.testing.assert_array_equal(X[[0, 1, 4]], images[[3, 19, 0]])
    np.testing.assert_array_equal(X[[2, 3]], np.zeros((2, 12), np.float32))
    np.testing.assert_array_equal(dyo.to_host((8,), np.uint8)[:5], np.array([labels[3], labels[19], 0, 0, labels[0]], np.uint8))


def test_weight_initialisation_moments_and_rules(ops, L):
    """znn_init_he_normal draws N(0, 2/fan_in) (src/nn.zig:1336-1350); the model-level call applies the modules' rule:
    He-normal weights with each module's fan-in, zero biases, unit norm gains.  The random stream itself is not the
    reference's (parity of the stream is unpinned), so the check is on moments, determinism and the rule."""
    from znn_b200.models import Model
    n, fan_in = 1 << 20, 512
    d = ops.DevBuf(n * 4)
    L.call("znn_init_he_normal", d.ptr, n, fan_in, 1234)
    w = d.to_host((n,)).astype(np.float64)
    std = np.sqrt(2.0 / fan_in)
    assert abs(w.mean()) < 4 * std / np.sqrt(n)
    assert abs(w.std() / std - 1.0) < 0.01
    assert abs(((w / std) ** 4).mean() - 3.0) < 0.1                       # kurtosis of a normal
    assert np.abs(w / std).max() < 6.0                                    # 24-bit uniforms bound the tail
    L.call("znn_init_he_normal", d.ptr, n, fan_in, 1234)
    np.testing.assert_array_equal(d.to_host((n,)), w.astype(np.float32))  # same seed, same values
    L.call("znn_init_he_normal", d.ptr, n, fan_in, 1235)
    assert not np.array_equal(d.to_host((n,)), w.astype(np.float32))
    L.call("znn_fill_normal", d.ptr, n, C.c_float(2.0), C.c_float(0.5), 7)
    v = d.to_host((n,)).astype(np.float64)
    assert abs(v.mean() - 2.0) < 0.005 and abs(v.std() - 0.5) < 0.005
    L.call("znn_fill_uniform", d.ptr, n, C.c_float(-1.0), C.c_float(3.0), 7)
    u = d.to_host((n,)).astype(np.float64)
    assert u.min() >= -1.0 and u.max() < 3.0 and abs(u.mean() - 1.0) < 0.01 and abs(u.var() - 16.0 / 12.0) < 0.01
    cfg = (61, 24, 32, 4, 2)
    m = Model("gpt", cfg, arena_bytes=64 << 20)
    L.call("znn_model_init_weights", m.h, 99)
    P = m.get_params()
    for name, shape, _, fan in m.params:
        a = P[name].astype(np.float64)
        if name.endswith(".bias"):
            assert not a.any(), name
        elif fan == 0:
            assert (a == 1.0).all(), name
        else:
            s = np.sqrt(2.0 / fan)
            assert abs(a.std() / s - 1.0) < 0.15 and abs(a.mean()) < 0.2 * s, (name, a.std(), s)
    # a model initialised this way trains: the loss falls
    r = np.random.default_rng(0)
    x = r.integers(0, 61, (4, 24)).astype(np.float32)
    t = r.integers(0, 61, (4, 24)).astype(np.int32)
    m.set_option("lr", 0.05)
    losses = [m.train_step(x, t, seq=24) for _ in range(8)]
    assert losses[-1] < losses[0]


def test_arena_and_param_slab_entry_points(ops, L):
    """The per-step arena (Graph.arena's analogue) and the contiguous parameter slabs as a host with its own Graph
    would use them: allocate, compute into the memory, reset, step the optimizer over the slab."""
    a = C.c_void_p()
    L.call("znn_arena_create", 1 << 20, C.byref(a))
    p1, p2 = C.c_void_p(), C.c_void_p()
    L.call("znn_arena_alloc", a, 1000, C.byref(p1))
    L.call("znn_arena_alloc", a, 4096, C.byref(p2))
    assert p1.value % 256 == 0 and p2.value == p1.value + 1024
    used, high, cap = C.c_size_t(), C.c_size_t(), C.c_size_t()
    L.call("znn_arena_usage", a, C.byref(used), C.byref(high), C.byref(cap))
    assert (used.value, high.value, cap.value) == (1024 + 4096, 1024 + 4096, 1 << 20)
    with pytest.raises(RuntimeError, match="exhausted"):
        L.call("znn_arena_alloc", a, 2 << 20, C.byref(p2))
    L.call("znn_arena_reset", a)
    p3 = C.c_void_p()
    L.call("znn_arena_alloc", a, 16, C.byref(p3))
    assert p3.value == p1.value
    L.call("znn_arena_destroy", a)

    counts = (C.c_size_t * 3)(10, 7, 33)
    s = C.c_void_p()
    L.call("znn_param_slab_create", counts, 3, C.byref(s))
    total = C.c_size_t()
    L.call("znn_param_slab_total", s, C.byref(total))
    assert total.value == 12 + 8 + 36
    r = np.random.default_rng(2)
    W, G = [], []
    for i, n in enumerate((10, 7, 33)):
        w, g, v, off = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_size_t()
        L.call("znn_param_slab_tensor", s, i, C.byref(w), C.byref(g), C.byref(v), C.byref(off))
        assert off.value % 4 == 0
        wi, gi = r.standard_normal(n).astype(np.float32), r.standard_normal(n).astype(np.float32)
        L.call("znn_memcpy_h2d", w, wi.ctypes.data, wi.nbytes)
        L.call("znn_memcpy_h2d", g, gi.ctypes.data, gi.nbytes)
        L.call("znn_sync")
        W.append((w, wi))
        G.append((g, gi))
    L.call("znn_param_slab_sgd_step", s, C.c_float(0.1), C.c_float(0.0), C.c_float(1.0))
    for (w, wi), (g, gi) in zip(W, G):
        out = np.empty_like(wi)
        L.call("znn_memcpy_d2h", out.ctypes.data, w, out.nbytes)
        np.testing.assert_array_equal(out, (wi - (np.float32(0.1) * gi)).astype(np.float32))
    L.call("znn_param_slab_zero_grad", s)
    for g, gi in G:
        out = np.empty_like(gi)
        L.call("znn_memcpy_d2h", out.ctypes.data, g, out.nbytes)
        assert not out.any()
    L.call("znn_param_slab_destroy", s)


def test_cuda_graph_survives_scratch_growth_and_option_changes(ops, L):
    """A captured training step holds raw scratch addresses and baked-in scalars.  After (a) an evaluation at a larger
    batch and a large direct GEMM that make the scratch blocks grow (the old blocks are freed) and (b) a change of the
    learning rate, the replaying model must keep producing exactly what an eager model produces."""
    from znn_b200.models import Model
    dims = (784, 128, 64, 10)
    r = np.random.default_rng(9)
    P0 = models.init_params("mlp", dims, seed=10)
    batches = [((r.integers(0, 256, (64, 784)) / 255.0).astype(np.float32), r.integers(0, 10, 64).astype(np.int32))
               for _ in range(8)]
    big_x = (r.integers(0, 256, (4096, 784)) / 255.0).astype(np.float32)
    A = r.standard_normal((300, 8200), np.float32)       # unaligned-K product on the planes path: grows slot 0
    finals = []
    for use_graph in (0, 1):
        m = Model("mlp", dims, arena_bytes=256 << 20)
        m.set_params(P0)
        m.set_option("lr", 0.05)
        m.set_option("momentum", 0.9)
        m.set_option("cuda_graph", use_graph)
        dx, dt = ops.DevBuf(64 * 784 * 4), ops.DevBuf(64 * 4)
        losses = []
        for i, (x, t) in enumerate(batches):
            if i == 4:
                m.forward(big_x, classes=10)                                  # larger batch: scratch may grow
                ops.set_gemm_path(3)
                ops.sgemm(111, 112, 300, 300, 8199, 1.0, A[:, :8199].copy(), 8199, A[:, :8199].copy(), 8199, 0.0,
                          np.zeros((300, 300), np.float32), 300)
                ops.set_gemm_path(0)
                m.set_option("lr", 0.01)                                      # a schedule step
            L.call("znn_memcpy_h2d", dx.ptr, x.ctypes.data, x.nbytes)
            L.call("znn_memcpy_h2d", dt.ptr, t.ctypes.data, t.nbytes)
            L.call("znn_sync")
            loss = C.c_float()
            L.call("znn_model_train_step", m.h, dx.ptr, dt.ptr, 64, 0, 1, C.byref(loss))
            losses.append(loss.value)
        finals.append((losses, m.get_params(), m.graph_replays()))
        m.close()
    assert finals[0][0] == finals[1][0]
    for k in finals[0][1]:
        np.testing.assert_array_equal(finals[0][1][k], finals[1][1][k])
    assert finals[1][2] >= 4
    assert status(L) == 0


def test_two_host_threads_with_their_own_streams(ops, L):
    """Each host thread launches on its own stream (znn_set_stream) and gets its own scratch blocks, so concurrent
    split-K and planes-path products do not trample each other's partial sums."""
    import torch
    r = np.random.default_rng(12)
    cases = []
    for i in range(2):
        A = r.standard_normal((300 + 4 * i, 4100), np.float32)
        B = r.standard_normal((4100, 200), np.float32)
        cases.append((A, B, A.astype(np.float64) @ B.astype(np.float64)))
    streams = [torch.cuda.Stream() for _ in range(2)]
    errs, outs = [None, None], [None, None]

    def work(i):
        try:
            L.call("znn_init", 0)
            L.call("znn_set_stream", C.c_void_p(streams[i].cuda_stream))
            A, B, _ = cases[i]
            dA, dB = ops.DevBuf.from_host(A), ops.DevBuf.from_host(B)
            dC = ops.DevBuf(A.shape[0] * 200 * 4)
            for _ in range(20):
                L.call("znn_sgemm", 101, 111, 111, A.shape[0], 200, 4100, C.c_float(1.0), dA.ptr, 4100, dB.ptr, 200,
                       C.c_float(0.0), dC.ptr, 200)
            outs[i] = dC.to_host((A.shape[0], 200))
            L.call("znn_set_stream", None)
        except Exception as e:   # noqa: BLE001
            errs[i] = e

    th = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert errs == [None, None], errs
    for i in range(2):
        e = np.linalg.norm(outs[i] - cases[i][2]) / np.linalg.norm(cases[i][2])
        assert e <= 1e-5, (i, e)
    assert status(L) == 0


def test_one_thread_drives_two_devices(ops, L):
    """znn_set_device: one host thread alternates between two GPUs; every per-device resource (stream, scratch, status
    word, the kernels' shared-memory attribute) must exist on both."""
    n = C.c_int()
    L.call("znn_device_count", C.byref(n))
    if n.value < 2:
        pytest.skip("needs two GPUs")
    r = np.random.default_rng(13)
    A, B = r.standard_normal((512, 1024), np.float32), r.standard_normal((1024, 384), np.float32)
    exact = A.astype(np.float64) @ B.astype(np.float64)
    try:
        bufs = {}
        for dev in (0, 1):
            L.call("znn_set_device", dev)
            bufs[dev] = (ops.DevBuf.from_host(A), ops.DevBuf.from_host(B), ops.DevBuf(512 * 384 * 4))
        for rep in range(3):
            for dev in (1, 0):
                L.call("znn_set_device", dev)
                dA, dB, dC = bufs[dev]
                L.call("znn_sgemm", 101, 111, 111, 512, 384, 1024, C.c_float(1.0), dA.ptr, 1024, dB.ptr, 384, C.c_float(0.0),
                       dC.ptr, 384)
        for dev in (0, 1):
            L.call("znn_set_device", dev)
            got = bufs[dev][2].to_host((512, 384))
            assert np.linalg.norm(got - exact) / np.linalg.norm(exact) <= 1e-5
            assert status(L) == 0
            for b in bufs[dev]:
                b.free()
    finally:
        L.call("znn_set_device", 0)
