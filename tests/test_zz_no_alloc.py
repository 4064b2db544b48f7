"""znn_softmax_xent_fwd_static: the SoftmaxCrossEntropy forward for callers that must not
allocate (fixed memory budgets, threads that cannot block in cudaMalloc).  It keeps its
per-row losses in a fixed device array inside the library, so its output must equal the
regular entry point's and the CPU oracle's -- on a first call and again on a second call that reuses the array
with different, smaller inputs.  This file sorts last so that it runs after every other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL = 1e-5   # the tolerance of the row-wise parity tests


def _both(ops, L, X, t):
    M, N = X.shape
    stream = C.c_void_p()
    L.call("znn_get_stream", C.byref(stream))
    dX, dt = ops.DevBuf.from_host(X), ops.DevBuf.from_host(t)
    p_ref, l_ref = ops.DevBuf(X.nbytes), ops.DevBuf(4)
    p_new, l_new = ops.DevBuf(X.nbytes), ops.DevBuf(4)
    L.call("znn_softmax_xent_fwd", dX.ptr, dt.ptr, p_ref.ptr, l_ref.ptr, M, N)
    L.call("znn_softmax_xent_fwd_static", dX.ptr, dt.ptr, p_new.ptr, l_new.ptr, M, N, stream)
    L.call("znn_sync")
    return (p_ref.to_host((M, N)), l_ref.to_host((1,))), (p_new.to_host((M, N)), l_new.to_host((1,)))


def test_static_scratch_matches_regular_entry_point_twice():
    from znn_b200 import ops
    from znn_b200._lib import ZnnError, lib
    ops.init(0)
    L = lib()
    r = np.random.default_rng(2024)
    for M, N in ((4096, 1000), (37, 10)):        # second call: fewer rows, stale rows stay in the array
        X = (r.standard_normal((M, N)) * 3.0).astype(np.float32)
        t = r.integers(0, N, M).astype(np.int32)
        (p_ref, l_ref), (p_new, l_new) = _both(ops, L, X, t)
        assert np.isfinite(l_new).all() and float(l_new[0]) > 0.0
        np.testing.assert_allclose(p_new, p_ref, rtol=RTOL, atol=1e-12)
        np.testing.assert_allclose(l_new, l_ref, rtol=RTOL)
        # and against the CPU oracle's restatement of the reference loop (src/autodiff.zig:196-238)
        from oracle import zo
        l_cpu, p_cpu = zo.softmax_xent_fwd(X, t)
        np.testing.assert_allclose(p_new, p_cpu, rtol=RTOL, atol=1e-12)
        np.testing.assert_allclose(l_new, np.asarray(l_cpu).reshape(-1), rtol=RTOL)
    # beyond the fixed array: refused on the host, nothing is launched
    big = 65537
    with pytest.raises(ZnnError) as ei:
        L.call("znn_softmax_xent_fwd_static", 1, 1, 1, 1, big, 4, None)
    assert ei.value.code == -1 and "65536" in str(ei.value)
