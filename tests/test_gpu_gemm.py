"""znn_sgemm (the cblas_sgemm boundary) against the CPU oracle and an fp64 arbiter.

Bar (from the workload definition): normwise relative error <= 1e-5 against the
reference sgemm on N(0,1) inputs, for the forward product and both backward
products, on every code path: fp32-FMA kernel (1), tcgen05 one-CTA tiles (2) and
CTA-pair tiles (3) over pre-split operand planes, CTA-pair tiles reading the
operands in place (4), and the automatic choice (0).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NT, T = 111, 112
TOL = 1e-5


@pytest.fixture(scope="module")
def ops():
    from znn_b200 import ops as _ops
    _ops.init(0)
    yield _ops
    _ops.set_gemm_path(0)


def rel_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(1e-30, np.linalg.norm(want)))


def make(ta, tb, M, N, K, seed, lda_pad=0, ldb_pad=0):
    r = np.random.default_rng(seed)
    a_shape = (M, K + lda_pad) if ta == NT else (K, M + lda_pad)
    b_shape = (K, N + ldb_pad) if tb == NT else (N, K + ldb_pad)
    return r.standard_normal(a_shape, np.float32), r.standard_normal(b_shape, np.float32)


def run_case(ops, zo, path, ta, tb, M, N, K, alpha=1.0, beta=0.0, lda_pad=0, ldb_pad=0, ldc_pad=0, seed=0):
    A, B = make(ta, tb, M, N, K, seed, lda_pad, ldb_pad)
    r = np.random.default_rng(seed + 1)
    C0 = r.standard_normal((M, N + ldc_pad), np.float32)
    lda, ldb, ldc = A.shape[1], B.shape[1], N + ldc_pad
    want = C0.copy()
    zo.sgemm(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, want, ldc, naive=True)
    got = C0.copy()
    ops.set_gemm_path(path)
    ops.sgemm(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, got, ldc)
    if path == 4:
        # in-place operand reads need 16-byte aligned leading dimensions; otherwise the planes path runs
        assert ops.last_gemm_path() == (4 if (lda % 4 == 0 and ldb % 4 == 0) else 3)
    elif path != 0:
        assert ops.last_gemm_path() == path
    if ldc_pad:  # columns beyond N are not touched
        np.testing.assert_array_equal(got[:, N:], C0[:, N:])
    e = rel_err(got[:, :N], want[:, :N])
    assert e <= TOL, f"path {path} {ta},{tb} {M}x{N}x{K} alpha={alpha} beta={beta}: rel err {e:.3e} vs oracle"
    return got


SMALL = [(2, 2, 3), (1, 1, 1), (64, 10, 784), (64, 128, 784), (33, 65, 17), (128, 256, 32), (130, 258, 70),
         (256, 256, 256), (200, 64, 96), (300, 72, 1000)]


@pytest.mark.parametrize("path", [1, 2, 3, 4])
@pytest.mark.parametrize("M,N,K", SMALL)
def test_forward_nn(ops, zo, path, M, N, K):
    run_case(ops, zo, path, NT, NT, M, N, K, seed=M + N + K)


@pytest.mark.parametrize("path", [1, 2, 3, 4])
@pytest.mark.parametrize("ta,tb", [(NT, T), (T, NT), (T, T)])
@pytest.mark.parametrize("M,N,K", [(64, 10, 784), (130, 258, 70), (256, 128, 512), (132, 260, 72), (384, 320, 96)])
def test_transposed_accumulate(ops, zo, path, ta, tb, M, N, K):
    """The backward calls: dA += dC.B^T (NoTrans,Trans) and dB += A^T.dC (Trans,NoTrans), beta = 1."""
    run_case(ops, zo, path, ta, tb, M, N, K, beta=1.0, seed=7 * M + N)


@pytest.mark.parametrize("path", [1, 2, 3, 4])
def test_alpha_beta_and_leading_dimensions(ops, zo, path):
    run_case(ops, zo, path, NT, NT, 150, 90, 200, alpha=0.5, beta=-2.0, lda_pad=3, ldb_pad=5, ldc_pad=7, seed=3)
    run_case(ops, zo, path, T, T, 129, 257, 65, alpha=2.0, beta=0.0, lda_pad=1, ldb_pad=2, ldc_pad=1, seed=4)
    # padded but TMA-readable leading dimensions: the in-place path must honour them
    run_case(ops, zo, path, NT, NT, 152, 92, 200, alpha=0.5, beta=-2.0, lda_pad=4, ldb_pad=8, ldc_pad=4, seed=5)
    run_case(ops, zo, path, T, NT, 136, 264, 68, alpha=1.5, beta=1.0, lda_pad=8, ldb_pad=4, ldc_pad=0, seed=6)


def test_beta_zero_ignores_old_c(ops):
    """beta == 0 must overwrite C even when it holds NaN (the reference memsets, cblas.zig:56-60)."""
    r = np.random.default_rng(5)
    for path in (1, 2, 3, 4):
        A, B = r.standard_normal((128, 64), np.float32), r.standard_normal((64, 256), np.float32)
        Cm = np.full((128, 256), np.nan, np.float32)
        ops.set_gemm_path(path)
        ops.sgemm(NT, NT, 128, 256, 64, 1.0, A, 64, B, 256, 0.0, Cm, 256)
        assert np.isfinite(Cm).all()


def test_degenerate(ops, zo):
    ops.set_gemm_path(0)
    Cm = np.ones((4, 5), np.float32)
    A, B = np.ones((4, 1), np.float32), np.ones((1, 5), np.float32)
    ops.sgemm(NT, NT, 4, 5, 0, 1.0, A, 1, B, 5, 0.0, Cm, 5)      # K == 0: C = beta*C
    assert (Cm == 0).all()
    Cm = np.full((4, 5), 3.0, np.float32)
    ops.sgemm(NT, NT, 4, 5, 1, 0.0, A, 1, B, 5, 0.5, Cm, 5)      # alpha == 0
    assert (Cm == 1.5).all()
    ops.sgemm(NT, NT, 0, 5, 1, 1.0, A, 1, B, 5, 0.0, Cm, 5)      # empty M: no-op


@pytest.mark.parametrize("path", [1, 2, 3, 4])
def test_batched(ops, zo, path):
    """BatchMatMul forward/backward shapes of attention (per (b,h) slices)."""
    r = np.random.default_rng(11)
    nb, Tn, hs = 6, 96, 64
    q = r.standard_normal((nb, Tn, hs), np.float32)
    kt = r.standard_normal((nb, hs, Tn), np.float32)
    ops.set_gemm_path(path)
    got = ops.batch_matmul_fwd(q, kt)
    want = zo.batch_matmul_fwd(q, kt)
    assert rel_err(got, want) <= TOL
    dC = r.standard_normal((nb, Tn, Tn), np.float32)
    g = [np.zeros_like(q), np.zeros_like(kt)]
    h = [np.zeros_like(q), np.zeros_like(kt)]
    ops.batch_matmul_bwd(q, kt, dC, g[0], g[1])
    zo.batch_matmul_bwd(q, kt, dC, h[0], h[1])
    assert rel_err(g[0], h[0]) <= TOL and rel_err(g[1], h[1]) <= TOL


@pytest.mark.parametrize("path", [2, 3, 4, 0])
@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (1024, 1024, 1024), (64, 4096, 4096), (4096, 64, 4096)])
def test_sweep_shapes_vs_fp64(ops, zo, path, M, N, K):
    """Workload-definition sweep shapes that the fp64 arbiter finishes quickly on the CPU."""
    A, B = make(NT, NT, M, N, K, seed=M ^ N ^ K)
    ops.set_gemm_path(path)
    got = ops.matmul_fwd(A, B)
    exact = A.astype(np.float64) @ B.astype(np.float64)
    e = rel_err(got, exact)
    assert e <= TOL, f"{M}x{N}x{K} path {path}: rel err {e:.3e} vs fp64"
    dC = np.random.default_rng(9).standard_normal((M, N), np.float32)
    dA, dB = np.zeros_like(A), np.zeros_like(B)
    ops.matmul_bwd(A, B, dC, dA, dB)
    assert rel_err(dA, dC.astype(np.float64) @ B.astype(np.float64).T) <= TOL
    assert rel_err(dB, A.astype(np.float64).T @ dC.astype(np.float64)) <= TOL


def test_full_size_rows_vs_fp64(ops):
    """8192^3: sampled output rows against exact arithmetic, plus linearity in A."""
    n = 8192
    r = np.random.default_rng(8192)
    A, B = r.standard_normal((n, n), np.float32), r.standard_normal((n, n), np.float32)
    ops.set_gemm_path(0)
    got = ops.matmul_fwd(A, B)
    rows = r.choice(n, 24, replace=False)
    exact = A[rows].astype(np.float64) @ B.astype(np.float64)
    e = rel_err(got[rows], exact)
    assert e <= TOL, f"8192^3 sampled rows: rel err {e:.3e} vs fp64"
    got2 = ops.matmul_fwd(A * np.float32(2.0), B)   # scaling by a power of two is exact
    np.testing.assert_array_equal(got2, got * np.float32(2.0))


@pytest.mark.parametrize("path", [2, 3, 4])
@pytest.mark.parametrize("ta,tb,M,N,K", [(T, NT, 768, 768, 8192), (T, NT, 300, 200, 4100), (NT, NT, 256, 512, 2048),
                                          (NT, T, 128, 64, 4096)])
def test_split_k_parameter_gradient_shapes(ops, path, ta, tb, M, N, K):
    """Few output tiles, long contraction (dW = X^T dY): K is split over CTAs and reduced in a fixed
    order; accumulate semantics (beta = 1) and bit-reproducibility must hold."""
    from znn_b200._lib import lib
    A, B = make(ta, tb, M, N, K, seed=K + M)
    C0 = np.random.default_rng(4).standard_normal((M, N), np.float32)
    a64 = A.astype(np.float64) if ta == NT else A.astype(np.float64).T
    b64 = B.astype(np.float64) if tb == NT else B.astype(np.float64).T
    exact = a64 @ b64 + C0
    ops.set_gemm_path(path)
    outs = []
    for splitk in (1, 1, 0):
        lib().call("znn_gemm_set_splitk", splitk)
        got = C0.copy()
        ops.sgemm(ta, tb, M, N, K, 1.0, A, A.shape[1], B, B.shape[1], 1.0, got, N)
        outs.append(got)
        e = rel_err(got, exact)
        assert e <= TOL, f"split-K={splitk} {M}x{N}x{K}: rel err {e:.3e} vs fp64"
    lib().call("znn_gemm_set_splitk", 1)
    np.testing.assert_array_equal(outs[0], outs[1])          # deterministic reduction order


def test_tensor_core_ignores_low_mantissa_bits(ops):
    """The in-place path feeds raw fp32 tiles as the hi operand (conv mode 1) on the strength of the tensor
    core dropping the 13 low mantissa bits of a tf32 operand.  Mode 0 clears them explicitly: both must give
    bit-identical results, for K-major and MN-major operands."""
    from znn_b200._lib import lib
    r = np.random.default_rng(123)
    ops.set_gemm_path(4)
    for ta, tb in ((NT, NT), (T, NT), (NT, T)):
        A, B = make(ta, tb, 512, 384, 1024, seed=9)
        outs = []
        for mode in (0, 1):
            lib().call("znn_gemm_set_conv_mode", mode)
            got = np.zeros((512, 384), np.float32)
            ops.sgemm(ta, tb, 512, 384, 1024, 1.0, A, A.shape[1], B, B.shape[1], 0.0, got, 384)
            assert ops.last_gemm_path() == 4
            outs.append(got)
        np.testing.assert_array_equal(outs[0], outs[1])
    lib().call("znn_gemm_set_conv_mode", 1)


@pytest.mark.parametrize("ta,tb,M,N,K,batch", [(NT, NT, 2048, 2048, 96, 4), (NT, T, 1024, 64, 512, 20), (T, NT, 768, 384, 800, 9),
                                               (T, NT, 64, 1024, 256, 24), (NT, NT, 520, 1000, 72, 11)])
@pytest.mark.parametrize("beta", [0.0, 1.0])
def test_in_place_kernel_many_work_units_per_cta_pair(ops, ta, tb, M, N, K, batch, beta):
    """The in-place kernel is persistent: each CTA pair walks several output tiles, with pipeline stages and
    accumulator buffers carried across tiles (odd chunk counts shift the buffer parity from tile to tile).
    More tiles than the GPU has CTA pairs, ragged edges, beta on and off, against fp64."""
    r = np.random.default_rng(M + N + K + batch)
    A = r.standard_normal((batch, M, K) if ta == NT else (batch, K, M), np.float32)
    B = r.standard_normal((batch, K, N) if tb == NT else (batch, N, K), np.float32)
    C0 = r.standard_normal((batch, M, N), np.float32)
    got = C0.copy()
    ops.set_gemm_path(4)
    try:
        ops.sgemm_batched(ta, tb, M, N, K, 0.75, A, A.shape[2], A[0].size, B, B.shape[2], B[0].size, beta, got, N, M * N, batch)
        assert ops.last_gemm_path() == 4
    finally:
        ops.set_gemm_path(0)
    a64 = A.astype(np.float64) if ta == NT else A.astype(np.float64).transpose(0, 2, 1)
    b64 = B.astype(np.float64) if tb == NT else B.astype(np.float64).transpose(0, 2, 1)
    want = 0.75 * (a64 @ b64) + beta * C0
    for b in range(batch):
        assert rel_err(got[b], want[b]) <= TOL, f"slice {b}"


@pytest.mark.parametrize("T_,hd,batch", [(1024, 64, 3), (768, 64, 2), (520, 32, 2)])
def test_triangular_hints_of_the_causal_attention_products(ops, T_, hd, batch):
    """znn_sgemm_batched_strided_tri: the six products around a causal softmax with their structure hints give
    what the unhinted products give wherever the result may be read (everything, except above the diagonal
    for ZNN_TRI_C_LOWER)."""
    r = np.random.default_rng(T_ + hd)
    f32 = np.float32
    Q, Kt = r.standard_normal((batch, T_, hd), f32), r.standard_normal((batch, hd, T_), f32)
    V, dO = r.standard_normal((batch, T_, hd), f32), r.standard_normal((batch, T_, hd), f32)
    low = np.tril(np.ones((T_, T_), f32))
    P = (r.standard_normal((batch, T_, T_), f32) * low).astype(f32)      # lower-triangular, exact zeros above
    dS = (r.standard_normal((batch, T_, T_), f32) * low).astype(f32)
    ops.set_gemm_path(4)
    try:
        def both(ta, tb, M, N, K, A, B, beta, tri):
            C0 = r.standard_normal((batch, M, N), f32)
            lda, ldb = A.shape[2], B.shape[2]
            full = ops.sgemm_batched(ta, tb, M, N, K, 1.0, A, lda, A[0].size, B, ldb, B[0].size, beta, C0.copy(), N, M * N, batch)
            hint = ops.sgemm_batched_tri(ta, tb, M, N, K, 1.0, A, lda, A[0].size, B, ldb, B[0].size, beta, C0.copy(), N, M * N,
                                         batch, tri)
            assert ops.last_gemm_path() == 4
            return full, hint
        # S = Q.Kt: only the lower triangle is read
        full, hint = both(NT, NT, T_, T_, hd, Q, Kt, 0.0, ops.TRI_C_LOWER)
        assert rel_err(np.tril(hint), np.tril(full)) <= 1e-6
        # O = P.V, dQ = dS.Kt^T: left operand lower-triangular
        for (A, B, tb, N, beta) in ((P, V, NT, hd, 0.0), (dS, Kt, T, hd, 1.0)):
            full, hint = both(NT, tb, T_, N, T_, A, B, beta, ops.TRI_A_LOWER)
            assert rel_err(hint, full) <= 1e-6
        # dP = dO.V^T accumulated: only the lower triangle is read
        full, hint = both(NT, T, T_, T_, hd, dO, V, 1.0, ops.TRI_C_LOWER)
        assert rel_err(np.tril(hint), np.tril(full)) <= 1e-6
        # dV = P^T.dO: left operand upper-triangular after the transpose
        full, hint = both(T, NT, T_, hd, T_, P, dO, 1.0, ops.TRI_A_UPPER)
        assert rel_err(hint, full) <= 1e-6
        # dKt = Q^T.dS: right operand lower-triangular
        full, hint = both(T, NT, hd, T_, T_, Q, dS, 1.0, ops.TRI_B_LOWER)
        assert rel_err(hint, full) <= 1e-6
    finally:
        ops.set_gemm_path(0)


def test_persistent_and_per_tile_launch_give_the_same_bits(ops):
    """znn_gemm_set_persistent: the persistent walk and one CTA pair per tile run the same arithmetic per element;
    and no bounded device-side wait expired anywhere in this module (znn_gemm_wait_record stays all zero)."""
    import ctypes as C
    from znn_b200._lib import lib
    r = np.random.default_rng(77)
    M, N, K = 1536, 1280, 640
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32)
    C0 = r.standard_normal((M, N), np.float32)
    res = []
    ops.set_gemm_path(4)
    try:
        for pers in (1, 0):
            lib().call("znn_gemm_set_persistent", pers)
            got = C0.copy()
            ops.sgemm(NT, NT, M, N, K, 1.0, A, K, B, N, 1.0, got, N)
            assert ops.last_gemm_path() == 4
            res.append(got)
    finally:
        lib().call("znn_gemm_set_persistent", 1)
        ops.set_gemm_path(0)
    np.testing.assert_array_equal(res[0], res[1])
    rec = (C.c_int * 16)()
    lib().call("znn_gemm_wait_record", rec)
    assert list(rec) == [0] * 16


@pytest.mark.parametrize("n", [2048, 4096])
def test_square_sweep_2048_4096_vs_fp64(ops, n):
    """The two sweep sizes between the L2-resident shapes and 8192^3 (4096^3 is where the tail split of the
    persistent walk engages): forward, dA and dB against exact arithmetic on sampled rows."""
    r = np.random.default_rng(n)
    A, B = r.standard_normal((n, n), np.float32), r.standard_normal((n, n), np.float32)
    dC = r.standard_normal((n, n), np.float32)
    ops.set_gemm_path(0)
    C = ops.matmul_fwd(A, B)
    dA, dB = np.zeros_like(A), np.zeros_like(B)
    ops.matmul_bwd(A, B, dC, dA, dB)
    assert ops.last_gemm_path() == 4
    rows = r.choice(n, 32, replace=False)
    A64, B64, dC64 = A.astype(np.float64), B.astype(np.float64), dC.astype(np.float64)
    for name, got, exact in (("C", C[rows], A64[rows] @ B64), ("dA", dA[rows], dC64[rows] @ B64.T),
                             ("dB", dB[rows], A64[:, rows].T @ dC64)):
        e = rel_err(got, exact)
        assert e <= TOL, f"{n}^3 {name}: rel err {e:.3e} vs fp64"


def test_full_size_backward_rows_vs_fp64(ops):
    """8192^3: dA += dC.B^T and dB += A^T.dC (beta = 1 into zeroed gradients) on sampled rows against exact arithmetic."""
    n = 8192
    r = np.random.default_rng(8193)
    A, B = r.standard_normal((n, n), np.float32), r.standard_normal((n, n), np.float32)
    dC = r.standard_normal((n, n), np.float32)
    ops.set_gemm_path(0)
    dA, dB = np.zeros_like(A), np.zeros_like(B)
    ops.matmul_bwd(A, B, dC, dA, dB)
    rows = r.choice(n, 16, replace=False)
    e = rel_err(dA[rows], dC[rows].astype(np.float64) @ B.astype(np.float64).T)
    assert e <= TOL, f"8192^3 dA sampled rows: rel err {e:.3e} vs fp64"
    e = rel_err(dB[rows], A[:, rows].astype(np.float64).T @ dC.astype(np.float64))
    assert e <= TOL, f"8192^3 dB sampled rows: rel err {e:.3e} vs fp64"


@pytest.mark.parametrize("form", ["beta1", "bias", "plain"])
def test_tail_split_on_and_off(ops, form):
    """znn_gemm_set_tail_split: 4096 x 4096 x 1024 has 256 tiles for 74 CTA pairs, so the last round of the persistent
    walk is 46 % full and its tiles are cut into K-slices added by tail_reduce_kernel.  With the split on and off the
    product must agree with exact arithmetic, with accumulation (beta = 1) and with a fused bias, and the split
    result must be bit-reproducible run to run (fixed slice order)."""
    from znn_b200._lib import lib
    M = N = 4096
    K = 1024
    r = np.random.default_rng(77)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32)
    C0 = r.standard_normal((M, N), np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    rows = r.choice(M, 24, replace=False)
    exact = A[rows].astype(np.float64) @ B.astype(np.float64)
    if form == "beta1":
        exact = exact + C0[rows]
    elif form == "bias":
        exact = exact + bias[None, :]
    ops.set_gemm_path(4)
    outs = []
    try:
        for split in (1, 1, 0):
            lib().call("znn_gemm_set_tail_split", split)
            lib().call("znn_launch_count", C.byref(C.c_longlong()), 1)
            if form == "bias":
                got = ops.linear_fwd(A, B, bias)
            else:
                got = C0.copy()
                ops.sgemm(NT, NT, M, N, K, 1.0, A, K, B, N, 1.0 if form == "beta1" else 0.0, got, N)
            n = C.c_longlong()
            lib().call("znn_launch_count", C.byref(n), 1)
            assert ops.last_gemm_path() == 4
            # the split adds exactly one launch (tail_reduce_kernel); host uploads launch nothing
            outs.append((got, n.value))
            e = rel_err(got[rows], exact)
            assert e <= TOL, f"tail split {split} {form}: rel err {e:.3e} vs fp64"
    finally:
        lib().call("znn_gemm_set_tail_split", 1)
    np.testing.assert_array_equal(outs[0][0], outs[1][0])
    assert outs[0][1] == outs[2][1] + 1, (outs[0][1], outs[2][1])
    ops.check_device_status()


def _gelu64(h):
    from math import erf, sqrt
    return 0.5 * h * (1.0 + np.vectorize(erf)(h / sqrt(2.0)))


def _gelu_grad64(h):
    from math import erf, sqrt, pi
    cdf = 0.5 * (1.0 + np.vectorize(erf)(h / sqrt(2.0)))
    return cdf + h * np.exp(-0.5 * h * h) / sqrt(2.0 * pi)


@pytest.mark.parametrize("M,K,N", [(1024, 384, 256), (1000, 200, 516), (1024, 256, 1280), (2048, 768, 3072)])
@pytest.mark.parametrize("act,res", [(0, True), (1, False), (2, False), (1, True)])
def test_linear_with_activation_and_residual_epilogue(ops, M, K, N, act, res):
    """znn_linear_fwd_ex: the activation (src/autodiff.zig:148-165) and the residual add (src/nn.zig:996-1021) in the
    GEMM epilogue, against the same steps in float64; the pre-activation copy equals the plain fused Linear bit for bit."""
    ops.set_gemm_path(0)
    r = np.random.default_rng(M + K + N + 7 * act)
    X = r.standard_normal((M, K), np.float32)
    W = (r.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    b = r.standard_normal(N).astype(np.float32)
    R = r.standard_normal((M, N), np.float32) if res else None
    Y, H = ops.linear_fwd_ex(X, W, b, act, R, want_pre=True)
    h64 = X.astype(np.float64) @ W.astype(np.float64) + b
    if res:
        h64 = h64 + R
    y64 = h64 if act == 0 else (np.maximum(h64, 0.0) if act == 1 else _gelu64(h64))
    scale = float(np.abs(h64).max())
    assert float(np.abs(H - h64).max()) <= 1e-5 * scale
    assert float(np.abs(Y - y64).max()) <= 1e-5 * scale
    if not res:
        np.testing.assert_array_equal(H, ops.linear_fwd(X, W, b))
    # the activation of the stored pre-activation, by the stand-alone kernel, equals the fused output to rounding
    if act == 1:
        np.testing.assert_array_equal(Y, np.maximum(H, 0.0))
    elif act == 2:
        assert float(np.abs(Y - ops.gelu_fwd(H)).max()) <= 1e-6 * scale


@pytest.mark.parametrize("M,K,N", [(1024, 256, 384), (1000, 516, 200), (2048, 3072, 768)])
@pytest.mark.parametrize("x_act", [1, 2])
@pytest.mark.parametrize("fresh", [1, 0])
def test_linear_backward_with_activation_gradient_epilogue(ops, M, K, N, x_act, fresh):
    """znn_linear_bwd_ex: dX = (dY.W^T) o act'(x_pre) in the epilogue of the data-gradient product, stored or added."""
    ops.set_gemm_path(0)
    r = np.random.default_rng(M + K + N + x_act)
    pre = r.standard_normal((M, K), np.float32)
    X = (np.maximum(pre, 0.0) if x_act == 1 else _gelu64(pre.astype(np.float64))).astype(np.float32)
    W = (r.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    dY = r.standard_normal((M, N), np.float32)
    dX0 = r.standard_normal((M, K), np.float32)
    dX, dW, db = dX0.copy(), np.zeros((K, N), np.float32), np.zeros(N, np.float32)
    ops.linear_bwd_ex(X, W, dY, dX, dW, db, pre, x_act, fresh)
    g = dY.astype(np.float64) @ W.astype(np.float64).T
    g = g * ((pre > 0) if x_act == 1 else _gelu_grad64(pre.astype(np.float64)))
    want = g + (0.0 if fresh else dX0)
    scale = float(np.abs(want).max())
    assert float(np.abs(dX - want).max()) <= 1e-5 * scale
    dW64 = X.astype(np.float64).T @ dY
    assert float(np.abs(dW - dW64).max()) <= 1e-5 * float(np.abs(dW64).max())
    assert float(np.abs(db - dY.sum(0, dtype=np.float64)).max()) <= 3e-5 * float(np.abs(dY.sum(0)).max())


def test_fused_epilogue_refuses_small_products(ops):
    """Below the tensor-core threshold the epilogue forms do not exist: a clear refusal, the caller keeps the two ops."""
    from znn_b200._lib import ZnnError
    X, W, b = np.ones((64, 32), np.float32), np.ones((32, 64), np.float32), np.zeros(64, np.float32)
    with pytest.raises(ZnnError):
        ops.linear_fwd_ex(X, W, b, act=1)


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (8, 4096, 2048), (20, 3000, 1284), (32, 1028, 2048)])
@pytest.mark.parametrize("ta,tb", [(111, 111), (111, 112), (112, 111), (112, 112)])
def test_skinny_products_run_transposed(ops, M, N, K, ta, tb):
    """8..64 rows against a wide, long matrix: computed as the transposed product and written back by a small kernel
    (path 5); values against float64, with beta = 1 and a leading dimension wider than N, and against the ordinary path."""
    from znn_b200 import _lib
    L = _lib.lib()
    ops.set_gemm_path(0)
    r = np.random.default_rng(M + N + K + ta + tb)
    A = r.standard_normal((M, K) if ta == 111 else (K, M)).astype(np.float32)
    B = r.standard_normal((K, N) if tb == 111 else (N, K)).astype(np.float32)
    ldc = N + 8
    C0 = r.standard_normal((M, ldc)).astype(np.float32)
    opA = A if ta == 111 else A.T
    opB = B if tb == 111 else B.T
    want = 0.5 * (opA.astype(np.float64) @ opB.astype(np.float64)) + C0[:, :N]
    got = ops.sgemm(ta, tb, M, N, K, 0.5, A, A.shape[1], B, B.shape[1], 1.0, C0.copy(), ldc)
    assert L.dll.znn_gemm_last_path() == 5
    scale = float(np.abs(want).max())
    assert float(np.abs(got[:, :N] - want).max()) <= 1e-5 * scale
    np.testing.assert_array_equal(got[:, N:], C0[:, N:])          # the padding columns are not touched
    L.call("znn_gemm_set_skinny", 0)
    try:
        ref = ops.sgemm(ta, tb, M, N, K, 0.5, A, A.shape[1], B, B.shape[1], 1.0, C0.copy(), ldc)
        assert L.dll.znn_gemm_last_path() != 5
    finally:
        L.call("znn_gemm_set_skinny", 1)
    assert float(np.abs(got[:, :N] - ref[:, :N]).max()) <= 1e-5 * scale   # (below 64 rows the ordinary path is the fp32-FMA kernel)


def test_skinny_linear_with_bias(ops):
    """The fused Linear of a 64-row batch (decode): bias added by the write-back kernel."""
    ops.set_gemm_path(0)
    r = np.random.default_rng(64)
    X = r.standard_normal((64, 768)).astype(np.float32)
    W = (r.standard_normal((768, 3072)) / 28.0).astype(np.float32)
    b = r.standard_normal(3072).astype(np.float32)
    got = ops.linear_fwd(X, W, b)
    want = X.astype(np.float64) @ W.astype(np.float64) + b
    assert float(np.abs(got - want).max()) <= 1e-5 * float(np.abs(want).max())


def test_grouped_products_shared_input_and_bias_per_slice(ops):
    """znn_sgemm_grouped, kcat = 0: three Linear layers on one input (the q, k, v projections, src/nn.zig:776-793) in one
    launch: A shared (stride 0), weights and biases at a uniform stride inside one parameter block, outputs in slices."""
    ops.set_gemm_path(0)
    r = np.random.default_rng(301)
    M, K, N, nb = 1024, 256, 384, 3
    X = r.standard_normal((M, K)).astype(np.float32)
    sW = K * N + N + 4                                   # weight, bias, a little padding: as in a parameter slab
    params = r.standard_normal(nb * sW).astype(np.float32)
    sY = 2 * M * N                                       # value and gradient buffers alternate in the arena
    Y = np.zeros(nb * sY, np.float32)
    ops.sgemm_grouped(111, 111, M, N, K, 1.0, X, K, 0, params, N, sW, 0.0, Y, N, sY, nb, bias=params[K * N:], sbias=sW)
    for s_ in range(nb):
        W = params[s_ * sW: s_ * sW + K * N].reshape(K, N).astype(np.float64)
        b = params[s_ * sW + K * N: s_ * sW + K * N + N].astype(np.float64)
        want = X.astype(np.float64) @ W + b
        got = Y[s_ * sY: s_ * sY + M * N].reshape(M, N)
        assert float(np.abs(got - want).max()) <= 1e-5 * float(np.abs(want).max())
        assert not Y[s_ * sY + M * N: (s_ + 1) * sY].any()           # the gap between the slices is untouched


def test_grouped_weight_gradients_and_concatenated_data_gradient(ops):
    """kcat = 0 with beta = 1 (dW_s += X^T.dY_s, X shared) and kcat = 1 (dX += sum_s dY_s.W_s^T as one product whose
    contraction runs through the slices)."""
    ops.set_gemm_path(0)
    r = np.random.default_rng(302)
    M, K, N, nb = 2048, 256, 256, 3
    X = r.standard_normal((M, K)).astype(np.float32)
    sY = 2 * M * N
    dY = np.zeros(nb * sY, np.float32)
    for s_ in range(nb):
        dY[s_ * sY: s_ * sY + M * N] = r.standard_normal(M * N).astype(np.float32)
    sW = K * N + N + 4
    W = r.standard_normal(nb * sW).astype(np.float32)
    dW0 = r.standard_normal(nb * sW).astype(np.float32)
    dW = dW0.copy()
    ops.sgemm_grouped(112, 111, K, N, M, 1.0, X, K, 0, dY, N, sY, 1.0, dW, N, sW, nb)
    dX0 = r.standard_normal((M, K)).astype(np.float32)
    dX = dX0.copy()
    ops.sgemm_grouped(111, 112, M, K, N, 1.0, dY, N, sY, W, N, sW, 1.0, dX, K, 0, nb, kcat=1)
    want_dx = dX0.astype(np.float64)
    for s_ in range(nb):
        g = dY[s_ * sY: s_ * sY + M * N].reshape(M, N).astype(np.float64)
        want = dW0[s_ * sW: s_ * sW + K * N].reshape(K, N) + X.astype(np.float64).T @ g
        got = dW[s_ * sW: s_ * sW + K * N].reshape(K, N)
        assert float(np.abs(got - want).max()) <= 1e-5 * float(np.abs(want).max())
        np.testing.assert_array_equal(dW[s_ * sW + K * N: (s_ + 1) * sW], dW0[s_ * sW + K * N: (s_ + 1) * sW])
        want_dx += g @ W[s_ * sW: s_ * sW + K * N].reshape(K, N).astype(np.float64).T
    assert float(np.abs(dX - want_dx).max()) <= 1e-5 * float(np.abs(want_dx).max())
