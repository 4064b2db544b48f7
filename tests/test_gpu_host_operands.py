"""znn_sgemm_host / znn_matmul_host_fwd_bwd: the GEMM boundary with HOST operands, as the reference's
binding passes them (src/cblas.zig:17-34 receives host slices), pipelined by panels inside the shim.

The checker is the CPU oracle's sgemm on the same arrays; the bar is the GEMM bar (normwise relative
error <= 1e-5).  Panel counts are forced so that ragged last panels, leading-dimension padding, both
transposes, beta != 0 and gradient accumulation all cross the panel seams.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NT, T = 111, 112
TOL = 1e-5


@pytest.fixture(scope="module")
def ops():
    from znn_b200 import ops as _ops
    _ops.init(0)
    _ops.set_gemm_path(0)
    return _ops


def rel_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(1e-30, np.linalg.norm(want)))


@pytest.mark.parametrize("panels", [0, 1, 3])
@pytest.mark.parametrize("ta,tb", [(NT, NT), (NT, T), (T, NT), (T, T)])
@pytest.mark.parametrize("M,N,K,pad", [(1, 1, 1, 0), (300, 200, 100, 0), (515, 260, 96, 3), (1000, 384, 512, 4)])
def test_sgemm_host_matches_oracle(ops, zo, panels, ta, tb, M, N, K, pad):
    r = np.random.default_rng(M * 7 + N + K + ta + tb)
    A = r.standard_normal((M, K + pad) if ta == NT else (K, M + pad), np.float32)
    B = r.standard_normal((K, N + pad) if tb == NT else (N, K + pad), np.float32)
    C0 = r.standard_normal((M, N + pad), np.float32)
    for alpha, beta in ((1.0, 0.0), (0.5, 1.0), (-1.25, 0.75)):
        want, got = C0.copy(), C0.copy()
        zo.sgemm(ta, tb, M, N, K, alpha, A, A.shape[1], B, B.shape[1], beta, want, N + pad, naive=True)
        ops.sgemm_host(ta, tb, M, N, K, alpha, A, A.shape[1], B, B.shape[1], beta, got, N + pad, panels=panels)
        if pad:
            np.testing.assert_array_equal(got[:, N:], C0[:, N:])
        e = rel_err(got[:, :N], want[:, :N])
        assert e <= TOL, f"{ta},{tb} {M}x{N}x{K} panels={panels} alpha={alpha} beta={beta}: {e:.3e}"


def test_sgemm_host_beta_zero_ignores_old_c(ops):
    r = np.random.default_rng(3)
    A, B = r.standard_normal((260, 64), np.float32), r.standard_normal((64, 130), np.float32)
    got = np.full((260, 130), np.nan, np.float32)
    ops.sgemm_host(NT, NT, 260, 130, 64, 1.0, A, 64, B, 130, 0.0, got, 130, panels=2)
    assert np.isfinite(got).all()
    assert rel_err(got, A.astype(np.float64) @ B.astype(np.float64)) <= TOL


def test_sgemm_host_degenerate(ops):
    A, B = np.ones((4, 4), np.float32), np.ones((4, 4), np.float32)
    Cm = np.full((4, 4), 2.0, np.float32)
    ops.sgemm_host(NT, NT, 0, 4, 4, 1.0, A, 4, B, 4, 0.0, Cm, 4)          # M = 0: nothing happens
    assert (Cm == 2.0).all()
    ops.sgemm_host(NT, NT, 4, 4, 0, 1.0, A, 4, B, 4, 0.5, Cm, 4)          # K = 0: C = beta * C
    assert (Cm == 1.0).all()
    ops.sgemm_host(NT, NT, 4, 4, 4, 0.0, A, 4, B, 4, 3.0, Cm, 4)          # alpha = 0: C = beta * C
    assert (Cm == 3.0).all()
    with pytest.raises(RuntimeError):
        ops.sgemm_host(NT, NT, 4, 4, 4, 1.0, A, 3, B, 4, 0.0, Cm, 4)      # lda too small
    with pytest.raises(RuntimeError):
        ops.sgemm_host(NT, NT, 4, 4, 4, 1.0, A, 4, B, 4, 0.0, Cm, 3)      # ldc too small


@pytest.mark.parametrize("panels", [0, 1, 3])
@pytest.mark.parametrize("M,K,N", [(2, 3, 2), (130, 70, 258), (1000, 300, 700), (2304, 256, 640)])
def test_matmul_host_fwd_bwd_matches_oracle(ops, zo, panels, M, K, N):
    r = np.random.default_rng(M + K + N)
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32)
    dC = r.standard_normal((M, N), np.float32)
    wC = zo.matmul_fwd(A, B)
    wdA, wdB = np.zeros((M, K), np.float32), np.zeros((K, N), np.float32)
    zo.matmul_bwd(A, B, dC, wdA, wdB)
    Cm, dA, dB = ops.matmul_host_fwd_bwd(A, B, dC, panels=panels)
    for name, got, want in (("C", Cm, wC), ("dA", dA, wdA), ("dB", dB, wdB)):
        e = rel_err(got, want)
        assert e <= TOL, f"{name} {M}x{K}x{N} panels={panels}: {e:.3e}"
    # the reference accumulates gradients: a second backward doubles them
    zo.matmul_bwd(A, B, dC, wdA, wdB)
    Cm2, dA2, dB2 = ops.matmul_host_fwd_bwd(A, B, dC, dA=dA, dB=dB, panels=panels)
    np.testing.assert_array_equal(Cm2, Cm)
    assert rel_err(dA2, wdA) <= TOL and rel_err(dB2, wdB) <= TOL


def test_matmul_host_partial_outputs(ops, zo):
    r = np.random.default_rng(11)
    A, B = r.standard_normal((300, 64), np.float32), r.standard_normal((64, 200), np.float32)
    dC = r.standard_normal((300, 200), np.float32)
    Cm, dA, dB = ops.matmul_host_fwd_bwd(A, B)                      # forward only
    assert dA is None and dB is None and rel_err(Cm, zo.matmul_fwd(A, B)) <= TOL
    _, dA, dB = ops.matmul_host_fwd_bwd(A, B, dC, want_dA=False)    # requires_grad false on A
    wdB = np.zeros_like(B)
    zo.matmul_bwd(A, B, dC, None, wdB)
    assert dA is None and rel_err(dB, wdB) <= TOL


def test_matmul_host_same_bits_as_device_resident_calls(ops):
    """The panels cut M and N on tile boundaries, so each element is produced by the same kernel
    arithmetic as in one whole-matrix call on the same path."""
    r = np.random.default_rng(5)
    M, K, N = 2048, 512, 1024
    A, B = r.standard_normal((M, K), np.float32), r.standard_normal((K, N), np.float32)
    ops.set_gemm_path(4)
    try:
        whole = np.zeros((M, N), np.float32)
        ops.sgemm(NT, NT, M, N, K, 1.0, A, K, B, N, 0.0, whole, N)
        piped, _, _ = ops.matmul_host_fwd_bwd(A, B, panels=4)
    finally:
        ops.set_gemm_path(0)
    np.testing.assert_array_equal(piped, whole)
