"""The fused causal-attention kernels (znn_attn_fwd / znn_attn_bwd) against the CPU oracle running the reference's
literal operator sequence (src/nn.zig:796-906): batchMatMul(Q, K^T) -> mulScalar -> add(-1e9 mask) -> softmax ->
batchMatMul(P, V), and its backward arms in reverse.  Bar: normwise relative error <= 1e-5 for O, dQ, dK and dV."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5


@pytest.fixture(scope="module")
def ops():
    from znn_b200 import ops as _ops
    from znn_b200._lib import lib
    _ops.init(0)
    # a short limit for the device-side waits of this module (0.2 s): a stalled pipeline ends the test, not the run
    lib().call("znn_debug_set_wait_limit", 400000000)
    yield _ops
    lib().call("znn_debug_set_wait_limit", 0)


@pytest.fixture()
def blas():
    from oracle import zo
    ptr, info = zo.find_host_cblas()
    if ptr is not None:
        zo.bind_sgemm(ptr)
    yield
    zo.bind_sgemm(None)


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(1e-30, np.linalg.norm(b)))


def oracle_attention(Q, K, V, dO, scale):
    """[B, nh, T, hs] arrays through the oracle's operator loops, forward and backward, literally as the reference."""
    from oracle import zo
    B, nh, T, hs = Q.shape
    Kt = zo.transpose_fwd(K, 2, 3)
    S = zo.batch_matmul_fwd(Q, Kt)
    Ss = zo.mul_scalar_fwd(S, scale)
    mask = np.zeros((B, nh, T, T), np.float32)
    iu = np.triu_indices(T, 1)
    mask[:, :, iu[0], iu[1]] = -1e9
    P = zo.softmax_fwd(zo.add_fwd(Ss, mask))
    O = zo.batch_matmul_fwd(P, V)
    dP, dV = np.zeros_like(P), np.zeros_like(V)
    zo.batch_matmul_bwd(P, V, dO, dP, dV)
    dM = np.zeros_like(P)
    zo.softmax_bwd(P, dP, dM)
    dS = np.zeros_like(P)
    zo.mul_scalar_bwd(dM, scale, dS)          # add's backward passes dM through unchanged
    dQ, dKt = np.zeros_like(Q), np.zeros_like(Kt)
    zo.batch_matmul_bwd(Q, Kt, dS, dQ, dKt)
    dK = np.zeros_like(K)
    zo.transpose_bwd(dKt, dK, 2, 3)
    return O, dQ, dK, dV


@pytest.mark.parametrize("B,nh,T,hs", [(2, 2, 256, 64), (1, 3, 1024, 64), (2, 2, 520, 32), (1, 1, 64, 64), (1, 2, 388, 64)])
@pytest.mark.parametrize("layout", ["bhtd", "bthd"])
def test_fused_attention_matches_the_literal_sequence(ops, blas, B, nh, T, hs, layout):
    r = np.random.default_rng(T * 7 + hs + nh)
    Q, K, V, dO = (r.standard_normal((B, nh, T, hs), np.float32) for _ in range(4))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hs)))
    Oo, dQo, dKo, dVo = oracle_attention(Q, K, V, dO, scale)
    tr = (lambda a: np.ascontiguousarray(a.transpose(0, 2, 1, 3))) if layout == "bthd" else (lambda a: a)
    back = (lambda a: a.transpose(0, 2, 1, 3)) if layout == "bthd" else (lambda a: a)
    O, LSE = ops.attn_fwd(tr(Q), tr(K), tr(V), scale, layout)
    e = rel(back(O), Oo)
    assert e <= TOL, f"O: {e:.3e}"
    dQ, dK, dV = ops.attn_bwd(tr(Q), tr(K), tr(V), O, tr(dO), LSE, scale, layout)
    for name, got, want in (("dQ", dQ, dQo), ("dK", dK, dKo), ("dV", dV, dVo)):
        e = rel(back(got), want)
        assert e <= TOL, f"{name}: {e:.3e}"


def test_fused_attention_accumulates_and_skips_null_gradients(ops):
    r = np.random.default_rng(5)
    B, nh, T, hs = 1, 2, 320, 64
    Q, K, V, dO = (r.standard_normal((B, nh, T, hs), np.float32) for _ in range(4))
    O, LSE = ops.attn_fwd(Q, K, V, 0.125)
    dQ, dK, dV = ops.attn_bwd(Q, K, V, O, dO, LSE, 0.125)
    g0 = [r.standard_normal((B, nh, T, hs), np.float32) for _ in range(3)]
    aQ, aK, aV = ops.attn_bwd(Q, K, V, O, dO, LSE, 0.125, grads=g0)
    for got, base, inc in ((aQ, g0[0], dQ), (aK, g0[1], dK), (aV, g0[2], dV)):
        np.testing.assert_array_equal(got, base + inc)
    only = ops.attn_bwd(Q, K, V, O, dO, LSE, 0.125, want=(False, True, False))
    assert only[0] is None and only[2] is None
    np.testing.assert_array_equal(only[1], dK)                     # deterministic
    # scaling the upstream gradient by a power of two scales every gradient exactly
    dQ2, dK2, dV2 = ops.attn_bwd(Q, K, V, O, dO * np.float32(4.0), LSE, 0.125)
    np.testing.assert_array_equal(dV2, dV * np.float32(4.0))
    np.testing.assert_array_equal(dQ2, dQ * np.float32(4.0))


def test_fused_attention_rejects_what_it_cannot_run(ops):
    from znn_b200._lib import ZnnError, lib
    buf = ops.DevBuf(1 << 20)
    with pytest.raises(ZnnError) as ei:
        lib().call("znn_attn_fwd", buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 1, 1, 64, 48, 48, 64 * 48, 64 * 48, 0.1)
    assert ei.value.code == -6
    with pytest.raises(ZnnError) as ei:
        lib().call("znn_attn_fwd", buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 1, 1, 66, 64, 64, 66 * 64, 66 * 64, 0.1)
    assert ei.value.code == -6


@pytest.mark.parametrize("layout", ["bhtd", "bthd"])
def test_precomputed_remainder_planes_equal_in_kernel_conversion(ops, layout):
    """Default form: converter warps split every landed tile inside the kernel.  The other form
    (znn_debug_set_attn_planes(1)) makes the remainder (lo) planes of the shared-memory operands once in a pre-pass and
    loads them by TMA.  Same arithmetic on the same values: every output bit-identical."""
    from znn_b200._lib import lib
    r = np.random.default_rng(77)
    B, nh, T, hs = 2, 3, 712, 64
    shape = (B, nh, T, hs) if layout == "bhtd" else (B, T, nh, hs)
    Q, K, V, dO = (r.standard_normal(shape, np.float32) for _ in range(4))
    res = []
    try:
        for planes in (1, 0):
            lib().call("znn_debug_set_attn_planes", planes)
            O, LSE = ops.attn_fwd(Q, K, V, 0.125, layout)
            res.append((O, LSE) + tuple(ops.attn_bwd(Q, K, V, O, dO, LSE, 0.125, layout)))
    finally:
        lib().call("znn_debug_set_attn_planes", 0)
    for a, b in zip(res[0], res[1]):
        np.testing.assert_array_equal(a, b)


def test_issue_order_of_the_second_products_does_not_change_a_bit(ops):
    """By default the MMA issuer issues a block's second product as soon as its inputs are there, possibly before the
    next block's first product; znn_debug_set_attn_issue_order(1) keeps the fixed order.  The two products of different
    blocks use different buffers, so every output is bit-identical."""
    from znn_b200._lib import lib
    r = np.random.default_rng(78)
    B, nh, T, hs = 2, 5, 1000, 64
    Q, K, V, dO = (r.standard_normal((B, T, nh, hs), np.float32) for _ in range(4))
    res = []
    try:
        for in_order in (1, 0):
            lib().call("znn_debug_set_attn_issue_order", in_order)
            O, LSE = ops.attn_fwd(Q, K, V, 0.125, "bthd")
            res.append((O, LSE) + tuple(ops.attn_bwd(Q, K, V, O, dO, LSE, 0.125, "bthd")))
    finally:
        lib().call("znn_debug_set_attn_issue_order", 0)
    for a, b in zip(res[0], res[1]):
        np.testing.assert_array_equal(a, b)


def test_unit_schedule_table_does_not_change_a_bit(ops):
    """The work units are dealt to the CTA pairs by a host-made table (longest unit to the least loaded pair) or, with
    znn_debug_set_attn_schedule(0), by the kernel's own arithmetic.  Each unit is computed by exactly one pair with the
    same arithmetic: outputs are bit-identical.  96 units of 1-4 row blocks on 74 pairs: several units per pair."""
    from znn_b200._lib import lib
    r = np.random.default_rng(79)
    B, nh, T, hs = 4, 12, 520, 64
    Q, K, V, dO = (r.standard_normal((B, T, nh, hs), np.float32) for _ in range(4))
    res = []
    try:
        for sched in (0, 1):
            lib().call("znn_debug_set_attn_schedule", sched)
            O, LSE = ops.attn_fwd(Q, K, V, 0.125, "bthd")
            res.append((O, LSE) + tuple(ops.attn_bwd(Q, K, V, O, dO, LSE, 0.125, "bthd")))
    finally:
        lib().call("znn_debug_set_attn_schedule", 1)
    for a, b in zip(res[0], res[1]):
        np.testing.assert_array_equal(a, b)
