"""Host-array front end of the C ABI: every function copies its numpy inputs to
the device, makes ONE call through libznn_cuda.so, and copies the result back.

The names and argument meaning mirror the reference's operator arms
(src/autodiff.zig Op.forward / Op.backward), so parity tests read like the
reference's own tests.  Backward functions accumulate into the gradient arrays
passed in (a None gradient = requires_grad false), as the reference does.
"""
import ctypes as C

import numpy as np

from ._lib import lib

ROW_MAJOR, NO_TRANS, TRANS = 101, 111, 112

_inited = {}


def init(device=0):
    """Select the device for this thread and create the per-device state."""
    lib().call("znn_init", device)
    _inited[device] = True


def _ensure():
    if not _inited:
        init(0)


class DevBuf:
    """A device allocation owned by Python (znn_malloc / znn_free)."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        lib().call("znn_malloc", C.byref(p), self.nbytes)
        self.ptr = p.value if self.nbytes else None

    @classmethod
    def from_host(cls, arr):
        arr = np.ascontiguousarray(arr)
        b = cls(arr.nbytes)
        if arr.nbytes:
            lib().call("znn_memcpy_h2d", b.ptr, arr.ctypes.data, arr.nbytes)
            lib().call("znn_sync")  # arr may be a temporary
        return b

    def to_host(self, shape, dtype=np.float32):
        out = np.empty(shape, dtype)
        if out.nbytes:
            lib().call("znn_memcpy_d2h", out.ctypes.data, self.ptr, out.nbytes)
        return out

    def into(self, arr):
        if arr.nbytes:
            lib().call("znn_memcpy_d2h", arr.ctypes.data, self.ptr, arr.nbytes)

    def free(self):
        if self.ptr:
            lib().call("znn_free", self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _up(a, dtype=np.float32):
    if a is None:
        return None
    return DevBuf.from_host(np.ascontiguousarray(a, dtype=dtype))


def _ptr(b):
    return b.ptr if b is not None else None


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def check_device_status():
    st = C.c_int(0)
    lib().call("znn_device_status", C.byref(st), 1)
    if st.value:
        raise RuntimeError(f"device status word = {st.value}: a bounded device-side wait expired")


def set_gemm_path(path):
    lib().call("znn_gemm_set_path", int(path))


def last_gemm_path():
    return lib().dll.znn_gemm_last_path()


def sgemm(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, Cm, ldc):
    """cblas_sgemm on host arrays (row-major). Cm is updated in place and returned."""
    _ensure()
    dA, dB, dC = _up(A), _up(B), _up(Cm)
    lib().call("znn_sgemm", ROW_MAJOR, ta, tb, M, N, K, alpha, dA.ptr, lda, dB.ptr, ldb, beta, dC.ptr, ldc)
    check_device_status()
    dC.into(Cm)
    return Cm


def sgemm_host(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, Cm, ldc, panels=0):
    """cblas_sgemm straight on host arrays: ONE call, the shim pipelines copies and panels itself."""
    _ensure()
    for a in (A, B, Cm):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    lib().call("znn_sgemm_host", ROW_MAJOR, ta, tb, M, N, K, alpha, A.ctypes.data, lda, B.ctypes.data, ldb, beta,
               Cm.ctypes.data, ldc, panels)
    check_device_status()
    return Cm


def matmul_host_fwd_bwd(A, B, dC=None, want_dA=True, want_dB=True, dA=None, dB=None, panels=0):
    """MatMul forward + backward on host arrays in one pipelined call.  With dA/dB given the
    gradients are accumulated into them (the reference's +=); otherwise fresh arrays are returned."""
    _ensure()
    A, B = _f(A), _f(B)
    M, K = A.shape
    N = B.shape[1]
    Cm = np.empty((M, N), np.float32)
    acc = int(dA is not None or dB is not None)
    if dC is not None:
        dC = _f(dC)
        if not acc:
            dA = np.empty((M, K), np.float32) if want_dA else None
            dB = np.empty((K, N), np.float32) if want_dB else None
    p = lambda a: a.ctypes.data if a is not None else None
    lib().call("znn_matmul_host_fwd_bwd", p(A), p(B), p(dC), p(Cm), p(dA), p(dB), M, K, N, acc, panels)
    check_device_status()
    return Cm, dA, dB


def sgemm_batched(ta, tb, M, N, K, alpha, A, lda, sa, B, ldb, sb, beta, Cm, ldc, sc, batch):
    _ensure()
    dA, dB, dC = _up(A), _up(B), _up(Cm)
    lib().call("znn_sgemm_batched_strided", ta, tb, M, N, K, alpha, dA.ptr, lda, sa, dB.ptr, ldb, sb, beta,
               dC.ptr, ldc, sc, batch)
    check_device_status()
    dC.into(Cm)
    return Cm


def sgemm_grouped(ta, tb, M, N, K, alpha, A, lda, sa, B, ldb, sb, beta, Cm, ldc, sc, batch, bias=None, sbias=0, kcat=0):
    """znn_sgemm_grouped on host arrays (flat float32 buffers holding the slices at the given strides)."""
    _ensure()
    dA, dB, dC, db = _up(A), _up(B), _up(Cm), _up(bias)
    lib().call("znn_sgemm_grouped", ta, tb, M, N, K, alpha, dA.ptr, lda, sa, dB.ptr, ldb, sb, beta, dC.ptr, ldc, sc, batch,
               _ptr(db), sbias, kcat)
    check_device_status()
    dC.into(Cm)
    return Cm


TRI_NONE, TRI_C_LOWER, TRI_A_LOWER, TRI_A_UPPER, TRI_B_LOWER = 0, 1, 2, 3, 4


def sgemm_batched_tri(ta, tb, M, N, K, alpha, A, lda, sa, B, ldb, sb, beta, Cm, ldc, sc, batch, tri):
    """znn_sgemm_batched_strided_tri on host arrays (triangular-structure hint, see include/znn_cuda.h)."""
    _ensure()
    dA, dB, dC = _up(A), _up(B), _up(Cm)
    lib().call("znn_sgemm_batched_strided_tri", ta, tb, M, N, K, alpha, dA.ptr, lda, sa, dB.ptr, ldb, sb, beta,
               dC.ptr, ldc, sc, batch, tri)
    check_device_status()
    dC.into(Cm)
    return Cm


def matmul_fwd(A, B):
    A, B = _f(A), _f(B)
    M, K = A.shape
    N = B.shape[1]
    out = np.zeros((M, N), np.float32)
    return sgemm(NO_TRANS, NO_TRANS, M, N, K, 1.0, A, K, B, N, 0.0, out, N)


def linear_fwd(X, W, bias):
    """Linear.forward as one fused call: Y = X.W + bias (the bias is added in the GEMM epilogue)."""
    _ensure()
    X, W, bias = _f(X), _f(W), _f(bias).reshape(-1)
    M, K = X.shape
    N = W.shape[1]
    dX, dW, db = _up(X), _up(W), _up(bias)
    out = DevBuf(M * N * 4)
    lib().call("znn_linear_fwd", dX.ptr, dW.ptr, db.ptr, out.ptr, M, K, N)
    check_device_status()
    return out.to_host((M, N))


def linear_fwd_ex(X, W, bias, act=0, residual=None, want_pre=False):
    """Linear with the activation (1 ReLU, 2 GELU) and / or the residual add in the GEMM epilogue; returns Y (and the
    pre-activation h when asked)."""
    _ensure()
    X, W, bias = _f(X), _f(W), _f(bias).reshape(-1)
    M, K = X.shape
    N = W.shape[1]
    dX, dW, db = _up(X), _up(W), _up(bias)
    dr = _up(_f(residual)) if residual is not None else None
    out = DevBuf(M * N * 4)
    pre = DevBuf(M * N * 4) if want_pre else None
    lib().call("znn_linear_fwd_ex", dX.ptr, dW.ptr, db.ptr, out.ptr, pre.ptr if pre else None, dr.ptr if dr else None,
               M, K, N, act)
    check_device_status()
    if want_pre:
        return out.to_host((M, N)), pre.to_host((M, N))
    return out.to_host((M, N))


def linear_bwd_ex(X, W, dY, dX, dW, dbias, x_pre, x_act, dx_fresh):
    """Backward of Linear whose input is act(x_pre): dX receives the gradient with respect to x_pre."""
    _ensure()
    M, K = X.shape
    N = W.shape[1]
    x, w, dy, dx, dw, db, xp = _up(_f(X)), _up(_f(W)), _up(_f(dY)), _up(dX), _up(dW), _up(dbias), _up(_f(x_pre))
    lib().call("znn_linear_bwd_ex", x.ptr, w.ptr, dy.ptr, _ptr(dx), _ptr(dw), _ptr(db), M, K, N, xp.ptr, x_act, dx_fresh)
    check_device_status()
    for host, dev in ((dX, dx), (dW, dw), (dbias, db)):
        if host is not None:
            dev.into(host)


def matmul_bwd(A, B, dC, dA=None, dB=None):
    M, K = A.shape
    N = B.shape[1]
    if dA is not None:
        sgemm(NO_TRANS, TRANS, M, K, N, 1.0, dC, N, B, N, 1.0, dA, K)
    if dB is not None:
        sgemm(TRANS, NO_TRANS, K, N, M, 1.0, A, K, dC, N, 1.0, dB, N)


def batch_matmul_fwd(A, B):
    A, B = _f(A), _f(B)
    M, K = A.shape[-2:]
    N = B.shape[-1]
    nb = int(np.prod(A.shape[:-2]))
    out = np.zeros(A.shape[:-2] + (M, N), np.float32)
    return sgemm_batched(NO_TRANS, NO_TRANS, M, N, K, 1.0, A, K, M * K, B, N, K * N, 0.0, out, N, M * N, nb)


def batch_matmul_bwd(A, B, dC, dA=None, dB=None):
    M, K = A.shape[-2:]
    N = B.shape[-1]
    nb = int(np.prod(A.shape[:-2]))
    if dA is not None:
        sgemm_batched(NO_TRANS, TRANS, M, K, N, 1.0, dC, N, M * N, B, N, K * N, 1.0, dA, K, M * K, nb)
    if dB is not None:
        sgemm_batched(TRANS, NO_TRANS, K, N, M, 1.0, A, K, M * K, dC, N, M * N, 1.0, dB, N, K * N, nb)


def add_bias_fwd(A, bias):
    _ensure()
    A, bias = _f(A), _f(bias)
    dA, db = _up(A), _up(bias)
    dC = DevBuf(A.nbytes)
    lib().call("znn_add_bias_fwd", dA.ptr, db.ptr, dC.ptr, A.shape[0], A.shape[1])
    return dC.to_host(A.shape)


def add_bias_bwd(dC, dA=None, dbias=None):
    _ensure()
    d_dC, d_dA, d_db = _up(dC), _up(dA), _up(dbias)
    lib().call("znn_add_bias_bwd", d_dC.ptr, _ptr(d_dA), _ptr(d_db), dC.shape[0], dC.shape[1])
    if dA is not None:
        d_dA.into(dA)
    if dbias is not None:
        d_db.into(dbias)


def _unary_fwd(name, A):
    _ensure()
    A = _f(A)
    dA = _up(A)
    dC = DevBuf(A.nbytes)
    lib().call(name, dA.ptr, dC.ptr, A.size)
    return dC.to_host(A.shape)


def _unary_bwd(name, A, dC, dA):
    _ensure()
    a, g, o = _up(A), _up(dC), _up(dA)
    lib().call(name, a.ptr, g.ptr, o.ptr, A.size)
    o.into(dA)


def relu_fwd(A):
    return _unary_fwd("znn_relu_fwd", A)


def gelu_fwd(A):
    return _unary_fwd("znn_gelu_fwd", A)


def relu_bwd(A, dC, dA):
    _unary_bwd("znn_relu_bwd", A, dC, dA)


def gelu_bwd(A, dC, dA):
    _unary_bwd("znn_gelu_bwd", A, dC, dA)


def gelu_bwd_set(A, dC, dA):
    """Stores the gradient into dA (whatever it held) instead of adding it."""
    _unary_bwd("znn_gelu_bwd_set", A, dC, dA)


def softmax_xent_fwd(logits, targets, u8=False):
    _ensure()
    logits = _f(logits)
    M, N = logits.shape
    dl = _up(logits)
    dt = _up(targets, np.uint8 if u8 else np.int32)
    dp, dloss = DevBuf(logits.nbytes), DevBuf(4)
    lib().call("znn_softmax_xent_fwd_u8" if u8 else "znn_softmax_xent_fwd", dl.ptr, dt.ptr, dp.ptr, dloss.ptr, M, N)
    return dloss.to_host((1,)), dp.to_host((M, N))


def softmax_xent_bwd(probs, targets, dlogits, u8=False):
    _ensure()
    M, N = probs.shape
    dp, dt, dg = _up(probs), _up(targets, np.uint8 if u8 else np.int32), _up(dlogits)
    lib().call("znn_softmax_xent_bwd_u8" if u8 else "znn_softmax_xent_bwd", dp.ptr, dt.ptr, dg.ptr, M, N)
    dg.into(dlogits)


def softmax_fwd(A):
    _ensure()
    A = _f(A)
    D = A.shape[-1]
    dA, dC = _up(A), DevBuf(A.nbytes)
    lib().call("znn_softmax_fwd", dA.ptr, dC.ptr, A.size // D, D)
    return dC.to_host(A.shape)


def softmax_bwd(Y, dY, dA):
    _ensure()
    D = Y.shape[-1]
    y, g, o = _up(Y), _up(dY), _up(dA)
    lib().call("znn_softmax_bwd", y.ptr, g.ptr, o.ptr, Y.size // D, D)
    o.into(dA)


def causal_softmax_fwd(S, scale):
    _ensure()
    S = _f(S)
    T = S.shape[-1]
    dS, dP = _up(S), DevBuf(S.nbytes)
    lib().call("znn_causal_softmax_fwd", dS.ptr, scale, dP.ptr, S.size // (T * T), T)
    return dP.to_host(S.shape)


def causal_softmax_bwd(P, dP, scale, dS):
    _ensure()
    T = P.shape[-1]
    p, g, o = _up(P), _up(dP), _up(dS)
    lib().call("znn_causal_softmax_bwd", p.ptr, g.ptr, scale, o.ptr, P.size // (T * T), T)
    o.into(dS)


def causal_softmax_bwd_set(P, dP, scale, dS):
    """Stores the gradient into dS (zeros above the diagonal) instead of adding it."""
    _ensure()
    T = P.shape[-1]
    p, g, o = _up(P), _up(dP), _up(dS)
    lib().call("znn_causal_softmax_bwd_set", p.ptr, g.ptr, scale, o.ptr, P.size // (T * T), T)
    o.into(dS)


def adam_step(w, g, m, v, lr, beta1, beta2, eps, t, grad_scale=1.0):
    """In place on the host arrays w, m, v."""
    _ensure()
    dw, dg, dm, dv = _up(w), _up(g), _up(m), _up(v)
    lib().call("znn_adam_step", dw.ptr, dg.ptr, dm.ptr, dv.ptr, lr, beta1, beta2, eps, t, grad_scale, w.size)
    dw.into(w)
    dm.into(m)
    dv.into(v)


def attn_dscores(dO, V, P, scale):
    """dS = scale * P o (dO.V^T - D), D = rowsum(dO o O) with O = P.V (computed here on the host in fp64 -> fp32);
    returns dS (tiles entirely above the diagonal keep the zeros they are given here)."""
    _ensure()
    dO, V, P = _f(dO), _f(V), _f(P)
    ns, T, hs = dO.shape
    O = (P.astype(np.float64) @ V.astype(np.float64))
    D = np.ascontiguousarray((dO.astype(np.float64) * O).sum(-1).astype(np.float32))
    d_do, d_v, d_p, d_d = _up(dO), _up(V), _up(P), _up(D)
    out = np.zeros((ns, T, T), np.float32)
    d_out = _up(out)
    lib().call("znn_attn_dscores", d_do.ptr, d_v.ptr, d_p.ptr, d_d.ptr, scale, d_out.ptr, T, hs, ns)
    check_device_status()
    d_out.into(out)
    return out


def _attn_layout(shape, layout):
    if layout == "bhtd":
        B, nh, T, hs = shape
        return B, nh, T, hs, hs, T * hs, nh * T * hs
    B, T, nh, hs = shape
    return B, nh, T, hs, nh * hs, hs, T * nh * hs


def attn_fwd(Q, K, V, scale, layout="bhtd"):
    """Fused causal attention forward.  layout 'bhtd': arrays are [B, nh, T, hs]; 'bthd': [B, T, nh, hs].
    Returns (O in the same layout, LSE [B*nh, T])."""
    _ensure()
    Q, K, V = _f(Q), _f(K), _f(V)
    B, nh, T, hs, ld, sh, sb = _attn_layout(Q.shape, layout)
    dQ_, dK_, dV_ = _up(Q), _up(K), _up(V)
    dO, dL = DevBuf(Q.nbytes), DevBuf(B * nh * T * 4)
    lib().call("znn_attn_fwd", dQ_.ptr, dK_.ptr, dV_.ptr, dO.ptr, dL.ptr, B, nh, T, hs, ld, sh, sb, scale)
    check_device_status()
    return dO.to_host(Q.shape), dL.to_host((B * nh, T))


def attn_bwd(Q, K, V, O, dO, LSE, scale, layout="bhtd", grads=None, want=(True, True, True)):
    """Fused causal attention backward: returns (dQ, dK, dV).  With grads = (dQ0, dK0, dV0) the results are added to
    them (the reference's +=)."""
    _ensure()
    Q, K, V, O, dO, LSE = _f(Q), _f(K), _f(V), _f(O), _f(dO), _f(LSE)
    B, nh, T, hs, ld, sh, sb = _attn_layout(Q.shape, layout)
    bufs = [_up(a) for a in (Q, K, V, O, dO, LSE)]
    outs = []
    for i, w in enumerate(want):
        if not w:
            outs.append(None)
        elif grads is not None:
            outs.append(_up(grads[i]))
        else:
            outs.append(DevBuf(Q.nbytes))
    lib().call("znn_attn_bwd", *[b.ptr for b in bufs], *[_ptr(o) for o in outs], B, nh, T, hs, ld, sh, sb, scale,
               1 if grads is not None else 0)
    check_device_status()
    return tuple(o.to_host(Q.shape) if o is not None else None for o in outs)


def rowdot(A, B):
    _ensure()
    A, B = _f(A), _f(B)
    rows, D = A.shape
    a, b, o = _up(A), _up(B), DevBuf(rows * 4)
    lib().call("znn_rowdot", a.ptr, b.ptr, o.ptr, rows, D)
    return o.to_host((rows,))


def rmsnorm_fwd(X, G, eps):
    _ensure()
    X, G = _f(X), _f(G)
    D = X.shape[-1]
    x, g, y = _up(X), _up(G), DevBuf(X.nbytes)
    lib().call("znn_rmsnorm_fwd", x.ptr, g.ptr, eps, y.ptr, X.size // D, D)
    return y.to_host(X.shape)


def rmsnorm_bwd(X, G, dY, eps, dX=None, dG=None):
    _ensure()
    D = X.shape[-1]
    x, g, dy, dx, dg = _up(X), _up(G), _up(dY), _up(dX), _up(dG)
    lib().call("znn_rmsnorm_bwd", x.ptr, g.ptr, dy.ptr, eps, _ptr(dx), _ptr(dg), X.size // D, D)
    if dX is not None:
        dx.into(dX)
    if dG is not None:
        dg.into(dG)


def layernorm_fwd(X, G, Bt, eps):
    _ensure()
    X, G, Bt = _f(X), _f(G), _f(Bt)
    D = X.shape[-1]
    x, g, b, y = _up(X), _up(G), _up(Bt), DevBuf(X.nbytes)
    lib().call("znn_layernorm_fwd", x.ptr, g.ptr, b.ptr, eps, y.ptr, X.size // D, D)
    return y.to_host(X.shape)


def layernorm_bwd(X, G, dY, eps, dX=None, dG=None, dB=None):
    _ensure()
    D = X.shape[-1]
    x, g, dy, dx, dg, db = _up(X), _up(G), _up(dY), _up(dX), _up(dG), _up(dB)
    lib().call("znn_layernorm_bwd", x.ptr, g.ptr, dy.ptr, eps, _ptr(dx), _ptr(dg), _ptr(db), X.size // D, D)
    for host, dev in ((dX, dx), (dG, dg), (dB, db)):
        if host is not None:
            dev.into(host)


def conv2d_fwd(X, W, bias=None, pad=0):
    _ensure()
    X, W = _f(X), _f(W)
    N, Ci, H, Wd = X.shape
    Co, _, KH, KW = W.shape
    Ho, Wo = H + 2 * pad - KH + 1, Wd + 2 * pad - KW + 1
    x, w, b = _up(X), _up(W), _up(bias)
    y = DevBuf(N * Co * Ho * Wo * 4)
    lib().call("znn_conv2d_fwd", x.ptr, w.ptr, _ptr(b), y.ptr, N, Ci, H, Wd, Co, KH, KW, pad)
    return y.to_host((N, Co, Ho, Wo))


def conv2d_bwd(X, W, dY, dX=None, dW=None, dbias=None, pad=0):
    _ensure()
    N, Ci, H, Wd = X.shape
    Co, _, KH, KW = W.shape
    x, w, dy, dx, dw, db = _up(X), _up(W), _up(dY), _up(dX), _up(dW), _up(dbias)
    lib().call("znn_conv2d_bwd", x.ptr, w.ptr, dy.ptr, _ptr(dx), _ptr(dw), _ptr(db), N, Ci, H, Wd, Co, KH, KW, pad)
    for host, dev in ((dX, dx), (dW, dw), (dbias, db)):
        if host is not None:
            dev.into(host)


def maxpool2d_fwd(X, pool, stride, want_idx=False):
    _ensure()
    X = _f(X)
    N, Cc, H, W = X.shape
    Ho, Wo = H // stride, W // stride
    x = _up(X)
    y = DevBuf(N * Cc * Ho * Wo * 4)
    idx = DevBuf(N * Cc * Ho * Wo * 4) if want_idx else None
    lib().call("znn_maxpool2d_fwd", x.ptr, y.ptr, _ptr(idx), N, Cc, H, W, pool, stride)
    out = y.to_host((N, Cc, Ho, Wo))
    return (out, idx.to_host((N, Cc, Ho, Wo), np.int32)) if want_idx else out


def maxpool2d_bwd(X, dY, dX, pool, stride):
    _ensure()
    N, Cc, H, W = X.shape
    x, dy, dx = _up(X), _up(dY), _up(dX)
    lib().call("znn_maxpool2d_bwd", x.ptr, dy.ptr, dx.ptr, N, Cc, H, W, pool, stride)
    dx.into(dX)


def embedding_fwd(W, ids):
    _ensure()
    W, ids = _f(W), _f(ids)
    V, D = W.shape
    w, i = _up(W), _up(ids)
    y = DevBuf(ids.size * D * 4)
    lib().call("znn_embedding_fwd", w.ptr, i.ptr, y.ptr, ids.size, D, V)
    return y.to_host(ids.shape + (D,))


def embedding_bwd(ids, dY, dW):
    _ensure()
    ids = _f(ids)
    V, D = dW.shape
    i, dy, dw = _up(ids), _up(dY), _up(dW)
    lib().call("znn_embedding_bwd", i.ptr, dy.ptr, dw.ptr, ids.size, D, V)
    dw.into(dW)


def transpose_fwd(A, d0, d1):
    _ensure()
    A = _f(A)
    dims = np.array(A.shape, dtype=np.int64)
    oshape = list(A.shape)
    oshape[d0], oshape[d1] = oshape[d1], oshape[d0]
    a, c = _up(A), DevBuf(A.nbytes)
    lib().call("znn_transpose_fwd", a.ptr, c.ptr, dims.ctypes.data, A.ndim, d0, d1)
    return c.to_host(tuple(oshape))


def transpose_bwd(dC, dA, d0, d1):
    _ensure()
    dims = np.array(dA.shape, dtype=np.int64)
    g, o = _up(dC), _up(dA)
    lib().call("znn_transpose_bwd", g.ptr, o.ptr, dims.ctypes.data, dA.ndim, d0, d1)
    o.into(dA)


def add_fwd(A, B):
    _ensure()
    A, B = _f(A), _f(B)
    a, b, c = _up(A), _up(B), DevBuf(A.nbytes)
    lib().call("znn_add_fwd", a.ptr, b.ptr, c.ptr, A.size)
    return c.to_host(A.shape)


def accumulate(src, dst):
    _ensure()
    s, d = _up(src), _up(dst)
    lib().call("znn_accumulate", s.ptr, d.ptr, dst.size)
    d.into(dst)


def mul_scalar_fwd(A, v):
    _ensure()
    A = _f(A)
    a, c = _up(A), DevBuf(A.nbytes)
    lib().call("znn_mul_scalar_fwd", a.ptr, v, c.ptr, A.size)
    return c.to_host(A.shape)


def mul_scalar_bwd(dC, v, dA):
    _ensure()
    g, o = _up(dC), _up(dA)
    lib().call("znn_mul_scalar_bwd", g.ptr, v, o.ptr, dA.size)
    o.into(dA)


def argmax(A, dim):
    _ensure()
    A = _f(A)
    M, N = A.shape
    n_out = M if dim == 1 else N
    a, o = _up(A), DevBuf(n_out * 4)
    lib().call("znn_argmax", a.ptr, o.ptr, M, N, dim)
    return o.to_host((n_out,))


def sgd_step(w, g, v, lr, momentum, grad_scale=1.0):
    _ensure()
    dw, dg, dv = _up(w), _up(g), _up(v)
    lib().call("znn_sgd_step", dw.ptr, dg.ptr, _ptr(dv), lr, momentum, grad_scale, w.size)
    dw.into(w)
    if v is not None:
        dv.into(v)
