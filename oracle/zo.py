"""ctypes/numpy front end of the CPU oracle (libznn_oracle.so).

TEST INFRASTRUCTURE ONLY: tests, the smoke check and the bench's CPU-baseline
leg use this as the checker.  Product code never imports it.

Every function takes and returns contiguous float32 numpy arrays and forwards
to the C restatement in znn_oracle.c, which cites the reference loop it follows.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libznn_oracle.so")

ROW_MAJOR, NO_TRANS, TRANS = 101, 111, 112


def build(force=False):
    """Compile the C restatement with the Makefile next to this file."""
    src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("znn_oracle.c", "znn_oracle.h"))
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < src_m:
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


_SGEMM_T = C.CFUNCTYPE(None, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float,
                       C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_int)


def find_host_cblas():
    """Locate a host CBLAS sgemm with the LP64 C ABI of src/cblas.zig:17-34.

    Returns (function pointer as int, description) or (None, reason).  Looks for
    a system OpenBLAS first, then the OpenBLAS that scipy bundles.
    """
    import glob
    cands = []
    for pat in ("/usr/lib/x86_64-linux-gnu/libopenblas.so*", "/usr/lib/x86_64-linux-gnu/libcblas.so*"):
        cands += [(p, "cblas_sgemm") for p in sorted(glob.glob(pat))]
    try:
        import scipy
        base = os.path.join(os.path.dirname(os.path.dirname(scipy.__file__)), "scipy.libs")
        cands += [(p, "scipy_cblas_sgemm") for p in sorted(glob.glob(os.path.join(base, "libscipy_openblas-*.so")))]
    except Exception:
        pass
    for path, sym in cands:
        try:
            h = C.CDLL(path)
            fn = getattr(h, sym)
            nthreads = None
            for tsym in ("scipy_openblas_get_num_threads", "openblas_get_num_threads"):
                if hasattr(h, tsym):
                    nthreads = getattr(h, tsym)()
                    break
            return C.cast(fn, C.c_void_p).value, {"path": path, "symbol": sym, "threads": nthreads, "handle": h}
        except (OSError, AttributeError):
            continue
    return None, {"reason": "no LP64 cblas_sgemm found"}


def bind_sgemm(ptr):
    """ptr=None -> in-tree fallback loops (Linux behaviour); else a host CBLAS."""
    lib().zo_bind_sgemm(C.c_void_p(ptr))


def sgemm(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, Cm, ldc, naive=False):
    fn = lib().zo_sgemm_naive if naive else lib().zo_sgemm
    fn(C.c_int(ROW_MAJOR), C.c_int(ta), C.c_int(tb), C.c_int(M), C.c_int(N), C.c_int(K), C.c_float(alpha),
       _p(A), C.c_int(lda), _p(B), C.c_int(ldb), C.c_float(beta), _p(Cm), C.c_int(ldc))
    return Cm


def sgemm_f64(ta, tb, M, N, K, A, lda, B, ldb):
    out = np.zeros((M, N), dtype=np.float64)
    lib().zo_sgemm_f64(C.c_int(ta), C.c_int(tb), C.c_int(M), C.c_int(N), C.c_int(K), _p(A), C.c_int(lda),
                       _p(B), C.c_int(ldb), _p(out), C.c_int(N))
    return out


def matmul_fwd(A, B):
    A, B = _f(A), _f(B)
    M, K = A.shape
    N = B.shape[1]
    out = np.empty((M, N), np.float32)
    lib().zo_matmul_fwd(_p(A), _p(B), _p(out), C.c_int(M), C.c_int(K), C.c_int(N))
    return out


def matmul_bwd(A, B, dC, dA=None, dB=None):
    """Accumulates into dA / dB in place (either may be None)."""
    M, K = A.shape
    N = B.shape[1]
    lib().zo_matmul_bwd(_p(A), _p(B), _p(dC), _p(dA), _p(dB), C.c_int(M), C.c_int(K), C.c_int(N))


def batch_matmul_fwd(A, B):
    A, B = _f(A), _f(B)
    M, K = A.shape[-2:]
    N = B.shape[-1]
    nb = int(np.prod(A.shape[:-2]))
    out = np.empty(A.shape[:-2] + (M, N), np.float32)
    lib().zo_batch_matmul_fwd(_p(A), _p(B), _p(out), C.c_int(nb), C.c_int(M), C.c_int(K), C.c_int(N))
    return out


def batch_matmul_bwd(A, B, dC, dA=None, dB=None):
    M, K = A.shape[-2:]
    N = B.shape[-1]
    nb = int(np.prod(A.shape[:-2]))
    lib().zo_batch_matmul_bwd(_p(A), _p(B), _p(dC), _p(dA), _p(dB), C.c_int(nb), C.c_int(M), C.c_int(K), C.c_int(N))


def add_bias_fwd(A, bias):
    A, bias = _f(A), _f(bias)
    out = np.empty_like(A)
    lib().zo_add_bias_fwd(_p(A), _p(bias), _p(out), C.c_int(A.shape[0]), C.c_int(A.shape[1]))
    return out


def add_bias_bwd(dC, dA=None, dbias=None):
    lib().zo_add_bias_bwd(_p(dC), _p(dA), _p(dbias), C.c_int(dC.shape[0]), C.c_int(dC.shape[1]))


def _unary(name, A):
    A = _f(A)
    out = np.empty_like(A)
    getattr(lib(), name)(_p(A), _p(out), C.c_size_t(A.size))
    return out


def relu_fwd(A):
    return _unary("zo_relu_fwd", A)


def gelu_fwd(A):
    return _unary("zo_gelu_fwd", A)


def relu_bwd(A, dC, dA):
    lib().zo_relu_bwd(_p(A), _p(dC), _p(dA), C.c_size_t(A.size))


def gelu_bwd(A, dC, dA):
    lib().zo_gelu_bwd(_p(A), _p(dC), _p(dA), C.c_size_t(A.size))


def softmax_xent_fwd(logits, targets):
    logits = _f(logits)
    t = np.ascontiguousarray(targets, dtype=np.int32)
    M, N = logits.shape
    probs = np.empty_like(logits)
    loss = np.zeros(1, np.float32)
    lib().zo_softmax_xent_fwd(_p(logits), _p(t), _p(probs), _p(loss), C.c_int(M), C.c_int(N))
    return loss, probs


def softmax_xent_bwd(probs, targets, dlogits):
    t = np.ascontiguousarray(targets, dtype=np.int32)
    M, N = probs.shape
    lib().zo_softmax_xent_bwd(_p(probs), _p(t), _p(dlogits), C.c_int(M), C.c_int(N))


def softmax_fwd(A):
    A = _f(A)
    D = A.shape[-1]
    out = np.empty_like(A)
    lib().zo_softmax_fwd(_p(A), _p(out), C.c_size_t(A.size // D), C.c_int(D))
    return out


def softmax_bwd(Y, dY, dA):
    D = Y.shape[-1]
    lib().zo_softmax_bwd(_p(Y), _p(dY), _p(dA), C.c_size_t(Y.size // D), C.c_int(D))


def causal_softmax_fwd(S, scale):
    S = _f(S)
    T = S.shape[-1]
    out = np.empty_like(S)
    lib().zo_causal_softmax_fwd(_p(S), C.c_float(scale), _p(out), C.c_int(S.size // (T * T)), C.c_int(T))
    return out


def causal_softmax_bwd(P, dP, scale, dS):
    T = P.shape[-1]
    lib().zo_causal_softmax_bwd(_p(P), _p(dP), C.c_float(scale), _p(dS), C.c_int(P.size // (T * T)), C.c_int(T))


def rmsnorm_fwd(X, G, eps):
    X, G = _f(X), _f(G)
    D = X.shape[-1]
    out = np.empty_like(X)
    lib().zo_rmsnorm_fwd(_p(X), _p(G), C.c_float(eps), _p(out), C.c_size_t(X.size // D), C.c_int(D))
    return out


def rmsnorm_bwd(X, G, dY, eps, dX=None, dG=None):
    D = X.shape[-1]
    lib().zo_rmsnorm_bwd(_p(X), _p(G), _p(dY), C.c_float(eps), _p(dX), _p(dG), C.c_size_t(X.size // D), C.c_int(D))


def layernorm_fwd(X, G, Bt, eps):
    X, G, Bt = _f(X), _f(G), _f(Bt)
    D = X.shape[-1]
    out = np.empty_like(X)
    lib().zo_layernorm_fwd(_p(X), _p(G), _p(Bt), C.c_float(eps), _p(out), C.c_size_t(X.size // D), C.c_int(D))
    return out


def layernorm_bwd(X, G, dY, eps, dX=None, dG=None, dB=None):
    D = X.shape[-1]
    lib().zo_layernorm_bwd(_p(X), _p(G), _p(dY), C.c_float(eps), _p(dX), _p(dG), _p(dB),
                           C.c_size_t(X.size // D), C.c_int(D))


def conv2d_fwd(X, W, bias=None, pad=0):
    X, W = _f(X), _f(W)
    N, Ci, H, Wd = X.shape
    Co, _, KH, KW = W.shape
    Ho, Wo = H + 2 * pad - KH + 1, Wd + 2 * pad - KW + 1
    out = np.empty((N, Co, Ho, Wo), np.float32)
    b = _f(bias) if bias is not None else None
    lib().zo_conv2d_fwd(_p(X), _p(W), _p(b), _p(out), *(C.c_int(v) for v in (N, Ci, H, Wd, Co, KH, KW, pad)))
    return out


def conv2d_bwd(X, W, dY, dX=None, dW=None, dbias=None, pad=0):
    N, Ci, H, Wd = X.shape
    Co, _, KH, KW = W.shape
    lib().zo_conv2d_bwd(_p(X), _p(W), _p(dY), _p(dX), _p(dW), _p(dbias),
                        *(C.c_int(v) for v in (N, Ci, H, Wd, Co, KH, KW, pad)))


def maxpool2d_fwd(X, pool, stride, want_idx=False):
    X = _f(X)
    N, Cc, H, W = X.shape
    Ho, Wo = H // stride, W // stride
    out = np.empty((N, Cc, Ho, Wo), np.float32)
    idx = np.empty((N, Cc, Ho, Wo), np.int32) if want_idx else None
    lib().zo_maxpool2d_fwd(_p(X), _p(out), _p(idx), *(C.c_int(v) for v in (N, Cc, H, W, pool, stride)))
    return (out, idx) if want_idx else out


def maxpool2d_bwd(X, dY, dX, pool, stride):
    N, Cc, H, W = X.shape
    lib().zo_maxpool2d_bwd(_p(X), _p(dY), _p(dX), *(C.c_int(v) for v in (N, Cc, H, W, pool, stride)))


def embedding_fwd(W, ids):
    W, ids = _f(W), _f(ids)
    D = W.shape[1]
    out = np.empty(ids.shape + (D,), np.float32)
    lib().zo_embedding_fwd(_p(W), _p(ids), _p(out), C.c_size_t(ids.size), C.c_int(D))
    return out


def embedding_bwd(ids, dY, dW):
    ids = _f(ids)
    lib().zo_embedding_bwd(_p(ids), _p(dY), _p(dW), C.c_size_t(ids.size), C.c_int(dW.shape[1]))


def transpose_fwd(A, d0, d1):
    A = _f(A)
    dims = np.array(A.shape, dtype=np.int64)
    oshape = list(A.shape)
    oshape[d0], oshape[d1] = oshape[d1], oshape[d0]
    out = np.empty(oshape, np.float32)
    lib().zo_transpose_fwd(_p(A), _p(out), _p(dims), C.c_int(A.ndim), C.c_int(d0), C.c_int(d1))
    return out


def transpose_bwd(dC, dA, d0, d1):
    dims = np.array(dA.shape, dtype=np.int64)
    lib().zo_transpose_bwd(_p(dC), _p(dA), _p(dims), C.c_int(dA.ndim), C.c_int(d0), C.c_int(d1))


def add_fwd(A, B):
    A, B = _f(A), _f(B)
    out = np.empty_like(A)
    lib().zo_add_fwd(_p(A), _p(B), _p(out), C.c_size_t(A.size))
    return out


def accumulate(src, dst):
    lib().zo_accumulate(_p(src), _p(dst), C.c_size_t(src.size))


def mul_scalar_fwd(A, v):
    A = _f(A)
    out = np.empty_like(A)
    lib().zo_mul_scalar_fwd(_p(A), C.c_float(v), _p(out), C.c_size_t(A.size))
    return out


def mul_scalar_bwd(dC, v, dA):
    lib().zo_mul_scalar_bwd(_p(dC), C.c_float(v), _p(dA), C.c_size_t(dC.size))


def argmax(A, dim):
    A = _f(A)
    M, N = A.shape
    out = np.empty(M if dim == 1 else N, np.float32)
    lib().zo_argmax(_p(A), _p(out), C.c_int(M), C.c_int(N), C.c_int(dim))
    return out


def adam_step(w, g, m, v, lr, beta1, beta2, eps, t):
    """AdamOptimizer.step (src/optim.zig:133-151) in place; t = step count after the increment."""
    lib().zo_adam_step(_p(w), _p(g), _p(m), _p(v), C.c_float(lr), C.c_float(beta1), C.c_float(beta2), C.c_float(eps),
                       C.c_float(t), C.c_size_t(w.size))


def sgd_step(w, g, v, lr, momentum):
    lib().zo_sgd_step(_p(w), _p(g), _p(v), C.c_float(lr), C.c_float(momentum), C.c_size_t(w.size))
