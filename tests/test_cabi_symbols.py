"""The C-ABI library loads and exports every symbol the headers under include/ declare."""
import ctypes
import os

import pytest

from znn_b200 import _lib


@pytest.fixture(scope="module")
def dll():
    if not os.path.exists(_lib.LIB_PATH):
        from znn_b200 import build
        build.build()
    return ctypes.CDLL(_lib.LIB_PATH)


def test_header_declares_the_hot_path():
    names = {n for n, _ in _lib.declared_functions()}
    for must in ("znn_sgemm", "znn_sgemm_batched_strided", "znn_add_bias_fwd", "znn_add_bias_bwd", "znn_relu_fwd",
                 "znn_gelu_bwd", "znn_softmax_xent_fwd", "znn_softmax_xent_bwd", "znn_causal_softmax_fwd",
                 "znn_rmsnorm_bwd", "znn_layernorm_fwd", "znn_conv2d_fwd", "znn_conv2d_bwd", "znn_maxpool2d_fwd",
                 "znn_embedding_bwd", "znn_transpose_fwd", "znn_argmax", "znn_sgd_step"):
        assert must in names


def test_every_declared_symbol_is_exported(dll):
    for header in _lib.ALL_HEADERS:
        decl = _lib.declared_functions(header)
        assert decl, header
        missing = [n for n, _ in decl if not hasattr(dll, n)]
        assert not missing, f"declared in {header} but not exported: {missing}"


def test_zig_binding_declares_every_function_of_the_cuda_header():
    """znn_b200/bindings/cuda.zig is the reference-side binding file: one `pub extern fn` per function of
    include/znn_cuda.h, with the same number of parameters."""
    import re
    here = os.path.dirname(os.path.abspath(_lib.__file__))
    zig = open(os.path.join(here, "bindings", "cuda.zig")).read()
    decls = {m.group(1): m.group(2) for m in re.finditer(r"pub extern fn (\w+)\(([^)]*)\)", zig)}
    header = [h for h in _lib.ALL_HEADERS if h.endswith("znn_cuda.h")][0]
    for name, types in _lib.declared_functions(header):
        assert name in decls, f"{name} missing from cuda.zig"
        nargs = len([a for a in decls[name].split(",") if a.strip()])
        assert nargs == len(types), f"{name}: {nargs} parameters in cuda.zig, {len(types)} in the header"


def test_ctypes_signatures_resolve():
    L = _lib.lib()
    for name, types in _lib.all_declared_functions():
        assert len(getattr(L.dll, name).argtypes) == len(types)


def test_no_silent_cpu_fallback(dll):
    """Without a CUDA device, initialisation must fail loudly (never fall back)."""
    n = ctypes.c_int(0)
    rc = dll.znn_device_count(ctypes.byref(n))
    if rc == 0 and n.value > 0:
        pytest.skip("a CUDA device is present")
    assert dll.znn_init(0) != 0
    buf = ctypes.create_string_buffer(256)
    dll.znn_last_error(buf, 256)
    assert b"no CUDA device" in buf.value
