"""ctypes binding of libznn_cuda.so (the C ABI declared in include/znn_cuda.h).

There is no fallback: if the shared object is missing or a call fails, an
exception is raised.
"""
import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libznn_cuda.so")
HEADER = os.path.join(os.path.dirname(HERE), "include", "znn_cuda.h")
HOST_HEADER = os.path.join(os.path.dirname(HERE), "include", "znn_host.h")
DEBUG_HEADER = os.path.join(os.path.dirname(HERE), "include", "znn_debug.h")
ALL_HEADERS = (HEADER, HOST_HEADER, DEBUG_HEADER)

_CTYPES = {
    "int": C.c_int, "float": C.c_float, "double": C.c_double, "size_t": C.c_size_t, "long long": C.c_longlong,
    "void*": C.c_void_p, "const void*": C.c_void_p, "void**": C.POINTER(C.c_void_p),
    "float*": C.c_void_p, "const float*": C.c_void_p, "int*": C.POINTER(C.c_int),
    "int32_t*": C.c_void_p, "const int32_t*": C.c_void_p, "const uint8_t*": C.c_void_p,
    "const int64_t*": C.c_void_p, "char*": C.c_char_p, "const char*": C.c_char_p, "long long*": C.POINTER(C.c_longlong),
    "double*": C.POINTER(C.c_double), "const double*": C.c_void_p, "const long long*": C.c_void_p,
    "const int*": C.c_void_p, "znn_graph*": C.c_void_p, "znn_model*": C.c_void_p,
    "znn_graph**": C.POINTER(C.c_void_p), "znn_model**": C.POINTER(C.c_void_p),
    "uint8_t*": C.c_void_p, "float**": C.POINTER(C.c_void_p), "uint8_t**": C.POINTER(C.c_void_p),
    "unsigned*": C.POINTER(C.c_uint), "size_t*": C.POINTER(C.c_size_t),
    "znn_loader*": C.c_void_p, "znn_loader**": C.POINTER(C.c_void_p),
    "unsigned long long": C.c_ulonglong, "unsigned long long*": C.POINTER(C.c_ulonglong),
    "znn_arena*": C.c_void_p, "znn_arena**": C.POINTER(C.c_void_p),
    "znn_param_slab*": C.c_void_p, "znn_param_slab**": C.POINTER(C.c_void_p),
    "const size_t*": C.c_void_p, "const float**": C.c_void_p, "unsigned": C.c_uint,
    "znn_debug_allreduce_fn": C.c_void_p,
}


class ZnnError(RuntimeError):
    def __init__(self, code, text, fn):
        super().__init__(f"{fn} failed with code {code}: {text}")
        self.code = code


def declared_functions(header=HEADER):
    """[(name, [ctype strings])] for every `int znn_*(...)` prototype in the header."""
    src = open(header).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    out = []
    for m in re.finditer(r"\bint\s+(znn_\w+)\s*\(([^)]*)\)\s*;", src):
        name, args = m.group(1), m.group(2).strip()
        types = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                a = re.sub(r"\s*\b\w+$", "", a) if not a.endswith("*") else a   # drop the parameter name
                a = re.sub(r"\s*\*\s*", "*", a).strip()
                types.append(a)
        out.append((name, types))
    return out


def all_declared_functions():
    out = []
    for h in ALL_HEADERS:
        out += declared_functions(h)
    return out


class _Lib:
    def __init__(self):
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m znn_b200.build` (nvcc, sm_100a). "
                "There is no CPU or PyTorch fallback.")
        self.dll = C.CDLL(LIB_PATH)
        for name, types in all_declared_functions():
            fn = getattr(self.dll, name)
            fn.restype = C.c_int
            fn.argtypes = [_CTYPES[t] for t in types]

    def last_error(self):
        buf = C.create_string_buffer(512)
        self.dll.znn_last_error(buf, 512)
        return buf.value.decode(errors="replace")

    def call(self, name, *args):
        rc = getattr(self.dll, name)(*args)
        if rc != 0:
            raise ZnnError(rc, self.last_error(), name)
        return rc


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = _Lib()
    return _lib
