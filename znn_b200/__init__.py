"""znn_b200: B200 (sm_100a) implementation of the dense-contraction hot path of
chen-gz/znn behind a C ABI (include/znn_cuda.h, libznn_cuda.so).

`znn_b200.ops` is the host-array front end used by the parity tests;
`znn_b200.build` compiles the shared object in-tree.  Nothing here falls back
to the CPU: without the CUDA library or a device every call raises.
"""
from ._lib import LIB_PATH, ZnnError, declared_functions, lib  # noqa: F401
