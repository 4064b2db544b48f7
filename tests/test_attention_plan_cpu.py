"""Host side of the fused attention kernels: how the work units are dealt to the CTA pairs (no GPU needed: the library
loads without a device and znn_debug_attn_plan is host arithmetic)."""
import ctypes as C
import os

import pytest

from znn_b200._lib import LIB_PATH


@pytest.fixture(scope="module")
def dll():
    if not os.path.exists(LIB_PATH):
        from znn_b200 import build
        build.build()
    d = C.CDLL(LIB_PATH)
    d.znn_debug_attn_plan.restype = C.c_int
    d.znn_debug_attn_plan.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    return d


def plan(dll, rows_first, nslices, T, pairs, table):
    units = (C.c_int * pairs)()
    blocks = (C.c_int * pairs)()
    rc = dll.znn_debug_attn_plan(rows_first, nslices, T, pairs, table, units, blocks)
    assert rc == 0      # the table form also checks that every unit appears exactly once
    return list(units), list(blocks)


@pytest.mark.parametrize("rows_first", [1, 0])
@pytest.mark.parametrize("nslices,T,pairs", [(96, 1024, 74), (256, 256, 74), (48, 520, 74), (7, 2048, 5), (3, 64, 74), (1, 4096, 74)])
def test_table_holds_every_unit_once_and_all_blocks(dll, rows_first, nslices, T, pairs):
    nrb, ncb = (T + 255) // 256, (T + 63) // 64
    # blocks of row block rb: forward / dQ walk the key blocks up to the diagonal, dK / dV from the diagonal to the end
    per_rb = [min(ncb, (min(T, 256 * rb + 256) + 63) // 64) if rows_first else ncb - 4 * rb for rb in range(nrb)]
    for table in (1, 0):
        units, blocks = plan(dll, rows_first, nslices, T, pairs, table)
        assert sum(units) == nslices * nrb
        assert sum(blocks) == nslices * sum(per_rb)


def test_table_balances_the_gpt_shape_better_than_round_dealing(dll):
    """96 slices x 1024 positions on 74 pairs: 384 units of 4, 8, 12 and 16 blocks, 51.9 blocks per pair on average."""
    for rows_first in (1, 0):
        _, by_rounds = plan(dll, rows_first, 96, 1024, 74, 0)
        units, by_table = plan(dll, rows_first, 96, 1024, 74, 1)
        assert max(by_rounds) == 56
        assert max(by_table) <= 53
        assert max(units) <= 7
