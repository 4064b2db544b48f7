"""The data-parallel bucket schedule (which gradient bucket's all-reduce starts when, during the backward sweep) run
on the CPU against stand-in reductions: firing order, a late rank, and a rank whose reduction fails.  No GPU: the
schedule is host bookkeeping, and failures are made on the host."""
import ctypes as C
import threading
import time

import numpy as np

from znn_b200._lib import lib

FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_size_t, C.c_size_t)


def run_schedule(offsets, total, bucket_floats, uses, order, fn):
    n = len(offsets)
    off = (C.c_size_t * n)(*offsets)
    us = (C.c_int * n)(*uses)
    od = (C.c_int * max(1, len(order)))(*order)
    nb = C.c_int()
    cb = FN(fn)
    rc = lib().dll.znn_debug_bucket_schedule_run(off, n, C.c_size_t(total), C.c_size_t(bucket_floats), us, od, len(order),
                                                  C.cast(cb, C.c_void_p), None, C.byref(nb))
    return rc, nb.value


def test_buckets_fire_when_their_last_reader_has_run():
    # six parameters of 10 floats, buckets of >= 20 floats: {0,1} {2,3} {4,5}; the sweep finishes them back to front
    offsets, total = [0, 10, 20, 30, 40, 50], 60
    uses = [1, 2, 1, 1, 1, 0]                      # parameter 5 is never read this step
    fired = []
    rc, nb = run_schedule(offsets, total, 20, uses, [4, 3, 2, 1, 0, 1], lambda ctx, b, c: fired.append((b, c)) or 0)
    assert rc == 0 and nb == 3
    # bucket {4,5} completes with the first event (5 has no readers), {2,3} after events 3 and 2, {0,1} only once
    # parameter 1's second reader has run
    assert fired == [(40, 20), (20, 20), (0, 20)]
    # nothing complete during the sweep: finish() fires everything in slab order
    fired.clear()
    rc, _ = run_schedule(offsets, total, 20, [1] * 6, [0, 2, 4], lambda ctx, b, c: fired.append((b, c)) or 0)
    assert rc == 0 and fired == [(0, 20), (20, 20), (40, 20)]
    # one bucket for everything
    fired.clear()
    rc, nb = run_schedule(offsets, total, 1000, [1] * 6, [5, 4, 3, 2, 1, 0], lambda ctx, b, c: fired.append((b, c)) or 0)
    assert rc == 0 and nb == 1 and fired == [(0, 60)]


def test_a_failing_reduction_stops_the_step():
    fired = []

    def fn(ctx, b, c):
        fired.append(b)
        return -5 if b == 20 else 0

    rc, _ = run_schedule([0, 10, 20, 30, 40, 50], 60, 20, [1] * 6, [5, 4, 3, 2, 1, 0], fn)
    assert rc == -5
    assert fired == [40, 20]                       # the bucket after the failure is never started
    buf = C.create_string_buffer(256)
    lib().dll.znn_last_error(buf, 256)
    assert b"returned -5" in buf.value


class FakeWorld:
    """An all-reduce over `world` threads: every rank deposits its slice, a barrier, every rank reads the sum."""

    def __init__(self, world, timeout):
        self.world, self.timeout = world, timeout
        self.barrier = threading.Barrier(world)
        self.parts = [None] * world

    def allreduce(self, rank, grads, begin, count, delay=0.0, fail=False):
        if delay:
            time.sleep(delay)
        if fail:
            self.barrier.abort()                   # this rank leaves; the others learn of it at their barrier
            return -5
        try:
            self.parts[rank] = grads[begin:begin + count].copy()
            self.barrier.wait(self.timeout)
            total = np.sum(self.parts, axis=0, dtype=np.float32)
            self.barrier.wait(self.timeout)
            grads[begin:begin + count] = total
            return 0
        except threading.BrokenBarrierError:
            return -5


def run_ranks(world, delays, fail_rank=None, fail_bucket=None):
    offsets, total = [0, 16, 32, 48], 64
    order = [3, 2, 1, 0]
    rng = np.random.default_rng(0)
    grads = [rng.standard_normal(total).astype(np.float32) for _ in range(world)]
    want = np.sum(grads, axis=0, dtype=np.float32)
    fw = FakeWorld(world, timeout=5.0)
    rcs = [None] * world

    def rank_main(r):
        def fn(ctx, b, c):
            return fw.allreduce(r, grads[r], b, c, delay=delays[r], fail=(r == fail_rank and b == fail_bucket))
        rcs[r], _ = run_schedule(offsets, total, 32, [1] * 4, order, fn)

    th = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    t0 = time.time()
    for t in th:
        t.start()
    for t in th:
        t.join(30)
    assert not any(t.is_alive() for t in th), "a rank is stuck"
    return rcs, grads, want, time.time() - t0


def test_two_ranks_agree_even_when_one_is_late():
    rcs, grads, want, _ = run_ranks(2, delays=[0.0, 0.05])
    assert rcs == [0, 0]
    for g in grads:
        np.testing.assert_array_equal(g, want)


def test_an_erroring_rank_ends_every_rank_with_an_error_not_a_hang():
    rcs, _, _, elapsed = run_ranks(2, delays=[0.0, 0.0], fail_rank=1, fail_bucket=0)
    assert rcs[1] == -5                            # the failing rank reports its own error
    assert rcs[0] == -5                            # the healthy rank's reduction ends with an error as well
    assert elapsed < 20
