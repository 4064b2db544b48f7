"""Data-parallel training on 2 GPUs (one process per GPU, NCCL gradient all-reduce overlapped with
backward) against single-GPU training on the whole batch.  Skipped on boxes with one GPU."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CFG = {"vocab_size": 64, "block_size": 32, "n_embd": 64, "n_head": 4, "n_layer": 2}
DIMS = (64, 32, 64, 4, 2)
STEPS, GLOBAL_B, T = 4, 8, 32


def _batches():
    r = np.random.default_rng(77)
    for _ in range(STEPS):
        x = r.integers(0, 64, (GLOBAL_B, T)).astype(np.float32)
        t = np.concatenate([x[:, 1:], r.integers(0, 64, (GLOBAL_B, 1))], axis=1).astype(np.int32)
        yield x, t


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_dir, overlap):
    sys.path.insert(0, ROOT)
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    import ctypes as C
    import torch.distributed as dist
    from oracle import models
    from znn_b200._lib import lib
    from znn_b200.models import Model
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L = lib()
    L.call("znn_init", rank)
    uid = C.create_string_buffer(128)
    if rank == 0:
        L.call("znn_dp_unique_id", uid)
    box = [uid.raw]
    dist.broadcast_object_list(box, src=0)
    L.call("znn_dp_init", world, rank, box[0])
    m = Model("gpt", DIMS, arena_bytes=256 << 20)
    m.set_params(models.init_params("gpt", CFG, seed=6, scheme="n002"))
    m.set_option("lr", 0.05)
    m.set_option("momentum", 0.9)
    m.set_option("dp_overlap", overlap)
    m.set_option("dp_bucket_floats", 20000)          # several buckets even for this small model
    losses = []
    for x, t in _batches():
        lo, hi = rank * GLOBAL_B // world, (rank + 1) * GLOBAL_B // world
        losses.append(m.train_step(x[lo:hi], t[lo:hi], seq=T))
    P = m.get_params()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), losses=np.array(losses), **P)
    m.close()
    L.call("znn_dp_finalize")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("overlap", [1, 0])
def test_two_gpu_dp_matches_single_gpu(tmp_path, overlap):
    import ctypes as C
    import torch.multiprocessing as mp
    from oracle import models
    from znn_b200 import ops
    from znn_b200._lib import lib
    from znn_b200.models import Model
    n = C.c_int()
    lib().call("znn_device_count", C.byref(n))
    if n.value < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_rank_main, args=(2, _free_port(), str(tmp_path), overlap), nprocs=2, join=True)
    r0, r1 = (np.load(os.path.join(str(tmp_path), f"rank{i}.npz")) for i in (0, 1))
    ops.init(0)
    m = Model("gpt", DIMS, arena_bytes=256 << 20)
    P0 = models.init_params("gpt", CFG, seed=6, scheme="n002")
    m.set_params(P0)
    m.set_option("lr", 0.05)
    m.set_option("momentum", 0.9)
    for s, (x, t) in enumerate(_batches()):
        loss = m.train_step(x, t, seq=T)
        dp_loss = 0.5 * (r0["losses"][s] + r1["losses"][s])        # mean of the shard means
        assert abs(dp_loss - loss) <= 1e-4 * abs(loss), (s, dp_loss, loss)
    P = m.get_params()
    for k in P:
        np.testing.assert_array_equal(r0[k], r1[k])                # replicas stay identical
        scale = max(float(np.abs(P[k]).max()), 1e-3)
        assert float(np.abs(r0[k] - P[k]).max()) <= 1e-4 * scale, k
