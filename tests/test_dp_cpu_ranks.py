"""Data-parallel scheme on CPU ranks (gloo, world_size 2): each rank runs the ORACLE training step on
its shard of the batch, the parameter gradients are summed over ranks and the optimizer applies them
with grad_scale = 1/world -- the same recipe the CUDA path uses with NCCL.  The result must match one
process training on the whole batch (SoftmaxCrossEntropy backward scales by 1/M_local and ignores the
upstream gradient, src/autodiff.zig:758-774, so the scaling can only be applied to the reduced grads)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _trainer(models, kind, P0, cfg, adam):
    if adam:
        return models.OracleTrainer(kind, P0, cfg, lr=0.001, adam=adam)
    return models.OracleTrainer(kind, P0, cfg, lr=0.05, momentum=0.9)


def _rank_main(rank, world, port, kind, cfg, steps, out_dir, adam=None):
    sys.path.insert(0, ROOT)
    from oracle import models
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    P0 = models.init_params(kind, cfg, seed=5)
    tr = _trainer(models, kind, P0, cfg, adam)
    r = np.random.default_rng(17)                      # every rank draws the same global batches
    G = 8
    losses = []
    for _ in range(steps):
        x = (r.integers(0, 256, (G, 784)).astype(np.float32) / np.float32(255.0)).astype(np.float32)
        t = r.integers(0, 10, G).astype(np.int32)
        lo, hi = rank * G // world, (rank + 1) * G // world
        loss, _ = tr.loss_and_grads(x[lo:hi], t[lo:hi])
        flat = torch.from_numpy(np.concatenate([tr.grads[k].reshape(-1) for k in tr.P]))
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)    # the one exchange step
        off, red = 0, {}
        for k in tr.P:
            n = tr.P[k].size
            red[k] = flat[off:off + n].numpy().reshape(tr.P[k].shape)
            off += n
        tr.apply(red, grad_scale=1.0 / world)
        lt = torch.tensor([loss], dtype=torch.float64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        losses.append(float(lt.item()) / world)
    if rank == 0:
        np.savez(os.path.join(out_dir, "dp.npz"), losses=np.array(losses), **tr.P)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("kind,cfg,adam", [("mlp", (784, 32, 16, 10), None), ("cnn_ref", None, None),
                                           ("mlp", (784, 32, 16, 10), (0.9, 0.999, 1e-6))])
def test_two_cpu_ranks_match_single_process(tmp_path, kind, cfg, adam):
    sys.path.insert(0, ROOT)
    from oracle import models, zo
    zo.build()
    steps, world = 5, 2
    mp.spawn(_rank_main, args=(world, _free_port(), kind, cfg, steps, str(tmp_path), adam), nprocs=world, join=True)
    got = np.load(os.path.join(str(tmp_path), "dp.npz"))
    P0 = models.init_params(kind, cfg, seed=5)
    tr = _trainer(models, kind, P0, cfg, adam)
    r = np.random.default_rng(17)
    for s in range(steps):
        x = (r.integers(0, 256, (8, 784)).astype(np.float32) / np.float32(255.0)).astype(np.float32)
        t = r.integers(0, 10, 8).astype(np.int32)
        loss, _ = tr.step(x, t)
        assert abs(got["losses"][s] - loss) <= 1e-5 * abs(loss), (s, got["losses"][s], loss)
    for k in tr.P:
        scale = max(1e-30, float(np.abs(tr.P[k]).max()))
        assert float(np.abs(got[k] - tr.P[k]).max()) <= 1e-5 * scale, k
