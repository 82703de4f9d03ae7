"""The batch-sharded path on CPU: two gloo ranks compute their shard's gradients (with the oracle,
there being no GPU here), all-reduce the fused dW||dB buffer, and must reproduce the single-process
full-batch result.  Mirrors the sharded configuration: per-sample seeds, contiguous batch slices."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import dp
from oracle import oracle

GLOBAL_BATCH, C, HW = 8, 8, 10


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _shard_grads(start, stop):
    x = dp.seeded_samples((C, HW, HW), 5000, start, stop).numpy()
    go = dp.seeded_samples((C, HW, HW), 7000, start, stop).numpy()
    gw = torch.Generator().manual_seed(4999)
    w = ((torch.rand(C, C, 3, 3, generator=gw) * 2 - 1) / (C * 9) ** 0.5).numpy()
    g = oracle.geometry(x.shape, C, (3, 3), padding=(1, 1))
    return oracle.dweight(g, x, go, f64=True), oracle.dbias(g, go, f64=True), w


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    start, stop = dp.shard_range(GLOBAL_BATCH, rank, world)
    dw, db, _ = _shard_grads(start, stop)
    rdw, rdb = dp.allreduce_grads(torch.from_numpy(dw), torch.from_numpy(db))
    np.save(os.path.join(out_dir, f"dw{rank}.npy"), rdw.numpy())
    np.save(os.path.join(out_dir, f"db{rank}.npy"), rdb.numpy())
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_full_batch_gradients(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    full_dw, full_db, _ = _shard_grads(0, GLOBAL_BATCH)
    for rank in range(world):
        dw = np.load(tmp_path / f"dw{rank}.npy")
        db = np.load(tmp_path / f"db{rank}.npy")
        assert oracle.rel_l2(dw, full_dw) < 1e-6
        assert oracle.rel_l2(db, full_db) < 1e-6


def test_shards_cover_the_global_batch_for_every_world_size():
    full = dp.seeded_samples((2, 3, 3), 5000, 0, 8)
    for world in (1, 2, 4, 8):
        parts = [dp.seeded_samples((2, 3, 3), 5000, *dp.shard_range(8, r, world)) for r in range(world)]
        assert torch.equal(torch.cat(parts), full)
    with pytest.raises(ValueError, match="evenly"):
        dp.shard_range(10, 0, 4)
    with pytest.raises(ValueError, match="invalid rank"):
        dp.shard_range(8, 2, 2)


def test_allreduce_is_identity_without_a_process_group():
    dw, db = torch.randn(4, 2, 3, 3), torch.randn(4)
    rdw, rdb = dp.allreduce_grads(dw, db)
    assert torch.equal(rdw, dw) and torch.equal(rdb, db)
