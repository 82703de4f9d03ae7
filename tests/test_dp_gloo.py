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
    # the gradients live in one fused buffer dW || dB, as the kernels write them: ONE collective, no copy
    flat, vdw, vdb = dp.fused_gradient_buffer(dw.shape, True, torch.empty(0))
    vdw.copy_(torch.from_numpy(dw))
    vdb.copy_(torch.from_numpy(db))
    rdw, rdb = dp.allreduce_grads(vdw, vdb)
    assert rdw.data_ptr() == flat.data_ptr() and rdb.data_ptr() == vdb.data_ptr()
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


def test_fused_buffer_views_and_the_packing_fallback_agree():
    dw, db = torch.randn(4, 2, 3, 3), torch.randn(4)
    flat, vdw, vdb = dp.fused_gradient_buffer(dw.shape, True, dw)
    assert flat.numel() == dw.numel() + db.numel() and vdw.shape == dw.shape and vdb.shape == db.shape
    vdw.copy_(dw)
    vdb.copy_(db)
    assert torch.equal(flat, torch.cat([dw.reshape(-1), db]))
    flat2, vdw2, none = dp.fused_gradient_buffer(dw.shape, False, dw)
    assert none is None and flat2.numel() == dw.numel()
    rdw, rdb = dp.allreduce_grads(dw, None)
    assert torch.equal(rdw, dw) and rdb is None


def _late_rank(port, hold_s):
    """Rank 0 of a two-rank job that comes up but never publishes the communicator id."""
    import datetime
    import time
    store = torch.distributed.TCPStore("127.0.0.1", port, 2, True, timeout=datetime.timedelta(seconds=30))
    time.sleep(hold_s)
    del store


def test_a_rank_that_never_publishes_the_id_times_out_on_the_host():
    """Failure detection stays on the host: the id travels through a key-value store with a bounded wait, so
    a missing rank 0 is an exception on the others after the timeout, before any GPU work is queued."""
    import datetime
    import time
    port = _free_port()
    ctx = mp.get_context("spawn")
    holder = ctx.Process(target=_late_rank, args=(port, 6.0))
    holder.start()
    try:
        store = None
        for _ in range(50):  # the server process needs a moment to listen
            try:
                store = torch.distributed.TCPStore("127.0.0.1", port, 2, False, timeout=datetime.timedelta(seconds=5))
                break
            except Exception:
                time.sleep(0.1)
        assert store is not None
        t0 = time.time()
        with pytest.raises(Exception):
            dp.exchange_unique_id(store, 1, lambda: b"", timeout_s=1.0)
        assert time.time() - t0 < 5.0
    finally:
        holder.join(timeout=15)
        if holder.is_alive():
            holder.terminate()


def test_the_id_reaches_the_other_ranks_through_the_store():
    import datetime
    port = _free_port()
    server = torch.distributed.TCPStore("127.0.0.1", port, 1, True, timeout=datetime.timedelta(seconds=10))
    uid = bytes(range(128))
    assert dp.exchange_unique_id(server, 0, lambda: uid) == uid
    assert dp.exchange_unique_id(server, 1, lambda: b"unused", timeout_s=2.0) == uid
