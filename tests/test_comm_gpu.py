"""The data-parallel exchange through the C ABI (b200_comm_*, b200_allreduce_sum_f32) and through the
torch_vulkan module.  One rank on one GPU here; a two-rank case runs as two child processes when the box
has two GPUs (the id travels through a TCP store, as dp.exchange_unique_id does it)."""
import ctypes
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import b200conv

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_communicator_all_reduce_is_the_identity():
    b200conv.init()
    L = b200conv.lib()
    assert L.b200_comm_size() == 0 and L.b200_comm_rank() == -1
    with pytest.raises(b200conv.B200Error, match="b200_comm_init has not been called"):
        b200conv.allreduce_sum_f32(b200conv.DeviceBuffer(16).ptr, 4)
    uid = b200conv.comm_unique_id()
    assert len(uid) == 128
    b200conv.comm_init(0, 1, uid, timeout_ms=30000)
    try:
        assert L.b200_comm_size() == 1 and L.b200_comm_rank() == 0
        with pytest.raises(b200conv.B200Error, match="already initialised"):
            b200conv.comm_init(0, 1, uid)
        x = np.random.default_rng(0).standard_normal(100003, dtype=np.float32)
        v = b200conv.DeviceView(x)
        before = b200conv.launch_count()
        b200conv.allreduce_sum_f32(v.ptr, x.size)
        np.testing.assert_array_equal(v.buf.to_numpy(x.shape), x)
        assert b200conv.launch_count() == before + 1
        b200conv.allreduce_sum_f32(v.ptr, 0)      # empty buffers are accepted
    finally:
        b200conv.comm_destroy()
    assert L.b200_comm_size() == 0
    b200conv.comm_destroy()                          # idempotent
    with pytest.raises(b200conv.B200Error, match="invalid rank"):
        b200conv.comm_init(2, 2, uid)


def test_vulkan_tensors_all_reduce_through_the_module():
    import torch
    import torch_vulkan
    import dp
    uid = torch_vulkan.comm_unique_id()
    torch_vulkan.comm_init(0, 1, uid, 30000)
    try:
        assert torch_vulkan.comm_size() == 1
        t = torch.arange(12, dtype=torch.float32).reshape(3, 4)
        v = t.to("vulkan")
        assert torch_vulkan.all_reduce_(v) is v
        torch.testing.assert_close(v.cpu(), t)
        flat, dw, db = dp.fused_gradient_buffer((4, 2, 3, 3), True, v)
        assert flat.device.type == "vulkan" and dw.shape == (4, 2, 3, 3) and db.shape == (4,)
        rdw, rdb = dp.allreduce_grads(dw, db)       # views of one buffer: one collective, nothing copied
        assert rdw.data_ptr() == dw.data_ptr() and rdb.data_ptr() == db.data_ptr()
        with pytest.raises(RuntimeError, match="contiguous FP32"):
            torch_vulkan.all_reduce_(v.t())
    finally:
        torch_vulkan.comm_destroy()


_CHILD = r"""
import datetime, os, sys
import numpy as np
sys.path.insert(0, sys.argv[4]); sys.path.insert(0, os.path.join(sys.argv[4], "pytorch-vulkan_b200"))
import torch
import b200conv, dp
rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
b200conv.init(rank)
store = torch.distributed.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=60))
uid = dp.exchange_unique_id(store, rank, b200conv.comm_unique_id, timeout_s=60.0)
b200conv.comm_init(rank, world, uid, timeout_ms=60000)
x = np.full(1 << 20, float(rank + 1), np.float32)
v = b200conv.DeviceView(x)
b200conv.allreduce_sum_f32(v.ptr, x.size)
out = v.buf.to_numpy(x.shape)
assert (out == world * (world + 1) / 2).all(), out[:4]
store.set(f"done{rank}", b"1")
store.wait([f"done{r}" for r in range(world)], datetime.timedelta(seconds=60))   # leave between steps, together
b200conv.comm_destroy()
print("rank", rank, "ok")
"""


def test_two_ranks_on_two_gpus_sum_their_buffers():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", _CHILD, str(r), "2", str(port), ROOT], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
