"""Batch-sharded (data-parallel) execution of the convolution path.

Forward and dInput are rank-local; dWeight and dBias are sums over samples, so the only
exchange step is one all-reduce of the fused buffer dW || dB per layer (NCCL over NVLink on
GPUs, gloo in the CPU tests).  The reference backend is single-device (README.md:50,137 of the
reference); this module is the multi-GPU plumbing the B200 build adds around the same operators.

Inputs for the sharded configuration are generated per global sample index, so every rank
count sees the same global batch.
"""
from __future__ import annotations

import torch


def shard_range(global_batch: int, rank: int, world: int):
    """Contiguous slice [start, stop) of the global batch owned by `rank`."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"invalid rank {rank} for world size {world}")
    if global_batch % world != 0:
        raise ValueError(f"global batch {global_batch} does not split evenly over {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def seeded_samples(sample_shape, base_seed: int, start: int, stop: int, scale: float = 1.0) -> torch.Tensor:
    """Samples start..stop-1 of a global batch; sample i ~ N(0,1) from Generator(base_seed + i)."""
    out = torch.empty((stop - start, *sample_shape), dtype=torch.float32)
    for i in range(start, stop):
        g = torch.Generator().manual_seed(base_seed + i)
        out[i - start] = torch.randn(sample_shape, generator=g) * scale
    return out


def fused_gradient_buffer(w_shape, with_bias: bool, like: torch.Tensor):
    """One flat buffer dW || dB on `like`'s device plus the two views into it.  The dWeight and dBias
    kernels write their results straight into the views, so the exchange needs no concatenation."""
    n_w = 1
    for d in w_shape:
        n_w *= int(d)
    n_b = int(w_shape[0]) if with_bias else 0
    flat = torch.empty(n_w + n_b, dtype=torch.float32, device=like.device)
    return flat, flat[:n_w].view(*w_shape), (flat[n_w:] if with_bias else None)


def allreduce_fused_(flat: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over ranks of a fused gradient buffer with ONE collective.  Tensors of the "vulkan"
    device go through the library's own communicator (torch_vulkan.all_reduce_, NCCL behind the C ABI);
    anything else through torch.distributed (gloo in the CPU tests)."""
    if flat.device.type == "vulkan":
        import torch_vulkan
        if torch_vulkan.comm_size() > 1:
            torch_vulkan.all_reduce_(flat)
        return flat
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    return flat


def allreduce_grads(dw: torch.Tensor, db: torch.Tensor | None, group=None):
    """Sum dW (and dB) over ranks with ONE collective.  When the two are already views of one fused buffer
    (fused_gradient_buffer) nothing is copied; otherwise they are packed into one first.
    Returns the reduced (dw, db)."""
    if db is not None and dw.is_contiguous() and db.is_contiguous() and dw.untyped_storage().data_ptr() == \
            db.untyped_storage().data_ptr() and db.storage_offset() == dw.storage_offset() + dw.numel():
        flat = torch.as_strided(dw, (dw.numel() + db.numel(),), (1,), dw.storage_offset())
        allreduce_fused_(flat, group)
        return dw, db
    parts = [dw.reshape(-1)] + ([db.reshape(-1)] if db is not None else [])
    fused = torch.cat(parts) if len(parts) > 1 else parts[0].clone()
    allreduce_fused_(fused, group)
    out_dw = fused[:dw.numel()].view_as(dw)
    out_db = fused[dw.numel():].view_as(db) if db is not None else None
    return out_dw, out_db


def exchange_unique_id(store, rank: int, make_id, key: str = "b200_comm_id", timeout_s: float = 60.0) -> bytes:
    """Rank 0 publishes the communicator id on a host key-value store (torch.distributed.TCPStore or
    anything with set / get / wait); the others fetch it.  A rank 0 that never shows up makes the others
    raise after `timeout_s` instead of waiting forever."""
    import datetime
    if rank == 0:
        uid = make_id()
        store.set(key, uid)
        return uid
    store.wait([key], datetime.timedelta(seconds=timeout_s))
    return bytes(store.get(key))
