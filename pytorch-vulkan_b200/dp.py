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


def allreduce_grads(dw: torch.Tensor, db: torch.Tensor | None, group=None):
    """Sum dW (and dB) over ranks with ONE collective on the fused buffer dW || dB.
    Returns views into the reduced buffer shaped like the inputs."""
    import torch.distributed as dist
    parts = [dw.reshape(-1)] + ([db.reshape(-1)] if db is not None else [])
    fused = torch.cat(parts)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(fused, op=dist.ReduceOp.SUM, group=group)
    out_dw = fused[:dw.numel()].view_as(dw)
    out_db = fused[dw.numel():].view_as(db) if db is not None else None
    return out_dw, out_db
