"""CPU restatement of the reference's GroupNorm shaders.  TEST INFRASTRUCTURE ONLY.

numpy, in the order of operations of csrc/shaders/group_norm_forward.comp,
group_norm_backward_input.comp and group_norm_backward_affine.comp of the reference; `dtype` selects
the arithmetic (float32 as the shaders, float64 for a tight check).  Only the order of the
128-lane tree reduction is not reproduced: sums are numpy pairwise sums.

Parity status: pinned against PyTorch CPU FP64 `native_group_norm` / `native_group_norm_backward`
on the seeds and shapes of the reference's tests/test_native_group_norm.py
(tests/test_group_norm_oracle.py, tests/golden/group_norm_cases.npz).  Only tests import this module.
"""
from __future__ import annotations

import numpy as np


def forward(x, groups, weight=None, bias=None, eps=1e-5, dtype=np.float32):
    """(y, mean [n, groups], rstd [n, groups]).  group_norm_forward.comp:17-55."""
    f = np.dtype(dtype).type
    x = np.asarray(x)
    n, c = x.shape[:2]
    blocks = x.reshape(n, groups, -1).astype(dtype)            # :23 one contiguous block per (sample, group)
    count = blocks.shape[2]
    center = blocks[:, :, :1]                                  # :25
    mean = center[:, :, 0] + (blocks - center).sum(axis=2, dtype=dtype) / f(count)   # :26-34
    d = blocks - mean[:, :, None]
    with np.errstate(divide="ignore"):
        rstd = f(1) / np.sqrt((d * d).sum(axis=2, dtype=dtype) / f(count) + f(eps))   # :36-47
    gamma = np.ones(c, dtype) if weight is None else np.asarray(weight).astype(dtype)
    beta = np.zeros(c, dtype) if bias is None else np.asarray(bias).astype(dtype)
    z = (d * rstd[:, :, None]).reshape(n, c, -1)
    y = z * gamma[None, :, None] + beta[None, :, None]         # :53
    return y.reshape(x.shape).astype(dtype), mean.astype(dtype), rstd.astype(dtype)


def backward(grad, x, mean, rstd, groups, weight=None, mask=(True, True, True), dtype=np.float32):
    """(dx, dw, db), None where masked off.  group_norm_backward_input.comp:17-46 and
    group_norm_backward_affine.comp:12-32."""
    f = np.dtype(dtype).type
    x, grad = np.asarray(x), np.asarray(grad)
    n, c = x.shape[:2]
    xs, gs = x.reshape(n, c, -1).astype(dtype), grad.reshape(n, c, -1).astype(dtype)
    gamma = np.ones(c, dtype) if weight is None else np.asarray(weight).astype(dtype)
    m = np.repeat(np.asarray(mean).astype(dtype).reshape(n, groups), c // groups, axis=1)[:, :, None]
    r = np.repeat(np.asarray(rstd).astype(dtype).reshape(n, groups), c // groups, axis=1)[:, :, None]
    z = (xs - m) * r
    dx = dw = db = None
    if mask[0]:
        v = gs * gamma[None, :, None]
        count = f(xs.shape[2] * (c // groups))
        a = v.reshape(n, groups, -1).sum(axis=2, dtype=dtype) / count
        b = (v * z).reshape(n, groups, -1).sum(axis=2, dtype=dtype) / count
        a = np.repeat(a, c // groups, axis=1)[:, :, None]
        b = np.repeat(b, c // groups, axis=1)[:, :, None]
        dx = (r * (v - a - z * b)).reshape(x.shape).astype(dtype)
    if mask[1]:
        dw = (gs * z).sum(axis=(0, 2), dtype=dtype).astype(dtype)
    if mask[2]:
        db = gs.sum(axis=(0, 2), dtype=dtype).astype(dtype)
    return dx, dw, db
