"""CPU restatement of the reference's BatchNorm shaders.  TEST INFRASTRUCTURE ONLY.

numpy, one channel at a time, in the order of operations of the shaders
(csrc/shaders/batch_norm_forward.comp, batch_norm_eval.comp, batch_norm_backward.comp of the
reference); `dtype` selects the arithmetic (float32 as the shaders, float64 for a tight check).
Only the order of the 128-lane tree reduction is not reproduced: sums are numpy pairwise sums.

Parity status: pinned against PyTorch CPU FP64 `native_batch_norm` / `native_batch_norm_backward`
on the reference's own seeded cases (tests/test_batch_norm.py of the reference uses the same ground
truth): tests/test_batch_norm_oracle.py and tests/golden/batch_norm_cases.npz.
Only tests import this module.
"""
from __future__ import annotations

import numpy as np


def _channels(x):
    """[n, c, ...] -> [c, n * s] view order of the shader's address(r, c) (batch_norm_forward.comp:16)."""
    n, c = x.shape[:2]
    return np.moveaxis(x.reshape(n, c, -1), 1, 0).reshape(c, -1)


def _restore(rows, shape):
    n, c = shape[:2]
    return np.moveaxis(rows.reshape(c, n, -1), 0, 1).reshape(shape)


def forward(x, weight=None, bias=None, running_mean=None, running_var=None, training=True, momentum=0.1, eps=1e-5,
            dtype=np.float32):
    """(y, save_mean, save_inv, running_mean', running_var').  batch_norm_forward.comp:18-55 and
    batch_norm_eval.comp:20-30; save_* are empty in evaluation mode (batch_norm.cpp:37-38)."""
    f = np.dtype(dtype).type
    rows = _channels(np.asarray(x)).astype(dtype)
    c, m = rows.shape
    eps, momentum = f(eps), f(momentum)
    gamma = np.ones(c, dtype) if weight is None else np.asarray(weight).astype(dtype)
    beta = np.zeros(c, dtype) if bias is None else np.asarray(bias).astype(dtype)
    rm = None if running_mean is None else np.asarray(running_mean).astype(dtype).copy()
    rv = None if running_var is None else np.asarray(running_var).astype(dtype).copy()
    if training:
        origin = rows[:, :1]                                         # :25 origin = x[c*s]
        shifted = rows - origin
        mean_shift = shifted.sum(axis=1, dtype=dtype) / f(m)         # :27-30
        centered = shifted - mean_shift[:, None]                     # :33
        m2 = (centered * centered).sum(axis=1, dtype=dtype)
        variance = m2 / f(m)                                         # :36
        with np.errstate(divide="ignore", invalid="ignore"):
            inv = np.where((variance == 0) & (eps == 0), f(0), f(1) / np.sqrt(variance + eps))  # :37
            mean = origin[:, 0] + mean_shift
            if rm is not None:
                rm = (f(1) - momentum) * rm + momentum * mean        # :40
            if rv is not None:
                rv = (f(1) - momentum) * rv + momentum * (m2 / f(m - 1))  # :41 (0/0 = NaN for m == 1)
        save_mean, save_inv = mean.astype(dtype), inv.astype(dtype)
    else:
        if rm is None or rv is None:
            raise ValueError("evaluation requires running statistics")   # batch_norm.cpp:27-28
        centered = rows - rm[:, None]
        inv = f(1) / np.sqrt(rv + eps)                               # :45
        save_mean = save_inv = np.empty((0,), dtype)
    y = (centered * inv[:, None]) * gamma[:, None] + beta[:, None]   # :52
    return _restore(y.astype(dtype), np.asarray(x).shape), save_mean, save_inv, rm, rv


def backward(grad, x, weight, mean, inv_or_var, training=True, eps=1e-5, mask=(True, True, True), dtype=np.float32):
    """(dx, dw, db), None where masked off.  batch_norm_backward.comp:18-66."""
    f = np.dtype(dtype).type
    xs, gs = _channels(np.asarray(x)).astype(dtype), _channels(np.asarray(grad)).astype(dtype)
    c, m = xs.shape
    mean = np.asarray(mean).astype(dtype)
    inv = np.asarray(inv_or_var).astype(dtype)
    if not training:
        inv = f(1) / np.sqrt(inv + f(eps))                           # :22
    gamma = np.ones(c, dtype) if weight is None else np.asarray(weight).astype(dtype)
    want_dx, want_dw, want_db = mask
    if not any(mask):
        return None, None, None
    if training and m == 2:                                          # :26-38 algebraic pair derivative
        dg = f(0.5) * gs[:, 0] - f(0.5) * gs[:, 1]
        dw = ((xs[:, 0] - xs[:, 1]) * dg) * inv
        db = gs[:, 0] + gs[:, 1]
        v = (dg * gamma) * (((f(eps) * inv) * inv) * inv)
        dx = np.stack([v, -v], axis=1)
        return (_restore(dx.astype(dtype), np.asarray(x).shape) if want_dx else None,
                dw.astype(dtype) if want_dw else None, db.astype(dtype) if want_db else None)
    centered = xs - mean[:, None]
    a = gs.sum(axis=1, dtype=dtype)                                  # :41-46
    b = (centered * gs).sum(axis=1, dtype=dtype)
    residual = np.zeros(c, dtype)
    if training:
        residual = centered.sum(axis=1, dtype=dtype) / f(m)          # :50
        b = np.where(residual != 0, b - residual * a, b)             # :52
    dw, db = b * inv, a                                              # :56
    dx = None
    if want_dx:
        v = gs
        if training:                                                 # :61
            v = gs - (a[:, None] / f(m) + ((centered - residual[:, None]) * (b[:, None] / f(m))) * inv[:, None] * inv[:, None])
        dx = _restore((v * (inv * gamma)[:, None]).astype(dtype), np.asarray(x).shape)
    return dx, dw.astype(dtype) if want_dw else None, db.astype(dtype) if want_db else None
