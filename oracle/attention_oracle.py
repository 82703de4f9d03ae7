"""CPU restatement of the reference's attention shader.  TEST INFRASTRUCTURE ONLY.

numpy FP64 (or FP32) restatement of csrc/shaders/sdpa_training.comp of the reference without
dropout: scores q k^T * scale + mask with keys j > i hidden when causal (:16), the per-row
log-sum-exp and probabilities (:21-30), the three input gradients and the mask gradient (:33-45); masks are additive
floats or booleans (False hides the key).

Parity status: pinned against PyTorch CPU FP64 `scaled_dot_product_attention` and its autograd on
seeded inputs in tests/test_attention_oracle.py (the reference's tests/test_attention.py compares
with the same operator).  Only tests import this module.
"""
from __future__ import annotations

import numpy as np


def _scores(q, k, mask, causal, scale, dtype):
    s = np.einsum("bid,bjd->bij", q.astype(dtype), k.astype(dtype)) * dtype(scale)
    if mask is not None:
        mask = np.asarray(mask)
        # masktype 2 (bool): a zero byte hides the key; masktype 1: added to the scaled score (sdpa_training.comp:16)
        s = np.where(mask, s, -np.inf) if mask.dtype == np.bool_ else s + mask.astype(dtype)
    if causal:
        i, j = np.arange(s.shape[1])[:, None], np.arange(s.shape[2])[None, :]
        s = np.where(j > i, -np.inf, s)
    return s


def forward(q, k, v, mask=None, causal=False, scale=None, dtype=np.float64):
    """(out [b, tq, dv], lse [b, tq]); rows with every key hidden give zeros and -inf."""
    dtype = np.dtype(dtype).type
    scale = 1.0 / np.sqrt(q.shape[2]) if scale is None else scale
    s = _scores(q, k, mask, causal, scale, dtype)
    with np.errstate(divide="ignore", invalid="ignore"):
        mx = s.max(axis=2, keepdims=True) if s.shape[2] else np.full(s.shape[:2] + (1,), -np.inf)
        safe = np.where(np.isfinite(mx), mx, 0.0)
        e = np.exp(s - safe)
        total = e.sum(axis=2, keepdims=True)
        lse = np.where(total > 0, safe + np.log(total), -np.inf)
        p = np.where(total > 0, e / np.where(total > 0, total, 1.0), 0.0)
    out = np.einsum("bij,bje->bie", p, v.astype(dtype))
    return out.astype(dtype), lse[:, :, 0].astype(dtype)


def backward(grad, q, k, v, out, lse, mask=None, causal=False, scale=None, dtype=np.float64, mask_grad=False):
    """(dq, dk, dv), and with mask_grad the gradient of the additive mask, `ds` before the scale (:38,40)."""
    dtype = np.dtype(dtype).type
    scale = 1.0 / np.sqrt(q.shape[2]) if scale is None else scale
    s = _scores(q, k, mask, causal, scale, dtype)
    lse = np.asarray(lse).astype(dtype)[:, :, None]
    with np.errstate(invalid="ignore"):
        p = np.where(np.isfinite(lse), np.exp(s - np.where(np.isfinite(lse), lse, 0.0)), 0.0)
    g = grad.astype(dtype)
    dv = np.einsum("bij,bie->bje", p, g)
    dp = np.einsum("bie,bje->bij", g, v.astype(dtype))
    delta = (g * np.asarray(out).astype(dtype)).sum(axis=2, keepdims=True)
    dm = p * (dp - delta)
    ds = dm * dtype(scale)
    dq = np.einsum("bij,bjd->bid", ds, k.astype(dtype))
    dk = np.einsum("bij,bid->bjd", ds, q.astype(dtype))
    grads = dq.astype(dtype), dk.astype(dtype), dv.astype(dtype)
    return grads + (dm.astype(dtype),) if mask_grad else grads
