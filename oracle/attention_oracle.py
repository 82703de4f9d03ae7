"""CPU restatement of the reference's attention shader.  TEST INFRASTRUCTURE ONLY.

numpy FP64 (or FP32) restatement of csrc/shaders/sdpa_training.comp of the reference (dropout through the
Philox4x32-10 stream of csrc/shaders/philox.glsl, pinned on the algorithm's published known-answer vectors): scores q k^T * scale + mask with keys j > i hidden when causal (:16), the per-row
log-sum-exp and probabilities (:21-30), the three input gradients and the mask gradient (:33-45); masks are additive
floats or booleans (False hides the key).

Parity status: pinned against PyTorch CPU FP64 `scaled_dot_product_attention` and its autograd on
seeded inputs in tests/test_attention_oracle.py (the reference's tests/test_attention.py compares
with the same operator).  Only tests import this module.
"""
from __future__ import annotations

import numpy as np


def philox4x32_10(counter, key):
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11), vectorised:
    counter [..., 4] and key [..., 2] of uint32 -> [..., 4] uint32.  The round of csrc/shaders/philox.glsl:3-10."""
    c = [np.asarray(counter[..., i], np.uint64) for i in range(4)]
    k0, k1 = np.asarray(key[..., 0], np.uint64), np.asarray(key[..., 1], np.uint64)
    m32 = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = np.uint64(0xD2511F53) * c[0], np.uint64(0xCD9E8D57) * c[2]
        c = [(p1 >> np.uint64(32)) ^ c[1] ^ k0, p1 & m32, (p0 >> np.uint64(32)) ^ c[3] ^ k1, p0 & m32]
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & m32, (k1 + np.uint64(0xBB67AE85)) & m32
    return np.stack(c, axis=-1).astype(np.uint32)


def dropout_weights(shape, p, rng):
    """Weight of every score, flattened index i = (b*tq + row)*tk + key: 0 if dropped, else 1/(1-p)
    (sdpa_training.comp:17 `dropped`; philox.glsl:11-12: block i/4 at counter offset + block, word i%4, uniform from the
    top 24 bits).  rng = (seed, offset), both 64-bit."""
    if p == 0:
        return np.ones(shape)
    if p >= 1:
        return np.zeros(shape)
    seed, offset = int(rng[0]), int(rng[1])
    n = int(np.prod(shape))
    blocks = np.arange((n + 3) // 4, dtype=np.uint64)
    low = (np.uint64(offset & 0xFFFFFFFF) + blocks) & np.uint64(0xFFFFFFFF)
    high = (np.uint64(offset >> 32) + (low < np.uint64(offset & 0xFFFFFFFF)).astype(np.uint64)) & np.uint64(0xFFFFFFFF)
    counter = np.stack([low, high, np.zeros_like(low), np.zeros_like(low)], axis=-1)
    key = np.broadcast_to(np.array([seed & 0xFFFFFFFF, seed >> 32], np.uint64), (len(blocks), 2))
    words = philox4x32_10(counter, key).reshape(-1)[:n]
    uniform = (words >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)
    return np.where(uniform >= np.float32(p), 1.0 / (1.0 - np.float32(p)), 0.0).astype(np.float64).reshape(shape)


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


def forward(q, k, v, mask=None, causal=False, scale=None, dtype=np.float64, dropout=0.0, rng=None):
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
    out = np.einsum("bij,bje->bie", p * dropout_weights(p.shape, dropout, rng).astype(dtype), v.astype(dtype))
    return out.astype(dtype), lse[:, :, 0].astype(dtype)


def backward(grad, q, k, v, out, lse, mask=None, causal=False, scale=None, dtype=np.float64, mask_grad=False, dropout=0.0, rng=None):
    """(dq, dk, dv), and with mask_grad the gradient of the additive mask, `ds` before the scale (:38,40)."""
    dtype = np.dtype(dtype).type
    scale = 1.0 / np.sqrt(q.shape[2]) if scale is None else scale
    s = _scores(q, k, mask, causal, scale, dtype)
    lse = np.asarray(lse).astype(dtype)[:, :, None]
    with np.errstate(invalid="ignore"):
        p = np.where(np.isfinite(lse), np.exp(s - np.where(np.isfinite(lse), lse, 0.0)), 0.0)
    g = grad.astype(dtype)
    w = dropout_weights(p.shape, dropout, rng).astype(dtype)
    dv = np.einsum("bij,bie->bje", p * w, g)
    dp = np.einsum("bie,bje->bij", g, v.astype(dtype))
    delta = (g * np.asarray(out).astype(dtype)).sum(axis=2, keepdims=True)
    dm = p * (dp * w - delta)
    ds = dm * dtype(scale)
    dq = np.einsum("bij,bjd->bid", ds, k.astype(dtype))
    dk = np.einsum("bij,bid->bjd", ds, q.astype(dtype))
    grads = dq.astype(dtype), dk.astype(dtype), dv.astype(dtype)
    return grads + (dm.astype(dtype),) if mask_grad else grads
