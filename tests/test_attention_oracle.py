"""Pins the attention oracle against PyTorch CPU FP64 scaled_dot_product_attention and its autograd
(the ground truth of the reference's tests/test_attention.py) on seeded inputs."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import attention_oracle as att

CASES = [  # (batch, tq, tk, d, dv, causal, masked)
    (2, 5, 7, 8, 8, False, False), (3, 16, 16, 4, 6, True, False), (1, 9, 12, 16, 16, False, True),
    (2, 33, 33, 8, 8, True, True), (4, 1, 10, 8, 3, False, False),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_oracle_matches_pytorch_fp64(case):
    batch, tq, tk, d, dv, causal, masked = case
    gen = torch.Generator().manual_seed(sum(case[:5]))
    q = torch.randn(batch, tq, d, generator=gen, dtype=torch.float64, requires_grad=True)
    k = torch.randn(batch, tk, d, generator=gen, dtype=torch.float64, requires_grad=True)
    v = torch.randn(batch, tk, dv, generator=gen, dtype=torch.float64, requires_grad=True)
    mask = torch.randn(batch, tq, tk, generator=gen, dtype=torch.float64) if masked else None
    grad = torch.randn(batch, tq, dv, generator=gen, dtype=torch.float64)
    full = mask
    if causal:   # PyTorch refuses a mask together with is_causal: fold the triangle into the mask
        tri = torch.full((tq, tk), float("-inf"), dtype=torch.float64).triu(1)
        full = tri if mask is None else mask + tri
    want = F.scaled_dot_product_attention(q, k, v, attn_mask=full)
    wdq, wdk, wdv = torch.autograd.grad(want, (q, k, v), grad)
    n = lambda t: None if t is None else t.detach().numpy()
    out, lse = att.forward(n(q), n(k), n(v), n(mask), causal)
    np.testing.assert_allclose(out, n(want), rtol=1e-10, atol=1e-12)
    dq, dk, dv_ = att.backward(n(grad), n(q), n(k), n(v), out, lse, n(mask), causal)
    for got, exp in ((dq, wdq), (dk, wdk), (dv_, wdv)):
        np.testing.assert_allclose(got, n(exp), rtol=1e-9, atol=1e-11)


def test_rows_with_every_key_hidden():
    q, k, v = np.ones((1, 2, 4)), np.ones((1, 3, 4)), np.ones((1, 3, 2))
    mask = np.zeros((1, 2, 3))
    mask[0, 1] = -np.inf
    out, lse = att.forward(q, k, v, mask)
    assert np.isneginf(lse[0, 1]) and (out[0, 1] == 0).all() and np.isfinite(lse[0, 0])


@pytest.mark.parametrize("shape", [(2, 5, 7, 4, 6), (3, 37, 19, 8, 3)])
def test_bool_masks_and_the_mask_gradient_match_pytorch_fp64(shape):
    """Cases in the manner of the reference's tests/test_complete_attention.py:6-24: a bool mask and a float mask
    that requires a gradient, scale 0.37."""
    batch, tq, tk, d, dv = shape
    gen = torch.Generator().manual_seed(432)
    q, k, v = (torch.randn(s, generator=gen, dtype=torch.float64, requires_grad=True) for s in ((batch, tq, d), (batch, tk, d), (batch, tk, dv)))
    grad = torch.randn(batch, tq, dv, generator=gen, dtype=torch.float64)
    keep = torch.rand(batch, tq, tk, generator=gen) > 0.3
    keep[:, :, 0] = True
    want = F.scaled_dot_product_attention(q, k, v, attn_mask=keep, scale=0.37)
    want.backward(grad)
    n = lambda t: t.detach().numpy()
    out, lse = att.forward(n(q), n(k), n(v), n(keep), scale=0.37)
    np.testing.assert_allclose(out, n(want), rtol=1e-10, atol=1e-12)
    for got, ref in zip(att.backward(n(grad), n(q), n(k), n(v), out, lse, n(keep), scale=0.37), (q.grad, k.grad, v.grad)):
        np.testing.assert_allclose(got, n(ref), rtol=1e-9, atol=1e-11)
    for t in (q, k, v):
        t.grad = None
    add = torch.randn(batch, tq, tk, generator=gen, dtype=torch.float64, requires_grad=True)
    F.scaled_dot_product_attention(q, k, v, attn_mask=add, scale=0.37).backward(grad)
    out, lse = att.forward(n(q), n(k), n(v), n(add), scale=0.37)
    dq, dk, dvv, dm = att.backward(n(grad), n(q), n(k), n(v), out, lse, n(add), scale=0.37, mask_grad=True)
    np.testing.assert_allclose(dm, n(add.grad), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dq, n(q.grad), rtol=1e-9, atol=1e-11)
