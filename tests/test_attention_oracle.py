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


def test_philox_known_answers():
    """Known-answer vectors of Philox4x32-10 from the Random123 distribution (kat_vectors: counter, key -> output)."""
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for counter, key, want in kat:
        got = att.philox4x32_10(np.array([counter], np.uint32), np.array([key], np.uint32))[0]
        assert tuple(int(v) for v in got) == want


def test_dropout_oracle_statistics_and_autograd_identity():
    """The weights are 0 or 1/(1-p) with the right frequency, consecutive calls (offset advanced) differ, and the
    gradients are those of the same masked softmax computed by PyTorch with the oracle's own mask."""
    shape, p = (3, 40, 52), 0.35
    w = att.dropout_weights(shape, p, (42, 0))
    assert set(np.unique(w)) == {0.0, 1.0 / (1.0 - np.float32(p))}
    assert abs((w == 0).mean() - p) < 0.02
    assert (att.dropout_weights(shape, p, (42, (np.prod(shape) + 3) // 4)) != w).any()
    assert (att.dropout_weights(shape, 0.0, None) == 1).all() and (att.dropout_weights(shape, 1.0, None) == 0).all()
    gen = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(s, generator=gen, dtype=torch.float64, requires_grad=True) for s in ((3, 40, 8), (3, 52, 8), (3, 52, 6)))
    grad = torch.randn(3, 40, 6, generator=gen, dtype=torch.float64)
    probs = torch.softmax(q @ k.transpose(1, 2) * 0.37, dim=-1)
    want = (probs * torch.from_numpy(w)) @ v
    want.backward(grad)
    n = lambda t: t.detach().numpy()
    out, lse = att.forward(n(q), n(k), n(v), scale=0.37, dropout=p, rng=(42, 0))
    np.testing.assert_allclose(out, n(want), rtol=1e-10, atol=1e-12)
    for got, ref in zip(att.backward(n(grad), n(q), n(k), n(v), out, lse, scale=0.37, dropout=p, rng=(42, 0)), (q.grad, k.grad, v.grad)):
        np.testing.assert_allclose(got, n(ref), rtol=1e-9, atol=1e-11)
