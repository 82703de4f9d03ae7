"""Pins the N-d convolution restatement (oracle/convnd_oracle.py) against PyTorch's CPU convolutions, the ground truth of the
reference's own test for this path (tests/test_complete_spatial_recurrent.py:7-48 of the reference: same ranks, groups,
strides, paddings, dilations and output paddings), plus int64 forward with wrapping products."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import convnd_oracle


def reference_case(rank, transposed, groups, seed=91):
    gen = torch.Generator().manual_seed(seed)
    spatial = (4, 5, 6)[-rank:]
    co = 8
    x = torch.randn((2, 4, *spatial), generator=gen)
    kernel = (2, 3, 2)[-rank:]
    w = torch.randn((4, co // groups, *kernel) if transposed else (co, 4 // groups, *kernel), generator=gen)
    b = torch.randn(co, generator=gen)
    kw = dict(stride=(1, 2, 2)[-rank:], padding=(1, 1, 0)[-rank:], dilation=(1, 1, 2)[-rank:], groups=groups)
    if transposed:
        kw["output_padding"] = (0, 1, 1)[-rank:]
    return x, w, b, kw


def torch_fn(rank, transposed):
    return getattr(F, f"conv_transpose{rank}d" if transposed else f"conv{rank}d")


@pytest.mark.parametrize("rank,transposed", [(1, False), (2, False), (3, False), (1, True), (2, True), (3, True)])
@pytest.mark.parametrize("groups", [1, 2, 4])
def test_restatement_matches_torch_cpu(rank, transposed, groups):
    x, w, b, kw = reference_case(rank, transposed, groups)
    xd, wd, bd = (t.double().requires_grad_() for t in (x, w, b))
    want = torch_fn(rank, transposed)(xd, wd, bd, **kw)
    grad = torch.randn(want.shape, generator=torch.Generator().manual_seed(5), dtype=torch.float64)
    want.backward(grad)
    okw = dict(stride=kw["stride"], padding=kw["padding"], dilation=kw["dilation"], output_padding=kw.get("output_padding", 0),
               transposed=transposed, groups=groups)
    got = convnd_oracle.forward(x.numpy(), w.numpy(), b.numpy(), **okw)
    assert got.shape == tuple(want.shape)
    np.testing.assert_allclose(got, want.detach().numpy(), rtol=1e-12, atol=1e-12)
    dx, dw, db = convnd_oracle.backward(grad.numpy(), x.numpy(), w.numpy(), **okw)
    np.testing.assert_allclose(dx, xd.grad.numpy(), rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(dw, wd.grad.numpy(), rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(db, bd.grad.numpy(), rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("rank,transposed", [(2, False), (3, False), (3, True)])
def test_int64_forward_is_exact_and_wraps(rank, transposed):
    gen = torch.Generator().manual_seed(7)
    spatial = (4, 5, 6)[-rank:]
    x = torch.randint(-9, 9, (2, 4, *spatial), generator=gen, dtype=torch.int64)
    kernel = (2, 3, 2)[-rank:]
    w = torch.randint(-5, 5, (4, 4, *kernel) if transposed else (8, 2, *kernel), generator=gen, dtype=torch.int64)
    b = torch.randint(-100, 100, (8,), generator=gen, dtype=torch.int64)
    kw = dict(stride=(1, 2, 2)[-rank:], padding=(1, 1, 0)[-rank:], dilation=(1, 1, 2)[-rank:], groups=2)
    okw = dict(kw, transposed=transposed, output_padding=(0, 1, 1)[-rank:] if transposed else 0)
    if transposed:
        kw["output_padding"] = (0, 1, 1)[-rank:]
    want = torch_fn(rank, transposed)(x, w, b, **kw).numpy()
    got = convnd_oracle.forward(x.numpy(), w.numpy(), b.numpy(), **okw)
    assert got.dtype == np.int64 and np.array_equal(got, want)
    # products beyond 2^63 wrap, as 64-bit integer arithmetic on the device does
    big = convnd_oracle.forward(x.numpy() * (1 << 40), w.numpy() * (1 << 30), None, **okw)
    assert np.array_equal(big, (torch_fn(rank, transposed)(x * (1 << 40), w * (1 << 30), None, **kw)).numpy())
