"""Batched matrix product (bmm) against FP64 ground truth through the C ABI and against PyTorch CPU
through the PrivateUse1 operators, on the shapes and view styles of the reference's
tests/test_native_bmm.py (:8-11 there)."""
import numpy as np
import pytest
import torch

import b200conv
import torch_vulkan  # noqa: F401  (registers the device)
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-4
SHAPES = [(1, 2, 3, 7), (2, 8, 16, 11), (4, 16, 8, 32), (8, 32, 32, 32), (2, 2, 128, 4), (3, 256, 96, 128), (16, 128, 64, 128)]


def _views(style, batch, m, k, n, seed):
    """(a, b) numpy views of the given style: logical shapes [batch, m, k] and [batch, k, n]."""
    rng = np.random.default_rng(seed)
    r = lambda *s: rng.standard_normal(s, dtype=np.float32)
    if style == "contiguous":
        return r(batch, m, k), r(batch, k, n)
    if style == "right_transpose":
        return r(batch, m, k), r(batch, n, k).transpose(0, 2, 1)
    if style == "both":
        return r(batch, k, m).transpose(0, 2, 1), r(batch, n, k).transpose(0, 2, 1)
    if style == "offset":
        return r(batch, m + 1, k + 1)[:, :m, :k], r(batch, k + 1, n + 1)[:, :k, :n]
    if style == "batch_broadcast":
        return np.broadcast_to(r(1, m, k), (batch, m, k)), np.broadcast_to(r(1, k, n), (batch, k, n))
    if style == "shared_right":   # one right-hand matrix for all batches: a single product
        return r(batch, m, k), np.broadcast_to(r(1, k, n), (batch, k, n))
    raise ValueError(style)


STYLES = ["contiguous", "right_transpose", "both", "offset", "batch_broadcast", "shared_right"]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("style", STYLES)
def test_bmm_through_the_c_abi(shape, style):
    batch, m, k, n = shape
    a, b = _views(style, batch, m, k, n, 82 + sum(shape))
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    got = b200conv.bmm(a, b)
    assert got.shape == want.shape
    assert oracle.rel_l2(got, want) <= GATE


@pytest.mark.parametrize("shape", [(2, 8, 16, 32), (4, 16, 32, 16), (8, 32, 32, 32), (3, 256, 96, 128), (16, 128, 64, 128),
                                   (5, 130, 40, 72), (64, 128, 64, 64)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("style", STYLES)
def test_batched_tensor_core_kernel(shape, style):
    # every batch in one launch pair: forced onto the tcgen05 kernel, also for the strided views
    batch, m, k, n = shape
    a, b = _views(style, batch, m, k, n, 11 + sum(shape))
    got = b200conv.bmm(a, b, algo="tc")
    assert b200conv.last_kernel() in ("tc_bmm", "tc_gemm")   # tc_gemm: a shared right-hand matrix folds into one product
    assert oracle.rel_l2(got, np.matmul(a.astype(np.float64), b.astype(np.float64))) <= GATE
    assert b200conv.device_status() == 0


def test_empty_contraction_gives_zeros():
    got = b200conv.bmm(np.zeros((3, 5, 0), np.float32), np.zeros((3, 0, 4), np.float32))
    np.testing.assert_array_equal(got, np.zeros((3, 5, 4), np.float32))


@pytest.mark.parametrize("shape", SHAPES[:6], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("style", ["contiguous", "right_transpose", "both", "offset"])
def test_bmm_operator_and_autograd(shape, style):
    batch, m, k, n = shape
    a, b = _views(style, batch, m, k, n, 7 + sum(shape))
    base_a, base_b = torch.from_numpy(np.ascontiguousarray(a)), torch.from_numpy(np.ascontiguousarray(b))

    def run(device):
        # rebuild the same kind of view on the device: transposes and slices of dense device tensors
        ta, tb = base_a.to(device), base_b.to(device)
        if style in ("right_transpose", "both"):
            tb = tb.transpose(1, 2).contiguous().transpose(1, 2)
        if style == "both":
            ta = ta.transpose(1, 2).contiguous().transpose(1, 2)
        ta, tb = ta.detach().requires_grad_(), tb.detach().requires_grad_()
        out = torch.bmm(ta, tb)
        grad = torch.from_numpy(np.random.default_rng(5).standard_normal(out.shape, dtype=np.float32)).to(device)
        ga, gb = torch.autograd.grad(out, (ta, tb), grad)
        return out.detach(), ga, gb
    for got, want in zip(run("vulkan"), run("cpu")):
        assert got.device.type == "vulkan"
        torch.testing.assert_close(got.cpu(), want, rtol=2e-4, atol=2e-4)


def test_bmm_out_and_rejections():
    a, b = torch.randn(3, 8, 5), torch.randn(3, 5, 6)
    out = torch.empty(3, 8, 6).to("vulkan")
    torch.bmm(a.to("vulkan"), b.to("vulkan"), out=out)
    torch.testing.assert_close(out.cpu(), torch.bmm(a, b), rtol=2e-4, atol=2e-4)
    zero_k = torch.bmm(torch.empty(2, 3, 0).to("vulkan"), torch.empty(2, 0, 4).to("vulkan"))
    assert zero_k.shape == (2, 3, 4) and (zero_k.cpu() == 0).all()
    with pytest.raises(RuntimeError, match="matching batch dimensions and contraction size"):
        torch.ops.aten.bmm(a.to("vulkan"), torch.randn(3, 4, 6).to("vulkan"))
