"""GroupNorm through the PrivateUse1 ("vulkan") extension: the reference's operator-level tests
restated against the drop-in package (reference: tests/test_native_group_norm.py:9-44, :47-77)."""
import pytest
import torch
import torch.nn.functional as F

import torch_vulkan  # noqa: F401  (registers the device)

gpu = pytest.mark.gpu


def test_group_norm_operators_are_registered():
    for op in ("aten::native_group_norm", "aten::native_group_norm_backward"):
        assert torch._C._dispatch_has_kernel_for_dispatch_key(op, "PrivateUse1"), op


@gpu
@pytest.mark.parametrize("shape,groups", [((2, 8, 4, 5), 4), ((1, 8, 8, 8), 1), ((1, 12, 3, 7), 3), ((2, 16, 8), 8),
                                          ((2, 8, 2, 3, 4), 2), ((1, 8, 2, 2), 8), ((2, 4, 1, 1), 2), ((2, 32, 48, 48), 8)])
@pytest.mark.parametrize("affine", [False, True])
def test_group_norm_forward_backward_through_autograd(shape, groups, affine):
    torch.manual_seed(1000 + sum(shape) + groups)
    x = torch.randn(*shape, requires_grad=True)
    c = shape[1]
    w = torch.randn(c, requires_grad=True) if affine else None
    b = torch.randn(c, requires_grad=True) if affine else None
    on_device = lambda t: None if t is None else t.detach().to("vulkan").requires_grad_()
    xv, wv, bv = on_device(x), on_device(w), on_device(b)
    out, actual = F.group_norm(x, groups, w, b, 1e-5), F.group_norm(xv, groups, wv, bv, 1e-5)
    assert actual.device.type == "vulkan"
    torch.testing.assert_close(actual.cpu(), out, rtol=5e-4, atol=4e-5)
    grad = torch.randn_like(out)
    expected = torch.autograd.grad(out, tuple(v for v in (x, w, b) if v is not None), grad)
    grads = torch.autograd.grad(actual, tuple(v for v in (xv, wv, bv) if v is not None), grad.to("vulkan"))
    for got, want in zip(grads, expected):
        torch.testing.assert_close(got.cpu(), want, rtol=8e-4, atol=7e-5)


VIEWS = {
    "transpose_spatial": lambda t: t.transpose(-1, -2),
    "channels_last": lambda t: t.contiguous(memory_format=torch.channels_last),
    "offset": lambda t: t[:, :, :5, 1:],
    "expanded": lambda t: t[:1].expand(2, -1, -1, -1),
}


@gpu
@pytest.mark.parametrize("kind", sorted(VIEWS))
def test_group_norm_on_strided_views(kind):
    torch.manual_seed(901)
    raw = torch.randn(2, 8, 6, 7)
    x = VIEWS[kind](raw).detach().requires_grad_()
    xv = VIEWS[kind](raw.to("vulkan")).detach().requires_grad_()
    out, ov = F.group_norm(x, 4), F.group_norm(xv, 4)
    torch.testing.assert_close(ov.cpu(), out, atol=2e-4, rtol=5e-4)
    grad = torch.randn_like(out)
    expected = torch.autograd.grad(out, x, grad)[0]
    actual = torch.autograd.grad(ov, xv, grad.to("vulkan"))[0]
    torch.testing.assert_close(actual.cpu(), expected, atol=3e-4, rtol=5e-4)


@gpu
@pytest.mark.parametrize("mask", [(True, False, False), (False, True, False), (False, False, True), (True, True, True)])
def test_group_norm_output_mask_and_rejections(mask):
    torch.manual_seed(123)
    x, g, w = torch.randn(2, 8, 5, 6), torch.randn(2, 8, 5, 6), torch.randn(8)

    def run(device):
        xx, gg, ww = x.to(device), g.to(device), w.to(device)
        _, mean, rstd = torch.ops.aten.native_group_norm(xx, ww, None, 2, 8, 30, 4, 1e-5)
        return torch.ops.aten.native_group_norm_backward(gg, xx, mean, rstd, ww, 2, 8, 30, 4, list(mask))
    for yes, a, e in zip(mask, run("vulkan"), run("cpu")):
        if yes:
            torch.testing.assert_close(a.cpu(), e, rtol=8e-4, atol=7e-5)
        else:
            assert a is None
    with pytest.raises(RuntimeError, match="invalid batch, channel, group or spatial"):
        torch.ops.aten.native_group_norm(x.to("vulkan"), None, None, 2, 8, 30, 3, 1e-5)
    with pytest.raises(RuntimeError, match="weight must have C float elements"):
        torch.ops.aten.native_group_norm(x.to("vulkan"), torch.ones(7).to("vulkan"), None, 2, 8, 30, 4, 1e-5)
