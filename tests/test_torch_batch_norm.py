"""BatchNorm through the PrivateUse1 ("vulkan") extension: the reference's operator-level tests
restated against the drop-in package (reference: tests/test_batch_norm.py:8-60, :91-100)."""
import itertools

import pytest
import torch
import torch.nn.functional as F

import torch_vulkan  # noqa: F401  (registers the device)

gpu = pytest.mark.gpu


def test_every_batch_norm_spelling_is_registered():
    # the operator names of csrc/ops/batch_norm.cpp:121-126 of the reference
    for op in ("native_batch_norm", "_native_batch_norm_legit", "_native_batch_norm_legit.no_stats",
               "_native_batch_norm_legit_no_training", "_batch_norm_with_update", "_batch_norm_with_update_functional",
               "native_batch_norm_backward", "batch_norm_backward"):
        assert torch._C._dispatch_has_kernel_for_dispatch_key("aten::" + op, "PrivateUse1"), op


def _every_other(x, device):
    """x as every other element (offset 1) of the last axis of a longer device buffer."""
    width = x.shape[-1]
    store = torch.zeros((*x.shape[:-1], 2 * width + 3), dtype=x.dtype)
    store[..., 1:1 + 2 * width:2] = x
    return store.to(device)[..., 1:1 + 2 * width:2]


# the strided forms the reference's tests feed the operator (tests/test_batch_norm.py:8-17 of the reference)
LAYOUTS = {
    "contiguous": lambda x, device: x.to(device),
    "channels_last": lambda x, device: x.to(device).contiguous(memory_format=torch.channels_last),
    "transpose": lambda x, device: x.transpose(-1, -2).contiguous().to(device).transpose(-1, -2),
    "slice": _every_other,
    "broadcast": lambda x, device: x[:1].to(device).expand(x.shape),
}


def layout(x, kind, device):
    return LAYOUTS[kind](x, device)


@gpu
@pytest.mark.parametrize("shape,kind", [
    ((7, 5), "contiguous"), ((2, 3, 11), "slice"), ((2, 5, 7, 9), "channels_last"), ((2, 5, 7, 9), "transpose"),
    ((2, 3, 4, 5, 7), "slice"), ((3, 2, 4, 7), "broadcast"), ((2, 3, 2, 3, 2, 2), "transpose"),
    ((4, 8, 40, 40), "contiguous"), ((4, 8, 40, 40), "channels_last"),
])
@pytest.mark.parametrize("training,affine,stats", [(True, True, True), (True, False, False), (False, True, True),
                                                   (False, False, True)])
def test_native_batch_norm_and_backward(shape, kind, training, affine, stats):
    torch.manual_seed(90)
    x, g, c = torch.randn(shape), torch.randn(shape), shape[1]
    w = torch.randn(c) if affine else None
    b = torch.randn(c) if affine else None
    rm = torch.randn(c) if stats else None
    rv = torch.rand(c) + .3 if stats else None

    def execute(device):
        xx, gg = layout(x, kind, device), layout(g, kind, device)

        def vec(v):  # strided, offset channel vectors on the device: reads and the in-place update
            if v is None:
                return None
            return v.clone() if device == "cpu" else layout(v, "slice", device)
        ww, bb, mm, vv = map(vec, (w, b, rm, rv))
        out, mean, inv = torch.ops.aten.native_batch_norm(xx, ww, bb, mm, vv, training, .23, 1e-4)
        grads = torch.ops.aten.native_batch_norm_backward(gg, xx, ww, mm, vv, mean, inv, training, 1e-4, [True] * 3)
        return (out, mean, inv, *grads, *([mm, vv] if stats else []))
    ref, got = execute("cpu"), execute("vulkan")
    for a, e in zip(got, ref):
        assert a.device.type == "vulkan"
        torch.testing.assert_close(a.cpu(), e, rtol=3e-4, atol=3e-5)
    if kind == "channels_last":   # the layout is kept, as PyTorch's CPU kernels keep it
        assert got[0].is_contiguous(memory_format=torch.channels_last)
        assert got[3].is_contiguous(memory_format=torch.channels_last)


@gpu
@pytest.mark.parametrize("mask", list(itertools.product([False, True], repeat=3)))
@pytest.mark.parametrize("training", [False, True])
def test_output_masks(mask, training):
    torch.manual_seed(8)
    x = torch.randn(2, 5, 7)
    g, w, m, v = torch.randn_like(x), torch.randn(5), torch.randn(5), torch.rand(5) + .5

    def run(device):
        xx, gg, ww, mm, vv = [t.to(device) for t in (x, g, w, m, v)]
        _, sm, si = torch.ops.aten.native_batch_norm(xx, ww, None, mm, vv, training, .1, 1e-5)
        return torch.ops.aten.native_batch_norm_backward(gg, xx, ww, mm, vv, sm, si, training, 1e-5, mask)
    for yes, a, e in zip(mask, run("vulkan"), run("cpu")):
        if yes:
            torch.testing.assert_close(a.cpu(), e, rtol=3e-4, atol=3e-5)
        else:
            assert a is None


@gpu
@pytest.mark.parametrize("training", [True, False])
def test_functional_batch_norm_through_autograd(training):
    torch.manual_seed(77)
    x, go = torch.randn(4, 6, 9, 9), torch.randn(4, 6, 9, 9)
    w, b, rm, rv = torch.randn(6), torch.randn(6), torch.randn(6), torch.rand(6) + .5

    def run(device):
        xx = x.to(device).requires_grad_()
        ww, bb = w.to(device).requires_grad_(), b.to(device).requires_grad_()
        mm, vv = rm.to(device), rv.to(device)
        y = F.batch_norm(xx, mm, vv, ww, bb, training, 0.1, 1e-5)
        y.backward(go.to(device))
        return y.detach(), xx.grad, ww.grad, bb.grad, mm, vv
    for a, e in zip(run("vulkan"), run("cpu")):
        torch.testing.assert_close(a.cpu(), e, rtol=4e-4, atol=4e-5)


@gpu
def test_single_sample_rejections_and_evaluation_outputs():
    x = torch.ones(1, 3).to("vulkan")
    m, v = torch.zeros(3).to("vulkan"), torch.ones(3).to("vulkan")
    y, mean, inv = torch.ops.aten.native_batch_norm(x, None, None, m, v, True, .1, 1e-5)
    torch.testing.assert_close(y.cpu(), torch.zeros(1, 3))
    assert v.cpu().isnan().all()   # unbiased variance of one sample (tests/test_batch_norm.py:91-100 of the reference)
    y, mean, inv = torch.ops.aten.native_batch_norm(x, None, None, m, torch.ones(3).to("vulkan"), False, .1, 1e-5)
    assert mean.numel() == 0 and inv.numel() == 0
    with pytest.raises(RuntimeError, match="evaluation requires running statistics"):
        torch.ops.aten.native_batch_norm(x, None, None, None, None, False, .1, 1e-5)
    with pytest.raises(RuntimeError, match="expects a channel vector"):
        torch.ops.aten.native_batch_norm(x, torch.ones(4).to("vulkan"), None, m, v, True, .1, 1e-5)
    with pytest.raises(RuntimeError, match="gradient shape mismatch"):
        torch.ops.aten.native_batch_norm_backward(torch.ones(2, 3).to("vulkan"), x, None, m, v, mean, inv, False, 1e-5,
                                                  [True] * 3)
