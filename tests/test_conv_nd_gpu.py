"""Transposed and 1-D convolutions, which the reference routes through its generic N-d path
(csrc/ops/convolution_nd.cpp of the reference), against PyTorch CPU on the same seeded inputs:
through the C ABI (FP64 ground truth, gate 1e-4 relative L2) and through the PrivateUse1 operators
with autograd (tolerances of the reference's convolution tests, tests/test_conv_universality.py:36-44)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import b200conv
import torch_vulkan  # noqa: F401  (registers the device)
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-4

# (x shape, cout, kernel, stride, padding, output_padding, dilation, groups)
TRANSPOSED = [
    ((2, 6, 7, 9), 4, (3, 3), (1, 1), (0, 0), (0, 0), (1, 1), 1),
    ((2, 8, 9, 8), 6, (3, 3), (2, 2), (1, 1), (1, 1), (1, 1), 1),       # the usual x2 upsampling block
    ((1, 6, 5, 6), 9, (4, 2), (3, 2), (1, 0), (2, 1), (1, 1), 3),       # grouped, ragged kernel, output padding
    ((2, 4, 6, 5), 4, (3, 3), (1, 2), (2, 1), (0, 1), (2, 2), 2),       # dilated; output padding below the stride
    ((2, 64, 16, 16), 32, (2, 2), (2, 2), (0, 0), (0, 0), (1, 1), 1),   # U-Net up-convolution: tensor-core kernels
    ((2, 64, 12, 12), 64, (4, 4), (2, 2), (1, 1), (0, 0), (1, 1), 1),
]


def _transposed_inputs(case, seed):
    xshape, cout, kernel, stride, padding, output_padding, dilation, groups = case
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(*xshape, generator=gen)
    w = torch.randn(xshape[1], cout // groups, *kernel, generator=gen) * 0.2
    b = torch.randn(cout, generator=gen)
    return x, w, b, dict(stride=stride, padding=padding, output_padding=output_padding, dilation=dilation, groups=groups)


@pytest.mark.parametrize("case", TRANSPOSED, ids=lambda c: "x".join(map(str, c[0])) + f"-co{c[1]}-g{c[7]}")
@pytest.mark.parametrize("algo", ["auto", "direct"])
def test_conv_transpose2d_through_the_c_abi(case, algo):
    x, w, b, kw = _transposed_inputs(case, 31 + sum(case[0]))
    want = F.conv_transpose2d(x.double(), w.double(), b.double(), **kw).numpy()
    got = b200conv.conv_transpose2d_forward(x.numpy(), w.numpy(), b.numpy(), algo=algo, **kw)
    assert got.shape == want.shape
    assert oracle.rel_l2(got, want) <= GATE
    no_bias = b200conv.conv_transpose2d_forward(x.numpy(), w.numpy(), None, algo=algo, **kw)
    assert oracle.rel_l2(no_bias, F.conv_transpose2d(x.double(), w.double(), None, **kw).numpy()) <= GATE


def _check_autograd(run, tensors):
    """run(tensors...) on CPU and on the device; outputs and all gradients must agree."""
    cpu = [t.clone().requires_grad_() for t in tensors]
    dev = [t.to("vulkan").requires_grad_() for t in tensors]
    out_cpu, out_dev = run(*cpu), run(*dev)
    assert out_dev.device.type == "vulkan" and out_dev.shape == out_cpu.shape
    torch.testing.assert_close(out_dev.cpu(), out_cpu, atol=4e-4, rtol=3e-4)
    grad = torch.randn_like(out_cpu)
    expected = torch.autograd.grad(out_cpu, cpu, grad_outputs=grad)
    actual = torch.autograd.grad(out_dev, dev, grad_outputs=grad.to("vulkan"))
    for a, e in zip(actual, expected):
        assert a.device.type == "vulkan"
        torch.testing.assert_close(a.cpu(), e, atol=5e-4, rtol=4e-4)


@pytest.mark.parametrize("case", TRANSPOSED, ids=lambda c: "x".join(map(str, c[0])) + f"-co{c[1]}-g{c[7]}")
def test_conv_transpose2d_operator_and_gradients(case):
    x, w, b, kw = _transposed_inputs(case, 57 + sum(case[0]))
    _check_autograd(lambda xx, ww, bb: F.conv_transpose2d(xx, ww, bb, **kw), (x, w, b))


@pytest.mark.parametrize("xshape,cout,k,stride,padding,dilation,groups", [
    ((2, 6, 33), 8, 3, 1, 1, 1, 1), ((1, 4, 50), 6, 5, 2, 2, 1, 2), ((3, 8, 17), 8, 3, 1, 2, 2, 8), ((2, 64, 200), 64, 3, 1, 1, 1, 1),
])
def test_conv1d_operator_and_gradients(xshape, cout, k, stride, padding, dilation, groups):
    gen = torch.Generator().manual_seed(sum(xshape) + cout)
    x = torch.randn(*xshape, generator=gen)
    w = torch.randn(cout, xshape[1] // groups, k, generator=gen) * 0.3
    b = torch.randn(cout, generator=gen)
    _check_autograd(lambda xx, ww, bb: F.conv1d(xx, ww, bb, stride, padding, dilation, groups), (x, w, b))


@pytest.mark.parametrize("xshape,cout,k,stride,padding,output_padding,groups", [
    ((2, 6, 20), 4, 4, 2, 1, 0, 1), ((1, 8, 15), 6, 3, 3, 0, 2, 2),
])
def test_conv_transpose1d_operator_and_gradients(xshape, cout, k, stride, padding, output_padding, groups):
    gen = torch.Generator().manual_seed(sum(xshape) + cout)
    x = torch.randn(*xshape, generator=gen)
    w = torch.randn(xshape[1], cout // groups, k, generator=gen) * 0.3
    b = torch.randn(cout, generator=gen)
    _check_autograd(lambda xx, ww, bb: F.conv_transpose1d(xx, ww, bb, stride, padding, output_padding, groups), (x, w, b))


def test_rejections():
    x = torch.randn(1, 4, 5, 5).to("vulkan")
    w = torch.randn(4, 2, 3, 3).to("vulkan")
    with pytest.raises(RuntimeError, match="invalid output padding"):
        torch.ops.aten.convolution(x, w, None, [1, 1], [0, 0], [1, 1], True, [1, 1], 1)
    with pytest.raises(RuntimeError, match="weight/channel/group mismatch"):
        torch.ops.aten.convolution_overrideable(x, torch.randn(3, 2, 3, 3).to("vulkan"), None, [1, 1], [0, 0], [1, 1], True,
                                                [0, 0], 1)
    with pytest.raises(RuntimeError, match="one or two spatial dimensions"):
        F.conv3d(torch.randn(1, 2, 4, 4, 4).to("vulkan"), torch.randn(2, 2, 3, 3, 3).to("vulkan"))
