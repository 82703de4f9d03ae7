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
from oracle import convnd_oracle, oracle

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
    with pytest.raises(RuntimeError, match="matching FP32/int64 tensors"):
        F.conv3d(torch.randn(1, 2, 4, 4, 4).to("vulkan"), torch.randn(2, 2, 3, 3, 3).double().to("vulkan"))
    over = lambda xx, ww, bb=None: torch.ops.aten.convolution_overrideable(xx, ww, bb, [1, 1, 1], [0, 0, 0], [1, 1, 1], False, [0, 0, 0], 1)
    dev = lambda *shape: torch.randn(*shape).to("vulkan")
    with pytest.raises(RuntimeError, match="weight/channel/group mismatch"):
        over(dev(1, 3, 4, 4, 4), dev(2, 2, 3, 3, 3))
    with pytest.raises(RuntimeError, match="invalid bias"):
        over(dev(1, 2, 4, 4, 4), dev(2, 2, 3, 3, 3), dev(3))
    with pytest.raises(RuntimeError, match="invalid or oversized output shape"):
        over(dev(1, 2, 2, 4, 4), dev(2, 2, 3, 3, 3))


# ---- three spatial dimensions and int64: the generic one-thread-per-output kernel ----------------------------------
def _nd_case(rank, transposed, groups, seed=91):
    """Shapes and parameters of the reference's own test of this path (tests/test_complete_spatial_recurrent.py:7-37)."""
    gen = torch.Generator().manual_seed(seed)
    spatial, kernel, co = (4, 5, 6)[-rank:], (2, 3, 2)[-rank:], 8
    x = torch.randn((2, 4, *spatial), generator=gen)
    w = torch.randn((4, co // groups, *kernel) if transposed else (co, 4 // groups, *kernel), generator=gen)
    b = torch.randn(co, generator=gen)
    kw = dict(stride=(1, 2, 2)[-rank:], padding=(1, 1, 0)[-rank:], dilation=(1, 1, 2)[-rank:], groups=groups)
    if transposed:
        kw["output_padding"] = (0, 1, 1)[-rank:]
    return x, w, b, kw


def _okw(kw, transposed):
    return dict(stride=kw["stride"], padding=kw["padding"], dilation=kw["dilation"], output_padding=kw.get("output_padding", 0),
                transposed=transposed, groups=kw["groups"])


@pytest.mark.parametrize("rank,transposed", [(1, False), (2, False), (3, False), (1, True), (2, True), (3, True)])
@pytest.mark.parametrize("groups", [1, 2, 4])
def test_generic_kernel_through_the_c_abi(rank, transposed, groups):
    x, w, b, kw = _nd_case(rank, transposed, groups)
    okw = _okw(kw, transposed)
    want = convnd_oracle.forward(x.numpy(), w.numpy(), b.numpy(), **okw)
    got = b200conv.convnd_forward(x.numpy(), w.numpy(), b.numpy(), **okw)
    assert got.shape == want.shape and oracle.rel_l2(got, want) <= 1e-6
    assert b200conv.last_kernel() == "convnd_forward"
    grad = torch.randn(want.shape, generator=torch.Generator().manual_seed(3)).numpy()
    wdx, wdw, wdb = convnd_oracle.backward(grad, x.numpy(), w.numpy(), **okw)
    dx, dw, db = b200conv.convnd_backward(grad, x.numpy(), w.numpy(), **okw)
    assert oracle.rel_l2(dx, wdx) <= 1e-6 and oracle.rel_l2(dw, wdw) <= 1e-6 and oracle.rel_l2(db, wdb) <= 1e-6
    only_dw = b200conv.convnd_backward(grad, x.numpy(), w.numpy(), mask=(False, True, False), **okw)
    assert only_dw[0] is None and only_dw[2] is None and np.array_equal(only_dw[1], dw)


@pytest.mark.parametrize("generic", [True, False], ids=["generic-kernel", "tensor-core-decomposition"])
def test_generic_kernel_on_a_video_sized_block(generic, monkeypatch):
    """A 3-D residual block shape (16 frames of 56x56, 16 -> 32 channels, 3x3x3, stride (1,2,2)) against the restatement,
    through the one-thread-per-output kernel (pinned by B200_CONV3D_GENERIC) and through the decomposition."""
    if generic:
        monkeypatch.setenv("B200_CONV3D_GENERIC", "1")
    else:
        monkeypatch.setenv("B200_CONV3D_DECOMPOSE", "1")
    gate = 2e-6 if generic else 2e-5
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(1, 16, 8, 28, 28, generator=gen).numpy()
    w = (torch.randn(32, 16, 3, 3, 3, generator=gen) * 0.1).numpy()
    b = torch.randn(32, generator=gen).numpy()
    okw = dict(stride=(1, 2, 2), padding=1, dilation=1, groups=1)
    want = convnd_oracle.forward(x, w, b, **okw)
    got = b200conv.convnd_forward(x, w, b, **okw)
    assert b200conv.last_kernel().startswith("convnd_forward" if generic else "conv3d_forward")
    assert oracle.rel_l2(got, want) <= gate
    grad = torch.randn(want.shape, generator=gen).numpy()
    for g, e in zip(b200conv.convnd_backward(grad, x, w, **okw), convnd_oracle.backward(grad, x, w, **okw)):
        assert oracle.rel_l2(g, e) <= gate


@pytest.mark.parametrize("rank,transposed", [(1, False), (2, False), (3, False), (2, True), (3, True)])
def test_int64_forward_is_bit_exact(rank, transposed):
    gen = torch.Generator().manual_seed(7 + rank)
    spatial, kernel = (4, 5, 6)[-rank:], (2, 3, 2)[-rank:]
    x = torch.randint(-9, 9, (2, 4, *spatial), generator=gen, dtype=torch.int64)
    w = torch.randint(-5, 5, (4, 4, *kernel) if transposed else (8, 2, *kernel), generator=gen, dtype=torch.int64)
    b = torch.randint(-100, 100, (8,), generator=gen, dtype=torch.int64)
    okw = dict(stride=(1, 2, 2)[-rank:], padding=(1, 1, 0)[-rank:], dilation=(1, 1, 2)[-rank:], groups=2, transposed=transposed,
               output_padding=(0, 1, 1)[-rank:] if transposed else 0)
    for xs, ws, bias in ((1, 1, b.numpy()), (1 << 40, 1 << 30, None)):       # the second pair wraps past 2^63
        want = convnd_oracle.forward(x.numpy() * xs, w.numpy() * ws, bias, **okw)
        got = b200conv.convnd_forward(x.numpy() * xs, w.numpy() * ws, bias, **okw)
        assert got.dtype == np.int64 and np.array_equal(got, want)
    assert b200conv.last_kernel() == "convnd_forward_int64"
    # through the operator: an int64 tensor on the device takes the same kernel
    fn = getattr(F, f"conv_transpose{rank}d" if transposed else f"conv{rank}d")
    kw = {k: v for k, v in okw.items() if k != "transposed" and (transposed or k != "output_padding")}
    dev = fn(x.to("vulkan"), w.to("vulkan"), b.to("vulkan"), **kw)
    assert dev.dtype == torch.int64 and torch.equal(dev.cpu(), fn(x, w, b, **kw))


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("groups", [1, 2, 4])
@pytest.mark.parametrize("layout", ["contiguous", "offset", "channels_last"])
def test_conv3d_operator_and_gradients(transposed, groups, layout):
    """The reference's own 3-D test (tests/test_complete_spatial_recurrent.py:7-37): same shapes, views and tolerances."""
    x, w, b, kw = _nd_case(3, transposed, groups)
    if layout == "offset":
        def view(t):
            base = torch.empty((*t.shape[:-1], t.shape[-1] * 2 + 1), device="vulkan")
            out = base[..., 1::2]
            out.copy_(t.to("vulkan"))
            return out.detach().requires_grad_()
        refs = [t.clone().requires_grad_() for t in (x, w, b)]
        vals = [view(x), view(w), b.to("vulkan").requires_grad_()]
    else:
        if layout == "channels_last":
            x = x.contiguous(memory_format=torch.channels_last_3d)
        refs = [t.clone().requires_grad_() for t in (x, w, b)]
        vals = [t.to("vulkan").requires_grad_() for t in (x, w, b)]
    fn = F.conv_transpose3d if transposed else F.conv3d
    expected, actual = fn(*refs, **kw), fn(*vals, **kw)
    grad = torch.randn_like(expected)
    expected.backward(grad)
    actual.backward(grad.to("vulkan"))
    torch.testing.assert_close(actual.cpu(), expected, rtol=3e-4, atol=1e-4)
    for a, e in zip(vals, refs):
        torch.testing.assert_close(a.grad.cpu(), e.grad, rtol=4e-4, atol=2e-4)


@pytest.mark.parametrize("transposed", [False, True])
def test_conv3d_empty_batch(transposed):
    """An empty batch gives an empty result and a zero dW (tests/test_complete_spatial_recurrent.py:40-48 of the reference).
    Through the C ABI: PyTorch resolves an empty-batch convolution itself, with elementwise operators, before the backend's
    convolution operator is reached."""
    x = np.empty((0, 2, 3, 4, 5), np.float32)
    w = torch.randn((2, 3, 2, 2, 2) if transposed else (3, 2, 2, 2, 2)).numpy()
    y = b200conv.convnd_forward(x, w, None, transposed=transposed)
    assert y.shape == ((0, 3, 4, 5, 6) if transposed else (0, 3, 2, 3, 4))
    dx, dw, db = b200conv.convnd_backward(np.empty(y.shape, np.float32), x, w, transposed=transposed)
    assert dx.shape == x.shape and (dw == 0).all() and dw.shape == w.shape and (db == 0).all()


@pytest.mark.parametrize("case", [TRANSPOSED[4], TRANSPOSED[5], ((2, 128, 12, 12), 128, (3, 3), (1, 1), (1, 1), (0, 0), (1, 1), 1)],
                         ids=["up2x2", "up4x4s2", "3x3s1-128"])
def test_transposed_bias_rides_in_the_tensor_core_epilogue(case):
    """With a tcgen05 (or Winograd) kernel the bias of a transposed convolution costs no extra launch."""
    x, w, b, kw = _transposed_inputs(case, 77)
    b200conv.conv_transpose2d_forward(x.numpy(), w.numpy(), None, algo="tc", **kw)      # warm: one-time attribute calls
    n0 = b200conv.launch_count()
    plain = b200conv.conv_transpose2d_forward(x.numpy(), w.numpy(), None, algo="tc", **kw)
    n1 = b200conv.launch_count()
    biased = b200conv.conv_transpose2d_forward(x.numpy(), w.numpy(), b.numpy(), algo="tc", **kw)
    n2 = b200conv.launch_count()
    assert n2 - n1 == n1 - n0
    want = F.conv_transpose2d(x.double(), w.double(), b.double(), **kw).numpy()
    assert oracle.rel_l2(biased, want) <= GATE
    np.testing.assert_allclose(biased - plain, np.broadcast_to(b.numpy()[None, :, None, None], plain.shape), atol=2e-5)


# ---- 3-D convolutions with 16 or more channels per group: depth taps on the 2-D tensor-core kernels ----------------
WIDE3D = [  # (x shape, cout, kernel, stride, padding, dilation, groups)
    ((2, 32, 6, 10, 9), 48, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1),
    ((1, 64, 5, 12, 12), 64, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1),
    ((2, 32, 7, 9, 8), 32, (2, 3, 2), (2, 1, 2), (1, 1, 0), (1, 1, 2), 1),       # strides and dilation: dInput through the 2-D dInput kernels + strided add
    ((2, 64, 6, 8, 8), 64, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 2),       # two groups of 32: likewise
    ((1, 32, 4, 7, 7), 32, (5, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1),       # depth taps that reach no input depth at all
    ((2, 48, 8, 6, 6), 32, (3, 1, 1), (1, 1, 1), (0, 0, 0), (2, 1, 1), 1),       # "valid" in depth with dilation 2
    ((2, 32, 9, 11, 10), 64, (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), 1),     # stride 2 everywhere (a video stem's shape)
    ((1, 32, 6, 8, 8), 32, (3, 3, 3), (1, 1, 1), (3, 3, 3), (1, 1, 1), 1),       # padding beyond the filter reach
]


@pytest.mark.parametrize("case", WIDE3D, ids=lambda c: "x".join(map(str, c[0])) + f"-co{c[1]}-k{'x'.join(map(str, c[2]))}-g{c[6]}")
def test_conv3d_on_the_tensor_core_kernels(case, monkeypatch):
    monkeypatch.setenv("B200_CONV3D_DECOMPOSE", "1")      # these shapes are below the size from which it is chosen
    xshape, cout, kernel, stride, padding, dilation, groups = case
    gen = torch.Generator().manual_seed(sum(xshape) + cout)
    x = torch.randn(*xshape, generator=gen).numpy()
    w = (torch.randn(cout, xshape[1] // groups, *kernel, generator=gen) / np.sqrt(xshape[1] // groups * np.prod(kernel))).numpy()
    b = torch.randn(cout, generator=gen).numpy()
    okw = dict(stride=stride, padding=padding, dilation=dilation, groups=groups)
    want = convnd_oracle.forward(x, w, b, **okw)
    got = b200conv.convnd_forward(x, w, b, **okw)
    assert b200conv.last_kernel().startswith("conv3d_forward")
    assert got.shape == want.shape and oracle.rel_l2(got, want) <= 2e-5
    assert oracle.rel_l2(b200conv.convnd_forward(x, w, None, **okw), convnd_oracle.forward(x, w, None, **okw)) <= 2e-5
    grad = torch.randn(want.shape, generator=gen).numpy()
    for g, e in zip(b200conv.convnd_backward(grad, x, w, **okw), convnd_oracle.backward(grad, x, w, **okw)):
        assert oracle.rel_l2(g, e) <= 2e-5
    assert b200conv.device_status() == 0


def test_conv3d_wide_operator_and_gradients(monkeypatch):
    """The operator on a wide 3-D layer (tensor-core decomposition) agrees with the generic kernel and with PyTorch CPU."""
    monkeypatch.setenv("B200_CONV3D_DECOMPOSE", "1")
    torch.manual_seed(14)
    x, w, b = torch.randn(2, 32, 5, 9, 9), torch.randn(32, 32, 3, 3, 3) * 0.05, torch.randn(32)
    fn = lambda xx, ww, bb: F.conv3d(xx, ww, bb, padding=1)
    _check_autograd(fn, (x, w, b))
    fast = fn(x.to("vulkan"), w.to("vulkan"), b.to("vulkan")).cpu()
    monkeypatch.setenv("B200_CONV3D_GENERIC", "1")
    slow = fn(x.to("vulkan"), w.to("vulkan"), b.to("vulkan")).cpu()
    torch.testing.assert_close(fast, slow, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("xshape,cout,kernel,stride,padding,output_padding,groups", [
    ((2, 32, 4, 5, 6), 32, (2, 2, 2), (2, 2, 2), (0, 0, 0), (0, 0, 0), 1),       # the x2 up-convolution of a 3-D U-Net
    ((1, 64, 3, 6, 6), 32, (3, 3, 3), (1, 1, 1), (1, 1, 1), (0, 0, 0), 1),
    ((2, 32, 4, 5, 5), 48, (3, 3, 2), (2, 1, 2), (1, 1, 0), (1, 0, 1), 1),       # output padding, mixed strides
    ((1, 64, 3, 5, 5), 64, (2, 3, 3), (1, 2, 1), (0, 1, 1), (0, 1, 0), 2),       # two groups
])
def test_conv_transpose3d_on_the_tensor_core_kernels(xshape, cout, kernel, stride, padding, output_padding, groups, monkeypatch):
    monkeypatch.setenv("B200_CONV3D_DECOMPOSE", "1")
    gen = torch.Generator().manual_seed(sum(xshape) + cout + 5)
    x = torch.randn(*xshape, generator=gen).numpy()
    w = (torch.randn(xshape[1], cout // groups, *kernel, generator=gen) / np.sqrt(xshape[1] // groups * np.prod(kernel))).numpy()
    b = torch.randn(cout, generator=gen).numpy()
    okw = dict(stride=stride, padding=padding, dilation=1, output_padding=output_padding, transposed=True, groups=groups)
    want = convnd_oracle.forward(x, w, b, **okw)
    got = b200conv.convnd_forward(x, w, b, **okw)
    assert b200conv.last_kernel().startswith("conv_transpose3d_forward")
    assert got.shape == want.shape and oracle.rel_l2(got, want) <= 2e-5
    grad = torch.randn(want.shape, generator=gen).numpy()
    for g, e in zip(b200conv.convnd_backward(grad, x, w, **okw), convnd_oracle.backward(grad, x, w, **okw)):
        assert oracle.rel_l2(g, e) <= 2e-5
    assert b200conv.device_status() == 0
    # and through the operator with autograd
    tkw = dict(stride=stride, padding=padding, output_padding=output_padding, groups=groups)
    _check_autograd(lambda xx, ww, bb: F.conv_transpose3d(xx, ww, bb, **tkw), (torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b)))


@pytest.mark.parametrize("xshape,cout,kernel,stride,padding,groups", [
    ((2, 3, 6, 20, 20), 24, (3, 5, 5), (1, 2, 2), (1, 2, 2), 1),      # a video stem: three input channels
    ((2, 8, 5, 12, 12), 8, (3, 3, 3), (1, 1, 1), (1, 1, 1), 2),       # four channels per group
    ((1, 12, 4, 9, 9), 40, (2, 3, 3), (2, 1, 1), (0, 1, 1), 1),
])
def test_conv3d_narrow_layers_through_the_decomposition(xshape, cout, kernel, stride, padding, groups, monkeypatch):
    """Fewer than 16 channels per group: the 2-D candidates per depth tap into a scratch, added into the result."""
    monkeypatch.setenv("B200_CONV3D_DECOMPOSE", "1")
    gen = torch.Generator().manual_seed(sum(xshape) + cout)
    x = torch.randn(*xshape, generator=gen).numpy()
    w = (torch.randn(cout, xshape[1] // groups, *kernel, generator=gen) * 0.1).numpy()
    b = torch.randn(cout, generator=gen).numpy()
    okw = dict(stride=stride, padding=padding, dilation=1, groups=groups)
    want = convnd_oracle.forward(x, w, b, **okw)
    got = b200conv.convnd_forward(x, w, b, **okw)
    assert b200conv.last_kernel().startswith("conv3d_forward") and oracle.rel_l2(got, want) <= 2e-5
    grad = torch.randn(want.shape, generator=gen).numpy()
    for g, e in zip(b200conv.convnd_backward(grad, x, w, **okw), convnd_oracle.backward(grad, x, w, **okw)):
        assert oracle.rel_l2(g, e) <= 2e-5
