"""Parity of the fused forward entry point (bias + residual + ReLU in the epilogue, optional
channels-last result) against PyTorch CPU FP64 on the same seeded inputs."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import b200conv
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-4


def _rand(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape, dtype=np.float32) * scale).astype(np.float32)


def _reference(x, w, b, res, relu, args):
    y = F.conv2d(torch.from_numpy(np.ascontiguousarray(x)).double(), torch.from_numpy(w).double(),
                 None if b is None else torch.from_numpy(b).double(), **args)
    if res is not None:
        y = y + torch.from_numpy(np.ascontiguousarray(res)).double()
    if relu:
        y = torch.relu(y)
    return y.numpy()


CASES = [
    # (xshape, cout, kernel, conv args): strip-kernel geometries (NCHW and channels-last results) ...
    ((2, 64, 14, 14), 64, (3, 3), dict(padding=(1, 1))),
    ((2, 32, 9, 11), 48, (3, 3), dict(padding=(1, 1))),              # ragged column tile
    ((1, 128, 12, 12), 256, (1, 1), dict()),
    ((2, 64, 15, 15), 96, (3, 3), dict(stride=(2, 2), padding=(1, 1))),
    ((2, 64, 8, 8), 64, (3, 3), dict(padding=(1, 1), groups=2)),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c[0])) + f"-co{c[1]}")
@pytest.mark.parametrize("channels_last", [False, True], ids=["nchw_out", "nhwc_out"])
@pytest.mark.parametrize("ops", ["bias_relu", "residual", "bias_residual_relu", "plain"])
def test_fused_forward_on_strip_geometries(case, channels_last, ops):
    xshape, cout, kernel, kw = case
    args = dict(stride=kw.get("stride", (1, 1)), padding=kw.get("padding", (0, 0)), dilation=kw.get("dilation", (1, 1)),
                groups=kw.get("groups", 1))
    g = oracle.geometry(xshape, cout, kernel, **args)
    seed = sum(xshape) + cout
    x, w = _rand(g.x_shape, seed), _rand(g.w_shape, seed + 1, 0.1)
    b = _rand((cout,), seed + 2) if "bias" in ops else None
    res = _rand(g.y_shape, seed + 3) if "residual" in ops else None
    if res is not None and channels_last:   # a channels-last residual for a channels-last result
        res = np.ascontiguousarray(res.transpose(0, 2, 3, 1)).transpose(0, 3, 1, 2)
    relu = "relu" in ops
    got = b200conv.conv2d_forward_fused(x, w, b, residual=res, relu=relu, channels_last=channels_last, algo="tc", **args)
    assert b200conv.last_kernel() == "tc_strip_forward_fused"
    assert b200conv.device_status() == 0
    want = _reference(x, w, b, res, relu, args)
    assert oracle.rel_l2(got, want) <= GATE
    if relu:
        assert (got >= 0).all()


def test_fused_forward_falls_back_to_an_elementwise_pass():
    # 8 -> 8 channels: CUDA-core candidate; NCHW result works, a channels-last one is declined
    x, w, b = _rand((2, 8, 10, 10), 1), _rand((8, 8, 3, 3), 2, 0.2), _rand((8,), 3)
    res = _rand((2, 8, 10, 10), 4)
    args = dict(stride=(1, 1), padding=(1, 1), dilation=(1, 1), groups=1)
    got = b200conv.conv2d_forward_fused(x, w, b, residual=res, relu=True, **args)
    assert not b200conv.last_kernel().startswith("tc_strip")
    assert oracle.rel_l2(got, _reference(x, w, b, res, True, args)) <= GATE
    with pytest.raises(b200conv.B200Error, match="incompatible"):
        b200conv.conv2d_forward_fused(x, w, b, channels_last=True, **args)


def test_fused_forward_matches_the_plain_entry_point_bit_for_bit_without_post_ops():
    x, w, b = _rand((2, 64, 12, 12), 7), _rand((64, 64, 3, 3), 8, 0.1), _rand((64,), 9)
    args = dict(stride=(1, 1), padding=(1, 1), dilation=(1, 1), groups=1)
    plain = b200conv.conv2d_forward(x, w, b, algo="tc", **args)
    fused = b200conv.conv2d_forward_fused(x, w, b, algo="tc", **args)
    np.testing.assert_array_equal(plain, fused)
    fused_cl = b200conv.conv2d_forward_fused(x, w, b, channels_last=True, algo="tc", **args)
    np.testing.assert_array_equal(plain, fused_cl)


@pytest.mark.parametrize("xshape,cout,kernel,kw", [
    ((2, 64, 14, 14), 64, (3, 3), dict(padding=(1, 1))),                       # strip kernel: channels-last written by the epilogue
    ((2, 64, 15, 15), 96, (3, 3), dict(stride=(2, 2), padding=(1, 1))),
    ((2, 6, 9, 7), 5, (3, 2), dict(padding=(1, 0), dilation=(1, 2))),           # small: CUDA-core candidate plus one elementwise pass
    ((1, 8, 10, 10), 8, (3, 3), dict(padding=(1, 1), groups=8)),
])
@pytest.mark.parametrize("channels_last_out", [False, True])
def test_fused_operator_under_the_torch_vulkan_namespace(xshape, cout, kernel, kw, channels_last_out):
    """torch.ops.torch_vulkan.conv2d_fused (and the torch_vulkan.conv2d_fused helper) against PyTorch CPU FP64."""
    import torch_vulkan
    gen = torch.Generator().manual_seed(sum(xshape) + cout)
    groups = kw.get("groups", 1)
    x = torch.randn(*xshape, generator=gen)
    w = torch.randn(cout, xshape[1] // groups, *kernel, generator=gen) * 0.1
    b = torch.randn(cout, generator=gen)
    want_plain = F.conv2d(x.double(), w.double(), b.double(), **kw)
    res = torch.randn(want_plain.shape, generator=gen)
    want = torch.relu(want_plain + res.double())
    xd = x.to("vulkan").contiguous(memory_format=torch.channels_last) if channels_last_out else x.to("vulkan")
    got = torch_vulkan.conv2d_fused(xd, w.to("vulkan"), b.to("vulkan"), res.to("vulkan"), relu=True, channels_last_out=channels_last_out,
                                    **kw)
    assert got.device.type == "vulkan" and got.shape == want.shape
    assert got.is_contiguous(memory_format=torch.channels_last if channels_last_out else torch.contiguous_format)
    assert oracle.rel_l2(got.cpu().numpy(), want.numpy()) <= GATE
    plain = torch.ops.torch_vulkan.conv2d_fused(x.to("vulkan"), w.to("vulkan"), None, None, False, list(kw.get("stride", (1, 1))),
                                                list(kw.get("padding", (0, 0))), list(kw.get("dilation", (1, 1))), groups, False)
    assert oracle.rel_l2(plain.cpu().numpy(), (want_plain - b.double().view(1, -1, 1, 1)).numpy()) <= GATE
    with pytest.raises(RuntimeError, match="residual must have the result's shape"):
        torch_vulkan.conv2d_fused(x.to("vulkan"), w.to("vulkan"), residual=x.to("vulkan")[:, :1], **kw)
