"""The PrivateUse1 ("vulkan") extension: the reference's own conv/mm/runtime tests restated
against the drop-in package (reference: tests/test_convolution.py, tests/test_conv_universality.py,
tests/test_conv_dispatch.py:183-208,336-342, tests/test_fused_addmm.py, tests/test_direct_mm_out.py,
tests/test_complete_runtime.py, tests/test_fp32_contracts.py:126-143)."""
import pytest
import torch
import torch.nn.functional as F

import torch_vulkan

gpu = pytest.mark.gpu


def test_backend_registers_the_overrideable_pair_and_device_module():
    # tests/test_convolution.py:15-20 of the reference
    for op in ("aten::convolution_overrideable", "aten::convolution_backward_overrideable", "aten::mm", "aten::addmm"):
        assert torch._C._dispatch_has_kernel_for_dispatch_key(op, "PrivateUse1"), op
    assert torch.device("vulkan").type == "vulkan"
    assert torch.vulkan is torch_vulkan
    for name in ("is_available", "is_hardware_accelerated", "device_name", "synchronize", "performance_options",
                 "conv_dispatch_stats", "clear_conv_dispatch_cache", "cache_stats", "queue_stats", "gpu_timing_stats",
                 "execution_stats", "reset_execution_stats", "Stream", "Event", "manual_seed", "current_stream",
                 "default_stream", "set_stream", "device_count", "current_device"):
        assert hasattr(torch_vulkan, name), name
    assert set(torch_vulkan.performance_options()) >= {"gpu_resident", "deferred_submissions",
                                                       "adamw_multitensor_requested"}
    with pytest.raises(RuntimeError, match="logical device 0"):
        torch_vulkan.synchronize("vulkan:17")


@gpu
@pytest.mark.parametrize("shape,channels,kernel,stride,padding,dilation,groups,bias", [
    ((2, 3, 9, 11), 4, 3, 1, 1, 1, 1, True),
    ((1, 2, 11, 12), 3, 3, 2, 1, 1, 1, False),
    ((2, 4, 8, 7), 6, 3, 1, 2, 2, 2, True),
    ((1, 8, 8, 8), 8, 1, 1, 0, 1, 8, True),
    ((2, 64, 20, 20), 64, 3, 1, 1, 1, 1, True),   # large enough for the tcgen05 kernels
])
def test_conv2d_forward_backward_through_autograd(shape, channels, kernel, stride, padding, dilation, groups, bias):
    torch.manual_seed(72)
    inp = torch.randn(*shape, requires_grad=True)
    weight = torch.randn(channels, shape[1] // groups, kernel, kernel, requires_grad=True)
    b = torch.randn(channels, requires_grad=True) if bias else None
    out = F.conv2d(inp, weight, b, stride, padding, dilation, groups)
    grad = torch.randn_like(out)
    refs = (inp, weight, b) if b is not None else (inp, weight)
    cpu_grad = torch.autograd.grad(out, refs, grad_outputs=grad)
    x_vk = inp.detach().to("vulkan").requires_grad_()
    w_vk = weight.detach().to("vulkan").requires_grad_()
    b_vk = b.detach().to("vulkan").requires_grad_() if b is not None else None
    out_vk = F.conv2d(x_vk, w_vk, b_vk, stride, padding, dilation, groups)
    assert out_vk.device.type == "vulkan"
    torch.testing.assert_close(out_vk.cpu(), out, rtol=2e-4, atol=3e-4)
    vg = (x_vk, w_vk, b_vk) if b_vk is not None else (x_vk, w_vk)
    gradients = torch.autograd.grad(out_vk, vg, grad_outputs=grad.to("vulkan"))
    for actual, expected in zip(gradients, cpu_grad):
        assert actual.device.type == "vulkan"
        torch.testing.assert_close(actual.cpu(), expected, rtol=3e-4, atol=3e-4)
    assert torch_vulkan.execution_stats()["cpu_fallback_calls"] == 0
    assert torch_vulkan.device_status() == 0


@gpu
@pytest.mark.parametrize("layout", ["transpose", "channels_last", "slice", "offset", "broadcast"])
@pytest.mark.parametrize("algorithm", ["direct", "optimized", "auto"])
def test_strided_views_and_output_masks(layout, algorithm, monkeypatch):
    monkeypatch.setenv("TORCH_VULKAN_CONV_BACKWARD_ALGO", algorithm)
    torch.manual_seed(700)
    def view(t):
        if layout == "transpose": return t.transpose(2, 3)
        if layout == "channels_last": return t.contiguous(memory_format=torch.channels_last)
        if layout == "slice": return t[:, :, 1::2, ::2]
        if layout == "offset": return t[1:]
        return t[:1].expand(3, -1, -1, -1)
    base = torch.randn(3, 6, 13, 15)
    weight_base = torch.randn(10, 3, 3, 5)
    bias_base = torch.randn(20)
    x, xv = view(base), view(base.to("vulkan"))   # views applied after the transfer: device strides survive
    w, wv = weight_base.transpose(2, 3), weight_base.to("vulkan").transpose(2, 3)
    b, bv = bias_base[1::2], bias_base.to("vulkan")[1::2]
    args = ([1, 2], [2, 1], [1, 1], 2)
    ref = F.conv2d(x, w, b, *args)
    out = F.conv2d(xv, wv, bv, *args)
    torch.testing.assert_close(out.cpu(), ref, atol=4e-4, rtol=3e-4)
    grad_base = torch.randn(*ref.shape[:-1], ref.shape[-1] * 2)
    grad, gradv = grad_base[..., 1::2], grad_base.to("vulkan")[..., 1::2]
    def backward(go, inp, wt, mask):
        return torch.ops.aten.convolution_backward.default(go, inp, wt, [10], args[0], args[1], args[2], False,
                                                           [0, 0], 2, mask)
    for mask in ([True, True, True], [True, False, False], [False, True, False], [False, False, True]):
        expected = backward(grad, x, w, mask)
        actual = backward(gradv, xv, wv, mask)
        for enabled, a, e in zip(mask, actual, expected):
            if enabled:
                torch.testing.assert_close(a.cpu(), e, atol=5e-4, rtol=4e-4)
            else:
                assert a is None


@gpu
def test_dispatch_stats_env_controls_and_rejections(monkeypatch):
    x = torch.randn(2, 64, 16, 16).to("vulkan")
    w = torch.randn(64, 64, 3, 3).to("vulkan")
    torch_vulkan.clear_conv_dispatch_cache()
    F.conv2d(x, w, padding=1)
    stats = torch_vulkan.conv_dispatch_stats()
    assert stats.get("selected_forward_tiled_tcgen05", 0) == 1, stats
    monkeypatch.setenv("TORCH_VULKAN_CONV_ALGO", "direct")
    F.conv2d(x, w, padding=1)
    assert torch_vulkan.conv_dispatch_stats().get("selected_forward_direct", 0) == 1
    monkeypatch.setenv("TORCH_VULKAN_CONV_ALGO", "winograd")
    with pytest.raises(RuntimeError, match="incompatible|exceeds"):
        F.conv2d(torch.randn(1, 2, 9, 9).to("vulkan"), torch.randn(3, 2, 3, 5).to("vulkan"))
    monkeypatch.setenv("TORCH_VULKAN_CONV_ALGO", "bogus")
    with pytest.raises(RuntimeError, match="invalid algorithm"):
        F.conv2d(x, w, padding=1)
    monkeypatch.delenv("TORCH_VULKAN_CONV_ALGO")
    monkeypatch.setenv("TORCH_VULKAN_CONV_WORKSPACE_MB", "5000")
    with pytest.raises(RuntimeError, match="WORKSPACE_MB"):
        F.conv2d(x, w, padding=1)
    monkeypatch.delenv("TORCH_VULKAN_CONV_WORKSPACE_MB")
    # tests/test_conv_universality.py:96-101: effective kernel larger than the padded input
    with pytest.raises(RuntimeError):
        F.conv2d(torch.randn(1, 2, 2, 2).to("vulkan"), torch.randn(3, 2, 3, 3).to("vulkan"), stride=2)
    # tests/test_conv_dispatch.py:336-342
    with pytest.raises(RuntimeError, match="int32 coordinates"):
        F.conv2d(torch.randn(1, 1, 4, 4).to("vulkan"), torch.randn(1, 1, 1, 1).to("vulkan"), stride=(2 ** 31, 1))
    with pytest.raises(RuntimeError):
        torch.zeros(1, device="vulkan:17")


@gpu
def test_autotuner_times_candidates_once_and_reuses_the_plan(monkeypatch):
    # tests/test_conv_dispatch.py:115-160 of the reference: the first call of a geometry tunes and caches,
    # repeats hit the cache, a different memory layout is a different plan, results stay correct
    monkeypatch.setenv("TORCH_VULKAN_CONV_AUTOTUNE", "1")
    torch.manual_seed(3)
    xc, wc = torch.randn(2, 32, 12, 12) * 0.2, torch.randn(32, 32, 3, 3) * 0.2
    x = xc.to("vulkan").requires_grad_()
    w = wc.to("vulkan").requires_grad_()
    torch_vulkan.clear_conv_dispatch_cache()
    y = F.conv2d(x, w, padding=1)
    stats = torch_vulkan.conv_dispatch_stats()
    assert stats["misses"] == 1 and stats["tunes"] == 1 and stats["hits"] == 0 and stats["entries"] == 1, stats
    assert stats["candidates_timed"] >= 2, stats
    assert stats.get("candidates_timed_forward_tiled_tcgen05", 0) == 1, stats
    F.conv2d(x, w, padding=1)
    stats = torch_vulkan.conv_dispatch_stats()
    assert stats["hits"] == 1 and stats["tunes"] == 1 and stats["entries"] == 1, stats
    go = torch.randn(2, 32, 12, 12) * 0.3
    y.backward(go.to("vulkan"))   # dInput and dWeight tune separately
    stats = torch_vulkan.conv_dispatch_stats()
    assert stats["tunes"] == 3 and stats["entries"] == 3, stats
    torch.testing.assert_close(y.cpu(), F.conv2d(xc, wc, padding=1), atol=3e-5, rtol=4e-4)
    xr, wr = xc.clone().requires_grad_(), wc.clone().requires_grad_()
    F.conv2d(xr, wr, padding=1).backward(go)
    torch.testing.assert_close(x.grad.cpu(), xr.grad, atol=5e-5, rtol=5e-4)
    torch.testing.assert_close(w.grad.cpu(), wr.grad, atol=5e-5, rtol=5e-4)
    F.conv2d(x.detach().contiguous(memory_format=torch.channels_last), w.detach(), padding=1)
    stats = torch_vulkan.conv_dispatch_stats()
    assert stats["misses"] == 4 and stats["entries"] == 4, stats   # another layout class: another plan
    monkeypatch.setenv("TORCH_VULKAN_CONV_AUTOTUNE", "2")
    with pytest.raises(RuntimeError, match="AUTOTUNE"):
        F.conv2d(x, w, padding=1)


@gpu
def test_mm_addmm_and_copies():
    torch.manual_seed(3)
    a, b = torch.randn(70, 33), torch.randn(50, 33)
    av, bv = a.to("vulkan"), b.to("vulkan")
    torch.testing.assert_close(torch.mm(av, bv.t()).cpu(), a @ b.t(), rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(torch.mm(torch.tensor([[1., 2.], [3., 4.]]).to("vulkan"),
                                        torch.tensor([[5., 6.], [7., 8.]]).to("vulkan")).cpu(),
                               torch.tensor([[19., 22.], [43., 50.]]))
    bias = torch.randn(50)
    for beta, alpha in ((1.0, 1.0), (0.0, 1.0), (0.5, -2.0)):
        got = torch.addmm(bias.to("vulkan"), av, bv.t(), beta=beta, alpha=alpha)
        torch.testing.assert_close(got.cpu(), torch.addmm(bias, a, b.t(), beta=beta, alpha=alpha), rtol=2e-4, atol=2e-4)
    out = torch.empty(0, device="vulkan")
    torch.mm(av, bv.t(), out=out)
    torch.testing.assert_close(out.cpu(), a @ b.t(), rtol=2e-4, atol=2e-4)
    assert torch.mm(torch.zeros(0, 4).to("vulkan"), torch.zeros(4, 5).to("vulkan")).shape == (0, 5)
    assert torch.equal(torch.mm(torch.zeros(3, 0).to("vulkan"), torch.zeros(0, 5).to("vulkan")).cpu(), torch.zeros(3, 5))
    # strided copies both ways, item(), zeros/full factories
    t = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)
    tv = t.to("vulkan")
    assert torch.equal(tv.transpose(0, 2).cpu(), t.transpose(0, 2))
    assert torch.equal(tv[:, 1:, ::2].contiguous().cpu(), t[:, 1:, ::2])
    tv[:, 0, :] = torch.ones(2, 4)
    t[:, 0, :] = 1
    assert torch.equal(tv.cpu(), t)
    assert tv[1, 2, 3].item() == 23.0
    assert torch.equal(torch.zeros(3, 5, device="vulkan").cpu(), torch.zeros(3, 5))
    assert torch.equal(torch.full((2, 2), 1.5, device="vulkan").cpu(), torch.full((2, 2), 1.5))
    assert torch_vulkan.execution_stats()["host_read_calls"] > 0


@gpu
def test_streams_events_and_channels_last_factory():
    # tests/test_complete_runtime.py:6-32 and tests/test_fp32_contracts.py:126-138 of the reference
    s = torch_vulkan.Stream()
    start, end = torch_vulkan.Event(enable_timing=True), torch_vulkan.Event(enable_timing=True)
    x = torch.randn(4, 32, 24, 24).to("vulkan")
    w = torch.randn(32, 32, 3, 3).to("vulkan")
    with s:
        start.record()
        y = F.conv2d(x, w, padding=1)
        end.record()
    end.synchronize()
    assert start.elapsed_time(end) >= 0.0
    assert end.query()
    torch_vulkan.synchronize()
    xc = torch.randn(2, 32, 10, 10).contiguous(memory_format=torch.channels_last)
    xv = xc.to("vulkan").requires_grad_()
    wv = w.detach().clone().requires_grad_()
    out = F.conv2d(xv, wv, padding=1)
    assert out.is_contiguous()  # always NCHW, like the reference
    ref = F.conv2d(xc, w.cpu(), padding=1)
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4)
    assert torch_vulkan.device_name().startswith("NVIDIA")
    assert torch_vulkan.is_hardware_accelerated()
