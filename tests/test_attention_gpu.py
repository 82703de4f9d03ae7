"""Scaled dot-product attention on the device against the FP64 oracle (C ABI) and against PyTorch
CPU through the PrivateUse1 operators the reference registers
(_scaled_dot_product_flash_attention_for_cpu and its backward, csrc/ops/attention.cpp:43 there)."""
import numpy as np
import pytest
import torch

import b200conv
import torch_vulkan  # noqa: F401  (registers the device)
from oracle import attention_oracle as att
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-4

CASES = [  # (batch, tq, tk, d, dv, causal, masked)
    (2, 5, 7, 8, 8, False, False), (3, 16, 16, 4, 6, True, False), (1, 9, 12, 16, 16, False, True),
    (2, 33, 33, 8, 8, True, True), (4, 1, 10, 8, 3, False, False),
    (4, 256, 256, 64, 64, False, False), (2, 512, 384, 64, 64, True, False), (3, 200, 300, 40, 72, False, True),
]


def _inputs(case):
    batch, tq, tk, d, dv, causal, masked = case
    rng = np.random.default_rng(sum(case[:5]))
    r = lambda *s: rng.standard_normal(s, dtype=np.float32)
    return r(batch, tq, d), r(batch, tk, d), r(batch, tk, dv), (r(batch, tq, tk) if masked else None), r(batch, tq, dv)


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_attention_through_the_c_abi(case):
    q, k, v, mask, grad = _inputs(case)
    causal = case[5]
    out, lse = b200conv.attention_forward(q, k, v, mask, causal)
    wout, wlse = att.forward(q, k, v, mask, causal)
    assert oracle.rel_l2(out, wout) <= GATE
    np.testing.assert_allclose(lse, wlse, rtol=1e-4, atol=1e-4)
    dq, dk, dv = b200conv.attention_backward(grad, q, k, v, out, lse, mask, causal)
    for got, want in zip((dq, dk, dv), att.backward(grad, q, k, v, wout, wlse, mask, causal)):
        assert oracle.rel_l2(got, want) <= 2 * GATE
    assert b200conv.device_status() == 0


def test_hidden_rows_and_empty_keys():
    q, k, v = (np.ones(s, np.float32) for s in ((1, 2, 4), (1, 3, 4), (1, 3, 2)))
    mask = np.zeros((1, 2, 3), np.float32)
    mask[0, 1] = -np.inf
    out, lse = b200conv.attention_forward(q, k, v, mask)
    assert np.isneginf(lse[0, 1]) and (out[0, 1] == 0).all() and np.isfinite(lse[0, 0])
    dq, dk, dv = b200conv.attention_backward(np.ones((1, 2, 2), np.float32), q, k, v, out, lse, mask)
    assert np.isfinite(dq).all() and (dq[0, 1] == 0).all()
    out, lse = b200conv.attention_forward(q, np.zeros((1, 0, 4), np.float32), np.zeros((1, 0, 2), np.float32))
    assert (out == 0).all() and np.isneginf(lse).all()


@pytest.mark.parametrize("causal,masked", [(False, False), (True, False), (False, True)])
def test_flash_attention_operator_pair(causal, masked):
    torch.manual_seed(5)
    q, k, v = torch.randn(2, 3, 40, 16), torch.randn(2, 3, 48 if not causal else 40, 16), torch.randn(2, 3, 48 if not causal else 40, 16)
    mask = torch.randn(2, 3, 40, k.size(2)) if masked else None
    grad = torch.randn(2, 3, 40, 16)

    def run(device):
        to = lambda t: None if t is None else t.to(device)
        out, lse = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(to(q), to(k), to(v), 0.0, causal, attn_mask=to(mask))
        grads = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu_backward(to(grad), to(q), to(k), to(v), out, lse, 0.0,
                                                                                    causal, attn_mask=to(mask))
        return (out, lse, *grads)
    for got, want in zip(run("vulkan"), run("cpu")):
        assert got.device.type == "vulkan"
        torch.testing.assert_close(got.cpu(), want, rtol=3e-4, atol=3e-4)
    with pytest.raises(RuntimeError, match="do not support dropout"):
        torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(q.to("vulkan"), k.to("vulkan"), v.to("vulkan"), 0.5, False)


def test_operator_returns_zero_log_sum_exp_for_rows_with_every_key_hidden():
    """The reference's operator replaces the -inf log-sum-exp of such rows with 0
    (csrc/ops/attention.cpp, cpu_flash_forward_native); its backward then sees probability 0 there."""
    torch.manual_seed(11)
    q, k, v = torch.randn(1, 2, 6, 8), torch.randn(1, 2, 5, 8), torch.randn(1, 2, 5, 8)
    mask = torch.zeros(1, 2, 6, 5)
    mask[0, 1, 3] = float("-inf")
    grad = torch.randn(1, 2, 6, 8)
    dev = lambda t: t.to("vulkan")
    out, lse = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(dev(q), dev(k), dev(v), 0.0, False, attn_mask=dev(mask))
    lse_h, out_h = lse.cpu(), out.cpu()
    assert torch.isfinite(lse_h).all() and lse_h[0, 1, 3] == 0 and (out_h[0, 1, 3] == 0).all()
    dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu_backward(dev(grad), dev(q), dev(k), dev(v), out, lse,
                                                                                    0.0, False, attn_mask=dev(mask))
    assert torch.isfinite(dq.cpu()).all() and (dq.cpu()[0, 1, 3] == 0).all()
    # the visible rows agree with the oracle on the same inputs
    wout, wlse = att.forward(q.reshape(2, 6, 8).numpy(), k.reshape(2, 5, 8).numpy(), v.reshape(2, 5, 8).numpy(),
                             mask.reshape(2, 6, 5).numpy(), False)
    keep = np.isfinite(wlse)
    np.testing.assert_allclose(lse_h.reshape(2, 6).numpy()[keep], wlse[keep], rtol=1e-4, atol=1e-4)
    with pytest.raises(RuntimeError, match="same head size"):
        torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(dev(q), dev(k), dev(torch.randn(1, 2, 5, 4)), 0.0, False)


@pytest.mark.parametrize("shape", [(2, 5, 7, 4, 6), (2, 137, 19, 8, 3), (2, 4, 141, 7, 129), (3, 128, 256, 64, 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_bool_masks_and_the_mask_gradient_through_the_c_abi(shape, causal):
    batch, tq, tk, d, dv = shape
    rng = np.random.default_rng(432 + tq)
    r = lambda *s: rng.standard_normal(s, dtype=np.float32)
    q, k, v, grad = r(batch, tq, d), r(batch, tk, d), r(batch, tk, dv), r(batch, tq, dv)
    keep = rng.random((batch, tq, tk)) > 0.3
    keep[:, 0] = False                        # a row with every key hidden
    out, lse = b200conv.attention_forward(q, k, v, keep, causal, scale=0.37)
    wout, wlse = att.forward(q, k, v, keep, causal, scale=0.37)
    assert oracle.rel_l2(out, wout) <= GATE and (out[:, 0] == 0).all() and np.isneginf(lse[:, 0]).all()
    np.testing.assert_allclose(lse, wlse, rtol=1e-4, atol=1e-4)
    for got, want in zip(b200conv.attention_backward(grad, q, k, v, out, lse, keep, causal, scale=0.37),
                         att.backward(grad, q, k, v, wout, wlse, keep, causal, scale=0.37)):
        assert np.isfinite(got).all() and oracle.rel_l2(got, want) <= 2 * GATE
    add = r(batch, tq, tk)
    out, lse = b200conv.attention_forward(q, k, v, add, causal, scale=0.37)
    wout, wlse = att.forward(q, k, v, add, causal, scale=0.37)
    got = b200conv.attention_backward(grad, q, k, v, out, lse, add, causal, scale=0.37, mask_grad=True)
    want = att.backward(grad, q, k, v, wout, wlse, add, causal, scale=0.37, mask_grad=True)
    assert len(got) == 4 and got[3].shape == (batch, tq, tk)
    for a, e in zip(got, want):
        assert oracle.rel_l2(a, e) <= 2 * GATE
    # the mask gradient is the score gradient before the scale: hidden (causal) keys get exactly zero
    if causal:
        i, j = np.arange(tq)[:, None], np.arange(tk)[None, :]
        assert (got[3][:, j > i] == 0).all()


@pytest.mark.parametrize("shape", [(2, 3, 5, 7, 4, 6), (1, 2, 137, 19, 8, 3), (2, 1, 4, 141, 7, 129)])
@pytest.mark.parametrize("kind", ["none", "causal", "bool", "float"])
def test_scaled_dot_product_attention_forward_backward(shape, kind):
    """The reference's tests/test_complete_attention.py:6-24 with its tolerances; the float mask has the scores' full
    shape here, the broadcast [1, 1, L, S] form is test_broadcast_float_mask_receives_its_gradient below."""
    import torch.nn.functional as F
    torch.manual_seed(432)
    b, h, l, s, d, e = shape
    q, k, v = [torch.randn(size, requires_grad=True) for size in [(b, h, l, d), (b, h, s, d), (b, h, s, e)]]
    mask = None
    if kind == "bool":
        mask = torch.rand(l, s) > .3
        mask[0] = False
    if kind == "float":
        mask = torch.randn(b, h, l, s, requires_grad=True)
    inputs = [x.detach().to("vulkan").requires_grad_() for x in (q, k, v)]
    mv = mask.detach().to("vulkan").requires_grad_(mask.requires_grad) if mask is not None else None
    a = F.scaled_dot_product_attention(q, k, v, mask, is_causal=kind == "causal", scale=.37)
    z = F.scaled_dot_product_attention(*inputs, mv, is_causal=kind == "causal", scale=.37)
    assert z.device.type == "vulkan"
    g = torch.randn_like(a)
    a.backward(g)
    z.backward(g.to("vulkan"))
    # rows whose keys are all hidden: PyTorch's CPU math path returns NaN there, the device operator zeros, as the reference's
    want = torch.nan_to_num(a.detach(), nan=0.0)
    torch.testing.assert_close(z.detach().cpu(), want, rtol=4e-4, atol=4e-5)
    for x, y in zip(inputs, (q, k, v)):
        torch.testing.assert_close(x.grad.cpu(), torch.nan_to_num(y.grad, nan=0.0), rtol=6e-4, atol=7e-5)
    if mask is not None and mask.requires_grad:
        torch.testing.assert_close(mv.grad.cpu(), mask.grad, rtol=6e-4, atol=7e-5)


def test_scaled_dot_product_attention_gqa_without_grad_and_rejections():
    import torch.nn.functional as F
    torch.manual_seed(3)
    q, k, v = torch.randn(2, 4, 7, 5), torch.randn(2, 2, 9, 5), torch.randn(2, 2, 9, 3)
    with torch.no_grad():
        got = F.scaled_dot_product_attention(q.to("vulkan"), k.to("vulkan"), v.to("vulkan"), enable_gqa=True)
    torch.testing.assert_close(got.cpu(), F.scaled_dot_product_attention(q, k, v, enable_gqa=True), rtol=3e-4, atol=3e-5)
    with pytest.raises(RuntimeError, match="invalid attention dropout"):
        torch.ops.torch_vulkan.attention_forward(q[0].to("vulkan"), q[0].to("vulkan"), q[0].to("vulkan"), torch.empty(0).to("vulkan"), 1.5, False, 1.0)
    # dropout_p = 1 drops every probability: zero output and zero gradients (tests/test_complete_attention.py:36-45 there)
    qd = q.to("vulkan").requires_grad_()
    full = F.scaled_dot_product_attention(qd, qd.detach(), qd.detach(), dropout_p=1.0)
    full.backward(torch.ones_like(full))
    assert (full.detach().cpu() == 0).all() and (qd.grad.cpu() == 0).all()
    with pytest.raises(RuntimeError, match="Attention mask must be bool or FP32"):
        F.scaled_dot_product_attention(q.to("vulkan"), q.to("vulkan"), q.to("vulkan"), attn_mask=torch.zeros(7, 7, dtype=torch.float64).to("vulkan"))
    with pytest.raises(RuntimeError, match="attention mask shape/dtype mismatch"):
        torch.ops.torch_vulkan.attention_forward(q[0].to("vulkan"), q[0].to("vulkan"), q[0].to("vulkan"), torch.zeros(4, 7, 6).to("vulkan"),
                                                 0.0, False, 1.0)


@pytest.mark.parametrize("batch,qlen,klen,dv", [(0, 3, 4, 5), (2, 0, 4, 5), (2, 3, 0, 5), (2, 3, 4, 0)])
def test_attention_empty_dimensions(batch, qlen, klen, dv):
    """tests/test_complete_attention.py:47-57 of the reference."""
    import torch.nn.functional as F
    q, k, v = torch.randn(batch, qlen, 7, requires_grad=True), torch.randn(batch, klen, 7, requires_grad=True), torch.randn(batch, klen, dv, requires_grad=True)
    inputs = [x.detach().to("vulkan").requires_grad_() for x in (q, k, v)]
    expected = F.scaled_dot_product_attention(q, k, v)
    actual = F.scaled_dot_product_attention(*inputs)
    expected.backward(torch.ones_like(expected))
    actual.backward(torch.ones_like(expected).to("vulkan"))
    torch.testing.assert_close(actual.cpu(), expected)
    for a, b in zip(inputs, (q, k, v)):
        torch.testing.assert_close(a.grad.cpu(), b.grad)


@pytest.mark.parametrize("shape", [(2, 5, 7, 4, 6), (2, 137, 19, 8, 3), (3, 128, 256, 64, 64)])
@pytest.mark.parametrize("p", [0.1, 0.35, 0.9])
def test_dropout_stream_through_the_c_abi(shape, p):
    """Forward and all gradients with dropout against the oracle drawing the same Philox stream (seed, offset)."""
    batch, tq, tk, d, dv = shape
    rng = np.random.default_rng(tq + tk)
    r = lambda *s: rng.standard_normal(s, dtype=np.float32)
    q, k, v, grad, add = r(batch, tq, d), r(batch, tk, d), r(batch, tk, dv), r(batch, tq, dv), r(batch, tq, tk)
    stream = (0x1234567887654321, 0xFFFFFFF0)       # the block counter carries into the high offset word
    out, lse = b200conv.attention_forward(q, k, v, add, True, scale=0.37, dropout=p, rng=stream)
    wout, wlse = att.forward(q, k, v, add, True, scale=0.37, dropout=p, rng=stream)
    assert oracle.rel_l2(out, wout) <= GATE
    np.testing.assert_allclose(lse, wlse, rtol=1e-4, atol=1e-4)
    got = b200conv.attention_backward(grad, q, k, v, out, lse, add, True, scale=0.37, mask_grad=True, dropout=p, rng=stream)
    want = att.backward(grad, q, k, v, wout, wlse, add, True, scale=0.37, mask_grad=True, dropout=p, rng=stream)
    for a, e in zip(got, want):
        assert oracle.rel_l2(a, e) <= 2 * GATE
    other, _ = b200conv.attention_forward(q, k, v, add, True, scale=0.37, dropout=p, rng=(stream[0], stream[1] + 1))
    assert not np.array_equal(other, out)


def test_scaled_dot_product_attention_with_dropout_is_seeded_and_consistent():
    """tests/test_complete_attention.py:36-45 of the reference: the same seed gives the same mask, and the gradient agrees
    with finite differences taken under that mask; here also with the oracle drawing the stream from offset 0."""
    import torch.nn.functional as F
    import torch_vulkan
    torch.manual_seed(1)
    q, k, v = (torch.randn(1, 2, 9, 8) for _ in range(3))
    dev = [t.to("vulkan").requires_grad_() for t in (q, k, v)]
    torch_vulkan.manual_seed(42)
    out = F.scaled_dot_product_attention(*dev, dropout_p=0.35)
    out.backward(torch.ones_like(out))
    torch_vulkan.manual_seed(42)
    again = F.scaled_dot_product_attention(*[t.detach() for t in dev], dropout_p=0.35)
    assert torch.equal(again.cpu(), out.detach().cpu())
    later = F.scaled_dot_product_attention(*[t.detach() for t in dev], dropout_p=0.35)        # the offset has advanced
    assert not torch.equal(later.cpu(), out.detach().cpu())
    n = lambda t: t.reshape(2, 9, 8).numpy()
    want, wlse = att.forward(n(q), n(k), n(v), dropout=0.35, rng=(42, 0))
    assert oracle.rel_l2(out.detach().cpu().reshape(2, 9, 8).numpy(), want) <= GATE
    grads = att.backward(np.ones((2, 9, 8), np.float32), n(q), n(k), n(v), want, wlse, dropout=0.35, rng=(42, 0))
    for g, e in zip(dev, grads):
        assert oracle.rel_l2(g.grad.cpu().reshape(2, 9, 8).numpy(), e) <= 2 * GATE


@pytest.mark.parametrize("shape,dims,keepdim", [((4, 5, 6), (1,), False), ((4, 5, 6), (0, 2), True), ((3, 1, 7, 9), None, False),
                                               ((2, 3, 4, 5, 6), (0, 1, 3), False), ((64, 300), (0,), False), ((5000,), (0,), False)])
def test_sum_over_a_dimension_list(shape, dims, keepdim):
    torch.manual_seed(3)
    x = torch.randn(*shape)
    want = x.double().sum() if dims is None else x.double().sum(dim=dims, keepdim=keepdim)
    xd = x.to("vulkan")
    got = xd.sum() if dims is None else xd.sum(dim=dims, keepdim=keepdim)
    assert got.device.type == "vulkan" and got.shape == want.shape
    torch.testing.assert_close(got.cpu().double(), want, rtol=1e-5, atol=1e-5)
    if len(shape) >= 2:        # a transposed (strided) view sums the same
        xt = xd.transpose(0, -1)
        torch.testing.assert_close(xt.sum(dim=0).cpu().double(), x.transpose(0, -1).double().sum(dim=0), rtol=1e-5, atol=1e-5)
    with pytest.raises(RuntimeError, match="only FP32"):
        torch.ones(3, dtype=torch.int64).to("vulkan").sum()


@pytest.mark.parametrize("gqa", [False, True])
def test_attention_broadcast_and_gqa_with_gradients(gqa):
    """tests/test_complete_attention.py:26-33 of the reference: broadcast batch, grouped-query heads, `.sum().backward()`."""
    import torch.nn.functional as F
    torch.manual_seed(8)
    q = torch.randn(2, 4, 7, 5, requires_grad=True)
    k = torch.randn(1, 2 if gqa else 4, 9, 5, requires_grad=True)
    v = torch.randn(2, 2 if gqa else 4, 9, 3, requires_grad=True)
    vs = [x.detach().to("vulkan").requires_grad_() for x in (q, k, v)]
    a = F.scaled_dot_product_attention(q, k, v, enable_gqa=gqa)
    b = F.scaled_dot_product_attention(*vs, enable_gqa=gqa)
    a.sum().backward()
    b.sum().backward()
    torch.testing.assert_close(b.detach().cpu(), a.detach(), rtol=3e-4, atol=3e-5)
    for x, y in zip(vs, (q, k, v)):
        torch.testing.assert_close(x.grad.cpu(), y.grad, rtol=5e-4, atol=5e-5)


def test_broadcast_float_mask_receives_its_gradient():
    """The float-mask case of tests/test_complete_attention.py:6-24 as the reference writes it: a [1, 1, L, S] mask that
    requires a gradient, broadcast over batch and heads."""
    import torch.nn.functional as F
    torch.manual_seed(432)
    b, h, l, s, d, e = 2, 3, 5, 7, 4, 6
    q, k, v = [torch.randn(size, requires_grad=True) for size in [(b, h, l, d), (b, h, s, d), (b, h, s, e)]]
    mask = torch.randn(1, 1, l, s, requires_grad=True)
    inputs = [x.detach().to("vulkan").requires_grad_() for x in (q, k, v)]
    mv = mask.detach().to("vulkan").requires_grad_()
    a = F.scaled_dot_product_attention(q, k, v, mask, scale=.37)
    z = F.scaled_dot_product_attention(*inputs, mv, scale=.37)
    g = torch.randn_like(a)
    a.backward(g)
    z.backward(g.to("vulkan"))
    torch.testing.assert_close(z.detach().cpu(), a.detach(), rtol=4e-4, atol=4e-5)
    for x, y in zip(inputs, (q, k, v)):
        torch.testing.assert_close(x.grad.cpu(), y.grad, rtol=6e-4, atol=7e-5)
    torch.testing.assert_close(mv.grad.cpu(), mask.grad, rtol=6e-4, atol=7e-5)
