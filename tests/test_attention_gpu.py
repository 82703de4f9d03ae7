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
