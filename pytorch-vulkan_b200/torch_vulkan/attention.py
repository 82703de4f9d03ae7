"""F.scaled_dot_product_attention on "vulkan" tensors, with a device-resident backward.

Mirrors the reference's module of the same name (torch_vulkan/attention.py there): the composite
aten::scaled_dot_product_attention is overridden at the backend's autograd key, so that the saved
tensors and the gradients belong to the two device operators torch_vulkan::attention_forward /
attention_backward (csrc/torch_backend/attention_ops.cpp here, csrc/ops/attention.cpp:16-34 there)
instead of the softmax/matmul decomposition.  Operands of any leading shape are flattened to
[batch, tokens, dim]; masks may be bool (False hides the key) or float32 (added to the scores; its
gradient is returned when it requires one); grouped-query attention repeats the key/value heads.
Dropout draws from the backend's counter-based stream (torch_vulkan.manual_seed).
"""
import math

import torch

__all__ = ["scaled_dot_product_attention"]


class _DeviceAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, dropout, causal, scale):
        out, lse, state = torch.ops.torch_vulkan.attention_forward(q, k, v, mask, dropout, causal, scale)
        ctx.save_for_backward(q, k, v, mask, out, lse, state)
        ctx.settings = (dropout, causal, scale)
        return out

    @staticmethod
    def backward(ctx, grad):
        q, k, v, mask, out, lse, state = ctx.saved_tensors
        dropout, causal, scale = ctx.settings
        dq, dk, dv, dmask = torch.ops.torch_vulkan.attention_backward(grad, q, k, v, mask, out, lse, dropout, causal, scale, state)
        return dq, dk, dv, (dmask if ctx.needs_input_grad[3] else None), None, None, None


def _flatten_leading(t, leading):
    """[*leading-broadcastable, rows, cols] -> [prod(leading), rows, cols]."""
    return t.expand(*leading, *t.shape[-2:]).reshape(math.prod(leading), *t.shape[-2:])


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None, enable_gqa=False):
    for t in (query, key, value):
        if t.dtype != torch.float32 or t.ndim < 2:
            raise RuntimeError("Vulkan attention currently requires FP32 tensors with rank >=2")
    if query.shape[-1] != key.shape[-1] or key.shape[-2] != value.shape[-2] or query.shape[-1] == 0:
        raise RuntimeError("Attention feature or sequence dimensions mismatch")
    if enable_gqa:
        if min(query.ndim, key.ndim, value.ndim) < 3 or key.shape[-3] != value.shape[-3] or query.shape[-3] % key.shape[-3]:
            raise RuntimeError("Invalid grouped-query attention head counts")
        heads, repeat = query.shape[-3], query.shape[-3] // key.shape[-3]

        def per_query_head(t):  # [..., kv_heads, S, E] -> [..., heads, S, E], each kv head serving `repeat` query heads
            widened = t.unsqueeze(-3).expand(*t.shape[:-2], repeat, *t.shape[-2:])
            return widened.reshape(*t.shape[:-3], heads, *t.shape[-2:])
        key, value = per_query_head(key), per_query_head(value)
    leading = torch.broadcast_shapes(query.shape[:-2], key.shape[:-2], value.shape[:-2])
    q, k, v = (_flatten_leading(t, leading) for t in (query, key, value))
    if attn_mask is None:
        mask = query.new_empty((0,))
    elif attn_mask.dtype in (torch.bool, torch.float32):
        mask = attn_mask.expand(*leading, q.shape[-2], k.shape[-2]).reshape(q.shape[0], q.shape[-2], k.shape[-2])
    else:
        raise RuntimeError("Attention mask must be bool or FP32")
    factor = float(scale) if scale is not None else 1.0 / math.sqrt(query.shape[-1])
    out = _DeviceAttention.apply(q, k, v, mask, float(dropout_p), bool(is_causal), factor)
    return out.reshape(*leading, q.shape[-2], v.shape[-1])


# The composite operator is replaced at the autograd key (training) and at the backend key (no_grad / inference).
_autograd_lib = torch.library.Library("aten", "IMPL", "AutogradPrivateUse1")
_autograd_lib.impl("scaled_dot_product_attention", scaled_dot_product_attention)
_backend_lib = torch.library.Library("aten", "IMPL", "PrivateUse1")
_backend_lib.impl("scaled_dot_product_attention", scaled_dot_product_attention)


@torch.library.register_fake("torch_vulkan::attention_forward")
def _forward_meta(q, k, v, mask, dropout, causal, scale):
    return (q.new_empty((q.shape[0], q.shape[1], v.shape[2])), q.new_empty(q.shape[:2]),
            torch.empty(4, dtype=torch.int64, device="cpu"))


@torch.library.register_fake("torch_vulkan::attention_backward")
def _backward_meta(grad, q, k, v, mask, out, lse, dropout, causal, scale, state):
    return q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape), q.new_empty((q.shape[0], q.shape[1], k.shape[1]))
