// ATen registrations on PrivateUse1 for scaled dot-product attention: the operator pair the
// reference registers (csrc/ops/attention.cpp:36-43), _scaled_dot_product_flash_attention_for_cpu and
// its backward, with its shape checks and messages (:39).  [B, H, T, D] operands are made
// contiguous and handed to b200_attention_forward / _backward as B*H batches; a 2-D or 4-D additive
// FP32 mask is expanded to the scores' shape as there (:38).  Dropout is not supported, as there.
#include <torch/library.h>

#include <cmath>
#include <optional>
#include <tuple>

#include "backend.h"

namespace torch_vulkan {
namespace {

at::Tensor packed(const at::Tensor& t) {
  if (t.is_contiguous()) return t;
  auto out = at::empty(t.sizes(), t.options());
  if (t.numel())
    B200_TORCH_CHECK(b200_gather_strided(out.data_ptr(), t.const_data_ptr(), (int)t.dim(), t.sizes().data(), t.strides().data(),
                                         (int)t.element_size(), backend_stream()));
  return out;
}

void check(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double dropout) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4,
              "scaled_dot_product_attention_flash_attention: Accept only 4 dims inputs shape of {B, H, T, K}");
  TORCH_CHECK(q.scalar_type() == at::kFloat && k.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat,
              "Vulkan attention requires FP32 input");
  TORCH_CHECK(dropout == 0, "scaled_dot_product_attention_flash_attention: Currently do not support dropout > 0");
  TORCH_CHECK(q.size(3) == v.size(3) && k.size(3) == v.size(3),
              "scaled_dot_product_attention_flash_attention: Q/K/V should have the same head size");
  TORCH_CHECK(q.sizes().slice(0, 2) == k.sizes().slice(0, 2) && q.sizes().slice(0, 2) == v.sizes().slice(0, 2) &&
                  k.size(2) == v.size(2),
              "attention batch/head/sequence mismatch");
}

// The mask as a dense [B, H, Tq, Tk] tensor, or undefined.
at::Tensor dense_mask(const at::Tensor& q, const at::Tensor& k, const std::optional<at::Tensor>& mask) {
  if (!mask || !mask->defined()) return at::Tensor();
  TORCH_CHECK(mask->scalar_type() == at::kFloat,
              "scaled_dot_product_attention_flash_attention: Attention mask is the same data type as query");
  TORCH_CHECK(mask->dim() == 2 || mask->dim() == 4, "scaled_dot_product_attention_flash_attention: Attention mask dim in {2, 4}");
  TORCH_CHECK(mask->device() == q.device(), "attention mask device mismatch");
  return packed(mask->expand({q.size(0), q.size(1), q.size(2), k.size(2)}));
}

struct Workspace {
  at::Tensor hold;
  size_t bytes;
  Workspace(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, bool backward, const at::TensorOptions& opts) {
    bytes = b200_attention_workspace(batch, tq, tk, d, dv, backward ? 1 : 0);
    hold = at::empty({(int64_t)(bytes / 4) + 1}, opts);
  }
};

std::tuple<at::Tensor, at::Tensor> attention_forward(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double dropout,
                                                     bool causal, const std::optional<at::Tensor>& mask, std::optional<double> scale) {
  check(q, k, v, dropout);
  const int64_t batch = q.size(0) * q.size(1), tq = q.size(2), tk = k.size(2), d = q.size(3), dv = v.size(3);
  const at::Tensor qc = packed(q), kc = packed(k), vc = packed(v), mc = dense_mask(q, k, mask);
  auto out = at::empty({q.size(0), q.size(1), tq, dv}, q.options());
  auto lse = at::empty({q.size(0), q.size(1), tq}, q.options());
  Workspace ws(batch, tq, tk, d, dv, false, q.options());
  B200_TORCH_CHECK(b200_attention_forward(batch, tq, tk, d, dv, qc.const_data_ptr<float>(), kc.const_data_ptr<float>(),
                                          vc.const_data_ptr<float>(), mc.defined() ? mc.const_data_ptr<float>() : nullptr,
                                          causal ? 1 : 0, (float)scale.value_or(1.0 / std::sqrt((double)d)), out.data_ptr<float>(),
                                          lse.data_ptr<float>(), ws.hold.data_ptr(), ws.bytes, backend_stream()));
  // rows with every key hidden: the reference's operator returns 0 for them, not -inf (attention.cpp, cpu_flash_forward_native)
  B200_TORCH_CHECK(b200_attention_lse_finite(lse.data_ptr<float>(), lse.numel(), backend_stream()));
  return {out, lse};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> attention_backward(const at::Tensor& grad, const at::Tensor& q, const at::Tensor& k,
                                                                  const at::Tensor& v, const at::Tensor& out, const at::Tensor& lse,
                                                                  double dropout, bool causal, const std::optional<at::Tensor>& mask,
                                                                  std::optional<double> scale) {
  if (!grad.defined()) return {at::Tensor(), at::Tensor(), at::Tensor()};
  check(q, k, v, dropout);
  const int64_t batch = q.size(0) * q.size(1), tq = q.size(2), tk = k.size(2), d = q.size(3), dv = v.size(3);
  TORCH_CHECK(grad.sizes() == out.sizes() && out.dim() == 4 && out.size(2) == tq && out.size(3) == dv && lse.numel() == batch * tq,
              "attention backward shape mismatch");
  const at::Tensor gc = packed(grad), qc = packed(q), kc = packed(k), vc = packed(v), oc = packed(out), lc = packed(lse),
                   mc = dense_mask(q, k, mask);
  auto dq = at::empty(q.sizes(), q.options()), dk = at::empty(k.sizes(), k.options()), dvalue = at::empty(v.sizes(), v.options());
  Workspace ws(batch, tq, tk, d, dv, true, q.options());
  B200_TORCH_CHECK(b200_attention_backward(batch, tq, tk, d, dv, gc.const_data_ptr<float>(), qc.const_data_ptr<float>(),
                                           kc.const_data_ptr<float>(), vc.const_data_ptr<float>(),
                                           mc.defined() ? mc.const_data_ptr<float>() : nullptr, oc.const_data_ptr<float>(),
                                           lc.const_data_ptr<float>(), causal ? 1 : 0,
                                           (float)scale.value_or(1.0 / std::sqrt((double)d)), dq.data_ptr<float>(),
                                           dk.data_ptr<float>(), dvalue.data_ptr<float>(), ws.hold.data_ptr(), ws.bytes,
                                           backend_stream()));
  return {dq, dk, dvalue};
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_scaled_dot_product_flash_attention_for_cpu", &attention_forward);
  m.impl("_scaled_dot_product_flash_attention_for_cpu_backward", &attention_backward);
}

}  // namespace torch_vulkan
