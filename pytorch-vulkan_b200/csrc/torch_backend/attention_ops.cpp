// Scaled dot-product attention on PrivateUse1, the two layers the reference registers:
//   torch_vulkan::attention_forward / attention_backward (csrc/ops/attention.cpp:16-34): [batch, tokens, dim] operands, a
//     mask of the scores' shape that is empty, FP32 (additive) or bool (false hides the key), the saved log-sum-exp, and a
//     backward that also returns the gradient of the additive mask.  The Python module torch_vulkan.attention routes
//     F.scaled_dot_product_attention here.
//   aten::_scaled_dot_product_flash_attention_for_cpu and its backward (:36-43), with their shape checks and messages:
//     [B, H, T, D] operands reshaped to B*H batches, a 2-D or 4-D additive FP32 mask expanded to the scores' shape (:38).
// Operands are made contiguous and handed to b200_attention_forward / _backward.  Dropout draws from the backend's
// Philox stream (seed from torch_vulkan.manual_seed, offset advanced per call), whose four state words travel from
// the forward to the backward operator as a CPU tensor, as in the reference (attention.cpp:17-18,25).
#include <torch/library.h>

#include <array>
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

struct Workspace {
  at::Tensor hold;
  size_t bytes;
  Workspace(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, bool backward, const at::TensorOptions& opts) {
    bytes = b200_attention_workspace(batch, tq, tk, d, dv, backward ? 1 : 0);
    hold = at::empty({(int64_t)(bytes / 4) + 1}, opts);
  }
};

// ---- [batch, tokens, dim] operators ---------------------------------------------------------------------------------
int mask_kind(const at::Tensor& q, const at::Tensor& k, const at::Tensor& mask) {
  if (!mask.defined() || !mask.numel()) return B200_MASK_NONE;
  TORCH_CHECK(mask.sizes() == at::IntArrayRef({q.size(0), q.size(1), k.size(1)}) &&
                  (mask.scalar_type() == at::kFloat || mask.scalar_type() == at::kBool),
              "attention mask shape/dtype mismatch");
  return mask.scalar_type() == at::kBool ? B200_MASK_BYTES : B200_MASK_ADDITIVE;
}

void check3(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& mask, double dropout) {
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.size(0) == k.size(0) && k.size(0) == v.size(0) &&
                  q.size(2) == k.size(2) && k.size(1) == v.size(1),
              "attention dimensions mismatch");
  TORCH_CHECK(q.scalar_type() == at::kFloat && k.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat,
              "Vulkan attention requires FP32 input");
  TORCH_CHECK(q.device() == k.device() && k.device() == v.device() && (!mask.defined() || !mask.numel() || mask.device() == q.device()),
              "attention devices mismatch");
  TORCH_CHECK(dropout >= 0 && dropout <= 1, "invalid attention dropout");
}

// The four words of the random stream as the CPU int64 tensor the operator pair hands from forward to backward
// (attention.cpp:18 of the reference); zeros when no stream is drawn from.
at::Tensor rng_metadata(const std::array<uint32_t, 4>& state = {0, 0, 0, 0}) {
  auto t = at::empty({4}, at::TensorOptions().dtype(at::kLong).device(at::kCPU));
  for (int i = 0; i < 4; ++i) t.data_ptr<int64_t>()[i] = state[i];
  return t;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> attention_forward3(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                                                  const at::Tensor& mask, double dropout, bool causal, double scale) {
  check3(q, k, v, mask, dropout);
  const int kind = mask_kind(q, k, mask);
  const int64_t batch = q.size(0), tq = q.size(1), tk = k.size(1), d = q.size(2), dv = v.size(2);
  auto out = at::empty({batch, tq, dv}, q.options().memory_format(at::MemoryFormat::Contiguous));
  auto lse = at::empty({batch, tq}, q.options().memory_format(at::MemoryFormat::Contiguous));
  // a stream is reserved exactly when the reference reserves one (attention.cpp:17): a quarter block per score
  std::array<uint32_t, 4> state = {0, 0, 0, 0};
  if (dropout > 0 && dropout < 1) state = reserve_random_blocks(((uint64_t)batch * tq * tk + 3) / 4);
  if (!lse.numel()) return {out, lse, rng_metadata(state)};
  if (!out.numel()) {  // no value features: nothing to weigh, the reference reports a zero log-sum-exp (attention.cpp:20)
    lse.zero_();
    return {out, lse, rng_metadata(state)};
  }
  const at::Tensor qc = packed(q), kc = packed(k), vc = packed(v), mc = kind ? packed(mask) : at::Tensor();
  Workspace ws(batch, tq, tk, d, dv, false, q.options());
  B200_TORCH_CHECK(b200_attention_forward(batch, tq, tk, d, dv, qc.const_data_ptr<float>(), kc.const_data_ptr<float>(),
                                          vc.const_data_ptr<float>(), kind ? mc.const_data_ptr() : nullptr, kind, causal ? 1 : 0,
                                          (float)scale, (float)dropout, state.data(), out.data_ptr<float>(), lse.data_ptr<float>(),
                                          ws.hold.data_ptr(), ws.bytes, backend_stream()));
  return {out, lse, rng_metadata(state)};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> attention_backward3(const at::Tensor& grad, const at::Tensor& q,
                                                                               const at::Tensor& k, const at::Tensor& v,
                                                                               const at::Tensor& mask, const at::Tensor& out,
                                                                               const at::Tensor& lse, double dropout, bool causal,
                                                                               double scale, const at::Tensor& rng) {
  TORCH_CHECK(rng.device().is_cpu() && rng.scalar_type() == at::kLong && rng.numel() == 4 && rng.is_contiguous(),
              "Invalid attention RNG metadata");
  check3(q, k, v, mask, dropout);
  TORCH_CHECK(grad.sizes() == out.sizes() && out.dim() == 3 && out.size(0) == q.size(0) && out.size(1) == q.size(1) &&
                  out.size(2) == v.size(2) && lse.sizes() == q.sizes().slice(0, 2),
              "attention backward shape mismatch");
  const int kind = mask_kind(q, k, mask);
  const int64_t batch = q.size(0), tq = q.size(1), tk = k.size(1), d = q.size(2), dv = v.size(2);
  const auto dense = [](const at::Tensor& like) { return like.options().memory_format(at::MemoryFormat::Contiguous); };
  auto dq = at::empty(q.sizes(), dense(q)), dk = at::empty(k.sizes(), dense(k)), dvalue = at::empty(v.sizes(), dense(v));
  auto dm = at::empty({batch, tq, tk}, dense(q));
  std::array<uint32_t, 4> state;
  for (int i = 0; i < 4; ++i) state[i] = (uint32_t)rng.const_data_ptr<int64_t>()[i];
  const at::Tensor gc = packed(grad), qc = packed(q), kc = packed(k), vc = packed(v), oc = packed(out), lc = packed(lse),
                   mc = kind ? packed(mask) : at::Tensor();
  Workspace ws(batch, tq, tk, d, dv, true, q.options());
  const auto ptr = [](const at::Tensor& t) { return t.numel() ? t.const_data_ptr<float>() : nullptr; };
  const auto out_ptr = [](at::Tensor& t) { return t.numel() ? t.data_ptr<float>() : nullptr; };
  // the entry point zero-fills whatever gradient has elements when a dimension is empty; it wants non-null results
  static float placeholder;
  const auto want = [&](at::Tensor& t) { float* p = out_ptr(t); return p ? p : &placeholder; };
  B200_TORCH_CHECK(b200_attention_backward(batch, tq, tk, d, dv, ptr(gc), ptr(qc), ptr(kc), ptr(vc), kind ? mc.const_data_ptr() : nullptr,
                                           kind, ptr(oc), ptr(lc), causal ? 1 : 0, (float)scale, (float)dropout, state.data(), want(dq),
                                           want(dk), want(dvalue), out_ptr(dm), ws.hold.data_ptr(), ws.bytes, backend_stream()));
  return {dq, dk, dvalue, dm};
}

// ---- the flash-attention-for-CPU operator pair ------------------------------------------------------------------------
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

// The mask as a dense [B*H, Tq, Tk] tensor, or an empty one.
at::Tensor flash_mask(const at::Tensor& q, const at::Tensor& k, const std::optional<at::Tensor>& mask) {
  if (!mask || !mask->defined()) return at::empty({0}, q.options());
  TORCH_CHECK(mask->scalar_type() == at::kFloat,
              "scaled_dot_product_attention_flash_attention: Attention mask is the same data type as query");
  TORCH_CHECK(mask->dim() == 2 || mask->dim() == 4, "scaled_dot_product_attention_flash_attention: Attention mask dim in {2, 4}");
  TORCH_CHECK(mask->device() == q.device(), "attention mask device mismatch");
  return packed(mask->expand({q.size(0), q.size(1), q.size(2), k.size(2)})).view({q.size(0) * q.size(1), q.size(2), k.size(2)});
}

at::Tensor heads_as_batches(const at::Tensor& t) { return packed(t).view({t.size(0) * t.size(1), t.size(2), t.size(3)}); }

std::tuple<at::Tensor, at::Tensor> flash_forward(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double dropout, bool causal,
                                                 const std::optional<at::Tensor>& mask, std::optional<double> scale) {
  check(q, k, v, dropout);
  auto [out, lse, rng] = attention_forward3(heads_as_batches(q), heads_as_batches(k), heads_as_batches(v), flash_mask(q, k, mask), 0,
                                            causal, scale.value_or(1.0 / std::sqrt((double)q.size(3))));
  // rows with every key hidden: this operator returns 0 for them, not -inf (attention.cpp, cpu_flash_forward_native)
  B200_TORCH_CHECK(b200_attention_lse_finite(lse.numel() ? lse.data_ptr<float>() : nullptr, lse.numel(), backend_stream()));
  return {out.view({q.size(0), q.size(1), q.size(2), v.size(3)}), lse.view({q.size(0), q.size(1), q.size(2)})};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> flash_backward(const at::Tensor& grad, const at::Tensor& q, const at::Tensor& k,
                                                              const at::Tensor& v, const at::Tensor& out, const at::Tensor& lse,
                                                              double dropout, bool causal, const std::optional<at::Tensor>& mask,
                                                              std::optional<double> scale) {
  if (!grad.defined()) return {at::Tensor(), at::Tensor(), at::Tensor()};
  check(q, k, v, dropout);
  const int64_t batch = q.size(0) * q.size(1), tq = q.size(2);
  TORCH_CHECK(grad.sizes() == out.sizes() && out.dim() == 4 && out.size(2) == tq && out.size(3) == v.size(3) && lse.numel() == batch * tq,
              "attention backward shape mismatch");
  auto [dq, dk, dvalue, dm] = attention_backward3(heads_as_batches(grad), heads_as_batches(q), heads_as_batches(k), heads_as_batches(v),
                                                  flash_mask(q, k, mask), heads_as_batches(out), packed(lse).view({batch, tq}), 0, causal,
                                                  scale.value_or(1.0 / std::sqrt((double)q.size(3))), rng_metadata());
  return {dq.view(q.sizes()), dk.view(k.sizes()), dvalue.view(v.sizes())};
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(torch_vulkan, m) {
  m.def("attention_forward(Tensor q, Tensor k, Tensor v, Tensor mask, float dropout, bool causal, float scale) -> (Tensor, Tensor, Tensor)");
  m.def("attention_backward(Tensor grad, Tensor q, Tensor k, Tensor v, Tensor mask, Tensor output, Tensor lse, float dropout, "
        "bool causal, float scale, Tensor state) -> (Tensor, Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(torch_vulkan, PrivateUse1, m) {
  m.impl("attention_forward", &attention_forward3);
  m.impl("attention_backward", &attention_backward3);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_scaled_dot_product_flash_attention_for_cpu", &flash_forward);
  m.impl("_scaled_dot_product_flash_attention_for_cpu_backward", &flash_backward);
}

}  // namespace torch_vulkan
