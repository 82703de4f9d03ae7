// ATen registrations on PrivateUse1 for GroupNorm.  Host-side mirror of the reference's
// csrc/ops/group_norm.cpp: native_group_norm and native_group_norm_backward with its argument
// checks and messages (:80-92, :118-131), the empty-batch results (:93, :132) and undefined
// gradients for masked-off outputs.  Operands are made contiguous on the device first, as the
// reference packs them (:97-99, :134-135).  Where the reference falls back to PyTorch's CPU
// kernels (ineligible shapes, :94-96), this extension raises: it registers no host computation.
#include <torch/library.h>

#include <array>
#include <optional>
#include <tuple>

#include "backend.h"

namespace torch_vulkan {
namespace {

using Optional = std::optional<at::Tensor>;
using Three = std::tuple<at::Tensor, at::Tensor, at::Tensor>;

bool present(const Optional& t) { return t && t->defined(); }

at::Tensor packed(const at::Tensor& t) {
  if (t.is_contiguous()) return t;
  auto out = at::empty(t.sizes(), t.options());
  if (t.numel())
    B200_TORCH_CHECK(b200_gather_strided(out.data_ptr(), t.const_data_ptr(), (int)t.dim(), t.sizes().data(), t.strides().data(),
                                         (int)t.element_size(), backend_stream()));
  return out;
}

bool channel_vector(const Optional& v, const at::Tensor& x, int64_t c) {
  return !present(v) || (v->device() == x.device() && v->scalar_type() == at::kFloat && v->numel() == c);
}

Three group_norm(const at::Tensor& x, const Optional& weight, const Optional& bias, c10::SymInt N, c10::SymInt C, c10::SymInt HxW,
                 int64_t group, double eps) {
  const int64_t n = N.expect_int(), c = C.expect_int(), hw = HxW.expect_int();
  TORCH_CHECK(group > 0 && n >= 0 && c > 0 && hw > 0 && c % group == 0,
              "native_group_norm: invalid batch, channel, group or spatial dimensions");
  TORCH_CHECK(x.scalar_type() == at::kFloat, "Vulkan native_group_norm currently requires FP32");
  TORCH_CHECK(x.numel() == n * c * hw, "native_group_norm: input does not have N*C*HxW elements");
  TORCH_CHECK(channel_vector(weight, x, c), "native_group_norm: weight must have C float elements");
  TORCH_CHECK(channel_vector(bias, x, c), "native_group_norm: bias must have C float elements");
  auto out = at::empty(x.sizes(), x.options());
  auto mean = at::empty({n, group}, x.options());
  auto rstd = at::empty({n, group}, x.options());
  if (n == 0) return {out, mean, rstd};
  const at::Tensor xc = packed(x);
  const at::Tensor wc = present(weight) ? packed(*weight) : at::Tensor();
  const at::Tensor bc = present(bias) ? packed(*bias) : at::Tensor();
  B200_TORCH_CHECK(b200_group_norm_forward(n, c, hw, group, xc.const_data_ptr<float>(),
                                           wc.defined() ? wc.const_data_ptr<float>() : nullptr,
                                           bc.defined() ? bc.const_data_ptr<float>() : nullptr, (float)eps, out.data_ptr<float>(),
                                           mean.data_ptr<float>(), rstd.data_ptr<float>(), backend_stream()));
  return {out, mean, rstd};
}

Three group_norm_backward(const at::Tensor& grad, const at::Tensor& x, const at::Tensor& mean, const at::Tensor& rstd,
                          const Optional& weight, c10::SymInt N, c10::SymInt C, c10::SymInt HxW, int64_t group,
                          std::array<bool, 3> mask) {
  const int64_t n = N.expect_int(), c = C.expect_int(), hw = HxW.expect_int();
  TORCH_CHECK(group > 0 && n >= 0 && c > 0 && hw > 0 && c % group == 0, "native_group_norm_backward: invalid geometry");
  TORCH_CHECK(grad.sizes() == x.sizes() && mean.numel() == n * group && rstd.numel() == n * group,
              "native_group_norm_backward: input and saved statistic shape mismatch");
  TORCH_CHECK(x.scalar_type() == at::kFloat && grad.scalar_type() == at::kFloat && mean.scalar_type() == at::kFloat &&
                  rstd.scalar_type() == at::kFloat,
              "native_group_norm_backward: FP32 only");
  TORCH_CHECK(channel_vector(weight, x, c), "native_group_norm_backward: invalid gamma");
  at::Tensor dx, dw, db;
  if (n == 0) {
    if (mask[0]) dx = at::empty(x.sizes(), x.options());
    if (mask[1]) dw = at::empty({c}, x.options()).zero_();
    if (mask[2]) db = at::empty({c}, x.options()).zero_();
    return {dx, dw, db};
  }
  if (!mask[0] && !mask[1] && !mask[2]) return {dx, dw, db};
  const at::Tensor xc = packed(x), gc = packed(grad), mc = packed(mean), rc = packed(rstd);
  const at::Tensor wc = present(weight) ? packed(*weight) : at::Tensor();
  if (mask[0]) dx = at::empty(x.sizes(), x.options());
  if (mask[1]) dw = at::empty({c}, x.options());
  if (mask[2]) db = at::empty({c}, x.options());
  const size_t ws_bytes = b200_group_norm_workspace(n, c, hw, group);
  at::Tensor ws = at::empty({(int64_t)(ws_bytes + 3) / 4 + 1}, x.options());
  B200_TORCH_CHECK(b200_group_norm_backward(n, c, hw, group, gc.const_data_ptr<float>(), xc.const_data_ptr<float>(),
                                            mc.const_data_ptr<float>(), rc.const_data_ptr<float>(),
                                            wc.defined() ? wc.const_data_ptr<float>() : nullptr,
                                            mask[0] ? dx.data_ptr<float>() : nullptr, mask[1] ? dw.data_ptr<float>() : nullptr,
                                            mask[2] ? db.data_ptr<float>() : nullptr, ws.data_ptr(), ws_bytes, backend_stream()));
  return {dx, dw, db};
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("native_group_norm", &group_norm);
  m.impl("native_group_norm_backward", &group_norm_backward);
}

}  // namespace torch_vulkan
