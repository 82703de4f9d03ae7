// ATen registrations on PrivateUse1 for BatchNorm.  Host-side mirror of the reference's
// csrc/ops/batch_norm.cpp: the same eight operator names (:121-126), argument checks and
// messages (:9-20, :27-28, :88-92), empty save_mean / save_inv in evaluation mode (:37-38) and
// undefined gradients for masked-off outputs (:96).  Device work is b200_batch_norm_forward /
// b200_batch_norm_backward; nothing is computed on the host.
//
// One difference in layout: a dense channels-last input (4-D or 5-D) is consumed in place and its
// output / input gradient come back channels-last, where the reference first packs to the
// contiguous form and returns contiguous tensors (:30, :36).  Every other strided input is
// gathered to the contiguous form on the device first, as there.
#include <torch/library.h>

#include <algorithm>
#include <array>
#include <numeric>
#include <optional>
#include <tuple>
#include <vector>

#include "backend.h"

namespace torch_vulkan {
namespace {

using Optional = std::optional<at::Tensor>;
using Three = std::tuple<at::Tensor, at::Tensor, at::Tensor>;

bool present(const Optional& t) { return t && t->defined(); }

void check_tensor(const at::Tensor& t) {
  TORCH_CHECK(t.device().type() == c10::DeviceType::PrivateUse1 && t.scalar_type() == at::kFloat,
              "Vulkan BatchNorm supports FP32 Vulkan tensors only");
}
void check_vector(const at::Tensor& t, int64_t c) {
  check_tensor(t);
  TORCH_CHECK(t.dim() == 1 && t.numel() == c, "Vulkan BatchNorm expects a channel vector");
}
void check_input(const at::Tensor& x) {
  check_tensor(x);
  TORCH_CHECK(x.dim() >= 2 && x.dim() <= 8 && x.numel() > 0, "Vulkan BatchNorm requires nonempty rank 2 to 8 input");
}

// The memory format whose dense form the kernels can read in place, if the tensor has one.
std::optional<at::MemoryFormat> channels_last_format(const at::Tensor& x) {
  if (x.is_contiguous()) return std::nullopt;
  if (x.dim() == 4 && x.is_contiguous(at::MemoryFormat::ChannelsLast)) return at::MemoryFormat::ChannelsLast;
  if (x.dim() == 5 && x.is_contiguous(at::MemoryFormat::ChannelsLast3d)) return at::MemoryFormat::ChannelsLast3d;
  return std::nullopt;
}

at::Tensor dense(const at::Tensor& t, at::MemoryFormat format) {
  if (t.is_contiguous(format)) return t;
  auto out = at::empty(t.sizes(), t.options().memory_format(format));
  // the gather writes row-major over the extents it is given: hand it the dimensions in the
  // destination's memory order (largest stride first), with the source's strides permuted alike
  std::vector<int64_t> order(t.dim());
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return out.stride(a) > out.stride(b); });
  std::vector<int64_t> sizes, strides;
  for (int64_t d : order) sizes.push_back(t.size(d)), strides.push_back(t.stride(d));
  B200_TORCH_CHECK(b200_gather_strided(out.data_ptr(), t.const_data_ptr(), (int)t.dim(), sizes.data(), strides.data(),
                                       (int)t.element_size(), backend_stream()));
  return out;
}

struct Workspace {
  at::Tensor hold;
  void* ptr = nullptr;
  size_t bytes = 0;
  Workspace(int64_t n, int64_t c, int64_t s, int layout, const at::TensorOptions& opts) {
    bytes = b200_batch_norm_workspace(n, c, s, layout);
    TORCH_CHECK(bytes > 0, "Vulkan backend (B200): ", b200_last_error());
    hold = at::empty({(int64_t)((bytes + 3) / 4)}, opts);
    ptr = hold.data_ptr();
  }
};

const float* vec_ptr(const Optional& t) { return present(t) ? t->const_data_ptr<float>() : nullptr; }
int64_t vec_stride(const Optional& t) { return present(t) ? t->stride(0) : 0; }

Three batch_norm(const at::Tensor& input, const Optional& weight, const Optional& bias, const Optional& running_mean,
                 const Optional& running_var, bool training, double momentum, double eps) {
  check_input(input);
  const int64_t n = input.size(0), c = input.size(1), s = input.numel() / n / c;
  TORCH_CHECK(training || (present(running_mean) && present(running_var)),
              "Vulkan BatchNorm evaluation requires running statistics");
  for (const auto* t : {&weight, &bias, &running_mean, &running_var})
    if (present(*t)) check_vector(**t, c);
  const auto cl = channels_last_format(input);
  const at::MemoryFormat format = cl.value_or(at::MemoryFormat::Contiguous);
  const int layout = cl ? B200_BN_INTERLEAVED : B200_BN_PLANAR;
  const at::Tensor x = dense(input, format);
  auto y = at::empty(input.sizes(), input.options().memory_format(format));
  auto mean = at::empty({training ? c : 0}, input.options());
  auto inv = at::empty({training ? c : 0}, input.options());
  Workspace ws(n, c, s, layout, input.options());
  // running statistics are written in place through their own strides (batch_norm.cpp:39-40)
  float* rm = present(running_mean) ? running_mean->data_ptr<float>() : nullptr;
  float* rv = present(running_var) ? running_var->data_ptr<float>() : nullptr;
  B200_TORCH_CHECK(b200_batch_norm_forward(n, c, s, layout, x.const_data_ptr<float>(), vec_ptr(weight), vec_stride(weight),
                                           vec_ptr(bias), vec_stride(bias), rm, vec_stride(running_mean), rv,
                                           vec_stride(running_var), training ? 1 : 0, (float)momentum, (float)eps,
                                           y.data_ptr<float>(), training ? mean.data_ptr<float>() : nullptr,
                                           training ? inv.data_ptr<float>() : nullptr, ws.ptr, ws.bytes, backend_stream()));
  return {y, mean, inv};
}

Three batch_norm_backward(const at::Tensor& grad, const at::Tensor& input, const Optional& weight,
                          const Optional& running_mean, const Optional& running_var, const Optional& save_mean,
                          const Optional& save_inv, bool training, double eps, std::array<bool, 3> mask) {
  check_input(input);
  check_input(grad);
  TORCH_CHECK(input.sizes() == grad.sizes(), "Vulkan BatchNorm gradient shape mismatch");
  const int64_t n = input.size(0), c = input.size(1), s = input.numel() / n / c;
  const auto& mean = training ? save_mean : running_mean;
  const auto& inv = training ? save_inv : running_var;
  TORCH_CHECK(present(mean) && present(inv), "Vulkan BatchNorm backward requires statistics");
  check_vector(*mean, c);
  check_vector(*inv, c);
  if (present(weight)) check_vector(*weight, c);
  at::Tensor dx, dw, db;
  if (!mask[0] && !mask[1] && !mask[2]) return {dx, dw, db};
  const auto cl = channels_last_format(input);
  const at::MemoryFormat format = cl.value_or(at::MemoryFormat::Contiguous);
  const int layout = cl ? B200_BN_INTERLEAVED : B200_BN_PLANAR;
  const at::Tensor x = dense(input, format), g = dense(grad, format);
  if (mask[0]) dx = at::empty(input.sizes(), input.options().memory_format(format));
  if (mask[1]) dw = at::empty({c}, input.options());
  if (mask[2]) db = at::empty({c}, input.options());
  Workspace ws(n, c, s, layout, input.options());
  B200_TORCH_CHECK(b200_batch_norm_backward(n, c, s, layout, g.const_data_ptr<float>(), x.const_data_ptr<float>(),
                                            vec_ptr(weight), vec_stride(weight), mean->const_data_ptr<float>(),
                                            mean->stride(0), inv->const_data_ptr<float>(), inv->stride(0), training ? 1 : 0,
                                            (float)eps, mask[0] ? dx.data_ptr<float>() : nullptr,
                                            mask[1] ? dw.data_ptr<float>() : nullptr, mask[2] ? db.data_ptr<float>() : nullptr,
                                            ws.ptr, ws.bytes, backend_stream()));
  return {dx, dw, db};
}

// The newer operator spellings are the same two computations under other signatures, as in the
// reference (batch_norm.cpp:114-119).
using Four = std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor>;
using Six = std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>;

Three legit(const at::Tensor& input, const Optional& weight, const Optional& bias, at::Tensor& running_mean,
            at::Tensor& running_var, bool training, double momentum, double eps) {
  return batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps);
}
Three legit_no_stats(const at::Tensor& input, const Optional& weight, const Optional& bias, bool training, double momentum,
                     double eps) {
  return batch_norm(input, weight, bias, {}, {}, training, momentum, eps);
}
Three legit_no_training(const at::Tensor& input, const Optional& weight, const Optional& bias, const at::Tensor& running_mean,
                        const at::Tensor& running_var, double momentum, double eps) {
  return batch_norm(input, weight, bias, running_mean, running_var, /*training=*/false, momentum, eps);
}
Four with_update(const at::Tensor& input, const Optional& weight, const Optional& bias, at::Tensor& running_mean,
                 at::Tensor& running_var, double momentum, double eps) {
  Three r = batch_norm(input, weight, bias, running_mean, running_var, /*training=*/true, momentum, eps);
  auto reserve = at::empty({0}, input.options().dtype(at::kByte));  // no reserve space on this backend
  return {std::get<0>(r), std::get<1>(r), std::get<2>(r), reserve};
}
Six with_update_functional(const at::Tensor& input, const Optional& weight, const Optional& bias, const at::Tensor& running_mean,
                           const at::Tensor& running_var, double momentum, double eps) {
  at::Tensor new_mean = running_mean.clone(), new_var = running_var.clone();
  Four r = with_update(input, weight, bias, new_mean, new_var, momentum, eps);
  return {std::get<0>(r), std::get<1>(r), std::get<2>(r), std::get<3>(r), new_mean, new_var};
}
Three backward_with_reserve(const at::Tensor& grad, const at::Tensor& input, const at::Tensor& weight,
                            const Optional& running_mean, const Optional& running_var, const Optional& save_mean,
                            const Optional& save_var, bool update, double eps, std::array<bool, 3> mask,
                            const at::Tensor& /*reserve*/) {
  Optional w;
  if (weight.defined()) w = weight;
  return batch_norm_backward(grad, input, w, running_mean, running_var, save_mean, save_var, update, eps, mask);
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("native_batch_norm", &batch_norm);
  m.impl("_native_batch_norm_legit", &legit);
  m.impl("_native_batch_norm_legit.no_stats", &legit_no_stats);
  m.impl("_native_batch_norm_legit_no_training", &legit_no_training);
  m.impl("_batch_norm_with_update", &with_update);
  m.impl("_batch_norm_with_update_functional", &with_update_functional);
  m.impl("native_batch_norm_backward", &batch_norm_backward);
  m.impl("batch_norm_backward", &backward_with_reserve);
}

}  // namespace torch_vulkan
