// ATen registrations on PrivateUse1 for the convolution path and the tensor plumbing its
// callers need.  Host-side mirror of the reference's operator layer:
//   convolution_overrideable / convolution_backward_overrideable  csrc/ops/convolution.cpp:641-702
//   controls (env flags, re-read on every call)                  csrc/ops/convolution.cpp:402-422
//   dispatch statistics                                          csrc/ops/convolution.cpp:523-538,625-635
//   mm / mm.out / addmm                                          csrc/ops/mm.cpp:244-383,835-917,1092-1109
//   empty / empty_strided / copies / views / resize_ / item      csrc/ops/mm.cpp:498-681,942-991,1054-1067
// No operator here computes on the host: device work is the C ABI's, and there is no CPU
// fallback registration (unregistered operators raise PyTorch's usual "not implemented" error).
#include "backend.h"

#include <ATen/EmptyTensor.h>
#include <ATen/native/Resize.h>
#include <ATen/ops/_reshape_alias_native.h>
#include <ATen/ops/as_strided_native.h>
#include <ATen/ops/view_native.h>
#include <torch/library.h>

#include <algorithm>
#include <array>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <functional>
#include <mutex>
#include <sstream>
#include <unordered_map>

namespace torch_vulkan {

static bool on_device(const at::Tensor& t) { return t.device().type() == c10::DeviceType::PrivateUse1; }
static const c10::DispatchKeySet kKeys(c10::DispatchKey::PrivateUse1);

// ---- allocation ------------------------------------------------------------------------------
static at::Tensor empty_memory_format(c10::SymIntArrayRef size, std::optional<at::ScalarType> dtype,
                                      std::optional<at::Layout>, std::optional<at::Device> device,
                                      std::optional<bool>, std::optional<at::MemoryFormat> memory_format) {
  if (device) validate_device(*device);
  return at::detail::empty_generic(C10_AS_INTARRAYREF_SLOW(size), backend_allocator(), kKeys,
                                   dtype.value_or(at::kFloat), memory_format);
}
static at::Tensor empty_strided(c10::SymIntArrayRef size, c10::SymIntArrayRef stride,
                                std::optional<at::ScalarType> dtype, std::optional<at::Layout>,
                                std::optional<at::Device> device, std::optional<bool>) {
  if (device) validate_device(*device);
  return at::detail::empty_strided_generic(C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride),
                                           backend_allocator(), kKeys, dtype.value_or(at::kFloat));
}

// ---- copies ------------------------------------------------------------------------------------
static bool dense_standard(const at::Tensor& t) { return t.is_contiguous(); }

static at::Tensor device_contiguous(const at::Tensor& t) {  // strided device view -> dense device tensor
  if (dense_standard(t)) return t;
  auto out = at::empty(t.sizes(), t.options());
  if (t.numel())
    B200_TORCH_CHECK(b200_gather_strided(out.data_ptr(), t.const_data_ptr(), (int)t.dim(), t.sizes().data(),
                                         t.strides().data(), (int)t.element_size(), backend_stream()));
  return out;
}

// dst (device, any strides) <- dense device tensor of the same dtype and shape
static void device_assign(const at::Tensor& dst, const at::Tensor& dense) {
  if (!dst.numel()) return;
  if (dense_standard(dst))
    B200_TORCH_CHECK(b200_memcpy(dst.data_ptr(), dense.const_data_ptr(), dst.nbytes(), B200_D2D, backend_stream()));
  else
    B200_TORCH_CHECK(b200_scatter_strided(dst.data_ptr(), dense.const_data_ptr(), (int)dst.dim(), dst.sizes().data(),
                                          dst.strides().data(), (int)dst.element_size(), backend_stream()));
}

static at::Tensor copy_from(const at::Tensor& src, const at::Tensor& dst, bool /*non_blocking*/) {
  TORCH_CHECK(src.element_size() <= 8 && dst.element_size() <= 8, "Vulkan copy: unsupported element size");
  if (!on_device(src)) {  // host -> device
    TORCH_CHECK(src.device().is_cpu() && on_device(dst), "Vulkan copy: unsupported device pair");
    const auto host = src.to(dst.scalar_type()).expand(dst.sizes()).contiguous();
    if (!host.numel()) return dst;
    if (dense_standard(dst)) {
      B200_TORCH_CHECK(b200_memcpy(dst.data_ptr(), host.const_data_ptr(), host.nbytes(), B200_H2D, backend_stream()));
    } else {
      auto staged = at::empty(dst.sizes(), dst.options());
      B200_TORCH_CHECK(b200_memcpy(staged.data_ptr(), host.const_data_ptr(), host.nbytes(), B200_H2D, backend_stream()));
      device_assign(dst, staged);
    }
    // the host tensor may be pageable and is released on return
    B200_TORCH_CHECK(b200_stream_sync(backend_stream()));
    return dst;
  }
  if (!on_device(dst)) {  // device -> host
    TORCH_CHECK(dst.device().is_cpu(), "Vulkan copy: unsupported device pair");
    const auto dense = device_contiguous(src.expand(dst.sizes()));
    auto host = at::empty(dense.sizes(), dense.options().device(at::kCPU));
    if (dense.numel()) {
      B200_TORCH_CHECK(b200_memcpy(host.data_ptr(), dense.const_data_ptr(), dense.nbytes(), B200_D2H, backend_stream()));
      B200_TORCH_CHECK(b200_stream_sync(backend_stream()));
      note_host_read(dense.nbytes());
    }
    dst.copy_(host);
    return dst;
  }
  // device -> device
  if (src.scalar_type() != dst.scalar_type()) {  // dtype conversion is not part of this path: stage through the host
    ++execution_stats().cpu_fallback_calls;
    return copy_from(src.cpu().to(dst.scalar_type()), dst, false);
  }
  device_assign(dst, device_contiguous(src.expand(dst.sizes())));
  return dst;
}

static void resize_storage(const at::Tensor& self, size_t bytes) {
  auto* impl = self.storage().unsafeGetStorageImpl();
  if (bytes <= impl->nbytes()) return;
  auto next = backend_allocator()->allocate(bytes);
  if (impl->nbytes() && impl->data())
    B200_TORCH_CHECK(b200_memcpy(next.get(), impl->data(), impl->nbytes(), B200_D2D, backend_stream()));
  impl->set_data_ptr_noswap(std::move(next));
  impl->set_nbytes(bytes);
}

static const at::Tensor& resize_(const at::Tensor& self, c10::SymIntArrayRef size,
                                 std::optional<at::MemoryFormat> memory_format) {
  const auto sizes = C10_AS_INTARRAYREF_SLOW(size);
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  resize_storage(self, (size_t)(self.storage_offset() + numel) * self.element_size());
  self.unsafeGetTensorImpl()->set_sizes_contiguous(sizes);
  if (memory_format && *memory_format != at::MemoryFormat::Preserve && *memory_format != at::MemoryFormat::Contiguous)
    self.unsafeGetTensorImpl()->empty_tensor_restride(*memory_format);
  return self;
}

static at::Tensor copy_from_and_resize(const at::Tensor& src, const at::Tensor& dst) {
  if (dst.sizes() != src.sizes()) {
    std::vector<c10::SymInt> sz(src.sizes().begin(), src.sizes().end());
    resize_(dst, sz, std::nullopt);
  }
  return copy_from(src, dst, false);
}

static at::Scalar local_scalar_dense(const at::Tensor& self) {
  TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(), " elements cannot be converted to Scalar");
  return self.cpu().item();
}

static at::Tensor& fill_scalar(at::Tensor& self, const at::Scalar& value) {
  if (!self.numel()) return self;
  if (value.toDouble() == 0.0 && dense_standard(self)) {
    B200_TORCH_CHECK(b200_memset(self.data_ptr(), 0, self.nbytes(), backend_stream()));
    return self;
  }
  copy_from(at::full(self.sizes(), value, self.options().device(at::kCPU)), self, false);
  return self;
}
static at::Tensor& zero_(at::Tensor& self) { return fill_scalar(self, 0); }

// ---- views -------------------------------------------------------------------------------------
static at::Tensor view(const at::Tensor& self, c10::SymIntArrayRef size) {
  return at::native::view(self, C10_AS_INTARRAYREF_SLOW(size));
}
static at::Tensor as_strided(const at::Tensor& self, c10::SymIntArrayRef size, c10::SymIntArrayRef stride,
                             std::optional<c10::SymInt> storage_offset) {
  std::optional<int64_t> off;
  if (storage_offset) off = storage_offset->expect_int();
  return at::native::as_strided_tensorimpl(self, C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride), off);
}
static at::Tensor reshape_alias(const at::Tensor& self, c10::SymIntArrayRef size, c10::SymIntArrayRef stride) {
  return at::native::_reshape_alias(self, C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride));
}

// ---- convolution -------------------------------------------------------------------------------
static std::mutex plan_mutex;
static std::map<std::string, uint64_t> plan_stats;
// Plans found by the opt-in autotuner (TORCH_VULKAN_CONV_AUTOTUNE=1), FIFO of at most 256, keyed by
// phase, budget, the sixteen geometry parameters and the memory layout class of each operand -- never
// by addresses (csrc/ops/convolution.cpp:523-554 of the reference).
static std::unordered_map<std::string, int> plan_cache;
static std::deque<std::string> plan_fifo;
static constexpr size_t kMaxConvPlans = 256;

std::map<std::string, uint64_t> conv_dispatch_stats() {
  std::lock_guard<std::mutex> lock(plan_mutex);
  auto result = plan_stats;
  for (const char* key : {"hits", "misses", "tunes", "evictions", "candidates_timed"}) result[key] += 0;
  result["entries"] = plan_cache.size();
  return result;
}
void clear_conv_dispatch_cache() {
  std::lock_guard<std::mutex> lock(plan_mutex);
  plan_cache.clear();
  plan_fifo.clear();
  plan_stats.clear();
}

static size_t workspace_limit() {
  const char* value = std::getenv("TORCH_VULKAN_CONV_WORKSPACE_MB");
  if (!value || !*value) return 64ull * 1024 * 1024;
  char* end = nullptr;
  const auto mb = std::strtoull(value, &end, 10);
  TORCH_CHECK(*value != '-' && end != value && *end == '\0' && mb <= 4096,
              "TORCH_VULKAN_CONV_WORKSPACE_MB must be an integer in [0,4096]");
  return mb * 1024 * 1024;
}

// Maps the reference's env controls onto this library's candidates.  forward: auto / direct /
// tiled / depthwise / winograd; backward: auto / direct / optimized.  "tiled"/"optimized" force the
// implicit-GEMM family (tcgen05 when the geometry allows, CUDA cores otherwise); the GLSL tile
// menu (TORCH_VULKAN_CONV_TILE) has no meaning here and is validated, then ignored.
static int requested_algo(int phase, const b200_conv_params& p) {
  const char* name = phase == B200_PHASE_FORWARD ? "TORCH_VULKAN_CONV_ALGO" : "TORCH_VULKAN_CONV_BACKWARD_ALGO";
  const char* raw = std::getenv(name);
  const std::string algo = raw && *raw ? raw : "auto";
  const bool fwd = phase == B200_PHASE_FORWARD;
  TORCH_CHECK(algo == "auto" || algo == "direct" ||
                  (fwd ? algo == "tiled" || algo == "depthwise" || algo == "winograd" : algo == "optimized"),
              name, " has an invalid algorithm (forward: auto/direct/tiled/depthwise/winograd; backward: auto/direct/optimized)");
  const char* tile = std::getenv("TORCH_VULKAN_CONV_TILE");
  if (tile && *tile) {
    bool known = false;
    for (const char* t : {"auto", "base", "wide", "tall", "register", "register3", "register3_hoist"}) known |= !std::strcmp(tile, t);
    TORCH_CHECK(known, "TORCH_VULKAN_CONV_TILE must be auto/base/wide/tall/register/register3/register3_hoist");
  }
  const char* tune = std::getenv("TORCH_VULKAN_CONV_AUTOTUNE");
  TORCH_CHECK(!tune || !*tune || !std::strcmp(tune, "0") || !std::strcmp(tune, "1"),
              "TORCH_VULKAN_CONV_AUTOTUNE must be 0 or 1");
  if (algo == "direct") return B200_ALGO_DIRECT;
  if (algo == "winograd") return B200_ALGO_WINOGRAD;
  if (algo == "depthwise") {
    TORCH_CHECK(p.groups == p.cin, "Forced Vulkan convolution forward candidate depthwise exceeds device limits, "
                                   "workspace budget, or operator applicability");
    return B200_ALGO_DIRECT;
  }
  if (algo == "tiled" || algo == "optimized") {
    const int tc = b200_conv2d_select(&p, phase, B200_ALGO_TC, 0);
    return tc == B200_ALGO_TC ? B200_ALGO_TC : B200_ALGO_TILED;
  }
  return B200_ALGO_AUTO;
}

static bool autotune_enabled() {
  const char* tune = std::getenv("TORCH_VULKAN_CONV_AUTOTUNE");
  return tune && !std::strcmp(tune, "1");
}

static const char* phase_name(int phase) {
  static const char* names[] = {"forward", "dinput", "dweight", "dbias"};
  return names[phase];
}
static const char* candidate_name(int algo, int phase) {
  switch (algo) {
    case B200_ALGO_DIRECT: return "direct";
    case B200_ALGO_TILED: return phase == B200_PHASE_DBIAS ? "reduce" : "tiled_simt";
    case B200_ALGO_TC: return "tiled_tcgen05";
    case B200_ALGO_WINOGRAD: return "winograd_f4";
    default: return "auto";
  }
}

// Runs one candidate: (algorithm id, workspace pointer, workspace bytes) -> B200_* code.
using ConvRunner = std::function<int(int, void*, size_t)>;

// Memory layout class of an operand for the plan key: 0 contiguous NCHW, 1 channels-last, 2 other.
static int layout_class(const at::Tensor& t) {
  if (t.is_contiguous()) return 0;
  if (t.dim() == 4 && t.is_contiguous(at::MemoryFormat::ChannelsLast)) return 1;
  return 2;
}

// Opt-in autotuner (csrc/ops/convolution.cpp:570-624 of the reference): on a cache miss every
// shortlisted candidate is warmed once and timed five times in rotated order with the stream
// synchronised around each run; the heuristic's choice is replaced only by a candidate whose median
// is more than 5 % faster.  Returns the algorithm id to run (B200_ALGO_AUTO keeps the heuristic).
static int tuned_algo(const b200_conv_params& p, int phase, size_t budget, const std::string& layouts,
                      const at::TensorOptions& opts, const ConvRunner& run) {
  const int heuristic = b200_conv2d_select(&p, phase, B200_ALGO_AUTO, budget);
  std::vector<int> available;
  for (int c : {B200_ALGO_DIRECT, B200_ALGO_TILED, B200_ALGO_TC, B200_ALGO_WINOGRAD})
    if (b200_conv2d_select(&p, phase, c, budget) == c && b200_conv2d_workspace(&p, phase, c, budget) <= budget)
      available.push_back(c);
  if (std::find(available.begin(), available.end(), heuristic) == available.end()) return B200_ALGO_AUTO;
  std::ostringstream key;
  key << b200_device_name() << ':' << phase << ':' << budget << ':' << layouts;
  for (const int v : {p.n, p.cin, p.cout, p.h, p.w, p.kh, p.kw, p.oh, p.ow, p.sh, p.sw, p.ph, p.pw, p.dh, p.dw, p.groups})
    key << ':' << v;
  {
    std::lock_guard<std::mutex> lock(plan_mutex);
    const auto it = plan_cache.find(key.str());
    if (it != plan_cache.end() && std::find(available.begin(), available.end(), it->second) != available.end()) {
      ++plan_stats["hits"];
      return it->second;
    }
    ++plan_stats["misses"];
  }
  // bound the tuning cost: the one-thread-per-output kernels are only timed on small problems
  const long double work = (long double)p.n * p.cout * p.oh * p.ow * (p.cin / p.groups) * p.kh * p.kw;
  std::vector<int> shortlist;
  for (int c : available)
    if (c != B200_ALGO_DIRECT || work <= 8000000 || c == heuristic) shortlist.push_back(c);
  const auto trial = [&](int c) {
    // candidate-specific scratch allocation and release are part of what is timed
    const size_t need = b200_conv2d_workspace(&p, phase, c, budget);
    at::Tensor scratch;
    if (need) scratch = at::empty({(int64_t)need}, opts.dtype(at::kByte));
    B200_TORCH_CHECK(run(c, need ? scratch.data_ptr() : nullptr, need));
    B200_TORCH_CHECK(b200_stream_sync(backend_stream()));
  };
  B200_TORCH_CHECK(b200_stream_sync(backend_stream()));
  for (int c : shortlist) trial(c);
  std::vector<std::array<double, 5>> samples(shortlist.size());
  for (int repeat = 0; repeat < 5; ++repeat)
    for (size_t j = 0; j < shortlist.size(); ++j) {
      const size_t i = (j + repeat) % shortlist.size();
      const auto start = std::chrono::steady_clock::now();
      trial(shortlist[i]);
      samples[i][repeat] = std::chrono::duration<double, std::nano>(std::chrono::steady_clock::now() - start).count();
    }
  for (auto& sample : samples) std::sort(sample.begin(), sample.end());
  const size_t incumbent = std::find(shortlist.begin(), shortlist.end(), heuristic) - shortlist.begin();
  int selected = heuristic;
  double best = samples[incumbent][2];
  for (size_t i = 0; i < shortlist.size(); ++i)
    if (samples[i][2] < best * 0.95) {  // marginal differences are timing noise: keep the heuristic
      best = samples[i][2];
      selected = shortlist[i];
    }
  {
    std::lock_guard<std::mutex> lock(plan_mutex);
    ++plan_stats["tunes"];
    plan_stats["candidates_timed"] += shortlist.size();
    for (int c : shortlist) ++plan_stats[std::string("candidates_timed_") + phase_name(phase) + "_" + candidate_name(c, phase)];
    if (!plan_cache.count(key.str())) {
      if (plan_cache.size() >= kMaxConvPlans) {
        plan_cache.erase(plan_fifo.front());
        plan_fifo.pop_front();
        ++plan_stats["evictions"];
      }
      plan_fifo.push_back(key.str());
    }
    plan_cache[key.str()] = selected;
  }
  return selected;
}

// Resolves the candidate (env controls, autotuner, heuristic), enforces the workspace budget,
// allocates the scratch and runs it.  The tuner's trial runs write the same output; the winner is
// executed again afterwards so that the visible result always belongs to the recorded plan.
static void plan_and_run(const b200_conv_params& p, int phase, const at::TensorOptions& opts, const std::string& layouts,
                         const ConvRunner& run) {
  const size_t budget = workspace_limit();
  int requested = phase == B200_PHASE_DBIAS ? B200_ALGO_AUTO : requested_algo(phase, p);
  if (requested == B200_ALGO_AUTO && phase != B200_PHASE_DBIAS && autotune_enabled())
    requested = tuned_algo(p, phase, budget, layouts, opts, run);
  const int chosen = b200_conv2d_select(&p, phase, requested, budget);
  TORCH_CHECK(chosen >= 0, "Forced Vulkan convolution ", phase_name(phase), " candidate: ", b200_last_error());
  int algo = requested;
  size_t need = b200_conv2d_workspace(&p, phase, requested, budget);
  if (chosen == B200_ALGO_TC && (phase == B200_PHASE_FORWARD || phase == B200_PHASE_DINPUT) && need > budget) {
    // the weight stage images do not fit the budget: a forced request fails like the reference's
    // forced tiled dWeight with a zero budget, an automatic one takes the CUDA-core kernel
    TORCH_CHECK(requested == B200_ALGO_AUTO, "Forced Vulkan convolution ", phase_name(phase),
                " candidate exceeds device limits, workspace budget, or operator applicability");
    algo = B200_ALGO_TILED;
    need = 0;
  }
  if (phase == B200_PHASE_DWEIGHT && requested != B200_ALGO_AUTO && requested != B200_ALGO_DIRECT && need == 0 &&
      (int64_t)p.n * p.oh * p.ow > 256 && budget == 0)
    TORCH_CHECK(false, "Forced Vulkan convolution dweight candidate exceeds device limits, workspace budget, "
                       "or operator applicability");
  at::Tensor scratch;
  if (need) scratch = at::empty({(int64_t)need}, opts.dtype(at::kByte));
  {
    std::lock_guard<std::mutex> lock(plan_mutex);
    const int shown = algo == B200_ALGO_AUTO ? chosen : b200_conv2d_select(&p, phase, algo, budget);
    ++plan_stats[std::string("selected_") + phase_name(phase) + "_" + candidate_name(shown, phase)];
    if (phase == B200_PHASE_DWEIGHT && need) {
      const size_t dw_bytes = sizeof(float) * (size_t)p.cout * (p.cin / p.groups) * p.kh * p.kw;
      plan_stats["dweight_tiled_split_count_total"] += need / dw_bytes;
      plan_stats["dweight_tiled_workspace_bytes_total"] += need;
      ++plan_stats["dweight_tiled_dispatches"];
    }
  }
  B200_TORCH_CHECK(run(algo, need ? scratch.data_ptr() : nullptr, need));
}

static b200_view4 view_of(const at::Tensor& t) {
  b200_view4 v{t.const_data_ptr<float>(), {0, 0, 0, 0}};
  for (int64_t d = 0; d < t.dim(); ++d) v.stride[d] = t.stride(d);
  if (t.dim() == 3) v.stride[3] = t.stride(2), v.stride[2] = 0;  // [N, C, L] read as [N, C, 1, L]
  return v;
}
static void require_fp32_device(const at::Tensor& t) {
  TORCH_CHECK(on_device(t) && t.scalar_type() == at::kFloat, "Vulkan convolution requires FP32 Vulkan tensors");
}

// One convolution call resolved to the 2-D geometry the library computes with.  A 1-D convolution
// is the 2-D one with a single row.  For a transposed convolution `p` describes the ordinary
// convolution whose input gradient it is (its "input" is this call's result), as
// b200_conv_transpose2d_forward expects; the reference routes both through convolution_nd
// (csrc/ops/convolution.cpp:647,674; csrc/ops/convolution_nd.cpp:11-37).
struct ConvCall {
  b200_conv_params p;
  bool transposed;
  std::vector<int64_t> result_shape;  // of the forward result
};

// ---- generic N-d branch: 3-D convolutions and int64 tensors --------------------------------------
// The reference sends every rank and both dtypes through one generic shader (csrc/ops/convolution_nd.cpp:51-74);
// here FP32 calls over one or two spatial dimensions take the Conv2D kernels below and only what those do not
// cover (three spatial dimensions, int64) runs the generic kernel, on packed operands as in the reference.
static bool takes_nd_branch(const at::Tensor& input) { return input.dim() == 5 || input.scalar_type() == at::kLong; }

struct ConvNdCall {
  b200_convnd_params p;
  std::vector<int64_t> result_shape;
};

static ConvNdCall convnd_call(const at::Tensor& x, const at::Tensor& w, c10::SymIntArrayRef stride, c10::SymIntArrayRef pad,
                              c10::SymIntArrayRef dilation, bool transposed, c10::SymIntArrayRef output_pad,
                              const c10::SymInt& groups) {
  const int rank = (int)x.dim() - 2;
  TORCH_CHECK(rank >= 1 && rank <= 3 && w.dim() == x.dim(), "convolution: expected matching rank 3, 4 or 5 tensors");
  TORCH_CHECK((x.scalar_type() == at::kFloat || x.scalar_type() == at::kLong) && w.scalar_type() == x.scalar_type() &&
                  x.device() == w.device() && on_device(x),
              "convolution: expected matching FP32/int64 tensors on the same device");
  TORCH_CHECK((int)stride.size() == rank && (int)pad.size() == rank && (int)dilation.size() == rank && (int)output_pad.size() == rank,
              "convolution: spatial parameter rank mismatch");
  int64_t in[3], k[3], s[3], p[3], d[3], op[3];
  for (int a = 0; a < rank; ++a) {
    in[a] = x.size(a + 2), k[a] = w.size(a + 2), s[a] = stride[a].expect_int(), p[a] = pad[a].expect_int();
    d[a] = dilation[a].expect_int(), op[a] = output_pad[a].expect_int();
  }
  ConvNdCall call{};
  const int rc = b200_convnd_geometry(&call.p, rank, x.size(0), x.size(1), in, w.size(0), w.size(1), k, s, p, d, op, transposed,
                                      groups.expect_int());
  TORCH_CHECK(rc == 0, b200_last_error());
  call.result_shape = {call.p.n, call.p.cout};
  for (int a = 0; a < rank; ++a) call.result_shape.push_back(call.p.out[3 - rank + a]);
  return call;
}

static at::Tensor convnd_forward(const at::Tensor& x, const at::Tensor& w, const std::optional<at::Tensor>& bias,
                                 c10::SymIntArrayRef stride, c10::SymIntArrayRef pad, c10::SymIntArrayRef dilation, bool transposed,
                                 c10::SymIntArrayRef output_pad, const c10::SymInt& groups) {
  const ConvNdCall call = convnd_call(x, w, stride, pad, dilation, transposed, output_pad, groups);
  auto out = at::empty(call.result_shape, x.options().memory_format(at::MemoryFormat::Contiguous));
  at::Tensor b;
  if (bias && bias->defined()) {
    TORCH_CHECK(bias->dim() == 1 && bias->numel() == call.p.cout && bias->device() == x.device() &&
                    bias->scalar_type() == x.scalar_type(),
                "convolution: invalid bias");
    b = device_contiguous(*bias);
  }
  if (!out.numel()) return out;
  const at::Tensor xc = device_contiguous(x), wc = device_contiguous(w);
  B200_TORCH_CHECK(b200_convnd_forward(&call.p, xc.const_data_ptr(), wc.const_data_ptr(), b.defined() ? b.const_data_ptr() : nullptr,
                                       out.data_ptr(), x.scalar_type() == at::kLong, backend_stream()));
  return out;
}

static std::tuple<at::Tensor, at::Tensor, at::Tensor> convnd_backward(const at::Tensor& grad, const at::Tensor& x, const at::Tensor& w,
                                                                      c10::SymIntArrayRef stride, c10::SymIntArrayRef pad,
                                                                      c10::SymIntArrayRef dilation, bool transposed,
                                                                      c10::SymIntArrayRef output_pad, const c10::SymInt& groups,
                                                                      std::array<bool, 3> mask) {
  const ConvNdCall call = convnd_call(x, w, stride, pad, dilation, transposed, output_pad, groups);
  TORCH_CHECK(grad.sizes() == at::IntArrayRef(call.result_shape) && grad.scalar_type() == at::kFloat && grad.device() == x.device() &&
                  x.scalar_type() == at::kFloat,
              "convolution backward: invalid gradient");
  const at::Tensor xc = device_contiguous(x), wc = device_contiguous(w), gc = device_contiguous(grad);
  const auto dense = [](const at::Tensor& like) { return like.options().memory_format(at::MemoryFormat::Contiguous); };
  at::Tensor dx, dw, db;
  if (mask[0]) dx = at::empty(x.sizes(), dense(x));
  if (mask[1]) dw = at::empty(w.sizes(), dense(w));
  if (mask[2]) db = at::empty({call.p.cout}, dense(w));
  const auto ptr = [](const at::Tensor& t) { return t.defined() && t.numel() ? t.data_ptr<float>() : nullptr; };
  B200_TORCH_CHECK(b200_convnd_backward(&call.p, gc.numel() ? gc.const_data_ptr<float>() : nullptr,
                                        xc.numel() ? xc.const_data_ptr<float>() : nullptr, wc.const_data_ptr<float>(), ptr(dx), ptr(dw),
                                        ptr(db), backend_stream()));
  return {dx, dw, db};
}

static ConvCall conv_call(const at::Tensor& input, const at::Tensor& weight, c10::SymIntArrayRef stride,
                          c10::SymIntArrayRef padding, c10::SymIntArrayRef dilation, bool transposed,
                          c10::SymIntArrayRef output_padding, const c10::SymInt& groups_sym) {
  const int64_t rank = input.dim() - 2;
  TORCH_CHECK((rank == 1 || rank == 2) && weight.dim() == input.dim(), "convolution: expected matching rank 3 or 4 tensors");
  TORCH_CHECK((int64_t)stride.size() == rank && (int64_t)padding.size() == rank && (int64_t)dilation.size() == rank &&
                  (int64_t)output_padding.size() == rank,
              "convolution: spatial parameter rank mismatch");
  require_fp32_device(input);
  require_fp32_device(weight);
  // spatial parameters as (row, column) pairs; the missing row of a 1-D call is the identity
  auto pair = [&](c10::SymIntArrayRef v, int64_t fill) {
    return rank == 2 ? std::array<int64_t, 2>{v[0].expect_int(), v[1].expect_int()} : std::array<int64_t, 2>{fill, v[0].expect_int()};
  };
  const auto s = pair(stride, 1), pad = pair(padding, 0), d = pair(dilation, 1), op = pair(output_padding, 0);
  const int64_t groups = groups_sym.expect_int();
  const int64_t h = rank == 2 ? input.size(2) : 1, w = input.size(rank + 1);
  const int64_t kh = rank == 2 ? weight.size(2) : 1, kw = weight.size(rank + 1);
  ConvCall call{};
  call.transposed = transposed;
  int rc;
  if (!transposed) {
    TORCH_CHECK(op[0] == 0 && op[1] == 0, "convolution: invalid output padding");
    rc = b200_conv2d_geometry(&call.p, input.size(0), input.size(1), weight.size(0), h, w, weight.size(1), kh, kw, s[0], s[1],
                              pad[0], pad[1], d[0], d[1], groups);
    TORCH_CHECK(rc == 0, "Vulkan ", b200_last_error());
    call.result_shape = {call.p.n, call.p.cout, call.p.oh, call.p.ow};
  } else {
    TORCH_CHECK(groups > 0 && weight.size(0) == input.size(1), "convolution: weight/channel/group mismatch");
    for (int i = 0; i < 2; ++i)
      TORCH_CHECK(op[i] >= 0 && (op[i] < s[i] || op[i] < d[i]), "convolution: invalid output padding");
    const int64_t oh = (h - 1) * s[0] - 2 * pad[0] + d[0] * (kh - 1) + op[0] + 1;
    const int64_t ow = (w - 1) * s[1] - 2 * pad[1] + d[1] * (kw - 1) + op[1] + 1;
    TORCH_CHECK(oh > 0 && ow > 0, "convolution: invalid or oversized output shape");
    rc = b200_conv2d_geometry(&call.p, input.size(0), weight.size(1) * groups, weight.size(0), oh, ow, weight.size(1), kh, kw,
                              s[0], s[1], pad[0], pad[1], d[0], d[1], groups);
    TORCH_CHECK(rc == 0, "Vulkan ", b200_last_error());
    TORCH_CHECK(call.p.oh == h && call.p.ow == w, "convolution: invalid or oversized output shape");
    call.result_shape = {call.p.n, call.p.cin, call.p.h, call.p.w};
  }
  if (rank == 1) call.result_shape.erase(call.result_shape.begin() + 2);
  return call;
}

static at::Tensor convolution_overrideable(const at::Tensor& input, const at::Tensor& weight,
                                           const std::optional<at::Tensor>& bias, c10::SymIntArrayRef stride,
                                           c10::SymIntArrayRef padding, c10::SymIntArrayRef dilation, bool transposed,
                                           c10::SymIntArrayRef output_padding, c10::SymInt groups) {
  if (takes_nd_branch(input)) return convnd_forward(input, weight, bias, stride, padding, dilation, transposed, output_padding, groups);
  const ConvCall call = conv_call(input, weight, stride, padding, dilation, transposed, output_padding, groups);
  const b200_conv_params& p = call.p;
  const float* bias_ptr = nullptr;
  int64_t bias_stride = 0;
  if (bias && bias->defined()) {
    TORCH_CHECK(bias->numel() == call.result_shape[1] && bias->scalar_type() == at::kFloat && on_device(*bias),
                "Vulkan convolution: bias shape/dtype mismatch");
    bias_ptr = bias->const_data_ptr<float>();
    bias_stride = bias->dim() ? bias->stride(bias->dim() - 1) : 0;
  }
  auto result = at::empty(call.result_shape, input.options());  // always contiguous, as in the reference
  const std::string layouts = std::to_string(layout_class(input)) + std::to_string(layout_class(weight));
  if (call.transposed) {
    plan_and_run(p, B200_PHASE_DINPUT, input.options(), layouts + "t", [&](int algo, void* ws, size_t ws_bytes) {
      return b200_conv_transpose2d_forward(&p, view_of(input), view_of(weight), bias_ptr, bias_stride, result.data_ptr<float>(),
                                           ws, ws_bytes, algo, backend_stream());
    });
    return result;
  }
  plan_and_run(p, B200_PHASE_FORWARD, input.options(), layouts, [&](int algo, void* ws, size_t ws_bytes) {
    return b200_conv2d_forward(&p, view_of(input), view_of(weight), bias_ptr, bias_stride, result.data_ptr<float>(), ws,
                               ws_bytes, algo, backend_stream());
  });
  return result;
}

static std::tuple<at::Tensor, at::Tensor, at::Tensor> convolution_backward_overrideable(
    const at::Tensor& grad_output, const at::Tensor& input, const at::Tensor& weight, c10::SymIntArrayRef stride,
    c10::SymIntArrayRef padding, c10::SymIntArrayRef dilation, bool transposed, c10::SymIntArrayRef output_padding,
    c10::SymInt groups, std::array<bool, 3> output_mask) {
  if (takes_nd_branch(input))
    return convnd_backward(grad_output, input, weight, stride, padding, dilation, transposed, output_padding, groups, output_mask);
  const ConvCall call = conv_call(input, weight, stride, padding, dilation, transposed, output_padding, groups);
  const b200_conv_params& p = call.p;
  TORCH_CHECK(grad_output.sizes() == at::IntArrayRef(call.result_shape), "Vulkan convolution backward: output gradient shape mismatch");
  require_fp32_device(grad_output);
  const std::string layouts = std::to_string(layout_class(input)) + std::to_string(layout_class(weight)) +
                              std::to_string(layout_class(grad_output)) + (call.transposed ? "t" : "");
  // Ordinary convolution: dx = dInput(dy, w), dw = dWeight(x, dy).  Transposed: the roles swap,
  // dx = forward(dy, w) and dw = dWeight(dy as the input, x as the output gradient).
  const at::Tensor& conv_in = call.transposed ? grad_output : input;    // the tensor with p's input extent
  const at::Tensor& conv_out = call.transposed ? input : grad_output;  // the tensor with p's output extent
  at::Tensor dx, dw, db;
  if (output_mask[0]) {
    dx = at::empty(input.sizes(), input.options().memory_format(at::MemoryFormat::Contiguous));
    if (call.transposed) {
      plan_and_run(p, B200_PHASE_FORWARD, input.options(), layouts, [&](int algo, void* ws, size_t ws_bytes) {
        return b200_conv2d_forward(&p, view_of(grad_output), view_of(weight), nullptr, 0, dx.data_ptr<float>(), ws, ws_bytes,
                                   algo, backend_stream());
      });
    } else {
      plan_and_run(p, B200_PHASE_DINPUT, input.options(), layouts, [&](int algo, void* ws, size_t ws_bytes) {
        return b200_conv2d_dinput(&p, view_of(grad_output), view_of(weight), dx.data_ptr<float>(), ws, ws_bytes, algo,
                                  backend_stream());
      });
    }
  }
  if (output_mask[1]) {
    dw = at::empty(weight.sizes(), weight.options().memory_format(at::MemoryFormat::Contiguous));
    plan_and_run(p, B200_PHASE_DWEIGHT, input.options(), layouts, [&](int algo, void* ws, size_t ws_bytes) {
      return b200_conv2d_dweight(&p, view_of(conv_in), view_of(conv_out), dw.data_ptr<float>(), ws, ws_bytes, algo,
                                 backend_stream());
    });
  }
  if (output_mask[2]) {
    // the bias gradient sums grad_output over samples and positions; for a transposed call that
    // tensor has p's input extent, described here as the output of a 1x1 convolution
    b200_conv_params pb = p;
    if (call.transposed) {
      const int rc = b200_conv2d_geometry(&pb, p.n, p.cin, p.cin, p.h, p.w, p.cin, 1, 1, 1, 1, 0, 0, 1, 1, 1);
      TORCH_CHECK(rc == 0, "Vulkan ", b200_last_error());
    }
    db = at::empty({pb.cout}, weight.options());
    plan_and_run(pb, B200_PHASE_DBIAS, input.options(), layouts, [&](int, void* ws, size_t ws_bytes) {
      return b200_conv2d_dbias(&pb, view_of(grad_output), db.data_ptr<float>(), ws, ws_bytes, backend_stream());
    });
  }
  return {dx, dw, db};
}

// ---- torch_vulkan::conv2d_fused ------------------------------------------------------------------------
// y = act(conv2d(x, w) + bias + residual) in one call, optionally produced channels-last: the convolution
// together with the add.Tensor / relu that follow it in a residual block, which the reference runs as
// separate operators (csrc/ops/mm.cpp:1094-1097).  With the tcgen05 strip kernel all of it happens in the
// kernel's epilogue and the channels-last result is written directly; other candidates compute the dense
// result, apply one elementwise pass, and a channels-last request is then a strided copy.  Forward only:
// the operator records no autograd graph.
static at::Tensor conv2d_fused(const at::Tensor& input, const at::Tensor& weight, const std::optional<at::Tensor>& bias,
                               const std::optional<at::Tensor>& residual, bool relu, at::IntArrayRef stride, at::IntArrayRef padding,
                               at::IntArrayRef dilation, int64_t groups, bool channels_last_out) {
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 4, "conv2d_fused: expected 4-D input and weight");
  TORCH_CHECK(stride.size() == 2 && padding.size() == 2 && dilation.size() == 2, "convolution: spatial parameter rank mismatch");
  require_fp32_device(input);
  require_fp32_device(weight);
  b200_conv_params p;
  const int rc = b200_conv2d_geometry(&p, input.size(0), input.size(1), weight.size(0), input.size(2), input.size(3), weight.size(1),
                                      weight.size(2), weight.size(3), stride[0], stride[1], padding[0], padding[1], dilation[0],
                                      dilation[1], groups);
  TORCH_CHECK(rc == 0, "Vulkan ", b200_last_error());
  const std::vector<int64_t> shape = {p.n, p.cout, p.oh, p.ow};
  const float* bias_ptr = nullptr;
  int64_t bias_stride = 0;
  if (bias && bias->defined()) {
    TORCH_CHECK(bias->numel() == p.cout && bias->scalar_type() == at::kFloat && on_device(*bias), "Vulkan convolution: bias shape/dtype mismatch");
    bias_ptr = bias->const_data_ptr<float>();
    bias_stride = bias->dim() ? bias->stride(bias->dim() - 1) : 0;
  }
  b200_view4 res{nullptr, {0, 0, 0, 0}};
  if (residual && residual->defined()) {
    require_fp32_device(*residual);
    TORCH_CHECK(residual->sizes() == at::IntArrayRef(shape), "conv2d_fused: the residual must have the result's shape");
    res = view_of(*residual);
  }
  // the channels-last epilogue belongs to the strip kernel; everything else produces the dense layout first
  const bool strip = channels_last_out && b200_conv2d_select(&p, B200_PHASE_FORWARD, B200_ALGO_TC, workspace_limit()) == B200_ALGO_TC &&
                     b200_conv2d_tc_route(&p, B200_PHASE_FORWARD, view_of(input)) == 0;
  at::Tensor direct, dense;
  bool last_cl = false;
  const std::string layouts = std::to_string(layout_class(input)) + std::to_string(layout_class(weight)) + "f";
  plan_and_run(p, B200_PHASE_FORWARD, input.options(), layouts, [&](int algo, void* ws, size_t ws_bytes) {
    const int resolved = b200_conv2d_select(&p, B200_PHASE_FORWARD, algo, workspace_limit());
    const bool cl_now = strip && resolved == B200_ALGO_TC && ws_bytes >= b200_conv2d_workspace(&p, B200_PHASE_FORWARD, B200_ALGO_TC, workspace_limit());
    at::Tensor& target = cl_now ? direct : dense;
    last_cl = cl_now;
    if (!target.defined())
      target = at::empty(shape, input.options().memory_format(cl_now ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous));
    return b200_conv2d_forward_fused(&p, view_of(input), view_of(weight), bias_ptr, bias_stride, res, relu ? 1 : 0, target.data_ptr<float>(),
                                     cl_now ? 1 : 0, ws, ws_bytes, algo, backend_stream());
  });
  // the last run is the recorded plan's (the tuner's trials come first): its target holds the result
  if (last_cl) return direct;
  if (!channels_last_out) return dense;
  auto out = at::empty(shape, input.options().memory_format(at::MemoryFormat::ChannelsLast));
  device_assign(out, dense);
  return out;
}

// ---- sum over a dimension list -------------------------------------------------------------------------
// The one reduction the autograd graphs of this backend's operators need: expand's backward (`sum_to_size`) for a
// broadcast attention mask or grouped-query key / value heads, and `.sum()` of a result.  FP32 only, any strides
// (reference: sum_dim / sum_all, csrc/ops/reduce.cpp:24-35; its integer and fallback branches are not built).
static at::Tensor sum_dim(const at::Tensor& x, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype) {
  TORCH_CHECK(on_device(x) && x.scalar_type() == at::kFloat && dtype.value_or(at::kFloat) == at::kFloat,
              "Vulkan sum: only FP32 tensors are implemented by this backend build");
  TORCH_CHECK(x.dim() <= 8, "Vulkan sum: at most 8 dimensions");
  std::array<unsigned char, 8> reduce{};
  if (!dim.has_value() || dim->empty()) {
    for (int64_t d = 0; d < x.dim(); ++d) reduce[d] = 1;
  } else {
    for (int64_t d : *dim) reduce[at::maybe_wrap_dim(d, x.dim())] = 1;
  }
  std::vector<int64_t> shape;
  for (int64_t d = 0; d < x.dim(); ++d) {
    if (!reduce[d]) shape.push_back(x.size(d));
    else if (keepdim) shape.push_back(1);
  }
  auto out = at::empty(shape, x.options().memory_format(at::MemoryFormat::Contiguous));
  if (out.numel())
    B200_TORCH_CHECK(b200_sum_strided(out.data_ptr<float>(), x.numel() ? x.const_data_ptr<float>() : nullptr, (int)x.dim(),
                                      x.sizes().data(), x.strides().data(), reduce.data(), backend_stream()));
  return out;
}
static at::Tensor sum_all(const at::Tensor& x, std::optional<at::ScalarType> dtype) { return sum_dim(x, std::nullopt, false, dtype); }

// ---- mm / addmm ----------------------------------------------------------------------------------
static void gemm_into(const at::Tensor& a, const at::Tensor& b, const float* bias, float alpha, float beta,
                      at::Tensor& out) {
  B200_TORCH_CHECK(b200_gemm(a.size(0), b.size(1), a.size(1), a.const_data_ptr<float>(), a.stride(0), a.stride(1),
                             b.const_data_ptr<float>(), b.stride(0), b.stride(1), bias, alpha, beta,
                             out.data_ptr<float>(), B200_ALGO_AUTO, backend_stream()));
}
static void check_mm(const at::Tensor& a, const at::Tensor& b) {
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "mm: both arguments must be matrices");
  TORCH_CHECK(a.size(1) == b.size(0), "mm: matrix shapes cannot be multiplied (", a.size(0), "x", a.size(1), " and ",
              b.size(0), "x", b.size(1), ")");
  TORCH_CHECK(on_device(a) && on_device(b) && a.scalar_type() == at::kFloat && b.scalar_type() == at::kFloat,
              "Vulkan mm supports FP32 Vulkan tensors only");
}
static at::Tensor mm(const at::Tensor& a, const at::Tensor& b) {
  check_mm(a, b);
  auto out = at::empty({a.size(0), b.size(1)}, a.options());
  if (!out.numel()) return out;
  if (!a.size(1)) return torch_vulkan::zero_(out);
  gemm_into(a, b, nullptr, 1.f, 0.f, out);
  return out;
}
static at::Tensor& mm_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {
  check_mm(a, b);
  const std::vector<int64_t> shape = {a.size(0), b.size(1)};
  if (out.sizes() != at::IntArrayRef(shape)) {
    std::vector<c10::SymInt> sz(shape.begin(), shape.end());
    resize_(out, sz, std::nullopt);
  }
  if (!out.numel()) return out;
  // the output may alias an operand or be a strided view: compute into a fresh tensor first
  auto result = torch_vulkan::mm(a, b);
  copy_from(result, out, false);
  return out;
}
static at::Tensor addmm(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta,
                        const at::Scalar& alpha) {
  TORCH_CHECK(mat1.dim() == 2 && mat2.dim() == 2, "addmm: mat1 and mat2 must be matrices");
  TORCH_CHECK(mat1.size(1) == mat2.size(0), "addmm: matrix shapes cannot be multiplied");
  TORCH_CHECK(self.device() == mat1.device() && self.device() == mat2.device(),
              "addmm: all tensors must be on the same device");
  TORCH_CHECK(self.scalar_type() == mat1.scalar_type() && self.scalar_type() == mat2.scalar_type(),
              "addmm: all tensors must have the same dtype");
  const std::vector<int64_t> shape = {mat1.size(0), mat2.size(1)};
  const auto expanded = self.expand(shape);  // validates broadcasting even when beta is zero
  check_mm(mat1, mat2);
  auto out = at::empty(shape, mat1.options());
  if (!out.numel()) return out;
  const float b = beta.toFloat(), a = alpha.toFloat();
  TORCH_CHECK(self.dim() <= 1 || (self.dim() == 2 && self.size(0) == 1) || b == 0.f,
              "Vulkan addmm: only a bias broadcast along rows (1-D, or [1,N]) is fused by this backend build");
  at::Tensor bias = device_contiguous(self.dim() == 0 ? self.expand({shape[1]}) : self.reshape({-1}).expand({shape[1]}));
  gemm_into(mat1, mat2, bias.const_data_ptr<float>(), a, b, out);
  return out;
}

// ---- bmm -------------------------------------------------------------------------------------------
// bmm / bmm.out of the reference (csrc/ops/bmm.cpp:16-110): rank-3 FP32 operands with arbitrary
// strides (transposed, offset, batch-broadcast views are read in place), zeros for an empty
// contraction.  Integer and complex operands, which the reference sends elsewhere, are not built.
static at::Tensor bmm(const at::Tensor& a, const at::Tensor& b) {
  TORCH_CHECK(a.device() == b.device() && a.dim() == 3 && b.dim() == 3 && a.size(0) == b.size(0) && a.size(2) == b.size(1),
              "Vulkan bmm: expected matching batch dimensions and contraction size");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "Vulkan bmm: dtype mismatch");
  TORCH_CHECK(on_device(a) && a.scalar_type() == at::kFloat, "Vulkan bmm supports FP32 Vulkan tensors only");
  const int64_t batch = a.size(0), m = a.size(1), k = a.size(2), n = b.size(2);
  auto out = at::empty({batch, m, n}, a.options());
  if (!out.numel()) return out;
  if (k == 0) return torch_vulkan::zero_(out);
  B200_TORCH_CHECK(b200_bmm(batch, m, n, k, a.const_data_ptr<float>(), a.stride(0), a.stride(1), a.stride(2),
                            b.const_data_ptr<float>(), b.stride(0), b.stride(1), b.stride(2), out.data_ptr<float>(),
                            B200_ALGO_AUTO, backend_stream()));
  return out;
}
static at::Tensor& bmm_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {
  TORCH_CHECK(out.device() == a.device() && a.device() == b.device(), "Vulkan bmm.out: all tensors must be on the same device");
  auto result = torch_vulkan::bmm(a, b);  // the destination may alias an operand or be a strided view
  if (out.sizes() != result.sizes()) {
    std::vector<c10::SymInt> sz(result.sizes().begin(), result.sizes().end());
    resize_(out, sz, std::nullopt);
  }
  if (out.numel()) copy_from(result, out, false);
  return out;
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("empty.memory_format", &empty_memory_format);
  m.impl("empty_strided", &empty_strided);
  m.impl("_copy_from", &copy_from);
  m.impl("_copy_from_and_resize", &copy_from_and_resize);
  m.impl("_local_scalar_dense", &local_scalar_dense);
  m.impl("fill_.Scalar", &fill_scalar);
  m.impl("zero_", &zero_);
  m.impl("resize_", &resize_);
  m.impl("view", &view);
  m.impl("as_strided", &as_strided);
  m.impl("_reshape_alias", &reshape_alias);
  m.impl("convolution_overrideable", &convolution_overrideable);
  m.impl("convolution_backward_overrideable", &convolution_backward_overrideable);
  m.impl("sum.dim_IntList", &sum_dim);
  m.impl("sum", &sum_all);
  m.impl("mm", &mm);
  m.impl("mm.out", &mm_out);
  m.impl("addmm", &addmm);
  m.impl("bmm", &bmm);
  m.impl("bmm.out", &bmm_out);
}

TORCH_LIBRARY_FRAGMENT(torch_vulkan, m) {
  m.def("conv2d_fused(Tensor input, Tensor weight, Tensor? bias, Tensor? residual, bool relu, int[2] stride, int[2] padding, "
        "int[2] dilation, int groups, bool channels_last_out) -> Tensor");
}

TORCH_LIBRARY_IMPL(torch_vulkan, PrivateUse1, m) { m.impl("conv2d_fused", &conv2d_fused); }

}  // namespace torch_vulkan
