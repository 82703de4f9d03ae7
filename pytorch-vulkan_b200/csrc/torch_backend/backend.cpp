// PrivateUse1 backend registration: device guard, hooks, allocator adaptor and the `_C`
// Python module.  Host-side mirror of the reference's csrc/torch_vulkan.cpp with the Vulkan
// engine/context/allocator replaced by the CUDA runtime behind the C ABI:
//   VulkanGuardImpl  (csrc/torch_vulkan.cpp:40-108)  -> GuardImpl below (CUDA stream + events)
//   VulkanHooks      (csrc/torch_vulkan.cpp:134-155) -> Hooks below
//   VulkanAllocator  (csrc/vulkan_allocator.cpp)     -> DeviceAllocator over b200_malloc/b200_free
//   pybind `_C`      (csrc/torch_vulkan.cpp:246-283) -> same function names
#include "backend.h"

#include <ATen/CPUGeneratorImpl.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <torch/csrc/Stream.h>
#include <torch/extension.h>

#include <atomic>
#include <mutex>

namespace torch_vulkan {

static thread_local c10::StreamId current_stream_id = 0;
static std::atomic<int64_t> next_stream_id{1};

void validate_device(c10::Device d) {
  TORCH_CHECK(d.type() == c10::DeviceType::PrivateUse1 && (!d.has_index() || d.index() == 0),
              "Vulkan backend supports only logical device 0");
}

void* backend_stream() {
  static void* stream = [] {
    void* s = nullptr;
    B200_TORCH_CHECK(b200_init(-1));
    B200_TORCH_CHECK(b200_stream_create(&s));
    return s;
  }();
  return stream;
}

ExecutionStats& execution_stats() {
  static ExecutionStats s;
  return s;
}

namespace {
std::mutex rng_mutex;
uint64_t rng_seed = 67280421310721ull, rng_offset = 0;   // PyTorch's default seed value until manual_seed is called
}  // namespace
void set_random_seed(uint64_t seed) {
  std::lock_guard<std::mutex> lock(rng_mutex);
  rng_seed = seed;
  rng_offset = 0;
}
uint64_t random_seed() {
  std::lock_guard<std::mutex> lock(rng_mutex);
  return rng_seed;
}
std::array<uint32_t, 4> reserve_random_blocks(uint64_t blocks) {
  std::lock_guard<std::mutex> lock(rng_mutex);
  TORCH_CHECK(blocks <= UINT64_MAX - rng_offset, "Vulkan RNG counter exhausted");
  const std::array<uint32_t, 4> state = {uint32_t(rng_seed), uint32_t(rng_seed >> 32), uint32_t(rng_offset), uint32_t(rng_offset >> 32)};
  rng_offset += blocks;
  return state;
}
static std::mutex stats_mutex;
void note_host_read(size_t bytes) {
  std::lock_guard<std::mutex> lock(stats_mutex);
  auto& s = execution_stats();
  ++s.host_read_calls;
  s.host_read_bytes += bytes;
  if (bytes > s.host_read_max_bytes) s.host_read_max_bytes = bytes;
}

// ---- allocator -----------------------------------------------------------------------------
struct DeviceAllocator final : public c10::Allocator {
  static void release(void* p) {
    if (p) b200_free(p, backend_stream());
  }
  c10::DataPtr allocate(size_t n) override {
    void* p = nullptr;
    if (n) B200_TORCH_CHECK(b200_malloc(&p, n, backend_stream()));
    return {p, p, &release, c10::Device(c10::DeviceType::PrivateUse1, 0)};
  }
  c10::DeleterFnPtr raw_deleter() const override { return &release; }
  void copy_data(void* dest, const void* src, std::size_t count) const override {
    B200_TORCH_CHECK(b200_memcpy(dest, src, count, B200_D2D, backend_stream()));
  }
};
c10::Allocator* backend_allocator() {
  static DeviceAllocator a;
  return &a;
}

// ---- device guard ----------------------------------------------------------------------------
struct BackendEvent {
  void* handle = nullptr;
  bool timing = false;
};

struct GuardImpl final : public c10::impl::DeviceGuardImplInterface {
  static c10::Device dev() { return c10::Device(c10::DeviceType::PrivateUse1, 0); }
  c10::DeviceType type() const override { return c10::DeviceType::PrivateUse1; }
  c10::Device exchangeDevice(c10::Device d) const override { validate_device(d); return dev(); }
  c10::Device getDevice() const override { return dev(); }
  void setDevice(c10::Device d) const override { validate_device(d); }
  void uncheckedSetDevice(c10::Device) const noexcept override {}
  c10::Stream getStream(c10::Device) const override { return c10::Stream(c10::Stream::UNSAFE, dev(), current_stream_id); }
  c10::Stream getDefaultStream(c10::Device d) const override { validate_device(d); return c10::Stream(c10::Stream::DEFAULT, dev()); }
  c10::Stream exchangeStream(c10::Stream s) const override {
    auto old = c10::Stream(c10::Stream::UNSAFE, dev(), current_stream_id);
    current_stream_id = s.id();
    return old;
  }
  c10::Stream getNewStream(c10::Device d, int priority = 0) const override {
    validate_device(d);
    TORCH_CHECK(priority == 0, "Vulkan stream priorities are unsupported");
    return c10::Stream(c10::Stream::UNSAFE, dev(), next_stream_id.fetch_add(1));
  }
  c10::Stream getStreamFromGlobalPool(c10::Device d, bool = false) const override { return getNewStream(d, 0); }
  c10::DeviceIndex deviceCount() const noexcept override { return 1; }
  bool queryStream(const c10::Stream&) const override { return b200_stream_query(backend_stream()) == 1; }
  void synchronizeStream(const c10::Stream&) const override { B200_TORCH_CHECK(b200_stream_sync(backend_stream())); }
  void synchronizeDevice(const c10::DeviceIndex index) const override {
    TORCH_CHECK(index == 0 || index == -1, "Invalid Vulkan device");
    B200_TORCH_CHECK(b200_device_sync());
  }
  void record(void** event, const c10::Stream& stream, const c10::DeviceIndex index, const c10::EventFlag flag) const override {
    validate_device(stream.device());
    TORCH_CHECK(index == -1 || index == 0, "Invalid Vulkan event device");
    TORCH_CHECK(flag != c10::EventFlag::INVALID, "Invalid event flag");
    const bool timing = flag == c10::EventFlag::BACKEND_DEFAULT;
    auto* e = static_cast<BackendEvent*>(*event);
    if (e && e->timing != timing) {
      b200_event_destroy(e->handle);
      e->handle = nullptr;
    }
    if (!e) {
      e = new BackendEvent();
      *event = e;
    }
    if (!e->handle) B200_TORCH_CHECK(b200_event_create(&e->handle, timing ? 1 : 0));
    e->timing = timing;
    B200_TORCH_CHECK(b200_event_record(e->handle, backend_stream()));
  }
  void destroyEvent(void* event, const c10::DeviceIndex) const noexcept override {
    auto* e = static_cast<BackendEvent*>(event);
    if (!e) return;
    if (e->handle) b200_event_destroy(e->handle);
    delete e;
  }
  void block(void*, const c10::Stream&) const override {
    // every logical stream maps to the one in-order CUDA stream: a recorded event already
    // precedes whatever is enqueued next
  }
  bool queryEvent(void* event) const override {
    auto* e = static_cast<BackendEvent*>(event);
    return !e || !e->handle || b200_event_query(e->handle) == 1;
  }
  void synchronizeEvent(void* event) const override {
    auto* e = static_cast<BackendEvent*>(event);
    if (e && e->handle) B200_TORCH_CHECK(b200_event_sync(e->handle));
  }
  double elapsedTime(void* first, void* second, const c10::DeviceIndex) const override {
    auto* a = static_cast<BackendEvent*>(first);
    auto* b = static_cast<BackendEvent*>(second);
    TORCH_CHECK(a && b && a->handle && b->handle, "Both events must be recorded");
    TORCH_CHECK(a->timing && b->timing, "Event timing was not enabled");
    TORCH_CHECK(queryEvent(first) && queryEvent(second), "Events have not completed");
    float ms = 0.f;
    B200_TORCH_CHECK(b200_event_elapsed_ms(a->handle, b->handle, &ms));
    return ms;
  }
  void recordDataPtrOnStream(const c10::DataPtr&, const c10::Stream&) const override {}
};
C10_REGISTER_GUARD_IMPL(PrivateUse1, GuardImpl);

// ---- hooks -------------------------------------------------------------------------------------
struct Hooks final : public at::PrivateUse1HooksInterface {
  // Device RNG is outside the convolution path; a host generator stands in so that code which
  // only asks for "the default generator" keeps working.
  const at::Generator& getDefaultGenerator(c10::DeviceIndex index) const override {
    TORCH_CHECK(index == -1 || index == 0, "Invalid Vulkan generator device");
    static at::Generator g = at::detail::createCPUGenerator();
    return g;
  }
  at::Generator getNewGenerator(c10::DeviceIndex = -1) const override { return at::detail::createCPUGenerator(); }
  bool isBuilt() const override { return true; }
  bool isAvailable() const override { return true; }
  bool hasPrimaryContext(c10::DeviceIndex index) const override { return index == 0; }
  c10::DeviceIndex deviceCount() const override { return 1; }
  c10::DeviceIndex getCurrentDevice() const override { return 0; }
  void setCurrentDevice(c10::DeviceIndex index) const override {
    TORCH_CHECK(index == 0, "Vulkan backend supports only logical device 0");
  }
  c10::DeviceIndex exchangeDevice(c10::DeviceIndex index) const override { setCurrentDevice(index); return 0; }
  c10::DeviceIndex maybeExchangeDevice(c10::DeviceIndex index) const override { return exchangeDevice(index); }
  c10::Device getDeviceFromPtr(void*) const override { return c10::Device(c10::DeviceType::PrivateUse1, 0); }
  void init() const override { backend_stream(); }
  void resizePrivateUse1Bytes(const c10::Storage& storage, size_t bytes) const override {
    auto* impl = storage.unsafeGetStorageImpl();
    const size_t old_bytes = impl->nbytes();
    if (bytes <= old_bytes) return;
    auto next = backend_allocator()->allocate(bytes);
    if (old_bytes && impl->data())
      B200_TORCH_CHECK(b200_memcpy(next.get(), impl->data(), old_bytes, B200_D2D, backend_stream()));
    impl->set_data_ptr_noswap(std::move(next));
    impl->set_nbytes(bytes);
    impl->set_allocator(backend_allocator());
    impl->set_resizable(true);
  }
};
static Hooks backend_hooks;

// ---- Python module ---------------------------------------------------------------------------
static py::dict dict_of(const std::map<std::string, uint64_t>& m) {
  py::dict d;
  for (const auto& kv : m) d[py::str(kv.first)] = kv.second;
  return d;
}

static bool is_available() { return b200_init(-1) == B200_OK; }

PYBIND11_MODULE(_C, m) {
  m.def("_conv_dispatch_stats", [] { return dict_of(conv_dispatch_stats()); });
  m.def("_clear_conv_dispatch_cache", &clear_conv_dispatch_cache);
  m.def("_set_shader_dir", [](const std::string&) {});  // no shaders: kernels are linked in
  m.def("_device_name", [] {
    B200_TORCH_CHECK(b200_init(-1));
    return std::string(b200_device_name());
  });
  m.def("_is_available", &is_available);
  m.def("_is_hardware_accelerated", &is_available);
  m.def("_synchronize", [] { B200_TORCH_CHECK(b200_stream_sync(backend_stream())); });
  m.def("_execution_stats", [] {
    const auto& s = execution_stats();
    py::dict d;
    d["cpu_fallback_calls"] = s.cpu_fallback_calls;
    d["host_read_calls"] = s.host_read_calls;
    d["host_read_bytes"] = s.host_read_bytes;
    d["host_read_max_bytes"] = s.host_read_max_bytes;
    return d;
  });
  m.def("_reset_execution_stats", [] { execution_stats() = ExecutionStats(); });
  m.def("_manual_seed", [](uint64_t seed) { set_random_seed(seed); });
  m.def("_initial_seed", [] { return random_seed(); });
  m.def("_current_stream", [] {
    return py::reinterpret_steal<py::object>(THPStream_Wrap(
        c10::Stream(c10::Stream::UNSAFE, c10::Device(c10::DeviceType::PrivateUse1, 0), current_stream_id)));
  });
  m.def("_default_stream", [] {
    return py::reinterpret_steal<py::object>(
        THPStream_Wrap(c10::Stream(c10::Stream::DEFAULT, c10::Device(c10::DeviceType::PrivateUse1, 0))));
  });
  m.def("_set_stream_id", [](int64_t id) {
    TORCH_CHECK(id >= 0 && id < next_stream_id.load(), "Unknown Vulkan stream");
    current_stream_id = id;
  });
  m.def("_execution_mode", [] {
    py::dict d;  // memory is always device-resident and work is always queued asynchronously
    d["gpu_resident"] = true;
    d["deferred_submissions"] = true;
    return d;
  });
  m.def("_queue_stats", [] {
    py::dict d;
    d["submissions"] = b200_launch_count();
    d["recorded_ops"] = b200_launch_count();
    d["largest_batch"] = 1;
    return d;
  });
  m.def("_gpu_timing_stats", [] { return py::dict(); });
  m.def("_runtime_hotpath_stats", [] { return py::dict(); });
  m.def("_cache_stats", [] {
    uint64_t s[4] = {0, 0, 0, 0};
    b200_mem_stats(s);
    py::dict d;
    for (const char* k : {"algo_hits", "algo_misses", "seq_reuses", "seq_creates", "algo_evictions", "bound_algorithms",
                          "bound_cached_buffer_bytes", "pipeline_hits", "pipeline_misses", "pipeline_evictions",
                          "pipeline_entries"})
      d[k] = 0;
    d["allocator_bytes_in_use"] = s[0];
    d["allocator_bytes_cached"] = s[1];
    d["allocator_device_allocs"] = s[2];
    d["allocator_cache_hits"] = s[3];
    return d;
  });
  m.def("_clear_algorithm_cache", [] { b200_empty_cache(); });
  m.def("_device_status", [](bool clear) {
    int v = 0;
    B200_TORCH_CHECK(b200_device_status(&v, clear ? 1 : 0));
    return v;
  });
  // data-parallel exchange: NCCL behind the C ABI, on the backend's current stream
  m.def("_comm_unique_id", [] {
    char id[128];
    B200_TORCH_CHECK(b200_comm_unique_id(id));
    return py::bytes(id, sizeof id);
  });
  m.def("_comm_init", [](int rank, int nranks, const std::string& id, int timeout_ms) {
    TORCH_CHECK(id.size() == 128, "the communicator id is 128 bytes");
    if (timeout_ms > 0) B200_TORCH_CHECK(b200_comm_set_timeout_ms(timeout_ms));
    B200_TORCH_CHECK(b200_comm_init(rank, nranks, id.data()));
  });
  m.def("_comm_destroy", [] { B200_TORCH_CHECK(b200_comm_destroy()); });
  m.def("_comm_size", [] { return b200_comm_size(); });
  m.def("_all_reduce_", [](at::Tensor& t) {
    TORCH_CHECK(t.device().type() == c10::DeviceType::PrivateUse1, "all_reduce_: expected a vulkan tensor");
    TORCH_CHECK(t.scalar_type() == at::kFloat && t.is_contiguous(), "all_reduce_: expected a contiguous FP32 tensor");
    if (t.numel())
      B200_TORCH_CHECK(b200_allreduce_sum_f32(t.data_ptr<float>(), (size_t)t.numel(), backend_stream()));
    return t;
  });
  m.def("_launch_count", [] { return b200_launch_count(); });
  m.def("_last_kernel", [] { return std::string(b200_last_kernel()); });

  c10::register_privateuse1_backend("vulkan");
  at::RegisterPrivateUse1HooksInterface(&backend_hooks);
  c10::SetAllocator(c10::DeviceType::PrivateUse1, backend_allocator());
}

}  // namespace torch_vulkan
