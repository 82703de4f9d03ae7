// Shared declarations of the PyTorch PrivateUse1 ("vulkan") extension.  The extension holds
// host logic only; every byte moved and every FLOP computed on the device goes through the
// C ABI in include/b200conv.h.
#pragma once
#include <ATen/ATen.h>
#include <c10/core/Allocator.h>

#include <cstdint>
#include <map>
#include <string>

#include "../../../include/b200conv.h"

namespace torch_vulkan {

// TORCH_CHECK on a C-ABI status, carrying the library's message.
#define B200_TORCH_CHECK(expr)                                                       \
  do {                                                                               \
    const int rc__ = (expr);                                                         \
    TORCH_CHECK(rc__ >= 0, "Vulkan backend (B200): ", b200_last_error());            \
  } while (0)

// All logical streams share one in-order CUDA stream, as all streams of the reference share
// one queue (csrc/torch_vulkan.cpp:34-35,91-94).
void* backend_stream();
c10::Allocator* backend_allocator();
void validate_device(c10::Device d);  // "only logical device 0" (csrc/vulkan_device.h:8)

// counters read by torch_vulkan.execution_stats() (csrc/execution_audit.h:7-10)
struct ExecutionStats {
  uint64_t cpu_fallback_calls = 0, host_read_calls = 0, host_read_bytes = 0, host_read_max_bytes = 0;
};
ExecutionStats& execution_stats();
void note_host_read(size_t bytes);

std::map<std::string, uint64_t> conv_dispatch_stats();
void clear_conv_dispatch_cache();

}  // namespace torch_vulkan
