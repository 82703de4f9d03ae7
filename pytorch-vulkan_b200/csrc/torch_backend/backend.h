// Shared declarations of the PyTorch PrivateUse1 ("vulkan") extension.  The extension holds
// host logic only; every byte moved and every FLOP computed on the device goes through the
// C ABI in include/b200conv.h.
#pragma once
#include <array>
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

// The device random stream: a 64-bit seed and a 64-bit counter offset, as VulkanGenerator keeps them
// (csrc/vulkan_generator.h:11-19 of the reference).  reserve_random_blocks hands out {seed low, seed high, offset low,
// offset high} and advances the offset by `blocks` (csrc/vulkan_generator.cpp:17-20); set_random_seed restarts the
// stream at offset 0 (torch_vulkan.manual_seed).
void set_random_seed(uint64_t seed);
uint64_t random_seed();
std::array<uint32_t, 4> reserve_random_blocks(uint64_t blocks);
void note_host_read(size_t bytes);

std::map<std::string, uint64_t> conv_dispatch_stats();
void clear_conv_dispatch_cache();

}  // namespace torch_vulkan
