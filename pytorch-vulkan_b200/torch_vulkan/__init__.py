"""torch_vulkan: drop-in device module for the "vulkan" PrivateUse1 backend, B200 edition.

Same entry points as the reference package (torch_vulkan/__init__.py:56-257 of the reference):
importing it loads ``_C``, which renames PrivateUse1 to "vulkan", installs the device guard,
hooks and allocator, and registers the FP32 Conv2D operators (plus mm/addmm and the tensor
plumbing around them) whose device work runs in hand-written sm_100a CUDA kernels through the
C ABI of ``libb200conv.so``.  There is no CPU fallback: operators outside the convolution path
raise PyTorch's "not implemented for PrivateUse1" error.

    import torch, torch_vulkan
    x = torch.randn(8, 64, 56, 56).to("vulkan")
    y = torch.nn.functional.conv2d(x, w.to("vulkan"), padding=1)   # tcgen05 implicit GEMM
    y.cpu()
"""
import contextlib
import os
import sys

import torch

from torch_vulkan import _C  # registers the backend


def _tensor_vulkan(self, *args, **kwargs):
    if args:
        raise TypeError("tensor.vulkan() takes no positional arguments")
    return self.to(device="vulkan", **kwargs)


torch.Tensor.vulkan = _tensor_vulkan


def is_available() -> bool:
    """True when an sm_100 device can be bound."""
    return _C._is_available()


def is_hardware_accelerated() -> bool:
    return _C._is_hardware_accelerated()


def _validate_device(value=None):
    """The backend exposes exactly one logical device; anything else is refused, as in the reference."""
    if value is None:
        return
    if isinstance(value, torch.Stream):
        value = value.device
    if isinstance(value, int):
        kind, index = "vulkan", value
    else:
        parsed = torch.device(value)
        kind, index = parsed.type, parsed.index
    if kind != "vulkan" or (index is not None and index != 0):
        raise RuntimeError("Vulkan backend supports logical device 0")


def synchronize(device=None) -> None:
    """Wait until all queued device work has completed."""
    _validate_device(device)
    _C._synchronize()


def performance_options() -> dict:
    state = dict(_C._execution_mode())
    state["adamw_multitensor_requested"] = os.environ.get("TORCH_VULKAN_ADAMW_DISABLE_MULTITENSOR") != "1"
    return state


def gpu_timing_stats() -> dict:
    return _C._gpu_timing_stats()


def queue_stats() -> dict:
    return _C._queue_stats()


def device_name() -> str:
    return _C._device_name()


def device(index: int = 0) -> torch.device:
    return torch.device("vulkan", index)


def runtime_hotpath_stats() -> dict:
    return _C._runtime_hotpath_stats()


def cache_stats() -> dict:
    return _C._cache_stats()


def clear_algorithm_cache():
    _C._clear_algorithm_cache()


def device_count() -> int:
    return 1 if is_available() else 0


def current_device() -> int:
    return 0


def _is_in_bad_fork() -> bool:
    return False


# The backend keeps one counter-based random stream (64-bit seed, 64-bit offset; the reference's VulkanGenerator):
# attention dropout draws from it.  Random tensor factories are outside this build: tensors are drawn on the host.
def manual_seed_all(seed: int) -> None:
    _C._manual_seed(int(seed) & ((1 << 64) - 1))


def manual_seed(seed: int) -> None:
    manual_seed_all(seed)


def initial_seed() -> int:
    return _C._initial_seed()


def seed() -> None:
    manual_seed_all(int.from_bytes(os.urandom(8), "little") >> 1)


def seed_all() -> None:
    seed()


def get_rng_state(device="vulkan"):
    _validate_device(device)
    return torch.tensor([_C._initial_seed() & ((1 << 63) - 1)], dtype=torch.int64)   # the seed; the offset restarts at 0


def set_rng_state(state, device="vulkan"):
    _validate_device(device)
    manual_seed_all(int(state.reshape(-1)[0]))


torch._register_device_module("vulkan", sys.modules[__name__])
has_fp64 = False


def conv_dispatch_stats() -> dict:
    """Counters of the convolution dispatcher: ``selected_<phase>_<candidate>`` with phases
    forward/dinput/dweight/dbias and candidates direct / tiled_simt / tiled_tcgen05 / reduce /
    winograd_f4, plus the split-K totals of dWeight."""
    return _C._conv_dispatch_stats()


def clear_conv_dispatch_cache() -> None:
    _C._clear_conv_dispatch_cache()


def set_device(value):
    _validate_device(value)


def current_stream(device=None):
    _validate_device(device)
    return _C._current_stream()


def default_stream(device=None):
    _validate_device(device)
    return _C._default_stream()


def set_stream(value):
    if value is not None:
        _validate_device(value.device)
        _C._set_stream_id(value.stream_id)


def stream(value):
    return value if value is not None else contextlib.nullcontext()


class Stream(torch.Stream):
    """A stream of the one logical device (each is its own CUDA stream underneath)."""

    def __new__(cls, device="vulkan", priority=0):
        _validate_device(device)
        return torch.Stream.__new__(cls, device=device, priority=priority)


class Event(torch.Event):
    """An event of the one logical device; events cannot be shared between processes."""

    def __new__(cls, enable_timing=False, blocking=False, interprocess=False):
        if interprocess:
            raise RuntimeError("Interprocess Vulkan events are unsupported")
        options = dict(enable_timing=enable_timing, blocking=blocking)
        return torch.Event(device="vulkan", **options)


# ---- batch sharding over GPUs (one process per GPU; the reference is single-device) -------------------
def comm_unique_id() -> bytes:
    """Rank 0 creates the communicator id (128 opaque bytes) and sends it to every rank by any host channel."""
    return _C._comm_unique_id()


def comm_init(rank: int, nranks: int, unique_id: bytes, timeout_ms: int = 0) -> None:
    """Join the communicator; raises after the timeout if a rank never joins."""
    _C._comm_init(rank, nranks, unique_id, timeout_ms)


def comm_destroy() -> None:
    _C._comm_destroy()


def comm_size() -> int:
    """Number of ranks of the communicator, 0 before comm_init."""
    return _C._comm_size()


def all_reduce_(tensor: torch.Tensor) -> torch.Tensor:
    """In-place sum of a contiguous FP32 vulkan tensor over all ranks (NCCL over NVLink), queued on the
    current stream like any other operator."""
    return _C._all_reduce_(tensor)


def execution_stats():
    """CPU-fallback and host-read counters (the former stays 0: there is no fallback)."""
    return _C._execution_stats()


def reset_execution_stats():
    synchronize()
    _C._reset_execution_stats()


def device_status(clear: bool = False) -> int:
    """0 unless a bounded device-side wait of a tcgen05 kernel gave up."""
    return _C._device_status(clear)


def conv2d_fused(input, weight, bias=None, residual=None, relu=False, stride=1, padding=0, dilation=1, groups=1,
                 channels_last_out=False):
    """act(conv2d(input, weight) + bias + residual) in one device call (torch.ops.torch_vulkan.conv2d_fused), the result
    optionally produced channels-last.  Forward only: no autograd graph is recorded."""
    pair = lambda v: [v, v] if isinstance(v, int) else list(v)
    return torch.ops.torch_vulkan.conv2d_fused(input, weight, bias, residual, bool(relu), pair(stride), pair(padding),
                                               pair(dilation), int(groups), bool(channels_last_out))


from torch_vulkan import attention as _attention  # noqa: E402,F401  (routes F.scaled_dot_product_attention to the device operators)
