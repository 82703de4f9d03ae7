// Runtime of the B200 Conv2D library: device selection, error text, the
// stream-ordered caching allocator, copies, streams and events.
//
// This replaces the reference's Vulkan runtime for the convolution path:
//  - VulkanContext device pick / deferred command sequence / fences
//    (csrc/vulkan_context.cpp:59-83,172-211,493-523) -> cudaSetDevice + CUDA streams/events;
//  - VulkanAllocator's exact-size free list with deferred reuse while commands are
//    queued (csrc/vulkan_allocator.cpp:33-47,123-154) -> size-bucketed free lists whose
//    blocks carry the stream and an event of their release point;
//  - conv2d_pack / native_pack strided materialisation (csrc/ops/convolution.cpp:62-99)
//    -> gather/scatter kernels used only by copy plumbing (convolution reads views in place).
#include "common.cuh"

#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace b200 {

static thread_local std::string t_error;
static thread_local const char* t_kernel = "";
std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  t_error = buf;
}
int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  t_error = buf;
  return code;
}
int cuda_fail(cudaError_t e, const char* what) {
  return fail(B200_ECUDA, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}
void note_kernel(const char* name) { t_kernel = name; }
int launch_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  return B200_OK;
}

// ---- device state ------------------------------------------------------------------------
static std::mutex g_init_mutex;
static int g_device = -1;
static int g_sms = 0;
static char g_name[256] = "";
static int* g_status_word = nullptr;

int* device_status_word() { return g_status_word; }
int read_device_status(int* out) {
  if (!g_status_word) return fail(B200_ECUDA, "device status word is not allocated");
  B200_CUDA(cudaMemcpy(out, g_status_word, sizeof(int), cudaMemcpyDeviceToHost));
  return B200_OK;
}
int clear_device_status() {
  if (g_status_word) B200_CUDA(cudaMemset(g_status_word, 0, sizeof(int)));
  return B200_OK;
}

int ensure_init() {
  if (g_device >= 0) {
    // Worker threads (autograd) start with device 0 current; keep them on the library's device.
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur != g_device) cudaSetDevice(g_device);
    return B200_OK;
  }
  return b200_init(-1);
}
bool library_is_initialised() { return g_device >= 0; }
// Planning code may run before a device is bound (host-only callers): assume a full B200.
int sm_count() { return g_sms > 0 ? g_sms : 148; }

// ---- caching allocator -------------------------------------------------------------------
struct Block {
  void* ptr = nullptr;
  size_t size = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t event = nullptr;  // recorded at the release point
};
static std::mutex g_alloc_mutex;
static std::unordered_map<void*, Block> g_live;
static std::multimap<size_t, Block> g_free;
static std::vector<cudaEvent_t> g_event_pool;
static uint64_t g_in_use = 0, g_cached = 0, g_device_allocs = 0, g_hits = 0;

static size_t round_size(size_t bytes) {
  if (bytes == 0) bytes = 1;
  if (bytes < (1u << 20)) return (bytes + 511) & ~size_t(511);
  return (bytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);
}
static cudaEvent_t take_event() {
  if (!g_event_pool.empty()) {
    cudaEvent_t e = g_event_pool.back();
    g_event_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  return e;
}
static void release_all_cached_locked() {
  for (auto& kv : g_free) {
    cudaFree(kv.second.ptr);
    if (kv.second.event) g_event_pool.push_back(kv.second.event);
  }
  g_free.clear();
  g_cached = 0;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_init(int device_ordinal) {
  std::lock_guard<std::mutex> lock(g_init_mutex);
  if (g_device >= 0) {
    if (device_ordinal >= 0 && device_ordinal != g_device)
      return fail(B200_EINVAL, "library already bound to device %d (one device per process)", g_device);
    return B200_OK;
  }
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(B200_ECUDA, "no CUDA device available (%s); this library has no CPU fallback",
                e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  int dev = device_ordinal;
  if (dev < 0) {
    // One process per GPU: honour the launcher's LOCAL_RANK when several devices are visible.
    const char* lr = getenv("LOCAL_RANK");
    dev = lr ? atoi(lr) % count : 0;
  }
  if (dev >= count) return fail(B200_EINVAL, "device ordinal %d out of range (count %d)", dev, count);
  B200_CUDA(cudaSetDevice(dev));
  cudaDeviceProp prop;
  B200_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10)
    return fail(B200_ECUDA, "device %s is sm_%d%d; this library contains sm_100a code only", prop.name,
                prop.major, prop.minor);
  snprintf(g_name, sizeof g_name, "%s", prop.name);
  g_sms = prop.multiProcessorCount;
  B200_CUDA(cudaMalloc(&g_status_word, 256));
  B200_CUDA(cudaMemset(g_status_word, 0, 256));
  g_device = dev;
  return B200_OK;
}

const char* b200_last_error(void) { return t_error.c_str(); }
const char* b200_device_name(void) { return ensure_init() == B200_OK ? g_name : ""; }
int b200_device_sm_count(void) { return ensure_init() == B200_OK ? g_sms : 0; }
uint64_t b200_launch_count(void) { return g_launches.load(); }
const char* b200_last_kernel(void) { return t_kernel; }

int b200_malloc(void** ptr, size_t bytes, void* stream) {
  if (!ptr) return fail(B200_EINVAL, "b200_malloc: null out pointer");
  if (int rc = ensure_init()) return rc;
  const size_t size = round_size(bytes);
  cudaStream_t st = (cudaStream_t)stream;
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  // Best fit in [size, size + size/4]; a block released on another stream is only
  // taken once its release point has been reached.
  for (auto it = g_free.lower_bound(size); it != g_free.end() && it->first <= size + size / 4; ++it) {
    Block b = it->second;
    if (b.stream != st && b.event && cudaEventQuery(b.event) != cudaSuccess) {
      cudaGetLastError();
      continue;
    }
    g_free.erase(it);
    if (b.event) g_event_pool.push_back(b.event);
    b.event = nullptr;
    b.stream = st;
    g_cached -= b.size;
    g_in_use += b.size;
    ++g_hits;
    g_live[b.ptr] = b;
    *ptr = b.ptr;
    return B200_OK;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, size);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaDeviceSynchronize();
    release_all_cached_locked();
    e = cudaMalloc(&p, size);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B200_ENOMEM, "out of device memory allocating %zu bytes (%llu in use)", size,
                (unsigned long long)g_in_use);
  }
  ++g_device_allocs;
  Block b;
  b.ptr = p;
  b.size = size;
  b.stream = st;
  g_live[p] = b;
  g_in_use += size;
  *ptr = p;
  return B200_OK;
}

int b200_free(void* ptr, void* stream) {
  if (!ptr) return B200_OK;
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  auto it = g_live.find(ptr);
  if (it == g_live.end()) return fail(B200_EINVAL, "b200_free: pointer %p was not allocated by b200_malloc", ptr);
  Block b = it->second;
  g_live.erase(it);
  b.stream = (cudaStream_t)stream;
  b.event = take_event();
  if (b.event && cudaEventRecord(b.event, b.stream) != cudaSuccess) {
    cudaGetLastError();
    g_event_pool.push_back(b.event);
    b.event = nullptr;
  }
  g_in_use -= b.size;
  g_cached += b.size;
  g_free.emplace(b.size, b);
  return B200_OK;
}

int b200_empty_cache(void) {
  if (g_device < 0) return B200_OK;
  B200_CUDA(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  release_all_cached_locked();
  return B200_OK;
}

int b200_mem_stats(uint64_t out[4]) {
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  out[0] = g_in_use;
  out[1] = g_cached;
  out[2] = g_device_allocs;
  out[3] = g_hits;
  return B200_OK;
}

int b200_host_alloc(void** ptr, size_t bytes) {
  if (int rc = ensure_init()) return rc;
  B200_CUDA(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocDefault));
  return B200_OK;
}
int b200_host_free(void* ptr) {
  if (ptr) B200_CUDA(cudaFreeHost(ptr));
  return B200_OK;
}

int b200_memcpy(void* dst, const void* src, size_t bytes, int kind, void* stream) {
  if (int rc = ensure_init()) return rc;
  if (bytes == 0) return B200_OK;
  cudaMemcpyKind k = kind == B200_H2D ? cudaMemcpyHostToDevice
                   : kind == B200_D2H ? cudaMemcpyDeviceToHost
                   : kind == B200_D2D ? cudaMemcpyDeviceToDevice : cudaMemcpyDefault;
  if (kind < B200_H2D || kind > B200_D2D) return fail(B200_EINVAL, "b200_memcpy: bad kind %d", kind);
  B200_CUDA(cudaMemcpyAsync(dst, src, bytes, k, (cudaStream_t)stream));
  return B200_OK;
}
int b200_memset(void* dst, int value, size_t bytes, void* stream) {
  if (int rc = ensure_init()) return rc;
  if (bytes) B200_CUDA(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
  return B200_OK;
}

int b200_stream_create(void** stream) {
  if (int rc = ensure_init()) return rc;
  cudaStream_t s;
  B200_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return B200_OK;
}
int b200_stream_destroy(void* stream) {
  if (stream) B200_CUDA(cudaStreamDestroy((cudaStream_t)stream));
  return B200_OK;
}
int b200_stream_sync(void* stream) {
  if (int rc = ensure_init()) return rc;
  B200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return B200_OK;
}
int b200_stream_query(void* stream) {
  if (int rc = ensure_init()) return rc;
  cudaError_t e = cudaStreamQuery((cudaStream_t)stream);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) { cudaGetLastError(); return 0; }
  return cuda_fail(e, "cudaStreamQuery");
}
int b200_device_sync(void) {
  if (int rc = ensure_init()) return rc;
  B200_CUDA(cudaDeviceSynchronize());
  return B200_OK;
}
int b200_event_create(void** event, int enable_timing) {
  if (int rc = ensure_init()) return rc;
  cudaEvent_t e;
  B200_CUDA(cudaEventCreateWithFlags(&e, enable_timing ? cudaEventDefault : cudaEventDisableTiming));
  *event = e;
  return B200_OK;
}
int b200_event_destroy(void* event) {
  if (event) B200_CUDA(cudaEventDestroy((cudaEvent_t)event));
  return B200_OK;
}
int b200_event_record(void* event, void* stream) {
  if (int rc = ensure_init()) return rc;
  B200_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
  return B200_OK;
}
int b200_event_sync(void* event) {
  if (int rc = ensure_init()) return rc;
  B200_CUDA(cudaEventSynchronize((cudaEvent_t)event));
  return B200_OK;
}
int b200_event_query(void* event) {
  if (int rc = ensure_init()) return rc;
  cudaError_t e = cudaEventQuery((cudaEvent_t)event);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) { cudaGetLastError(); return 0; }
  return cuda_fail(e, "cudaEventQuery");
}
int b200_stream_wait_event(void* stream, void* event) {
  if (int rc = ensure_init()) return rc;
  B200_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
  return B200_OK;
}
int b200_event_elapsed_ms(void* first, void* second, float* ms) {
  B200_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)first, (cudaEvent_t)second));
  return B200_OK;
}

}  // extern "C"

// ---- strided gather / scatter ------------------------------------------------------------
namespace b200 {
struct StridedDesc {
  int ndim;
  long long size[8];
  long long stride[8];
};

template <typename T, bool kScatter>
__global__ void __launch_bounds__(256) strided_copy_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                           StridedDesc d, long long total) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    long long r = i, addr = 0;
#pragma unroll 1
    for (int k = d.ndim - 1; k >= 0; --k) {
      const long long q = r / d.size[k];
      addr += (r - q * d.size[k]) * d.stride[k];
      r = q;
    }
    if (kScatter) dst[addr] = src[i];
    else dst[i] = src[addr];
  }
}

template <bool kScatter>
static int strided_copy(void* dst, const void* src, int ndim, const int64_t* sizes, const int64_t* strides,
                        int elem_bytes, cudaStream_t st) {
  if (int rc = ensure_init()) return rc;
  if (ndim < 0 || ndim > 8) return fail(B200_EINVAL, "strided copy supports at most 8 dimensions (got %d)", ndim);
  StridedDesc d;
  d.ndim = ndim;
  long long total = 1;
  for (int i = 0; i < ndim; ++i) {
    d.size[i] = sizes[i];
    d.stride[i] = strides[i];
    total *= sizes[i];
  }
  if (total == 0) return B200_OK;
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
  switch (elem_bytes) {
    case 1: strided_copy_kernel<uint8_t, kScatter><<<grid, 256, 0, st>>>((uint8_t*)dst, (const uint8_t*)src, d, total); break;
    case 2: strided_copy_kernel<uint16_t, kScatter><<<grid, 256, 0, st>>>((uint16_t*)dst, (const uint16_t*)src, d, total); break;
    case 4: strided_copy_kernel<uint32_t, kScatter><<<grid, 256, 0, st>>>((uint32_t*)dst, (const uint32_t*)src, d, total); break;
    case 8: strided_copy_kernel<uint64_t, kScatter><<<grid, 256, 0, st>>>((uint64_t*)dst, (const uint64_t*)src, d, total); break;
    default: return fail(B200_EINVAL, "strided copy: unsupported element size %d", elem_bytes);
  }
  count_launch();
  return launch_check("strided_copy_kernel");
}
}  // namespace b200

// ---- strided sum over a subset of the dimensions --------------------------------------------------------------------
namespace b200 {
struct ReduceDesc {
  int kept_dims, reduced_dims;
  long long kept_size[8], kept_stride[8], red_size[8], red_stride[8];
  long long red_total;
};
// One warp per result element: its lanes stride over the reduced elements (FP32 partial sums of at most
// red_total / 32 terms each), then a shuffle tree in a fixed order.
__global__ void __launch_bounds__(256) sum_strided_kernel(float* __restrict__ dst, const float* __restrict__ src, ReduceDesc d,
                                                          long long outputs) {
  const long long out = blockIdx.x * 8ll + (threadIdx.x >> 5);
  if (out >= outputs) return;
  const int lane = threadIdx.x & 31;
  long long r = out, base = 0;
  for (int k = d.kept_dims - 1; k >= 0; --k) {
    const long long q = r / d.kept_size[k];
    base += (r - q * d.kept_size[k]) * d.kept_stride[k];
    r = q;
  }
  float acc = 0.f;
  for (long long e = lane; e < d.red_total; e += 32) {
    long long t = e, off = base;
    for (int k = d.reduced_dims - 1; k >= 0; --k) {
      const long long q = t / d.red_size[k];
      off += (t - q * d.red_size[k]) * d.red_stride[k];
      t = q;
    }
    acc += src[off];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dst[out] = acc;
}
}  // namespace b200

extern "C" int b200_sum_strided(float* dst, const float* src, int ndim, const int64_t* sizes, const int64_t* strides,
                                const unsigned char* reduce, void* stream) {
  using namespace b200;
  if (int rc = ensure_init()) return rc;
  if (ndim < 0 || ndim > 8 || (ndim > 0 && (!sizes || !strides || !reduce))) return fail(B200_EINVAL, "strided sum supports at most 8 dimensions (got %d)", ndim);
  ReduceDesc d{};
  d.red_total = 1;
  long long outputs = 1;
  for (int i = 0; i < ndim; ++i) {
    if (sizes[i] < 0) return fail(B200_EINVAL, "strided sum: negative extent");
    if (reduce[i]) {
      d.red_size[d.reduced_dims] = sizes[i]; d.red_stride[d.reduced_dims++] = strides[i];
      d.red_total *= sizes[i];
    } else {
      d.kept_size[d.kept_dims] = sizes[i]; d.kept_stride[d.kept_dims++] = strides[i];
      outputs *= sizes[i];
    }
  }
  if (outputs == 0) return B200_OK;
  if (!dst || (!src && d.red_total > 0)) return fail(B200_EINVAL, "strided sum: null tensor");
  if (outputs > 8ll * 2147483647ll) return fail(B200_ERANGE, "strided sum: too many results");
  sum_strided_kernel<<<(unsigned)((outputs + 7) / 8), 256, 0, (cudaStream_t)stream>>>(dst, src, d, outputs);
  count_launch();
  return launch_check("sum_strided_kernel");
}

extern "C" int b200_gather_strided(void* dst, const void* src, int ndim, const int64_t* sizes,
                                   const int64_t* strides, int elem_bytes, void* stream) {
  return b200::strided_copy<false>(dst, src, ndim, sizes, strides, elem_bytes, (cudaStream_t)stream);
}
// strided dst += contiguous src (FP32): accumulation of partial results into a view of a larger tensor
namespace b200 {
__global__ void __launch_bounds__(256) strided_add_kernel(float* __restrict__ dst, const float* __restrict__ src, StridedDesc d, long long total) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    long long r = i, addr = 0;
#pragma unroll 1
    for (int k = d.ndim - 1; k >= 0; --k) {
      const long long q = r / d.size[k];
      addr += (r - q * d.size[k]) * d.stride[k];
      r = q;
    }
    dst[addr] += src[i];
  }
}
}  // namespace b200
extern "C" int b200_scatter_add_strided(float* dst, const float* src, int ndim, const int64_t* sizes, const int64_t* strides, void* stream) {
  using namespace b200;
  if (int rc = ensure_init()) return rc;
  if (ndim < 0 || ndim > 8) return fail(B200_EINVAL, "strided copy supports at most 8 dimensions (got %d)", ndim);
  StridedDesc d;
  d.ndim = ndim;
  long long total = 1;
  for (int i = 0; i < ndim; ++i) { d.size[i] = sizes[i]; d.stride[i] = strides[i]; total *= sizes[i]; }
  if (total == 0) return B200_OK;
  if (!dst || !src) return fail(B200_EINVAL, "strided add: null tensor");
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
  strided_add_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(dst, src, d, total);
  count_launch();
  return launch_check("strided_add_kernel");
}

extern "C" int b200_scatter_strided(void* dst, const void* src, int ndim, const int64_t* sizes,
                                    const int64_t* strides, int elem_bytes, void* stream) {
  return b200::strided_copy<true>(dst, src, ndim, sizes, strides, elem_bytes, (cudaStream_t)stream);
}
