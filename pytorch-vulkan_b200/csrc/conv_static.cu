// dWeight for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a weight
// gradient: an application that has handed the whole device to its own memory pool (a further
// cudaMalloc fails, or steals from the pool), or a latency-critical loop that cannot afford the
// implicit device-wide synchronisation cudaMalloc and cudaFree may perform.  The regular entry
// point, b200_conv2d_dweight, leaves the split-K scratch to the caller; this variant carries its
// own: a fixed array in the library's device image.  It never calls cudaMalloc, cudaFree or any
// allocating routine, and it needs b200_init to have run earlier (initialisation allocates; this
// call does not).
//
// Cost and limits, stated plainly:
//  * the array is B200_STATIC_SCRATCH_BYTES (16 MiB) and every GPU that loads the library holds
//    it until the process exits, whether or not this entry point is ever called;
//  * a gradient is accepted only if two split-K partials of it fit (2 * numel(dW) * 4 bytes
//    <= 16 MiB), otherwise the call fails with B200_EWORKSPACE and a message naming both sizes;
//  * all calls share the one array.  Each call overwrites every partial it later reads, so
//    nothing has to be cleared between calls, but two calls whose kernels overlap on the GPU
//    (different streams, or different host threads on different streams) race on it: issue them
//    on one stream, or order them with events;
//  * the first call on a device looks up the array's device address (cudaGetSymbolAddress) and
//    caches it; make that first call outside any stream capture.
#include "common.cuh"

#include <algorithm>
#include <mutex>

namespace b200 {

constexpr size_t kStaticScratchBytes = B200_STATIC_SCRATCH_BYTES;

// In host code this name is only a handle for the runtime: it is not a device address and must
// never be handed to a kernel.  The address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

static std::mutex g_static_mutex;
static float* g_static_address[64] = {};  // per device ordinal, filled on first use

// The caller has run ensure_init() just before, which makes the library's device current on this
// thread, so the ordinal read here is the library's own (one device per process); the address is
// resolved with that device current, as cudaGetSymbolAddress requires.
static int static_scratch_address(float** out) {
  int dev = -1;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200_EINVAL, "device ordinal %d is outside the supported range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_address[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static split-K scratch)");
    if (!p) return fail(B200_ECUDA, "static split-K scratch has no device address");
    g_static_address[dev] = static_cast<float*>(p);
  }
  *out = g_static_address[dev];
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_conv2d_dweight_static(const b200_conv_params* p, b200_view4 x, b200_view4 dy, float* dw,
                                          void* stream) {
  if (!p) return fail(B200_EINVAL, "null convolution parameters");
  if (!(p->n > 0 && p->cin > 0 && p->cout > 0 && p->h > 0 && p->w > 0 && p->kh > 0 && p->kw > 0 && p->oh > 0 &&
        p->ow > 0 && p->sh > 0 && p->sw > 0 && p->dh > 0 && p->dw > 0 && p->ph >= 0 && p->pw >= 0 &&
        p->groups > 0 && p->cin % p->groups == 0 && p->cout % p->groups == 0))
    return fail(B200_EINVAL, "convolution: invalid shapes or parameters");
  if (!x.ptr || !dy.ptr || !dw) return fail(B200_EINVAL, "convolution dWeight: null tensor");
  if (!library_is_initialised())
    return fail(B200_ECUDA, "b200_conv2d_dweight_static: call b200_init first (initialisation allocates, this call does not)");
  if (int rc = ensure_init()) return rc;  // already initialised: only makes the library's device current
  const ConvGeom g = to_geom(*p);
  const long long positions = (long long)g.n * g.oh * g.ow;
  const long long cols = (long long)g.cig * g.kh * g.kw;
  const size_t dw_bytes = (size_t)g.cout * cols * sizeof(float);
  int splits = 1, span = (int)positions;
  float* scratch = nullptr;
  if (positions > 256) {
    if (2 * dw_bytes > kStaticScratchBytes)
      return fail(B200_EWORKSPACE,
                  "b200_conv2d_dweight_static: this weight gradient is %zu bytes and two split-K partials of it "
                  "exceed the %zu-byte static workspace; use b200_conv2d_dweight with caller-provided scratch",
                  dw_bytes, kStaticScratchBytes);
    // Enough partials for about four CTAs per SM, at most what the array holds; spans stay
    // multiples of the K tile (16 positions).
    const long long tiles = div_up64(cols, 64) * div_up64(g.cog, 64) * g.groups;
    long long want = std::max<long long>(2, div_up64(4ll * sm_count(), tiles));
    want = std::min<long long>(want, div_up64(positions, 256));
    want = std::min<long long>(want, (long long)(kStaticScratchBytes / dw_bytes));
    want = std::max<long long>(want, 2);
    const long long s = div_up64(div_up64(positions, want), 16) * 16;
    span = (int)s;
    splits = (int)div_up64(positions, s);
    if (splits > 1)
      if (int rc = static_scratch_address(&scratch)) return rc;
  }
  note_kernel(splits > 1 ? "simt_igemm_dweight+finalize(static scratch)" : "simt_igemm_dweight");
  return simt_igemm_dweight(g, to_view(x), to_view(dy), dw, scratch, splits, span, (cudaStream_t)stream);
}
