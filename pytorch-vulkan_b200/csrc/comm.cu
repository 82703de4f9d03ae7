// Data-parallel exchange step of the convolution path: one process per GPU, the batch sharded over
// ranks, forward and dInput rank-local, and the weight / bias gradients summed over ranks with an NCCL
// all-reduce (over NVLink / NVSwitch) on a stream the caller chooses, so that the sum of one layer's
// gradients can run under the next layer's kernels.
//
// The reference backend is single-device (csrc/torch_vulkan.cpp:105-107 of the reference: deviceCount
// is 1), so these entry points have no counterpart there.
//
// NCCL is bound at run time (dlopen of libnccl.so.2): a process that never shards loads no
// communication library, and a process that already carries NCCL (PyTorch's) shares that copy.
// Initialisation is non-blocking with a wall-clock bound: a rank that never joins makes the others
// return B200_ECUDA after the timeout, with the half-built communicator aborted, instead of hanging.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

namespace b200 {
namespace {

struct Nccl {
  void* handle = nullptr;
  decltype(&ncclGetUniqueId) get_unique_id = nullptr;
  decltype(&ncclCommInitRankConfig) init_rank_config = nullptr;
  decltype(&ncclCommGetAsyncError) async_error = nullptr;
  decltype(&ncclAllReduce) all_reduce = nullptr;
  decltype(&ncclCommDestroy) destroy = nullptr;
  decltype(&ncclCommAbort) abort = nullptr;
  decltype(&ncclGetErrorString) error_string = nullptr;
  decltype(&ncclGetVersion) version = nullptr;
};

std::mutex g_comm_mutex;
Nccl g_nccl;
ncclComm_t g_comm = nullptr;
int g_rank = -1, g_nranks = 0;
int g_timeout_ms = 60000;

int load_nccl() {
  if (g_nccl.handle) return B200_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names)
    if ((h = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
  if (!h) return fail(B200_ECUDA, "comm: libnccl.so.2 cannot be loaded (%s)", dlerror());
  Nccl t;
  t.handle = h;
  bool ok = true;
  auto sym = [&](const char* name) {
    void* p = dlsym(h, name);
    if (!p) ok = false;
    return p;
  };
  t.get_unique_id = reinterpret_cast<decltype(t.get_unique_id)>(sym("ncclGetUniqueId"));
  t.init_rank_config = reinterpret_cast<decltype(t.init_rank_config)>(sym("ncclCommInitRankConfig"));
  t.async_error = reinterpret_cast<decltype(t.async_error)>(sym("ncclCommGetAsyncError"));
  t.all_reduce = reinterpret_cast<decltype(t.all_reduce)>(sym("ncclAllReduce"));
  t.destroy = reinterpret_cast<decltype(t.destroy)>(sym("ncclCommDestroy"));
  t.abort = reinterpret_cast<decltype(t.abort)>(sym("ncclCommAbort"));
  t.error_string = reinterpret_cast<decltype(t.error_string)>(sym("ncclGetErrorString"));
  t.version = reinterpret_cast<decltype(t.version)>(sym("ncclGetVersion"));
  if (!ok) return fail(B200_ECUDA, "comm: the loaded NCCL library lacks a required symbol");
  g_nccl = t;
  return B200_OK;
}

int nccl_fail(ncclResult_t r, const char* what) {
  return fail(B200_ECUDA, "comm: %s failed: %s", what, g_nccl.error_string ? g_nccl.error_string(r) : "?");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_comm_unique_id(void* out128) {
  static_assert(sizeof(ncclUniqueId) == 128, "the unique id travels as 128 opaque bytes");
  if (!out128) return fail(B200_EINVAL, "comm: null id buffer");
  std::lock_guard<std::mutex> lock(g_comm_mutex);
  if (int rc = load_nccl()) return rc;
  ncclUniqueId id;
  const ncclResult_t r = g_nccl.get_unique_id(&id);
  if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  memcpy(out128, &id, sizeof id);
  return B200_OK;
}

int b200_comm_set_timeout_ms(int timeout_ms) {
  if (timeout_ms <= 0) return fail(B200_EINVAL, "comm: the timeout must be positive");
  std::lock_guard<std::mutex> lock(g_comm_mutex);
  g_timeout_ms = timeout_ms;
  return B200_OK;
}

int b200_comm_init(int rank, int nranks, const void* unique_id128) {
  if (nranks < 1 || rank < 0 || rank >= nranks || !unique_id128)
    return fail(B200_EINVAL, "comm: invalid rank %d of %d or null id", rank, nranks);
  if (int rc = ensure_init()) return rc;  // binds the library's device on this thread
  std::lock_guard<std::mutex> lock(g_comm_mutex);
  if (g_comm) return fail(B200_EINVAL, "comm: already initialised (rank %d of %d); destroy it first", g_rank, g_nranks);
  if (int rc = load_nccl()) return rc;
  ncclUniqueId id;
  memcpy(&id, unique_id128, sizeof id);
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;  // return at once; completion is polled below under a wall-clock bound
  // The exchange usually runs under compute kernels whose CTAs fill an SM's register file, so every SM a collective CTA
  // sits on delays one compute CTA: B200_COMM_MAX_CTAS bounds how many the all-reduce may use (unset: NCCL's choice).
  if (const char* e = getenv("B200_COMM_MAX_CTAS")) {
    const int ctas = atoi(e);
    if (ctas >= 1 && ctas <= 64) { cfg.minCTAs = 1; cfg.maxCTAs = ctas; }
  }
  // ... and B200_COMM_MIN_CTAS how few: an exchange that nothing overlaps (the default of the benchmark's sweep) is
  // served best by many
  if (const char* e = getenv("B200_COMM_MIN_CTAS")) {
    const int ctas = atoi(e);
    if (ctas >= 1 && ctas <= 64) { cfg.minCTAs = ctas; if (cfg.maxCTAs != NCCL_CONFIG_UNDEF_INT && cfg.maxCTAs < ctas) cfg.maxCTAs = ctas; }
  }
  ncclComm_t comm = nullptr;
  ncclResult_t r = g_nccl.init_rank_config(&comm, nranks, id, rank, &cfg);
  if (r != ncclSuccess && r != ncclInProgress) return nccl_fail(r, "ncclCommInitRankConfig");
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(g_timeout_ms);
  ncclResult_t state = ncclInProgress;
  while (true) {
    r = g_nccl.async_error(comm, &state);
    if (r != ncclSuccess) { state = r; break; }
    if (state != ncclInProgress) break;
    if (std::chrono::steady_clock::now() > deadline) {
      g_nccl.abort(comm);
      return fail(B200_ECUDA, "comm: rank %d of %d gave up after %d ms waiting for the other ranks (communicator aborted)",
                  rank, nranks, g_timeout_ms);
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
  if (state != ncclSuccess) {
    if (comm) g_nccl.abort(comm);
    return nccl_fail(state, "communicator initialisation");
  }
  g_comm = comm;
  g_rank = rank;
  g_nranks = nranks;
  return B200_OK;
}

int b200_comm_rank(void) { return g_comm ? g_rank : -1; }
int b200_comm_size(void) { return g_comm ? g_nranks : 0; }

int b200_allreduce_sum_f32(float* buf, size_t count, void* stream) {
  if (int rc = ensure_init()) return rc;
  if (count == 0) return B200_OK;
  if (!buf) return fail(B200_EINVAL, "comm: null buffer");
  std::lock_guard<std::mutex> lock(g_comm_mutex);
  if (!g_comm) return fail(B200_EINVAL, "comm: b200_comm_init has not been called");
  ncclResult_t r = g_nccl.all_reduce(buf, buf, count, ncclFloat32, ncclSum, g_comm, (cudaStream_t)stream);
  // a non-blocking communicator may answer "in progress" while it queues the operation
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(g_timeout_ms);
  while (r == ncclInProgress) {
    ncclResult_t state = ncclSuccess;
    const ncclResult_t q = g_nccl.async_error(g_comm, &state);
    if (q != ncclSuccess) return nccl_fail(q, "ncclCommGetAsyncError");
    r = state;
    if (r == ncclInProgress && std::chrono::steady_clock::now() > deadline) {
      g_nccl.abort(g_comm);
      g_comm = nullptr;
      return fail(B200_ECUDA, "comm: all-reduce did not enqueue within %d ms (communicator aborted)", g_timeout_ms);
    }
    if (r == ncclInProgress) {
      if (getenv("B200_COMM_POLL_SLEEP")) std::this_thread::sleep_for(std::chrono::microseconds(50));
      else std::this_thread::yield();   // the enqueue takes tens of microseconds: sleeping through it doubles the call's latency
    }
  }
  if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce");
  count_launch();
  return B200_OK;
}

int b200_comm_destroy(void) {
  std::lock_guard<std::mutex> lock(g_comm_mutex);
  if (!g_comm) return B200_OK;
  const ncclResult_t r = g_nccl.destroy(g_comm);
  g_comm = nullptr;
  g_rank = -1;
  g_nranks = 0;
  if (r != ncclSuccess && r != ncclInProgress) return nccl_fail(r, "ncclCommDestroy");
  return B200_OK;
}

}  // extern "C"
