// Shared host/device helpers of the B200 Conv2D library (internal; the public
// surface is include/b200conv.h).
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/b200conv.h"

namespace b200 {

// ---- error reporting ---------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define B200_CUDA(expr)                                         \
  do {                                                          \
    cudaError_t e__ = (expr);                                   \
    if (e__ != cudaSuccess) return ::b200::cuda_fail(e__, #expr); \
  } while (0)

int ensure_init();
bool library_is_initialised();  // true once b200_init has bound a device
int sm_count();
extern std::atomic<uint64_t> g_launches;
void note_kernel(const char* name);
inline void count_launch(int n = 1) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// Checks the launch of the kernel named `what`; to be used right after <<<>>>.
int launch_check(const char* what);

// ---- device-side geometry ------------------------------------------------------------------
struct View4 {
  const float* ptr;
  long long s0, s1, s2, s3;
};
inline View4 to_view(const b200_view4& v) { return {v.ptr, v.stride[0], v.stride[1], v.stride[2], v.stride[3]}; }
inline View4 contiguous_view(const float* p, long long d1, long long d2, long long d3) {
  return {p, d1 * d2 * d3, d2 * d3, d3, 1};
}

struct ConvGeom {
  int n, cin, cout, h, w, kh, kw, oh, ow, sh, sw, ph, pw, dh, dw, groups;
  int cig, cog;  // channels per group
};
inline ConvGeom to_geom(const b200_conv_params& p) {
  return {p.n, p.cin, p.cout, p.h, p.w, p.kh, p.kw, p.oh, p.ow, p.sh, p.sw, p.ph, p.pw, p.dh, p.dw, p.groups,
          p.cin / p.groups, p.cout / p.groups};
}

static inline int64_t div_up64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Division of 0 <= n < 2^31 by a divisor fixed at launch time as one multiply-high and a shift:
// with s = ceil(log2 d) and m = ceil(2^(31+s) / d), floor(n / d) = (n * m) >> (31 + s) because the
// excess m*d - 2^(31+s) is below d <= 2^s and n is below 2^31.  Kernels use it to turn a padded
// pixel index into (image, row, column) without the long division sequence.
struct FastDiv {
  uint32_t d = 1, mul = 0, shr = 0;
  FastDiv() = default;
  explicit FastDiv(uint32_t divisor) : d(divisor) {
    if (d > 1) {
      uint32_t s = 0;
      while ((1ull << s) < d) ++s;
      mul = (uint32_t)(((1ull << (31 + s)) + d - 1) / d);
      shr = s - 1;  // after taking the high 32 bits of the product
    }
  }
#ifdef __CUDACC__
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : (__umulhi(n, mul) >> shr); }
#endif
  uint32_t host_div(uint32_t n) const { return d == 1 ? n : (uint32_t)(((uint64_t)n * mul) >> 32) >> shr; }
};

// ---- kernel families (each returns a B200_* code) -------------------------------------------
// CUDA-core paths (conv_simt.cu)
int simt_direct(const ConvGeom& g, int phase, View4 a, View4 b, const float* bias, long long bias_stride,
                float* out, cudaStream_t st);
int simt_igemm_forward(const ConvGeom& g, View4 x, View4 w, const float* bias, long long bias_stride, float* y,
                       cudaStream_t st);
int simt_igemm_dinput(const ConvGeom& g, View4 dy, View4 w, float* dx, cudaStream_t st);
// splits >= 1; when splits > 1 `partial` holds splits*numel(dw) floats and a finalize pass sums
// them in ascending order into dw.
int simt_igemm_dweight(const ConvGeom& g, View4 x, View4 dy, float* dw, float* partial, int splits, int span,
                       cudaStream_t st);
int finalize_splits(const float* partial, float* out, long long count, int splits, cudaStream_t st);
int dbias_reduce(const ConvGeom& g, View4 dy, float* db, float* partial, int slabs, cudaStream_t st);
int simt_gemm(long long M, long long N, long long K, const float* A, long long sa0, long long sa1, const float* B,
              long long sb0, long long sb1, const float* bias, float alpha, float beta, float* C, cudaStream_t st);

// grouped 3x3 convolutions with 4 or 8 channels per group (conv_group_small.cu)
bool group_small_supported(const ConvGeom& g);
size_t group_small_dweight_workspace(const ConvGeom& g);
int group_small_conv(const ConvGeom& g, bool is_dx, View4 in, View4 w, const float* bias, long long bias_stride, float* out, cudaStream_t st);
int group_small_dweight(const ConvGeom& g, View4 x, View4 dy, float* dw, float* ws, size_t ws_bytes, cudaStream_t st);

// tcgen05 paths (conv_tc.cu)
bool tc_supported(const ConvGeom& g, int phase);
size_t tc_workspace(const ConvGeom& g, int phase, size_t budget, int* splits_out, int* span_out);
int tc_forward(const ConvGeom& g, View4 x, View4 w, const float* bias, long long bias_stride, float* y,
               void* ws, size_t ws_bytes, cudaStream_t st);
// bias (may be null) is indexed by the result's channel: the bias of a transposed convolution, whose forward pass this is.
// *bias_applied tells whether the kernel that ran added it (the CUDA-core fallback does not).
int tc_dinput(const ConvGeom& g, View4 dy, View4 w, const float* bias, long long bias_stride, float* dx, void* ws, size_t ws_bytes,
              cudaStream_t st, bool* bias_applied = nullptr);
int tc_dweight(const ConvGeom& g, View4 x, View4 dy, float* dw, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_bmm(long long batch, long long M, long long N, long long K, const float* A, long long sa_b, long long sa0, long long sa1,
           const float* B, long long sb_b, long long sb0, long long sb1, float* C, cudaStream_t st);
int tc_gemm(long long M, long long N, long long K, const float* A, long long sa0, long long sa1, const float* B,
            long long sb0, long long sb1, const float* bias, float alpha, float beta, float* C, cudaStream_t st);

// persistent strip kernel for stride-1 "same" convolutions (conv_tc_strip.cu)
bool strip_supported(const ConvGeom& g, int phase);
// What the strip kernel's epilogue may fuse behind alpha*acc + beta*bias: a residual tensor of the
// output's logical shape [n][channels][h][w] (any strides) and a ReLU.
struct StripPostOps {
  View4 residual{nullptr, 0, 0, 0, 0};
  int relu = 0;
};
// Per-group element offsets that turn the grouped 1x1 convolution into a batched GEMM (tc_bmm).
struct StripBatch {
  long long act_group_extra = 0, w_group_extra = 0, out_pitch = 0, out_group = 0;
};
int strip_conv(const ConvGeom& g, bool is_dx, View4 act, View4 w, const float* bias, long long bias_stride, float* out,
               void* ws, size_t ws_bytes, cudaStream_t st, bool rowmajor = false, float alpha = 1.f, float beta = 1.f,
               const float* staged_images = nullptr,  // images already written for strip_column_tile()
               const StripPostOps* post = nullptr, const StripBatch* batch = nullptr);
// elementwise residual add / ReLU on a contiguous NCHW result (conv_simt.cu), for candidates without a fused epilogue
int post_ops_nchw(float* y, const ConvGeom& g, const StripPostOps& post, cudaStream_t st);
// y[n][c][plane] += bias[c] on a contiguous result (conv_simt.cu)
int bias_add_nchw(float* y, long long n, int channels, long long plane, const float* bias, long long bias_stride, cudaStream_t st);
bool strip_view_addressable(const ConvGeom& g, bool is_dx, const View4& act, const StripBatch* batch);
int tc_route(const ConvGeom& g, bool is_dx, const View4& act);  // 0 strip, 1 gather, 2 CUDA-core implicit GEMM (conv_tc.cu)
// transposed strip kernel (conv_tc_tstrip.cu): filter on M, up to 256 pixels on N; contiguous NCHW results
bool tstrip_supported(const ConvGeom& g, int phase);
size_t tstrip_workspace(const ConvGeom& g, int phase);
int tstrip_conv(const ConvGeom& g, bool is_dx, View4 act, View4 w, const float* bias, long long bias_stride, float* out,
                void* ws, size_t ws_bytes, cudaStream_t st);
int strip_column_tile(const ConvGeom& g, bool is_dx);   // column tile the plan picks, 0 if unsupported
size_t strip_workspace(const ConvGeom& g, int phase);  // bytes of the weight stage images

// Winograd F(4x4,3x3) forward / dInput (winograd.cu)
bool winograd_supported(const ConvGeom& g, int phase);
size_t winograd_workspace(const ConvGeom& g, int phase, size_t budget);
int winograd_conv(const ConvGeom& g, bool is_dx, View4 act, View4 w, const float* bias, long long bias_stride, float* out,
                  void* ws, size_t ws_bytes, cudaStream_t st);

// dWeight strip kernel (dweight_tc_strip.cu)
bool dweight_strip_supported(const ConvGeom& g);
size_t dweight_strip_workspace(const ConvGeom& g, size_t budget);
int dweight_strip(const ConvGeom& g, View4 x, View4 dy, float* dw, void* ws, size_t ws_bytes, cudaStream_t st);

int* device_status_word();  // device memory, zero unless a bounded wait gave up
int read_device_status(int* out);
int clear_device_status();

}  // namespace b200
