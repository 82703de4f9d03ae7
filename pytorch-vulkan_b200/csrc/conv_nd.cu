// Generic N-d convolution (1 to 3 spatial dimensions, ordinary and transposed, FP32 and int64 forward): one thread
// per output element, contiguous operands.  This is the branch the reference's convolution entry point takes for
// everything that is not a plain FP32 Conv2D (csrc/ops/convolution_nd.cpp:51-74,
// shaders convolution_nd.comp / convolution_nd_int64.comp, also one invocation per output element).  The 2-D and
// 1-D FP32 cases never come here: they run the Conv2D kernels; what remains is 3-D convolution and integer tensors.
//
// Three-dimensional FP32 convolutions with at least 16 channels per group on both sides do not run that kernel: they
// are decomposed over the depth taps into 2-D convolutions on the tcgen05 kernels (conv3d_* below), each depth tap a
// batch of depth slices read through a strided view, the partial results accumulated through the fused epilogue's
// residual input.  The generic kernel remains for everything else (and as the fallback when a step declines).
//
//   ordinary     y[n, co, o]  = b[co] + sum_{ci in group, k} x[n, ci, o*s - p + k*d] * w[co, ci_local, k]
//   transposed   y[n, co, o]  = b[co] + sum_{ci in group, k : (o + p - k*d) = i*s} x[n, ci, i] * w[ci, co_local, k]
// and the three gradients of either (mode 1: dx, 2: dw, 3: db), each again one thread per result element.
#include "common.cuh"

#include <algorithm>
#include <cstdlib>
#include <vector>

namespace b200 {
namespace cnd {

struct Nd {
  long long n, cin, cout, groups;
  int in[3], out[3], k[3], s[3], p[3], d[3];   // depth, height, width (missing leading dimensions are 1)
  int transposed;
};

__device__ __forceinline__ long long vol(const int (&v)[3]) { return (long long)v[0] * v[1] * v[2]; }

// position of the operand that pairs with result position `o` under tap `k`:
//   gather  (ordinary forward, transposed dx):  i = o*s - p + k*d, valid if inside
//   scatter (transposed forward, ordinary dx):  i = (o + p - k*d) / s, valid if divisible and inside
__device__ __forceinline__ bool pair_pos(const Nd& g, bool scatter, const int (&o)[3], const int (&k)[3], const int (&lim)[3], int (&i)[3]) {
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    int v;
    if (scatter) {
      v = o[a] + g.p[a] - k[a] * g.d[a];
      if (v < 0 || v % g.s[a] != 0) return false;
      v /= g.s[a];
    } else {
      v = o[a] * g.s[a] - g.p[a] + k[a] * g.d[a];
      if (v < 0) return false;
    }
    if (v >= lim[a]) return false;
    i[a] = v;
  }
  return true;
}

// mode 0: forward (y from x, w, bias).  mode 1: dx from grad, w.  T = float or long long (mode 0 only).
template <typename T>
__global__ void __launch_bounds__(256) convnd_map_kernel(Nd g, int mode, const T* __restrict__ src, const T* __restrict__ w,
                                                         const T* __restrict__ bias, T* __restrict__ dst, long long total) {
  const long long idx = blockIdx.x * 256ll + threadIdx.x;
  if (idx >= total) return;
  // the result lives on the output grid (mode 0) or on the input grid (mode 1)
  const bool on_out = mode == 0;
  const int (&rs)[3] = on_out ? g.out : g.in;     // extent of the result
  const int (&ss)[3] = on_out ? g.in : g.out;     // extent of the operand it reads
  const long long rc = on_out ? g.cout : g.cin, sc = on_out ? g.cin : g.cout;
  long long r = idx;
  int o[3];
  o[2] = (int)(r % rs[2]); r /= rs[2];
  o[1] = (int)(r % rs[1]); r /= rs[1];
  o[0] = (int)(r % rs[0]); r /= rs[0];
  const long long c = r % rc, n = r / rc;
  const long long rcg = rc / g.groups, scg = sc / g.groups, grp = c / rcg, cl = c % rcg;
  // ordinary forward and transposed dx gather; transposed forward and ordinary dx scatter
  const bool scatter = (mode == 0) == (g.transposed != 0);
  const long long kvol = vol(g.k);
  T acc = (mode == 0 && bias) ? bias[c] : T(0);
  for (long long c2l = 0; c2l < scg; ++c2l) {
    const long long c2 = grp * scg + c2l;
    const T* plane = src + (n * sc + c2) * vol(ss);
    // weight layout: ordinary [cout][cin/g][k], transposed [cin][cout/g][k]; (co, ci) in terms of (c, c2):
    // the result channel is cout in mode 0 and cin in mode 1
    const long long co = on_out ? c : c2, col = on_out ? cl : c2l, ci = on_out ? c2 : c, cil = on_out ? c2l : cl;
    const T* wk = g.transposed ? w + (ci * (g.cout / g.groups) + col) * kvol : w + (co * (g.cin / g.groups) + cil) * kvol;
    int k[3], i[3];
    for (k[0] = 0; k[0] < g.k[0]; ++k[0])
      for (k[1] = 0; k[1] < g.k[1]; ++k[1])
        for (k[2] = 0; k[2] < g.k[2]; ++k[2])
          if (pair_pos(g, scatter, o, k, ss, i))
            acc += plane[((long long)i[0] * ss[1] + i[1]) * ss[2] + i[2]] * wk[((long long)k[0] * g.k[1] + k[1]) * g.k[2] + k[2]];
  }
  dst[idx] = acc;
}

// mode 2: dw[., ., k] = sum over samples and positions of grad * x.  One thread per weight element.
__global__ void __launch_bounds__(256) convnd_dw_kernel(Nd g, const float* __restrict__ grad, const float* __restrict__ x,
                                                        float* __restrict__ dw, long long total) {
  const long long idx = blockIdx.x * 256ll + threadIdx.x;
  if (idx >= total) return;
  long long r = idx;
  int k[3];
  k[2] = (int)(r % g.k[2]); r /= g.k[2];
  k[1] = (int)(r % g.k[1]); r /= g.k[1];
  k[0] = (int)(r % g.k[0]); r /= g.k[0];
  const long long cig = g.cin / g.groups, cog = g.cout / g.groups;
  long long co, ci;
  if (g.transposed) { const long long col = r % cog; ci = r / cog; co = (ci / cig) * cog + col; }
  else { const long long cil = r % cig; co = r / cig; ci = (co / cog) * cig + cil; }
  float acc = 0.f;
  for (long long n = 0; n < g.n; ++n) {
    const float* gp = grad + (n * g.cout + co) * vol(g.out);
    const float* xp = x + (n * g.cin + ci) * vol(g.in);
    int o[3], i[3];
    // ordinary: grad lives on the output grid o, x at o*s - p + k*d.  transposed: x on the input grid i, grad at
    // i*s - p + k*d.  Either way: walk the grid that is indexed directly, gather from the other.
    const int (&walk)[3] = g.transposed ? g.in : g.out;
    const int (&other)[3] = g.transposed ? g.out : g.in;
    const float* pw = g.transposed ? xp : gp;
    const float* po = g.transposed ? gp : xp;
    for (o[0] = 0; o[0] < walk[0]; ++o[0])
      for (o[1] = 0; o[1] < walk[1]; ++o[1])
        for (o[2] = 0; o[2] < walk[2]; ++o[2])
          if (pair_pos(g, false, o, k, other, i))
            acc += pw[((long long)o[0] * walk[1] + o[1]) * walk[2] + o[2]] * po[((long long)i[0] * other[1] + i[1]) * other[2] + i[2]];
  }
  dw[idx] = acc;
}

// mode 3: db[co] = sum grad[:, co, ...].  One warp per channel, lanes stride over the elements, fixed-order tree.
__global__ void __launch_bounds__(256) convnd_db_kernel(Nd g, const float* __restrict__ grad, float* __restrict__ db) {
  const long long co = blockIdx.x * 8ll + (threadIdx.x >> 5);
  if (co >= g.cout) return;
  const int lane = threadIdx.x & 31;
  const long long v = vol(g.out);
  float acc = 0.f;
  for (long long n = 0; n < g.n; ++n) {
    const float* p = grad + (n * g.cout + co) * v;
    for (long long e = lane; e < v; e += 32) acc += p[e];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) db[co] = acc;
}

// rows[r][c] = bias[c] (or 0): the start value of the channels-last accumulation buffer
__global__ void __launch_bounds__(256) fill_rows_kernel(float* __restrict__ dst, const float* __restrict__ bias, long long rows, int c) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i < rows * c) dst[i] = bias ? __ldg(bias + (int)(i % c)) : 0.f;
}

static Nd to_nd(const b200_convnd_params& p) {
  Nd g{};
  g.n = p.n; g.cin = p.cin; g.cout = p.cout; g.groups = p.groups; g.transposed = p.transposed;
  for (int a = 0; a < 3; ++a) {
    g.in[a] = (int)p.in[a]; g.out[a] = (int)p.out[a]; g.k[a] = (int)p.k[a];
    g.s[a] = (int)p.stride[a]; g.p[a] = (int)p.pad[a]; g.d[a] = (int)p.dilation[a];
  }
  return g;
}

// ---- 3-D convolution on the 2-D tensor-core kernels ------------------------------------------------------------------
// y[n, :, od] = bias + sum_kd conv2d(x[n, :, od*sd - pd + kd*dd], w[:, :, kd]): for every depth tap kd and sample n ONE 2-D
// call whose batch is the range of output depths that tap reaches inside the input (view with batch stride sd * plane
// pitch, no copy).  The calls accumulate in a channels-last buffer [n][od][oh][ow][cout] through
// b200_conv2d_forward_fused (residual = the buffer itself), which starts as the bias rows and is transposed into the
// contiguous result at the end.  dInput (stride 1, one group) is the same with the filter view flipped and transposed
// (negative strides); dWeight runs the 2-D dWeight per (kd, n) into a scratch [n][kd][cout][cin/g][kh][kw], summed over
// n and scattered into dW.
struct Scratch {   // blocks of the library's stream-ordered allocator, released on scope exit
  cudaStream_t st;
  std::vector<void*> blocks;
  explicit Scratch(cudaStream_t s) : st(s) {}
  ~Scratch() { for (void* p : blocks) b200_free(p, st); }
  int get(void** out, size_t bytes) {
    if (int rc = b200_malloc(out, bytes ? bytes : 16, st)) return rc;
    blocks.push_back(*out);
    return B200_OK;
  }
};

// A transposed convolution is the input gradient of the ordinary convolution with the same weight whose input is the
// transposed call's result: that convolution's parameters (input and output extents and channel counts swapped).
static b200_convnd_params mirrored(const b200_convnd_params& p) {
  b200_convnd_params m = p;
  m.transposed = 0;
  m.cin = p.cout; m.cout = p.cin;
  for (int a = 0; a < 3; ++a) { m.in[a] = p.out[a]; m.out[a] = p.in[a]; }
  return m;
}

static bool conv3d_takes(const b200_convnd_params& p) {
  if (getenv("B200_CONV3D_GENERIC")) return false;   // testing aid: pins the generic kernel
  if (p.rank != 3 || p.transposed || p.n <= 0) return false;
  const long long plane = p.out[1] * p.out[2];
  if (!(p.in[0] * p.in[1] * p.in[2] > 0 && plane > 0 && p.n * p.out[0] * plane * std::max(p.cin, p.cout) < (1ll << 40))) return false;
  // small problems stay on the single launch of the generic kernel: the decomposition costs a few launches per depth tap and sample
  const long long macs = p.n * p.out[0] * plane * p.cout * (p.cin / p.groups) * p.k[0] * p.k[1] * p.k[2];
  return macs >= (1ll << 24) || getenv("B200_CONV3D_DECOMPOSE") != nullptr;   // (testing aid: decompose whatever the size)
}
// the fused channels-last accumulation needs the tcgen05 strip kernel: 16 or more channels per group on both sides
static bool conv3d_wide(const b200_convnd_params& p) { return p.cin / p.groups >= 16 && p.cout / p.groups >= 16; }
// output depths [lo, hi] that tap kd reads inside the input: 0 <= od*sd - pd + kd*dd < D
static void depth_range(const b200_convnd_params& p, long long kd, long long* lo, long long* hi) {
  const long long off = kd * p.dilation[0] - p.pad[0], sd = p.stride[0];
  *lo = off >= 0 ? 0 : (-off + sd - 1) / sd;
  *hi = std::min<long long>(p.out[0] - 1, (p.in[0] - 1 - off) >= 0 ? (p.in[0] - 1 - off) / sd : -1);
}

// Narrow layers (fewer than 16 channels per group on a side): the 2-D forward candidates per (kd, n) into a contiguous
// scratch [depths][cout][oh][ow], added into the slice of y those depths are (y starts as the bias planes).
static int conv3d_forward_general(const b200_convnd_params& p, const float* x, const float* w, const float* bias, float* y, cudaStream_t st) {
  const long long D = p.in[0], H = p.in[1], W = p.in[2], OD = p.out[0], OH = p.out[1], OW = p.out[2], cig = p.cin / p.groups;
  const long long kvol2 = p.k[1] * p.k[2];
  Scratch scratch(st);
  B200_CUDA(cudaMemsetAsync(y, 0, (size_t)(p.n * p.cout * OD * OH * OW) * sizeof(float), st));
  if (bias)
    if (int rc = bias_add_nchw(y, p.n, (int)p.cout, OD * OH * OW, bias, 1, st)) return rc;
  float* part = nullptr;
  if (int rc = scratch.get((void**)&part, (size_t)(OD * p.cout * OH * OW) * sizeof(float))) return rc;
  size_t ws_bytes = 0;
  void* ws = nullptr;
  for (long long kd = 0; kd < p.k[0]; ++kd) {
    long long lo, hi;
    depth_range(p, kd, &lo, &hi);
    if (hi < lo) continue;
    b200_conv_params p2;
    if (int rc = b200_conv2d_geometry(&p2, hi - lo + 1, p.cin, p.cout, H, W, cig, p.k[1], p.k[2], p.stride[1], p.stride[2], p.pad[1], p.pad[2],
                                      p.dilation[1], p.dilation[2], p.groups))
      return rc;
    if (p2.oh != OH || p2.ow != OW) return fail(B200_EINVAL, "convolution: invalid or oversized output shape");
    const size_t need = b200_conv2d_workspace(&p2, B200_PHASE_FORWARD, B200_ALGO_AUTO, (size_t)1 << 40);
    if (need > ws_bytes) {
      if (int rc = scratch.get(&ws, need)) return rc;
      ws_bytes = need;
    }
    const b200_view4 wv{w + kd * kvol2, {cig * p.k[0] * kvol2, p.k[0] * kvol2, p.k[2], 1}};
    const long long d0 = lo * p.stride[0] - p.pad[0] + kd * p.dilation[0];
    for (long long n = 0; n < p.n; ++n) {
      const b200_view4 xv{x + (n * p.cin * D + d0) * H * W, {p.stride[0] * H * W, D * H * W, W, 1}};
      if (int rc = b200_conv2d_forward(&p2, xv, wv, nullptr, 0, part, need ? ws : nullptr, need, B200_ALGO_AUTO, st)) return rc;
      const int64_t sizes[4] = {hi - lo + 1, p.cout, OH, OW};
      const int64_t strides[4] = {OH * OW, OD * OH * OW, OW, 1};
      if (int rc = b200_scatter_add_strided(y + (n * p.cout * OD + lo) * OH * OW, part, 4, sizes, strides, st)) return rc;
    }
  }
  return B200_OK;
}

static int conv3d_forward(const b200_convnd_params& p, const float* x, const float* w, const float* bias, float* y, cudaStream_t st) {
  if (!conv3d_wide(p)) return conv3d_forward_general(p, x, w, bias, y, st);
  const long long D = p.in[0], H = p.in[1], W = p.in[2], OD = p.out[0], OH = p.out[1], OW = p.out[2], cig = p.cin / p.groups;
  const long long kvol2 = p.k[1] * p.k[2];
  Scratch scratch(st);
  float* acc = nullptr;   // [n][od][oh][ow][cout]
  const long long rows = p.n * OD * OH * OW;
  if (int rc = scratch.get((void**)&acc, (size_t)rows * p.cout * sizeof(float))) return rc;
  fill_rows_kernel<<<(unsigned)div_up64(rows * p.cout, 256), 256, 0, st>>>(acc, bias, rows, (int)p.cout);
  count_launch();
  if (int rc = launch_check("fill_rows_kernel")) return rc;
  size_t ws_bytes = 0;
  void* ws = nullptr;
  for (long long kd = 0; kd < p.k[0]; ++kd) {
    long long lo, hi;
    depth_range(p, kd, &lo, &hi);
    if (hi < lo) continue;
    b200_conv_params p2;
    if (int rc = b200_conv2d_geometry(&p2, hi - lo + 1, p.cin, p.cout, H, W, cig, p.k[1], p.k[2], p.stride[1], p.stride[2], p.pad[1], p.pad[2],
                                      p.dilation[1], p.dilation[2], p.groups))
      return rc;
    if (p2.oh != OH || p2.ow != OW) return fail(B200_EINVAL, "convolution: invalid or oversized output shape");
    if (b200_conv2d_select(&p2, B200_PHASE_FORWARD, B200_ALGO_TC, (size_t)1 << 40) != B200_ALGO_TC)
      return conv3d_forward_general(p, x, w, bias, y, st);   // y has not been touched yet
    const size_t need = b200_conv2d_workspace(&p2, B200_PHASE_FORWARD, B200_ALGO_TC, (size_t)1 << 40);
    if (need > ws_bytes) {
      if (int rc = scratch.get(&ws, need)) return rc;
      ws_bytes = need;
    }
    const b200_view4 wv{w + kd * kvol2, {cig * p.k[0] * kvol2, p.k[0] * kvol2, p.k[2], 1}};
    for (long long n = 0; n < p.n; ++n) {
      const long long d0 = lo * p.stride[0] - p.pad[0] + kd * p.dilation[0];
      const b200_view4 xv{x + (n * p.cin * D + d0) * H * W, {p.stride[0] * H * W, D * H * W, W, 1}};
      float* block = acc + (n * OD + lo) * OH * OW * p.cout;
      const b200_view4 res{block, {OH * OW * p.cout, 1, OW * p.cout, p.cout}};
      const int rc = b200_conv2d_forward_fused(&p2, xv, wv, nullptr, 0, res, 0, block, 1, ws, ws_bytes, B200_ALGO_TC, st);
      if (rc) return rc;   // B200_EUNSUPPORTED from the first call: the caller runs the generic kernel instead
    }
  }
  // [n][od][oh][ow][cout] -> contiguous [n][cout][od][oh][ow]
  const int64_t sizes[5] = {p.n, p.cout, OD, OH, OW};
  const int64_t strides[5] = {OD * OH * OW * p.cout, 1, OH * OW * p.cout, OW * p.cout, p.cout};
  return b200_gather_strided(y, acc, 5, sizes, strides, 4, st);
}

// dx[n, :, id] = sum_kd conv2d(dy[n, :, id + pd - kd*dd], flip(w[:, :, kd])^T), stride 1 in all three dimensions, one group
// The general form (strides, groups): the 2-D dInput kernels per (kd, n) into a contiguous scratch [depths][cin][h][w],
// added into the slice of dx those depths are (dx starts as zeros).  An input depth id receives tap kd from the output
// depth od with od*sd = id + pd - kd*dd: for sd > 1 those id are every sd-th depth.
static int conv3d_dinput_general(const b200_convnd_params& p, const float* grad, const float* w, float* dx, cudaStream_t st) {
  const long long D = p.in[0], H = p.in[1], W = p.in[2], OD = p.out[0], OH = p.out[1], OW = p.out[2], cig = p.cin / p.groups;
  const long long kvol2 = p.k[1] * p.k[2];
  Scratch scratch(st);
  B200_CUDA(cudaMemsetAsync(dx, 0, (size_t)(p.n * p.cin * D * H * W) * sizeof(float), st));
  float* part = nullptr;
  if (int rc = scratch.get((void**)&part, (size_t)(OD * p.cin * H * W) * sizeof(float))) return rc;
  size_t ws_bytes = 0;
  void* ws = nullptr;
  for (long long kd = 0; kd < p.k[0]; ++kd) {
    long long lo, hi;
    depth_range(p, kd, &lo, &hi);   // output depths whose tap kd lies inside the input
    if (hi < lo) continue;
    b200_conv_params p2;
    if (int rc = b200_conv2d_geometry(&p2, hi - lo + 1, p.cin, p.cout, H, W, cig, p.k[1], p.k[2], p.stride[1], p.stride[2], p.pad[1], p.pad[2],
                                      p.dilation[1], p.dilation[2], p.groups))
      return rc;
    if (p2.oh != OH || p2.ow != OW) return B200_EUNSUPPORTED;
    const size_t need = b200_conv2d_workspace(&p2, B200_PHASE_DINPUT, B200_ALGO_AUTO, (size_t)1 << 40);
    if (need > ws_bytes) {
      if (int rc = scratch.get(&ws, need)) return rc;
      ws_bytes = need;
    }
    const b200_view4 wv{w + kd * kvol2, {cig * p.k[0] * kvol2, p.k[0] * kvol2, p.k[2], 1}};
    const long long d0 = lo * p.stride[0] - p.pad[0] + kd * p.dilation[0];   // input depth of the first of them
    for (long long n = 0; n < p.n; ++n) {
      const b200_view4 gv{grad + (n * p.cout * OD + lo) * OH * OW, {OH * OW, OD * OH * OW, OW, 1}};
      if (int rc = b200_conv2d_dinput(&p2, gv, wv, part, need ? ws : nullptr, need, B200_ALGO_AUTO, st)) return rc;
      const int64_t sizes[4] = {hi - lo + 1, p.cin, H, W};
      const int64_t strides[4] = {p.stride[0] * H * W, D * H * W, W, 1};
      if (int rc = b200_scatter_add_strided(dx + (n * p.cin * D + d0) * H * W, part, 4, sizes, strides, st)) return rc;
    }
  }
  return B200_OK;
}

static int conv3d_dinput(const b200_convnd_params& p, const float* grad, const float* w, float* dx, cudaStream_t st) {
  if (p.groups != 1 || p.stride[0] != 1 || p.stride[1] != 1 || p.stride[2] != 1 || !conv3d_wide(p)) return conv3d_dinput_general(p, grad, w, dx, st);
  const long long D = p.in[0], H = p.in[1], W = p.in[2], OD = p.out[0], OH = p.out[1], OW = p.out[2];
  const long long kvol2 = p.k[1] * p.k[2];
  const long long ph2 = p.dilation[1] * (p.k[1] - 1) - p.pad[1], pw2 = p.dilation[2] * (p.k[2] - 1) - p.pad[2];
  if (ph2 < 0 || pw2 < 0) return conv3d_dinput_general(p, grad, w, dx, st);   // padding beyond the filter reach
  Scratch scratch(st);
  float* acc = nullptr;   // [n][d][h][w][cin]
  const long long rows = p.n * D * H * W;
  if (int rc = scratch.get((void**)&acc, (size_t)rows * p.cin * sizeof(float))) return rc;
  fill_rows_kernel<<<(unsigned)div_up64(rows * p.cin, 256), 256, 0, st>>>(acc, nullptr, rows, (int)p.cin);
  count_launch();
  if (int rc = launch_check("fill_rows_kernel")) return rc;
  size_t ws_bytes = 0;
  void* ws = nullptr;
  for (long long kd = 0; kd < p.k[0]; ++kd) {
    // input depths id with 0 <= id + pd - kd*dd < OD
    const long long off = p.pad[0] - kd * p.dilation[0];
    const long long lo = std::max<long long>(0, -off), hi = std::min<long long>(D - 1, OD - 1 - off);
    if (hi < lo) continue;
    b200_conv_params p2;   // the 2-D convolution dy -> dx: cout input channels, cin output channels, flipped filter
    if (int rc = b200_conv2d_geometry(&p2, hi - lo + 1, p.cout, p.cin, OH, OW, p.cout, p.k[1], p.k[2], 1, 1, ph2, pw2, p.dilation[1],
                                      p.dilation[2], 1))
      return rc;
    if (p2.oh != H || p2.ow != W) return B200_EUNSUPPORTED;
    if (b200_conv2d_select(&p2, B200_PHASE_FORWARD, B200_ALGO_TC, (size_t)1 << 40) != B200_ALGO_TC) return conv3d_dinput_general(p, grad, w, dx, st);
    const size_t need = b200_conv2d_workspace(&p2, B200_PHASE_FORWARD, B200_ALGO_TC, (size_t)1 << 40);
    if (need > ws_bytes) {
      if (int rc = scratch.get(&ws, need)) return rc;
      ws_bytes = need;
    }
    // filter of that convolution: [cin][cout][kh][kw] = w[co][ci][kd][kh-1-ky][kw-1-kx]
    const b200_view4 wv{w + kd * kvol2 + (kvol2 - 1), {p.k[0] * kvol2, p.cin * p.k[0] * kvol2, -p.k[2], -1}};
    for (long long n = 0; n < p.n; ++n) {
      const b200_view4 gv{grad + (n * p.cout * OD + (lo + off)) * OH * OW, {OH * OW, OD * OH * OW, OW, 1}};
      float* block = acc + (n * D + lo) * H * W * p.cin;
      const b200_view4 res{block, {H * W * p.cin, 1, W * p.cin, p.cin}};
      if (int rc = b200_conv2d_forward_fused(&p2, gv, wv, nullptr, 0, res, 0, block, 1, ws, ws_bytes, B200_ALGO_TC, st)) return rc;
    }
  }
  const int64_t sizes[5] = {p.n, p.cin, D, H, W};
  const int64_t strides[5] = {D * H * W * p.cin, 1, H * W * p.cin, W * p.cin, p.cin};
  return b200_gather_strided(dx, acc, 5, sizes, strides, 4, st);
}

// dw[:, :, kd] = sum_n dWeight2d(x[n, :, od*sd - pd + kd*dd], dy[n, :, od])
static int conv3d_dweight(const b200_convnd_params& p, const float* grad, const float* x, float* dw, cudaStream_t st) {
  const long long D = p.in[0], H = p.in[1], W = p.in[2], OD = p.out[0], OH = p.out[1], OW = p.out[2], cig = p.cin / p.groups;
  const long long kvol2 = p.k[1] * p.k[2], slice = p.cout * cig * kvol2;
  Scratch scratch(st);
  float* parts = nullptr;   // [n][kd][cout][cin/g][kh][kw]
  float* sums = nullptr;    // [kd][cout][cin/g][kh][kw]
  if (int rc = scratch.get((void**)&parts, (size_t)(p.n * p.k[0] * slice) * sizeof(float))) return rc;
  if (int rc = scratch.get((void**)&sums, (size_t)(p.k[0] * slice) * sizeof(float))) return rc;
  B200_CUDA(cudaMemsetAsync(parts, 0, (size_t)(p.n * p.k[0] * slice) * sizeof(float), st));   // taps that reach no depth stay zero
  size_t ws_bytes = 0;
  void* ws = nullptr;
  for (long long kd = 0; kd < p.k[0]; ++kd) {
    long long lo, hi;
    depth_range(p, kd, &lo, &hi);
    if (hi < lo) continue;
    b200_conv_params p2;
    if (int rc = b200_conv2d_geometry(&p2, hi - lo + 1, p.cin, p.cout, H, W, cig, p.k[1], p.k[2], p.stride[1], p.stride[2], p.pad[1], p.pad[2],
                                      p.dilation[1], p.dilation[2], p.groups))
      return rc;
    const size_t need = b200_conv2d_workspace(&p2, B200_PHASE_DWEIGHT, B200_ALGO_AUTO, (size_t)256 << 20);
    if (need > ws_bytes) {
      if (int rc = scratch.get(&ws, need)) return rc;
      ws_bytes = need;
    }
    for (long long n = 0; n < p.n; ++n) {
      const long long d0 = lo * p.stride[0] - p.pad[0] + kd * p.dilation[0];
      const b200_view4 xv{x + (n * p.cin * D + d0) * H * W, {p.stride[0] * H * W, D * H * W, W, 1}};
      const b200_view4 gv{grad + (n * p.cout * OD + lo) * OH * OW, {OH * OW, OD * OH * OW, OW, 1}};
      if (int rc = b200_conv2d_dweight(&p2, xv, gv, parts + (n * p.k[0] + kd) * slice, need ? ws : nullptr, need, B200_ALGO_AUTO, st)) return rc;
    }
  }
  // sum over n, then [kd][cout][cin/g][kh*kw] -> dw[cout][cin/g][kd][kh*kw]
  const int64_t psizes[2] = {p.n, p.k[0] * slice}, pstrides[2] = {p.k[0] * slice, 1};
  const unsigned char reduce[2] = {1, 0};
  if (int rc = b200_sum_strided(sums, parts, 2, psizes, pstrides, reduce, st)) return rc;
  const int64_t sizes[3] = {p.k[0], p.cout * cig, kvol2}, strides[3] = {kvol2, p.k[0] * kvol2, 1};
  return b200_scatter_strided(dw, sums, 3, sizes, strides, 4, st);
}

}  // namespace cnd
}  // namespace b200

using namespace b200;

extern "C" {

int b200_convnd_geometry(b200_convnd_params* out, int rank, int64_t n, int64_t cin, const int64_t* in_sizes, int64_t w0,
                         int64_t w1, const int64_t* kernel, const int64_t* stride, const int64_t* pad, const int64_t* dilation,
                         const int64_t* output_pad, int transposed, int64_t groups) {
  if (!out || !in_sizes || !kernel || !stride || !pad || !dilation || !output_pad) return fail(B200_EINVAL, "convolution: null argument");
  if (rank < 1 || rank > 3) return fail(B200_EINVAL, "convolution: expected matching rank 3, 4 or 5 tensors");
  if (!(groups > 0 && cin > 0 && cin % groups == 0)) return fail(B200_EINVAL, "convolution: invalid groups/input channels");
  if (w0 <= 0 || w1 <= 0) return fail(B200_EINVAL, "convolution: empty weight dimension");
  const int64_t cout = transposed ? w1 * groups : w0;
  if (!(cout % groups == 0 && (transposed ? w0 == cin : w1 * groups == cin)))
    return fail(B200_EINVAL, "convolution: weight/channel/group mismatch");
  b200_convnd_params g{};
  g.rank = rank; g.n = n; g.cin = cin; g.cout = cout; g.groups = groups; g.transposed = transposed ? 1 : 0;
  for (int a = 0; a < 3; ++a) { g.in[a] = g.out[a] = g.k[a] = g.stride[a] = g.dilation[a] = 1; g.pad[a] = 0; }
  for (int a = 0; a < rank; ++a) {
    const int d = 3 - rank + a;
    const int64_t in = in_sizes[a], k = kernel[a], s = stride[a], p = pad[a], di = dilation[a], op = output_pad[a];
    if (k <= 0) return fail(B200_EINVAL, "convolution: empty weight dimension");
    if (!(in > 0 && s > 0 && di > 0 && p >= 0 && op >= 0)) return fail(B200_EINVAL, "convolution: invalid spatial parameters");
    if (!(transposed ? (op < s || op < di) : op == 0)) return fail(B200_EINVAL, "convolution: invalid output padding");
    if (!(in <= INT32_MAX && k <= INT32_MAX && s <= INT32_MAX && p <= INT32_MAX / 2 && di <= INT32_MAX && (k - 1) <= INT32_MAX / di &&
          (in - 1) <= INT32_MAX / s))
      return fail(B200_ERANGE, "convolution: spatial addressing exceeds int32");
    const int64_t effective = (k - 1) * di + 1;
    const int64_t o = transposed ? (in - 1) * s - 2 * p + effective + op : (in + 2 * p - effective) / s + 1;
    if (!((transposed || in + 2 * p >= effective) && o > 0 && o <= INT32_MAX && o * s + effective + p <= INT32_MAX))
      return fail(B200_EINVAL, "convolution: invalid or oversized output shape");
    g.in[d] = in; g.out[d] = o; g.k[d] = k; g.stride[d] = s; g.pad[d] = p; g.dilation[d] = di;
  }
  *out = g;
  return B200_OK;
}

int b200_convnd_forward(const b200_convnd_params* p, const void* x, const void* w, const void* bias, void* y, int is_int64,
                        void* stream) {
  if (!p) return fail(B200_EINVAL, "convolution: null parameters");
  if (int rc = ensure_init()) return rc;
  const cnd::Nd g = cnd::to_nd(*p);
  const long long total = p->n * p->cout * p->out[0] * p->out[1] * p->out[2];
  if (total == 0) return B200_OK;
  if (!x || !w || !y) return fail(B200_EINVAL, "convolution: null tensor");
  const unsigned blocks = (unsigned)div_up64(total, 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (!is_int64 && cnd::conv3d_takes(*p)) {
    const int rc = cnd::conv3d_forward(*p, (const float*)x, (const float*)w, (const float*)bias, (float*)y, st);
    if (rc != B200_EUNSUPPORTED) {
      note_kernel("conv3d_forward: depth taps on the 2-D tcgen05 kernels");
      return rc;
    }
  }
  if (!is_int64 && p->transposed && p->rank == 3) {   // the input gradient of the mirrored convolution, plus the bias
    const b200_convnd_params m = cnd::mirrored(*p);
    if (cnd::conv3d_takes(m)) {
      int rc = cnd::conv3d_dinput(m, (const float*)x, (const float*)w, (float*)y, st);
      if (rc == B200_OK && bias)
        rc = bias_add_nchw((float*)y, p->n, (int)p->cout, (long long)(p->out[0] * p->out[1] * p->out[2]), (const float*)bias, 1, st);
      if (rc != B200_EUNSUPPORTED) {
        note_kernel("conv_transpose3d_forward: depth taps on the 2-D tcgen05 kernels");
        return rc;
      }
    }
  }
  if (is_int64)
    cnd::convnd_map_kernel<long long><<<blocks, 256, 0, st>>>(g, 0, (const long long*)x, (const long long*)w, (const long long*)bias,
                                                             (long long*)y, total);
  else
    cnd::convnd_map_kernel<float><<<blocks, 256, 0, st>>>(g, 0, (const float*)x, (const float*)w, (const float*)bias, (float*)y, total);
  count_launch();
  note_kernel(is_int64 ? "convnd_forward_int64" : "convnd_forward");
  return launch_check("convnd_map_kernel");
}

int b200_convnd_backward(const b200_convnd_params* p, const float* grad, const float* x, const float* w, float* dx, float* dw,
                         float* db, void* stream) {
  if (!p) return fail(B200_EINVAL, "convolution: null parameters");
  if (int rc = ensure_init()) return rc;
  const cnd::Nd g = cnd::to_nd(*p);
  cudaStream_t st = (cudaStream_t)stream;
  const long long in_total = p->n * p->cin * p->in[0] * p->in[1] * p->in[2];
  const long long w_total = (p->transposed ? p->cin * (p->cout / p->groups) : p->cout * (p->cin / p->groups)) * p->k[0] * p->k[1] * p->k[2];
  const long long out_total = p->n * p->cout * p->out[0] * p->out[1] * p->out[2];
  if ((dx || dw || db) && out_total && !grad) return fail(B200_EINVAL, "convolution backward: null gradient");
  if (p->transposed && p->rank == 3 && out_total > 0 && in_total > 0) {
    // gradients of a transposed call through the mirrored convolution: dx = its forward pass over grad, dw = its
    // dWeight with grad as the input and x as the output gradient
    const b200_convnd_params m = cnd::mirrored(*p);
    if (cnd::conv3d_takes(m)) {
      if (dx && w) {
        const int rc = cnd::conv3d_forward(m, grad, w, nullptr, dx, st);
        if (rc != B200_EUNSUPPORTED) { if (rc) return rc; dx = nullptr; }
      }
      if (dw && w_total && x) {
        const int rc = cnd::conv3d_dweight(m, x, grad, dw, st);
        if (rc != B200_EUNSUPPORTED) { if (rc) return rc; dw = nullptr; }
      }
    }
  }
  const bool on_2d = cnd::conv3d_takes(*p) && out_total > 0;
  if (dx && in_total && on_2d && w) {
    const int rc = cnd::conv3d_dinput(*p, grad, w, dx, st);
    if (rc != B200_EUNSUPPORTED) {
      if (rc) return rc;
      dx = nullptr;   // done
    }
  }
  if (dw && w_total && on_2d && x) {
    const int rc = cnd::conv3d_dweight(*p, grad, x, dw, st);
    if (rc != B200_EUNSUPPORTED) {
      if (rc) return rc;
      dw = nullptr;
    }
  }
  if (dx && in_total) {
    if (!w) return fail(B200_EINVAL, "convolution backward: null weight");
    cnd::convnd_map_kernel<float><<<(unsigned)div_up64(in_total, 256), 256, 0, st>>>(g, 1, grad, w, nullptr, dx, in_total);
    count_launch();
    if (int rc = launch_check("convnd_map_kernel")) return rc;
  }
  if (dw && w_total) {
    if (!x && in_total) return fail(B200_EINVAL, "convolution backward: null input");
    cnd::convnd_dw_kernel<<<(unsigned)div_up64(w_total, 256), 256, 0, st>>>(g, grad, x, dw, w_total);
    count_launch();
    if (int rc = launch_check("convnd_dw_kernel")) return rc;
  }
  if (db && p->cout) {
    cnd::convnd_db_kernel<<<(unsigned)div_up64(p->cout, 8), 256, 0, st>>>(g, grad, db);
    count_launch();
    if (int rc = launch_check("convnd_db_kernel")) return rc;
  }
  note_kernel("convnd_backward");
  return B200_OK;
}

}  // extern "C"
