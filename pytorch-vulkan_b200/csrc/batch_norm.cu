// BatchNorm forward (training / evaluation) and backward for FP32 tensors viewed as
// [outer][channels][inner].  Replaces the batch_norm_forward / batch_norm_eval /
// batch_norm_backward shaders of the reference (csrc/shaders/batch_norm_*.comp) and their
// host side (csrc/ops/batch_norm.cpp:21-113).
//
// All kernels are bound by HBM traffic, not arithmetic: training forward reads the tensor
// twice and writes it once, backward reads two tensors twice and writes one.  They therefore
// run on the CUDA cores with 16-byte loads, several loads in flight per lane, and grids of a
// few CTAs per SM; nothing here is GEMM-shaped.
//
// Two arrangements cover every shape:
//   rows     inner >= 256: the channel's elements lie in `outer` contiguous planes.  A warp
//            streams one plane segment at a time (like the reference's one-workgroup-per-channel
//            loop, but with the channel cut into (channel, slab) CTAs).
//   columns  inner < 256 (channels-last tensors have inner == 1): the tensor is a matrix of
//            `outer` rows by channels*inner columns; eight lanes cover 32 adjacent columns of a
//            row with one 16-byte load each and every column keeps its own statistics, which
//            the finalize kernel merges per channel.
// Statistics are kept as (count, mean relative to the channel's first element, sum of squared
// deviations) and merged pairwise, the streaming form of the reference's shifted two-pass
// reduction (batch_norm_forward.comp:27-38): no E[x^2]-E[x]^2 cancellation for data with a
// large common offset, and the low part of the mean survives into the normalisation.
#include <cstdlib>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsInnerMin = 256;  // planes at least this long use the rows arrangement
constexpr int kSegment = 2048;      // most floats of a plane one warp streams per unit

struct Moments {
  float n, mean, m2;
};

__device__ __forceinline__ Moments merge(Moments a, Moments b) {
  const float n = a.n + b.n;
  if (!(n > 0.f)) return a;
  const float d = b.mean - a.mean, f = b.n / n;
  return {n, a.mean + d * f, a.m2 + b.m2 + d * d * a.n * f};
}

__device__ __forceinline__ Moments shfl_moments(Moments m, int o) {
  return {__shfl_xor_sync(0xffffffffu, m.n, o), __shfl_xor_sync(0xffffffffu, m.mean, o), __shfl_xor_sync(0xffffffffu, m.m2, o)};
}

__device__ __forceinline__ Moments warp_merge(Moments m) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = merge(m, shfl_moments(m, o));
  return m;
}

// Sums around a thread-local shift k (a sample of the data), turned into Moments relative to the
// channel origin when a unit ends.
struct Shifted {
  float n = 0.f, s = 0.f, q = 0.f;
  __device__ __forceinline__ void add(float v, float k) {
    const float d = v - k;
    s += d;
    q = fmaf(d, d, q);
    n += 1.f;
  }
  __device__ __forceinline__ Moments moments(float k, float origin) const {
    if (!(n > 0.f)) return {0.f, 0.f, 0.f};
    const float mean_d = s / n;
    return {n, (k - origin) + mean_d, fmaxf(q - s * mean_d, 0.f)};
  }
};

// Geometry shared by all kernels of one call.
struct BnShape {
  int outer, c, inner;  // logical [outer][c][inner]
  int cols;             // c * inner
  int slabs;            // partial results per column (columns) or per channel (rows)
  int per;              // units (rows arrangement) or rows (columns) per slab
  int segs, seg_len;    // rows: segments per plane and their length (a multiple of 4)
  int part_inner;       // partial entries per channel and slab: inner (columns) or 1 (rows)
  float m;              // outer * inner, the reduction length
};

// ---- forward: statistics -----------------------------------------------------------------

// rows arrangement: grid (c, slabs); part[slab * c + ch].
__global__ void __launch_bounds__(kThreads, 8) bn_stats_rows_kernel(const float* __restrict__ x, BnShape sh, Moments* part) {
  const int ch = blockIdx.x, slab = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = sh.outer * sh.segs, per = sh.per;
  const int u0 = slab * per, u1 = min(units, u0 + per);
  const float origin = __ldg(x + (size_t)ch * sh.inner);
  Moments acc = {0.f, 0.f, 0.f};
  for (int u = u0 + warp; u < u1; u += kThreads / 32) {
    const int img = u / sh.segs, off = (u - img * sh.segs) * sh.seg_len, len = min(sh.seg_len, sh.inner - off);
    const float* base = x + ((size_t)img * sh.c + ch) * sh.inner + off;
    const float k = __ldg(base + min(lane, len - 1));
    Shifted t;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(base) & 15) == 0) {
      const float4* v4 = reinterpret_cast<const float4*>(base);
      const int quads = len >> 2;
      int q = lane;
      for (; q + 96 < quads; q += 128) {
        const float4 a0 = __ldg(v4 + q), a1 = __ldg(v4 + q + 32), a2 = __ldg(v4 + q + 64), a3 = __ldg(v4 + q + 96);
        t.add(a0.x, k), t.add(a0.y, k), t.add(a0.z, k), t.add(a0.w, k);
        t.add(a1.x, k), t.add(a1.y, k), t.add(a1.z, k), t.add(a1.w, k);
        t.add(a2.x, k), t.add(a2.y, k), t.add(a2.z, k), t.add(a2.w, k);
        t.add(a3.x, k), t.add(a3.y, k), t.add(a3.z, k), t.add(a3.w, k);
      }
      for (; q < quads; q += 32) {
        const float4 a = __ldg(v4 + q);
        t.add(a.x, k), t.add(a.y, k), t.add(a.z, k), t.add(a.w, k);
      }
      done = quads * 4;
    }
    for (int e = done + lane; e < len; e += 32) t.add(__ldg(base + e), k);
    acc = merge(acc, t.moments(k, origin));
  }
  __shared__ Moments warp_part[kThreads / 32];
  acc = warp_merge(acc);
  if (lane == 0) warp_part[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    Moments m = warp_part[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) m = merge(m, warp_part[w]);
    part[(size_t)slab * sh.c + ch] = m;
  }
}

// columns arrangement: grid (ceil(cols / (8 V)), slabs); V adjacent columns per thread (V = 4 needs
// cols % 4 == 0 and a 16-byte aligned tensor); part[slab * cols + col].
template <int V>
__global__ void __launch_bounds__(kThreads, 5) bn_stats_cols_kernel(const float* __restrict__ x, BnShape sh, Moments* part) {
  const int cl = (threadIdx.x & 7) * V, prow = threadIdx.x >> 3, slab = blockIdx.y;
  const int col0 = blockIdx.x * 8 * V + cl;
  const int per = sh.per;
  const int r0 = slab * per, r1 = min(sh.outer, r0 + per);
  const bool live = col0 < sh.cols;  // V == 4: cols % 4 == 0, so a live quad is whole
  float origin[V];
  Moments acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int col = min(col0 + j, sh.cols - 1);
    origin[j] = __ldg(x + (size_t)(col / sh.inner) * sh.inner);
    acc[j] = {0.f, 0.f, 0.f};
  }
  if (live) {
    // chunks of at most 64 rows per thread between conversions keep the shifted sums short
    for (int rc = r0 + prow; rc < r1; rc += 32 * 64) {
      const int rend = min(r1, rc + 32 * 64);
      const float* src = x + (size_t)rc * sh.cols + col0;
      float k[V];
      Shifted t[V];
      if (V == 4) {
        const float4 kv = __ldg(reinterpret_cast<const float4*>(src));
        k[0] = kv.x, k[1 % V] = kv.y, k[2 % V] = kv.z, k[3 % V] = kv.w;
      } else {
        k[0] = __ldg(src);
      }
      int r = rc;
      const size_t step = (size_t)32 * sh.cols;
      if (V == 4) {
        for (; r + 96 < rend; r += 128, src += 4 * step) {
          const float4 a0 = __ldg(reinterpret_cast<const float4*>(src));
          const float4 a1 = __ldg(reinterpret_cast<const float4*>(src + step));
          const float4 a2 = __ldg(reinterpret_cast<const float4*>(src + 2 * step));
          const float4 a3 = __ldg(reinterpret_cast<const float4*>(src + 3 * step));
          t[0].add(a0.x, k[0]), t[1 % V].add(a0.y, k[1 % V]), t[2 % V].add(a0.z, k[2 % V]), t[3 % V].add(a0.w, k[3 % V]);
          t[0].add(a1.x, k[0]), t[1 % V].add(a1.y, k[1 % V]), t[2 % V].add(a1.z, k[2 % V]), t[3 % V].add(a1.w, k[3 % V]);
          t[0].add(a2.x, k[0]), t[1 % V].add(a2.y, k[1 % V]), t[2 % V].add(a2.z, k[2 % V]), t[3 % V].add(a2.w, k[3 % V]);
          t[0].add(a3.x, k[0]), t[1 % V].add(a3.y, k[1 % V]), t[2 % V].add(a3.z, k[2 % V]), t[3 % V].add(a3.w, k[3 % V]);
        }
        for (; r < rend; r += 32, src += step) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(src));
          t[0].add(a.x, k[0]), t[1 % V].add(a.y, k[1 % V]), t[2 % V].add(a.z, k[2 % V]), t[3 % V].add(a.w, k[3 % V]);
        }
      } else {
        for (; r + 96 < rend; r += 128, src += 4 * step) {
          const float a0 = __ldg(src), a1 = __ldg(src + step), a2 = __ldg(src + 2 * step), a3 = __ldg(src + 3 * step);
          t[0].add(a0, k[0]), t[0].add(a1, k[0]), t[0].add(a2, k[0]), t[0].add(a3, k[0]);
        }
        for (; r < rend; r += 32, src += step) t[0].add(__ldg(src), k[0]);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = merge(acc[j], t[j].moments(k[j], origin[j]));
    }
  }
  // the 32 row-lanes of a column: four share a warp (lanes l, l+8, l+16, l+24), the eight warps
  // meet in shared memory
  __shared__ Moments sm[kThreads / 32][8 * V + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    acc[j] = merge(acc[j], shfl_moments(acc[j], 8));
    acc[j] = merge(acc[j], shfl_moments(acc[j], 16));
    if (lane < 8) sm[warp][cl + j] = acc[j];
  }
  __syncthreads();
  if (threadIdx.x < 8 * V) {
    const int col = blockIdx.x * 8 * V + threadIdx.x;
    if (col < sh.cols) {
      Moments m = sm[0][threadIdx.x];
#pragma unroll
      for (int w = 1; w < kThreads / 32; ++w) m = merge(m, sm[w][threadIdx.x]);
      part[(size_t)slab * sh.cols + col] = m;
    }
  }
}

struct BnForwardVectors {
  const float *weight, *bias;
  float *running_mean, *running_var;
  long long w_stride, b_stride, rm_stride, rv_stride;
  float *save_mean, *save_inv;
  float eps, momentum;
};

// One warp per channel merges the partial statistics, writes the saved mean and inverse standard
// deviation, updates the running statistics (batch_norm_forward.comp:39-44) and leaves the
// normalisation coefficients {origin, mean - origin, inv * gamma, beta}.
__global__ void __launch_bounds__(kThreads) bn_stats_finalize_kernel(const float* __restrict__ x, BnShape sh, const Moments* part,
                                                                      BnForwardVectors v, float4* coef) {
  const int ch = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (ch >= sh.c) return;
  const int entries = sh.slabs * sh.part_inner;
  const int pcols = sh.c * sh.part_inner;
  // the channel's scalars first: their latency hides behind the merge
  const float origin = __ldg(x + (size_t)ch * sh.inner);
  const float gamma = v.weight ? v.weight[ch * v.w_stride] : 1.f;
  const float beta = v.bias ? v.bias[ch * v.b_stride] : 0.f;
  const float old_mean = v.running_mean ? v.running_mean[ch * v.rm_stride] : 0.f;
  const float old_var = v.running_var ? v.running_var[ch * v.rv_stride] : 0.f;
  Moments m = {0.f, 0.f, 0.f};
  for (int t = lane; t < entries; t += 32) {
    const int slab = t / sh.part_inner, j = t - slab * sh.part_inner;
    m = merge(m, part[(size_t)slab * pcols + (size_t)ch * sh.part_inner + j]);
  }
  m = warp_merge(m);
  if (lane != 0) return;
  const float variance = m.m2 / sh.m;
  const float inv = (variance == 0.f && v.eps == 0.f) ? 0.f : 1.f / sqrtf(variance + v.eps);
  const float mean = origin + m.mean;
  v.save_mean[ch] = mean;
  v.save_inv[ch] = inv;
  if (v.running_mean) v.running_mean[ch * v.rm_stride] = (1.f - v.momentum) * old_mean + v.momentum * mean;
  if (v.running_var) v.running_var[ch * v.rv_stride] = (1.f - v.momentum) * old_var + v.momentum * (m.m2 / (sh.m - 1.f));
  coef[ch] = make_float4(origin, m.mean, inv * gamma, beta);
}

// Evaluation: coefficients straight from the running statistics (batch_norm_eval.comp:24-29).
__global__ void bn_eval_coef_kernel(int c, BnForwardVectors v, float4* coef) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  const float mean = v.running_mean[ch * v.rm_stride];
  const float inv = 1.f / sqrtf(v.running_var[ch * v.rv_stride] + v.eps);
  const float gamma = v.weight ? v.weight[ch * v.w_stride] : 1.f;
  const float beta = v.bias ? v.bias[ch * v.b_stride] : 0.f;
  coef[ch] = make_float4(mean, 0.f, inv * gamma, beta);
}

// ---- forward: normalisation ----------------------------------------------------------------

struct ChannelOf {
  FastDiv inner, c;
  int nc;
  __device__ __forceinline__ int operator()(uint32_t i) const {
    const uint32_t plane = inner.div(i);
    return (int)(plane - c.div(plane) * (uint32_t)nc);
  }
};

__device__ __forceinline__ float normalise(float v, float4 k) { return ((v - k.x) - k.y) * k.z + k.w; }

// y = ((x - origin) - mean_rel) * (inv * gamma) + beta over the flat tensor.  UNIFORM: the four
// elements of a 16-byte group share a channel (inner % 4 == 0), `ch` then indexes groups.
// POST: add a residual tensor of the same layout (res may be null) and / or clamp at zero before the
// store, the add + ReLU that follows a BatchNorm in a residual block.
struct BnPost {
  const float* res;
  int relu;
};
__device__ __forceinline__ float4 post_ops(float4 r, float4 add, int relu) {
  r.x += add.x, r.y += add.y, r.z += add.z, r.w += add.w;
  if (relu) r = make_float4(fmaxf(r.x, 0.f), fmaxf(r.y, 0.f), fmaxf(r.z, 0.f), fmaxf(r.w, 0.f));
  return r;
}

template <bool UNIFORM, bool POST>
__global__ void __launch_bounds__(kThreads) bn_apply_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                             const float4* __restrict__ coef, uint32_t total, ChannelOf ch, BnPost post) {
  const uint32_t quads = total >> 2, stride = gridDim.x * kThreads;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  const float4* r4 = reinterpret_cast<const float4*>(post.res);
  float4* y4 = reinterpret_cast<float4*>(y);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  auto one = [&](uint32_t q, float4 a, float4 add) {
    float4 r;
    if (UNIFORM) {
      const float4 k = __ldg(coef + ch(q));
      r = make_float4(normalise(a.x, k), normalise(a.y, k), normalise(a.z, k), normalise(a.w, k));
    } else {
      r = make_float4(normalise(a.x, __ldg(coef + ch(4 * q))), normalise(a.y, __ldg(coef + ch(4 * q + 1))),
                      normalise(a.z, __ldg(coef + ch(4 * q + 2))), normalise(a.w, __ldg(coef + ch(4 * q + 3))));
    }
    y4[q] = POST ? post_ops(r, add, post.relu) : r;
  };
  auto residual = [&](uint32_t q) { return POST && r4 ? __ldg(r4 + q) : zero; };
  uint32_t q = blockIdx.x * kThreads + threadIdx.x;
  for (; q < quads && q + 3 * (uint64_t)stride < quads; q += 4 * stride) {
    const float4 a0 = __ldg(x4 + q), a1 = __ldg(x4 + q + stride), a2 = __ldg(x4 + q + 2 * stride), a3 = __ldg(x4 + q + 3 * stride);
    const float4 b0 = residual(q), b1 = residual(q + stride), b2 = residual(q + 2 * stride), b3 = residual(q + 3 * stride);
    one(q, a0, b0), one(q + stride, a1, b1), one(q + 2 * stride, a2, b2), one(q + 3 * stride, a3, b3);
  }
  for (; q < quads; q += stride) one(q, __ldg(x4 + q), residual(q));
}

// Channels-last with c % 4 == 0: a thread keeps one group of four channels, whose coefficients stay
// in registers, and walks down the rows.  `lanes` (a multiple of c / 4) threads take part.
template <bool POST>
__global__ void __launch_bounds__(kThreads) bn_apply_cols_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                  const float4* __restrict__ coef, uint32_t rows, uint32_t c4,
                                                                  uint32_t lanes, BnPost post) {
  const uint32_t t = blockIdx.x * kThreads + threadIdx.x;
  if (t >= lanes) return;
  const uint32_t r0 = t / c4, j = t - r0 * c4;
  const uint64_t rstep = lanes / c4;
  const float4 k0 = __ldg(coef + 4 * j), k1 = __ldg(coef + 4 * j + 1), k2 = __ldg(coef + 4 * j + 2), k3 = __ldg(coef + 4 * j + 3);
  const float4* x4 = reinterpret_cast<const float4*>(x) + j;
  const float4* r4 = post.res ? reinterpret_cast<const float4*>(post.res) + j : nullptr;
  float4* y4 = reinterpret_cast<float4*>(y) + j;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  auto one = [&](uint64_t row, float4 a, float4 add) {
    const float4 r = make_float4(normalise(a.x, k0), normalise(a.y, k1), normalise(a.z, k2), normalise(a.w, k3));
    y4[row * c4] = POST ? post_ops(r, add, post.relu) : r;
  };
  auto residual = [&](uint64_t row) { return POST && r4 ? __ldg(r4 + row * c4) : zero; };
  uint64_t r = r0;
  for (; r + 3 * rstep < rows; r += 4 * rstep) {
    const float4 a0 = __ldg(x4 + r * c4), a1 = __ldg(x4 + (r + rstep) * c4), a2 = __ldg(x4 + (r + 2 * rstep) * c4),
                 a3 = __ldg(x4 + (r + 3 * rstep) * c4);
    const float4 b0 = residual(r), b1 = residual(r + rstep), b2 = residual(r + 2 * rstep), b3 = residual(r + 3 * rstep);
    one(r, a0, b0), one(r + rstep, a1, b1), one(r + 2 * rstep, a2, b2), one(r + 3 * rstep, a3, b3);
  }
  for (; r < rows; r += rstep) one(r, __ldg(x4 + r * c4), residual(r));
}

// Scalar form: unaligned tensors and the last total % 4 elements ([first, total)).
__global__ void __launch_bounds__(kThreads) bn_apply_scalar_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                    const float4* __restrict__ coef, uint32_t first, uint32_t total,
                                                                    ChannelOf ch, BnPost post) {
  for (uint64_t i = first + blockIdx.x * (uint64_t)kThreads + threadIdx.x; i < total; i += (uint64_t)gridDim.x * kThreads) {
    float v = normalise(__ldg(x + i), __ldg(coef + ch((uint32_t)i)));
    if (post.res) v += __ldg(post.res + i);
    y[i] = post.relu ? fmaxf(v, 0.f) : v;
  }
}

// ---- backward: reductions -------------------------------------------------------------------

struct Sums {
  float a, b, r;  // sum g, sum (x - mean) g, sum (x - mean)
  __device__ __forceinline__ void add(float xv, float gv, float mean) {
    const float centered = xv - mean;
    a += gv;
    b = fmaf(centered, gv, b);
    r += centered;
  }
};

__device__ __forceinline__ Sums warp_sums(Sums s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s.a += __shfl_xor_sync(0xffffffffu, s.a, o);
    s.b += __shfl_xor_sync(0xffffffffu, s.b, o);
    s.r += __shfl_xor_sync(0xffffffffu, s.r, o);
  }
  return s;
}

struct BnBackwardVectors {
  const float *weight, *mean, *inv;
  long long w_stride, mean_stride, inv_stride;
  float *dw, *db;
  float eps;
  int training;
};

__global__ void __launch_bounds__(kThreads, 8) bn_bwd_rows_kernel(const float* __restrict__ x, const float* __restrict__ g, BnShape sh,
                                                                BnBackwardVectors v, Sums* part) {
  const int ch = blockIdx.x, slab = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = sh.outer * sh.segs, per = sh.per;
  const int u0 = slab * per, u1 = min(units, u0 + per);
  const float mean = v.mean[ch * v.mean_stride];
  Sums t = {0.f, 0.f, 0.f};
  for (int u = u0 + warp; u < u1; u += kThreads / 32) {
    const int img = u / sh.segs, off = (u - img * sh.segs) * sh.seg_len, len = min(sh.seg_len, sh.inner - off);
    const size_t at = ((size_t)img * sh.c + ch) * sh.inner + off;
    const float *xb = x + at, *gb = g + at;
    int done = 0;
    if (((reinterpret_cast<uintptr_t>(xb) | reinterpret_cast<uintptr_t>(gb)) & 15) == 0) {
      const float4 *x4 = reinterpret_cast<const float4*>(xb), *g4 = reinterpret_cast<const float4*>(gb);
      const int quads = len >> 2;
      int q = lane;
      for (; q + 32 < quads; q += 64) {
        const float4 a0 = __ldg(x4 + q), a1 = __ldg(x4 + q + 32), b0 = __ldg(g4 + q), b1 = __ldg(g4 + q + 32);
        t.add(a0.x, b0.x, mean), t.add(a0.y, b0.y, mean), t.add(a0.z, b0.z, mean), t.add(a0.w, b0.w, mean);
        t.add(a1.x, b1.x, mean), t.add(a1.y, b1.y, mean), t.add(a1.z, b1.z, mean), t.add(a1.w, b1.w, mean);
      }
      for (; q < quads; q += 32) {
        const float4 a = __ldg(x4 + q), b = __ldg(g4 + q);
        t.add(a.x, b.x, mean), t.add(a.y, b.y, mean), t.add(a.z, b.z, mean), t.add(a.w, b.w, mean);
      }
      done = quads * 4;
    }
    for (int e = done + lane; e < len; e += 32) t.add(__ldg(xb + e), __ldg(gb + e), mean);
  }
  __shared__ Sums warp_part[kThreads / 32];
  t = warp_sums(t);
  if (lane == 0) warp_part[warp] = t;
  __syncthreads();
  if (threadIdx.x == 0) {
    Sums s = warp_part[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) s.a += warp_part[w].a, s.b += warp_part[w].b, s.r += warp_part[w].r;
    part[(size_t)slab * sh.c + ch] = s;
  }
}

template <int V>
__global__ void __launch_bounds__(kThreads, 5) bn_bwd_cols_kernel(const float* __restrict__ x, const float* __restrict__ g, BnShape sh,
                                                                BnBackwardVectors v, Sums* part) {
  const int cl = (threadIdx.x & 7) * V, prow = threadIdx.x >> 3, slab = blockIdx.y;
  const int col0 = blockIdx.x * 8 * V + cl;
  const int per = sh.per;
  const int r0 = slab * per, r1 = min(sh.outer, r0 + per);
  float mean[V];
  Sums t[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int col = min(col0 + j, sh.cols - 1);
    mean[j] = v.mean[(col / sh.inner) * v.mean_stride];
    t[j] = {0.f, 0.f, 0.f};
  }
  if (col0 < sh.cols) {
    const size_t step = (size_t)32 * sh.cols;
    size_t at = (size_t)(r0 + prow) * sh.cols + col0;
    int r = r0 + prow;
    if (V == 4) {
      for (; r + 32 < r1; r += 64, at += 2 * step) {
        const float4 a0 = __ldg(reinterpret_cast<const float4*>(x + at)), a1 = __ldg(reinterpret_cast<const float4*>(x + at + step));
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(g + at)), b1 = __ldg(reinterpret_cast<const float4*>(g + at + step));
        t[0].add(a0.x, b0.x, mean[0]), t[1 % V].add(a0.y, b0.y, mean[1 % V]), t[2 % V].add(a0.z, b0.z, mean[2 % V]), t[3 % V].add(a0.w, b0.w, mean[3 % V]);
        t[0].add(a1.x, b1.x, mean[0]), t[1 % V].add(a1.y, b1.y, mean[1 % V]), t[2 % V].add(a1.z, b1.z, mean[2 % V]), t[3 % V].add(a1.w, b1.w, mean[3 % V]);
      }
      for (; r < r1; r += 32, at += step) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(x + at)), b = __ldg(reinterpret_cast<const float4*>(g + at));
        t[0].add(a.x, b.x, mean[0]), t[1 % V].add(a.y, b.y, mean[1 % V]), t[2 % V].add(a.z, b.z, mean[2 % V]), t[3 % V].add(a.w, b.w, mean[3 % V]);
      }
    } else {
      for (; r + 32 < r1; r += 64, at += 2 * step) {
        const float a0 = __ldg(x + at), a1 = __ldg(x + at + step), b0 = __ldg(g + at), b1 = __ldg(g + at + step);
        t[0].add(a0, b0, mean[0]), t[0].add(a1, b1, mean[0]);
      }
      for (; r < r1; r += 32, at += step) t[0].add(__ldg(x + at), __ldg(g + at), mean[0]);
    }
  }
  __shared__ Sums sm[kThreads / 32][8 * V + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < V; ++j) {
#pragma unroll
    for (int o = 8; o <= 16; o <<= 1) {
      t[j].a += __shfl_xor_sync(0xffffffffu, t[j].a, o);
      t[j].b += __shfl_xor_sync(0xffffffffu, t[j].b, o);
      t[j].r += __shfl_xor_sync(0xffffffffu, t[j].r, o);
    }
    if (lane < 8) sm[warp][cl + j] = t[j];
  }
  __syncthreads();
  if (threadIdx.x < 8 * V) {
    const int col = blockIdx.x * 8 * V + threadIdx.x;
    if (col < sh.cols) {
      Sums s = sm[0][threadIdx.x];
#pragma unroll
      for (int w = 1; w < kThreads / 32; ++w) s.a += sm[w][threadIdx.x].a, s.b += sm[w][threadIdx.x].b, s.r += sm[w][threadIdx.x].r;
      part[(size_t)slab * sh.cols + col] = s;
    }
  }
}

// One warp per channel: dw, db and the input-gradient coefficients
// {mean, residual, sum(g)/m, (b/m) inv^2} plus scale = inv * gamma (batch_norm_backward.comp:46-65).
// has_sums == 0: evaluation mode asked for dx only, nothing was reduced.
__global__ void __launch_bounds__(kThreads) bn_bwd_finalize_kernel(BnShape sh, const Sums* part, BnBackwardVectors v, int has_sums,
                                                                    float4* coef, float* scale) {
  const int ch = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (ch >= sh.c) return;
  double a = 0.0, b = 0.0, r = 0.0;
  if (has_sums) {
    const int entries = sh.slabs * sh.part_inner, pcols = sh.c * sh.part_inner;
    for (int t = lane; t < entries; t += 32) {
      const int slab = t / sh.part_inner, j = t - slab * sh.part_inner;
      const Sums s = part[(size_t)slab * pcols + (size_t)ch * sh.part_inner + j];
      a += s.a, b += s.b, r += s.r;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
      r += __shfl_xor_sync(0xffffffffu, r, o);
    }
  }
  if (lane != 0) return;
  float inv = v.inv[ch * v.inv_stride];
  if (!v.training) inv = 1.f / sqrtf(inv + v.eps);
  float fa = (float)a, fb = (float)b, residual = 0.f;
  if (v.training) {
    // the saved mean is rounded to FP32; its low part comes back from sum(x - mean)
    residual = (float)(r / (double)sh.m);
    if (residual != 0.f) fb = (float)(b - (double)residual * a);
  }
  if (v.dw) v.dw[ch] = fb * inv;
  if (v.db) v.db[ch] = fa;
  const float mean = v.mean[ch * v.mean_stride];
  const float gamma = v.weight ? v.weight[ch * v.w_stride] : 1.f;
  coef[ch] = v.training ? make_float4(mean, residual, fa / sh.m, (fb / sh.m) * inv * inv) : make_float4(mean, 0.f, 0.f, 0.f);
  scale[ch] = inv * gamma;
}

// Two values per channel in training mode: the reference switches to the algebraic derivative
// (batch_norm_backward.comp:24-37), which stays antisymmetric; so does this kernel.
__global__ void bn_bwd_pair_kernel(const float* __restrict__ x, const float* __restrict__ g, BnShape sh, BnBackwardVectors v, float* dx) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= sh.c) return;
  const size_t i0 = (size_t)ch * sh.inner;
  const size_t i1 = sh.inner == 2 ? i0 + 1 : (size_t)(sh.c + ch) * sh.inner;
  const float inv = v.inv[ch * v.inv_stride];
  const float dg = __fsub_rn(__fmul_rn(0.5f, g[i0]), __fmul_rn(0.5f, g[i1]));
  if (v.dw) v.dw[ch] = __fmul_rn(__fmul_rn(__fsub_rn(x[i0], x[i1]), dg), inv);
  if (v.db) v.db[ch] = g[i0] + g[i1];
  if (dx) {
    const float gamma = v.weight ? v.weight[ch * v.w_stride] : 1.f;
    const float val = (dg * gamma) * (((v.eps * inv) * inv) * inv);
    dx[i0] = val;
    dx[i1] = -val;
  }
}

// ---- backward: input gradient ----------------------------------------------------------------

template <bool TRAINING>
__device__ __forceinline__ float input_grad(float xv, float gv, float4 k, float scale) {
  if (TRAINING) gv -= k.z + ((xv - k.x) - k.y) * k.w;
  return gv * scale;
}

template <bool UNIFORM, bool TRAINING>
__global__ void __launch_bounds__(kThreads) bn_bwd_apply_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                 float* __restrict__ dx, const float4* __restrict__ coef,
                                                                 const float* __restrict__ scale, uint32_t total, ChannelOf ch) {
  const uint32_t quads = total >> 2, stride = gridDim.x * kThreads;
  const float4 *x4 = reinterpret_cast<const float4*>(x), *g4 = reinterpret_cast<const float4*>(g);
  float4* d4 = reinterpret_cast<float4*>(dx);
  auto one = [&](uint32_t q, float4 a, float4 b) {
    float4 r;
    if (UNIFORM) {
      const int c = ch(q);
      const float4 k = TRAINING ? __ldg(coef + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float s = __ldg(scale + c);
      r = make_float4(input_grad<TRAINING>(a.x, b.x, k, s), input_grad<TRAINING>(a.y, b.y, k, s),
                      input_grad<TRAINING>(a.z, b.z, k, s), input_grad<TRAINING>(a.w, b.w, k, s));
    } else {
      const int c0 = ch(4 * q), c1 = ch(4 * q + 1), c2 = ch(4 * q + 2), c3 = ch(4 * q + 3);
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      r = make_float4(input_grad<TRAINING>(a.x, b.x, TRAINING ? __ldg(coef + c0) : z, __ldg(scale + c0)),
                      input_grad<TRAINING>(a.y, b.y, TRAINING ? __ldg(coef + c1) : z, __ldg(scale + c1)),
                      input_grad<TRAINING>(a.z, b.z, TRAINING ? __ldg(coef + c2) : z, __ldg(scale + c2)),
                      input_grad<TRAINING>(a.w, b.w, TRAINING ? __ldg(coef + c3) : z, __ldg(scale + c3)));
    }
    d4[q] = r;
  };
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  uint32_t q = blockIdx.x * kThreads + threadIdx.x;
  for (; q < quads && q + (uint64_t)stride < quads; q += 2 * stride) {
    const float4 b0 = __ldg(g4 + q), b1 = __ldg(g4 + q + stride);
    const float4 a0 = TRAINING ? __ldg(x4 + q) : zero, a1 = TRAINING ? __ldg(x4 + q + stride) : zero;
    one(q, a0, b0), one(q + stride, a1, b1);
  }
  for (; q < quads; q += stride) one(q, TRAINING ? __ldg(x4 + q) : zero, __ldg(g4 + q));
}

// The channels-last form of the kernel above (c % 4 == 0): one group of four channels per thread.
template <bool TRAINING>
__global__ void __launch_bounds__(kThreads, 5) bn_bwd_apply_cols_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                      float* __restrict__ dx, const float4* __restrict__ coef,
                                                                      const float* __restrict__ scale, uint32_t rows, uint32_t c4,
                                                                      uint32_t lanes) {
  const uint32_t t = blockIdx.x * kThreads + threadIdx.x;
  if (t >= lanes) return;
  const uint32_t r0 = t / c4, j = t - r0 * c4;
  const uint64_t rstep = lanes / c4;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 k0 = TRAINING ? __ldg(coef + 4 * j) : zero, k1 = TRAINING ? __ldg(coef + 4 * j + 1) : zero,
               k2 = TRAINING ? __ldg(coef + 4 * j + 2) : zero, k3 = TRAINING ? __ldg(coef + 4 * j + 3) : zero;
  const float4 s = __ldg(reinterpret_cast<const float4*>(scale) + j);
  const float4 *x4 = reinterpret_cast<const float4*>(x) + j, *g4 = reinterpret_cast<const float4*>(g) + j;
  float4* d4 = reinterpret_cast<float4*>(dx) + j;
  auto one = [&](uint64_t row, float4 a, float4 b) {
    d4[row * c4] = make_float4(input_grad<TRAINING>(a.x, b.x, k0, s.x), input_grad<TRAINING>(a.y, b.y, k1, s.y),
                               input_grad<TRAINING>(a.z, b.z, k2, s.z), input_grad<TRAINING>(a.w, b.w, k3, s.w));
  };
  uint64_t r = r0;
  for (; r + rstep < rows; r += 2 * rstep) {
    const float4 b0 = __ldg(g4 + r * c4), b1 = __ldg(g4 + (r + rstep) * c4);
    const float4 a0 = TRAINING ? __ldg(x4 + r * c4) : zero, a1 = TRAINING ? __ldg(x4 + (r + rstep) * c4) : zero;
    one(r, a0, b0), one(r + rstep, a1, b1);
  }
  for (; r < rows; r += rstep) one(r, TRAINING ? __ldg(x4 + r * c4) : zero, __ldg(g4 + r * c4));
}

template <bool TRAINING>
__global__ void __launch_bounds__(kThreads) bn_bwd_apply_scalar_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                        float* __restrict__ dx, const float4* __restrict__ coef,
                                                                        const float* __restrict__ scale, uint32_t first, uint32_t total,
                                                                        ChannelOf ch) {
  for (uint64_t i = first + blockIdx.x * (uint64_t)kThreads + threadIdx.x; i < total; i += (uint64_t)gridDim.x * kThreads) {
    const int c = ch((uint32_t)i);
    dx[i] = input_grad<TRAINING>(TRAINING ? __ldg(x + i) : 0.f, __ldg(g + i), __ldg(coef + c), __ldg(scale + c));
  }
}

// ---- small tensors: one CTA per channel, one launch ------------------------------------------------
// When a channel's values are a few hundred KB at most and there are enough channels to fill the
// GPU, the three launches above cost more than the traffic.  Here one CTA owns a channel from the
// first read to the last write, as the reference's workgroup does (batch_norm_forward.comp:18-55,
// batch_norm_backward.comp:18-66), with a warp per image plane; the second pass finds the channel in
// L1 / L2.  Planar layout only.

// f(value) / f(x value, g value) over a plane of `len` floats, the warp's lanes striding it with
// 16-byte loads where the plane is aligned.
constexpr int kChannelThreads = 1024;  // 32 warps: a channel is spread over as many image planes at once as an SM holds

template <bool TWO, class F>
__device__ __forceinline__ void plane_stream(const float* __restrict__ p, const float* __restrict__ q, int len, int lane, F&& f) {
  int done = 0;
  if (((reinterpret_cast<uintptr_t>(p) | (TWO ? reinterpret_cast<uintptr_t>(q) : 0)) & 15) == 0) {
    const float4* p4 = reinterpret_cast<const float4*>(p);
    const float4* q4 = reinterpret_cast<const float4*>(q);
    const int quads = len >> 2;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    int i = lane;
    for (; i + 32 < quads; i += 64) {
      const float4 a0 = __ldg(p4 + i), a1 = __ldg(p4 + i + 32), b0 = TWO ? __ldg(q4 + i) : zero, b1 = TWO ? __ldg(q4 + i + 32) : zero;
      f(a0.x, b0.x), f(a0.y, b0.y), f(a0.z, b0.z), f(a0.w, b0.w);
      f(a1.x, b1.x), f(a1.y, b1.y), f(a1.z, b1.z), f(a1.w, b1.w);
    }
    for (; i < quads; i += 32) {
      const float4 a = __ldg(p4 + i), b = TWO ? __ldg(q4 + i) : zero;
      f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w);
    }
    done = quads * 4;
  }
  for (int e = done + lane; e < len; e += 32) f(__ldg(p + e), TWO ? __ldg(q + e) : 0.f);
}
// out[e] = f(a, b, r) over a plane; r is the residual value (0 when res is null).
template <bool TWO, class F>
__device__ __forceinline__ void plane_map(const float* __restrict__ p, const float* __restrict__ q, const float* __restrict__ res,
                                          float* __restrict__ out, int len, int lane, F&& f) {
  int done = 0;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(res) |
                         (TWO ? reinterpret_cast<uintptr_t>(q) : 0);
  if ((bits & 15) == 0) {
    const float4* p4 = reinterpret_cast<const float4*>(p);
    const float4* q4 = reinterpret_cast<const float4*>(q);
    const float4* r4 = reinterpret_cast<const float4*>(res);
    float4* o4 = reinterpret_cast<float4*>(out);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = lane; i < (len >> 2); i += 32) {
      const float4 a = __ldg(p4 + i), b = TWO ? __ldg(q4 + i) : zero, r = res ? __ldg(r4 + i) : zero;
      o4[i] = make_float4(f(a.x, b.x, r.x), f(a.y, b.y, r.y), f(a.z, b.z, r.z), f(a.w, b.w, r.w));
    }
    done = (len >> 2) * 4;
  }
  for (int e = done + lane; e < len; e += 32) out[e] = f(__ldg(p + e), TWO ? __ldg(q + e) : 0.f, res ? __ldg(res + e) : 0.f);
}

__global__ void __launch_bounds__(kChannelThreads) bn_forward_channel_kernel(const float* __restrict__ x, BnShape sh, BnForwardVectors v,
                                                                       BnPost post, float* __restrict__ y) {
  const int ch = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float origin = __ldg(x + (size_t)ch * sh.inner);
  const float gamma = v.weight ? v.weight[ch * v.w_stride] : 1.f;
  const float beta = v.bias ? v.bias[ch * v.b_stride] : 0.f;
  Moments acc = {0.f, 0.f, 0.f};
  for (int img = warp; img < sh.outer; img += kChannelThreads / 32) {
    const float* base = x + ((size_t)img * sh.c + ch) * sh.inner;
    const float k = __ldg(base + min(lane, sh.inner - 1));
    Shifted t;
    plane_stream<false>(base, nullptr, sh.inner, lane, [&](float xv, float) { t.add(xv, k); });
    acc = merge(acc, t.moments(k, origin));
  }
  __shared__ Moments warp_part[32];
  acc = warp_merge(acc);
  if (threadIdx.x < 32) warp_part[threadIdx.x] = Moments{0.f, 0.f, 0.f};
  __syncthreads();
  if (lane == 0) warp_part[warp] = acc;
  __syncthreads();
  const Moments m = warp_merge(warp_part[lane]);  // every warp folds the partial results itself
  const float variance = m.m2 / sh.m;
  const float inv = (variance == 0.f && v.eps == 0.f) ? 0.f : 1.f / sqrtf(variance + v.eps);
  if (threadIdx.x == 0) {
    const float mean = origin + m.mean;
    v.save_mean[ch] = mean;
    v.save_inv[ch] = inv;
    if (v.running_mean) {
      float* p = v.running_mean + ch * v.rm_stride;
      *p = (1.f - v.momentum) * *p + v.momentum * mean;
    }
    if (v.running_var) {
      float* p = v.running_var + ch * v.rv_stride;
      *p = (1.f - v.momentum) * *p + v.momentum * (m.m2 / (sh.m - 1.f));
    }
  }
  const float4 k4 = make_float4(origin, m.mean, inv * gamma, beta);
  for (int img = warp; img < sh.outer; img += kChannelThreads / 32) {
    const size_t at = ((size_t)img * sh.c + ch) * sh.inner;
    plane_map<false>(x + at, nullptr, post.res ? post.res + at : nullptr, y + at, sh.inner, lane, [&](float xv, float, float r) {
      const float o = normalise(xv, k4) + r;
      return post.relu ? fmaxf(o, 0.f) : o;
    });
  }
}

__global__ void __launch_bounds__(kChannelThreads) bn_backward_channel_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                        BnShape sh, BnBackwardVectors v, float* __restrict__ dx) {
  const int ch = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float mean = v.mean[ch * v.mean_stride];
  float inv = v.inv[ch * v.inv_stride];
  if (!v.training) inv = 1.f / sqrtf(inv + v.eps);
  const float gamma = v.weight ? v.weight[ch * v.w_stride] : 1.f;
  Sums t = {0.f, 0.f, 0.f};
  for (int img = warp; img < sh.outer; img += kChannelThreads / 32) {
    const size_t at = ((size_t)img * sh.c + ch) * sh.inner;
    plane_stream<true>(x + at, g + at, sh.inner, lane, [&](float xv, float gv) { t.add(xv, gv, mean); });
  }
  __shared__ Sums warp_part[32];
  t = warp_sums(t);
  if (threadIdx.x < 32) warp_part[threadIdx.x] = Sums{0.f, 0.f, 0.f};
  __syncthreads();
  if (lane == 0) warp_part[warp] = t;
  __syncthreads();
  const Sums s = warp_sums(warp_part[lane]);
  float fa = s.a, fb = s.b, residual = 0.f;
  if (v.training) {
    residual = s.r / sh.m;
    if (residual != 0.f) fb -= residual * fa;
  }
  if (threadIdx.x == 0) {
    if (v.dw) v.dw[ch] = fb * inv;
    if (v.db) v.db[ch] = fa;
  }
  if (!dx) return;
  const float4 k4 = make_float4(mean, residual, fa / sh.m, (fb / sh.m) * inv * inv);
  const float scale = inv * gamma;
  const bool training = v.training != 0;
  for (int img = warp; img < sh.outer; img += kChannelThreads / 32) {
    const size_t at = ((size_t)img * sh.c + ch) * sh.inner;
    plane_map<true>(x + at, g + at, nullptr, dx + at, sh.inner, lane, [&](float xv, float gv, float) {
      return training ? input_grad<true>(xv, gv, k4, scale) : input_grad<false>(xv, gv, k4, scale);
    });
  }
}

// One launch pays when a channel is tens to hundreds of KB and the channels fill the GPU.  Measured
// kernel times (64 images): 256 channels of 14x14 20 us against 26 us for the three launches, 128
// channels of 28x28 18 against 27; 512 channels of 7x7 (12 KB each) 31 against 21, so short channels
// keep the three-launch path.
bool channel_kernel_fits(const BnShape& sh, int layout) {
  static const bool enabled = !(getenv("B200_BN_ONE_LAUNCH") && getenv("B200_BN_ONE_LAUNCH")[0] == '0');  // testing aid
  if (!enabled) return false;
  const double channel_bytes = (double)sh.m * sizeof(float);
  return layout == B200_BN_PLANAR && sh.c >= 64 && channel_bytes >= 32.0 * 1024 && channel_bytes <= 256.0 * 1024 &&
         channel_bytes * sh.c <= 64.0 * 1024 * 1024;
}

// ---- host side ---------------------------------------------------------------------------------

struct BnPlan {
  BnShape sh;
  bool rows;
  size_t coef_bytes, scale_bytes, part_bytes;
};

int make_plan(int64_t n, int64_t c, int64_t s, int layout, BnPlan* out) {
  if (n <= 0 || c <= 0 || s <= 0) return fail(B200_EINVAL, "batch norm: empty tensor");
  if (layout != B200_BN_PLANAR && layout != B200_BN_INTERLEAVED) return fail(B200_EINVAL, "batch norm: unknown layout %d", layout);
  if (n > INT32_MAX || c > INT32_MAX || s > INT32_MAX || n * c > INT32_MAX / s)
    return fail(B200_ERANGE, "batch norm: more than INT32_MAX elements");
  BnPlan p{};
  BnShape& sh = p.sh;
  sh.c = (int)c;
  if (layout == B200_BN_PLANAR) sh.outer = (int)n, sh.inner = (int)s;
  else sh.outer = (int)(n * s), sh.inner = 1;
  sh.cols = sh.c * sh.inner;
  sh.m = (float)((double)n * (double)s);
  p.rows = sh.inner >= kRowsInnerMin;
  // CTAs wanted, from measurement: one wave of eight 32-register CTAs per SM for the rows kernels,
  // four per SM for the column kernels (48 registers, a longer epilogue per CTA)
  const int target = (p.rows ? 8 : 4) * sm_count();
  const int kMinUnits = 8, kMinRows = 512;  // least units (rows kernels) / rows (column kernels) per CTA
  if (p.rows) {
    sh.segs = (sh.inner + kSegment - 1) / kSegment;
    sh.seg_len = ((sh.inner + sh.segs - 1) / sh.segs + 3) & ~3;  // equal segments, 16-byte steps
    sh.part_inner = 1;
    // a CTA takes a multiple of eight units (one per warp and round), so no warp idles while the
    // others finish, and at least kMinUnits of them
    const int64_t units = (int64_t)sh.outer * sh.segs;
    int64_t slabs = (target + sh.c - 1) / sh.c;
    int64_t per = (units + slabs - 1) / slabs;
    if (per < kMinUnits) per = kMinUnits;
    per = (per + 7) / 8 * 8;
    sh.slabs = (int)((units + per - 1) / per);
    sh.per = (int)per;
  } else {
    sh.segs = 1;
    sh.seg_len = sh.inner;
    sh.part_inner = sh.inner;
    const int col_blocks = (sh.cols + 31) / 32;
    int64_t slabs = (target + col_blocks - 1) / col_blocks;
    int64_t per = (sh.outer + slabs - 1) / slabs;
    if (per < kMinRows) per = kMinRows;
    per = (per + 127) / 128 * 128;  // whole passes of 32 row-lanes x 4 loads
    sh.slabs = (int)((sh.outer + per - 1) / per);
    sh.per = (int)per;
  }
  if (sh.slabs > 65535) sh.slabs = 65535;
  p.coef_bytes = ((size_t)sh.c * sizeof(float4) + 255) & ~(size_t)255;
  p.scale_bytes = ((size_t)sh.c * sizeof(float) + 255) & ~(size_t)255;
  p.part_bytes = (size_t)sh.slabs * sh.c * sh.part_inner * sizeof(Moments);
  *out = p;
  return B200_OK;
}

ChannelOf channel_of(const BnShape& sh, bool uniform) {
  ChannelOf ch;
  ch.inner = FastDiv((uint32_t)(uniform ? sh.inner / 4 : sh.inner));
  ch.c = FastDiv((uint32_t)sh.c);
  ch.nc = sh.c;
  return ch;
}

int apply_grid(uint32_t work_items) {
  const int64_t want = ((int64_t)work_items + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 8;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_batch_norm_workspace(int64_t n, int64_t c, int64_t s, int layout) {
  if (ensure_init()) return 0;
  BnPlan p;
  if (make_plan(n, c, s, layout, &p)) return 0;
  return p.coef_bytes + p.scale_bytes + p.part_bytes;
}

int b200_batch_norm_forward(int64_t n, int64_t c, int64_t s, int layout, const float* x, const float* weight,
                            int64_t weight_stride, const float* bias, int64_t bias_stride, float* running_mean,
                            int64_t running_mean_stride, float* running_var, int64_t running_var_stride, int training,
                            float momentum, float eps, float* y, float* save_mean, float* save_inv, void* workspace,
                            size_t workspace_bytes, void* stream) {
  return b200_batch_norm_forward_fused(n, c, s, layout, x, weight, weight_stride, bias, bias_stride, running_mean,
                                       running_mean_stride, running_var, running_var_stride, training, momentum, eps, nullptr, 0, y,
                                       save_mean, save_inv, workspace, workspace_bytes, stream);
}

int b200_batch_norm_forward_fused(int64_t n, int64_t c, int64_t s, int layout, const float* x, const float* weight,
                                  int64_t weight_stride, const float* bias, int64_t bias_stride, float* running_mean,
                                  int64_t running_mean_stride, float* running_var, int64_t running_var_stride, int training,
                                  float momentum, float eps, const float* residual, int relu, float* y, float* save_mean,
                                  float* save_inv, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = ensure_init()) return rc;
  BnPlan p;
  if (int rc = make_plan(n, c, s, layout, &p)) return rc;
  if (!x || !y) return fail(B200_EINVAL, "batch norm: null tensor");
  if (!training && !(running_mean && running_var))
    return fail(B200_EINVAL, "batch norm: evaluation requires running statistics");
  if (training && !(save_mean && save_inv)) return fail(B200_EINVAL, "batch norm: training needs save_mean and save_inv");
  if (!workspace || !aligned16(workspace) || workspace_bytes < p.coef_bytes + p.scale_bytes + p.part_bytes)
    return fail(B200_EWORKSPACE, "batch norm: workspace missing, unaligned or smaller than b200_batch_norm_workspace()");
  cudaStream_t st = (cudaStream_t)stream;
  const BnShape& sh = p.sh;
  float4* coef = (float4*)workspace;
  Moments* part = (Moments*)((char*)workspace + p.coef_bytes + p.scale_bytes);
  BnForwardVectors v{weight, bias, running_mean, running_var, weight_stride, bias_stride, running_mean_stride,
                     running_var_stride, save_mean, save_inv, eps, momentum};
  const uint32_t total = (uint32_t)((int64_t)sh.outer * sh.cols);
  if (training && channel_kernel_fits(sh, layout)) {
    note_kernel(residual || relu ? "bn_forward_channel_fused" : "bn_forward_channel");
    bn_forward_channel_kernel<<<(unsigned)sh.c, kChannelThreads, 0, st>>>(x, sh, v, BnPost{residual, relu ? 1 : 0}, y);
    count_launch();
    return launch_check("bn_forward_channel_kernel");
  }
  if (training) {
    if (p.rows) {
      note_kernel("bn_stats_rows+finalize+apply");
      bn_stats_rows_kernel<<<dim3((unsigned)sh.c, (unsigned)sh.slabs), kThreads, 0, st>>>(x, sh, part);
    } else if (sh.cols % 4 == 0 && aligned16(x)) {
      note_kernel("bn_stats_cols+finalize+apply");
      bn_stats_cols_kernel<4><<<dim3((unsigned)((sh.cols + 31) / 32), (unsigned)sh.slabs), kThreads, 0, st>>>(x, sh, part);
    } else {
      note_kernel("bn_stats_cols+finalize+apply");
      bn_stats_cols_kernel<1><<<dim3((unsigned)((sh.cols + 7) / 8), (unsigned)sh.slabs), kThreads, 0, st>>>(x, sh, part);
    }
    count_launch();
    if (int rc = launch_check("bn_stats_kernel")) return rc;
    bn_stats_finalize_kernel<<<(sh.c + 7) / 8, kThreads, 0, st>>>(x, sh, part, v, coef);
    count_launch();
    if (int rc = launch_check("bn_stats_finalize_kernel")) return rc;
  } else {
    note_kernel("bn_eval_coef+apply");
    bn_eval_coef_kernel<<<(sh.c + 127) / 128, 128, 0, st>>>(sh.c, v, coef);
    count_launch();
    if (int rc = launch_check("bn_eval_coef_kernel")) return rc;
  }
  const BnPost post{residual, relu ? 1 : 0};
  const bool fused = residual || relu;
  if (fused) note_kernel(training ? "bn_stats+finalize+apply_fused" : "bn_eval_coef+apply_fused");
  if (aligned16(x) && aligned16(y) && aligned16(residual)) {
    const bool uniform = sh.inner % 4 == 0;
    const uint32_t quads = total >> 2;
    if (quads) {
      const int grid = apply_grid((quads + 3) / 4);
      const uint32_t c4 = (uint32_t)sh.c / 4, threads = (uint32_t)grid * kThreads;
      const uint32_t lanes = c4 ? threads / c4 * c4 : 0;
      if (sh.inner == 1 && sh.c % 4 == 0 && threads >= c4) {
        if (fused) bn_apply_cols_kernel<true><<<grid, kThreads, 0, st>>>(x, y, coef, (uint32_t)sh.outer, c4, lanes, post);
        else bn_apply_cols_kernel<false><<<grid, kThreads, 0, st>>>(x, y, coef, (uint32_t)sh.outer, c4, lanes, post);
      } else if (uniform) {
        if (fused) bn_apply_kernel<true, true><<<grid, kThreads, 0, st>>>(x, y, coef, total, channel_of(sh, true), post);
        else bn_apply_kernel<true, false><<<grid, kThreads, 0, st>>>(x, y, coef, total, channel_of(sh, true), post);
      } else {
        if (fused) bn_apply_kernel<false, true><<<grid, kThreads, 0, st>>>(x, y, coef, total, channel_of(sh, false), post);
        else bn_apply_kernel<false, false><<<grid, kThreads, 0, st>>>(x, y, coef, total, channel_of(sh, false), post);
      }
      count_launch();
      if (int rc = launch_check("bn_apply_kernel")) return rc;
    }
    if (total & 3) {
      bn_apply_scalar_kernel<<<1, kThreads, 0, st>>>(x, y, coef, total & ~3u, total, channel_of(sh, false), post);
      count_launch();
      if (int rc = launch_check("bn_apply_scalar_kernel")) return rc;
    }
  } else {
    bn_apply_scalar_kernel<<<apply_grid(total), kThreads, 0, st>>>(x, y, coef, 0, total, channel_of(sh, false), post);
    count_launch();
    if (int rc = launch_check("bn_apply_scalar_kernel")) return rc;
  }
  return B200_OK;
}

int b200_batch_norm_backward(int64_t n, int64_t c, int64_t s, int layout, const float* grad, const float* x,
                             const float* weight, int64_t weight_stride, const float* mean, int64_t mean_stride,
                             const float* inv_or_var, int64_t inv_stride, int training, float eps, float* dx, float* dw,
                             float* db, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = ensure_init()) return rc;
  BnPlan p;
  if (int rc = make_plan(n, c, s, layout, &p)) return rc;
  if (!x || !grad) return fail(B200_EINVAL, "batch norm backward: null tensor");
  if (!mean || !inv_or_var) return fail(B200_EINVAL, "batch norm backward requires statistics");
  if (!dx && !dw && !db) return B200_OK;
  if (!workspace || !aligned16(workspace) || workspace_bytes < p.coef_bytes + p.scale_bytes + p.part_bytes)
    return fail(B200_EWORKSPACE, "batch norm: workspace missing, unaligned or smaller than b200_batch_norm_workspace()");
  cudaStream_t st = (cudaStream_t)stream;
  const BnShape& sh = p.sh;
  float4* coef = (float4*)workspace;
  float* scale = (float*)((char*)workspace + p.coef_bytes);
  Sums* part = (Sums*)((char*)workspace + p.coef_bytes + p.scale_bytes);
  BnBackwardVectors v{weight, mean, inv_or_var, weight_stride, mean_stride, inv_stride, dw, db, eps, training ? 1 : 0};
  const uint32_t total = (uint32_t)((int64_t)sh.outer * sh.cols);
  if (training && n * s == 2) {
    note_kernel("bn_bwd_pair");
    bn_bwd_pair_kernel<<<(sh.c + 127) / 128, 128, 0, st>>>(x, grad, sh, v, dx);
    count_launch();
    return launch_check("bn_bwd_pair_kernel");
  }
  const int has_sums = training || dw || db;
  if (has_sums && channel_kernel_fits(sh, layout)) {
    note_kernel("bn_backward_channel");
    bn_backward_channel_kernel<<<(unsigned)sh.c, kChannelThreads, 0, st>>>(x, grad, sh, v, dx);
    count_launch();
    return launch_check("bn_backward_channel_kernel");
  }
  if (has_sums) {
    if (p.rows) {
      bn_bwd_rows_kernel<<<dim3((unsigned)sh.c, (unsigned)sh.slabs), kThreads, 0, st>>>(x, grad, sh, v, part);
    } else if (sh.cols % 4 == 0 && aligned16(x) && aligned16(grad)) {
      bn_bwd_cols_kernel<4><<<dim3((unsigned)((sh.cols + 31) / 32), (unsigned)sh.slabs), kThreads, 0, st>>>(x, grad, sh, v, part);
    } else {
      bn_bwd_cols_kernel<1><<<dim3((unsigned)((sh.cols + 7) / 8), (unsigned)sh.slabs), kThreads, 0, st>>>(x, grad, sh, v, part);
    }
    count_launch();
    if (int rc = launch_check("bn_bwd_reduce_kernel")) return rc;
  }
  note_kernel(has_sums ? (p.rows ? "bn_bwd_rows+finalize+apply" : "bn_bwd_cols+finalize+apply") : "bn_bwd_finalize+apply");
  bn_bwd_finalize_kernel<<<(sh.c + 7) / 8, kThreads, 0, st>>>(sh, part, v, has_sums, coef, scale);
  count_launch();
  if (int rc = launch_check("bn_bwd_finalize_kernel")) return rc;
  if (!dx) return B200_OK;
  const bool vec = aligned16(x) && aligned16(grad) && aligned16(dx);
  const bool uniform = sh.inner % 4 == 0;
  const uint32_t first_scalar = vec ? (total & ~3u) : 0;
  if (vec && (total >> 2)) {
    const int grid = apply_grid(((total >> 2) + 1) / 2);
    const ChannelOf ch = channel_of(sh, uniform);
    const uint32_t c4 = (uint32_t)sh.c / 4, threads = (uint32_t)grid * kThreads;
    if (sh.inner == 1 && sh.c % 4 == 0 && threads >= c4) {
      const uint32_t lanes = threads / c4 * c4;
      if (training) bn_bwd_apply_cols_kernel<true><<<grid, kThreads, 0, st>>>(x, grad, dx, coef, scale, (uint32_t)sh.outer, c4, lanes);
      else bn_bwd_apply_cols_kernel<false><<<grid, kThreads, 0, st>>>(x, grad, dx, coef, scale, (uint32_t)sh.outer, c4, lanes);
    } else if (training) {
      if (uniform) bn_bwd_apply_kernel<true, true><<<grid, kThreads, 0, st>>>(x, grad, dx, coef, scale, total, ch);
      else bn_bwd_apply_kernel<false, true><<<grid, kThreads, 0, st>>>(x, grad, dx, coef, scale, total, ch);
    } else {
      if (uniform) bn_bwd_apply_kernel<true, false><<<grid, kThreads, 0, st>>>(x, grad, dx, coef, scale, total, ch);
      else bn_bwd_apply_kernel<false, false><<<grid, kThreads, 0, st>>>(x, grad, dx, coef, scale, total, ch);
    }
    count_launch();
    if (int rc = launch_check("bn_bwd_apply_kernel")) return rc;
  }
  if (first_scalar < total) {
    const int grid = vec ? 1 : apply_grid(total);
    const ChannelOf ch = channel_of(sh, false);
    if (training) bn_bwd_apply_scalar_kernel<true><<<grid, kThreads, 0, st>>>(x, grad, dx, coef, scale, first_scalar, total, ch);
    else bn_bwd_apply_scalar_kernel<false><<<grid, kThreads, 0, st>>>(x, grad, dx, coef, scale, first_scalar, total, ch);
    count_launch();
    if (int rc = launch_check("bn_bwd_apply_scalar_kernel")) return rc;
  }
  return B200_OK;
}

}  // extern "C"
