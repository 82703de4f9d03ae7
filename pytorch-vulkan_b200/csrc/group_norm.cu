// GroupNorm forward and backward for contiguous FP32 [n][c][hw] tensors.  Replaces the
// group_norm_forward / group_norm_backward_input / group_norm_backward_affine shaders of the
// reference (csrc/shaders/group_norm_*.comp) and their host side (csrc/ops/group_norm.cpp:76-155).
//
// A (sample, group) block is c/groups adjacent planes, contiguous in memory.  As in the reference
// one CTA owns one block, but it is a CTA of 16 warps that each stream whole plane segments with
// 16-byte loads, and each kernel makes two passes over its block: the first reads it from HBM, the
// second finds it in L2 (at most three CTAs of a few hundred KB per SM are in flight, far below the
// 126 MB of L2).  HBM traffic is therefore one read and one write per tensor element:
//   forward   statistics (pass 1), normalise and write (pass 2)                    8 B / element
//   backward  the two group sums AND the per-(sample, channel) sums that the affine gradients
//             need (pass 1), input gradient (pass 2); a small second kernel adds the
//             per-sample sums over the batch                                     12 B / element
// The reference reads x and dy a third time for the affine gradients (one thread per channel
// walking the whole batch, group_norm_backward_affine.comp:16-29); here they fall out of pass 1.
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "tc_common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kSegment = 2048;   // most floats of a plane one warp streams per unit
constexpr int kMaxUnits = 4096;  // per-unit partial sums of a block live in shared memory
constexpr size_t kBulkSmemBytes = 200 * 1024;  // two resident blocks of the bulk-copy forward kernel
constexpr int kBulkThreads = 1024;             // its CTA: the only one on its SM, so all the warps the SM holds
constexpr int kBulkChannels = 256;             // most channels per group it takes

struct GnShape {
  int n, c, hw, groups, cpg;  // cpg = channels per group
  int segs, seg_len;          // a plane is cut into `segs` segments of `seg_len` floats (a multiple of 4)
  int units;                  // cpg * segs
  float count;                // cpg * hw
};

struct Moments {
  float n, mean, m2;
};
__device__ __forceinline__ Moments merge(Moments a, Moments b) {
  const float n = a.n + b.n;
  if (!(n > 0.f)) return a;
  const float d = b.mean - a.mean, f = b.n / n;
  return {n, a.mean + d * f, a.m2 + b.m2 + d * d * a.n * f};
}
__device__ __forceinline__ Moments warp_merge(Moments m) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Moments other = {__shfl_xor_sync(0xffffffffu, m.n, o), __shfl_xor_sync(0xffffffffu, m.mean, o),
                     __shfl_xor_sync(0xffffffffu, m.m2, o)};
    m = merge(m, other);
  }
  return m;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The warp walks `len` floats at p (and at q when TWO): f(a) or f(a, b) per element, 16-byte loads
// with four in flight per lane where both pointers are aligned.
template <bool TWO, class F>
__device__ __forceinline__ void warp_stream(const float* __restrict__ p, const float* __restrict__ q, int len, int lane, F&& f) {
  int done = 0;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p) | (TWO ? reinterpret_cast<uintptr_t>(q) : 0);
  if ((bits & 15) == 0) {
    const float4* p4 = reinterpret_cast<const float4*>(p);
    const float4* q4 = reinterpret_cast<const float4*>(q);
    const int quads = len >> 2;
    int i = lane;
    if (TWO) {
      for (; i + 32 < quads; i += 64) {
        const float4 a0 = __ldg(p4 + i), a1 = __ldg(p4 + i + 32), b0 = __ldg(q4 + i), b1 = __ldg(q4 + i + 32);
        f(a0.x, b0.x), f(a0.y, b0.y), f(a0.z, b0.z), f(a0.w, b0.w);
        f(a1.x, b1.x), f(a1.y, b1.y), f(a1.z, b1.z), f(a1.w, b1.w);
      }
      for (; i < quads; i += 32) {
        const float4 a = __ldg(p4 + i), b = __ldg(q4 + i);
        f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w);
      }
    } else {
      for (; i + 96 < quads; i += 128) {
        const float4 a0 = __ldg(p4 + i), a1 = __ldg(p4 + i + 32), a2 = __ldg(p4 + i + 64), a3 = __ldg(p4 + i + 96);
        f(a0.x, 0.f), f(a0.y, 0.f), f(a0.z, 0.f), f(a0.w, 0.f);
        f(a1.x, 0.f), f(a1.y, 0.f), f(a1.z, 0.f), f(a1.w, 0.f);
        f(a2.x, 0.f), f(a2.y, 0.f), f(a2.z, 0.f), f(a2.w, 0.f);
        f(a3.x, 0.f), f(a3.y, 0.f), f(a3.z, 0.f), f(a3.w, 0.f);
      }
      for (; i < quads; i += 32) {
        const float4 a = __ldg(p4 + i);
        f(a.x, 0.f), f(a.y, 0.f), f(a.z, 0.f), f(a.w, 0.f);
      }
    }
    done = quads * 4;
  }
  for (int e = done + lane; e < len; e += 32) f(__ldg(p + e), TWO ? __ldg(q + e) : 0.f);
}

// The same walk producing one output value per element: out[e] = f(a, b).  This is the last use of
// the inputs and the result is not read again here: streaming loads and stores (evict-first), so
// that the lines other CTAs still wait to re-read stay in L2.
template <bool TWO, class F>
__device__ __forceinline__ void warp_map(const float* __restrict__ p, const float* __restrict__ q, float* __restrict__ out, int len,
                                         int lane, F&& f) {
  int done = 0;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(out) | (TWO ? reinterpret_cast<uintptr_t>(q) : 0);
  if ((bits & 15) == 0) {
    const float4* p4 = reinterpret_cast<const float4*>(p);
    const float4* q4 = reinterpret_cast<const float4*>(q);
    float4* o4 = reinterpret_cast<float4*>(out);
    const int quads = len >> 2;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    int i = lane;
    for (; i + 32 < quads; i += 64) {
      const float4 a0 = __ldcs(p4 + i), a1 = __ldcs(p4 + i + 32);
      const float4 b0 = TWO ? __ldcs(q4 + i) : zero, b1 = TWO ? __ldcs(q4 + i + 32) : zero;
      __stcs(o4 + i, make_float4(f(a0.x, b0.x), f(a0.y, b0.y), f(a0.z, b0.z), f(a0.w, b0.w)));
      __stcs(o4 + i + 32, make_float4(f(a1.x, b1.x), f(a1.y, b1.y), f(a1.z, b1.z), f(a1.w, b1.w)));
    }
    for (; i < quads; i += 32) {
      const float4 a = __ldcs(p4 + i), b = TWO ? __ldcs(q4 + i) : zero;
      __stcs(o4 + i, make_float4(f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w)));
    }
    done = quads * 4;
  }
  for (int e = done + lane; e < len; e += 32) __stcs(out + e, f(__ldcs(p + e), TWO ? __ldcs(q + e) : 0.f));
}

// Unit u of a block: plane (channel within the group) and the segment's offset and length in it.
struct Unit {
  int plane, off, len;
};
__device__ __forceinline__ Unit unit_of(const GnShape& sh, int u) {
  const int plane = u / sh.segs, off = (u - plane * sh.segs) * sh.seg_len;
  return {plane, off, min(sh.seg_len, sh.hw - off)};
}

// ---- forward -----------------------------------------------------------------------------------
// grid = n * groups.  Mean and 1/sqrt(var + eps) per block (group_norm_forward.comp:24-47: shifted
// first pass, centred second pass; here one pass of pairwise-merged moments, each thread summing
// around a sample of its own segment), then y = (x - mean) * rstd * gamma[ch] + beta[ch] (:49-54).
__global__ void __launch_bounds__(kThreads, 3) gn_forward_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                 const float* __restrict__ beta, GnShape sh, float eps,
                                                                 float* __restrict__ y, float* __restrict__ means,
                                                                 float* __restrict__ rstds) {
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = row % sh.groups;
  const size_t base = ((size_t)(row / sh.groups) * sh.c + (size_t)group * sh.cpg) * sh.hw;
  const float* xb = x + base;
  const float origin = __ldg(xb);
  Moments acc = {0.f, 0.f, 0.f};
  for (int u = warp; u < sh.units; u += kWarps) {
    const Unit un = unit_of(sh, u);
    const float* p = xb + (size_t)un.plane * sh.hw + un.off;
    const float k = __ldg(p + min(lane, un.len - 1));
    float cnt = 0.f, s = 0.f, q = 0.f;
    warp_stream<false>(p, nullptr, un.len, lane, [&](float v, float) {
      const float d = v - k;
      s += d;
      q = fmaf(d, d, q);
      cnt += 1.f;
    });
    if (cnt > 0.f) {
      const float mean_d = s / cnt;
      acc = merge(acc, Moments{cnt, (k - origin) + mean_d, fmaxf(q - s * mean_d, 0.f)});
    }
  }
  __shared__ Moments warp_part[32];
  acc = warp_merge(acc);
  if (threadIdx.x < 32) warp_part[threadIdx.x] = Moments{0.f, 0.f, 0.f};
  __syncthreads();
  if (lane == 0) warp_part[warp] = acc;
  __syncthreads();
  // every warp folds the partial results itself; the mean stays relative to the origin so that its
  // low part survives in the subtraction below
  const Moments total = warp_merge(warp_part[lane]);
  const float mean_rel = total.mean, rstd = 1.f / sqrtf(total.m2 / sh.count + eps);
  if (threadIdx.x == 0) {
    means[row] = origin + mean_rel;
    rstds[row] = rstd;
  }
  for (int u = warp; u < sh.units; u += kWarps) {
    const Unit un = unit_of(sh, u);
    const int ch = group * sh.cpg + un.plane;
    const float scale = rstd * (gamma ? __ldg(gamma + ch) : 1.f), shift = beta ? __ldg(beta + ch) : 0.f;
    const size_t at = (size_t)un.plane * sh.hw + un.off;
    warp_map<false>(xb + at, nullptr, y + base + at, un.len, lane,
                    [&](float v, float) { return ((v - origin) - mean_rel) * scale + shift; });
  }
}

// The same computation with the block resident in shared memory: one thread brings the block in
// with bulk asynchronous copies (completion counted in bytes on an mbarrier), everybody computes
// the statistics and the result from shared memory, and while they do the copy of the CTA's next
// block is already in flight into the other buffer.  The block is read from HBM once and the
// bytes in flight do not depend on how many warps are waiting.  Used when two blocks fit
// but not four (100 KB < 2 * count * 4 bytes <= 200 KB: one CTA of 1024 threads per SM), planes are
// multiples of four floats, x is 16-byte aligned and every CTA gets four blocks or more.
// Every wait is bounded: a wait that gives up sets the status word and the CTA leaves.
__global__ void __launch_bounds__(kBulkThreads, 1) gn_forward_bulk_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                      const float* __restrict__ beta, GnShape sh, float eps,
                                                                      float* __restrict__ y, float* __restrict__ means,
                                                                      float* __restrict__ rstds, int blocks, FastDiv plane_quads,
                                                                      int* status) {
  extern __shared__ __align__(128) unsigned char gn_smem[];
  __shared__ __align__(8) unsigned long long full[2];
  __shared__ int abort_flag;
  __shared__ Moments warp_part[kBulkThreads / 32];
  __shared__ float2 affine[kBulkChannels];  // per channel of the group: rstd * gamma, beta
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t block_bytes = (uint32_t)(sh.cpg * sh.hw) * 4u;
  const int quads = (sh.cpg * sh.hw) >> 2;
  const uint32_t bar[2] = {tc::smem_u32(&full[0]), tc::smem_u32(&full[1])};
  if (threadIdx.x == 0) {
    tc::mbar_init(bar[0], 1);
    tc::mbar_init(bar[1], 1);
    abort_flag = 0;
    tc::fence_barrier_init();
  }
  __syncthreads();
  auto block_base = [&](int blk) { return ((size_t)(blk / sh.groups) * sh.c + (size_t)(blk % sh.groups) * sh.cpg) * sh.hw; };
  auto issue = [&](int blk, int b) {  // one thread: the whole block in pieces of at most 32 KB
    const char* src = reinterpret_cast<const char*>(x + block_base(blk));
    const uint32_t dst = tc::smem_u32(gn_smem) + (uint32_t)b * block_bytes;
    tc::mbar_expect_tx(bar[b], block_bytes);
    for (uint32_t off = 0; off < block_bytes; off += 32768u)
      tc::bulk_g2s(dst + off, src + off, min(32768u, block_bytes - off), bar[b]);
  };
  int it = 0, pending = -1;  // pending: buffer with a copy in flight that nobody has waited for yet
  if (threadIdx.x == 0 && (int)blockIdx.x < blocks) issue(blockIdx.x, 0);
  for (int blk = blockIdx.x; blk < blocks; blk += gridDim.x, ++it) {
    const int b = it & 1, next = blk + gridDim.x;
    pending = -1;
    if (next < blocks) {
      if (threadIdx.x == 0) issue(next, b ^ 1);  // that buffer's readers passed the barrier ending the previous round
      pending = b ^ 1;
    }
    if (!tc::mbar_wait(bar[b], (uint32_t)(it >> 1) & 1u, &abort_flag, status, tc::STATUS_TIMEOUT_TMA)) break;
    const float4* s4 = reinterpret_cast<const float4*>(gn_smem + (size_t)b * block_bytes);
    const float origin = reinterpret_cast<const float*>(s4)[0];
    // statistics: every thread sums around its own first value
    Moments acc = {0.f, 0.f, 0.f};
    if ((int)threadIdx.x < quads) {
      const float k = s4[threadIdx.x].x;
      float cnt = 0.f, s = 0.f, q = 0.f;
      for (int i = threadIdx.x; i < quads; i += kBulkThreads) {
        const float4 v = s4[i];
        const float d0 = v.x - k, d1 = v.y - k, d2 = v.z - k, d3 = v.w - k;
        s += (d0 + d1) + (d2 + d3);
        q = fmaf(d0, d0, fmaf(d1, d1, fmaf(d2, d2, fmaf(d3, d3, q))));
        cnt += 4.f;
      }
      const float mean_d = s / cnt;
      acc = Moments{cnt, (k - origin) + mean_d, fmaxf(q - s * mean_d, 0.f)};
    }
    acc = warp_merge(acc);
    if (lane == 0) warp_part[warp] = acc;
    __syncthreads();
    // every warp folds the 32 partial results itself: no second barrier, no serial chain
    const Moments total = warp_merge(warp_part[lane]);
    const float mean_rel = total.mean, rstd = 1.f / sqrtf(total.m2 / sh.count + eps);
    if (threadIdx.x == 0) {
      means[blk] = origin + mean_rel;
      rstds[blk] = rstd;
    }
    const int ch0 = (blk % sh.groups) * sh.cpg;
    if ((int)threadIdx.x < sh.cpg)
      affine[threadIdx.x] = make_float2(rstd * (gamma ? __ldg(gamma + ch0 + threadIdx.x) : 1.f), beta ? __ldg(beta + ch0 + threadIdx.x) : 0.f);
    __syncthreads();
    float4* y4 = reinterpret_cast<float4*>(y + block_base(blk));
#pragma unroll 4
    for (int i = threadIdx.x; i < quads; i += kBulkThreads) {
      const float2 ab = affine[plane_quads.div((uint32_t)i)];
      const float scale = ab.x, shift = ab.y;
      const float4 v = s4[i];
      __stcs(y4 + i, make_float4(((v.x - origin) - mean_rel) * scale + shift, ((v.y - origin) - mean_rel) * scale + shift,
                                 ((v.z - origin) - mean_rel) * scale + shift, ((v.w - origin) - mean_rel) * scale + shift));
    }
    __syncthreads();  // the buffer may be overwritten by the copy issued in the next round
  }
  // after a wait that gave up: do not leave while a copy into this CTA's shared memory may still land
  if (abort_flag && threadIdx.x == 0 && pending >= 0)
    tc::mbar_wait(bar[pending], (uint32_t)((it + 1) >> 1) & 1u, nullptr, status, tc::STATUS_TIMEOUT_TMA);
}

// ---- backward ------------------------------------------------------------------------------------
// grid = n * groups.  Pass 1: per unit s1 = sum dy, s2 = sum dy * z with z = (x - mean) * rstd.  The
// units of a plane add up (in unit order) to the per-(sample, channel) sums the affine gradients
// need; weighted by gamma they add up to the block's a and b (group_norm_backward_input.comp:26-37).
// Pass 2: dx = rstd * (gamma dy - a / count - z * b / count) (:38-45).
__global__ void __launch_bounds__(kThreads, 3) gn_backward_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                  const float* __restrict__ means, const float* __restrict__ rstds,
                                                                  const float* __restrict__ gamma, GnShape sh, float* __restrict__ dx,
                                                                  float* __restrict__ plane_sums) {
  extern __shared__ float unit_sums[];  // [units][2]
  __shared__ float totals[2];
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = row % sh.groups, sample = row / sh.groups;
  const size_t base = ((size_t)sample * sh.c + (size_t)group * sh.cpg) * sh.hw;
  const float mean = __ldg(means + row), rstd = __ldg(rstds + row);
  for (int u = warp; u < sh.units; u += kWarps) {
    const Unit un = unit_of(sh, u);
    const size_t at = base + (size_t)un.plane * sh.hw + un.off;
    float s1 = 0.f, s2 = 0.f;
    warp_stream<true>(x + at, dy + at, un.len, lane, [&](float xv, float gv) {
      s1 += gv;
      s2 = fmaf(gv, (xv - mean) * rstd, s2);
    });
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) unit_sums[2 * u] = s1, unit_sums[2 * u + 1] = s2;
  }
  __syncthreads();
  // per plane: add its segments in order; one warp then folds the planes into a and b
  for (int pl = threadIdx.x; pl < sh.cpg; pl += kThreads) {
    float s1 = 0.f, s2 = 0.f;
    for (int sgi = 0; sgi < sh.segs; ++sgi) s1 += unit_sums[2 * (pl * sh.segs + sgi)], s2 += unit_sums[2 * (pl * sh.segs + sgi) + 1];
    if (plane_sums) {
      const size_t at = ((size_t)sample * sh.c + (size_t)group * sh.cpg + pl) * 2;
      plane_sums[at] = s1, plane_sums[at + 1] = s2;
    }
    unit_sums[2 * pl * sh.segs] = s1, unit_sums[2 * pl * sh.segs + 1] = s2;  // the plane's first unit now holds its total
  }
  __syncthreads();
  if (!dx) return;
  if (warp == 0) {
    float a = 0.f, b = 0.f;
    for (int pl = lane; pl < sh.cpg; pl += 32) {
      const float w = gamma ? __ldg(gamma + group * sh.cpg + pl) : 1.f;
      a = fmaf(w, unit_sums[2 * pl * sh.segs], a);
      b = fmaf(w, unit_sums[2 * pl * sh.segs + 1], b);
    }
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) totals[0] = a / sh.count, totals[1] = b / sh.count;
  }
  __syncthreads();
  const float avg = totals[0], avg_z = totals[1];
  for (int u = warp; u < sh.units; u += kWarps) {
    const Unit un = unit_of(sh, u);
    const float w = gamma ? __ldg(gamma + group * sh.cpg + un.plane) : 1.f;
    const size_t at = base + (size_t)un.plane * sh.hw + un.off;
    warp_map<true>(x + at, dy + at, dx + at, un.len, lane, [&](float xv, float gv) {
      const float z = (xv - mean) * rstd;
      return rstd * (gv * w - avg - z * avg_z);
    });
  }
}

// dgamma[ch] = sum over samples of s2, dbeta[ch] = sum of s1 (the result of
// group_norm_backward_affine.comp:16-31).  One warp per channel: lane l adds samples l, l + 32, ...
// in order and the lanes are folded by shuffles, so the result does not depend on the launch.
__global__ void __launch_bounds__(256) gn_affine_kernel(const float* __restrict__ plane_sums, int n, int c, float* __restrict__ dgamma,
                                                        float* __restrict__ dbeta) {
  const int ch = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (ch >= c) return;
  float s1 = 0.f, s2 = 0.f;
  for (int b = lane; b < n; b += 32) {
    const float2 v = __ldg(reinterpret_cast<const float2*>(plane_sums) + (size_t)b * c + ch);
    s1 += v.x, s2 += v.y;
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  if (lane == 0) {
    if (dgamma) dgamma[ch] = s2;
    if (dbeta) dbeta[ch] = s1;
  }
}

int make_shape(int64_t n, int64_t c, int64_t hw, int64_t groups, GnShape* out) {
  if (!(groups > 0 && n > 0 && c > 0 && hw > 0 && c % groups == 0))
    return fail(B200_EINVAL, "native_group_norm: invalid batch, channel, group or spatial dimensions");
  if (n * groups > INT32_MAX || c > INT32_MAX || hw > INT32_MAX || (c / groups) * hw > INT32_MAX)
    return fail(B200_ERANGE, "native_group_norm: a (sample, group) block exceeds int32 indexing");
  GnShape sh{};
  sh.n = (int)n, sh.c = (int)c, sh.hw = (int)hw, sh.groups = (int)groups, sh.cpg = (int)(c / groups);
  if (sh.cpg > kMaxUnits) return fail(B200_EUNSUPPORTED, "native_group_norm: more than %d channels per group", kMaxUnits);
  int segs = (sh.hw + kSegment - 1) / kSegment;
  const int most = kMaxUnits / sh.cpg;  // keep cpg * segs within the shared-memory table
  if (segs > most) segs = most;
  sh.segs = segs;
  sh.seg_len = ((sh.hw + segs - 1) / segs + 3) & ~3;
  sh.segs = (sh.hw + sh.seg_len - 1) / sh.seg_len;  // rounding the length up can save a segment
  sh.units = sh.cpg * sh.segs;
  sh.count = (float)((double)sh.cpg * (double)sh.hw);
  *out = sh;
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_group_norm_workspace(int64_t n, int64_t c, int64_t hw, int64_t groups) {
  GnShape sh;
  if (make_shape(n, c, hw, groups, &sh)) return 0;
  return (size_t)n * (size_t)c * 2 * sizeof(float);
}

int b200_group_norm_forward(int64_t n, int64_t c, int64_t hw, int64_t groups, const float* x, const float* weight,
                            const float* bias, float eps, float* y, float* mean, float* rstd, void* stream) {
  if (int rc = ensure_init()) return rc;
  GnShape sh;
  if (int rc = make_shape(n, c, hw, groups, &sh)) return rc;
  if (!x || !y || !mean || !rstd) return fail(B200_EINVAL, "native_group_norm: null tensor");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t block_bytes = (size_t)sh.cpg * sh.hw * sizeof(float);
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  const int blocks = (int)(n * groups);
  const int bulk_grid = std::min(blocks, sm_count());
  // the resident form pays once the copy pipeline has rounds to overlap: four blocks or more per CTA
  if (aligned && sh.hw % 4 == 0 && sh.cpg <= kBulkChannels && 2 * block_bytes > kBulkSmemBytes / 2 && 2 * block_bytes <= kBulkSmemBytes &&
      blocks >= 4 * bulk_grid) {
    static std::once_flag once;
    static cudaError_t opt_in = cudaSuccess;
    std::call_once(once, [] {
      opt_in = cudaFuncSetAttribute(gn_forward_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBulkSmemBytes);
    });
    B200_CUDA(opt_in);
    note_kernel("gn_forward_bulk");
    gn_forward_bulk_kernel<<<bulk_grid, kBulkThreads, 2 * block_bytes, st>>>(x, weight, bias, sh, eps, y, mean, rstd, blocks,
                                                                            FastDiv((uint32_t)(sh.hw / 4)), device_status_word());
    count_launch();
    return launch_check("gn_forward_bulk_kernel");
  }
  note_kernel("gn_forward");
  gn_forward_kernel<<<(unsigned)(n * groups), kThreads, 0, st>>>(x, weight, bias, sh, eps, y, mean, rstd);
  count_launch();
  return launch_check("gn_forward_kernel");
}

int b200_group_norm_backward(int64_t n, int64_t c, int64_t hw, int64_t groups, const float* grad, const float* x,
                             const float* mean, const float* rstd, const float* weight, float* dx, float* dw, float* db,
                             void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = ensure_init()) return rc;
  GnShape sh;
  if (int rc = make_shape(n, c, hw, groups, &sh)) return rc;
  if (!grad || !x || !mean || !rstd) return fail(B200_EINVAL, "native_group_norm_backward: null tensor");
  if (!dx && !dw && !db) return B200_OK;
  const bool affine = dw || db;
  if (affine && (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 7) || workspace_bytes < (size_t)n * c * 2 * sizeof(float)))
    return fail(B200_EWORKSPACE, "native_group_norm_backward: workspace missing, unaligned or smaller than b200_group_norm_workspace()");
  cudaStream_t st = (cudaStream_t)stream;
  float* plane_sums = affine ? (float*)workspace : nullptr;
  note_kernel(affine ? "gn_backward+affine" : "gn_backward");
  gn_backward_kernel<<<(unsigned)(n * groups), kThreads, (size_t)sh.units * 2 * sizeof(float), st>>>(grad, x, mean, rstd, weight, sh,
                                                                                                      dx, plane_sums);
  count_launch();
  if (int rc = launch_check("gn_backward_kernel")) return rc;
  if (affine) {
    gn_affine_kernel<<<(unsigned)((c + 7) / 8), 256, 0, st>>>(plane_sums, (int)n, (int)c, dw, db);
    count_launch();
    if (int rc = launch_check("gn_affine_kernel")) return rc;
  }
  return B200_OK;
}

}  // extern "C"
