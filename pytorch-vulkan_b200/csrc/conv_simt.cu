// CUDA-core FP32 kernels of the Conv2D path: exact-FP32 candidates that accept every
// geometry and every strided view.  They are the "direct" and "tiled" candidates of the
// dispatcher and the fall-back for shapes the tcgen05 kernels do not take (tiny channel
// counts, ragged groups).  Arithmetic is FP32 FMA with a K-ascending accumulation per
// output, like the reference's tiled shaders.
//
// Reference arithmetic restated here (paths inside the reference tree):
//   direct:  csrc/shaders/conv2d_forward.comp:11-43, conv2d_backward_input.comp:10-47,
//            conv2d_backward_weight.comp:10-41, conv2d_backward_bias.comp:9-27
//   tiled:   csrc/shaders/conv2d_tiled_body.glsl:53-86,
//            conv2d_backward_input_tiled_body.glsl:49-93,
//            conv2d_backward_weight_tiled_body.glsl:42-70 + conv2d_backward_weight_finalize.comp:9-18
//   dBias:   csrc/shaders/conv2d_backward_bias_reduce.comp:9-24 (here: warp-shuffle tree)
//   GEMM:    csrc/shaders/matmul_strided.comp:1-65, matmul_strided_bias.comp:33-68
#include "common.cuh"

namespace b200 {

enum { PH_FWD = 0, PH_DX = 1, PH_DW = 2, PH_GEMM = 3 };

struct IgemmArgs {
  ConvGeom g;
  View4 a, b;  // fwd: a = w, b = x.  dx: a = w, b = dy.  dw: a = dy, b = x.  gemm: a = A, b = B (s0,s1 used)
  const float* bias;
  long long bias_stride;
  float* out;
  long long M, N, K;  // per-group GEMM extents
  int span;           // dW: positions per split
  float alpha, beta;  // gemm epilogue
};

// ---------------------------------------------------------------------------------------
// Operand fetchers.  (m, n, k) are indices inside one group's GEMM.
// ---------------------------------------------------------------------------------------
template <int PH>
__device__ __forceinline__ float fetch_a(const IgemmArgs& p, int group, long long m, long long k) {
  const ConvGeom& g = p.g;
  if (PH == PH_GEMM) return p.a.ptr[m * p.a.s0 + k * p.a.s1];
  const int taps = g.kh * g.kw;
  if (PH == PH_FWD) {  // W[oc][ci][ky][kx], k = (ci,ky,kx)
    const int ci = (int)(k / taps), rem = (int)(k % taps);
    const long long oc = (long long)group * g.cog + m;
    return p.a.ptr[oc * p.a.s0 + ci * p.a.s1 + (rem / g.kw) * p.a.s2 + (rem % g.kw) * p.a.s3];
  }
  if (PH == PH_DX) {  // W[oc][m][ky][kx], k = (co,ky,kx)
    const int co = (int)(k / taps), rem = (int)(k % taps);
    const long long oc = (long long)group * g.cog + co;
    return p.a.ptr[oc * p.a.s0 + m * p.a.s1 + (rem / g.kw) * p.a.s2 + (rem % g.kw) * p.a.s3];
  }
  // PH_DW: dY[b][oc][oy][ox], k = position
  const int spatial = g.oh * g.ow;
  const long long b = k / spatial;
  const int pos = (int)(k % spatial);
  const long long oc = (long long)group * g.cog + m;
  return p.a.ptr[b * p.a.s0 + oc * p.a.s1 + (pos / g.ow) * p.a.s2 + (pos % g.ow) * p.a.s3];
}

// Per-thread decode of the fixed N index of its B loads.
struct NCtx {
  bool valid;
  long long base;  // address contribution that does not depend on k
  int y0, x0;      // fwd: oy*sh-ph, ox*sw-pw.  dx: y+ph, x+pw.  dw: ky*dh-ph, kx*dw-pw
};

template <int PH>
__device__ __forceinline__ NCtx make_nctx(const IgemmArgs& p, int group, long long n) {
  const ConvGeom& g = p.g;
  NCtx c;
  c.valid = n < p.N;
  c.base = 0;
  c.y0 = c.x0 = 0;
  if (!c.valid) return c;
  if (PH == PH_GEMM) {
    c.base = n * p.b.s1;
  } else if (PH == PH_FWD) {
    const int spatial = g.oh * g.ow;
    const long long b = n / spatial;
    const int pos = (int)(n % spatial);
    c.y0 = (pos / g.ow) * g.sh - g.ph;
    c.x0 = (pos % g.ow) * g.sw - g.pw;
    c.base = b * p.b.s0 + (long long)group * g.cig * p.b.s1;
  } else if (PH == PH_DX) {
    const int spatial = g.h * g.w;
    const long long b = n / spatial;
    const int pos = (int)(n % spatial);
    c.y0 = pos / g.w + g.ph;
    c.x0 = pos % g.w + g.pw;
    c.base = b * p.b.s0 + (long long)group * g.cog * p.b.s1;
  } else {  // PH_DW: n = (ci,ky,kx)
    const int taps = g.kh * g.kw;
    const int ci = (int)(n / taps), rem = (int)(n % taps);
    c.y0 = (rem / g.kw) * g.dh - g.ph;
    c.x0 = (rem % g.kw) * g.dw - g.pw;
    c.base = ((long long)group * g.cig + ci) * p.b.s1;
  }
  return c;
}

template <int PH>
__device__ __forceinline__ float fetch_b(const IgemmArgs& p, const NCtx& c, long long k) {
  const ConvGeom& g = p.g;
  if (PH == PH_GEMM) return p.b.ptr[k * p.b.s0 + c.base];
  if (PH == PH_FWD) {
    const int taps = g.kh * g.kw;
    const int ci = (int)(k / taps), rem = (int)(k % taps);
    const int iy = c.y0 + (rem / g.kw) * g.dh, ix = c.x0 + (rem % g.kw) * g.dw;
    if (iy < 0 || iy >= g.h || ix < 0 || ix >= g.w) return 0.f;
    return p.b.ptr[c.base + ci * p.b.s1 + iy * p.b.s2 + ix * p.b.s3];
  }
  if (PH == PH_DX) {
    const int taps = g.kh * g.kw;
    const int co = (int)(k / taps), rem = (int)(k % taps);
    int yh = c.y0 - (rem / g.kw) * g.dh, xw = c.x0 - (rem % g.kw) * g.dw;
    if (yh < 0 || xw < 0) return 0.f;
    if (g.sh != 1 || g.sw != 1) {
      if (yh % g.sh != 0 || xw % g.sw != 0) return 0.f;
      yh /= g.sh;
      xw /= g.sw;
    }
    if (yh >= g.oh || xw >= g.ow) return 0.f;
    return p.b.ptr[c.base + co * p.b.s1 + yh * p.b.s2 + xw * p.b.s3];
  }
  // PH_DW: k = position
  const int spatial = g.oh * g.ow;
  const long long b = k / spatial;
  const int pos = (int)(k % spatial);
  const int iy = (pos / g.ow) * g.sh + c.y0, ix = (pos % g.ow) * g.sw + c.x0;
  if (iy < 0 || iy >= g.h || ix < 0 || ix >= g.w) return 0.f;
  return p.b.ptr[b * p.b.s0 + c.base + iy * p.b.s2 + ix * p.b.s3];
}

template <int PH>
__device__ __forceinline__ void store_out(const IgemmArgs& p, int group, int split, long long m, long long n,
                                          float v) {
  const ConvGeom& g = p.g;
  if (m >= p.M || n >= p.N) return;
  if (PH == PH_GEMM) {
    float r = p.alpha * v;  // alpha scales the product whether or not a bias follows
    if (p.bias && p.beta != 0.f) r += p.beta * p.bias[n * p.bias_stride];
    p.out[m * p.N + n] = r;
  } else if (PH == PH_FWD) {
    const int spatial = g.oh * g.ow;
    const long long b = n / spatial, pos = n % spatial, oc = (long long)group * g.cog + m;
    p.out[(b * g.cout + oc) * spatial + pos] = v + (p.bias ? p.bias[oc * p.bias_stride] : 0.f);
  } else if (PH == PH_DX) {
    const int spatial = g.h * g.w;
    const long long b = n / spatial, pos = n % spatial, ic = (long long)group * g.cig + m;
    p.out[(b * g.cin + ic) * spatial + pos] = v;
  } else {
    const long long oc = (long long)group * g.cog + m;
    p.out[((long long)split * g.cout + oc) * p.N + n] = v;
  }
}

// 64x64x16 block tile, 256 threads, 4x4 outputs per thread.
constexpr int BM = 64, BN = 64, BK = 16;

template <int PH>
__global__ void __launch_bounds__(256) simt_igemm_kernel(const IgemmArgs p) {
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tiles_m = (int)((p.M + BM - 1) / BM);
  const int group = blockIdx.y / tiles_m;
  const long long m0 = (long long)(blockIdx.y % tiles_m) * BM;
  const long long n0 = (long long)blockIdx.x * BN;
  const int split = blockIdx.z;
  long long k_begin = 0, k_end = p.K;
  if (PH == PH_DW) {
    k_begin = (long long)split * p.span;
    k_end = min(p.K, k_begin + p.span);
  }
  const NCtx nctx = make_nctx<PH>(p, group, n0 + (tid & 63));
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (long long k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + 256 * j;
      const int am = i >> 4, ak = i & 15;  // A: 16 consecutive threads walk K
      const long long m = m0 + am, k = k0 + ak;
      As[ak][am] = (m < p.M && k < k_end) ? fetch_a<PH>(p, group, m, k) : 0.f;
      const int bk = i >> 6;  // B: 64 consecutive threads walk N (n index fixed per thread)
      const long long kb = k0 + bk;
      Bs[bk][tid & 63] = (nctx.valid && kb < k_end) ? fetch_b<PH>(p, nctx, kb) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) store_out<PH>(p, group, split, m0 + ty * 4 + i, n0 + tx * 4 + j, acc[i][j]);
}

template <int PH>
static int launch_igemm(const IgemmArgs& p, int groups, int splits, cudaStream_t st, const char* name) {
  const long long gx = div_up64(p.N, BN), gy = div_up64(p.M, BM) * groups;
  if (gx > 2147483647ll || gy > 65535 || splits > 65535)
    return fail(B200_ERANGE, "%s: grid (%lld,%lld,%d) exceeds launch limits", name, gx, gy, splits);
  simt_igemm_kernel<PH><<<dim3((unsigned)gx, (unsigned)gy, (unsigned)splits), 256, 0, st>>>(p);
  count_launch();
  return launch_check(name);
}

int simt_igemm_forward(const ConvGeom& g, View4 x, View4 w, const float* bias, long long bias_stride, float* y,
                       cudaStream_t st) {
  IgemmArgs p{};
  p.g = g; p.a = w; p.b = x; p.bias = bias; p.bias_stride = bias_stride; p.out = y;
  p.M = g.cog; p.N = (long long)g.n * g.oh * g.ow; p.K = (long long)g.cig * g.kh * g.kw;
  return launch_igemm<PH_FWD>(p, g.groups, 1, st, "simt_igemm_forward");
}

int simt_igemm_dinput(const ConvGeom& g, View4 dy, View4 w, float* dx, cudaStream_t st) {
  IgemmArgs p{};
  p.g = g; p.a = w; p.b = dy; p.out = dx;
  p.M = g.cig; p.N = (long long)g.n * g.h * g.w; p.K = (long long)g.cog * g.kh * g.kw;
  return launch_igemm<PH_DX>(p, g.groups, 1, st, "simt_igemm_dinput");
}

__global__ void __launch_bounds__(256) finalize_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                       long long count, int splits) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= count) return;
  float sum = 0.f;
  for (int s = 0; s < splits; ++s) sum += partial[(long long)s * count + i];  // ascending: deterministic
  out[i] = sum;
}

int finalize_splits(const float* partial, float* out, long long count, int splits, cudaStream_t st) {
  finalize_kernel<<<(unsigned)div_up64(count, 256), 256, 0, st>>>(partial, out, count, splits);
  count_launch();
  return launch_check("finalize_kernel");
}

int simt_igemm_dweight(const ConvGeom& g, View4 x, View4 dy, float* dw, float* partial, int splits, int span,
                       cudaStream_t st) {
  IgemmArgs p{};
  p.g = g; p.a = dy; p.b = x;
  p.M = g.cog; p.N = (long long)g.cig * g.kh * g.kw; p.K = (long long)g.n * g.oh * g.ow;
  p.span = splits > 1 ? span : (int)p.K;
  p.out = splits > 1 ? partial : dw;
  if (int rc = launch_igemm<PH_DW>(p, g.groups, splits, st, "simt_igemm_dweight")) return rc;
  if (splits > 1) return finalize_splits(partial, dw, (long long)g.cout * p.N, splits, st);
  return B200_OK;
}

int simt_gemm(long long M, long long N, long long K, const float* A, long long sa0, long long sa1, const float* B,
              long long sb0, long long sb1, const float* bias, float alpha, float beta, float* C, cudaStream_t st) {
  IgemmArgs p{};
  p.a = {A, sa0, sa1, 0, 0};
  p.b = {B, sb0, sb1, 0, 0};
  p.bias = bias; p.bias_stride = 1; p.alpha = alpha; p.beta = beta; p.out = C;
  p.M = M; p.N = N; p.K = K;
  return launch_igemm<PH_GEMM>(p, 1, 1, st, "simt_gemm");
}

// ---------------------------------------------------------------------------------------
// Direct candidates: one thread per output element, loop order of the direct shaders.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) direct_forward_kernel(ConvGeom g, View4 x, View4 w, const float* bias,
                                                             long long bias_stride, float* y, long long total) {
  const long long idx = blockIdx.x * 128ll + threadIdx.x;
  if (idx >= total) return;
  const int hw = g.oh * g.ow;
  const int ow = (int)(idx % g.ow), oh = (int)((idx / g.ow) % g.oh);
  const int oc = (int)((idx / hw) % g.cout);
  const long long b = idx / ((long long)g.cout * hw);
  const int first_in = (oc / g.cog) * g.cig;
  float sum = bias ? bias[oc * bias_stride] : 0.f;
  for (int c = 0; c < g.cig; ++c)
    for (int kh = 0; kh < g.kh; ++kh) {
      const int ih = oh * g.sh - g.ph + kh * g.dh;
      if (ih < 0 || ih >= g.h) continue;
      for (int kw = 0; kw < g.kw; ++kw) {
        const int iw = ow * g.sw - g.pw + kw * g.dw;
        if (iw < 0 || iw >= g.w) continue;
        sum = fmaf(x.ptr[b * x.s0 + (first_in + c) * x.s1 + ih * x.s2 + iw * x.s3],
                   w.ptr[oc * w.s0 + c * w.s1 + kh * w.s2 + kw * w.s3], sum);
      }
    }
  y[idx] = sum;
}

__global__ void __launch_bounds__(128) direct_dinput_kernel(ConvGeom g, View4 go, View4 w, float* dx,
                                                            long long total) {
  const long long idx = blockIdx.x * 128ll + threadIdx.x;
  if (idx >= total) return;
  const int hw = g.h * g.w;
  const int iw = (int)(idx % g.w), ih = (int)((idx / g.w) % g.h);
  const int ic = (int)((idx / hw) % g.cin);
  const long long b = idx / ((long long)g.cin * hw);
  const int group = ic / g.cig, cg = ic % g.cig;
  float sum = 0.f;
  for (int co = 0; co < g.cog; ++co) {
    const int oc = group * g.cog + co;
    for (int kh = 0; kh < g.kh; ++kh) {
      const int ih0 = ih + g.ph - kh * g.dh;
      if (ih0 < 0 || ih0 % g.sh != 0) continue;
      const int out_h = ih0 / g.sh;
      if (out_h >= g.oh) continue;
      for (int kw = 0; kw < g.kw; ++kw) {
        const int iw0 = iw + g.pw - kw * g.dw;
        if (iw0 < 0 || iw0 % g.sw != 0) continue;
        const int out_w = iw0 / g.sw;
        if (out_w >= g.ow) continue;
        sum = fmaf(go.ptr[b * go.s0 + oc * go.s1 + out_h * go.s2 + out_w * go.s3],
                   w.ptr[oc * w.s0 + cg * w.s1 + kh * w.s2 + kw * w.s3], sum);
      }
    }
  }
  dx[idx] = sum;
}

__global__ void __launch_bounds__(128) direct_dweight_kernel(ConvGeom g, View4 x, View4 go, float* dw,
                                                             long long total) {
  const long long idx = blockIdx.x * 128ll + threadIdx.x;
  if (idx >= total) return;
  const int kw = (int)(idx % g.kw), kh = (int)((idx / g.kw) % g.kh);
  const int c = (int)((idx / (g.kw * g.kh)) % g.cig);
  const int oc = (int)(idx / ((long long)g.kw * g.kh * g.cig));
  const int ic = (oc / g.cog) * g.cig + c;
  float sum = 0.f;
  for (long long b = 0; b < g.n; ++b)
    for (int oh = 0; oh < g.oh; ++oh) {
      const int ih = oh * g.sh - g.ph + kh * g.dh;
      if (ih < 0 || ih >= g.h) continue;
      for (int ow = 0; ow < g.ow; ++ow) {
        const int iw = ow * g.sw - g.pw + kw * g.dw;
        if (iw < 0 || iw >= g.w) continue;
        sum = fmaf(x.ptr[b * x.s0 + ic * x.s1 + ih * x.s2 + iw * x.s3],
                   go.ptr[b * go.s0 + oc * go.s1 + oh * go.s2 + ow * go.s3], sum);
      }
    }
  dw[idx] = sum;
}

__global__ void __launch_bounds__(128) direct_dbias_kernel(ConvGeom g, View4 go, float* db) {
  const int oc = blockIdx.x * 128 + threadIdx.x;
  if (oc >= g.cout) return;
  float sum = 0.f;
  for (long long b = 0; b < g.n; ++b)
    for (int oh = 0; oh < g.oh; ++oh)
      for (int ow = 0; ow < g.ow; ++ow) sum += go.ptr[b * go.s0 + oc * go.s1 + oh * go.s2 + ow * go.s3];
  db[oc] = sum;
}

int simt_direct(const ConvGeom& g, int phase, View4 a, View4 b, const float* bias, long long bias_stride,
                float* out, cudaStream_t st) {
  long long total = 0;
  const char* name = "";
  switch (phase) {
    case B200_PHASE_FORWARD:
      total = (long long)g.n * g.cout * g.oh * g.ow;
      name = "direct_forward_kernel";
      direct_forward_kernel<<<(unsigned)div_up64(total, 128), 128, 0, st>>>(g, a, b, bias, bias_stride, out, total);
      break;
    case B200_PHASE_DINPUT:
      total = (long long)g.n * g.cin * g.h * g.w;
      name = "direct_dinput_kernel";
      direct_dinput_kernel<<<(unsigned)div_up64(total, 128), 128, 0, st>>>(g, a, b, out, total);
      break;
    case B200_PHASE_DWEIGHT:
      total = (long long)g.cout * g.cig * g.kh * g.kw;
      name = "direct_dweight_kernel";
      direct_dweight_kernel<<<(unsigned)div_up64(total, 128), 128, 0, st>>>(g, a, b, out, total);
      break;
    default:
      name = "direct_dbias_kernel";
      direct_dbias_kernel<<<(unsigned)div_up64(g.cout, 128), 128, 0, st>>>(g, a, out);
      break;
  }
  count_launch();
  return launch_check(name);
}

// ---------------------------------------------------------------------------------------
// dBias: bandwidth-bound reduction of dY over batch and positions.
// Two layouts: positions contiguous (NCHW-like) -> one CTA per (channel, batch slab) with a
// warp-shuffle tree; channels contiguous (channels-last) -> 32 channels per CTA, threads along
// channels.  Slab partials are summed in ascending order by finalize_kernel.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  return v;
}

// Planes contiguous (NCHW): one CTA per (channel, slab of images); each warp takes whole image
// planes (8 in flight per CTA), lanes stream the plane with 16-byte loads where it is aligned.
__global__ void __launch_bounds__(256) dbias_rows_kernel(ConvGeom g, View4 go, float* out, int slabs) {
  const int oc = blockIdx.x, slab = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (g.n + slabs - 1) / slabs;
  const int b0 = slab * per, b1 = min(g.n, b0 + per);
  const int sp = g.oh * g.ow;
  const bool dense = go.s3 == 1 && go.s2 == g.ow;
  float sum = 0.f;
  for (long long b = b0 + warp; b < b1; b += 8) {
    const float* base = go.ptr + b * go.s0 + oc * go.s1;
    if (dense) {
      int i = 0;
      if ((reinterpret_cast<uintptr_t>(base) & 15) == 0) {
        const float4* v4 = reinterpret_cast<const float4*>(base);
        const int quads = sp / 4;
        int q = lane;
        for (; q + 96 < quads; q += 128) {  // four independent loads in flight per lane
          const float4 a0 = __ldg(v4 + q), a1 = __ldg(v4 + q + 32), a2 = __ldg(v4 + q + 64), a3 = __ldg(v4 + q + 96);
          sum += ((a0.x + a0.y) + (a0.z + a0.w)) + ((a1.x + a1.y) + (a1.z + a1.w)) + ((a2.x + a2.y) + (a2.z + a2.w)) +
                 ((a3.x + a3.y) + (a3.z + a3.w));
        }
        for (; q < quads; q += 32) {
          const float4 v = __ldg(v4 + q);
          sum += (v.x + v.y) + (v.z + v.w);
        }
        i = quads * 4;
      }
      for (int q = i + lane; q < sp; q += 32) sum += __ldg(base + q);
    } else {
      for (int q = lane; q < sp; q += 32) sum += __ldg(base + (q / g.ow) * go.s2 + (q % g.ow) * go.s3);
    }
  }
  __shared__ float warp_part[8];
  sum = warp_sum(sum);
  if (lane == 0) warp_part[warp] = sum;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < 8 ? warp_part[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) out[(long long)slab * g.cout + oc] = v;
  }
}

// Channels contiguous (channels-last): one CTA per (block of 32 channels, slab of pixels); eight lanes
// cover the 32 channels of a pixel with one 16-byte load each, so a warp reads four whole 128-byte
// pieces per instruction and the CTA 32 pixels.  `dense` = pixels at a constant stride (true
// channels-last); otherwise the pixel index is split into (image, row, column).
__global__ void __launch_bounds__(256) dbias_channels_kernel(ConvGeom g, View4 go, float* out, int slabs, int dense) {
  const int c4 = (threadIdx.x & 7) * 4, prow = threadIdx.x >> 3, slab = blockIdx.y;  // 32 pixel rows per CTA pass
  const int oc0 = blockIdx.x * 32 + c4;
  const long long P = (long long)g.n * g.oh * g.ow;
  const long long per = (P + slabs - 1) / slabs;
  const long long p0 = slab * per, p1 = min(P, p0 + per);
  const int sp = g.oh * g.ow;
  const bool vec = oc0 + 3 < g.cout && ((reinterpret_cast<uintptr_t>(go.ptr) & 15) == 0) && go.s0 % 4 == 0 && go.s2 % 4 == 0 &&
                   go.s3 % 4 == 0;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  long long q = p0 + prow;
  if (dense && vec) {  // four independent 16-byte loads in flight per thread
    const float* src = go.ptr + oc0;
    for (; q + 96 < p1; q += 128) {
      const float4 a0 = __ldg(reinterpret_cast<const float4*>(src + q * go.s3));
      const float4 a1 = __ldg(reinterpret_cast<const float4*>(src + (q + 32) * go.s3));
      const float4 a2 = __ldg(reinterpret_cast<const float4*>(src + (q + 64) * go.s3));
      const float4 a3 = __ldg(reinterpret_cast<const float4*>(src + (q + 96) * go.s3));
      sum.x += (a0.x + a1.x) + (a2.x + a3.x); sum.y += (a0.y + a1.y) + (a2.y + a3.y);
      sum.z += (a0.z + a1.z) + (a2.z + a3.z); sum.w += (a0.w + a1.w) + (a2.w + a3.w);
    }
  }
  for (; q < p1; q += 32) {
    long long off;
    if (dense) off = q * go.s3;
    else {
      const long long b = q / sp;
      const int pos = (int)(q - b * sp);
      off = b * go.s0 + (pos / g.ow) * go.s2 + (pos % g.ow) * go.s3;
    }
    const float* src = go.ptr + off + oc0;
    if (vec) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(src));
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    } else {
      if (oc0 < g.cout) sum.x += __ldg(src);
      if (oc0 + 1 < g.cout) sum.y += __ldg(src + 1);
      if (oc0 + 2 < g.cout) sum.z += __ldg(src + 2);
      if (oc0 + 3 < g.cout) sum.w += __ldg(src + 3);
    }
  }
  __shared__ float4 part[32][9];
  part[prow][threadIdx.x & 7] = sum;
  __syncthreads();
  if (threadIdx.x < 32) {  // thread t sums channel t of the block over the 32 pixel rows, in order
    float v = 0.f;
#pragma unroll 8
    for (int i = 0; i < 32; ++i) v += reinterpret_cast<const float*>(&part[i][threadIdx.x >> 2])[threadIdx.x & 3];
    const int oc = blockIdx.x * 32 + threadIdx.x;
    if (oc < g.cout) out[(long long)slab * g.cout + oc] = v;
  }
}

// y (contiguous NCHW) += residual (any strides), then ReLU: the pass behind candidates whose kernels
// have no fused epilogue.
__global__ void __launch_bounds__(256) post_ops_kernel(float* __restrict__ y, ConvGeom g, View4 res, int relu, long long total) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= total) return;
  float v = y[i];
  if (res.ptr) {
    const int x = (int)(i % g.ow), yy = (int)((i / g.ow) % g.oh);
    const int c = (int)((i / ((long long)g.ow * g.oh)) % g.cout);
    const long long n = i / ((long long)g.ow * g.oh * g.cout);
    v += res.ptr[n * res.s0 + c * res.s1 + yy * res.s2 + x * res.s3];
  }
  if (relu) v = fmaxf(v, 0.f);
  y[i] = v;
}
int post_ops_nchw(float* y, const ConvGeom& g, const StripPostOps& post, cudaStream_t st) {
  if (!post.residual.ptr && !post.relu) return B200_OK;
  const long long total = (long long)g.n * g.cout * g.oh * g.ow;
  post_ops_kernel<<<(unsigned)div_up64(total, 256), 256, 0, st>>>(y, g, post.residual, post.relu, total);
  count_launch();
  return launch_check("post_ops_kernel");
}

// y[n][c][plane] += bias[c] on a contiguous result: one CTA per (sample, channel) plane at a time,
// 16-byte accesses where the plane is aligned.  The bias pass of the transposed convolution.
__global__ void __launch_bounds__(256) bias_planes_kernel(float* __restrict__ y, const float* __restrict__ bias, long long bias_stride,
                                                          int channels, int plane, long long planes) {
  for (long long pl = blockIdx.x; pl < planes; pl += gridDim.x) {
    const float b = __ldg(bias + (pl % channels) * bias_stride);
    float* p = y + pl * plane;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
      float4* p4 = reinterpret_cast<float4*>(p);
      const int quads = plane >> 2;
      for (int i = threadIdx.x; i < quads; i += 256) {
        float4 v = p4[i];
        v.x += b, v.y += b, v.z += b, v.w += b;
        p4[i] = v;
      }
      done = quads * 4;
    }
    for (int e = done + threadIdx.x; e < plane; e += 256) p[e] += b;
  }
}
int bias_add_nchw(float* y, long long n, int channels, long long plane, const float* bias, long long bias_stride, cudaStream_t st) {
  const long long planes = n * channels;
  if (planes == 0 || plane == 0) return B200_OK;
  const long long grid = planes < 8ll * sm_count() ? planes : 8ll * sm_count();
  bias_planes_kernel<<<(unsigned)grid, 256, 0, st>>>(y, bias, bias_stride, channels, (int)plane, planes);
  count_launch();
  return launch_check("bias_planes_kernel");
}

int dbias_reduce(const ConvGeom& g, View4 dy, float* db, float* partial, int slabs, cudaStream_t st) {
  if (slabs < 1 || !partial) slabs = 1;
  float* out = slabs > 1 ? partial : db;
  const bool channels_inner = dy.s1 == 1 && dy.s3 != 1;
  if (channels_inner) {
    // true channels-last: consecutive pixels of the whole batch sit at one constant stride
    const int dense = dy.s2 == (long long)g.ow * dy.s3 && dy.s0 == (long long)g.oh * dy.s2;
    dbias_channels_kernel<<<dim3((unsigned)div_up64(g.cout, 32), (unsigned)slabs), 256, 0, st>>>(g, dy, out, slabs, dense);
  } else {
    if (slabs > g.n) slabs = g.n;
    out = slabs > 1 ? partial : db;
    dbias_rows_kernel<<<dim3((unsigned)g.cout, (unsigned)slabs), 256, 0, st>>>(g, dy, out, slabs);
  }
  count_launch();
  if (int rc = launch_check("dbias_kernel")) return rc;
  if (slabs > 1) return finalize_splits(partial, db, g.cout, slabs, st);
  return B200_OK;
}

}  // namespace b200
