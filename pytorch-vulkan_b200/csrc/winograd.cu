// Winograd F(4x4,3x3) forward and dInput for 3x3, stride-1, dilation-1 convolutions.
//
//   Y = A^T [ sum_ci (G g G^T) .* (B^T d B) ] A      per 4x4 output tile (6x6 input tile)
//
// 36 multiplications per 16 outputs instead of 144: the contraction over channels shrinks 4x, which
// is the only way an FP32 convolution evaluated with three TF32 MMAs per product can pass one third
// of the tensor-core peak.  Three stages per chunk of tiles, all on the device:
//   1. input_transform_kernel   d (strided view, zero padded) -> V[tile][36][Cin]
//   2. the 36 channel contractions as ONE grouped 1x1 convolution over a `tiles`-pixel image
//      (36*groups groups) on the persistent tcgen05 strip kernel (split-precision FP32), row-major output
//      M[tile][36][Cout]
//   3. output_transform_kernel  A^T m A + bias -> y (contiguous NCHW, ragged edge tiles guarded)
// plus filter_transform_kernel  g -> U[36][Cout][Cin/groups] once per call (weights may change
// between calls).  dInput is the same pipeline on dY with the filter rotated by 180 degrees and its
// channel roles swapped.  The chunk size follows the caller's workspace budget.
//
// Replaces the reference's F(2x2,3x3) path: csrc/ops/convolution.cpp:257-335 (eligibility, three
// dispatches) and csrc/shaders/conv2d_winograd_{weights,input,gemm_output}.comp.
#include <cuda_bf16.h>

#include "common.cuh"
#include "tc_common.cuh"

#include <algorithm>

namespace b200 {
namespace wino {

__device__ __forceinline__ void bt6(const float (&i)[6], float (&o)[6]) {  // rows of B^T
  o[0] = 4.f * i[0] - 5.f * i[2] + i[4];
  o[1] = -4.f * i[1] - 4.f * i[2] + i[3] + i[4];
  o[2] = 4.f * i[1] - 4.f * i[2] - i[3] + i[4];
  o[3] = -2.f * i[1] - i[2] + 2.f * i[3] + i[4];
  o[4] = 2.f * i[1] - i[2] - 2.f * i[3] + i[4];
  o[5] = 4.f * i[1] - 5.f * i[3] + i[5];
}
__device__ __forceinline__ void g6(const float (&i)[3], float (&o)[6]) {  // rows of G
  o[0] = i[0] * 0.25f;
  o[1] = -(i[0] + i[1] + i[2]) * (1.f / 6.f);
  o[2] = -(i[0] - i[1] + i[2]) * (1.f / 6.f);
  o[3] = i[0] * (1.f / 24.f) + i[1] * (1.f / 12.f) + i[2] * (1.f / 6.f);
  o[4] = i[0] * (1.f / 24.f) - i[1] * (1.f / 12.f) + i[2] * (1.f / 6.f);
  o[5] = i[2];
}
__device__ __forceinline__ void at4(const float (&i)[6], float (&o)[4]) {  // rows of A^T
  o[0] = i[0] + i[1] + i[2] + i[3] + i[4];
  o[1] = i[1] - i[2] + 2.f * i[3] - 2.f * i[4];
  o[2] = i[1] + i[2] + 4.f * i[3] + 4.f * i[4];
  o[3] = i[1] - i[2] + 8.f * i[3] - 8.f * i[4] + i[5];
}

struct Tiling {
  int n, h, w;      // input map (for dInput: the dY map)
  int oh, ow;       // output map
  int ph, pw;       // offset of the first input row/column of tile (0,0) is (-ph, -pw)
  int th, tw;       // tiles per image
  long long tiles;  // n*th*tw
};

// U[p][co][ci] = (G g G^T)[p].  transposed: g'(ci -> row, co -> column) = g rotated by 180 degrees.
// U is written directly as the strip kernel's weight stage images for the grouped 1x1 product
// (group = p*groups + grp; TF32 hi and lo planes of bn rows x 32 channels, SWIZZLE_128B); rows that
// pad the last column tile are zeroed by the caller.
__global__ void __launch_bounds__(256) filter_transform_kernel(ConvGeom g, View4 w, int transposed, float* __restrict__ U,
                                                               long long pairs, int bn, int tiles_n) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= pairs) return;
  const int kc = transposed ? g.cog : g.cig, nc = transposed ? g.cig : g.cog;
  const int k = (int)(i % kc);
  const long long rg = i / kc;          // row over all groups: grp*nc + r
  const int r = (int)(rg % nc), grp = (int)(rg / nc);
  const int co = transposed ? k : r, ci = transposed ? r : k;
  const float* src = w.ptr + ((long long)grp * g.cog + co) * w.s0 + (long long)ci * w.s1;
  float gg[3][3];
#pragma unroll
  for (int y = 0; y < 3; ++y)
#pragma unroll
    for (int x = 0; x < 3; ++x) {
      const int sy = transposed ? 2 - y : y, sx = transposed ? 2 - x : x;
      gg[y][x] = src[sy * w.s2 + sx * w.s3];
    }
  float t[6][3];  // G g
#pragma unroll
  for (int x = 0; x < 3; ++x) {
    const float col[3] = {gg[0][x], gg[1][x], gg[2][x]};
    float o[6];
    g6(col, o);
#pragma unroll
    for (int y = 0; y < 6; ++y) t[y][x] = o[y];
  }
  const int cblocks = kc / 32;
  const long long within_image = ((long long)(r / bn) * cblocks + k / 32) * (bn * 64ll);  // start of the stage image
  const long long per_group = (long long)tiles_n * cblocks * (bn * 64ll);
#pragma unroll
  for (int y = 0; y < 6; ++y) {
    float o[6];
    g6(t[y], o);
#pragma unroll
    for (int x = 0; x < 6; ++x) {
      float hi, lo;
      tc::split_tf32(o[x], hi, lo);
      float* plane = U + ((long long)(y * 6 + x) * g.groups + grp) * per_group + within_image;
      plane[tc::sw128_offset(r % bn, k % 32) / 4] = hi;
      if (tc::CROSS_BF16) {
        __nv_bfloat16* cross = reinterpret_cast<__nv_bfloat16*>(plane + bn * 32);
        cross[tc::sw128_offset_bf16(r % bn, k % 32) / 2] = __float2bfloat16_rn(lo);
        cross[tc::sw128_offset_bf16(r % bn, 32 + k % 32) / 2] = __float2bfloat16_rn(hi);
      } else {
        plane[bn * 32 + tc::sw128_offset(r % bn, k % 32) / 4] = lo;
      }
    }
  }
}

// V[(t - t0)][p][c] = (B^T d B)[p] for tile t, channel c.  Block = 32 tiles (lane) x 8 channels
// (warp): loads are coalesced along the tile row for NCHW and sector-complete across the 8 warps
// for channels-last; results are staged in shared memory and written as 32-byte channel runs.
__global__ void __launch_bounds__(256) input_transform_kernel(Tiling tl, View4 x, int ctot, float* __restrict__ V,
                                                              long long t0, long long t1) {
  __shared__ float s[36][32][8 + 1];
  const int lane = threadIdx.x & 31, wq = threadIdx.x >> 5;
  const long long t = t0 + (long long)blockIdx.x * 32 + lane;
  const int c = blockIdx.y * 8 + wq;
  float d[6][6];
#pragma unroll
  for (int y = 0; y < 6; ++y)
#pragma unroll
    for (int xx = 0; xx < 6; ++xx) d[y][xx] = 0.f;
  if (t < t1 && c < ctot) {
    const int per = tl.th * tl.tw;
    const long long n = t / per;
    const int rem = (int)(t - n * per);
    const int ty = rem / tl.tw, tx = rem - ty * tl.tw;
    const int y0 = ty * 4 - tl.ph, x0 = tx * 4 - tl.pw;
    const float* src = x.ptr + n * x.s0 + (long long)c * x.s1;
#pragma unroll
    for (int y = 0; y < 6; ++y) {
      const int iy = y0 + y;
      if (iy < 0 || iy >= tl.h) continue;
#pragma unroll
      for (int xx = 0; xx < 6; ++xx) {
        const int ix = x0 + xx;
        if (ix >= 0 && ix < tl.w) d[y][xx] = __ldg(src + (long long)iy * x.s2 + (long long)ix * x.s3);
      }
    }
  }
  float tmp[6][6];  // B^T d
#pragma unroll
  for (int xx = 0; xx < 6; ++xx) {
    const float col[6] = {d[0][xx], d[1][xx], d[2][xx], d[3][xx], d[4][xx], d[5][xx]};
    float o[6];
    bt6(col, o);
#pragma unroll
    for (int y = 0; y < 6; ++y) tmp[y][xx] = o[y];
  }
#pragma unroll
  for (int y = 0; y < 6; ++y) {
    float o[6];
    bt6(tmp[y], o);
#pragma unroll
    for (int xx = 0; xx < 6; ++xx) s[y * 6 + xx][lane][wq] = o[xx];
  }
  __syncthreads();
  // 36 planes x 32 tiles x 2 float4 per block
  for (int i = threadIdx.x; i < 36 * 32 * 2; i += 256) {
    const int p = i >> 6, tt = (i >> 1) & 31, half = i & 1;
    const long long tg = t0 + (long long)blockIdx.x * 32 + tt;
    const int c0 = blockIdx.y * 8 + half * 4;
    if (tg < t1 && c0 < ctot) {
      const float4 v = make_float4(s[p][tt][half * 4], s[p][tt][half * 4 + 1], s[p][tt][half * 4 + 2], s[p][tt][half * 4 + 3]);
      *reinterpret_cast<float4*>(V + ((tg - t0) * 36 + p) * (long long)ctot + c0) = v;
    }
  }
}

// y[n][co][4x4 tile] = A^T m A + bias from M[(t - t0)][p][co].  Block = 32 channels (lane) x 8
// consecutive tiles (warp); the 4x4 results are staged in shared memory so that a warp writes runs
// of up to 32 consecutive pixels of one output row.
__global__ void __launch_bounds__(256) output_transform_kernel(Tiling tl, const float* __restrict__ M, int cout,
                                                               const float* __restrict__ bias, long long bias_stride,
                                                               float* __restrict__ y, long long t0, long long t1) {
  __shared__ float s[32][4][32 + 1];
  const int lane = threadIdx.x & 31, wq = threadIdx.x >> 5;
  const long long tbase = t0 + (long long)blockIdx.x * 8;
  const long long t = tbase + wq;
  const int co = blockIdx.y * 32 + lane;
  float o4[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) o4[a][b] = 0.f;
  if (t < t1 && co < cout) {
    float m[6][6];
    const float* src = M + (t - t0) * 36 * (long long)cout + co;
#pragma unroll
    for (int p = 0; p < 36; ++p) m[p / 6][p % 6] = __ldg(src + (long long)p * cout);
    float tmp[4][6];  // A^T m
#pragma unroll
    for (int xx = 0; xx < 6; ++xx) {
      const float col[6] = {m[0][xx], m[1][xx], m[2][xx], m[3][xx], m[4][xx], m[5][xx]};
      float o[4];
      at4(col, o);
#pragma unroll
      for (int a = 0; a < 4; ++a) tmp[a][xx] = o[a];
    }
    const float bv = bias ? __ldg(bias + (long long)co * bias_stride) : 0.f;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      float o[4];
      at4(tmp[a], o);
#pragma unroll
      for (int b = 0; b < 4; ++b) o4[a][b] = o[b] + bv;
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) s[lane][a][wq * 4 + b] = o4[a][b];
  __syncthreads();
  // (channel, row) pairs: 32*4 = 128 runs of 32 pixel slots; warp wq takes runs wq, wq+8, ...
  const int per = tl.th * tl.tw;
  const long long tl_t = tbase + (lane >> 2);   // tile of this lane's pixel slot
  const int bx = lane & 3;
  bool ok = tl_t < t1;
  long long n = 0;
  int ty = 0, tx = 0;
  if (ok) {
    n = tl_t / per;
    const int rem = (int)(tl_t - n * per);
    ty = rem / tl.tw;
    tx = rem - ty * tl.tw;
  }
  const int ox = tx * 4 + bx;
  for (int run = wq; run < 128; run += 8) {
    const int cc = run >> 2, a = run & 3;
    const int c = blockIdx.y * 32 + cc;
    const int oy = ty * 4 + a;
    if (ok && c < cout && oy < tl.oh && ox < tl.ow)
      y[((n * cout + c) * tl.oh + oy) * (long long)tl.ow + ox] = s[cc][a][lane];
  }
}

struct Plan {
  bool ok = false;
  int kc = 0, nc = 0;          // contraction / output channels per group
  long long tiles = 0;
  size_t u_bytes = 0, per_tile = 0;
};

static Plan make_plan(const ConvGeom& g, bool is_dx) {
  Plan p;
  if (g.kh != 3 || g.kw != 3 || g.sh != 1 || g.sw != 1 || g.dh != 1 || g.dw != 1) return p;
  if (is_dx && (g.ph > 2 || g.pw > 2)) return p;
  p.kc = is_dx ? g.cog : g.cig;
  p.nc = is_dx ? g.cig : g.cog;
  if (p.kc % 32 != 0 || p.nc < 16 || p.nc % 4 != 0) return p;
  const int oh = is_dx ? g.h : g.oh, ow = is_dx ? g.w : g.ow;
  p.tiles = (long long)g.n * ((oh + 3) / 4) * ((ow + 3) / 4);
  // the transformed filter is kept as the strip kernel's weight stage images
  ConvGeom gg{};
  gg.groups = 36 * g.groups; gg.cig = p.kc; gg.cog = p.nc; gg.kh = gg.kw = 1;
  p.u_bytes = (strip_workspace(gg, B200_PHASE_FORWARD) + 255) / 256 * 256;
  p.per_tile = sizeof(float) * 36ull * ((size_t)p.kc + p.nc) * g.groups;
  if (36ll * g.groups > 65535) return p;
  p.ok = true;
  return p;
}

}  // namespace wino

bool winograd_supported(const ConvGeom& g, int phase) {
  if (phase != B200_PHASE_FORWARD && phase != B200_PHASE_DINPUT) return false;
  return wino::make_plan(g, phase == B200_PHASE_DINPUT).ok;
}

// Workspace wanted (all tiles in one chunk) capped by the budget; 0 if even 128 tiles do not fit.
size_t winograd_workspace(const ConvGeom& g, int phase, size_t budget) {
  const wino::Plan p = wino::make_plan(g, phase == B200_PHASE_DINPUT);
  if (!p.ok) return 0;
  const size_t full = p.u_bytes + (size_t)p.tiles * p.per_tile + 256;
  const size_t least = p.u_bytes + (size_t)std::min<long long>(128, p.tiles) * p.per_tile + 256;
  if (budget < least) return 0;
  return std::min(full, budget);
}

int winograd_conv(const ConvGeom& g, bool is_dx, View4 act, View4 w, const float* bias, long long bias_stride,
                  float* out, void* ws, size_t ws_bytes, cudaStream_t st) {
  using namespace wino;
  const Plan p = make_plan(g, is_dx);
  if (!p.ok) return fail(B200_EUNSUPPORTED, "forced Winograd candidate is incompatible with this geometry");
  const size_t least = p.u_bytes + (size_t)std::min<long long>(128, p.tiles) * p.per_tile + 256;
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 15) || ws_bytes < least)
    return fail(B200_EWORKSPACE, "Winograd convolution exceeds the workspace budget: needs at least %zu bytes (got %zu)",
                least, ws_bytes);
  Tiling tl;
  tl.n = g.n;
  tl.h = is_dx ? g.oh : g.h;  tl.w = is_dx ? g.ow : g.w;
  tl.oh = is_dx ? g.h : g.oh; tl.ow = is_dx ? g.w : g.ow;
  tl.ph = is_dx ? 2 - g.ph : g.ph;
  tl.pw = is_dx ? 2 - g.pw : g.pw;
  tl.th = (tl.oh + 3) / 4; tl.tw = (tl.ow + 3) / 4;
  tl.tiles = p.tiles;
  const int ctot_in = p.kc * g.groups, ctot_out = p.nc * g.groups;
  float* U = (float*)ws;
  const size_t u_floats = p.u_bytes / sizeof(float);
  long long chunk = (long long)((ws_bytes - p.u_bytes) / p.per_tile);
  chunk = std::min(chunk, p.tiles);
  if (chunk < p.tiles) chunk = chunk / 128 * 128;
  if (chunk <= 0) return fail(B200_EWORKSPACE, "Winograd convolution exceeds the workspace budget");
  float* V = U + u_floats;
  float* M = V + (size_t)chunk * 36 * ctot_in;

  const long long pairs = (long long)g.cout * g.cig;
  int staged_bn = 0;  // column tile the images in U were written for

  // the 36 plane products as one grouped 1x1 convolution: group index = plane * groups + group
  ConvGeom gg{};
  gg.n = 1; gg.h = 1; gg.kh = gg.kw = 1; gg.oh = 1; gg.sh = gg.sw = 1; gg.dh = gg.dw = 1; gg.ph = gg.pw = 0;
  gg.groups = 36 * g.groups; gg.cig = p.kc; gg.cog = p.nc;
  gg.cin = gg.groups * p.kc; gg.cout = gg.groups * p.nc;
  for (long long t0 = 0; t0 < p.tiles; t0 += chunk) {
    const long long t1 = std::min(p.tiles, t0 + chunk), cnt = t1 - t0;
    input_transform_kernel<<<dim3((unsigned)div_up64(cnt, 32), (unsigned)div_up64(ctot_in, 8)), 256, 0, st>>>(
        tl, act, ctot_in, V, t0, t1);
    count_launch();
    if (int rc = launch_check("input_transform_kernel")) return rc;
    gg.w = (int)cnt; gg.ow = (int)cnt;
    const int bn = strip_column_tile(gg, false);  // depends on the number of tiles in the chunk
    if (bn <= 0) return fail(B200_EUNSUPPORTED, "Winograd plane product does not fit the strip kernel");
    if (bn != staged_bn) {
      const int tiles_n = (p.nc + bn - 1) / bn;
      if (p.nc % bn != 0) B200_CUDA(cudaMemsetAsync(U, 0, p.u_bytes, st));
      filter_transform_kernel<<<(unsigned)div_up64(pairs, 256), 256, 0, st>>>(g, w, is_dx ? 1 : 0, U, pairs, bn, tiles_n);
      count_launch();
      if (int rc = launch_check("filter_transform_kernel")) return rc;
      staged_bn = bn;
    }
    const View4 vact{V, 0, 1, 0, 36ll * ctot_in};
    if (int rc = strip_conv(gg, false, vact, View4{}, nullptr, 0, M, nullptr, 0, st, true, 1.f, 0.f, U)) return rc;
    output_transform_kernel<<<dim3((unsigned)div_up64(cnt, 8), (unsigned)div_up64(ctot_out, 32)), 256, 0, st>>>(
        tl, M, ctot_out, bias, bias_stride, out, t0, t1);
    count_launch();
    if (int rc = launch_check("output_transform_kernel")) return rc;
  }
  return B200_OK;
}

}  // namespace b200
