// CUDA-core kernels for grouped 3x3 convolutions with FEW channels per group (4 or 8 in and out), stride 1,
// dilation 1, padding 1: forward, dInput and dWeight.
//
// These are the groups=32 layers of a U-Net block at 128 / 256 channels.  With 4 or 8 channels per group the
// contraction per output is 36 or 72 long: the layers move 8 bytes per 9 to 18 FLOP, so their roofline is HBM, and
// an implicit-GEMM tile of 64 rows per group (conv_simt.cu) would spend nine tenths of its multiply-adds on padding.
// Here the tile follows the group instead: a thread block owns (image, group, 16 rows x 64 columns), brings the
// group's input tile (with its one-pixel halo) into shared memory once, and every thread keeps a 1 x 4 pixel strip
// of ALL the group's output channels in registers, so an input value is loaded once for up to 3 x 8 multiply-adds.
//   forward / dInput   one kernel; dInput runs it on dy with the filter rotated by 180 degrees and its channel roles
//                      exchanged (prepared in shared memory while the tile loads)
//   dWeight            each thread accumulates the (ci, 3, 3) block of one output channel over its pixel strips in registers; a block
//                      reduces them with warp shuffles and writes one partial per block; a second kernel sums the
//                      partials in ascending order (no atomics: results are identical from run to run)
// Inputs are read through their strides (NCHW: a warp reads consecutive pixels of a channel; channels-last: the
// channels of a pixel first); results are contiguous NCHW.
//
// Replaces csrc/shaders/conv2d_depthwise.comp:1-41 and the small-channel side of the heuristic
// (csrc/ops/convolution.cpp:459-463) of the reference for these geometries.
#include "common.cuh"

#include <algorithm>

namespace b200 {
namespace gcs {

constexpr int TH = 16;                   // rows of a dWeight tile (forward / dInput tiles come from the SX template parameter)
constexpr int IH = TH + 2;               // its input rows with halo
constexpr int THREADS = 256;

struct GArgs {
  View4 in;            // forward: x.  dInput: dy.  Logical [n][c][h][w]
  View4 w;             // [cout][cin/g][3][3]
  const float* bias;   // forward only
  long long bias_stride;
  float* out;          // contiguous [n][c][h][w]
  int n, c, h, w_, groups;
  int tiles_y, tiles_x;
  int transposed;      // dInput: use w[ci][co][2-ky][2-kx]
};

// y[n, g*CPG + co, y, x] = bias + sum_{ci, ky, kx} in[n, g*CPG + ci, y + ky - 1, x + kx - 1] * W[co][ci][ky][kx]
// SX strips of 4 pixels per tile row: the tile is (256 / SX) rows x (4 * SX) columns (16 x 64 for wide images,
// 32 x 32 for maps up to 32 columns, so that no thread idles on padding).
template <int CPG, int SX>
__global__ void __launch_bounds__(THREADS) gconv_fwd_kernel(const GArgs a) {
  constexpr int TWK = 4 * SX, THK = THREADS / SX;         // tile extent
  constexpr int IWK = TWK + 4, IHK = THK + 2;              // with halo; rows padded to a multiple of 4 floats
  __shared__ __align__(16) float s_in[CPG][IHK][IWK];
  __shared__ __align__(16) float s_w[CPG][3][3][CPG];   // [ci][ky][kx][co]: the co of one tap are one vector
  const int tid = threadIdx.x;
  int b = blockIdx.x;
  const int tx_tile = b % a.tiles_x; b /= a.tiles_x;
  const int ty_tile = b % a.tiles_y; b /= a.tiles_y;
  const int g = b % a.groups;
  const int n = b / a.groups;
  const int y0 = ty_tile * THK, x0 = tx_tile * TWK;
  const long long chan0 = (long long)g * CPG;

  // filter of the group
  for (int i = tid; i < CPG * CPG * 9; i += THREADS) {
    const int co = i % CPG, kx = (i / CPG) % 3, ky = (i / (CPG * 3)) % 3, ci = i / (CPG * 9);
    // forward: W[g*CPG + co][ci][ky][kx].  dInput: the output channel of this pass is the filter's input channel:
    // W[g*CPG + ci][co][2 - ky][2 - kx]
    const float v = a.transposed ? a.w.ptr[(chan0 + ci) * a.w.s0 + co * a.w.s1 + (2 - ky) * a.w.s2 + (2 - kx) * a.w.s3]
                                 : a.w.ptr[(chan0 + co) * a.w.s0 + ci * a.w.s1 + ky * a.w.s2 + kx * a.w.s3];
    s_w[ci][ky][kx][co] = v;
  }
  // input tile with halo (tile column c is image column x0 - 1 + c); out-of-image pixels are zero
  const float* src = a.in.ptr + n * a.in.s0 + chan0 * a.in.s1;
  const bool rows_vec = a.in.s3 == 1 && a.in.s2 % 4 == 0 && a.in.s1 % 4 == 0 && a.in.s0 % 4 == 0 &&
                        ((reinterpret_cast<uintptr_t>(a.in.ptr) & 15) == 0) && x0 + TWK <= a.w_;
  if (rows_vec) {
    // planes with contiguous rows: the interior of a tile row as 16-byte loads (all of a thread's loads are issued
    // before the first is used), the two halo columns as scalars
    constexpr int VEC = CPG * IHK * SX;                     // float4 pieces of the interior
#pragma unroll
    for (int i0 = 0; i0 < VEC; i0 += THREADS) {
      const int i = i0 + tid;
      if (VEC % THREADS == 0 || i < VEC) {
        const int c4 = i % SX, r = (i / SX) % IHK, ci = i / (SX * IHK);
        const int y = y0 - 1 + r;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (y >= 0 && y < a.h) v = __ldg(reinterpret_cast<const float4*>(src + ci * a.in.s1 + (long long)y * a.in.s2 + x0) + c4);
        float* d = &s_in[ci][r][1 + 4 * c4];
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
      }
    }
    for (int i = tid; i < CPG * IHK * 2; i += THREADS) {
      const int side = i & 1, r = (i >> 1) % IHK, ci = i / (2 * IHK);
      const int y = y0 - 1 + r, x = side ? x0 + TWK : x0 - 1;
      s_in[ci][r][side ? TWK + 1 : 0] = (y >= 0 && y < a.h && x >= 0 && x < a.w_) ? __ldg(src + ci * a.in.s1 + (long long)y * a.in.s2 + x) : 0.f;
    }
  } else if (a.in.s1 == 1) {   // channels-last: the channels of a pixel are adjacent
#pragma unroll 4
    for (int i = tid; i < CPG * IHK * (TWK + 2); i += THREADS) {
      const int ci = i % CPG, c = (i / CPG) % (TWK + 2), r = i / (CPG * (TWK + 2));
      const int y = y0 - 1 + r, x = x0 - 1 + c;
      s_in[ci][r][c] = (y >= 0 && y < a.h && x >= 0 && x < a.w_) ? __ldg(src + ci + (long long)y * a.in.s2 + (long long)x * a.in.s3) : 0.f;
    }
  } else {
#pragma unroll 4
    for (int i = tid; i < CPG * IHK * (TWK + 2); i += THREADS) {
      const int c = i % (TWK + 2), r = (i / (TWK + 2)) % IHK, ci = i / ((TWK + 2) * IHK);
      const int y = y0 - 1 + r, x = x0 - 1 + c;
      s_in[ci][r][c] = (y >= 0 && y < a.h && x >= 0 && x < a.w_) ? __ldg(src + ci * a.in.s1 + (long long)y * a.in.s2 + (long long)x * a.in.s3) : 0.f;
    }
  }
  __syncthreads();

  const int tx = tid % SX, ty = tid / SX;   // strip of 4 pixels: row ty, columns 4*tx .. 4*tx+3
  float acc[CPG][4];
#pragma unroll
  for (int co = 0; co < CPG; ++co)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[co][j] = 0.f;
#pragma unroll
  for (int ci = 0; ci < CPG; ++ci) {
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) {
      const float4 p0 = *reinterpret_cast<const float4*>(&s_in[ci][ty + ky][4 * tx]);
      const float2 p1 = *reinterpret_cast<const float2*>(&s_in[ci][ty + ky][4 * tx + 4]);
      const float v[6] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y};
#pragma unroll
      for (int kx = 0; kx < 3; ++kx) {
        float wv[CPG];
#pragma unroll
        for (int q = 0; q < CPG / 4; ++q) {
          const float4 t = *reinterpret_cast<const float4*>(&s_w[ci][ky][kx][4 * q]);
          wv[4 * q] = t.x; wv[4 * q + 1] = t.y; wv[4 * q + 2] = t.z; wv[4 * q + 3] = t.w;
        }
#pragma unroll
        for (int co = 0; co < CPG; ++co)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[co][j] = fmaf(v[j + kx], wv[co], acc[co][j]);
      }
    }
  }
  const int y = y0 + ty, x = x0 + 4 * tx;
  if (y >= a.h || x >= a.w_) return;
  const long long plane = (long long)a.h * a.w_;
  float* out = a.out + (n * (long long)a.c + chan0) * plane + (long long)y * a.w_ + x;
  const bool vec = x + 3 < a.w_ && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && (plane % 4 == 0);
#pragma unroll
  for (int co = 0; co < CPG; ++co) {
    const float bv = a.bias ? __ldg(a.bias + (chan0 + co) * a.bias_stride) : 0.f;
    float* p = out + co * plane;
    if (vec) {
      *reinterpret_cast<float4*>(p) = make_float4(acc[co][0] + bv, acc[co][1] + bv, acc[co][2] + bv, acc[co][3] + bv);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (x + j < a.w_) p[j] = acc[co][j] + bv;
    }
  }
}

// ---- dWeight -------------------------------------------------------------------------------------------------------
// dW[g*CPG + co][ci][ky][kx] = sum_{n, y, x} dy[n, g*CPG + co, y, x] * x[n, g*CPG + ci, y + ky - 1, x + kx - 1]
// A thread owns a strip of 4 pixels and COT output channels of the group and keeps the COT x CPG x 9 sums of its
// strips in registers over `tiles_per_block` tiles; the CPG / COT threads of a strip split the output channels.
struct GdwArgs {
  View4 x, dy;
  float* partial;      // [blocks per group][cout][CPG][9]
  int n, c, h, w_, groups;
  int tiles_y, tiles_x, tiles_per_block, blocks_per_group;
};

template <int CPG, int COT>
__global__ void __launch_bounds__(THREADS) gconv_dw_kernel(const GdwArgs a) {
  constexpr int NQ = CPG / COT;                 // threads per strip
  constexpr int STRIPS = THREADS / NQ;          // strips per tile
  constexpr int SW = STRIPS / TH;               // strips per tile row
  constexpr int DW_TW = SW * 4;                 // tile width in pixels
  constexpr int XW = DW_TW + 4;                 // input row with halo, padded to a multiple of 4
  __shared__ __align__(16) float s_x[CPG][IH][XW];
  __shared__ __align__(16) float s_dy[CPG][TH][DW_TW];
  const int tid = threadIdx.x;
  const int g = blockIdx.x / a.blocks_per_group, pb = blockIdx.x % a.blocks_per_group;
  const long long chan0 = (long long)g * CPG;
  const int q = tid / STRIPS, strip = tid % STRIPS;     // a warp holds one q (STRIPS >= 32)
  const int ty = strip / SW, sx = strip % SW;
  float acc[COT][CPG][9];
#pragma unroll
  for (int co = 0; co < COT; ++co)
#pragma unroll
    for (int ci = 0; ci < CPG; ++ci)
#pragma unroll
      for (int k = 0; k < 9; ++k) acc[co][ci][k] = 0.f;
  const int tiles_img = a.tiles_y * a.tiles_x, tiles_all = a.n * tiles_img;
  for (int it = 0; it < a.tiles_per_block; ++it) {
    const int t = pb * a.tiles_per_block + it;
    if (t >= tiles_all) break;
    const int n = t / tiles_img, rem = t % tiles_img;
    const int y0 = (rem / a.tiles_x) * TH, x0 = (rem % a.tiles_x) * DW_TW;
    __syncthreads();   // the previous tile has been consumed
    const float* px = a.x.ptr + n * a.x.s0 + chan0 * a.x.s1;
    const float* pd = a.dy.ptr + n * a.dy.s0 + chan0 * a.dy.s1;
    if (a.x.s1 == 1) {
#pragma unroll
      for (int i = tid; i < CPG * IH * (DW_TW + 2); i += THREADS) {
        const int ci = i % CPG, c = (i / CPG) % (DW_TW + 2), r = i / (CPG * (DW_TW + 2));
        const int y = y0 - 1 + r, x = x0 - 1 + c;
        s_x[ci][r][c] = (y >= 0 && y < a.h && x >= 0 && x < a.w_) ? __ldg(px + ci + (long long)y * a.x.s2 + (long long)x * a.x.s3) : 0.f;
      }
    } else {
#pragma unroll
      for (int i = tid; i < CPG * IH * (DW_TW + 2); i += THREADS) {
        const int c = i % (DW_TW + 2), r = (i / (DW_TW + 2)) % IH, ci = i / ((DW_TW + 2) * IH);
        const int y = y0 - 1 + r, x = x0 - 1 + c;
        s_x[ci][r][c] = (y >= 0 && y < a.h && x >= 0 && x < a.w_) ? __ldg(px + ci * a.x.s1 + (long long)y * a.x.s2 + (long long)x * a.x.s3) : 0.f;
      }
    }
    if (a.dy.s1 == 1) {
#pragma unroll
      for (int i = tid; i < CPG * TH * DW_TW; i += THREADS) {
        const int co = i % CPG, c = (i / CPG) % DW_TW, r = i / (CPG * DW_TW);
        const int y = y0 + r, x = x0 + c;
        s_dy[co][r][c] = (y < a.h && x < a.w_) ? __ldg(pd + co + (long long)y * a.dy.s2 + (long long)x * a.dy.s3) : 0.f;
      }
    } else {
#pragma unroll
      for (int i = tid; i < CPG * TH * DW_TW; i += THREADS) {
        const int c = i % DW_TW, r = (i / DW_TW) % TH, co = i / (DW_TW * TH);
        const int y = y0 + r, x = x0 + c;
        s_dy[co][r][c] = (y < a.h && x < a.w_) ? __ldg(pd + co * a.dy.s1 + (long long)y * a.dy.s2 + (long long)x * a.dy.s3) : 0.f;
      }
    }
    __syncthreads();
    float d[COT][4];
#pragma unroll
    for (int co = 0; co < COT; ++co) {
      const float4 t4 = *reinterpret_cast<const float4*>(&s_dy[q * COT + co][ty][4 * sx]);
      d[co][0] = t4.x; d[co][1] = t4.y; d[co][2] = t4.z; d[co][3] = t4.w;
    }
#pragma unroll
    for (int ci = 0; ci < CPG; ++ci) {
#pragma unroll
      for (int ky = 0; ky < 3; ++ky) {
        const float4 p0 = *reinterpret_cast<const float4*>(&s_x[ci][ty + ky][4 * sx]);
        const float2 p1 = *reinterpret_cast<const float2*>(&s_x[ci][ty + ky][4 * sx + 4]);
        const float v[6] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y};
#pragma unroll
        for (int kx = 0; kx < 3; ++kx)
#pragma unroll
          for (int co = 0; co < COT; ++co)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[co][ci][ky * 3 + kx] = fmaf(d[co][j], v[j + kx], acc[co][ci][ky * 3 + kx]);
      }
    }
  }
  // block reduction: shuffles inside a warp (one q per warp), then across the warps of a q in shared memory, in a
  // fixed order, so that the partial of a block is the same from run to run
  __shared__ float s_red[THREADS / 32][COT * CPG * 9];
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int co = 0; co < COT; ++co)
#pragma unroll
    for (int ci = 0; ci < CPG; ++ci)
#pragma unroll
      for (int k = 0; k < 9; ++k) {
        float v = acc[co][ci][k];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) s_red[warp][(co * CPG + ci) * 9 + k] = v;
      }
  __syncthreads();
  constexpr int WPQ = STRIPS / 32;   // warps per q
  for (int i = tid; i < CPG * CPG * 9; i += THREADS) {
    const int co = i / (CPG * 9), rest = i % (CPG * 9);
    const int qq = co / COT, col = (co % COT) * CPG * 9 + rest;
    float sum = 0.f;
    for (int wq = 0; wq < WPQ; ++wq) sum += s_red[qq * WPQ + wq][col];
    a.partial[((long long)pb * a.c + chan0 + co) * (CPG * 9) + rest] = sum;
  }
}

}  // namespace gcs

// 3x3, stride 1, dilation 1, padding 1, the same small channel count (4 or 8) in and out of every group
bool group_small_supported(const ConvGeom& g) {
  return g.kh == 3 && g.kw == 3 && g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1 && g.ph == 1 && g.pw == 1 && g.cig == g.cog &&
         (g.cig == 4 || g.cig == 8) && g.groups >= 2 && g.oh == g.h && g.ow == g.w;
}

static void dw_tiling(const ConvGeom& g, int* tiles_y, int* tiles_x, int* tiles_per_block, int* blocks_per_group) {
  const int tw = g.cig == 4 ? 16 : 8;   // one output channel per thread: 4 (8) threads share a strip, 64 (32) strips per tile
  *tiles_y = (g.h + gcs::TH - 1) / gcs::TH;
  *tiles_x = (g.w + tw - 1) / tw;
  const long long tiles_all = (long long)g.n * *tiles_y * *tiles_x;
  // enough blocks for about six per SM, at least sixteen tiles per block (the block reduction costs about as much as two tiles)
  long long bpg = std::max<long long>(1, std::min<long long>(tiles_all / 16, div_up64(6ll * sm_count(), g.groups)));
  *tiles_per_block = (int)div_up64(tiles_all, bpg);
  *blocks_per_group = (int)div_up64(tiles_all, *tiles_per_block);
}

size_t group_small_dweight_workspace(const ConvGeom& g) {
  int ty, tx, tpb, bpg;
  dw_tiling(g, &ty, &tx, &tpb, &bpg);
  return (size_t)bpg * g.cout * g.cig * 9 * sizeof(float);
}

int group_small_conv(const ConvGeom& g, bool is_dx, View4 in, View4 w, const float* bias, long long bias_stride, float* out, cudaStream_t st) {
  gcs::GArgs a{};
  a.in = in; a.w = w; a.bias = is_dx ? nullptr : bias; a.bias_stride = bias_stride; a.out = out;
  a.n = g.n; a.c = g.cin; a.h = g.h; a.w_ = g.w; a.groups = g.groups;
  const bool narrow = g.w <= 32;   // 32 x 32 tiles for small maps, 16 x 64 otherwise
  const int th = narrow ? 32 : 16, tw = narrow ? 32 : 64;
  a.tiles_y = (g.h + th - 1) / th; a.tiles_x = (g.w + tw - 1) / tw;
  a.transposed = is_dx ? 1 : 0;
  const long long blocks = (long long)g.n * g.groups * a.tiles_y * a.tiles_x;
  if (blocks > 2147483647ll) return fail(B200_ERANGE, "grouped convolution: grid exceeds launch limits");
  const unsigned nb = (unsigned)blocks;
  if (g.cig == 4) {
    if (narrow) gcs::gconv_fwd_kernel<4, 8><<<nb, gcs::THREADS, 0, st>>>(a);
    else gcs::gconv_fwd_kernel<4, 16><<<nb, gcs::THREADS, 0, st>>>(a);
  } else {
    if (narrow) gcs::gconv_fwd_kernel<8, 8><<<nb, gcs::THREADS, 0, st>>>(a);
    else gcs::gconv_fwd_kernel<8, 16><<<nb, gcs::THREADS, 0, st>>>(a);
  }
  count_launch();
  return launch_check("gconv_fwd_kernel");
}

int group_small_dweight(const ConvGeom& g, View4 x, View4 dy, float* dw, float* ws, size_t ws_bytes, cudaStream_t st) {
  gcs::GdwArgs a{};
  a.x = x; a.dy = dy; a.n = g.n; a.c = g.cin; a.h = g.h; a.w_ = g.w; a.groups = g.groups;
  dw_tiling(g, &a.tiles_y, &a.tiles_x, &a.tiles_per_block, &a.blocks_per_group);
  const size_t need = group_small_dweight_workspace(g);
  const long long count = (long long)g.cout * g.cig * 9;
  if (a.blocks_per_group > 1 && (!ws || ws_bytes < need))
    return fail(B200_EWORKSPACE, "grouped dWeight needs a workspace of %zu bytes (got %zu)", need, ws_bytes);
  a.partial = a.blocks_per_group > 1 ? ws : dw;   // one block per group writes dW directly ([cout][cig][9])
  const long long blocks = (long long)g.groups * a.blocks_per_group;
  if (g.cig == 4) gcs::gconv_dw_kernel<4, 1><<<(unsigned)blocks, gcs::THREADS, 0, st>>>(a);
  else gcs::gconv_dw_kernel<8, 1><<<(unsigned)blocks, gcs::THREADS, 0, st>>>(a);
  count_launch();
  if (int rc = launch_check("gconv_dw_kernel")) return rc;
  if (a.blocks_per_group > 1) return finalize_splits(ws, dw, count, a.blocks_per_group, st);
  return B200_OK;
}

}  // namespace b200
