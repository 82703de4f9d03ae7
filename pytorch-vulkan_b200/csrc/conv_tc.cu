// tcgen05 implicit-GEMM kernels for FP32 convolution on sm_100a.
//
// Numerics: every FP32 operand is split into two TF32 values (hi + lo) while it is staged into
// shared memory; each K block is multiplied three times (hi*hi, hi*lo, lo*hi) by tcgen05.mma
// kind::tf32 into one FP32 accumulator tile that lives in tensor memory (TMEM).
//
// Structure of one CTA (544 threads, one output tile of 128 rows x BN columns):
//   warps 0-7  producer group 0  \  gather activations straight from the caller's strided view
//   warps 8-15 producer group 1  /  (NCHW, channels-last, sliced ...), split them, and write the
//                                   128-byte-swizzled K-major operand tiles; the two groups take
//                                   alternate K blocks so global-load latency overlaps the MMAs
//   warp 16    allocates TMEM, issues the tcgen05.mma stream, commits stages back to producers
//   warps 0-15 afterwards read the accumulator with tcgen05.ld and store the result
// Stages are handed over with mbarriers; every wait is bounded (tc_common.cuh).
//
// Replaces the reference's tiled shaders (paths inside the reference tree):
//   forward  csrc/shaders/conv2d_tiled_body.glsl:53-86        (+ bias epilogue :19-25)
//   dInput   csrc/shaders/conv2d_backward_input_tiled_body.glsl:49-93
//   dWeight  csrc/shaders/conv2d_backward_weight_tiled_body.glsl:42-70 + conv2d_backward_weight_finalize.comp
//   GEMM     csrc/shaders/matmul_strided_reg.comp / matmul_strided_reg_bias.comp
#include "common.cuh"
#include "tc_common.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace b200 {
namespace tc {

constexpr int BLOCK_M = 128;
constexpr int KBLK = 32;  // FP32 elements per K block = one 128-byte swizzle row
constexpr int PRODUCER_WARPS = 16, GROUP_THREADS = 256;
constexpr int THREADS = (PRODUCER_WARPS + 1) * 32;

template <int BN>
struct TileCfg {
  static constexpr int STAGES = BN == 256 ? 2 : (BN == 128 ? 3 : 4);
  static constexpr int A_PLANE = BLOCK_M * 128;
  static constexpr int B_PLANE = BN * 128;
  static constexpr int STAGE_BYTES = 2 * A_PLANE + 2 * B_PLANE;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
};

struct Pipe {  // shared-memory addresses of the pipeline state
  uint32_t tiles, full, empty, accum, tmem_slot;
  volatile int* abort_flag;
  volatile uint32_t* tmem_slot_ptr;
  int* status;
};

template <int BN>
__device__ __forceinline__ Pipe pipe_setup(unsigned char* smem_raw, int producer_arrivals, int* status) {
  using Cfg = TileCfg<BN>;
  Pipe p;
  p.status = status;
  const uint32_t raw = smem_u32(smem_raw);
  p.tiles = (raw + 1023u) & ~1023u;
  unsigned char* ctrl = smem_raw + (p.tiles - raw) + Cfg::TILE_BYTES;
  p.full = smem_u32(ctrl);
  p.empty = p.full + 8 * Cfg::STAGES;
  p.accum = p.empty + 8 * Cfg::STAGES;
  p.tmem_slot = p.accum + 8;
  p.tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(ctrl + 8 * (2 * Cfg::STAGES + 1));
  p.abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * (2 * Cfg::STAGES + 1) + 4);
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(p.full + 8 * s, producer_arrivals);
      mbar_init(p.empty + 8 * s, 1);
    }
    mbar_init(p.accum, 1);
    *p.abort_flag = 0;
    fence_barrier_init();
  }
  if (threadIdx.x / 32 == PRODUCER_WARPS) tmem_alloc(p.tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return p;
}

// The MMA warp: for every K block, three tcgen05.mma passes (hi*hi, hi*lo, lo*hi), four K=8
// steps each, then hand the stage back.  Returns false if a bounded wait gave up.
template <int BN>
__device__ __forceinline__ void mma_loop(const Pipe& p, uint32_t tmem_acc, int kblocks) {
  using Cfg = TileCfg<BN>;
  constexpr uint32_t idesc = make_idesc_tf32(BLOCK_M, BN);
  const int lane = threadIdx.x & 31;
  for (int kb = 0; kb < kblocks; ++kb) {
    const int s = kb % Cfg::STAGES;
    const uint32_t it = (uint32_t)(kb / Cfg::STAGES);
    if (!mbar_wait(p.full + 8 * s, it & 1, p.abort_flag, p.status, STATUS_TIMEOUT_FULL)) return;
    tc_fence_after();
    if (lane == 0) {
      const uint32_t a_hi = p.tiles + s * Cfg::STAGE_BYTES, a_lo = a_hi + Cfg::A_PLANE;
      const uint32_t b_hi = a_lo + Cfg::A_PLANE, b_lo = b_hi + Cfg::B_PLANE;
      const uint64_t da_hi = make_kmajor_sw128_desc(a_hi), da_lo = make_kmajor_sw128_desc(a_lo);
      const uint64_t db_hi = make_kmajor_sw128_desc(b_hi), db_lo = make_kmajor_sw128_desc(b_lo);
      // small cross terms first, then the dominant term
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_lo + 2 * kk, db_hi + 2 * kk, idesc, (kb | kk) != 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_hi + 2 * kk, db_lo + 2 * kk, idesc, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_hi + 2 * kk, db_hi + 2 * kk, idesc, 1);
      umma_commit(p.empty + 8 * s);
    }
    __syncwarp();
  }
  if (lane == 0) umma_commit(p.accum);
  __syncwarp();
}

template <int BN>
__device__ __forceinline__ void pipe_teardown(const Pipe& p, uint32_t tmem_acc) {
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x / 32 == PRODUCER_WARPS) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, TileCfg<BN>::TMEM_COLS);
  }
}

// Copy one pre-split weight row block: lane = k.  Rows n0.. of the [rows_total][ktot] planes.
template <int BN>
__device__ __forceinline__ void produce_rows_kcontig(uint32_t plane_hi, uint32_t plane_lo, const float* __restrict__ hi,
                                                     const float* __restrict__ lo, long long row0, int rows_valid,
                                                     long long ktot, long long k0, int warp_in_group, int lane) {
  constexpr int ROWS_PER_WARP = BN / (GROUP_THREADS / 32), BATCH = 8;
#pragma unroll 1
  for (int r0 = 0; r0 < ROWS_PER_WARP; r0 += BATCH) {
    float vh[BATCH], vl[BATCH];
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {  // all loads of the batch in flight before the first store
      const int r = warp_in_group + (r0 + j) * (GROUP_THREADS / 32);
      vh[j] = vl[j] = 0.f;
      if (r < rows_valid) {
        const long long off = (row0 + r) * ktot + k0 + lane;
        vh[j] = __ldg(hi + off);
        vl[j] = __ldg(lo + off);
      }
    }
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      const int r = warp_in_group + (r0 + j) * (GROUP_THREADS / 32);
      const uint32_t o = sw128_offset(r, lane);
      sts_f32(plane_hi + o, vh[j]);
      sts_f32(plane_lo + o, vl[j]);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Forward and dInput: rows = pixels (128 per tile), columns = output channels of one group,
// K = (tap, channel) with 32 consecutive channels of one filter tap per K block.
// ---------------------------------------------------------------------------------------
struct ConvTcArgs {
  ConvGeom g;
  View4 act;                // forward: x.  dInput: dy
  const float* w_hi;        // [groups][nc][taps*kc] pre-split weights, K contiguous
  const float* w_lo;
  const float* bias;
  long long bias_stride;
  float* out;               // forward: y.  dInput: dx (contiguous NCHW)
  long long rows_total;     // pixels of the output map: n*oh*ow (forward) or n*h*w (dInput)
  int out_w, out_hw;        // width and plane size of the output map
  int kc, nc;               // reduction / output channels per group
  int cblocks, kblocks, tiles_n;
  int out_channels;         // cout (forward) or cin (dInput)
  int* status;
  // dInput with stride > 1: the rows of the implicit GEMM are ordered by input-pixel parity class
  // ("phase" (y % sh, x % sw)).  Every pixel of a phase is reached by the same subset of filter taps,
  // so a tile only runs the K blocks of those taps: no MMA is spent on the structurally-zero taps
  // (for stride 2 and a 3x3 filter that is 9/4 taps per pixel instead of 9).
  int phases;                          // 1 = plain row order
  int phase_tile_start[17];            // first M tile of each phase (prefix sums)
  unsigned long long phase_taps[16];   // bit t set: filter tap t contributes to this phase
};

__device__ __forceinline__ int nth_set_bit(unsigned long long mask, int n) {
  for (int i = 0; i < n; ++i) mask &= mask - 1;
  return __ffsll((long long)mask) - 1;
}

// Row r of M tile `tile` -> output pixel (batch, y, x); false if the row is padding.
struct RowMap {
  int phases, sh, sw, p, q, hp, wq, out_w, out_hw;
  long long rows_total, tile0;
  __device__ __forceinline__ bool decode(long long tile, int r, long long& b, int& py, int& px) const {
    if (phases == 1) {
      const long long pix = tile * BLOCK_M + r;
      if (pix >= rows_total) return false;
      b = pix / out_hw;
      const int pos = (int)(pix - b * out_hw);
      py = pos / out_w;
      px = pos - py * out_w;
      return true;
    }
    const long long idx = (tile - tile0) * BLOCK_M + r;
    const long long per = (long long)hp * wq;
    if (per == 0 || idx >= rows_total) return false;
    b = idx / per;
    const int pos = (int)(idx - b * per);
    const int yy = pos / wq;
    py = yy * sh + p;
    px = (pos - yy * wq) * sw + q;
    return true;
  }
};

template <int BN, bool IS_DX>
__global__ void __launch_bounds__(THREADS, 1) conv_tc_kernel(const ConvTcArgs a) {
  using Cfg = TileCfg<BN>;
  extern __shared__ unsigned char smem_raw[];
  const Pipe p = pipe_setup<BN>(smem_raw, GROUP_THREADS, a.status);
  const uint32_t tmem_acc = *p.tmem_slot_ptr;
  const ConvGeom& g = a.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = blockIdx.y / a.tiles_n;
  const int n0 = (blockIdx.y % a.tiles_n) * BN;
  const int cols_valid = min(BN, a.nc - n0);
  RowMap rm;
  rm.phases = 1; rm.out_w = a.out_w; rm.out_hw = a.out_hw; rm.rows_total = a.rows_total; rm.tile0 = 0;
  rm.sh = rm.sw = 1; rm.p = rm.q = 0; rm.hp = rm.wq = 0;
  unsigned long long tapmask = ~0ull;
  int kblocks = a.kblocks;
  if (IS_DX && a.phases > 1) {
    int ph = 0;
    while (ph + 1 < a.phases && (int)blockIdx.x >= a.phase_tile_start[ph + 1]) ++ph;
    rm.phases = a.phases; rm.sh = g.sh; rm.sw = g.sw; rm.p = ph / g.sw; rm.q = ph % g.sw;
    rm.hp = (g.h - rm.p + g.sh - 1) / g.sh;
    rm.wq = (g.w - rm.q + g.sw - 1) / g.sw;
    rm.rows_total = (long long)g.n * rm.hp * rm.wq;
    rm.tile0 = a.phase_tile_start[ph];
    tapmask = a.phase_taps[ph];
    kblocks = __popcll(tapmask) * a.cblocks;
  }

  if (warp == PRODUCER_WARPS) {
    mma_loop<BN>(p, tmem_acc, kblocks);
  } else {
    // ---- producers ----
    const int grp = warp >> 3, t = threadIdx.x & (GROUP_THREADS - 1);
    const int row = t & 127, khalf = t >> 7;  // this thread stages 16 channels of one pixel row
    long long base = 0, b = 0;
    int y0 = 0, x0 = 0, py = 0, px = 0;
    const bool row_ok = rm.decode(blockIdx.x, row, b, py, px);
    const bool vec_ok = a.act.s1 == 1 && ((reinterpret_cast<uintptr_t>(a.act.ptr) & 15) == 0) && a.act.s0 % 4 == 0 &&
                        a.act.s2 % 4 == 0 && a.act.s3 % 4 == 0;
    if (row_ok) {
      if (IS_DX) { y0 = py + g.ph; x0 = px + g.pw; }
      else { y0 = py * g.sh - g.ph; x0 = px * g.sw - g.pw; }
      base = b * a.act.s0 + (long long)group * a.kc * a.act.s1;
    }
    const long long ktot = (long long)g.kh * g.kw * a.kc;
    const long long wrow0 = (long long)group * a.nc + n0;
    for (int kb = grp; kb < kblocks; kb += 2) {
      const int s = kb % Cfg::STAGES;
      const uint32_t it = (uint32_t)(kb / Cfg::STAGES);
      const int tap_slot = kb / a.cblocks, cblk = kb - tap_slot * a.cblocks;
      const int tap = (IS_DX && a.phases > 1) ? nth_set_bit(tapmask, tap_slot) : tap_slot;
      const int c0 = cblk * KBLK + khalf * 16;
      const int ky = tap / g.kw, kx = tap - ky * g.kw;
      bool ok = row_ok;
      int iy, ix;
      if (IS_DX) {
        int yy = y0 - ky * g.dh, xx = x0 - kx * g.dw;
        ok = ok && yy >= 0 && xx >= 0;
        if (g.sh != 1 || g.sw != 1) {
          ok = ok && (yy % g.sh == 0) && (xx % g.sw == 0);
          yy /= g.sh;
          xx /= g.sw;
        }
        ok = ok && yy < g.oh && xx < g.ow;
        iy = yy; ix = xx;
      } else {
        iy = y0 + ky * g.dh; ix = x0 + kx * g.dw;
        ok = ok && iy >= 0 && iy < g.h && ix >= 0 && ix < g.w;
      }
      // Issue the global loads before waiting for the stage: they only need registers.
      float v[16];
      const float* src = a.act.ptr + base + (long long)c0 * a.act.s1 + (long long)iy * a.act.s2 + (long long)ix * a.act.s3;
      if (ok && vec_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 f = __ldg(reinterpret_cast<const float4*>(src) + j);
          v[4 * j] = f.x; v[4 * j + 1] = f.y; v[4 * j + 2] = f.z; v[4 * j + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = ok ? __ldg(src + j * a.act.s1) : 0.f;
      }
      if (!mbar_wait(p.empty + 8 * s, (it & 1) ^ 1, p.abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) break;
      const uint32_t a_hi = p.tiles + s * Cfg::STAGE_BYTES, a_lo = a_hi + Cfg::A_PLANE;
      const uint32_t b_hi = a_lo + Cfg::A_PLANE, b_lo = b_hi + Cfg::B_PLANE;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) split_tf32(v[q * 4 + j], h[j], l[j]);
        const uint32_t o = sw128_offset(row, khalf * 16 + q * 4);
        sts_f32x4(a_hi + o, h[0], h[1], h[2], h[3]);
        sts_f32x4(a_lo + o, l[0], l[1], l[2], l[3]);
      }
      produce_rows_kcontig<BN>(b_hi, b_lo, a.w_hi, a.w_lo, wrow0, cols_valid, ktot, (long long)tap * a.kc + cblk * KBLK, warp & 7, lane);
      fence_proxy_async();
      mbar_arrive(p.full + 8 * s);
    }
    // ---- epilogue: TMEM -> registers -> global ----
    if (mbar_wait(p.accum, 0, p.abort_flag, p.status, STATUS_TIMEOUT_ACCUM)) {
      tc_fence_after();
      const int q = warp & 3, chunk = warp >> 2;  // lane quarter of this warp, column chunk
      long long ob = 0, obase = 0;
      int opy = 0, opx = 0;
      const bool orow_ok = rm.decode(blockIdx.x, q * 32 + lane, ob, opy, opx);
      if (orow_ok) obase = (ob * a.out_channels + (long long)group * a.nc) * a.out_hw + (long long)opy * a.out_w + opx;
      constexpr int COLS_PER_WARP = BN / 4;
#pragma unroll 1
      for (int c = 0; c < COLS_PER_WARP; c += 32) {
        const int col0 = chunk * COLS_PER_WARP + c;
        if (col0 >= cols_valid) break;  // warp-uniform
        float v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)col0, v);
        if (orow_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + j;
            if (col < cols_valid) {
              float r = kblocks > 0 ? v[j] : 0.f;  // a phase no tap reaches has a zero gradient
              if (a.bias) r += __ldg(a.bias + ((long long)group * a.nc + n0 + col) * a.bias_stride);
              a.out[obase + (long long)(n0 + col) * a.out_hw] = r;
            }
          }
        }
      }
    }
  }
  pipe_teardown<BN>(p, tmem_acc);
}

// Weight staging: split W into TF32 hi/lo planes and reorder so that the reduction index of the
// phase is contiguous.  forward: [g][co][tap][ci];  dInput: [g][ci][tap][co].
__global__ void __launch_bounds__(256) prep_weights_kernel(ConvGeom g, View4 w, int is_dx, float* __restrict__ hi,
                                                           float* __restrict__ lo, long long total) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= total) return;
  const int taps = g.kh * g.kw;
  const int kc = is_dx ? g.cog : g.cig, nc = is_dx ? g.cig : g.cog;
  const int c = (int)(i % kc);
  const int tap = (int)((i / kc) % taps);
  const int r = (int)((i / ((long long)kc * taps)) % nc);
  const int grp = (int)(i / ((long long)kc * taps * nc));
  const int co = is_dx ? c : r, ci = is_dx ? r : c;
  const float v = w.ptr[((long long)grp * g.cog + co) * w.s0 + ci * w.s1 + (tap / g.kw) * w.s2 + (tap % g.kw) * w.s3];
  float h, l;
  split_tf32(v, h, l);
  hi[i] = h;
  lo[i] = l;
}


// ---------------------------------------------------------------------------------------
// dWeight: D[(tap,ci)][co] = sum over output positions of Xshifted[(tap,ci)][pos] * dY[co][pos].
// rows  = 128 (tap, ci) pairs of one group, columns = BN output channels, K = positions of one
// split (32 per K block, lane = position, so NCHW loads are coalesced).  Partials of the splits
// go to [split][cout][cig*taps] and are summed in ascending order by finalize_kernel.
// ---------------------------------------------------------------------------------------
struct DwTcArgs {
  ConvGeom g;
  View4 x, dy;
  float* out;            // dW itself (one split) or the partial buffer
  long long positions;   // n*oh*ow
  int span;              // positions per split (multiple of 32)
  int m_total;           // taps * cig
  int tiles_m, tiles_n;
  int* status;
};
struct DwRow {
  long long chan_off;  // (g*cig + ci) * x.s1, or -1 for a padding row
  int ydelta, xdelta;  // ky*dh - ph, kx*dw - pw
};
constexpr int DW_TABLE_BYTES = BLOCK_M * (int)sizeof(DwRow);

template <int BN>
__global__ void __launch_bounds__(THREADS, 1) dweight_tc_kernel(const DwTcArgs a) {
  using Cfg = TileCfg<BN>;
  extern __shared__ unsigned char smem_raw[];
  const Pipe p = pipe_setup<BN>(smem_raw, GROUP_THREADS, a.status);
  const uint32_t tmem_acc = *p.tmem_slot_ptr;
  const ConvGeom& g = a.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_group = a.tiles_m * a.tiles_n;
  const int group = blockIdx.x / tiles_per_group;
  const int tile = blockIdx.x - group * tiles_per_group;
  const int m0 = (tile / a.tiles_n) * BLOCK_M, n0 = (tile % a.tiles_n) * BN;
  const int split = blockIdx.y;
  const long long k_begin = (long long)split * a.span;
  const long long k_end = min(a.positions, k_begin + a.span);
  const int kblocks = (int)((k_end - k_begin + KBLK - 1) / KBLK);
  const int cols_valid = min(BN, g.cog - n0);
  const int taps = g.kh * g.kw;
  // row table, placed behind the pipeline control block
  DwRow* rows = reinterpret_cast<DwRow*>(smem_raw + (p.full - smem_u32(smem_raw)) + 256);
  if (threadIdx.x < BLOCK_M) {
    const int m = m0 + threadIdx.x;
    DwRow r;
    r.chan_off = -1; r.ydelta = 0; r.xdelta = 0;
    if (m < a.m_total) {
      const int tap = m / g.cig, ci = m - tap * g.cig;
      r.chan_off = ((long long)group * g.cig + ci) * a.x.s1;
      r.ydelta = (tap / g.kw) * g.dh - g.ph;
      r.xdelta = (tap % g.kw) * g.dw - g.pw;
    }
    rows[threadIdx.x] = r;
  }
  __syncthreads();

  if (warp == PRODUCER_WARPS) {
    mma_loop<BN>(p, tmem_acc, kblocks);
  } else {
    const int grp = warp >> 3, wi = warp & 7;
    const int ohw = g.oh * g.ow;
    const bool channels_last = a.x.s1 == 1 && a.dy.s1 == 1 && a.x.s3 != 1 && a.dy.s3 != 1;
    for (int kb = grp; kb < kblocks; kb += 2) {
      const int s = kb % Cfg::STAGES;
      const uint32_t it = (uint32_t)(kb / Cfg::STAGES);
      const long long pos = k_begin + (long long)kb * KBLK + lane;
      const bool ok = pos < k_end;
      long long xb = 0, yb = 0;
      int iy0 = 0, ix0 = 0;
      if (ok) {
        const long long b = pos / ohw;
        const int sp = (int)(pos - b * ohw);
        const int oy = sp / g.ow, ox = sp - oy * g.ow;
        iy0 = oy * g.sh; ix0 = ox * g.sw;
        xb = b * a.x.s0;
        yb = b * a.dy.s0 + (long long)oy * a.dy.s2 + (long long)ox * a.dy.s3;
      }
      if (!mbar_wait(p.empty + 8 * s, (it & 1) ^ 1, p.abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) break;
      const uint32_t a_hi = p.tiles + s * Cfg::STAGE_BYTES, a_lo = a_hi + Cfg::A_PLANE;
      const uint32_t b_hi = a_lo + Cfg::A_PLANE, b_lo = b_hi + Cfg::B_PLANE;
      if (channels_last) {
        // Channels-last operands: lane = row (32 consecutive channels are contiguous in memory), the
        // 32 pixels of the K block are walked four at a time; each pixel's coordinates come from the
        // lane that decoded it.  One 16-byte swizzled store per lane per four pixels.
        constexpr int ROW_BLOCKS = 4 + BN / 32;
#pragma unroll 1
        for (int rb = wi; rb < ROW_BLOCKS; rb += 8) {
          const bool is_a = rb < 4;
          const int r = (is_a ? rb : rb - 4) * 32 + lane;
          DwRow row;
          row.chan_off = -1; row.ydelta = 0; row.xdelta = 0;
          if (is_a) row = rows[r];
          const long long ychan = ((long long)group * g.cog + n0 + r) * a.dy.s1;
          const bool brow_ok = r < cols_valid;
          const uint32_t p_hi = is_a ? a_hi : b_hi, p_lo = is_a ? a_lo : b_lo;
#pragma unroll 1
          for (int kq = 0; kq < 8; kq += 2) {
            float v[8];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const int k = kq * 4 + kk;
              const bool kok = __shfl_sync(0xffffffffu, ok ? 1 : 0, k) != 0;
              const long long kxb = __shfl_sync(0xffffffffu, xb, k), kyb = __shfl_sync(0xffffffffu, yb, k);
              const int kiy = __shfl_sync(0xffffffffu, iy0, k), kix = __shfl_sync(0xffffffffu, ix0, k);
              float val = 0.f;
              if (is_a) {
                const int iy = kiy + row.ydelta, ix = kix + row.xdelta;
                if (kok && row.chan_off >= 0 && iy >= 0 && iy < g.h && ix >= 0 && ix < g.w)
                  val = __ldg(a.x.ptr + kxb + row.chan_off + (long long)iy * a.x.s2 + (long long)ix * a.x.s3);
              } else if (kok && brow_ok) {
                val = __ldg(a.dy.ptr + kyb + ychan);
              }
              v[kk] = val;
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              float h[4], l[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) split_tf32(v[half * 4 + j], h[j], l[j]);
              const uint32_t o = sw128_offset(r, (kq + half) * 4);
              sts_f32x4(p_hi + o, h[0], h[1], h[2], h[3]);
              sts_f32x4(p_lo + o, l[0], l[1], l[2], l[3]);
            }
          }
        }
        fence_proxy_async();
        mbar_arrive(p.full + 8 * s);
        continue;
      }
      // A rows: shifted input, 16 consecutive (tap, ci) rows per warp
#pragma unroll 1
      for (int r0 = 0; r0 < 16; r0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const DwRow row = rows[wi * 16 + r0 + j];
          const int iy = iy0 + row.ydelta, ix = ix0 + row.xdelta;
          const bool in = ok && row.chan_off >= 0 && iy >= 0 && iy < g.h && ix >= 0 && ix < g.w;
          v[j] = in ? __ldg(a.x.ptr + xb + row.chan_off + (long long)iy * a.x.s2 + (long long)ix * a.x.s3) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float h, l;
          split_tf32(v[j], h, l);
          const uint32_t o = sw128_offset(wi * 16 + r0 + j, lane);
          sts_f32(a_hi + o, h);
          sts_f32(a_lo + o, l);
        }
      }
      // B rows: output gradient, BN/8 consecutive channels per warp
      constexpr int BROWS = BN / 8;
#pragma unroll 1
      for (int r0 = 0; r0 < BROWS; r0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = wi * BROWS + r0 + j;
          const bool in = ok && r < cols_valid;
          v[j] = in ? __ldg(a.dy.ptr + yb + ((long long)group * g.cog + n0 + r) * a.dy.s1) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float h, l;
          split_tf32(v[j], h, l);
          const uint32_t o = sw128_offset(wi * BROWS + r0 + j, lane);
          sts_f32(b_hi + o, h);
          sts_f32(b_lo + o, l);
        }
      }
      fence_proxy_async();
      mbar_arrive(p.full + 8 * s);
    }
    // ---- epilogue: lane = (tap, ci) row, registers = consecutive output channels ----
    if (kblocks > 0 && mbar_wait(p.accum, 0, p.abort_flag, p.status, STATUS_TIMEOUT_ACCUM)) {
      tc_fence_after();
      const int q = warp & 3, chunk = warp >> 2;
      const int m = m0 + q * 32 + lane;
      const bool row_ok = m < a.m_total;
      const int tap = row_ok ? m / g.cig : 0, ci = row_ok ? m - tap * g.cig : 0;
      const long long cols = (long long)g.cig * taps;
      float* out = a.out + ((long long)split * g.cout + (long long)group * g.cog + n0) * cols + (long long)ci * taps + tap;
      constexpr int COLS_PER_WARP = BN / 4;
#pragma unroll 1
      for (int c = 0; c < COLS_PER_WARP; c += 32) {
        const int col0 = chunk * COLS_PER_WARP + c;
        if (col0 >= cols_valid) break;
        float v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)col0, v);
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < cols_valid) out[(long long)(col0 + j) * cols] = v[j];
        }
      }
    }
  }
  pipe_teardown<BN>(p, tmem_acc);
}

}  // namespace tc

using namespace tc;

static int pick_bn(int nc) { return nc <= 64 ? 64 : (nc <= 128 ? 128 : 256); }
static void tc_dweight_plan(const ConvGeom& g, size_t budget, int* splits_out, int* span_out, size_t* bytes_out);

// B200_CONV_TC_VARIANT=gather forces the per-tap gather kernel where the strip kernel would run
// (A/B measurements); anything else lets the strip kernel take the geometries it supports.
static bool strip_allowed() {
  const char* v = getenv("B200_CONV_TC_VARIANT");
  return !(v && !strcmp(v, "gather"));
}

bool tc_supported(const ConvGeom& g, int phase) {
  // the gather kernels need the reduction channels in blocks of 32; the strip kernel pads a ragged block
  const bool strip = (phase == B200_PHASE_FORWARD || phase == B200_PHASE_DINPUT) && strip_allowed() && strip_supported(g, phase);
  if (phase == B200_PHASE_FORWARD) return g.cog >= 16 && (g.cig % KBLK == 0 || strip);
  if (phase == B200_PHASE_DINPUT) return g.cig >= 16 && (g.cog % KBLK == 0 || strip);
  if (phase == B200_PHASE_DWEIGHT) return g.cog >= 16 && g.cig * g.kh * g.kw >= 32;
  return false;
}

// Split plan of the tcgen05 dWeight kernel: enough (tile, split) CTAs for about two per SM, every
// split at least eight K blocks long, partial buffer within the budget; spans are multiples of 32.
static void tc_dweight_plan(const ConvGeom& g, size_t budget, int* splits_out, int* span_out, size_t* bytes_out) {
  const long long positions = (long long)g.n * g.oh * g.ow;
  const int bn = pick_bn(g.cog);
  const long long tiles = div_up64((long long)g.cig * g.kh * g.kw, BLOCK_M) * div_up64(g.cog, bn) * g.groups;
  const size_t dw_bytes = sizeof(float) * (size_t)g.cout * g.cig * g.kh * g.kw;
  long long want = std::max<long long>(1, div_up64(2ll * sm_count(), tiles));
  want = std::min<long long>(want, std::max<long long>(1, positions / (8 * KBLK)));
  want = std::min<long long>(want, 65535);
  want = std::min<long long>(want, (long long)(budget / dw_bytes));
  long long span = positions, splits = 1;
  if (want >= 2) {
    span = div_up64(div_up64(positions, want), KBLK) * KBLK;
    splits = div_up64(positions, span);
  }
  *splits_out = (int)splits;
  *span_out = (int)std::min<long long>(span, 2147483616ll);
  *bytes_out = splits > 1 ? (size_t)splits * dw_bytes : 0;
}

size_t tc_workspace(const ConvGeom& g, int phase, size_t budget, int* splits_out, int* span_out) {
  (void)budget;
  if (splits_out) *splits_out = 1;
  if (span_out) *span_out = 0;
  if (phase == B200_PHASE_FORWARD || phase == B200_PHASE_DINPUT) {
    const size_t planes = 2 * sizeof(float) * (size_t)g.cout * g.cig * g.kh * g.kw;  // hi + lo
    size_t need = strip_allowed() && strip_supported(g, phase) ? std::max(planes, strip_workspace(g, phase)) : planes;
    if (strip_allowed() && tstrip_supported(g, phase)) need = std::max(need, tstrip_workspace(g, phase));
    return need;
  }
  if (phase == B200_PHASE_DWEIGHT && strip_allowed() && dweight_strip_supported(g)) {
    if (splits_out) *splits_out = 0;
    return dweight_strip_workspace(g, budget);
  }
  if (phase == B200_PHASE_DWEIGHT) {
    int splits, span;
    size_t bytes;
    tc_dweight_plan(g, budget, &splits, &span, &bytes);
    if (splits_out) *splits_out = splits;
    if (span_out) *span_out = span;
    return bytes;
  }
  return 0;
}

template <int BN, bool IS_DX>
static int launch_conv_tc(const ConvTcArgs& a, dim3 grid, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    B200_CUDA(cudaFuncSetAttribute(conv_tc_kernel<BN, IS_DX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   TileCfg<BN>::SMEM_BYTES));
    configured = true;
  }
  conv_tc_kernel<BN, IS_DX><<<grid, THREADS, TileCfg<BN>::SMEM_BYTES, st>>>(a);
  count_launch();
  return launch_check(IS_DX ? "conv_tc_kernel<dinput>" : "conv_tc_kernel<forward>");
}

static int conv_tc_run(const ConvGeom& g, bool is_dx, View4 act, View4 w, const float* bias, long long bias_stride,
                       float* out, void* ws, size_t ws_bytes, cudaStream_t st) {
  const size_t wcount = (size_t)g.cout * g.cig * g.kh * g.kw;
  if (!ws || ws_bytes < 2 * sizeof(float) * wcount)
    return fail(B200_EWORKSPACE, "tcgen05 convolution needs a workspace of %zu bytes (got %zu)",
                2 * sizeof(float) * wcount, ws_bytes);
  float* hi = (float*)ws;
  float* lo = hi + wcount;
  prep_weights_kernel<<<(unsigned)div_up64((long long)wcount, 256), 256, 0, st>>>(g, w, is_dx ? 1 : 0, hi, lo,
                                                                                  (long long)wcount);
  count_launch();
  if (int rc = launch_check("prep_weights_kernel")) return rc;
  ConvTcArgs a{};
  a.g = g; a.act = act; a.w_hi = hi; a.w_lo = lo; a.bias = bias; a.bias_stride = bias_stride; a.out = out;
  a.status = device_status_word();
  if (!a.status) return fail(B200_ECUDA, "device status word is not allocated");
  a.kc = is_dx ? g.cog : g.cig;
  a.nc = is_dx ? g.cig : g.cog;
  a.out_w = is_dx ? g.w : g.ow;
  a.out_hw = is_dx ? g.h * g.w : g.oh * g.ow;
  a.rows_total = (long long)g.n * a.out_hw;
  a.out_channels = is_dx ? g.cin : g.cout;
  a.cblocks = a.kc / KBLK;
  a.kblocks = g.kh * g.kw * a.cblocks;
  const int bn = pick_bn(a.nc);
  a.tiles_n = (a.nc + bn - 1) / bn;
  long long gx = div_up64(a.rows_total, BLOCK_M);
  const long long gy = (long long)g.groups * a.tiles_n;
  a.phases = 1;
  if (is_dx && (g.sh > 1 || g.sw > 1) && g.sh * g.sw <= 16 && g.kh * g.kw <= 64) {
    a.phases = g.sh * g.sw;
    long long tiles = 0;
    for (int ph = 0; ph < a.phases; ++ph) {
      const int p = ph / g.sw, q = ph % g.sw;
      const long long hp = (g.h - p + g.sh - 1) / g.sh, wq = (g.w - q + g.sw - 1) / g.sw;
      unsigned long long mask = 0;
      for (int ky = 0; ky < g.kh; ++ky)
        for (int kx = 0; kx < g.kw; ++kx)
          if (((p + g.ph - ky * g.dh) % g.sh + g.sh) % g.sh == 0 && ((q + g.pw - kx * g.dw) % g.sw + g.sw) % g.sw == 0)
            mask |= 1ull << (ky * g.kw + kx);
      a.phase_taps[ph] = mask;
      a.phase_tile_start[ph] = (int)tiles;
      tiles += div_up64((long long)g.n * hp * wq, BLOCK_M);
    }
    a.phase_tile_start[a.phases] = (int)tiles;
    gx = tiles;
  }
  if (gx > 2147483647ll || gy > 65535) return fail(B200_ERANGE, "tcgen05 convolution: grid exceeds launch limits");
  const dim3 grid((unsigned)gx, (unsigned)gy);
  if (is_dx) {
    if (bn == 64) return launch_conv_tc<64, true>(a, grid, st);
    if (bn == 128) return launch_conv_tc<128, true>(a, grid, st);
    return launch_conv_tc<256, true>(a, grid, st);
  }
  if (bn == 64) return launch_conv_tc<64, false>(a, grid, st);
  if (bn == 128) return launch_conv_tc<128, false>(a, grid, st);
  return launch_conv_tc<256, false>(a, grid, st);
}

// Which kernel takes a forward / dInput call that asked for the tcgen05 candidate:
//   0  the strip kernel (the normal case);
//   1  the gather kernel: the strip kernel declines at run time (a view that spans more elements than its
//      32-bit offsets address) and the reduction channels come in whole blocks of 32, which the gather
//      kernel needs (it has no ragged-block padding);
//   2  the CUDA-core implicit GEMM: everything else (a ragged channel count on such a view);
//   3  the transposed strip kernel, where most of a 128-channel tile is real output channels.
// Pure host arithmetic on the geometry and the view's strides; nothing is dereferenced.
int tc_route(const ConvGeom& g, bool is_dx, const View4& act) {
  const int kc = is_dx ? g.cog : g.cig;
  // 3: the transposed strip kernel (filter on M), which addresses the view with 64-bit offsets
  if (strip_allowed() && tstrip_supported(g, is_dx ? B200_PHASE_DINPUT : B200_PHASE_FORWARD)) return 3;
  if (strip_allowed() && strip_supported(g, is_dx ? B200_PHASE_DINPUT : B200_PHASE_FORWARD) &&
      strip_view_addressable(g, is_dx, act, nullptr))
    return 0;
  return kc % KBLK == 0 ? 1 : 2;
}

int tc_forward(const ConvGeom& g, View4 x, View4 w, const float* bias, long long bias_stride, float* y, void* ws,
               size_t ws_bytes, cudaStream_t st) {
  int route = tc_route(g, false, x);
  if (route == 3) {
    note_kernel("tc_tstrip_forward");
    const int rc = tstrip_conv(g, false, x, w, bias, bias_stride, y, ws, ws_bytes, st);
    if (rc != B200_EUNSUPPORTED) return rc;
    route = strip_supported(g, B200_PHASE_FORWARD) && strip_view_addressable(g, false, x, nullptr) ? 0 : (g.cig % KBLK == 0 ? 1 : 2);
  }
  if (route == 0) {
    note_kernel("tc_strip_forward");
    const int rc = strip_conv(g, false, x, w, bias, bias_stride, y, ws, ws_bytes, st);
    if (rc != B200_EUNSUPPORTED) return rc;  // e.g. more tiles than the kernel's 32-bit job indices
    route = g.cig % KBLK == 0 ? 1 : 2;
  }
  if (route == 1) {
    note_kernel("tc_igemm_forward");
    return conv_tc_run(g, false, x, w, bias, bias_stride, y, ws, ws_bytes, st);
  }
  note_kernel("simt_igemm_forward");
  return simt_igemm_forward(g, x, w, bias, bias_stride, y, st);
}
int tc_dinput(const ConvGeom& g, View4 dy, View4 w, const float* bias, long long bias_stride, float* dx, void* ws, size_t ws_bytes,
              cudaStream_t st, bool* bias_applied) {
  if (bias_applied) *bias_applied = bias != nullptr;
  int route = tc_route(g, true, dy);
  if (route == 3) {
    note_kernel("tc_tstrip_dinput");
    const int rc = tstrip_conv(g, true, dy, w, bias, bias_stride, dx, ws, ws_bytes, st);
    if (rc != B200_EUNSUPPORTED) return rc;
    route = strip_supported(g, B200_PHASE_DINPUT) && strip_view_addressable(g, true, dy, nullptr) ? 0 : (g.cog % KBLK == 0 ? 1 : 2);
  }
  if (route == 0) {
    note_kernel("tc_strip_dinput");
    const int rc = strip_conv(g, true, dy, w, bias, bias_stride, dx, ws, ws_bytes, st);
    if (rc != B200_EUNSUPPORTED) return rc;
    route = g.cog % KBLK == 0 ? 1 : 2;
  }
  if (route == 1) {
    note_kernel("tc_igemm_dinput");
    return conv_tc_run(g, true, dy, w, bias, bias_stride, dx, ws, ws_bytes, st);
  }
  note_kernel("simt_igemm_dinput");
  if (bias_applied) *bias_applied = false;  // the CUDA-core kernel has no bias term: the caller adds it
  return simt_igemm_dinput(g, dy, w, dx, st);
}
template <int BN>
static int launch_dweight_tc(const DwTcArgs& a, dim3 grid, cudaStream_t st) {
  constexpr int SMEM = TileCfg<BN>::SMEM_BYTES + DW_TABLE_BYTES;
  static bool configured = false;
  if (!configured) {
    B200_CUDA(cudaFuncSetAttribute(dweight_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured = true;
  }
  dweight_tc_kernel<BN><<<grid, THREADS, SMEM, st>>>(a);
  count_launch();
  return launch_check("dweight_tc_kernel");
}

int tc_dweight(const ConvGeom& g, View4 x, View4 dy, float* dw, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (strip_allowed() && dweight_strip_supported(g)) {
    note_kernel("tc_strip_dweight");
    const int rc = dweight_strip(g, x, dy, dw, ws, ws_bytes, st);
    if (rc != B200_EUNSUPPORTED) return rc;  // tensors beyond 32-bit element offsets take the gather kernel
    note_kernel("tc_igemm_dweight");
  }
  int splits, span;
  size_t bytes;
  tc_dweight_plan(g, ws ? ws_bytes : 0, &splits, &span, &bytes);
  DwTcArgs a{};
  a.g = g; a.x = x; a.dy = dy;
  a.positions = (long long)g.n * g.oh * g.ow;
  a.span = span;
  a.m_total = g.cig * g.kh * g.kw;
  const int bn = pick_bn(g.cog);
  a.tiles_m = (a.m_total + BLOCK_M - 1) / BLOCK_M;
  a.tiles_n = (g.cog + bn - 1) / bn;
  a.out = splits > 1 ? (float*)ws : dw;
  a.status = device_status_word();
  if (!a.status) return fail(B200_ECUDA, "device status word is not allocated");
  const long long gx = (long long)a.tiles_m * a.tiles_n * g.groups;
  if (gx > 2147483647ll) return fail(B200_ERANGE, "tcgen05 dWeight: grid exceeds launch limits");
  const dim3 grid((unsigned)gx, (unsigned)splits);
  int rc = bn == 64 ? launch_dweight_tc<64>(a, grid, st)
         : bn == 128 ? launch_dweight_tc<128>(a, grid, st) : launch_dweight_tc<256>(a, grid, st);
  if (rc) return rc;
  if (splits > 1) return finalize_splits((const float*)ws, dw, (long long)g.cout * a.m_total, splits, st);
  return B200_OK;
}


}  // namespace b200
