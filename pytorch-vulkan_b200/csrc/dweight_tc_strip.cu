// tcgen05 dWeight kernel for filters up to eight taps wide (any stride, padding, dilation, groups;
// at least 16 channels on both sides), FP32 via 3xTF32.
//
//   dW[co][ci][ky][kx] = sum over grid pixels q of  dY[q][co] * X_phase(ky,kx)[q + shift(ky,kx)][ci]
//
// The contraction runs over pixels, so both operands are staged pixel-major ("MN-major" for the
// tensor core): one 128-byte shared-memory row per pixel holding 32 channels, TF32 hi and lo
// planes, written in the 128-byte/32-byte-base swizzle that tcgen05 requires for 32-bit MN-major
// operands.  The M dimension of the MMA (4 blocks of 32 rows, at a programmable byte stride) is
// filled in one of two ways (plan_dw_strip):
//   strip   stride 1, output as large as the input: the vertical tap (ky) is a start-address
//           offset of ONE staged input strip and, with a block stride of `dilation_w` rows, its
//           four M blocks are the horizontal taps kx = 0..3: a single tcgen05.mma of shape
//           128 x BN x 8 accumulates up to four taps of a 32-channel block at once.  Two channel
//           blocks per CTA (two accumulators in TMEM) share every staged dY block.
//   blocks  everything else: four exact 32-pixel blocks per K block, the taps kx of one channel
//           block (each read from its own column phase and offset of a strided input) or four
//           channel blocks of a 1x1 filter.
// Every CTA owns one (channel tile, ky, column tile, pixel split); its 16 producer warps stream the
// input and dY blocks straight from the caller's strided views, one 32-row block per warp, several
// K blocks in flight.  Split partials land in [split][cout][kh*kw][cin/g] (channel fastest: the
// epilogue's lanes store neighbouring floats) and finalize_partials_kernel sums them in ascending
// split order (no atomics, run-to-run identical) while transposing into dW.
//
// Replaces csrc/shaders/conv2d_backward_weight_tiled_body.glsl:42-70 and
// conv2d_backward_weight_finalize.comp:9-18 of the reference for these geometries.
#include "common.cuh"
#include "tc_common.cuh"

#include <algorithm>
#include <mutex>
#include <cstdio>
#include <cstdlib>

namespace b200 {
namespace tcdw {
using namespace tc;

// BF16 cross terms (tc_common.cuh) in this kernel: bf16 planes of 64-byte rows (SWIZZLE_64B) with the
// same row-shift and block-stride tricks as the TF32 planes.  The kernel is bound by what its producers
// pull from L2 (about 15-20 bytes per clock and SM for 128-byte pieces, loads or bulk copies alike), so
// the cross terms pay only where they cut that traffic: an accumulator then takes BN instead of 2*BN
// TMEM columns, and FOUR channel blocks can share every staged dY block.  Measured: 128/256/512-channel
// 3x3 layers 12-20 % faster, 64-channel, 1x1 and strided ones 2-8 % slower -- so the plan turns them
// on exactly when it can use four accumulators (plan_dw_strip); everything else runs 3xTF32.

constexpr int KP = 32;          // pixels per K block (four K=8 MMA steps)
constexpr int XR = 40;          // rows of one staged input strip: KP + margin for the horizontal taps
constexpr int XOFF = 4;         // row of the strip that corresponds to the first pixel of the K block
constexpr int PRODUCER_WARPS = 16;
constexpr int MMA_WARP = PRODUCER_WARPS;
constexpr int THREADS = (PRODUCER_WARPS + 1) * 32;
constexpr int MAX_STAGES = 6;
constexpr int SMEM_LIMIT = 232448 - 2048;
// The tensor core adds into its FP32 accumulator with truncation, so the error of one accumulation chain
// grows linearly with its length (measured: 2e-4 relative after 32k pixels, i.e. 8k accumulation steps).
// A CTA therefore keeps a chain to CHUNK_KB K blocks (3072 pixels, 768 steps: about 1.4e-5): after each
// chunk the epilogue warps fold the accumulator into the CTA's slot of `out` with ordinary FP32 adds
// (round to nearest; the first chunk is a store, later ones are global reductions with a single writer per
// address) and the next chunk starts from zero.  A long reduction then costs one pass over the CTA's own
// output tile every few thousand pixels (about 5 us per fold: the staging pipeline runs dry while the epilogue
// warps, which are also producers, read the accumulator) instead of more splits and more scratch.
constexpr int CHUNK_KB = 96;

struct DwStripArgs {
  ConvGeom g;
  View4 x, dy;
  float* out;            // dW (one split) or the partial buffer [split][cout][cig*taps]
  int H, W, pr, pc;      // padded pixel space (see conv_tc_strip.cu)
  int q_total;           // padded pixels (below 2^31 - 64)
  FastDiv img_div, row_div, div_tasks, div_stages;
  int span, splits;      // padded pixels per split (multiple of KP)
  int xblocks;           // staged input blocks per CTA: 1 (one strip, taps in M through the block stride) or 4
  int partial_layout;    // 1: `out` is the split buffer [split][cout][kh*kw][cig] (channel fastest, so the epilogue's
                         // lanes store neighbouring floats); 0: dW itself, [cout][cig][kh*kw]
  int nacc;              // accumulators per CTA (strip arrangement: 1 or 2 channel blocks sharing the dY operand)
  int xr;                // rows staged per input block: XR (strip with tap margin) or KP (exact blocks)
  int blocks_are_taps;   // xblocks == 4: block j is tap kx = j of one channel block (strided filters) rather than
                         // channel block j of a 1x1 filter
  int sph, spw;          // stride: grid pixel (r, c) of phase (a, b) is the input pixel (r*sph + a, c*spw + b)
  int in_h, in_w, out_h, out_w;  // extents of x and of dY (the grid H x W covers both)
  unsigned blk_b[2], blk_dc[2];  // per tap kx (up to 8): column phase and whole-pixel column offset (signed), 8 bits each
  int kx_groups;                 // filters wider than four taps take ceil(kw / 4) CTAs, four taps each
  int ci_tiles, co_tiles;
  int stages;
  int chunk_kb;          // K blocks accumulated in tensor memory before the sum is folded into `out` (see CHUNK_KB)
  int* status;
  unsigned long long* prof;  // optional cycle counters of CTA (0,0) (B200_STRIP_PROFILE=1), else null
};

// role cycle probes: compiled in only with -DB200_ROLE_PROFILE=1 (see conv_tc_strip.cu)
#ifndef B200_ROLE_PROFILE
#define B200_ROLE_PROFILE 0
#endif
#define DPROF_ON(leader) (B200_ROLE_PROFILE && a.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (leader))
#define DPROF_T0(on) const long long prof_t0__ = (on) ? clock64() : 0
#define DPROF_ADD(on, slot) do { if (on) atomicAdd(a.prof + (slot), (unsigned long long)(clock64() - prof_t0__)); } while (0)

struct Ctrl {
  unsigned long long full[MAX_STAGES], empty[MAX_STAGES], accum[2], drained[2];
  uint32_t tmem_base;
  int abort_flag;
};

// byte offset of channel e (0..31) of row `row` in a plane using the 128B swizzle with 32-byte base
__device__ __forceinline__ uint32_t sw32b_offset(int row, int e) {
  return (uint32_t)(row * 128 + ((((e >> 3) ^ (row & 3)) << 5) | ((e & 7) << 2)));
}
// MN-major operand descriptor: blocks of 32 channels `lbo` bytes apart, 4-row groups 512 bytes apart
__device__ __forceinline__ uint64_t make_mn_desc(uint32_t addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(512u >> 4) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version of sm_100
  d |= (uint64_t)1 << 61;   // SWIZZLE_128B with 32-byte base
  return d;
}

// byte offset of channel e (0..31) of row `row` in a bf16 plane of 64-byte rows, SWIZZLE_64B
__device__ __forceinline__ uint32_t sw64_offset(int row, int e) {
  return (uint32_t)(row * 64 + ((((e >> 3) ^ ((row >> 1) & 3)) << 4) | ((e & 7) << 1)));
}
// MN-major descriptor of a bf16 plane (64-byte rows): blocks of 32 channels `lbo` bytes apart, 8-row
// groups 512 bytes apart, SWIZZLE_64B
__device__ __forceinline__ uint64_t make_mn_desc16(uint32_t addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(512u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;   // SWIZZLE_64B
  return d;
}

// One warp stages `rows` (<= 32, lane = row) x 32 channels of a pixel-major block: gather from
// the strided view, split into TF32 hi/lo, swizzled stores.  `q_first` is the padded pixel of row 0;
// rows outside [q_lo, q_hi) or on padding are written as zeros.
//
// With the 32-byte-base swizzle rows r and r+4 put the same 16-byte chunk into the same banks, so
// lanes 4-7 of every group of eight write the two chunks of a 32-byte pair in the opposite order
// (every 8-lane store wavefront is then conflict-free).  To keep that free of per-value selects the
// swapped lanes already LOAD their channels in swapped order: val[j] holds channel j ^ 4 there.
__device__ __forceinline__ bool stage_block(const View4& v, long long chan0, int chans, int H, int W, int row_pitch,
                                            int img_pitch, const FastDiv& img_div, const FastDiv& row_div, int q_first,
                                            int q_lo, int q_hi, int rows, int lane, bool vec_ok, float (&val)[32],
                                            int sph = 1, int spw = 1, int pa = 0, int pb = 0, int lim_h = 1 << 30,
                                            int lim_w = 1 << 30) {
  const int q = q_first + lane;
  bool ok = lane < rows && q >= q_lo && q < q_hi;
  const float* src = v.ptr;
  if (ok) {
    const int n = (int)img_div.div((uint32_t)q);
    const int rem = q - n * img_pitch;
    const int y = (int)row_div.div((uint32_t)rem), x = rem - y * row_pitch;
    const int ty = y * sph + pa, tx = x * spw + pb;  // position in the tensor
    ok = y < H && x < W && ty < lim_h && tx < lim_w;
    src += n * v.s0 + chan0 * v.s1 + (long long)ty * v.s2 + (long long)tx * v.s3;
  }
  const int sw = (lane >> 2) & 1;
  if (vec_ok && chans == 32) {
    // Channels-last: eight lanes fetch the 128 contiguous bytes of one pixel, four pixels per load
    // instruction; lane r computed the address of row r above and hands it to the lanes that fetch
    // it.  val[4i..4i+3] is then the 16-byte chunk (lane & 7) of row 4i + (lane >> 3): see
    // store_block_chunks.
    const unsigned long long mine = ok ? reinterpret_cast<unsigned long long>(src) : 0ull;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4* ps = reinterpret_cast<const float4*>(__shfl_sync(0xffffffffu, mine, 4 * i + (lane >> 3)));
      const float4 f = ps ? __ldg(ps + (lane & 7)) : make_float4(0.f, 0.f, 0.f, 0.f);
      val[4 * i] = f.x; val[4 * i + 1] = f.y; val[4 * i + 2] = f.z; val[4 * i + 3] = f.w;
    }
    return true;
  } else if (chans == 32) {
    // lane = pixel, one coalesced load per channel; 32-bit element offsets (the host checks that the
    // tensor is addressable with them) keep this at two instructions per value
    const int s1 = (int)v.s1;
    const float* pa = src + 4 * sw * s1;  // for j with bit 2 clear
    const float* pb = src - 4 * sw * s1;  // for j with bit 2 set
    if (__all_sync(0xffffffffu, ok)) {  // the common case away from padding: no predication
#pragma unroll
      for (int j = 0; j < 32; ++j) val[j] = __ldg(((j & 4) ? pb : pa) + j * s1);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) val[j] = ok ? __ldg(((j & 4) ? pb : pa) + j * s1) : 0.f;
    }
  } else {
    const int s1 = (int)v.s1;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int c = j ^ (sw << 2);
      val[j] = (ok && c < chans) ? __ldg(src + c * s1) : 0.f;
    }
  }
  return false;
}
// Where one staged block lives: the TF32 hi plane (128-byte rows) and either the FP32 lo plane or,
// with BF16 cross terms, the two bf16 planes (64-byte rows) of bf16(hi) and bf16(lo).
struct BlockPlanes {
  uint32_t hi, lo, h16, l16;
};
// Store for the channels-last load pattern: eight lanes write the eight 16-byte chunks of one row
// (a whole row per quarter warp: conflict-free in any swizzle).
template <bool DW_CROSS>
__device__ __forceinline__ void store_block_chunks(const float (&val)[32], int rows, int row0, const BlockPlanes& pl, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = 4 * i + (lane >> 3);
    if (r < rows) {
      float h[4], l[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) split_tf32_fast(val[4 * i + j], h[j], l[j]);
      const int c4 = (lane & 7) * 4;
      sts_f32x4(pl.hi + sw32b_offset(row0 + r, c4), h[0], h[1], h[2], h[3]);
      if (DW_CROSS) {
        const uint32_t o = sw64_offset(row0 + r, c4);
        sts_b32x2(pl.h16 + o, pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]));
        sts_b32x2(pl.l16 + o, pack_bf16x2(l[0], l[1]), pack_bf16x2(l[2], l[3]));
      } else {
        sts_f32x4(pl.lo + sw32b_offset(row0 + r, c4), l[0], l[1], l[2], l[3]);
      }
    }
  }
}
// Store for the lane = row pattern; val[j] holds channel j ^ 4 in lanes 4-7 of every eight (see stage_block).
template <bool DW_CROSS>
__device__ __forceinline__ void store_block(const float (&val)[32], int rows, int row0, const BlockPlanes& pl, int lane) {
  if (lane >= rows) return;
  const uint32_t sw = (uint32_t)((lane >> 2) & 1);
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    float h0[4], l0[4], h1[4], l1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      split_tf32_fast(val[m * 8 + j], h0[j], l0[j]);
      split_tf32_fast(val[m * 8 + 4 + j], h1[j], l1[j]);
    }
    const uint32_t oa = sw32b_offset(row0 + lane, m * 8) ^ (sw << 4), ob = oa ^ 16u;
    sts_f32x4(pl.hi + oa, h0[0], h0[1], h0[2], h0[3]);
    sts_f32x4(pl.hi + ob, h1[0], h1[1], h1[2], h1[3]);
    if (DW_CROSS) {
      // the eight channels of this group are one 16-byte chunk of a bf16 row; its two 8-byte halves
      // go where this lane's channel order puts them (64-byte rows need no bank-conflict swap)
      const uint32_t qa = sw64_offset(row0 + lane, m * 8) ^ (sw << 3), qb = qa ^ 8u;
      sts_b32x2(pl.h16 + qa, pack_bf16x2(h0[0], h0[1]), pack_bf16x2(h0[2], h0[3]));
      sts_b32x2(pl.h16 + qb, pack_bf16x2(h1[0], h1[1]), pack_bf16x2(h1[2], h1[3]));
      sts_b32x2(pl.l16 + qa, pack_bf16x2(l0[0], l0[1]), pack_bf16x2(l0[2], l0[3]));
      sts_b32x2(pl.l16 + qb, pack_bf16x2(l1[0], l1[1]), pack_bf16x2(l1[2], l1[3]));
    } else {
      sts_f32x4(pl.lo + oa, l0[0], l0[1], l0[2], l0[3]);
      sts_f32x4(pl.lo + ob, l1[0], l1[1], l1[2], l1[3]);
    }
  }
}

struct FoldArgs {
  float* out;            // this thread's first output element
  long long cols;        // element stride between output channels
  uint32_t acc;          // tensor-memory address of this warp's accumulator rows (buffer 0)
  uint32_t acc_buffer_cols, nbuf;  // column distance between the two accumulator buffers; 1 or 2 buffers
  uint32_t accum_bar, drained_bar; // shared-memory addresses of accum[0] / drained[0] (buffer b: + 8 * b)
  int cols_valid;
  bool row_ok;
  int* abort_flag;
  int* status;
};

// Folds one warp's accumulator rows into `out` after chunk `c` of the reduction (see CHUNK_KB): the first chunk is
// stored, later ones are added to what the same thread stored before.  Out of line on purpose: it runs once per
// 2048 pixels, and inlined it costs the producers' loop registers (that loop runs at the 96-register limit of a
// 17-warp CTA).
template <int BN, bool FUSE_HILO>
__device__ __noinline__ bool fold_accumulator(FoldArgs f, int c, bool more) {
  // chunk c used accumulator buffer c % nbuf, for the (c / nbuf)-th time
  const uint32_t buf = f.nbuf == 2 ? (uint32_t)c & 1u : 0u, use = f.nbuf == 2 ? (uint32_t)c >> 1 : (uint32_t)c;
  if (!mbar_wait(f.accum_bar + 8u * buf, use & 1u, f.abort_flag, f.status, STATUS_TIMEOUT_ACCUM)) return false;
  tc_fence_after();
  const bool add = c > 0;
  f.acc += buf * f.acc_buffer_cols;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 32) {
    if (c0 >= f.cols_valid) break;
    float v[32];
    tmem_ld32(f.acc + (uint32_t)c0, v);
    if (FUSE_HILO) {
      float v2[32];
      tmem_ld32(f.acc + (uint32_t)(BN + c0), v2);
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += v2[j];
    }
    if (f.row_ok) {
      float* p = f.out + c0 * f.cols;
      const int nvalid = f.cols_valid - c0;
      if (add) {
        // Reductions without a return value: the thread does not wait for the old values, so the accumulator is
        // handed back after the tensor-memory reads alone.  Every address has exactly one writer (this thread,
        // in program order), so the sums are the same from run to run.
#pragma unroll
        for (int j = 0; j < 32; ++j, p += f.cols)
          if (j < nvalid) atomicAdd(p, v[j]);
      } else if (nvalid >= 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j, p += f.cols) *p = v[j];
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j, p += f.cols)
          if (j < nvalid) *p = v[j];
      }
    }
  }
  if (more) {  // the accumulator may be overwritten now
    tc_fence_before();
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(f.drained_bar + 8u * buf);
  }
  return true;
}

template <int BN, bool DW_CROSS>
__global__ void __launch_bounds__(THREADS, 1) dweight_strip_kernel(const DwStripArgs a) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned long long prof_start = a.prof ? global_ns() : 0;
  // the pass that sums the split partials may take its place on the SMs now (it waits for this grid to finish)
  if (a.partial_layout) asm volatile("griddepcontrol.launch_dependents;");
  const ConvGeom& g = a.g;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  constexpr int NB = BN / 32;                                  // dY blocks per stage
  const uint32_t x_plane = (uint32_t)a.xr * 128u, x_bytes = (uint32_t)(a.nacc * a.xblocks) * 2u * x_plane;
  constexpr uint32_t y_plane = NB * KP * 128u;                 // all dY blocks of one plane
  const uint32_t stage_bytes = x_bytes + 2u * y_plane;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + (base - raw) + a.stages * stage_bytes);
  volatile int* abort_flag = &ctrl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int x_halves = a.xr > 32 ? 2 : 1;                      // a strip = rows 0..31 and 32..47; an exact block = 32 rows
  const int kx0 = (int)(blockIdx.x % (unsigned)a.kx_groups) * 4;  // first horizontal tap of this CTA
  // taps beyond the filter width of a narrow filter are not staged (their accumulator rows are never
  // stored); the last group of a wide filter stages zeros for them so that every CTA has the same jobs
  const int x_tasks = a.nacc * (a.blocks_are_taps ? min(4, g.kw) : a.xblocks) * x_halves;
  const int tasks = x_tasks + NB;                              // warp-sized staging jobs per K block
  // BN <= 128: the dY hi and lo planes (their 32-channel blocks are equally spaced) form ONE operand
  // of 2*BN columns, so x_hi*[dy_hi | dy_lo] is a single MMA; the epilogue adds the two halves.
  constexpr bool FUSE_HILO = BN <= 128 && !DW_CROSS;
  constexpr uint32_t ACC_COLS = FUSE_HILO ? 2 * BN : BN;
  // Two accumulator buffers where tensor memory has room (512 columns): the MMA thread then moves on to the
  // other buffer at a chunk boundary while the epilogue warps fold the finished one, instead of waiting for them.
  const uint32_t acc_buffer_cols = ACC_COLS * (uint32_t)a.nacc;   // 64..512, a power of two
  const uint32_t nbuf = acc_buffer_cols <= 256 ? 2u : 1u;
  const uint32_t tmem_cols = acc_buffer_cols * nbuf;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), (uint32_t)tasks * 32u);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->accum[b]), 1);
      mbar_init(smem_u32(&ctrl->drained[b]), (uint32_t)(4 * a.nacc));  // one arrival per epilogue warp
    }
    ctrl->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == MMA_WARP) tmem_alloc(smem_u32(&ctrl->tmem_base), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);

  // ---- which piece of dW this CTA owns ----
  int id = blockIdx.x / a.kx_groups;
  const int ci_tile = id % a.ci_tiles; id /= a.ci_tiles;
  const int ky = id % g.kh;            id /= g.kh;
  const int co_tile = id % a.co_tiles; id /= a.co_tiles;
  const int group = id;
  const int split = blockIdx.y;
  const int ci_per_tile = a.blocks_are_taps ? 32 : a.nacc * a.xblocks * 32;
  const int ci0 = ci_tile * ci_per_tile, co0 = co_tile * BN;
  const int cols_valid = min(BN, g.cog - co0);
  const int row_pitch = a.W + a.pc;
  const int img_pitch = (a.H + a.pr) * row_pitch;
  const int k_begin = split * a.span;  // < q_total
  const int k_end = a.q_total - k_begin > a.span ? k_begin + a.span : a.q_total;
  const int kblocks = (k_end - k_begin + KP - 1) / KP;
  // vertical tap: input row sph*(r + dr) + pa
  const int oy = ky * g.dh - g.ph;
  const int dr = oy >= 0 ? oy / a.sph : -((-oy + a.sph - 1) / a.sph), pa = oy - dr * a.sph;
  const int yshift = dr * row_pitch;

  if (warp == MMA_WARP) {
    // The whole warp runs the loop and waits on the barriers; one elected lane issues the tcgen05 instructions.  With
    // uniform control flow the descriptors live in uniform registers, which is where tcgen05.mma reads its operands
    // (issued from one divergent thread, every operand crossed over from the vector registers first, and that
    // crossing, not the tensor pipe, paced the kernel).  Stage indices are counted and descriptors are base + offset.
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_tf32(128, BN) | (1u << 15) | (1u << 16);  // both operands MN-major
      constexpr uint32_t idesc_wide = make_idesc_tf32(128, FUSE_HILO ? 2 * BN : BN) | (1u << 15) | (1u << 16);
      const uint32_t a_lbo = a.xblocks == 1 ? (uint32_t)g.dw * 128u : 2u * x_plane;
      // input rows start at the pixel shifted by -pad_w; hi plane then lo plane of each block
      const uint64_t da_base = make_mn_desc(base + (a.xblocks == 1 ? (uint32_t)(XOFF - g.pw + kx0 * g.dw) * 128u : 0u), a_lbo);
      const uint64_t db_base = make_mn_desc(base + x_bytes, KP * 128u);
      const uint32_t stage_d = stage_bytes >> 4, x_plane_d = x_plane >> 4;
      constexpr uint32_t y_plane_d = y_plane >> 4;
      // BF16 cross terms: the second plane of every block is split into bf16(hi) and bf16(lo) halves
      // of 64-byte rows; x_hi16 pairs with dy_lo16 and x_lo16 with dy_hi16
      constexpr uint32_t idesc16 = make_idesc_bf16(128, BN) | (1u << 15) | (1u << 16);
      const uint32_t a_lbo16 = a.xblocks == 1 ? (uint32_t)g.dw * 64u : 2u * x_plane;
      const uint64_t da16_base = make_mn_desc16(base + x_plane + (a.xblocks == 1 ? (uint32_t)(XOFF - g.pw + kx0 * g.dw) * 64u : 0u), a_lbo16);
      const uint64_t db16_base = make_mn_desc16(base + x_bytes + y_plane, KP * 64u);
      const bool pm = DPROF_ON(lane == 0);
      uint32_t s = 0, par = 0;
      int kb_in_chunk = 0;
      uint32_t chunk = 0, buf = 0;
      for (int kb = 0; kb < kblocks; ++kb, ++kb_in_chunk) {
        if (kb_in_chunk == a.chunk_kb) {
          // chunk boundary: hand the accumulator to the epilogue warps; before the next buffer is overwritten its
          // previous chunk (nbuf chunks back) must have been read
          if (leader) umma_commit(smem_u32(&ctrl->accum[buf]));
          ++chunk;
          kb_in_chunk = 0;
          buf = nbuf == 2 ? chunk & 1u : 0u;
          if (chunk >= nbuf) {
            const uint32_t prev_use = (chunk - nbuf) / nbuf;
            if (!warp_wait(smem_u32(&ctrl->drained[buf]), prev_use & 1u, abort_flag, a.status, STATUS_TIMEOUT_ACCUM)) break;
            tc_fence_after();
          }
        }
        { DPROF_T0(pm);
        if (!warp_wait(smem_u32(&ctrl->full[s]), par, abort_flag, a.status, STATUS_TIMEOUT_FULL)) break;
        DPROF_ADD(pm, 0); }
        DPROF_T0(pm);
        const uint64_t da_hi = da_base + s * stage_d;
        const uint64_t db_hi = db_base + s * stage_d, db_lo = db_hi + y_plane_d;
        if (leader)
        for (int u = 0; u < a.nacc; ++u) {  // channel blocks that share this dY block
          const uint32_t acc = tmem_acc + buf * acc_buffer_cols + (uint32_t)u * ACC_COLS;
          const uint64_t ua_hi = da_hi + (uint64_t)u * (2 * x_plane_d), ua_lo = ua_hi + x_plane_d;
          if constexpr (DW_CROSS) {
#pragma unroll
            for (int kg = 0; kg < KP / 8; ++kg) umma_tf32(acc, ua_hi + kg * 64, db_hi + kg * 64, idesc, (kb_in_chunk | kg) != 0);
            const uint64_t a_h16 = da16_base + s * stage_d + (uint64_t)u * (2 * x_plane_d), a_l16 = a_h16 + (x_plane_d >> 1);
            const uint64_t b_l16 = db16_base + s * stage_d, b_h16 = b_l16 + (y_plane_d >> 1);
#pragma unroll
            for (int kg = 0; kg < KP / 16; ++kg) umma_bf16(acc, a_h16 + kg * 64, b_l16 + kg * 64, idesc16, 1);  // 16 rows of 64 bytes
#pragma unroll
            for (int kg = 0; kg < KP / 16; ++kg) umma_bf16(acc, a_l16 + kg * 64, b_h16 + kg * 64, idesc16, 1);
          } else {
#pragma unroll
            for (int kg = 0; kg < KP / 8; ++kg) {  // 8 pixels = 8 rows of 128 bytes per MMA
              if (FUSE_HILO) {
                umma_tf32(acc, ua_hi + kg * 64, db_hi + kg * 64, idesc_wide, (kb_in_chunk | kg) != 0);
                umma_tf32(acc, ua_lo + kg * 64, db_hi + kg * 64, idesc, 1);
              } else {
                umma_tf32(acc, ua_lo + kg * 64, db_hi + kg * 64, idesc, (kb_in_chunk | kg) != 0);
                umma_tf32(acc, ua_hi + kg * 64, db_lo + kg * 64, idesc, 1);
                umma_tf32(acc, ua_hi + kg * 64, db_hi + kg * 64, idesc, 1);
              }
            }
          }
        }
        if (leader) umma_commit(smem_u32(&ctrl->empty[s]));
        if (++s == (uint32_t)a.stages) { s = 0; par ^= 1; }
        DPROF_ADD(pm, 1);
      }
      if (leader) umma_commit(smem_u32(&ctrl->accum[buf]));
    }
  } else {
    // ---- producers: job j of K block kb goes to warp (kb*tasks + j) % 16 ----
    const bool x_vec = a.x.s1 == 1 && ((reinterpret_cast<uintptr_t>(a.x.ptr) & 15) == 0) && a.x.s0 % 4 == 0 &&
                       a.x.s2 % 4 == 0 && a.x.s3 % 4 == 0;
    const bool y_vec = a.dy.s1 == 1 && ((reinterpret_cast<uintptr_t>(a.dy.ptr) & 15) == 0) && a.dy.s0 % 4 == 0 &&
                       a.dy.s2 % 4 == 0 && a.dy.s3 % 4 == 0;
    const int total_jobs = kblocks * tasks;  // kblocks <= 2^26, tasks <= 16
    // ---- folding the accumulator into `out` (warps 0 .. 4*nacc-1): lane = row of the accumulator = (block, channel) ----
    // Chunk c of the reduction is complete when the MMA thread's commit flips `accum` for the c-th time.  The first
    // chunk is stored, later ones are added to what this CTA stored before (same thread, same addresses: program order).
    const int chunks_total = (kblocks + a.chunk_kb - 1) / a.chunk_kb;
    const bool drains = warp < 4 * a.nacc;
    // what the fold needs, as plain values (the call is out of line: see fold_accumulator)
    FoldArgs fa;
    {
      const int taps = g.kh * g.kw;
      const int quarter = warp & 3, u = warp >> 2;
      // block index: horizontal tap (taps in M) or channel block (1x1 filter in the block arrangement)
      const bool taps_in_m = a.xblocks == 1 || a.blocks_are_taps;
      const int kx = taps_in_m ? kx0 + quarter : 0;
      const int ci = ci0 + u * 32 + (taps_in_m ? lane : quarter * 32 + lane);
      fa.cols = (long long)g.cig * taps;
      fa.row_ok = kx < g.kw && ci < g.cig;
      fa.out = a.out + ((long long)split * g.cout + (long long)group * g.cog + co0) * fa.cols +
               (a.partial_layout ? (long long)(ky * g.kw + kx) * g.cig + ci : (long long)ci * taps + ky * g.kw + kx);
      fa.acc = tmem_acc + (uint32_t)u * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      fa.cols_valid = cols_valid;
      fa.acc_buffer_cols = acc_buffer_cols;
      fa.nbuf = nbuf;
      fa.accum_bar = smem_u32(&ctrl->accum[0]);
      fa.drained_bar = smem_u32(&ctrl->drained[0]);
      fa.abort_flag = &ctrl->abort_flag;
      fa.status = a.status;
    }
    auto drain = [&](int c) -> bool { return fold_accumulator<BN, FUSE_HILO>(fa, c, c + (int)nbuf < chunks_total); };
    // consecutive jobs of a warp stay within `stages` K blocks of each other (a waiter that skipped
    // a whole phase of a stage's mbarrier would see the parity of an older phase and run ahead)
    const int warps_active = min(PRODUCER_WARPS, tasks * a.stages);
    const bool produces = warp < warps_active;
    bool alive = true;
    int job = warp;
    // chunk by chunk: this warp's staging jobs of the chunk (the inner loop is the hot one), then, for an
    // epilogue warp, the fold of that chunk -- so a warp never stages blocks of a later chunk before it has
    // folded the earlier one, and the MMA thread never waits for a fold that waits for this warp's blocks
    for (int chunk = 0; chunk < chunks_total && alive; ++chunk) {
    // ... except for the first `stages` K blocks of the next chunk, which it stages BEFORE folding: their slots
    // were last used by blocks of this chunk, so staging them depends on nothing the fold waits for, and the
    // MMA thread finds a full pipeline when the fold hands the accumulator back
    const int job_end = chunk + 1 < chunks_total ? min(total_jobs, ((chunk + 1) * a.chunk_kb + a.stages) * tasks) : total_jobs;
    for (; produces && job < job_end && alive; job += warps_active) {
      const int kb = (int)a.div_tasks.div((uint32_t)job), j = job - kb * tasks;
      const uint32_t round = a.div_stages.div((uint32_t)kb);
      const int s = kb - (int)round * a.stages;
      const int k0 = k_begin + kb * KP;
      const uint32_t xs = base + s * stage_bytes, ys = xs + x_bytes;
      float val[32];
      bool chunked;  // which register pattern stage_block used
      int rows, row0;
      BlockPlanes pl;
      const bool pp = DPROF_ON(threadIdx.x == 0);
      DPROF_T0(pp);
      if (j < x_tasks) {
        const int blk = x_halves == 2 ? j >> 1 : j, half = x_halves == 2 ? j & 1 : 0;
        rows = half ? XR - 32 : 32;
        row0 = half * 32;
        pl.hi = xs + (uint32_t)blk * 2u * x_plane;
        pl.lo = pl.hi + x_plane;
        pl.h16 = pl.lo;
        pl.l16 = pl.lo + x_plane / 2;
        if (a.xblocks == 1) {
          // one strip; the horizontal taps are its row offsets.  The input is needed wherever it
          // exists: no split-range clipping, only image bounds
          const int c0 = ci0 + blk * 32;  // strip blk of this CTA
          const int chans = max(0, min(32, g.cig - c0));
          chunked = stage_block(a.x, (long long)group * g.cig + c0, chans, a.H, a.W, row_pitch, img_pitch, a.img_div, a.row_div,
                      k0 + yshift - XOFF + row0, 0, a.q_total, rows, lane, x_vec, val);
        } else {
          // exact 32-pixel blocks: tap kx = blk of one channel block, or channel block blk of a 1x1 filter
          const int c0 = ci0 + (a.blocks_are_taps ? 0 : blk * 32);
          const int kx = kx0 + blk;  // tap of this block (blocks_are_taps)
          const int chans = (a.blocks_are_taps && kx >= g.kw) ? 0 : max(0, min(32, g.cig - c0));
          const unsigned tb = kx < 4 ? a.blk_b[0] >> (8 * kx) : a.blk_b[1] >> (8 * (kx - 4));
          const unsigned td = kx < 4 ? a.blk_dc[0] >> (8 * kx) : a.blk_dc[1] >> (8 * (kx - 4));
          const int pb = a.blocks_are_taps ? (int)(tb & 0xFFu) : 0;
          const int dc = a.blocks_are_taps ? (int)(signed char)(td & 0xFFu) : 0;
          chunked = stage_block(a.x, (long long)group * g.cig + c0, chans, a.H, a.W, row_pitch, img_pitch, a.img_div, a.row_div,
                      k0 + yshift + dc, 0, a.q_total, rows, lane, x_vec, val, a.sph, a.spw, pa, pb, a.in_h, a.in_w);
        }
      } else {
        const int blk = j - x_tasks;
        rows = 32;
        row0 = blk * KP;
        pl.hi = ys;
        pl.lo = ys + y_plane;
        pl.l16 = pl.lo;                 // [bf16(lo) blocks][bf16(hi) blocks]: x_hi16 meets dy_lo16
        pl.h16 = pl.lo + y_plane / 2;
        const int c0 = co0 + blk * 32;
        const int chans = max(0, min(32, g.cog - c0));
        // dY outside this split's pixel range must read as zero so that splits do not overlap
        chunked = stage_block(a.dy, (long long)group * g.cog + c0, chans, a.H, a.W, row_pitch, img_pitch, a.img_div, a.row_div,
                    k0, k_begin, k_end, rows, lane, y_vec, val, 1, 1, 0, 0, a.out_h, a.out_w);
      }
      DPROF_ADD(pp, 2);
      { const long long tw = pp ? clock64() : 0;
      if (!mbar_wait(smem_u32(&ctrl->empty[s]), (round & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_EMPTY)) { alive = false; break; }
      if (pp) atomicAdd(a.prof + 3, (unsigned long long)(clock64() - tw)); }
      { const long long tw = pp ? clock64() : 0;
      if (chunked) store_block_chunks<DW_CROSS>(val, rows, row0, pl, lane);
      else store_block<DW_CROSS>(val, rows, row0, pl, lane);
      fence_proxy_async();
      mbar_arrive(smem_u32(&ctrl->full[s]));
      if (pp) { atomicAdd(a.prof + 4, (unsigned long long)(clock64() - tw)); atomicAdd(a.prof + 5, 1ull); } }
    }
    if (drains && alive) {
      const bool pe = DPROF_ON(threadIdx.x == 0);
      DPROF_T0(pe);
      alive = drain(chunk);
      DPROF_ADD(pe, 7);
      if (pe) atomicAdd(a.prof + 8, 1ull);
    }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, tmem_cols);
  }
  if (a.prof && threadIdx.x == 0) {  // spread of CTA start times and lifetimes (ns)
    const unsigned long long now = global_ns();
    atomicMin(a.prof + 11, prof_start);
    atomicMax(a.prof + 12, prof_start);
    atomicMax(a.prof + 13, now);
    atomicMin(a.prof + 14, now - prof_start);
    atomicMax(a.prof + 15, now - prof_start);
  }
}

// Sum the split partials [split][cout][taps][cig] in ascending split order (run-to-run identical)
// and write dW[cout][cig][taps].  Threads follow the partial layout, so the reads, which are
// `splits` times the writes, are coalesced.
__global__ void __launch_bounds__(256) finalize_partials_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                                               long long count, int splits, int cig, int taps) {
  // launched with programmatic stream serialisation behind the kernel that writes the partials: its blocks may be
  // resident before that kernel has finished, and wait here until it has (and its stores are visible)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= count) return;
  float sum = 0.f;
  for (int s = 0; s < splits; ++s) sum += partial[(long long)s * count + i];
  const int ci = (int)(i % cig);
  const int tap = (int)((i / cig) % taps);
  const long long co = i / ((long long)cig * taps);
  dw[(co * cig + ci) * taps + tap] = sum;
}

struct DwStripPlan {
  bool ok = false;
  bool cross = false;  // BF16 cross terms (four accumulators)
  int bn = 0, xblocks = 1, nacc = 1, xr = XR, blocks_are_taps = 0, stages = 0, smem = 0, ci_tiles = 0, co_tiles = 0, splits = 1, span = 0;
  int gh = 0, gw = 0, pr = 0, pc = 0;  // pixel grid (covers dY and every phase sub-image of x) and its zero padding
  unsigned blk_b[2] = {0, 0}, blk_dc[2] = {0, 0};
  int kx_groups = 1;
  size_t bytes = 0;
};

static inline int floor_div(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }

// Two arrangements of the M dimension (4 blocks of 32 rows):
//   strip:  stride 1, output as large as the input, kw >= 2 (or few channels): one staged input
//           strip per K block, the horizontal taps are its row offsets;
//   blocks: everything else -- strides, any padding, 1x1: four exact 32-pixel blocks per K
//           block, either the taps kx = 0..3 of one channel block (each with its own column phase and
//           offset) or, for a 1x1 filter, four channel blocks.
static DwStripPlan plan_dw_strip(const ConvGeom& g, size_t budget) {
  DwStripPlan p;
  if (g.kw > 8 || g.cog < 16 || g.cig < 16) return p;
  p.kx_groups = (g.kw + 3) / 4;
  const bool same = g.sh == 1 && g.sw == 1 && g.oh == g.h && g.ow == g.w && 2 * g.ph == g.dh * (g.kh - 1) &&
                    2 * g.pw == g.dw * (g.kw - 1);
  // the last row a VALID tap's M block reads must be inside the strip (the unused blocks of the last
  // tap group read whatever follows in the stage; their accumulator rows are never stored)
  const bool strip_fits = same && g.pw <= XOFF && (g.kw - 1) * g.dw - g.pw + XOFF + KP <= XR;
  const bool pointwise = same && g.kh == 1 && g.kw == 1;
  if (strip_fits && !(pointwise && g.cig >= 64)) {
    p.xblocks = 1; p.xr = XR;
    p.gh = g.h; p.gw = g.w; p.pr = g.ph; p.pc = g.pw;
  } else {
    if (g.sh > 255 || g.sw > 255) return p;
    p.xblocks = 4; p.xr = KP;
    p.blocks_are_taps = pointwise ? 0 : 1;
    p.gh = std::max(g.oh, (g.h + g.sh - 1) / g.sh);
    p.gw = std::max(g.ow, (g.w + g.sw - 1) / g.sw);
    for (int ky = 0; ky < g.kh; ++ky) p.pr = std::max(p.pr, std::abs(floor_div(ky * g.dh - g.ph, g.sh)));
    for (int kx = 0; kx < g.kw; ++kx) {
      const int ox = kx * g.dw - g.pw, dc = floor_div(ox, g.sw);
      if (dc < -127 || dc > 127) return p;
      p.pc = std::max(p.pc, std::abs(dc));
      p.blk_b[kx / 4] |= (unsigned)(ox - dc * g.sw) << (8 * (kx % 4));
      p.blk_dc[kx / 4] |= ((unsigned)dc & 0xFFu) << (8 * (kx % 4));
    }
  }
  // Several channel blocks per CTA share every staged dY block (one TMEM accumulator each): less dY
  // staging per MMA.  The column tile then stays at 128 (TMEM holds 512 columns).
  if (p.xblocks == 1 && g.cig >= 64) {
    p.cross = g.cig >= 128 || getenv("B200_DW_FORCE_CROSS") != nullptr;
    p.nacc = p.cross && g.cig > 64 ? 4 : 2;
    p.bn = g.cog <= 64 ? 64 : 128;
  } else {
    p.bn = g.cog <= 64 ? 64 : (g.cog <= 128 ? 128 : 256);
  }
  const int y_stage = 2 * (p.bn / 32) * KP * 128;
  const int stage = p.nacc * p.xblocks * 2 * p.xr * 128 + y_stage;
  p.stages = std::min(MAX_STAGES, SMEM_LIMIT / stage);
  if (p.stages < 2) return p;
  p.smem = p.stages * stage + 1024 + (int)sizeof(Ctrl) + 64;
  const int ci_per_tile = p.blocks_are_taps ? 32 : p.nacc * p.xblocks * 32;
  p.ci_tiles = (g.cig + ci_per_tile - 1) / ci_per_tile;
  p.co_tiles = (g.cog + p.bn - 1) / p.bn;
  const long long q_total = (long long)g.n * (p.gh + p.pr) * (p.gw + p.pc);
  const long long tiles = (long long)p.ci_tiles * g.kh * p.kx_groups * p.co_tiles * g.groups;
  const size_t dw_bytes = sizeof(float) * (size_t)g.cout * g.cig * g.kh * g.kw;
  // Number of pixel splits: the one that minimises a small model of the run time in K-block units --
  // waves of CTAs (one CTA per SM is resident) x (K blocks per split + a fixed cost per CTA for
  // pipeline fill and the epilogue) + the finalize pass over the partials.  Every split at least 16
  // K blocks long; partials within budget.
  const long long kblocks_total = div_up64(q_total, KP);
  long long most = std::max<long long>(1, kblocks_total / 16);
  most = std::min<long long>(most, 65535);
  most = std::min<long long>(most, (long long)(budget / dw_bytes));
  most = std::min<long long>(most, 4ll * sm_count() / tiles + 1);
  const double cta_fixed = 10.0, finalize_per_split = (double)dw_bytes / 3.3e6;  // ~3 TB/s against ~1.1 us per K block
  long long want = 1;
  double best = 0.0;
  for (long long sp = 1; sp <= std::max<long long>(1, most); ++sp) {
    const double waves = (double)div_up64(tiles * sp, sm_count());
    const double cost = waves * ((double)div_up64(kblocks_total, sp) + cta_fixed) + (sp > 1 ? finalize_per_split * (double)sp : 0.0);
    if (sp == 1 || cost < best) { best = cost; want = sp; }
  }
  long long span = div_up64(q_total, KP) * KP, splits = 1;
  if (want >= 2) {
    span = div_up64(div_up64(q_total, want), KP) * KP;
    splits = div_up64(q_total, span);
  }
  if (q_total > 2147483647ll - (1 << 20)) return p;  // pixel indices are 32-bit in the kernel
  p.splits = (int)splits;
  p.span = (int)span;
  p.bytes = splits > 1 ? (size_t)splits * dw_bytes : 0;
  p.ok = true;
  return p;
}

}  // namespace tcdw

bool dweight_strip_supported(const ConvGeom& g) { return tcdw::plan_dw_strip(g, 0).ok; }
size_t dweight_strip_workspace(const ConvGeom& g, size_t budget) { return tcdw::plan_dw_strip(g, budget).bytes; }

template <int BN, bool CROSS>
static int launch_dw_strip(const tcdw::DwStripArgs& a, dim3 grid, int smem, cudaStream_t st) {
  // opt in once (thread-safe) to the full 227 KB of dynamic shared memory for this instantiation
  static std::once_flag once;
  static cudaError_t opt_in = cudaSuccess;
  std::call_once(once, [] { opt_in = cudaFuncSetAttribute(tcdw::dweight_strip_kernel<BN, CROSS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448); });
  B200_CUDA(opt_in);
  tcdw::dweight_strip_kernel<BN, CROSS><<<grid, tcdw::THREADS, smem, st>>>(a);
  count_launch();
  return launch_check("dweight_strip_kernel");
}

int dweight_strip(const ConvGeom& g, View4 x, View4 dy, float* dw, void* ws, size_t ws_bytes, cudaStream_t st) {
  using namespace tcdw;
  const DwStripPlan plan = plan_dw_strip(g, ws ? ws_bytes : 0);
  if (!plan.ok) return fail(B200_EUNSUPPORTED, "dWeight strip kernel does not take this geometry");
  // the kernel forms element offsets inside a tensor in 32 bits
  auto span = [](const View4& v, long long n, long long c, long long h, long long w) {
    return (n - 1) * std::llabs(v.s0) + (c - 1) * std::llabs(v.s1) + (h - 1) * std::llabs(v.s2) + (w - 1) * std::llabs(v.s3);
  };
  if (span(x, g.n, g.cin, g.h, g.w) > 2147483647ll - 64 * std::llabs(x.s1) || span(dy, g.n, g.cout, g.oh, g.ow) > 2147483647ll - 64 * std::llabs(dy.s1))
    return fail(B200_EUNSUPPORTED, "dWeight strip kernel: tensor too large for 32-bit element offsets");
  DwStripArgs a{};
  a.g = g; a.x = x; a.dy = dy;
  a.H = plan.gh; a.W = plan.gw; a.pr = plan.pr; a.pc = plan.pc;
  a.xr = plan.xr; a.blocks_are_taps = plan.blocks_are_taps; a.nacc = plan.nacc;
  a.sph = g.sh; a.spw = g.sw; a.in_h = g.h; a.in_w = g.w; a.out_h = g.oh; a.out_w = g.ow;
  a.blk_b[0] = plan.blk_b[0]; a.blk_b[1] = plan.blk_b[1]; a.blk_dc[0] = plan.blk_dc[0]; a.blk_dc[1] = plan.blk_dc[1];
  a.kx_groups = plan.kx_groups;
  a.q_total = (int)((long long)g.n * (a.H + a.pr) * (a.W + a.pc));
  a.img_div = FastDiv((uint32_t)((a.H + a.pr) * (a.W + a.pc)));
  a.row_div = FastDiv((uint32_t)(a.W + a.pc));
  a.span = plan.span; a.splits = plan.splits; a.xblocks = plan.xblocks;
  a.ci_tiles = plan.ci_tiles; a.co_tiles = plan.co_tiles; a.stages = plan.stages;
  {  // equal chunks of at most CHUNK_KB K blocks per CTA (a CTA reduces span / KP of them)
    int limit = CHUNK_KB;
    if (const char* e = getenv("B200_DW_CHUNK_KB")) limit = std::max(1, atoi(e));  // testing aid: chain length in K blocks
    const int kblocks = plan.span / KP;
    const int chunks = (kblocks + limit - 1) / limit;
    a.chunk_kb = std::max(1, (kblocks + chunks - 1) / std::max(1, chunks));
  }
  a.div_tasks = FastDiv((uint32_t)(plan.nacc * (plan.blocks_are_taps ? std::min(4, g.kw) : plan.xblocks) * (plan.xr > 32 ? 2 : 1) + plan.bn / 32));
  a.div_stages = FastDiv((uint32_t)plan.stages);
  a.out = plan.splits > 1 ? (float*)ws : dw;
  a.partial_layout = plan.splits > 1 ? 1 : 0;
  a.status = device_status_word();
  if (!a.status) return fail(B200_ECUDA, "device status word is not allocated");
  const long long gx = (long long)plan.ci_tiles * g.kh * plan.kx_groups * plan.co_tiles * g.groups;
  if (gx > 2147483647ll) return fail(B200_ERANGE, "dWeight strip kernel: grid exceeds launch limits");
  // rows of dW that no CTA writes (channel blocks beyond kw taps) do not exist: every (co, ci, ky, kx)
  // is covered: four taps per CTA, ceil(kw / 4) tap groups, and all ci tiles are enumerated
  const dim3 grid((unsigned)gx, (unsigned)plan.splits);
  static unsigned long long* prof_buf = nullptr;
  const char* prof_env = getenv("B200_STRIP_PROFILE");
  const bool profiling = B200_ROLE_PROFILE && prof_env && prof_env[0] == '1';
  if (profiling) {
    if (!prof_buf) B200_CUDA(cudaMalloc(&prof_buf, 16 * sizeof(unsigned long long)));
    B200_CUDA(cudaMemsetAsync(prof_buf, 0, 16 * sizeof(unsigned long long), st));
    B200_CUDA(cudaMemsetAsync(prof_buf + 11, 0xFF, sizeof(unsigned long long), st));
    B200_CUDA(cudaMemsetAsync(prof_buf + 14, 0xFF, sizeof(unsigned long long), st));
    a.prof = prof_buf;
  }
  int rc = plan.cross ? (plan.bn == 64 ? launch_dw_strip<64, true>(a, grid, plan.smem, st) : launch_dw_strip<128, true>(a, grid, plan.smem, st))
         : plan.bn == 64 ? launch_dw_strip<64, false>(a, grid, plan.smem, st)
         : plan.bn == 128 ? launch_dw_strip<128, false>(a, grid, plan.smem, st) : launch_dw_strip<256, false>(a, grid, plan.smem, st);
  if (rc) return rc;
  if (profiling) {
    unsigned long long h[16];
    B200_CUDA(cudaStreamSynchronize(st));
    B200_CUDA(cudaMemcpy(h, prof_buf, sizeof h, cudaMemcpyDeviceToHost));
    fprintf(stderr, "[dweight strip profile, CTA 0, cycles] bn=%d xblocks=%d stages=%d grid=%lldx%d kblocks/cta=%d | mma: wait_full %llu issue %llu | "
            "warp 0: jobs %llu load %llu wait_empty %llu store %llu | folds: %llu, cycles in them %llu (of which waiting for the accumulator %llu) | ns: last CTA start %llu, first start to last end %llu, CTA lifetime min %llu max %llu\n",
            plan.bn, plan.xblocks, plan.stages, gx, plan.splits, plan.span / KP, h[0], h[1], h[5], h[2], h[3], h[4], h[8], h[7], h[6], h[12] - h[11], h[13] - h[11], h[14], h[15]);
  }
  if (plan.splits > 1) {
    const long long count = (long long)g.cout * g.cig * g.kh * g.kw;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)div_up64(count, 256)); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    if (!getenv("B200_DW_NO_PDL")) { cfg.attrs = &attr; cfg.numAttrs = 1; }
    B200_CUDA(cudaLaunchKernelEx(&cfg, finalize_partials_kernel, (const float*)ws, dw, count, plan.splits, g.cig, g.kh * g.kw));
    count_launch();
    return launch_check("finalize_partials_kernel");
  }
  return B200_OK;
}

}  // namespace b200
