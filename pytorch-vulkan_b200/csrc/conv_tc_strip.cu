// Persistent tcgen05 implicit-GEMM kernel for convolution forward and dInput (any stride, padding,
// dilation and grouping; reduction channels in blocks of 32), FP32 by split precision (one TF32 pass
// for hi x hi, one BF16 pass for the cross terms: tc_common.cuh).  The same kernel is
// the GEMM behind mm/addmm and the plane product of the Winograd path.
//
// Idea: the kh*kw filter taps of one 32-channel block all read the same activations, shifted by
// whole pixels.  The activations of a tile are therefore staged ONCE per channel block as a
// "strip" in shared memory -- one 128-byte row (32 channels, TF32 hi and lo planes) per pixel of
// a zero-padded pixel grid -- and every tap's tcgen05.mma reads that strip through a matrix
// descriptor whose start address is moved by `shift(tap)` rows.  (The 128-byte swizzle is a
// function of the absolute shared-memory address, so a descriptor may start at any row.)
// Compared with gathering an operand tile per tap this issues kh*kw times fewer global loads,
// TF32 splits and shared-memory stores, which is what lets the tensor pipe stay busy.
//
// Padded pixel grid: `pc` zero columns after every row and `pr` zero rows after every image,
// q = (n*(H+pr) + y)*(W+pc) + x.  A tap offset (dr, dc) is then the constant row shift
// dr*(W+pc) + dc for every pixel, and reads that leave the image land on zero rows of the strip.
// Accumulator rows that fall on padding (or outside a smaller output) are discarded.
//
// Strides: with stride s the taps are grouped by the phase (row mod s, column mod s) of the pixels
// they touch -- input phases in forward (channel blocks are enumerated per phase, each with its own
// taps), output phases in dInput (column tiles are enumerated per phase; all read one dY strip).
// See TapTable and plan_strip.
//
// CTA roles (448 threads, persistent over tiles of 128 grid pixels x BN output channels):
//   warps 0-3    epilogue: tcgen05.ld of a finished accumulator, bias, coalesced stores
//   warps 4-11   strip producers: gather from the caller's strided view, TF32 split, swizzled stores
//   warp 12      (one thread) weight stages: one bulk copy (cp.async.bulk -> mbarrier complete_tx)
//                of a pre-split, pre-swizzled image per stage; stage_weights_kernel writes the
//                images once per call
//   warp 13      TMEM allocation; one thread issues the tcgen05.mma stream
// The accumulator is double-buffered in TMEM, so the epilogue of tile i overlaps the main loop of
// tile i+1.  All hand-offs are mbarriers with bounded waits.
//
// Replaces csrc/shaders/conv2d_tiled_body.glsl:53-86 and
// csrc/shaders/conv2d_backward_input_tiled_body.glsl:49-93 of the reference.
#include <cuda_bf16.h>

#include "common.cuh"
#include "strip_plan.cuh"
#include "tc_common.cuh"

#include <algorithm>
#include <mutex>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace b200 {
namespace tcs {
using namespace tc;

constexpr int BLOCK_M = 128, KBLK = 32;
// Warp roles: 4 epilogue warps, AW strip producers, the weight-copy warp, the MMA warp.  AW is 8, or 16 for layers
// whose producers set the pace (one tap per staged strip: 1x1 filters): twice the loads in flight per SM.
constexpr int EPI_WARPS = 4, W_WARPS = 1;
constexpr int strip_threads(int aw) { return (EPI_WARPS + aw + W_WARPS + 1) * 32; }
constexpr int MAX_STAGES = 4;
constexpr int SMEM_LIMIT = 232448 - 2048;  // 227 KB per CTA minus the control block and alignment slack

struct StripArgs {
  ConvGeom g;
  View4 act;              // forward: x.  dInput: dy
  const float* wp;        // weight stage images [groups][tiles_n][phase][cblock][tap of phase] of BN*256 bytes
  const float* bias;
  long long bias_stride;
  float* out;             // contiguous NCHW [n][out_channels][out_h][out_w] (or row-major, see below)
  int H, W, pr, pc;       // pixel grid shared by the strip and the accumulator rows, and its zero padding
  int act_h, act_w;       // extent of the activation tensor; grid pixel (r, c) of phase (a, b) reads (r*sph + a, c*spw + b)
  int out_h, out_w;       // extent of the output tensor (grid pixels beyond it are discarded)
  int sph, spw;           // forward: phases live on the reduction side (channel block -> phase)
  int osh, osw;           // dInput: phases live on the output side: column tile -> phase (a, b), grid pixel (r, c)
                          // is the output pixel (r*osh + a, c*osw + b); all phases read the same dY strip
  int phase_on_n;         // 1 in the dInput arrangement
  int tiles_pp;           // column tiles per phase (dInput), else tiles_n
  int kc, nc, out_channels;
  // batched GEMM (groups used as the batch): extra element offsets per group on top of the grouped
  // convolution's own (group * kc channels in, group * nc columns out); 0 / out_channels / nc otherwise
  long long act_group_extra, out_pitch, out_group;
  int cb_per_phase;       // kc / 32
  int cblocks;            // strips per tile: forward n_phase * cb_per_phase, dInput cb_per_phase
  int images_per_tile;    // forward: weight stages per tile = cb_per_phase * taps_total
  int tiles_n;
  int q_total;            // grid pixels incl. padding (below 2^31 - 2^20)
  FastDiv img_div, row_div;
  int tiles_m, tiles_total;
  int unit, units;        // tiles per scheduling unit, number of units (tiles_total = unit * units)
  int m_fastest;          // tile order (tile_coord)
  FastDiv div_tiles_n, div_tiles_m, div_tiles_pp, div_chunks, div_cblocks, div_cbpp, div_a_stages, div_unit;
  int halo, strip_rows;   // rows staged before the tile's first pixel; strip_rows is a multiple of 8
  int a_stages, w_stages;
  int out_rowmajor;       // 0: NCHW planes.  1: [pixel][channel] rows (channels-last / GEMM C)
  int out_vec4;           // row-major rows may be written with 16-byte stores
  int wide_producers;     // 1: the kernel instance with sixteen producer warps
  float alpha, beta;      // out = alpha * acc + beta * bias
  View4 res;              // optional residual added after the bias (logical shape of the output), ptr null = none
  int relu;               // clamp at zero last
  int wait_for_images;    // launched with programmatic stream serialisation behind stage_weights_kernel
  int* status;
  unsigned long long* prof;  // optional cycle counters of CTA 0 (B200_STRIP_PROFILE=1), else null
  TapTable tt;
};

struct Ctrl {  // lives behind the operand stages in shared memory
  unsigned long long a_full[MAX_STAGES], a_empty[MAX_STAGES], w_full[MAX_STAGES], w_empty[MAX_STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int shift[MAX_TAPS];
  unsigned char ph_a[MAX_PHASES], ph_b[MAX_PHASES], tap_start[MAX_PHASES + 1];
};

// Cycle accounting for one thread of each role in CTA 0 (diagnostics only).  The probes sit in the
// issuing loops, where every extra instruction costs tensor time, so they are compiled in only with
// -DB200_ROLE_PROFILE=1 (then B200_STRIP_PROFILE=1 in the environment prints them).
#ifndef B200_ROLE_PROFILE
#define B200_ROLE_PROFILE 0
#endif
#define PROF_ON(leader) (B200_ROLE_PROFILE && a.prof != nullptr && blockIdx.x == 0 && (leader))
#define PROF_T0(on) const long long prof_t0__ = (on) ? clock64() : 0
#define PROF_ADD(on, slot) do { if (on) atomicAdd(a.prof + (slot), (unsigned long long)(clock64() - prof_t0__)); } while (0)

// Tiles are dealt to CTAs in units of `unit` consecutive tiles, unit u to CTA u mod gridDim.  At any
// moment the CTAs then work on neighbouring pixel rows (their strips share DRAM pages and L2 lines),
// and with unit = all column tiles of a pixel-row tile a strided dInput gives every CTA the same mix
// of output phases, whose tap counts differ.
struct TileIter {
  int u, t, unit, units, step;
  __device__ explicit TileIter(const StripArgs& a) : u(blockIdx.x), t(0), unit(a.unit), units(a.units), step(gridDim.x) {}
  __device__ bool valid() const { return u < units; }
  __device__ int tile() const { return u * unit + t; }
  __device__ void next() { if (++t == unit) { t = 0; u += step; } }
};

// tile index -> (pixel-row tile, column tile, group).  Column tile fastest when tiles are dealt in
// units (see TileIter); otherwise the pixel-row tile runs fastest, so that the CTAs working at the same
// time share their weight stages (the heavier operand: BN*256 bytes per stage against 16 KB of raw
// activations) and L2 serves them as one stream.
struct TileCoord {
  int m_tile, n_tile, group;
};
__device__ __forceinline__ TileCoord tile_coord(const StripArgs& a, int tile) {
  TileCoord c;
  if (a.m_fastest) {
    const int rest = (int)a.div_tiles_m.div((uint32_t)tile);
    c.m_tile = tile - rest * a.tiles_m;
    c.group = (int)a.div_tiles_n.div((uint32_t)rest);
    c.n_tile = rest - c.group * a.tiles_n;
  } else {
    const int tn = (int)a.div_tiles_n.div((uint32_t)tile);
    c.n_tile = tile - tn * a.tiles_n;
    c.group = (int)a.div_tiles_m.div((uint32_t)tn);
    c.m_tile = tn - c.group * a.tiles_m;
  }
  return c;
}

template <int BN, int AW>
__global__ void __launch_bounds__(strip_threads(AW), 1) conv_strip_kernel(const StripArgs a) {
  constexpr int A_WARPS = AW, MMA_WARP = EPI_WARPS + AW + W_WARPS;
  extern __shared__ unsigned char smem_raw[];
  const unsigned long long prof_start = a.prof ? global_ns() : 0;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  const uint32_t a_stage_bytes = (uint32_t)a.strip_rows * 256u, a_plane = (uint32_t)a.strip_rows * 128u;
  constexpr uint32_t w_stage_bytes = BN * 256u, w_plane = BN * 128u;
  const uint32_t w_base = tiles_base + a.a_stages * a_stage_bytes;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + (w_base - raw) + a.w_stages * w_stage_bytes);
  volatile int* abort_flag = &ctrl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // For BN <= 128 the weight stage's hi and lo planes (adjacent in shared memory) are fed to the
  // tensor core as ONE operand of 2*BN rows: a single MMA of width 2*BN yields a_hi*b_hi in columns
  // [0,BN) and a_hi*b_lo in [BN,2BN), a second one of width BN adds a_lo*b_hi to [0,BN); the epilogue
  // sums the two halves.  Two MMAs read 14/18 of the shared-memory bytes that three do.
  constexpr bool FUSE_HILO = BN <= 128 && !CROSS_BF16;
  constexpr uint32_t ACC_COLS = FUSE_HILO ? 2 * BN : BN;
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->a_full[s]), (uint32_t)((a.strip_rows + 31) / 32) * 32u);
      mbar_init(smem_u32(&ctrl->a_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ctrl->acc_full[s]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[s]), EPI_WARPS * 32);
    }
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->w_full[s]), 1);  // the issuing thread's arrive.expect_tx; the copy completes the bytes
      mbar_init(smem_u32(&ctrl->w_empty[s]), 1);
    }
    ctrl->abort_flag = 0;
    fence_barrier_init();
  }
  // the tap table moves to shared memory: kernel parameters are not indexed dynamically
  if (threadIdx.x < MAX_TAPS) ctrl->shift[threadIdx.x] = a.tt.shift[threadIdx.x];
  if (threadIdx.x < MAX_PHASES) { ctrl->ph_a[threadIdx.x] = a.tt.a[threadIdx.x]; ctrl->ph_b[threadIdx.x] = a.tt.b[threadIdx.x]; }
  if (threadIdx.x <= MAX_PHASES) ctrl->tap_start[threadIdx.x] = a.tt.start[threadIdx.x];
  if (warp == MMA_WARP) tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);

  const int row_pitch = a.W + a.pc;
  const int img_pitch = (a.H + a.pr) * row_pitch;

  if (warp == MMA_WARP) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp runs the loop and waits on the barriers; one elected lane issues the tcgen05 instructions.
    // With uniform control flow the descriptors live in uniform registers, which is where tcgen05.mma reads its
    // operands (issued from one divergent thread, every operand crossed over from the vector registers first, and
    // that crossing paced the kernel).  Stage indices and parities are counted, not divided, and descriptors are
    // the stage's base plus an offset.
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_tf32(BLOCK_M, BN);
      constexpr uint32_t idesc_wide = make_idesc_tf32(BLOCK_M, FUSE_HILO ? 2 * BN : BN);
      constexpr uint32_t idesc_cross = make_idesc_bf16(BLOCK_M, BN);
      const uint64_t da_base = make_kmajor_sw128_desc(tiles_base + (uint32_t)a.halo * 128u);
      const uint64_t db_base = make_kmajor_sw128_desc(w_base);
      const uint32_t a_stage_d = a_stage_bytes >> 4, a_plane_d = a_plane >> 4;
      constexpr uint32_t w_stage_d = w_stage_bytes >> 4, w_plane_d = w_plane >> 4;
      uint32_t as = 0, a_par = 0, ws = 0, w_par = 0, t_count = 0;
      const bool pm = PROF_ON(lane == 0);
      bool alive = true;
      for (TileIter it(a); it.valid() && alive; it.next(), ++t_count) {
        const int tile = it.tile();
        const uint32_t ab = t_count & 1;
        { PROF_T0(pm);
        if (!warp_wait(smem_u32(&ctrl->acc_empty[ab]), ((t_count >> 1) & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_ACCUM)) break;
        PROF_ADD(pm, 0); }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + ab * ACC_COLS;
        const int n_tile = tile_coord(a, tile).n_tile;
        int phase = a.phase_on_n ? (int)a.div_tiles_pp.div((uint32_t)n_tile) : 0;  // dInput: the phase of this column tile
        int cbl = 0;
        uint32_t accumulate = 0;  // the tile's first MMA overwrites the accumulator
        for (int cb = 0; cb < a.cblocks && alive; ++cb) {
          { PROF_T0(pm);
          if (!warp_wait(smem_u32(&ctrl->a_full[as]), a_par, abort_flag, a.status, STATUS_TIMEOUT_FULL)) { alive = false; break; }
          PROF_ADD(pm, 1); }
          const uint64_t da_strip = da_base + as * a_stage_d;
          const int tap_end = ctrl->tap_start[phase + 1];
          for (int tap = ctrl->tap_start[phase]; tap < tap_end; ++tap) {
            const int sh = ctrl->shift[tap];
            { PROF_T0(pm);
            if (!warp_wait(smem_u32(&ctrl->w_full[ws]), w_par, abort_flag, a.status, STATUS_TIMEOUT_FULL)) { alive = false; break; }
            PROF_ADD(pm, 2); }
            PROF_T0(pm);
            const uint64_t da_hi = da_strip + (uint64_t)(long long)(sh * 8), da_lo = da_hi + a_plane_d;
            const uint64_t db_hi = db_base + ws * w_stage_d, db_lo = db_hi + w_plane_d;
            const uint32_t first = accumulate;
            accumulate = 1;
            if (!leader) {
            } else if (CROSS_BF16) {  // hi x hi in TF32, then both cross terms as one BF16 product over the second planes
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_hi + 2 * kk, db_hi + 2 * kk, idesc, first | (uint32_t)(kk != 0));
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem_acc, da_lo + 2 * kk, db_lo + 2 * kk, idesc_cross, 1);
            } else if (FUSE_HILO) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_hi + 2 * kk, db_hi + 2 * kk, idesc_wide, first | (uint32_t)(kk != 0));
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_lo + 2 * kk, db_hi + 2 * kk, idesc, 1);
            } else {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_lo + 2 * kk, db_hi + 2 * kk, idesc, first | (uint32_t)(kk != 0));
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_hi + 2 * kk, db_lo + 2 * kk, idesc, 1);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) umma_tf32(tmem_acc, da_hi + 2 * kk, db_hi + 2 * kk, idesc, 1);
            }
            if (leader) umma_commit(smem_u32(&ctrl->w_empty[ws]));
            if (++ws == (uint32_t)a.w_stages) { ws = 0; w_par ^= 1; }
            PROF_ADD(pm, 3);
          }
          if (alive && leader) umma_commit(smem_u32(&ctrl->a_empty[as]));
          if (++as == (uint32_t)a.a_stages) { as = 0; a_par ^= 1; }
          if (!a.phase_on_n && ++cbl == a.cb_per_phase) { cbl = 0; ++phase; }
        }
        if (alive && leader) umma_commit(smem_u32(&ctrl->acc_full[ab]));
      }
    }
  } else if (warp == EPI_WARPS + A_WARPS) {
    // ------------------------------ weight stages ------------------------------
    // One thread: each stage is a single bulk copy of a ready-made (split, swizzled) image.
    if (lane == 0) {
      uint32_t ws = 0, w_par = 1, issued = 0;
      bool alive = true;
      const bool pw = PROF_ON(true);
      // The kernel may have started while the staging kernel ahead of it was still running: only
      // this thread reads what that kernel writes, so only it waits for that kernel to finish.
      if (a.wait_for_images) asm volatile("griddepcontrol.wait;" ::: "memory");
      for (TileIter it(a); it.valid() && alive; it.next()) {
        const int tile = it.tile();
        const TileCoord tc_ = tile_coord(a, tile);
        const int n_tile = tc_.n_tile;
        const long long group = tc_.group;
        long long first_image;
        int images;
        if (a.phase_on_n) {  // images of a group: [phase][tile of the phase][channel block][tap of the phase]
          const int phase = (int)a.div_tiles_pp.div((uint32_t)n_tile), in_phase = n_tile - phase * a.tiles_pp;
          const int t0 = ctrl->tap_start[phase], ntap = ctrl->tap_start[phase + 1] - t0;
          images = a.cb_per_phase * ntap;
          first_image = ((group * a.tt.taps_total + t0) * a.tiles_pp + (long long)in_phase * ntap) * a.cb_per_phase;
        } else {
          images = a.images_per_tile;
          first_image = (group * a.tiles_n + n_tile) * a.images_per_tile;
        }
        const float* img = a.wp + first_image * (long long)(BN * 64);
        for (int i = 0; i < images; ++i, img += BN * 64) {
          { PROF_T0(pw);
          if (!mbar_wait(smem_u32(&ctrl->w_empty[ws]), w_par, abort_flag, a.status, STATUS_TIMEOUT_EMPTY)) { alive = false; break; }
          PROF_ADD(pw, 4); }
          const uint32_t full = smem_u32(&ctrl->w_full[ws]);
          mbar_expect_tx(full, w_stage_bytes);
          bulk_g2s(w_base + ws * w_stage_bytes, img, w_stage_bytes, full);
          ++issued;
          if (++ws == (uint32_t)a.w_stages) { ws = 0; w_par ^= 1; }
        }
      }
      // After an abort the MMA thread no longer consumes stages: wait (bounded) for the copies still
      // in flight so that none lands in shared memory of a finished CTA.
      if (!alive)
        for (uint32_t j = issued > (uint32_t)a.w_stages ? issued - a.w_stages : 0; j < issued; ++j)
          mbar_wait(smem_u32(&ctrl->w_full[j % a.w_stages]), (j / a.w_stages) & 1, nullptr, a.status, STATUS_TIMEOUT_FULL);
    }
  } else if (warp >= EPI_WARPS) {
    // ------------------------------ strip producers ------------------------------
    // A stage is staged as chunks of 32 rows, one warp per chunk (lane = row); chunk c of stage n
    // goes to warp (n*chunks + c) % 8, so short strips (1x1 filters) keep several stages in flight.
    const int aw = warp - EPI_WARPS;
    const int chunks = (a.strip_rows + 31) / 32;
    const bool vec_layout = a.act.s1 == 1 && a.kc % 4 == 0 && ((reinterpret_cast<uintptr_t>(a.act.ptr) & 15) == 0) &&
                        (a.act.s0 % 4 == 0) && (a.act.s2 % 4 == 0) && (a.act.s3 % 4 == 0) && (a.act_group_extra % 4 == 0);
    const bool chunked_layout = vec_layout && a.act.s3 < 256;  // eight lanes per pixel (see below)
    const int s1 = (int)a.act.s1;
    const int my_units = a.units > (int)blockIdx.x ? (a.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int my_tiles = my_units * a.unit;
    const int total_jobs = my_tiles * a.cblocks * chunks;  // below 2^31 (checked by the host)
    // A warp's consecutive jobs must not be more than a_stages stages apart: a waiter that skips a
    // whole phase of a stage's mbarrier would see the parity of an older phase and run ahead.
    const int a_warps = min(A_WARPS, chunks * a.a_stages);
    for (int job = aw; job < total_jobs && aw < a_warps; job += a_warps) {
      const uint32_t a_count = a.div_chunks.div((uint32_t)job);
      const int chunk = job - (int)a_count * chunks;
      const uint32_t tile_iter = a.div_cblocks.div(a_count);
      const int cb = (int)(a_count - tile_iter * a.cblocks);
      const uint32_t unit_iter = a.div_unit.div(tile_iter);
      const uint32_t tile = (blockIdx.x + unit_iter * gridDim.x) * a.unit + (tile_iter - unit_iter * a.unit);
      const TileCoord tc_ = tile_coord(a, (int)tile);
      const int group = tc_.group, m_tile = tc_.m_tile;
      const uint32_t a_round = a.div_a_stages.div(a_count);
      const uint32_t as = a_count - a_round * a.a_stages;
      const bool pa = PROF_ON(threadIdx.x == EPI_WARPS * 32);
      PROF_T0(pa);
      const int r = chunk * 32 + lane;
      const int q = m_tile * BLOCK_M - a.halo + r;
      bool ok = r < a.strip_rows && q >= 0 && q < a.q_total;
      const float* src = a.act.ptr;
      const int phase = a.phase_on_n ? 0 : (int)a.div_cbpp.div((uint32_t)cb), cbl = cb - phase * a.cb_per_phase;
      // the last channel block of a group may be ragged (channel counts that are no multiple of 32):
      // it takes the masked one-value-per-load path, channels beyond the group read as zero
      const int nvalid = min(KBLK, a.kc - cbl * KBLK);
      const bool chunked = chunked_layout && nvalid == KBLK, vec_ok = vec_layout && nvalid == KBLK;
      if (ok) {
        const int n = (int)a.img_div.div((uint32_t)q);
        const int rem = q - n * img_pitch;
        const int y = (int)a.row_div.div((uint32_t)rem), x = rem - y * row_pitch;
        const int iy = a.phase_on_n ? y : y * a.sph + ctrl->ph_a[phase], ix = a.phase_on_n ? x : x * a.spw + ctrl->ph_b[phase];
        ok = y < a.H && x < a.W && iy < a.act_h && ix < a.act_w;
        src += n * a.act.s0 + ((long long)group * a.kc + cbl * KBLK) * a.act.s1 + (long long)iy * a.act.s2 + (long long)ix * a.act.s3 +
               (long long)group * a.act_group_extra;
      }
      float v[KBLK];
      if (chunked) {
        // Channels-last: the 32 channels of a pixel are 128 contiguous bytes.  Eight lanes fetch one
        // pixel (16 bytes each), so a load instruction covers four whole rows; lane r computed row r's
        // address above and hands it to the lanes that fetch it.
        const unsigned long long mine = ok ? reinterpret_cast<unsigned long long>(src) : 0ull;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4* ps = reinterpret_cast<const float4*>(__shfl_sync(0xffffffffu, mine, 4 * i + (lane >> 3)));
          const float4 f = ps ? __ldg(ps + (lane & 7)) : make_float4(0.f, 0.f, 0.f, 0.f);
          v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
      } else if (vec_ok) {
        // wide pixels (1 KB apart and more): measured faster with one pixel per lane
#pragma unroll
        for (int j = 0; j < KBLK / 4; ++j) {
          const float4 f = ok ? __ldg(reinterpret_cast<const float4*>(src) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
          v[4 * j] = f.x; v[4 * j + 1] = f.y; v[4 * j + 2] = f.z; v[4 * j + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < KBLK; ++j) v[j] = (ok && j < nvalid) ? __ldg(src + j * s1) : 0.f;  // 32-bit offsets: two instructions per value
      }
      {
        const long long tw = pa ? clock64() : 0;
        if (!mbar_wait(smem_u32(&ctrl->a_empty[as]), (a_round & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_EMPTY)) break;
        if (pa) atomicAdd(a.prof + 6, (unsigned long long)(clock64() - tw));
      }
      const uint32_t p_hi = tiles_base + as * a_stage_bytes, p_lo = p_hi + a_plane;
      if (chunked) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int ri = chunk * 32 + 4 * i + (lane >> 3);  // strip_rows is a multiple of 8
          if (ri < a.strip_rows) {
            float h[4], l[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) split_tf32_fast(v[4 * i + j], h[j], l[j]);
            const int c4 = (lane & 7) * 4;  // first of this lane's four channels
            sts_f32x4(p_hi + sw128_offset(ri, c4), h[0], h[1], h[2], h[3]);
            if (CROSS_BF16) {
              sts_b32x2(p_lo + sw128_offset_bf16(ri, c4), pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]));
              sts_b32x2(p_lo + sw128_offset_bf16(ri, 32 + c4), pack_bf16x2(l[0], l[1]), pack_bf16x2(l[2], l[3]));
            } else {
              sts_f32x4(p_lo + sw128_offset(ri, c4), l[0], l[1], l[2], l[3]);
            }
          }
        }
      } else if (r < a.strip_rows) {
        if (CROSS_BF16) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {  // eight channels: two 16-byte chunks of the hi plane, one each of bf16(hi), bf16(lo)
            float h[8], l[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) split_tf32_fast(v[c * 8 + j], h[j], l[j]);
            sts_f32x4(p_hi + sw128_offset(r, c * 8), h[0], h[1], h[2], h[3]);
            sts_f32x4(p_hi + sw128_offset(r, c * 8 + 4), h[4], h[5], h[6], h[7]);
            sts_b32x4(p_lo + sw128_offset_bf16(r, c * 8), pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]),
                      pack_bf16x2(h[4], h[5]), pack_bf16x2(h[6], h[7]));
            sts_b32x4(p_lo + sw128_offset_bf16(r, 32 + c * 8), pack_bf16x2(l[0], l[1]), pack_bf16x2(l[2], l[3]),
                      pack_bf16x2(l[4], l[5]), pack_bf16x2(l[6], l[7]));
          }
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float h[4], l[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) split_tf32_fast(v[c * 4 + j], h[j], l[j]);
            const uint32_t o = sw128_offset(r, c * 4);
            sts_f32x4(p_hi + o, h[0], h[1], h[2], h[3]);
            sts_f32x4(p_lo + o, l[0], l[1], l[2], l[3]);
          }
        }
      }
      fence_proxy_async();
      mbar_arrive(smem_u32(&ctrl->a_full[as]));
      PROF_ADD(pa, 7);
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    // A warp reads the TMEM lane quarter (warp & 3); with 8 warps the 32-column chunks alternate
    // between warps w and w + 4.  One warp per scheduler runs at the latency of its dependent
    // instructions, so the per-element work is kept to a multiply-add and a store through a
    // running pointer; everything uniform (bias present, ragged last tile) is decided per chunk.
    const int quarter = warp & 3, half = warp >> 2;
    constexpr int HALVES = EPI_WARPS / 4;
    uint32_t t_count = 0;
    for (TileIter it(a); it.valid(); it.next(), ++t_count) {
      const int tile = it.tile();
      const TileCoord tc_ = tile_coord(a, tile);
      const int n_tile = tc_.n_tile, group = tc_.group, m_tile = tc_.m_tile;
      const int phase_n = (int)a.div_tiles_pp.div((uint32_t)n_tile);
      const int n0 = (n_tile - phase_n * a.tiles_pp) * BN;
      const int cols_valid = min(BN, a.nc - n0);
      const uint32_t ab = t_count & 1;
      const bool pe = PROF_ON(threadIdx.x == 0);
      // a dInput phase that no tap reaches (e.g. 1x1 filter with stride 2) gets zeros
      const bool has_taps = !a.phase_on_n || ctrl->tap_start[phase_n + 1] > ctrl->tap_start[phase_n];
      const int q = m_tile * BLOCK_M + quarter * 32 + lane;
      bool ok = q < a.q_total;
      long long obase = 0, res_off = 0;
      if (ok) {
        const long long n = a.img_div.div((uint32_t)q);
        const int rem = q - (int)n * img_pitch;
        int y = (int)a.row_div.div((uint32_t)rem), x = rem - y * row_pitch;
        ok = y < a.H && x < a.W;
        if (a.phase_on_n) { y = y * a.osh + ctrl->ph_a[phase_n]; x = x * a.osw + ctrl->ph_b[phase_n]; }
        ok = ok && y < a.out_h && x < a.out_w;
        res_off = n * a.res.s0 + ((long long)group * a.nc + n0) * a.res.s1 + (long long)y * a.res.s2 + (long long)x * a.res.s3;
        obase = a.out_rowmajor ? (((n * a.out_h + y) * a.out_w + x) * a.out_pitch + (long long)group * a.out_group + n0)
                               : (((n * a.out_channels + (long long)group * a.nc + n0) * a.out_h + y) * a.out_w + x);
      }
      const long long col_stride = a.out_rowmajor ? 1 : (long long)a.out_h * a.out_w;
      { PROF_T0(pe);
      if (!mbar_wait(smem_u32(&ctrl->acc_full[ab]), (t_count >> 1) & 1, abort_flag, a.status, STATUS_TIMEOUT_ACCUM)) break;
      PROF_ADD(pe, 8); }
      PROF_T0(pe);
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + ab * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const int chunks = (cols_valid + 31) / 32;
      bool released = false;
#pragma unroll 1
      for (int ch = half; ch < chunks; ch += HALVES) {
        const int c0 = ch * 32;
        float v[32];
        tmem_ld32(tmem_acc + (uint32_t)c0, v);
        if (FUSE_HILO) {
          float v2[32];
          tmem_ld32(tmem_acc + (uint32_t)(BN + c0), v2);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += v2[j];
        }
        if (ch + HALVES >= chunks) {  // this warp's last read of the accumulator: hand it back early
          tc_fence_before();
          mbar_arrive(smem_u32(&ctrl->acc_empty[ab]));
          released = true;
        }
        const int nvalid = min(32, cols_valid - c0);
        if (!has_taps) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (a.bias) {
          float bv = 0.f;  // lane j holds the bias of column c0 + j
          if (lane < nvalid) bv = a.beta * __ldg(a.bias + ((long long)group * a.nc + n0 + c0 + lane) * a.bias_stride);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaf(a.alpha, v[j], __shfl_sync(0xffffffffu, bv, j));
        } else if (a.alpha != 1.f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= a.alpha;
        }
        if (a.res.ptr && ok) {
          // all loads of the chunk are issued before the first add (one warp per scheduler runs at
          // the latency of its dependent instructions)
          const float* rp = a.res.ptr + res_off + c0 * a.res.s1;
          float r[32];
          if (nvalid == 32 && a.res.s1 == 1 && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 f = __ldg(reinterpret_cast<const float4*>(rp) + j);
              r[4 * j] = f.x; r[4 * j + 1] = f.y; r[4 * j + 2] = f.z; r[4 * j + 3] = f.w;
            }
          } else if (nvalid == 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __ldg(rp + j * a.res.s1);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = j < nvalid ? __ldg(rp + j * a.res.s1) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += r[j];
        }
        if (a.relu) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        }
        if (ok) {
          float* p = a.out + obase + c0 * col_stride;
          if (a.out_rowmajor && a.out_vec4 && nvalid == 32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(p)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else if (nvalid == 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j, p += col_stride) *p = v[j];
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j, p += col_stride)
              if (j < nvalid) *p = v[j];
          }
        }
      }
      if (!released) {  // no chunk for this warp in a narrow last tile
        tc_fence_before();
        mbar_arrive(smem_u32(&ctrl->acc_empty[ab]));
      }
      PROF_ADD(pe, 9);
      if (pe) atomicAdd(a.prof + 10, 1ull);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
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

// Split W[cout][cin/g][kh][kw] (any strides) into TF32 hi/lo parts laid out as the shared-memory
// images the MMA reads: image = [hi: bn rows x 128 B, SWIZZLE_128B][lo: same], row = output column of
// the tile (forward: co, dInput: ci; zero beyond nc), 32 reduction channels per row.  Images are
// ordered as the main loop consumes them: [group][n_tile][phase][channel block][tap of the phase],
// so a weight stage of the main kernel is one bulk copy from a running pointer.
__global__ void __launch_bounds__(256) stage_weights_kernel(ConvGeom g, View4 w, int is_dx, int bn, int tiles_pp,
                                                            TapTable tt, float* __restrict__ out, long long total,
                                                            long long w_group_extra) {
  // let the convolution kernel behind this one start its prologue and its activation strips now
  asm volatile("griddepcontrol.launch_dependents;");
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= total) return;
  const int kc = is_dx ? g.cog : g.cig, nc = is_dx ? g.cig : g.cog;
  const int cpp = (kc + KBLK - 1) / KBLK;
  // one thread per four adjacent reduction channels: a 16-byte piece of the swizzled row
  const int k = (int)(i % (KBLK / 4)) * 4;
  const int row = (int)((i / (KBLK / 4)) % bn);
  const long long image = i / ((long long)(KBLK / 4) * bn);
  int grp, n_tile, cbl, tap;
  if (is_dx) {  // [group][phase][tile of the phase][channel block][tap of the phase]
    const int per_group = tiles_pp * cpp * tt.taps_total;
    grp = (int)(image / per_group);
    const int local = (int)(image - (long long)grp * per_group);
    int phase = 0;
    while (phase + 1 < tt.n_phase && local >= tiles_pp * cpp * tt.start[phase + 1]) ++phase;
    const int rel = local - tiles_pp * cpp * tt.start[phase], ntap = tt.start[phase + 1] - tt.start[phase];
    n_tile = rel / (cpp * ntap);
    const int rel2 = rel - n_tile * cpp * ntap;
    cbl = rel2 / ntap;
    tap = tt.start[phase] + rel2 % ntap;
  } else {      // [group][tile][phase][channel block][tap of the phase]
    const int per_tile = cpp * tt.taps_total;
    const int local = (int)(image % per_tile);
    n_tile = (int)((image / per_tile) % tiles_pp);
    grp = (int)(image / ((long long)per_tile * tiles_pp));
    int phase = 0;
    while (phase + 1 < tt.n_phase && local >= cpp * tt.start[phase + 1]) ++phase;
    const int rel = local - cpp * tt.start[phase], ntap = tt.start[phase + 1] - tt.start[phase];
    cbl = rel / ntap;
    tap = tt.start[phase] + rel % ntap;
  }
  const int r = n_tile * bn + row, c = cbl * KBLK + k;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (r < nc) {  // rows beyond the column count and channels beyond a ragged last block are zero
    // forward: r is the output channel, c the input channel; dInput: the other way round
    const long long step = is_dx ? w.s0 : w.s1;
    const float* src = w.ptr + ((long long)grp * g.cog + (is_dx ? c : r)) * w.s0 + (long long)(is_dx ? r : c) * w.s1 +
                       tt.ky[tap] * w.s2 + tt.kx[tap] * w.s3 + grp * w_group_extra;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (c + j < kc) v[j] = __ldg(src + j * step);
  }
  float hi[4], lo[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) split_tf32(v[j], hi[j], lo[j]);
  float* plane = out + image * (bn * 64ll);
  *reinterpret_cast<float4*>(plane + sw128_offset(row, k) / 4) = make_float4(hi[0], hi[1], hi[2], hi[3]);
  if (CROSS_BF16) {  // second plane: [bf16(lo) x32 | bf16(hi) x32] per row, pairing with the activations' [hi | lo]
    unsigned char* cross = reinterpret_cast<unsigned char*>(plane + bn * 32);
    *reinterpret_cast<uint2*>(cross + sw128_offset_bf16(row, k)) = make_uint2(pack_bf16x2(lo[0], lo[1]), pack_bf16x2(lo[2], lo[3]));
    *reinterpret_cast<uint2*>(cross + sw128_offset_bf16(row, 32 + k)) = make_uint2(pack_bf16x2(hi[0], hi[1]), pack_bf16x2(hi[2], hi[3]));
  } else {
    *reinterpret_cast<float4*>(plane + bn * 32 + sw128_offset(row, k) / 4) = make_float4(lo[0], lo[1], lo[2], lo[3]);
  }
}

static inline int floor_div(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }


// Any stride / padding / dilation in both directions; the reduction channels must come in blocks of
// 32 and there must be at least 16 output columns.  Forward groups the taps by the phase of the
// INPUT pixel they read; dInput by the phase of the OUTPUT (dX) pixel they contribute to: dX pixel
// s*r + a receives tap ky iff (ky*d - pad) = a (mod s), from dY row r - floor((ky*d - pad) / s).
StripPlan plan_strip_geometry(const ConvGeom& g, bool is_dx) {
  StripPlan p;
  const int kc = is_dx ? g.cog : g.cig, nc = is_dx ? g.cig : g.cog;
  // a ragged last channel block is padded with zeros; below 16 channels the padding would more than
  // double the work and the CUDA-core kernels are the better choice
  if (kc < 16 || nc < 16 || g.kh * g.kw > MAX_TAPS) return p;
  if (g.sh * g.sw > MAX_PHASES || g.sh > 255 || g.sw > 255) return p;
  p.sph = g.sh; p.spw = g.sw;
  p.act_h = is_dx ? g.oh : g.h; p.act_w = is_dx ? g.ow : g.w;
  p.out_h = is_dx ? g.h : g.oh; p.out_w = is_dx ? g.w : g.ow;
  // the grid covers the unstrided tensor and every phase sub-image of the strided one
  p.gh = std::max(g.oh, (g.h + p.sph - 1) / p.sph);
  p.gw = std::max(g.ow, (g.w + p.spw - 1) / p.spw);
  // taps -> (phase, whole-pixel offset); forward reads x at s*o - pad + k*d, dInput reads dy at i + pad - k*d
  struct Tap { int phase, dr, dc, ky, kx; };
  Tap taps[MAX_TAPS];
  int ntaps = 0, dr_lo = 0, dr_hi = 0, dc_lo = 0, dc_hi = 0;
  for (int ky = 0; ky < g.kh; ++ky)
    for (int kx = 0; kx < g.kw; ++kx) {
      const int oy = ky * g.dh - g.ph, ox = kx * g.dw - g.pw;
      const int fr = floor_div(oy, p.sph), fc = floor_div(ox, p.spw);
      const int dr = is_dx ? -fr : fr, dc = is_dx ? -fc : fc;
      taps[ntaps++] = Tap{(oy - fr * p.sph) * p.spw + (ox - fc * p.spw), dr, dc, ky, kx};
      dr_lo = std::min(dr_lo, dr); dr_hi = std::max(dr_hi, dr);
      dc_lo = std::min(dc_lo, dc); dc_hi = std::max(dc_hi, dc);
    }
  p.pr = std::max(-dr_lo, dr_hi);
  p.pc = std::max(-dc_lo, dc_hi);
  if ((long long)g.n * (p.gh + p.pr) * (p.gw + p.pc) > 2147483647ll - (1 << 20)) return p;  // 32-bit pixel indices
  const int row_pitch = p.gw + p.pc;
  TapTable& tt = p.tt;
  memset(&tt, 0, sizeof tt);
  int lo = 0, hi = 0;
  for (int phase = 0; phase < p.sph * p.spw; ++phase) {
    int count = 0;
    for (int t = 0; t < ntaps; ++t)
      if (taps[t].phase == phase) {
        const int i = tt.taps_total++;
        tt.ky[i] = (unsigned char)taps[t].ky; tt.kx[i] = (unsigned char)taps[t].kx;
        tt.shift[i] = taps[t].dr * row_pitch + taps[t].dc;
        lo = std::min(lo, tt.shift[i]); hi = std::max(hi, tt.shift[i]);
        ++count;
      }
    if (count == 0 && !is_dx) continue;  // forward: a phase no tap reads is never staged (dInput: it is zero-filled)
    tt.a[tt.n_phase] = (unsigned char)(phase / p.spw); tt.b[tt.n_phase] = (unsigned char)(phase % p.spw);
    tt.start[tt.n_phase + 1] = (unsigned char)tt.taps_total;
    ++tt.n_phase;
  }
  p.shift_lo = lo; p.shift_hi = hi;
  p.halo = -lo;
  p.ok = true;
  return p;
}

static StripPlan plan_strip(const ConvGeom& g, bool is_dx) {
  StripPlan p = plan_strip_geometry(g, is_dx);
  if (!p.ok) return p;
  p.ok = false;
  const int nc = is_dx ? g.cig : g.cog;
  p.strip_rows = (BLOCK_M + p.shift_hi - p.shift_lo + 7) / 8 * 8;
  const int a_stage = p.strip_rows * 256;
  // Column tile: the widest tile makes the best use of shared-memory bandwidth per MMA, but a small
  // image gives few 128-pixel row tiles; pick the width with the lowest modelled time
  // waves(tiles / SMs) * width / efficiency(width).
  const long long tiles_m = div_up64((long long)g.n * (p.gh + p.pr) * (p.gw + p.pc), BLOCK_M);
  double best_cost = 0.0;
  bool single_tap = true;  // no phase has more than one tap (1x1 filters): every staged strip feeds one tap's MMAs only
  for (int ph = 0; ph < p.tt.n_phase; ++ph) single_tap = single_tap && p.tt.start[ph + 1] - p.tt.start[ph] <= 1;
  for (int bn : {256, 128, 64}) {
    if (bn > 64 && nc <= bn / 2) continue;  // do not pad the column tile by more than 2x
    const int w_stage = bn * 256;
    for (int a_stages : {4, 3, 2, 1}) {
      if (a_stages > 2 && a_stages * a_stage > SMEM_LIMIT / 2 && !single_tap) continue;  // deep strip pipelines only while cheap
                                                                                          // (or while the producers set the pace)
      const int left = SMEM_LIMIT - a_stages * a_stage;
      if (left < 2 * w_stage) continue;
      const long long tiles = tiles_m * ((nc + bn - 1) / bn) * g.groups * (is_dx ? p.sph * p.spw : 1);
      const double eff = bn == 256 ? 1.0 : (bn == 128 ? 0.85 : 0.55);
      const double cost = (double)div_up64(tiles, sm_count()) * bn / eff;
      if (!p.ok || cost < best_cost) {
        best_cost = cost;
        p.ok = true;
        p.bn = bn;
        p.a_stages = a_stages;
        p.w_stages = std::min(MAX_STAGES, left / w_stage);
        p.smem = a_stages * a_stage + p.w_stages * w_stage + 1024 + (int)sizeof(Ctrl) + 64;
      }
      break;  // the deepest strip pipeline that fits is the one to use for this width
    }
  }
  return p;
}

}  // namespace tcs

bool strip_supported(const ConvGeom& g, int phase) {
  if (phase != B200_PHASE_FORWARD && phase != B200_PHASE_DINPUT) return false;
  return tcs::plan_strip(g, phase == B200_PHASE_DINPUT).ok;
}
int strip_column_tile(const ConvGeom& g, bool is_dx) {
  const tcs::StripPlan p = tcs::plan_strip(g, is_dx);
  return p.ok ? p.bn : 0;
}
// Bytes of the weight stage images: hi and lo planes with the column count padded to the tile width.
// The width depends on the image count, so take the largest over the widths the plan may pick.
size_t strip_workspace(const ConvGeom& g, int phase) {
  const bool is_dx = phase == B200_PHASE_DINPUT;
  const size_t kc = is_dx ? g.cog : g.cig, nc = is_dx ? g.cig : g.cog;
  size_t cols = 0;
  for (size_t bn : {256, 128, 64}) cols = std::max(cols, (nc + bn - 1) / bn * bn);
  return 2 * sizeof(float) * (size_t)g.groups * cols * ((kc + 31) / 32 * 32) * g.kh * g.kw;  // ragged last channel block padded
}

template <int BN, int AW>
static int launch_strip_aw(const tcs::StripArgs& a, int grid, int smem, cudaStream_t st) {
  // opt in once (thread-safe) to the full 227 KB of dynamic shared memory for this instantiation
  static std::once_flag once;
  static cudaError_t opt_in = cudaSuccess;
  std::call_once(once, [] { opt_in = cudaFuncSetAttribute(tcs::conv_strip_kernel<BN, AW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448); });
  B200_CUDA(opt_in);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(tcs::strip_threads(AW)); cfg.dynamicSmemBytes = (size_t)smem; cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  if (a.wait_for_images) { cfg.attrs = &attr; cfg.numAttrs = 1; }
  B200_CUDA(cudaLaunchKernelEx(&cfg, tcs::conv_strip_kernel<BN, AW>, a));
  count_launch();
  return launch_check("conv_strip_kernel");
}
template <int BN>
static int launch_strip(const tcs::StripArgs& a, int grid, int smem, cudaStream_t st) {
  return a.wide_producers ? launch_strip_aw<BN, 16>(a, grid, smem, st) : launch_strip_aw<BN, 8>(a, grid, smem, st);
}

// The kernel forms element offsets inside the activation tensor in 32 bits: true when the view's
// extent (with the 64 channels a ragged block may look ahead) stays below 2^31 elements.
bool strip_view_addressable(const ConvGeom& g, bool is_dx, const View4& act, const StripBatch* batch) {
  const long long an = g.n, ac = is_dx ? g.cout : g.cin, ah = is_dx ? g.oh : g.h, aw = is_dx ? g.ow : g.w;
  const long long span = (an - 1) * std::llabs(act.s0) + (ac - 1) * std::llabs(act.s1) +
                         (ah - 1) * std::llabs(act.s2) + (aw - 1) * std::llabs(act.s3) +
                         (batch ? (g.groups - 1) * std::llabs(batch->act_group_extra) : 0);
  return span <= 2147483647ll - 64 * std::llabs(act.s1);
}

int strip_conv(const ConvGeom& g, bool is_dx, View4 act, View4 w, const float* bias, long long bias_stride, float* out,
               void* ws, size_t ws_bytes, cudaStream_t st, bool rowmajor, float alpha, float beta, const float* staged_images,
               const StripPostOps* post, const StripBatch* batch) {
  using namespace tcs;
  const StripPlan plan = plan_strip(g, is_dx);
  if (!plan.ok) return fail(B200_EUNSUPPORTED, "strip kernel does not take this geometry");
  const int kc = is_dx ? g.cog : g.cig, nc = is_dx ? g.cig : g.cog;
  const int tiles_pp = (nc + plan.bn - 1) / plan.bn;  // column tiles (per output phase in dInput)
  const int tiles_n = is_dx ? tiles_pp * plan.tt.n_phase : tiles_pp;
  const int cpp = (kc + KBLK - 1) / KBLK;  // channel blocks per group, the last one possibly ragged
  const long long wcount = (long long)g.groups * tiles_pp * plan.bn * cpp * KBLK * g.kh * g.kw;  // per plane
  const float* wp = staged_images;
  bool staged_here = false;
  if (!wp) {
    if (!ws || ws_bytes < 2 * sizeof(float) * (size_t)wcount || (reinterpret_cast<uintptr_t>(ws) & 15))
      return fail(B200_EWORKSPACE, "tcgen05 convolution needs a 16-byte aligned workspace of %zu bytes (got %zu)",
                  2 * sizeof(float) * (size_t)wcount, ws_bytes);
    stage_weights_kernel<<<(unsigned)div_up64(wcount / 4, 256), 256, 0, st>>>(g, w, is_dx ? 1 : 0, plan.bn, tiles_pp, plan.tt, (float*)ws, wcount / 4,
                                                                          batch ? batch->w_group_extra : 0);
    count_launch();
    if (int rc = launch_check("stage_weights_kernel")) return rc;
    wp = (const float*)ws;
    staged_here = true;
  }
  if (reinterpret_cast<uintptr_t>(wp) & 15) return fail(B200_EINVAL, "weight stage images must be 16-byte aligned");
  if (!strip_view_addressable(g, is_dx, act, batch))
    return fail(B200_EUNSUPPORTED, "strip kernel: activation tensor too large for 32-bit element offsets");
  StripArgs a{};
  a.g = g; a.act = act; a.wp = wp; a.bias = bias; a.bias_stride = bias_stride; a.out = out;
  a.H = plan.gh; a.W = plan.gw; a.pr = plan.pr; a.pc = plan.pc;
  a.act_h = plan.act_h; a.act_w = plan.act_w; a.out_h = plan.out_h; a.out_w = plan.out_w;
  a.sph = is_dx ? 1 : plan.sph; a.spw = is_dx ? 1 : plan.spw;
  a.osh = is_dx ? plan.sph : 1; a.osw = is_dx ? plan.spw : 1;
  a.phase_on_n = is_dx ? 1 : 0;
  a.tiles_pp = tiles_pp;
  a.tt = plan.tt;
  a.kc = kc;
  a.nc = nc;
  a.out_channels = is_dx ? g.cin : g.cout;
  a.act_group_extra = batch ? batch->act_group_extra : 0;
  a.out_pitch = batch ? batch->out_pitch : a.out_channels;
  a.out_group = batch ? batch->out_group : nc;
  a.cb_per_phase = cpp;
  a.cblocks = (is_dx ? 1 : plan.tt.n_phase) * a.cb_per_phase;
  a.images_per_tile = a.cb_per_phase * plan.tt.taps_total;
  a.tiles_n = tiles_n;
  a.q_total = (int)((long long)g.n * (a.H + a.pr) * (a.W + a.pc));
  a.img_div = FastDiv((uint32_t)((a.H + a.pr) * (a.W + a.pc)));
  a.row_div = FastDiv((uint32_t)(a.W + a.pc));
  a.tiles_m = (int)div_up64(a.q_total, BLOCK_M);
  a.halo = plan.halo; a.strip_rows = plan.strip_rows; a.a_stages = plan.a_stages; a.w_stages = plan.w_stages;
  {
    // one tap per staged strip (1x1 filters): the MMAs wait for the producers, so sixteen of them run (testing aid:
    // B200_STRIP_PRODUCERS=8|16 pins either)
    int most = 0;
    for (int ph = 0; ph < plan.tt.n_phase; ++ph) most = std::max(most, (int)plan.tt.start[ph + 1] - (int)plan.tt.start[ph]);
    // ... and only while the reduction side is the larger one (256 -> 64 channels forward: 90 -> 69 us); with more output
    // than input (its dInput) the epilogue's stores set the pace and the extra warps only take registers from it (61 -> 80 us)
    a.wide_producers = most <= 1 && kc > nc ? 1 : 0;
    if (const char* e = getenv("B200_STRIP_PRODUCERS")) a.wide_producers = atoi(e) == 16 ? 1 : 0;
  }
  const int chunks = (a.strip_rows + 31) / 32;
  const long long tiles_total = (long long)a.tiles_m * a.tiles_n * g.groups;
  if (tiles_total * a.cblocks * chunks > 2147483647ll - (1 << 20))
    return fail(B200_EUNSUPPORTED, "strip kernel: tile count exceeds 32-bit job indices");
  a.tiles_total = (int)tiles_total;
  // units of all column tiles of a pixel-row tile while that still leaves every SM two or more units
  a.unit = (tiles_total / a.tiles_n >= 2ll * sm_count()) ? a.tiles_n : 1;
  a.units = a.tiles_total / a.unit;
  a.m_fastest = (a.unit == 1 && a.tiles_n > 1) ? 1 : 0;
  a.div_unit = FastDiv((uint32_t)a.unit);
  a.div_tiles_n = FastDiv((uint32_t)a.tiles_n); a.div_tiles_m = FastDiv((uint32_t)a.tiles_m);
  a.div_tiles_pp = FastDiv((uint32_t)a.tiles_pp); a.div_chunks = FastDiv((uint32_t)chunks);
  a.div_cblocks = FastDiv((uint32_t)a.cblocks); a.div_cbpp = FastDiv((uint32_t)a.cb_per_phase);
  a.div_a_stages = FastDiv((uint32_t)a.a_stages);
  a.wait_for_images = staged_here ? 1 : 0;
  if (post && !is_dx) { a.res = post->residual; a.relu = post->relu; }
  a.out_rowmajor = rowmajor ? 1 : 0;
  a.alpha = alpha; a.beta = beta;
  a.out_vec4 = rowmajor && a.out_pitch % 4 == 0 && a.out_group % 4 == 0 && plan.bn % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
               a.nc % 4 == 0;
  a.status = device_status_word();
  if (!a.status) return fail(B200_ECUDA, "device status word is not allocated");
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
  const int grid = std::min(a.units, sm_count());
  if (profiling) {
    const int rc = plan.bn == 64 ? launch_strip<64>(a, grid, plan.smem, st)
                 : plan.bn == 128 ? launch_strip<128>(a, grid, plan.smem, st) : launch_strip<256>(a, grid, plan.smem, st);
    unsigned long long h[16];
    B200_CUDA(cudaStreamSynchronize(st));
    B200_CUDA(cudaMemcpy(h, prof_buf, sizeof h, cudaMemcpyDeviceToHost));
    fprintf(stderr, "[strip profile, CTA 0, cycles] bn=%d a_stages=%d w_stages=%d tiles=%llu | mma: wait_acc %llu wait_a %llu wait_w %llu issue %llu | "
            "w: wait_empty %llu convert %llu | a: wait_empty %llu stage_total %llu | epi: wait_acc %llu drain %llu | ns: CTA starts spread %llu, first start to last end %llu, CTA lifetime min %llu max %llu\n",
            plan.bn, plan.a_stages, plan.w_stages, h[10], h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[7], h[8], h[9], h[12] - h[11], h[13] - h[11], h[14], h[15]);
    return rc;
  }
  if (plan.bn == 64) return launch_strip<64>(a, grid, plan.smem, st);
  if (plan.bn == 128) return launch_strip<128>(a, grid, plan.smem, st);
  return launch_strip<256>(a, grid, plan.smem, st);
}


// C[M,N] = alpha * A*B + beta * bias[n] as a 1x1 convolution over an M-pixel image with K input and N
// output channels, written row-major.  Takes K >= 16 and N >= 16 (a ragged last block of K is padded
// with zeros); anything else is the caller's CUDA-core kernel.  The staged copy of B comes from the caching allocator and is released on `st`.
int tc_gemm(long long M, long long N, long long K, const float* A, long long sa0, long long sa1, const float* B,
            long long sb0, long long sb1, const float* bias, float alpha, float beta, float* C, cudaStream_t st) {
  if (K < 16 || N < 16 || M > 2147483647ll || N > 2147483647ll || K > 2147483647ll)
    return fail(B200_EUNSUPPORTED, "tcgen05 GEMM is incompatible with this shape (needs K >= 16 and N >= 16)");
  ConvGeom g{};
  g.n = 1; g.cin = (int)K; g.cout = (int)N; g.h = 1; g.w = (int)M; g.kh = g.kw = 1; g.oh = 1; g.ow = (int)M;
  g.sh = g.sw = 1; g.ph = g.pw = 0; g.dh = g.dw = 1; g.groups = 1; g.cig = (int)K; g.cog = (int)N;
  if (!tcs::plan_strip(g, false).ok) return fail(B200_EUNSUPPORTED, "tcgen05 GEMM is incompatible with this shape");
  const View4 act{A, 0, sa1, 0, sa0};   // [n=1][c=k][h=1][w=m]
  const View4 wv{B, sb1, sb0, 0, 0};    // [co=n][ci=k][1][1]
  void* ws = nullptr;
  const size_t ws_bytes = strip_workspace(g, B200_PHASE_FORWARD);
  if (int rc = b200_malloc(&ws, ws_bytes, st)) return rc;
  if (!bias || beta == 0.f) { bias = nullptr; beta = 0.f; }
  const int rc = strip_conv(g, false, act, wv, bias, 1, C, ws, ws_bytes, st, true, alpha, beta);
  b200_free(ws, st);
  return rc;
}

// C[b] = A[b] * B[b] for every batch in ONE launch pair: the batch rides on the kernel's group
// dimension (each group has its own weight images and its own block of reduction channels), with the
// three per-group offsets of StripBatch standing in for the grouped convolution's channel arithmetic.
int tc_bmm(long long batch, long long M, long long N, long long K, const float* A, long long sa_b, long long sa0, long long sa1,
           const float* B, long long sb_b, long long sb0, long long sb1, float* C, cudaStream_t st) {
  if (K < 16 || N < 16 || M > 2147483647ll || batch * N > 2147483647ll || batch * K > 2147483647ll || batch > 65535)
    return fail(B200_EUNSUPPORTED, "tcgen05 batched GEMM is incompatible with this shape (needs K >= 16 and N >= 16)");
  ConvGeom g{};
  g.n = 1; g.cin = (int)(batch * K); g.cout = (int)(batch * N); g.h = 1; g.w = (int)M; g.kh = g.kw = 1; g.oh = 1; g.ow = (int)M;
  g.sh = g.sw = 1; g.ph = g.pw = 0; g.dh = g.dw = 1; g.groups = (int)batch; g.cig = (int)K; g.cog = (int)N;
  if (!tcs::plan_strip(g, false).ok) return fail(B200_EUNSUPPORTED, "tcgen05 batched GEMM is incompatible with this shape");
  const View4 act{A, 0, sa1, 0, sa0};   // [n=1][c=(b,k)][h=1][w=m]
  const View4 wv{B, sb1, sb0, 0, 0};    // [co=(b,n)][ci=k][1][1]
  StripBatch sb;
  sb.act_group_extra = sa_b - K * sa1;  // group b starts b*K channels in: b*K*sa1 of the way to A[b]
  sb.w_group_extra = sb_b - N * sb1;
  sb.out_pitch = N;
  sb.out_group = M * N;
  void* ws = nullptr;
  const size_t ws_bytes = strip_workspace(g, B200_PHASE_FORWARD);
  if (int rc = b200_malloc(&ws, ws_bytes, st)) return rc;
  const int rc = strip_conv(g, false, act, wv, nullptr, 1, C, ws, ws_bytes, st, true, 1.f, 0.f, nullptr, nullptr, &sb);
  b200_free(ws, st);
  return rc;
}

}  // namespace b200
