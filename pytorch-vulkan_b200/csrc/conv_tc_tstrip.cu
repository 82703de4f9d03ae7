// Persistent tcgen05 implicit-GEMM kernel for convolution forward and dInput with the operand roles of
// conv_tc_strip.cu exchanged: the FILTER is the M operand (128 output channels per tile, zero padded) and the
// ACTIVATION STRIP is the N operand (up to 256 pixels of the zero-padded pixel grid per tile), so the
// accumulator holds [output channel][pixel].
//
// Why a second arrangement.  A tcgen05.mma reads both operands from shared memory at roughly 96 bytes per
// clock; with 128 pixels on M and N <= 128 output channels that read, not the tensor pipe, sets the pace
// (93 clocks for a 128x128x8 TF32 step that computes for 64), and the pixel tile is fixed at 128, which
// quantises badly (421 tiles on 148 SMs = 2.84 waves for 128 channels at 28x28).  With the filter on M
//   * the N extent is the pixel count, any multiple of 16 up to 256: a 128-channel layer issues 128x256x8
//     steps at the tensor pipe's own pace, and the tile width is chosen per layer so that the tiles fill
//     whole waves;
//   * each filter stage (one tap of 16 input channels) feeds twice the pixels, which halves the filter bytes
//     pulled from L2 per output.
// Everything else is the strip idea unchanged: the activations of a tile are staged once per channel block
// as one shared-memory row per pixel of the padded grid (q = (n*(H+pr) + y)*(W+pc) + x), a filter tap is a
// constant row shift applied through the operand descriptor's start address, strides are handled by tap
// phases (strip_plan.cuh), and FP32 comes from split precision: TF32 hi*hi plus one BF16 pass for both cross
// terms (tc_common.cuh).
//
// Shared-memory layout: channel blocks of 16 (64-byte rows, SWIZZLE_64B), so that a strip stage of 256 pixels
// plus halo is about 40 KB and three of them fit beside a ring of 32 KB filter stages (two taps each).  Per stage:
//   hi plane     rows x 64 B   TF32(x) for 16 channels
//   cross plane  rows x 64 B   [bf16(x_hi) x16 | bf16(x_lo) x16]     (filter: [bf16(w_lo) x16 | bf16(w_hi) x16])
//
// CTA roles (448 threads, persistent over tiles): warps 0-3 epilogue (tcgen05.ld, transpose through shared
// memory so that a warp stores 32 consecutive pixels of one channel, bias), warps 4-11 strip producers, warp 12
// one thread streaming filter stages with cp.async.bulk, warp 13 tensor-memory allocation and the MMA issue (the
// whole warp runs the loop, one elected lane issues).
// Two accumulators of 256 columns alternate, so the epilogue of a tile runs under the next tile's main loop.
// All hand-offs are mbarriers with bounded waits.
//
// Replaces csrc/shaders/conv2d_tiled_body.glsl:53-86 and conv2d_backward_input_tiled_body.glsl:49-93 of the
// reference for contiguous NCHW results with at least 65 output channels per group (below that half of every
// MMA would multiply padding, and conv_tc_strip.cu is the better arrangement).
#include "common.cuh"
#include "strip_plan.cuh"
#include "tc_common.cuh"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace b200 {
namespace tst {
using namespace tc;
using tcs::StripPlan;
using tcs::TapTable;
using tcs::MAX_PHASES;
using tcs::MAX_TAPS;

constexpr int TM = 128;          // filter rows (output channels) per tile
constexpr int KB = 16;           // reduction channels per stage
constexpr int ROWB = 64;         // bytes per plane row
constexpr int EPI_WARPS = 4;   // then AW strip producers (8, or 16 where the producers set the pace), the filter warp, the MMA warp
constexpr int tstrip_threads(int aw) { return (EPI_WARPS + aw + 2) * 32; }
constexpr int MAX_A_STAGES = 4, MAX_W_STAGES = 8;
constexpr uint32_t W_STAGE_BYTES = TM * ROWB * 2;   // hi plane + cross plane of one (tap, channel block)
constexpr uint32_t W_RING_BYTES = 2 * W_STAGE_BYTES;  // a ring stage holds the images of two consecutive taps: one wait and one
                                                      // commit per eight MMAs (the issuing warp is bound by its own instruction latencies)
constexpr int TBUF_BYTES = EPI_WARPS * 32 * 33 * 4;  // the epilogue's transpose tiles
constexpr int SMEM_LIMIT = 232448 - 2048;

struct TArgs {
  ConvGeom g;
  View4 act;              // forward: x.  dInput: dy
  const float* wp;        // filter stage images, W_STAGE_BYTES each, in the order the main loop consumes them
  const float* bias;
  long long bias_stride;
  float* out;             // contiguous NCHW [n][out_channels][out_h][out_w]
  int H, W, pr, pc;       // pixel grid shared by the strip rows and the accumulator columns, and its zero padding
  int act_h, act_w, out_h, out_w;
  int sph, spw;           // forward: phases on the reduction side (channel block -> phase)
  int osh, osw;           // dInput: phases on the output side (channel tile -> phase)
  int phase_on_m;         // 1 in the dInput arrangement
  int tiles_pp;           // channel tiles per phase (dInput), else tiles_m
  int kc, nc, out_channels;
  int cb_per_phase, cblocks, images_per_tile;
  int tiles_m, tiles_p, tiles_total;
  int pn;                 // pixels per tile: a multiple of 16, at most 256
  int q_total;
  FastDiv img_div, row_div, div_tiles_p, div_tiles_m, div_tiles_pp, div_chunks, div_cblocks, div_cbpp, div_a_stages;
  int halo, strip_rows;   // rows staged before a tile's first pixel; rows per stage (a multiple of 8)
  int a_stages, w_stages;
  int wait_for_images;
  int* status;
  unsigned long long* prof;   // optional cycle counters of CTA 0's MMA thread (-DB200_ROLE_PROFILE=1 and B200_STRIP_PROFILE=1)
  TapTable tt;
};

// tcgen05.fence::after_thread_sync after every operand-stage wait (measured: it costs about 300 clocks per stage,
// because it also waits behind the MMAs in flight; the mbarrier wait alone orders the stage's data before the MMA
// that reads it, so it is off)
#ifndef B200_STAGE_FENCE
#define B200_STAGE_FENCE 0
#endif
#ifndef B200_ROLE_PROFILE
#define B200_ROLE_PROFILE 0
#endif
#define TPROF(slot, stmt) do { if (B200_ROLE_PROFILE && a.prof && blockIdx.x == 0) { const long long t0__ = clock64(); stmt; atomicAdd(a.prof + (slot), (unsigned long long)(clock64() - t0__)); } else { stmt; } } while (0)

struct Ctrl {
  unsigned long long a_full[MAX_A_STAGES], a_empty[MAX_A_STAGES], w_full[MAX_W_STAGES], w_empty[MAX_W_STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int shift[MAX_TAPS];
  unsigned char ph_a[MAX_PHASES], ph_b[MAX_PHASES], tap_start[MAX_PHASES + 1];
};

// byte offset of 16-byte chunk `c` (0..3) of row `row` in a plane of 64-byte rows, SWIZZLE_64B
__device__ __host__ __forceinline__ uint32_t sw64_chunk(int row, int c) {
  return (uint32_t)(row * ROWB + ((c ^ ((row >> 1) & 3)) << 4));
}
// K-major operand descriptor for a plane of 64-byte rows, SWIZZLE_64B: 8-row groups 512 bytes apart
__device__ __forceinline__ uint64_t make_kmajor_sw64_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;   // SWIZZLE_64B
  return d;
}

struct TileCoord {
  int p_tile, m_tile, group;
};
// tile index -> (pixel tile, channel tile, group), pixel tile fastest: the CTAs that run at the same time
// then stream the same filter images, which L2 serves once
__device__ __forceinline__ TileCoord tile_coord(const TArgs& a, int tile) {
  TileCoord c;
  const int rest = (int)a.div_tiles_p.div((uint32_t)tile);
  c.p_tile = tile - rest * a.tiles_p;
  c.group = (int)a.div_tiles_m.div((uint32_t)rest);
  c.m_tile = rest - c.group * a.tiles_m;
  return c;
}

template <int AW>
__global__ void __launch_bounds__(tstrip_threads(AW), 1) conv_tstrip_kernel(const TArgs a) {
  constexpr int A_WARPS = AW, W_WARP = EPI_WARPS + AW, MMA_WARP = W_WARP + 1;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  const uint32_t a_plane = (uint32_t)a.strip_rows * ROWB, a_stage_bytes = 2u * a_plane;
  constexpr uint32_t w_plane = TM * ROWB;
  const uint32_t w_base = tiles_base + a.a_stages * a_stage_bytes;
  const uint32_t tbuf_base = w_base + a.w_stages * W_RING_BYTES;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + (tbuf_base - raw) + TBUF_BYTES);
  volatile int* abort_flag = &ctrl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t ACC_COLS = 256, TMEM_COLS = 512;
  const long long prof_c0 = (B200_ROLE_PROFILE && a.prof) ? clock64() : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_A_STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->a_full[s]), (uint32_t)((a.strip_rows + 31) / 32) * 32u);
      mbar_init(smem_u32(&ctrl->a_empty[s]), 1);
    }
    for (int s = 0; s < MAX_W_STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->w_full[s]), 1);
      mbar_init(smem_u32(&ctrl->w_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ctrl->acc_full[s]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[s]), EPI_WARPS * 32);
    }
    ctrl->abort_flag = 0;
    fence_barrier_init();
  }
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
  const int my_tiles = a.tiles_total > (int)blockIdx.x ? (a.tiles_total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

  if (warp == MMA_WARP) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp runs the loop and waits on the barriers; ONE elected lane issues the tcgen05 instructions.
    // Control flow and every descriptor are then uniform across the warp, so the compiler keeps them in uniform
    // registers, which is where tcgen05.mma takes its operands from: issued from a single divergent thread every
    // operand first crosses from the vector registers, and that (about 370 clocks per four MMAs, measured as
    // tensor-pipe idle time of 43 %) was what bounded the kernel.
    // D[128 filter rows][pn pixels] += W[128 x 8] * X[pn x 8]^T, both operands K-major
    const uint32_t idesc = make_idesc_tf32(TM, a.pn), idesc_cross = make_idesc_bf16(TM, a.pn);
    const uint64_t dx_base = make_kmajor_sw64_desc(tiles_base + (uint32_t)a.halo * ROWB);
    const uint64_t dw_base = make_kmajor_sw64_desc(w_base);
    const uint32_t a_stage_d = a_stage_bytes >> 4, a_plane_d = a_plane >> 4;
    constexpr uint32_t w_stage_d = W_STAGE_BYTES >> 4, w_plane_d = w_plane >> 4, w_ring_d = W_RING_BYTES >> 4;
    const bool leader = elect_one();
    uint32_t as = 0, a_par = 0, ws = 0, w_par = 0;
    bool alive = true;
    for (int t = 0; t < my_tiles && alive; ++t) {
      const int tile = (int)blockIdx.x + t * (int)gridDim.x;
      const uint32_t ab = (uint32_t)t & 1u;
      if (!warp_wait(smem_u32(&ctrl->acc_empty[ab]), (((uint32_t)t >> 1) & 1u) ^ 1u, abort_flag, a.status, STATUS_TIMEOUT_ACCUM)) break;
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + ab * ACC_COLS;
      const int m_tile = tile_coord(a, tile).m_tile;
      int phase = a.phase_on_m ? (int)a.div_tiles_pp.div((uint32_t)m_tile) : 0;
      int cbl = 0;
      uint32_t accumulate = 0;
      for (int cb = 0; cb < a.cblocks && alive; ++cb) {
        if (!warp_wait(smem_u32(&ctrl->a_full[as]), a_par, abort_flag, a.status, STATUS_TIMEOUT_FULL)) { alive = false; break; }
        const uint64_t dx_strip = dx_base + as * a_stage_d;
        const int tap_end = ctrl->tap_start[phase + 1];
        for (int tap = ctrl->tap_start[phase]; tap < tap_end; tap += 2) {
          const int sh0 = ctrl->shift[tap], sh1 = ctrl->shift[tap + 1 < tap_end ? tap + 1 : tap];
          const bool two = tap + 1 < tap_end;
          if (!warp_wait(smem_u32(&ctrl->w_full[ws]), w_par, abort_flag, a.status, STATUS_TIMEOUT_FULL)) { alive = false; break; }
          const uint64_t x0 = dx_strip + (uint64_t)(long long)(sh0 * (ROWB / 16)), x1 = dx_strip + (uint64_t)(long long)(sh1 * (ROWB / 16));
          const uint64_t w0 = dw_base + ws * w_ring_d, w1 = w0 + w_stage_d;
          if (leader) {
            umma_tf32(tmem_acc, w0, x0, idesc, accumulate);
            umma_tf32(tmem_acc, w0 + 2, x0 + 2, idesc, 1);
            umma_bf16(tmem_acc, w0 + w_plane_d, x0 + a_plane_d, idesc_cross, 1);
            umma_bf16(tmem_acc, w0 + w_plane_d + 2, x0 + a_plane_d + 2, idesc_cross, 1);
            if (two) {
              umma_tf32(tmem_acc, w1, x1, idesc, 1);
              umma_tf32(tmem_acc, w1 + 2, x1 + 2, idesc, 1);
              umma_bf16(tmem_acc, w1 + w_plane_d, x1 + a_plane_d, idesc_cross, 1);
              umma_bf16(tmem_acc, w1 + w_plane_d + 2, x1 + a_plane_d + 2, idesc_cross, 1);
            }
            umma_commit(smem_u32(&ctrl->w_empty[ws]));
          }
          accumulate = 1;
          if (++ws == (uint32_t)a.w_stages) { ws = 0; w_par ^= 1; }
        }
        if (alive && leader) umma_commit(smem_u32(&ctrl->a_empty[as]));
        if (++as == (uint32_t)a.a_stages) { as = 0; a_par ^= 1; }
        if (!a.phase_on_m && ++cbl == a.cb_per_phase) { cbl = 0; ++phase; }
      }
      if (alive && leader) umma_commit(smem_u32(&ctrl->acc_full[ab]));
    }
  } else if (warp == W_WARP) {
    // ------------------------------ filter stages (one thread) ------------------------------
    if (lane == 0) {
      uint32_t ws = 0, w_par = 1, issued = 0;
      bool alive = true;
      if (a.wait_for_images) asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int t = 0; t < my_tiles && alive; ++t) {
        const TileCoord tc_ = tile_coord(a, (int)blockIdx.x + t * (int)gridDim.x);
        const long long group = tc_.group;
        long long first_image;
        if (a.phase_on_m) {  // images of a group: [phase][tile of the phase][channel block][tap of the phase]
          const int phase = (int)a.div_tiles_pp.div((uint32_t)tc_.m_tile), in_phase = tc_.m_tile - phase * a.tiles_pp;
          const int t0 = ctrl->tap_start[phase], ntap = ctrl->tap_start[phase + 1] - t0;
          first_image = ((group * a.tt.taps_total + t0) * a.tiles_pp + (long long)in_phase * ntap) * a.cb_per_phase;
        } else {
          first_image = (group * a.tiles_m + tc_.m_tile) * a.images_per_tile;
        }
        // images are ordered [channel block][tap of the phase]: the two taps of a ring stage are adjacent in memory,
        // and a block with an odd tap count ends with a stage of one image
        const unsigned char* img = reinterpret_cast<const unsigned char*>(a.wp) + first_image * (long long)W_STAGE_BYTES;
        int phase = a.phase_on_m ? (int)a.div_tiles_pp.div((uint32_t)tc_.m_tile) : 0, cbl = 0;
        for (int cb = 0; cb < a.cblocks && alive; ++cb) {
          const int ntap = ctrl->tap_start[phase + 1] - ctrl->tap_start[phase];
          for (int tap = 0; tap < ntap; tap += 2) {
            const uint32_t bytes = tap + 1 < ntap ? W_RING_BYTES : W_STAGE_BYTES;
            if (!mbar_wait(smem_u32(&ctrl->w_empty[ws]), w_par, abort_flag, a.status, STATUS_TIMEOUT_EMPTY)) { alive = false; break; }
            const uint32_t full = smem_u32(&ctrl->w_full[ws]);
            mbar_expect_tx(full, bytes);
            bulk_g2s(w_base + ws * W_RING_BYTES, img, bytes, full);
            ++issued;
            if (++ws == (uint32_t)a.w_stages) { ws = 0; w_par ^= 1; }
            img += bytes;
          }
          if (!a.phase_on_m && ++cbl == a.cb_per_phase) { cbl = 0; ++phase; }
        }
      }
      // after an abort nobody consumes the stages: wait (bounded) for the copies still in flight
      if (!alive)
        for (uint32_t j = issued > (uint32_t)a.w_stages ? issued - a.w_stages : 0; j < issued; ++j)
          mbar_wait(smem_u32(&ctrl->w_full[j % a.w_stages]), (j / a.w_stages) & 1, nullptr, a.status, STATUS_TIMEOUT_FULL);
    }
  } else if (warp >= EPI_WARPS) {
    // ------------------------------ strip producers ------------------------------
    // A stage is staged as chunks of 32 rows, one warp per chunk; chunk c of stage n goes to warp
    // (n*chunks + c) % 8, so short strips keep several stages in flight.
    const int aw = warp - EPI_WARPS;
    const int chunks = (a.strip_rows + 31) / 32;
    const bool vec_layout = a.act.s1 == 1 && a.kc % 4 == 0 && ((reinterpret_cast<uintptr_t>(a.act.ptr) & 15) == 0) &&
                            (a.act.s0 % 4 == 0) && (a.act.s2 % 4 == 0) && (a.act.s3 % 4 == 0);
    const int s1 = (int)a.act.s1;
    const int total_jobs = my_tiles * a.cblocks * chunks;  // below 2^31 (checked by the host)
    // consecutive jobs of a warp stay within a_stages stages of each other (a waiter that skipped a whole
    // phase of a stage's mbarrier would see the parity of an older phase and run ahead)
    const int a_warps = min(A_WARPS, chunks * a.a_stages);
    for (int job = aw; job < total_jobs && aw < a_warps; job += a_warps) {
      const uint32_t a_count = a.div_chunks.div((uint32_t)job);
      const int chunk = job - (int)a_count * chunks;
      const uint32_t tile_iter = a.div_cblocks.div(a_count);
      const int cb = (int)(a_count - tile_iter * a.cblocks);
      const TileCoord tc_ = tile_coord(a, (int)(blockIdx.x + tile_iter * gridDim.x));
      const uint32_t a_round = a.div_a_stages.div(a_count);
      const uint32_t as = a_count - a_round * a.a_stages;
      const int phase = a.phase_on_m ? 0 : (int)a.div_cbpp.div((uint32_t)cb), cbl = cb - phase * a.cb_per_phase;
      const int nvalid = min(KB, a.kc - cbl * KB);
      const bool chunked = vec_layout && nvalid == KB;   // channels-last: four lanes fetch the 64 bytes of a pixel
      const int q0 = tc_.p_tile * a.pn - a.halo + chunk * 32;
      float v[KB];
      // row -> address of its first channel (0 = the row is padding)
      const float* src = nullptr;
      {
        const int r = chunk * 32 + lane, q = q0 + lane;
        if (r < a.strip_rows && q >= 0 && q < a.q_total) {
          const int n = (int)a.img_div.div((uint32_t)q);
          const int rem = q - n * img_pitch;
          const int y = (int)a.row_div.div((uint32_t)rem), x = rem - y * row_pitch;
          const int iy = a.phase_on_m ? y : y * a.sph + ctrl->ph_a[phase], ix = a.phase_on_m ? x : x * a.spw + ctrl->ph_b[phase];
          if (y < a.H && x < a.W && iy < a.act_h && ix < a.act_w)
            src = a.act.ptr + n * a.act.s0 + ((long long)tc_.group * a.kc + cbl * KB) * a.act.s1 + (long long)iy * a.act.s2 +
                  (long long)ix * a.act.s3;
        }
      }
      if (chunked) {
        // load i covers rows 8i .. 8i+7: lane -> (row 8i + lane/4, 16-byte piece lane%4)
        const unsigned long long mine = reinterpret_cast<unsigned long long>(src);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4* ps = reinterpret_cast<const float4*>(__shfl_sync(0xffffffffu, mine, 8 * i + (lane >> 2)));
          const float4 f = ps ? __ldg(ps + (lane & 3)) : make_float4(0.f, 0.f, 0.f, 0.f);
          v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < KB; ++j) v[j] = (src && j < nvalid) ? __ldg(src + j * s1) : 0.f;
      }
      if (!mbar_wait(smem_u32(&ctrl->a_empty[as]), (a_round & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_EMPTY)) break;
      const uint32_t p_hi = tiles_base + as * a_stage_bytes, p_cr = p_hi + a_plane;
      if (chunked) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = chunk * 32 + 8 * i + (lane >> 2);   // strip_rows is a multiple of 8
          if (r < a.strip_rows) {
            float h[4], l[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) split_tf32_fast(v[4 * i + j], h[j], l[j]);
            const int c = lane & 3;  // this lane's four channels: 4c .. 4c+3
            sts_f32x4(p_hi + sw64_chunk(r, c), h[0], h[1], h[2], h[3]);
            // cross plane: bf16(hi) of channels 0-15 in pieces 0-1, bf16(lo) in pieces 2-3; four values are 8 bytes
            sts_b32x2(p_cr + sw64_chunk(r, c >> 1) + (uint32_t)((c & 1) * 8), pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]));
            sts_b32x2(p_cr + sw64_chunk(r, 2 + (c >> 1)) + (uint32_t)((c & 1) * 8), pack_bf16x2(l[0], l[1]), pack_bf16x2(l[2], l[3]));
          }
        }
      } else {
        const int r = chunk * 32 + lane;
        if (r < a.strip_rows) {
          float h[KB], l[KB];
#pragma unroll
          for (int j = 0; j < KB; ++j) split_tf32_fast(v[j], h[j], l[j]);
#pragma unroll
          for (int c = 0; c < 4; ++c) sts_f32x4(p_hi + sw64_chunk(r, c), h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            sts_b32x4(p_cr + sw64_chunk(r, c), pack_bf16x2(h[8 * c], h[8 * c + 1]), pack_bf16x2(h[8 * c + 2], h[8 * c + 3]),
                      pack_bf16x2(h[8 * c + 4], h[8 * c + 5]), pack_bf16x2(h[8 * c + 6], h[8 * c + 7]));
            sts_b32x4(p_cr + sw64_chunk(r, 2 + c), pack_bf16x2(l[8 * c], l[8 * c + 1]), pack_bf16x2(l[8 * c + 2], l[8 * c + 3]),
                      pack_bf16x2(l[8 * c + 4], l[8 * c + 5]), pack_bf16x2(l[8 * c + 6], l[8 * c + 7]));
          }
        }
      }
      fence_proxy_async();
      mbar_arrive(smem_u32(&ctrl->a_full[as]));
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    // Warp w owns accumulator lanes 32w .. 32w+31 (output channels).  tcgen05.ld hands thread = channel its 32
    // consecutive pixels; a 32x33 shared-memory tile turns that into thread = pixel, so that each store
    // instruction writes 32 consecutive pixels of one channel plane.
    float* tb = reinterpret_cast<float*>(smem_raw + (tbuf_base - raw)) + warp * (32 * 33);
    for (int t = 0; t < my_tiles; ++t) {
      const TileCoord tc_ = tile_coord(a, (int)blockIdx.x + t * (int)gridDim.x);
      const int phase_m = a.phase_on_m ? (int)a.div_tiles_pp.div((uint32_t)tc_.m_tile) : 0;
      const int c0 = (tc_.m_tile - phase_m * a.tiles_pp) * TM + warp * 32;   // first channel (within the group) of this warp
      const int nch = min(32, a.nc - c0);                                       // channels of this warp that exist (may be <= 0)
      const uint32_t ab = (uint32_t)t & 1u;
      const bool has_taps = !a.phase_on_m || ctrl->tap_start[phase_m + 1] > ctrl->tap_start[phase_m];
      float bv = 0.f;  // lane j holds the bias of channel c0 + j
      if (a.bias && lane < nch) bv = __ldg(a.bias + ((long long)tc_.group * a.nc + c0 + lane) * a.bias_stride);
      if (!mbar_wait(smem_u32(&ctrl->acc_full[ab]), ((uint32_t)t >> 1) & 1u, abort_flag, a.status, STATUS_TIMEOUT_ACCUM)) break;
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + ab * ACC_COLS + ((uint32_t)(warp * 32) << 16);
      const int q_tile = tc_.p_tile * a.pn;
      const int cols = min(a.pn, a.q_total - q_tile);
      const int nchunks = (cols + 31) / 32;
      const long long plane = (long long)a.out_h * a.out_w;
      const long long te__ = (B200_ROLE_PROFILE && a.prof && blockIdx.x == 0 && threadIdx.x == 0) ? clock64() : 0;
      if (B200_ROLE_PROFILE && a.prof && blockIdx.x == 0 && threadIdx.x == 0) a.prof[10] = (unsigned long long)(te__ - prof_c0);
#pragma unroll 1
      for (int ch = 0; ch < nchunks; ++ch) {
        float v[32];
        tmem_ld32(tmem_acc + (uint32_t)(ch * 32), v);
        if (ch + 1 == nchunks) {  // last read of this accumulator: hand it back
          tc_fence_before();
          mbar_arrive(smem_u32(&ctrl->acc_empty[ab]));
        }
        if (nch <= 0) continue;
        // this lane's pixel of the chunk
        const int q = q_tile + ch * 32 + lane;
        bool ok = ch * 32 + lane < cols;
        long long obase = 0;
        if (ok) {
          const long long n = a.img_div.div((uint32_t)q);
          const int rem = q - (int)n * img_pitch;
          int y = (int)a.row_div.div((uint32_t)rem), x = rem - y * row_pitch;
          ok = y < a.H && x < a.W;
          if (a.phase_on_m) { y = y * a.osh + ctrl->ph_a[phase_m]; x = x * a.osw + ctrl->ph_b[phase_m]; }
          ok = ok && y < a.out_h && x < a.out_w;
          obase = ((n * a.out_channels + (long long)tc_.group * a.nc + c0) * a.out_h + y) * a.out_w + x;
        }
        __syncwarp();   // the previous chunk's reads of the tile are done
#pragma unroll
        for (int j = 0; j < 32; ++j) tb[lane * 33 + j] = has_taps ? v[j] : 0.f;   // [channel][pixel]
        __syncwarp();
        // every lane takes part in the shuffles (a pixel on padding only skips its stores)
        float* p = a.out + obase;
        if (nch == 32) {
#pragma unroll
          for (int c = 0; c < 32; ++c, p += plane) {
            const float val = tb[c * 33 + lane] + __shfl_sync(0xffffffffu, bv, c);
            if (ok) *p = val;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c, p += plane) {
            const float val = tb[c * 33 + lane] + __shfl_sync(0xffffffffu, bv, c);
            if (ok && c < nch) *p = val;
          }
        }
      }
      if (B200_ROLE_PROFILE && a.prof && blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(a.prof + 6, (unsigned long long)(clock64() - te__));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (B200_ROLE_PROFILE && a.prof && blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(a.prof + 5, (unsigned long long)(clock64() - prof_c0));
}

// Split W[cout][cin/g][kh][kw] (any strides) into TF32 hi / BF16 cross parts laid out as the shared-memory
// images the MMA reads: image = [hi: 128 rows x 64 B, SWIZZLE_64B][cross: same], row = output channel of the
// tile (forward: co, dInput: ci; zero beyond nc), 16 reduction channels per row.  Images are ordered as the
// main loop consumes them: forward [group][channel tile][phase][channel block][tap of the phase], dInput
// [group][phase][channel tile of the phase][channel block][tap of the phase].  One thread per four channels.
__global__ void __launch_bounds__(256) stage_filter16_kernel(ConvGeom g, View4 w, int is_dx, int tiles_pp, TapTable tt,
                                                             unsigned char* __restrict__ out, long long total) {
  asm volatile("griddepcontrol.launch_dependents;");
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= total) return;
  const int kc = is_dx ? g.cog : g.cig, nc = is_dx ? g.cig : g.cog;
  const int cpp = (kc + KB - 1) / KB;
  const int piece = (int)(i % 4), k = piece * 4;
  const int row = (int)((i / 4) % TM);
  const long long image = i / (4ll * TM);
  int grp, m_tile, cbl, tap;
  if (is_dx) {
    const int per_group = tiles_pp * cpp * tt.taps_total;
    grp = (int)(image / per_group);
    const int local = (int)(image - (long long)grp * per_group);
    int phase = 0;
    while (phase + 1 < tt.n_phase && local >= tiles_pp * cpp * tt.start[phase + 1]) ++phase;
    const int rel = local - tiles_pp * cpp * tt.start[phase], ntap = tt.start[phase + 1] - tt.start[phase];
    m_tile = rel / (cpp * ntap);
    const int rel2 = rel - m_tile * cpp * ntap;
    cbl = rel2 / ntap;
    tap = tt.start[phase] + rel2 % ntap;
  } else {
    const int per_tile = cpp * tt.taps_total;
    const int local = (int)(image % per_tile);
    m_tile = (int)((image / per_tile) % tiles_pp);
    grp = (int)(image / ((long long)per_tile * tiles_pp));
    int phase = 0;
    while (phase + 1 < tt.n_phase && local >= cpp * tt.start[phase + 1]) ++phase;
    const int rel = local - cpp * tt.start[phase], ntap = tt.start[phase + 1] - tt.start[phase];
    cbl = rel / ntap;
    tap = tt.start[phase] + rel % ntap;
  }
  const int r = m_tile * TM + row, c = cbl * KB + k;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (r < nc) {
    const long long step = is_dx ? w.s0 : w.s1;
    const float* src = w.ptr + ((long long)grp * g.cog + (is_dx ? c : r)) * w.s0 + (long long)(is_dx ? r : c) * w.s1 +
                       tt.ky[tap] * w.s2 + tt.kx[tap] * w.s3;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (c + j < kc) v[j] = __ldg(src + j * step);
  }
  float hi[4], lo[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) split_tf32(v[j], hi[j], lo[j]);
  unsigned char* img = out + image * (long long)W_STAGE_BYTES;
  *reinterpret_cast<float4*>(img + sw64_chunk(row, piece)) = make_float4(hi[0], hi[1], hi[2], hi[3]);
  unsigned char* cross = img + TM * ROWB;   // [bf16(lo) x16 | bf16(hi) x16], pairing with the activations' [hi | lo]
  *reinterpret_cast<uint2*>(cross + sw64_chunk(row, piece >> 1) + (piece & 1) * 8) = make_uint2(pack_bf16x2(lo[0], lo[1]), pack_bf16x2(lo[2], lo[3]));
  *reinterpret_cast<uint2*>(cross + sw64_chunk(row, 2 + (piece >> 1)) + (piece & 1) * 8) = make_uint2(pack_bf16x2(hi[0], hi[1]), pack_bf16x2(hi[2], hi[3]));
}

struct TPlan {
  bool ok = false;
  StripPlan geo;
  int pn = 0, strip_rows = 0, a_stages = 0, w_stages = 0, smem = 0;
  int tiles_pp = 0, tiles_m = 0, tiles_p = 0, cpp = 0;
  long long images = 0;   // filter stage images in total
};

// Clocks of one tcgen05.mma of 128 x pn x 8 (TF32) or x 16 (BF16): the tensor pipe needs pn / 2, the
// shared-memory operand read (4 KB of filter + 32 B per pixel) about 96 bytes per clock.
static double mma_clocks(int pn) { return std::max(pn / 2.0, (4096.0 + 32.0 * pn) / 96.0); }

// The pixel tile is the free parameter: wide tiles use the tensor pipe best, but the tile count should fill whole
// waves of SMs.  Modelled time = waves x (MMAs of a tile x clocks(pn) + a fixed cost per tile).
static TPlan plan_tstrip(const ConvGeom& g, bool is_dx) {
  TPlan p;
  p.geo = tcs::plan_strip_geometry(g, is_dx);
  if (!p.geo.ok) return p;
  const int kc = is_dx ? g.cog : g.cig, nc = is_dx ? g.cig : g.cog;
  const TapTable& tt = p.geo.tt;
  p.cpp = (kc + KB - 1) / KB;
  p.tiles_pp = (nc + TM - 1) / TM;
  p.tiles_m = is_dx ? p.tiles_pp * tt.n_phase : p.tiles_pp;
  p.images = (long long)g.groups * p.tiles_pp * p.cpp * tt.taps_total;
  const long long q_total = (long long)g.n * (p.geo.gh + p.geo.pr) * (p.geo.gw + p.geo.pc);
  // MMAs of one tile: forward runs every tap of every channel block, dInput the taps of the tile's phase (average)
  const double stages_per_tile = is_dx ? (double)p.cpp * tt.taps_total / std::max(1, tt.n_phase) : (double)p.cpp * tt.taps_total;
  const int span = p.geo.shift_hi - p.geo.shift_lo;
  double best = 0.0;
  int pn_hi = 256, pn_lo = 32;
  if (const char* e = getenv("B200_TSTRIP_PN")) pn_hi = pn_lo = std::max(16, std::min(256, atoi(e) / 16 * 16));  // testing aid
  for (int pn = pn_hi; pn >= pn_lo; pn -= 16) {
    const int rows = (pn + span + 7) / 8 * 8;
    const int a_stage = rows * ROWB * 2;
    int a_stages = 0, w_stages = 0;
    for (int as : {3, 2}) {
      const int left = SMEM_LIMIT - TBUF_BYTES - 1024 - (int)sizeof(Ctrl) - as * a_stage;
      if (left >= 2 * (int)W_RING_BYTES) { a_stages = as; w_stages = std::min(MAX_W_STAGES, left / (int)W_RING_BYTES); break; }
    }
    if (!a_stages) continue;
    const long long tiles = div_up64(q_total, pn) * p.tiles_m * g.groups;
    const double cost = (double)div_up64(tiles, sm_count()) * (stages_per_tile * (4.0 * mma_clocks(pn) + 120.0) + 3000.0);
    if (!p.ok || cost < best * 0.995) {   // ties go to the wider tile (fewer filter bytes per output)
      best = cost;
      p.ok = true;
      p.pn = pn; p.strip_rows = rows; p.a_stages = a_stages; p.w_stages = w_stages;
      p.tiles_p = (int)div_up64(q_total, pn);
      p.smem = a_stages * a_stage + w_stages * (int)W_RING_BYTES + TBUF_BYTES + 1024 + (int)sizeof(Ctrl) + 64;
    }
  }
  if (p.ok && (long long)p.tiles_p * p.tiles_m * g.groups * p.cpp * ((p.strip_rows + 31) / 32) > 2147483647ll - (1 << 20)) p.ok = false;
  return p;
}

}  // namespace tst

// The transposed arrangement pays when most of the 128 filter rows of a tile are real output channels.
bool tstrip_supported(const ConvGeom& g, int phase) {
  if (phase != B200_PHASE_FORWARD && phase != B200_PHASE_DINPUT) return false;
  const bool is_dx = phase == B200_PHASE_DINPUT;
  const int nc = is_dx ? g.cig : g.cog;
  const int last = nc % tst::TM;
  int least = 65;
  if (const char* e = getenv("B200_TSTRIP_MIN")) least = std::max(16, atoi(e));  // testing aid
  if (nc < least || (last != 0 && last < least && nc < 4 * tst::TM)) return false;   // at most a quarter of the rows may be padding
  // a 1x1 filter is bound by HBM and by the epilogue, not by the MMAs, and a strided dInput splits into phases of two
  // or three taps each: both keep the arrangement with pixels on M, whose epilogue stores straight from registers
  if (g.kh * g.kw < 4 || (is_dx && (g.sh > 1 || g.sw > 1))) return false;
  if (const char* v = getenv("B200_CONV_TC_VARIANT")) {
    if (!strcmp(v, "strip") || !strcmp(v, "gather")) return false;
  }
  return tst::plan_tstrip(g, is_dx).ok;
}
size_t tstrip_workspace(const ConvGeom& g, int phase) {
  const tst::TPlan p = tst::plan_tstrip(g, phase == B200_PHASE_DINPUT);
  return p.ok ? (size_t)p.images * tst::W_STAGE_BYTES : 0;
}

int tstrip_conv(const ConvGeom& g, bool is_dx, View4 act, View4 w, const float* bias, long long bias_stride, float* out,
                void* ws, size_t ws_bytes, cudaStream_t st) {
  using namespace tst;
  const TPlan plan = plan_tstrip(g, is_dx);
  if (!plan.ok) return fail(B200_EUNSUPPORTED, "transposed strip kernel does not take this geometry");
  const size_t need = (size_t)plan.images * W_STAGE_BYTES;
  if (!ws || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 15))
    return fail(B200_EWORKSPACE, "tcgen05 convolution needs a 16-byte aligned workspace of %zu bytes (got %zu)", need, ws_bytes);
  const int kc = is_dx ? g.cog : g.cig, nc = is_dx ? g.cig : g.cog;
  const long long pieces = plan.images * TM * 4;
  stage_filter16_kernel<<<(unsigned)div_up64(pieces, 256), 256, 0, st>>>(g, w, is_dx ? 1 : 0, plan.tiles_pp, plan.geo.tt,
                                                                         (unsigned char*)ws, pieces);
  count_launch();
  if (int rc = launch_check("stage_filter16_kernel")) return rc;

  TArgs a{};
  a.g = g; a.act = act; a.wp = (const float*)ws; a.bias = bias; a.bias_stride = bias_stride; a.out = out;
  a.H = plan.geo.gh; a.W = plan.geo.gw; a.pr = plan.geo.pr; a.pc = plan.geo.pc;
  a.act_h = plan.geo.act_h; a.act_w = plan.geo.act_w; a.out_h = plan.geo.out_h; a.out_w = plan.geo.out_w;
  a.sph = is_dx ? 1 : plan.geo.sph; a.spw = is_dx ? 1 : plan.geo.spw;
  a.osh = is_dx ? plan.geo.sph : 1; a.osw = is_dx ? plan.geo.spw : 1;
  a.phase_on_m = is_dx ? 1 : 0;
  a.tiles_pp = plan.tiles_pp;
  a.tt = plan.geo.tt;
  a.kc = kc; a.nc = nc;
  a.out_channels = is_dx ? g.cin : g.cout;
  a.cb_per_phase = plan.cpp;
  a.cblocks = (is_dx ? 1 : plan.geo.tt.n_phase) * plan.cpp;
  a.images_per_tile = plan.cpp * plan.geo.tt.taps_total;
  a.tiles_m = plan.tiles_m; a.tiles_p = plan.tiles_p;
  a.tiles_total = plan.tiles_p * plan.tiles_m * g.groups;
  a.pn = plan.pn;
  a.q_total = (int)((long long)g.n * (a.H + a.pr) * (a.W + a.pc));
  a.img_div = FastDiv((uint32_t)((a.H + a.pr) * (a.W + a.pc)));
  a.row_div = FastDiv((uint32_t)(a.W + a.pc));
  a.halo = plan.geo.halo; a.strip_rows = plan.strip_rows; a.a_stages = plan.a_stages; a.w_stages = plan.w_stages;
  const int chunks = (a.strip_rows + 31) / 32;
  a.div_tiles_p = FastDiv((uint32_t)a.tiles_p); a.div_tiles_m = FastDiv((uint32_t)a.tiles_m);
  a.div_tiles_pp = FastDiv((uint32_t)a.tiles_pp); a.div_chunks = FastDiv((uint32_t)chunks);
  a.div_cblocks = FastDiv((uint32_t)a.cblocks); a.div_cbpp = FastDiv((uint32_t)a.cb_per_phase);
  a.div_a_stages = FastDiv((uint32_t)a.a_stages);
  a.wait_for_images = 1;
  a.status = device_status_word();
  if (!a.status) return fail(B200_ECUDA, "device status word is not allocated");
  static unsigned long long* prof_buf = nullptr;
  const char* prof_env = getenv("B200_STRIP_PROFILE");
  const bool profiling = B200_ROLE_PROFILE && prof_env && prof_env[0] == '1';
  if (profiling) {
    if (!prof_buf) B200_CUDA(cudaMalloc(&prof_buf, 16 * sizeof(unsigned long long)));
    B200_CUDA(cudaMemsetAsync(prof_buf, 0, 16 * sizeof(unsigned long long), st));
    a.prof = prof_buf;
  }

  static std::once_flag once;
  static cudaError_t opt_in = cudaSuccess;
  std::call_once(once, [] {
    opt_in = cudaFuncSetAttribute(conv_tstrip_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (opt_in == cudaSuccess) opt_in = cudaFuncSetAttribute(conv_tstrip_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
  });
  B200_CUDA(opt_in);
  // A strided forward pass stages one strip per input phase and gets only one to four taps of MMAs out of it (a
  // stride-1 strip feeds all nine): the producers set the pace, so sixteen run (128 -> 128 channels, 56x56 stride 2:
  // 87 -> 81 us NCHW, 94 -> 73 us channels-last; stride-1 layers are unchanged either way).  B200_TSTRIP_PRODUCERS=8|16 pins it.
  bool wide = !is_dx && (g.sh > 1 || g.sw > 1);
  if (const char* e = getenv("B200_TSTRIP_PRODUCERS")) wide = atoi(e) == 16;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)std::min(a.tiles_total, sm_count())); cfg.blockDim = dim3(tstrip_threads(wide ? 16 : 8));
  cfg.dynamicSmemBytes = (size_t)plan.smem; cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  if (wide) B200_CUDA(cudaLaunchKernelEx(&cfg, conv_tstrip_kernel<16>, a));
  else B200_CUDA(cudaLaunchKernelEx(&cfg, conv_tstrip_kernel<8>, a));
  count_launch();
  if (profiling) {
    unsigned long long h[16];
    B200_CUDA(cudaStreamSynchronize(st));
    B200_CUDA(cudaMemcpy(h, prof_buf, sizeof h, cudaMemcpyDeviceToHost));
    fprintf(stderr, "[tstrip profile, CTA 0, cycles] pn=%d rows=%d a_stages=%d w_stages=%d tiles=%d (m %d x p %d) cblocks=%d | CTA %llu | mma: wait_acc %llu wait_strip %llu "
            "wait_filter %llu issue %llu over %llu stages | epilogue (all tiles) %llu | since CTA start: MMA loop begins %llu ends %llu, last epilogue begins %llu\n",
            a.pn, a.strip_rows, a.a_stages, a.w_stages, a.tiles_total, a.tiles_m, a.tiles_p, a.cblocks, h[5], h[0], h[1], h[2], h[3], h[4], h[6], h[8], h[9], h[10]);
  }
  return launch_check("conv_tstrip_kernel");
}

}  // namespace b200
