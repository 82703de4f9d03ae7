// Planner pieces shared by the two tcgen05 strip kernels (conv_tc_strip.cu, conv_tc_tstrip.cu): the padded pixel
// grid, the filter taps grouped by stride phase, and the row shifts that turn a tap into a descriptor offset.
#pragma once
#include "common.cuh"

namespace b200 {
namespace tcs {

constexpr int MAX_TAPS = 64, MAX_PHASES = 16;

// Filter taps grouped by the input phase they read.  With stride s the input row of output row oy
// and tap ky is s*oy + ky*d - pad = s*(oy + dr) + a with a = (ky*d - pad) mod s: tap ky reads the
// sub-image made of rows = a (mod s) ("phase a") at the whole-pixel offset dr.  Channel blocks are
// therefore enumerated per phase, and each phase runs only its own taps (stride 1: one phase, all taps).
struct TapTable {
  int n_phase = 0, taps_total = 0;
  unsigned char a[MAX_PHASES], b[MAX_PHASES];  // row / column phase of active phase i
  unsigned char start[MAX_PHASES + 1];         // taps of phase i: [start[i], start[i+1])
  unsigned char ky[MAX_TAPS], kx[MAX_TAPS];    // filter position of tap t
  int shift[MAX_TAPS];                         // strip row offset of tap t
};

struct StripPlan {
  bool ok = false;
  int bn = 0, a_stages = 0, w_stages = 0, strip_rows = 0, halo = 0, smem = 0;
  int gh = 0, gw = 0, pr = 0, pc = 0;  // pixel grid and its padding
  int act_h = 0, act_w = 0, out_h = 0, out_w = 0, sph = 1, spw = 1;
  int shift_lo = 0, shift_hi = 0;      // smallest / largest tap row shift (strip rows before / after a tile's pixels)
  TapTable tt;
};

// Geometry part of the plan (grid, padding, tap table, shifts); `ok` is false when the strip kernels do not take it.
StripPlan plan_strip_geometry(const ConvGeom& g, bool is_dx);

}  // namespace tcs
}  // namespace b200
