// C-ABI entry points of the convolution / GEMM path: geometry validation, candidate
// selection, workspace planning and dispatch to the kernel families.
//
// Host logic restated from the reference (paths inside the reference tree):
//   convolution_params            csrc/ops/convolution.cpp:101-156
//   dispatch element-count guards csrc/ops/convolution.cpp:559-560
//   applicable/candidates         csrc/ops/convolution.cpp:357-401
//   heuristic                     csrc/ops/convolution.cpp:423-482
//   weight_split_plan             csrc/ops/convolution.cpp:204-238
// The tile menu of the reference (base/wide/tall/register...) is a property of its GLSL
// shaders; here the candidates are direct / tiled (CUDA cores) / tc (tcgen05) / winograd.
#include "common.cuh"

#include <algorithm>
#include <climits>

namespace b200 {

struct SplitPlan {
  int splits = 1;
  int span = 0;
  size_t bytes = 0;
};

// Split-K plan of the CUDA-core dWeight kernel.  Like the reference's plan it never exceeds
// the caller's budget and keeps spans aligned to the K tile (16); unlike it, the number of
// partials is chosen to fill the machine (about four CTAs per SM) rather than fixed at 256
// positions, because on 148 SMs a 98-way split of a 147 KB gradient costs more in scratch
// traffic than it buys in parallelism.
static SplitPlan simt_dweight_plan(const ConvGeom& g, size_t budget) {
  SplitPlan plan;
  const long long positions = (long long)g.n * g.oh * g.ow;
  const long long cols = (long long)g.cig * g.kh * g.kw;
  const long long tiles = div_up64(cols, 64) * div_up64(g.cog, 64) * g.groups;
  const size_t dw_bytes = (size_t)g.cout * cols * sizeof(float);
  long long want = std::max<long long>(1, div_up64(4ll * std::max(1, sm_count()), tiles));
  want = std::min<long long>(want, div_up64(positions, 256));
  want = std::min<long long>(want, 65535);
  if (dw_bytes) want = std::min<long long>(want, (long long)(budget / dw_bytes));
  if (want < 2) {
    plan.span = (int)positions;
    return plan;
  }
  const long long span = div_up64(div_up64(positions, want), 16) * 16;
  plan.span = (int)span;
  plan.splits = (int)div_up64(positions, span);
  plan.bytes = plan.splits > 1 ? (size_t)plan.splits * dw_bytes : 0;
  return plan;
}

static int dbias_slabs(const ConvGeom& g, View4 dy, size_t budget) {
  const bool channels_inner = dy.s1 == 1 && dy.s3 != 1;
  const long long ctas = channels_inner ? div_up64(g.cout, 32) : g.cout;
  long long slabs = div_up64(4ll * std::max(1, sm_count()), ctas);
  // channels-last: a CTA pass covers 32 pixels, give every slab at least eight passes;
  // planes: a warp takes an image, a CTA eight of them
  const long long limit = channels_inner ? div_up64((long long)g.n * g.oh * g.ow, 256) : div_up64(g.n, 8);
  slabs = std::max<long long>(1, std::min<long long>(slabs, limit));
  slabs = std::min<long long>(slabs, (long long)(budget / (sizeof(float) * g.cout)));
  return (int)std::max<long long>(1, slabs);
}

static int check_params(const b200_conv_params* p) {
  if (!p) return fail(B200_EINVAL, "null convolution parameters");
  if (!(p->n > 0 && p->cin > 0 && p->cout > 0 && p->h > 0 && p->w > 0 && p->kh > 0 && p->kw > 0 && p->oh > 0 &&
        p->ow > 0 && p->sh > 0 && p->sw > 0 && p->dh > 0 && p->dw > 0 && p->ph >= 0 && p->pw >= 0 &&
        p->groups > 0 && p->cin % p->groups == 0 && p->cout % p->groups == 0))
    return fail(B200_EINVAL, "convolution: invalid shapes or parameters");
  return B200_OK;
}

// Returns the candidate to run, or a negative code when a forced one is not applicable.
static int select(const ConvGeom& g, int phase, int algo, size_t workspace) {
  const long long rows = (long long)g.n * g.oh * g.ow, cols = (long long)g.cig * g.kh * g.kw;
  if (phase == B200_PHASE_DBIAS) return algo == B200_ALGO_DIRECT ? B200_ALGO_DIRECT : B200_ALGO_TILED;
  switch (algo) {
    case B200_ALGO_DIRECT:
    case B200_ALGO_TILED:
      return algo;
    case B200_ALGO_TC:
      if (!tc_supported(g, phase))
        return fail(B200_EUNSUPPORTED, "forced tcgen05 candidate is incompatible with this geometry");
      return algo;
    case B200_ALGO_WINOGRAD:
      if (!winograd_supported(g, phase))
        return fail(B200_EUNSUPPORTED, "forced Winograd candidate is incompatible with this geometry or phase");
      return algo;
    case B200_ALGO_AUTO:
      break;
    default:
      return fail(B200_EINVAL, "unknown algorithm id %d", algo);
  }
  // Winograd F(4x4,3x3) runs three passes (input transform, 36 plane GEMMs, output transform) for 2.25x fewer multiplies;
  // it pays once both the channel contraction and the image are large.  Measured on 64 images, forward, microseconds,
  // direct tcgen05 kernel vs Winograd (NCHW; channels-last in brackets):
  //    512 ->  512 at  7x7     80 vs  78  (81 vs  83)     dInput  72 vs  85
  //    512 ->  512 at 14x14   177 vs 190 (177 vs 223)
  //    512 ->  512 at 28x28   697 vs 569 (704 vs 716)
  //   1024 -> 1024 at  7x7    230 vs 204 (229 vs 213)     dInput 215 vs 231
  //   1024 -> 1024 at 14x14   702 vs 550 (704 vs 639)
  //    256 ->  256 at 28x28   171 vs 227;  at 56x56  628 vs 805
  // so the rule is a product of both: 512 channels from 28x28, 1024 channels from 14x14.
  if ((phase == B200_PHASE_FORWARD || phase == B200_PHASE_DINPUT) && g.cig >= 512 && g.cog >= 512 &&
      (long long)g.cig * g.cog * g.oh * g.ow >= 512ll * 512 * 28 * 28 && winograd_supported(g, phase) &&
      winograd_workspace(g, phase, workspace) > 0)
    return B200_ALGO_WINOGRAD;
  // The tcgen05 forward / dInput kernels stage the split filter in the caller's workspace; a caller that
  // brings none (or too little) gets the CUDA-core kernels, which need no scratch.  dWeight runs unsplit
  // without a workspace.  (A forced B200_ALGO_TC keeps reporting the workspace error.)
  if (tc_supported(g, phase) &&
      (phase == B200_PHASE_DWEIGHT || tc_workspace(g, phase, workspace, nullptr, nullptr) <= workspace))
    return B200_ALGO_TC;
  // grouped 3x3 layers with 4 or 8 channels per group have kernels of their own behind the tiled candidate
  if (group_small_supported(g) && phase != B200_PHASE_DBIAS) return B200_ALGO_TILED;
  // Thresholds of the reference heuristic for leaving the one-thread-per-output kernels.
  if (phase == B200_PHASE_FORWARD) return (g.cog >= 8 && cols >= 16 && rows >= 32) ? B200_ALGO_TILED : B200_ALGO_DIRECT;
  if (phase == B200_PHASE_DINPUT)
    return (g.cig >= 2 && g.cog >= 8 && (long long)g.n * g.h * g.w >= 32) ? B200_ALGO_TILED : B200_ALGO_DIRECT;
  return rows >= 128 ? B200_ALGO_TILED : B200_ALGO_DIRECT;
}

// The automatic choice of Winograd is taken back for channels-last activations below 1024 channels: its input transform
// reads 6x6 patches of whole pixels and is slower there (measured, 512 channels, batch 32, forward, Winograd vs direct:
// 64x64 1869 vs ~1650 us, 33x33 599 vs ~485, 32x32 486 vs ~455; NCHW: 1322, 495, 374), while 1024 channels at 14x14 still
// win (639 vs 704 us).  Only where the direct tcgen05 kernel's stage images fit the workspace the caller brought.
static int reconsider_for_layout(const ConvGeom& g, int phase, int algo, int chosen, const b200_view4& act, size_t workspace) {
  if (algo != B200_ALGO_AUTO || chosen != B200_ALGO_WINOGRAD) return chosen;
  const bool channels_last = act.stride[1] == 1 && (long long)g.cig * g.groups > 1 && act.stride[3] != 1;
  if (!channels_last || g.cig >= 1024 || !tc_supported(g, phase)) return chosen;
  return tc_workspace(g, phase, workspace, nullptr, nullptr) <= workspace ? B200_ALGO_TC : chosen;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_conv2d_geometry(b200_conv_params* out, int64_t n, int64_t cin, int64_t cout, int64_t h, int64_t w,
                         int64_t wcin, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                         int64_t dh, int64_t dw, int64_t groups) {
  if (!out) return fail(B200_EINVAL, "null output");
  if (!(n > 0 && cin > 0 && cout > 0 && h > 0 && w > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0 && dh > 0 &&
        dw > 0 && ph >= 0 && pw >= 0 && groups > 0 && cin % groups == 0 && cout % groups == 0 &&
        wcin == cin / groups))
    return fail(B200_EINVAL, "convolution: invalid shapes or parameters");
  for (int64_t v : {h, w, kh, kw, sh, sw, ph, pw, dh, dw})
    if (v > INT32_MAX) return fail(B200_ERANGE, "convolution: spatial parameters exceed int32 coordinates");
  if (dh * (kh - 1) > INT32_MAX || dw * (kw - 1) > INT32_MAX)
    return fail(B200_ERANGE, "convolution: effective filter exceeds int32 coordinates");
  if (!(h + 2 * ph >= dh * (kh - 1) + 1 && w + 2 * pw >= dw * (kw - 1) + 1))
    return fail(B200_EINVAL, "convolution: effective kernel exceeds padded input");
  const int64_t oh = (h + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
  const int64_t ow = (w + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
  if (!(oh > 0 && ow > 0)) return fail(B200_EINVAL, "convolution: empty output");
  if ((oh - 1) * sh + dh * (kh - 1) > INT32_MAX || (ow - 1) * sw + dw * (kw - 1) > INT32_MAX ||
      h - 1 + ph > INT32_MAX || w - 1 + pw > INT32_MAX)
    return fail(B200_ERANGE, "convolution: spatial indexing exceeds int32 coordinates");
  // Element counts of x, w, y must fit uint32 (the reference's shaders index with uint);
  // n, cin, cout themselves must fit int32 for the kernels here.
  const long double lim = 4294967295.0L;
  if ((long double)n * cin * h * w > lim || (long double)cout * wcin * kh * kw > lim ||
      (long double)n * cout * oh * ow > lim || n > INT32_MAX || cin > INT32_MAX || cout > INT32_MAX)
    return fail(B200_ERANGE, "convolution: input/weight/output indexing overflow");
  *out = {(int32_t)n, (int32_t)cin, (int32_t)cout, (int32_t)h, (int32_t)w, (int32_t)kh, (int32_t)kw,
          (int32_t)oh, (int32_t)ow, (int32_t)sh, (int32_t)sw, (int32_t)ph, (int32_t)pw, (int32_t)dh,
          (int32_t)dw, (int32_t)groups};
  return B200_OK;
}

int b200_conv2d_select(const b200_conv_params* p, int phase, int algo, size_t workspace_bytes) {
  if (int rc = check_params(p)) return rc;
  return select(to_geom(*p), phase, algo, workspace_bytes);
}

int b200_conv2d_tc_route(const b200_conv_params* p, int phase, b200_view4 act) {
  if (int rc = check_params(p)) return rc;
  if (phase != B200_PHASE_FORWARD && phase != B200_PHASE_DINPUT) return fail(B200_EINVAL, "tc_route: forward or dInput only");
  const ConvGeom g = to_geom(*p);
  if (!tc_supported(g, phase)) return fail(B200_EUNSUPPORTED, "tcgen05 candidate is incompatible with this geometry");
  return tc_route(g, phase == B200_PHASE_DINPUT, to_view(act));
}

size_t b200_conv2d_workspace(const b200_conv_params* p, int phase, int algo, size_t budget_bytes) {
  if (check_params(p) != B200_OK) return 0;
  const ConvGeom g = to_geom(*p);
  const int chosen = select(g, phase, algo, budget_bytes);
  if (chosen < 0) return 0;
  if (phase == B200_PHASE_DBIAS) {
    const int slabs = dbias_slabs(g, contiguous_view(nullptr, g.cout, g.oh, g.ow), budget_bytes);
    // channels-last gradients may want more slabs; reserve for the larger of the two layouts
    View4 cl{nullptr, (long long)g.oh * g.ow * g.cout, 1, (long long)g.ow * g.cout, g.cout};
    const int slabs_cl = dbias_slabs(g, cl, budget_bytes);
    const int s = std::max(slabs, slabs_cl);
    return s > 1 ? (size_t)s * g.cout * sizeof(float) : 0;
  }
  if (chosen == B200_ALGO_TC) return tc_workspace(g, phase, budget_bytes, nullptr, nullptr);
  if (chosen == B200_ALGO_WINOGRAD) return winograd_workspace(g, phase, budget_bytes);
  if (chosen == B200_ALGO_TILED && phase == B200_PHASE_DWEIGHT) {
    if (group_small_supported(g) && group_small_dweight_workspace(g) <= budget_bytes) return group_small_dweight_workspace(g);
    return simt_dweight_plan(g, budget_bytes).bytes;
  }
  return 0;
}

int b200_conv2d_forward(const b200_conv_params* p, b200_view4 x, b200_view4 w, const float* bias,
                        int64_t bias_stride, float* y, void* workspace, size_t workspace_bytes, int algo,
                        void* stream) {
  if (int rc = check_params(p)) return rc;
  if (int rc = ensure_init()) return rc;
  if (!x.ptr || !w.ptr || !y) return fail(B200_EINVAL, "convolution forward: null tensor");
  const ConvGeom g = to_geom(*p);
  int chosen = select(g, B200_PHASE_FORWARD, algo, workspace ? workspace_bytes : 0);
  if (chosen < 0) return chosen;
  chosen = reconsider_for_layout(g, B200_PHASE_FORWARD, algo, chosen, x, workspace ? workspace_bytes : 0);
  cudaStream_t st = (cudaStream_t)stream;
  if (!bias) bias_stride = 0;
  switch (chosen) {
    case B200_ALGO_WINOGRAD:
      note_kernel("winograd_f4_forward");
      return winograd_conv(g, false, to_view(x), to_view(w), bias, bias_stride, y, workspace, workspace_bytes, st);
    case B200_ALGO_TC:
      note_kernel("tc_igemm_forward");
      return tc_forward(g, to_view(x), to_view(w), bias, bias_stride, y, workspace, workspace_bytes, st);
    case B200_ALGO_TILED:
      if (group_small_supported(g)) {   // few channels per group: the tile follows the group (conv_group_small.cu)
        note_kernel("group_small_forward");
        return group_small_conv(g, false, to_view(x), to_view(w), bias, bias_stride, y, st);
      }
      note_kernel("simt_igemm_forward");
      return simt_igemm_forward(g, to_view(x), to_view(w), bias, bias_stride, y, st);
    default:
      note_kernel("direct_forward");
      return simt_direct(g, B200_PHASE_FORWARD, to_view(x), to_view(w), bias, bias_stride, y, st);
  }
}

int b200_conv2d_forward_fused(const b200_conv_params* p, b200_view4 x, b200_view4 w, const float* bias,
                              int64_t bias_stride, b200_view4 residual, int relu, float* y, int y_channels_last,
                              void* workspace, size_t workspace_bytes, int algo, void* stream) {
  if (int rc = check_params(p)) return rc;
  if (int rc = ensure_init()) return rc;
  if (!x.ptr || !w.ptr || !y) return fail(B200_EINVAL, "fused convolution forward: null tensor");
  if ((relu != 0 && relu != 1) || (y_channels_last != 0 && y_channels_last != 1))
    return fail(B200_EINVAL, "fused convolution forward: relu and y_channels_last must be 0 or 1");
  const ConvGeom g = to_geom(*p);
  const int chosen = select(g, B200_PHASE_FORWARD, algo, workspace ? workspace_bytes : 0);
  if (chosen < 0) return chosen;
  cudaStream_t st = (cudaStream_t)stream;
  if (!bias) bias_stride = 0;
  StripPostOps post;
  post.residual = to_view(residual);
  post.relu = relu;
  // the strip kernel applies everything in its epilogue and can write [pixel][channel] rows
  if (chosen == B200_ALGO_TC && strip_supported(g, B200_PHASE_FORWARD)) {
    note_kernel("tc_strip_forward_fused");
    const int rc = strip_conv(g, false, to_view(x), to_view(w), bias, bias_stride, y, workspace, workspace_bytes, st,
                              y_channels_last != 0, 1.f, 1.f, nullptr, &post);
    if (rc != B200_EUNSUPPORTED) return rc;
  }
  if (y_channels_last)
    return fail(B200_EUNSUPPORTED, "fused convolution forward: a channels-last result is incompatible with this "
                                   "geometry's candidate (needs the tcgen05 strip kernel)");
  // every other candidate: plain forward, then one elementwise pass over the contiguous result
  if (int rc = b200_conv2d_forward(p, x, w, bias, bias_stride, y, workspace, workspace_bytes, algo, stream)) return rc;
  return post_ops_nchw(y, g, post, st);
}

// dInput with an optional per-channel bias on the result (the forward pass of a transposed convolution).  The tensor-core and
// Winograd kernels add it in their epilogue; after the CUDA-core kernels it is one more pass over the result.
static int dinput_with_bias(const b200_conv_params* p, b200_view4 dy, b200_view4 w, const float* bias, int64_t bias_stride, float* dx,
                            void* workspace, size_t workspace_bytes, int algo, void* stream) {
  if (int rc = check_params(p)) return rc;
  if (int rc = ensure_init()) return rc;
  if (!dy.ptr || !w.ptr || !dx) return fail(B200_EINVAL, "convolution dInput: null tensor");
  const ConvGeom g = to_geom(*p);
  int chosen = select(g, B200_PHASE_DINPUT, algo, workspace ? workspace_bytes : 0);
  if (chosen < 0) return chosen;
  chosen = reconsider_for_layout(g, B200_PHASE_DINPUT, algo, chosen, dy, workspace ? workspace_bytes : 0);
  cudaStream_t st = (cudaStream_t)stream;
  bool bias_applied = false;
  int rc;
  switch (chosen) {
    case B200_ALGO_WINOGRAD:
      note_kernel("winograd_f4_dinput");
      rc = winograd_conv(g, true, to_view(dy), to_view(w), bias, bias_stride, dx, workspace, workspace_bytes, st);
      bias_applied = true;
      break;
    case B200_ALGO_TC:
      note_kernel("tc_igemm_dinput");
      rc = tc_dinput(g, to_view(dy), to_view(w), bias, bias_stride, dx, workspace, workspace_bytes, st, &bias_applied);
      break;
    case B200_ALGO_TILED:
      if (group_small_supported(g)) {
        note_kernel("group_small_dinput");
        rc = group_small_conv(g, true, to_view(dy), to_view(w), nullptr, 0, dx, st);
      } else {
        note_kernel("simt_igemm_dinput");
        rc = simt_igemm_dinput(g, to_view(dy), to_view(w), dx, st);
      }
      break;
    default:
      note_kernel("direct_dinput");
      rc = simt_direct(g, B200_PHASE_DINPUT, to_view(dy), to_view(w), nullptr, 0, dx, st);
  }
  if (rc || !bias || bias_applied) return rc;
  // the result has p's input extent: [n, cin, h, w]
  return bias_add_nchw(dx, p->n, p->cin, (long long)p->h * p->w, bias, bias_stride, st);
}

int b200_conv2d_dinput(const b200_conv_params* p, b200_view4 dy, b200_view4 w, float* dx, void* workspace,
                       size_t workspace_bytes, int algo, void* stream) {
  return dinput_with_bias(p, dy, w, nullptr, 0, dx, workspace, workspace_bytes, algo, stream);
}

int b200_conv_transpose2d_forward(const b200_conv_params* p, b200_view4 x, b200_view4 w, const float* bias,
                                  int64_t bias_stride, float* y, void* workspace, size_t workspace_bytes, int algo,
                                  void* stream) {
  // the transposed convolution of x is the input gradient of the convolution p describes
  return dinput_with_bias(p, x, w, bias, bias_stride, y, workspace, workspace_bytes, algo, stream);
}

int b200_conv2d_dweight(const b200_conv_params* p, b200_view4 x, b200_view4 dy, float* dw, void* workspace,
                        size_t workspace_bytes, int algo, void* stream) {
  if (int rc = check_params(p)) return rc;
  if (int rc = ensure_init()) return rc;
  if (!x.ptr || !dy.ptr || !dw) return fail(B200_EINVAL, "convolution dWeight: null tensor");
  const ConvGeom g = to_geom(*p);
  const int chosen = select(g, B200_PHASE_DWEIGHT, algo, workspace ? workspace_bytes : 0);
  if (chosen < 0) return chosen;
  cudaStream_t st = (cudaStream_t)stream;
  if (!workspace) workspace_bytes = 0;
  switch (chosen) {
    case B200_ALGO_TC:
      note_kernel("tc_igemm_dweight");
      return tc_dweight(g, to_view(x), to_view(dy), dw, workspace, workspace_bytes, st);
    case B200_ALGO_TILED: {
      if (group_small_supported(g) && workspace_bytes >= group_small_dweight_workspace(g)) {
        note_kernel("group_small_dweight");
        return group_small_dweight(g, to_view(x), to_view(dy), dw, (float*)workspace, workspace_bytes, st);
      }
      const SplitPlan plan = simt_dweight_plan(g, workspace_bytes);
      note_kernel(plan.splits > 1 ? "simt_igemm_dweight+finalize" : "simt_igemm_dweight");
      return simt_igemm_dweight(g, to_view(x), to_view(dy), dw, (float*)workspace, plan.splits, plan.span, st);
    }
    default:
      note_kernel("direct_dweight");
      return simt_direct(g, B200_PHASE_DWEIGHT, to_view(x), to_view(dy), nullptr, 0, dw, st);
  }
}

int b200_conv2d_dbias(const b200_conv_params* p, b200_view4 dy, float* db, void* workspace,
                      size_t workspace_bytes, void* stream) {
  if (int rc = check_params(p)) return rc;
  if (int rc = ensure_init()) return rc;
  if (!dy.ptr || !db) return fail(B200_EINVAL, "convolution dBias: null tensor");
  const ConvGeom g = to_geom(*p);
  if (!workspace) workspace_bytes = 0;
  const int slabs = dbias_slabs(g, to_view(dy), workspace_bytes);
  note_kernel(slabs > 1 ? "dbias_reduce+finalize" : "dbias_reduce");
  return dbias_reduce(g, to_view(dy), db, (float*)workspace, slabs, (cudaStream_t)stream);
}

int b200_device_status(int* status, int clear) {
  if (int rc = ensure_init()) return rc;
  B200_CUDA(cudaDeviceSynchronize());
  if (status)
    if (int rc = read_device_status(status)) return rc;
  if (clear) return clear_device_status();
  return B200_OK;
}

int b200_gemm(int64_t M, int64_t N, int64_t K, const float* A, int64_t sa0, int64_t sa1, const float* B,
              int64_t sb0, int64_t sb1, const float* bias, float alpha, float beta, float* C, int algo,
              void* stream) {
  if (int rc = ensure_init()) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(B200_EINVAL, "gemm: negative extent");
  if (M == 0 || N == 0) return B200_OK;
  if (M > UINT32_MAX || N > UINT32_MAX || K > UINT32_MAX) return fail(B200_ERANGE, "gemm: matrix too large");
  if (!C || (K > 0 && (!A || !B))) return fail(B200_EINVAL, "gemm: null matrix");
  cudaStream_t st = (cudaStream_t)stream;
  if (algo == B200_ALGO_TC || (algo == B200_ALGO_AUTO && M >= 128 && N >= 64 && K >= 32)) {
    note_kernel("tc_gemm");
    const int rc = tc_gemm(M, N, K, A, sa0, sa1, B, sb0, sb1, bias, alpha, beta, C, st);
    if (rc != B200_EUNSUPPORTED || algo == B200_ALGO_TC) return rc;
  }
  note_kernel("simt_gemm");
  return simt_gemm(M, N, K, A, sa0, sa1, B, sb0, sb1, bias, alpha, beta, C, st);
}

int b200_bmm(int64_t batch, int64_t M, int64_t N, int64_t K, const float* A, int64_t sa_b, int64_t sa0, int64_t sa1,
             const float* B, int64_t sb_b, int64_t sb0, int64_t sb1, float* C, int algo, void* stream) {
  if (batch < 0) return fail(B200_EINVAL, "bmm: negative batch");
  if (batch == 0 || M == 0 || N == 0) return B200_OK;
  if (batch * M > UINT32_MAX / N) return fail(B200_ERANGE, "bmm: result too large");
  if (K == 0) {  // empty contraction: zeros (bmm.cpp:50-54)
    if (!C) return fail(B200_EINVAL, "bmm: null matrix");
    B200_CUDA(cudaMemsetAsync(C, 0, (size_t)(batch * M * N) * sizeof(float), (cudaStream_t)stream));
    return B200_OK;
  }
  // one right-hand matrix for every batch and left-hand rows at one constant stride: a single
  // product with batch * M rows
  if ((sb_b == 0 || batch == 1) && (batch == 1 || sa_b == M * sa0))
    return b200_gemm(batch * M, N, K, A, sa0, sa1, B, sb0, sb1, nullptr, 1.f, 0.f, C, algo, stream);
  // every batch in one launch pair on the tcgen05 kernel (the batch rides on its group dimension)
  // (a loop of small products is the alternative, so the batched kernel is taken from smaller shapes than b200_gemm's)
  if ((algo == B200_ALGO_TC || (algo == B200_ALGO_AUTO && M >= 64 && N >= 16 && K >= 16)) && A && B && C) {
    note_kernel("tc_bmm");
    const int rc = tc_bmm(batch, M, N, K, A, sa_b, sa0, sa1, B, sb_b, sb0, sb1, C, (cudaStream_t)stream);
    if (rc != B200_EUNSUPPORTED) return rc;
  }
  for (int64_t b = 0; b < batch; ++b)
    if (int rc = b200_gemm(M, N, K, A ? A + b * sa_b : nullptr, sa0, sa1, B ? B + b * sb_b : nullptr, sb0, sb1, nullptr, 1.f, 0.f,
                           C + b * M * N, algo, stream))
      return rc;
  return B200_OK;
}

}  // extern "C"
