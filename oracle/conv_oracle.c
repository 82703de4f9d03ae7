/*
 * CPU oracle for the FP32 Conv2D hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference backend's
 * convolution shaders so that the CUDA kernels can be checked against the
 * reference's own reduction orders on a machine that has no graphics stack.
 * It is never linked into, imported by, or called from the shipped library:
 * only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may use it.
 *
 * Parity status: PINNED.  The functions here are checked (tests/test_oracle.py)
 * against (a) the closed-form known-answer cases the reference's tests hold
 * (tests/test_conv_dispatch.py:315-333, tests/test_mm.py:29-36) and (b) golden
 * vectors produced by PyTorch's CPU convolution in FP64, which is the ground
 * truth the reference's own tests compare against
 * (tests/test_conv_dispatch.py:50-70, tests/test_convolution.py:21-40),
 * generated with the reference's seeds and shapes by tests/golden/make_golden.py.
 *
 * Every function cites the reference file:line whose arithmetic it follows.
 * All tensors are contiguous NCHW FP32 unless stated.  The `_f64` variants keep
 * the loop structure but accumulate in double; they are the "CPU float64
 * accumulation -> float32" oracle the reference's probes use
 * (benchmarks/probe_conv_dispatch.py:82-87).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

typedef struct {
  uint32_t n, cin, cout, h, w, kh, kw, oh, ow;
  uint32_t sh, sw, ph, pw, dh, dw, groups;
} oracle_conv_params; /* csrc/ops/convolution.cpp:45-52 (ConvParams, push-constant order) */

/* Geometry validation and output extent, csrc/ops/convolution.cpp:101-156.
 * Returns 0 and fills oh/ow, or a negative code naming the failed check:
 * -1 invalid shapes or parameters, -2 int32 coordinates, -3 effective kernel
 * exceeds padded input, -4 empty output. */
int oracle_conv_geometry(oracle_conv_params* p, int64_t n, int64_t cin, int64_t cout,
                         int64_t h, int64_t w, int64_t wcin, int64_t kh, int64_t kw,
                         int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                         int64_t dh, int64_t dw, int64_t groups) {
  if (!(n > 0 && cin > 0 && cout > 0 && h > 0 && w > 0 && kh > 0 && kw > 0 &&
        sh > 0 && sw > 0 && dh > 0 && dw > 0 && ph >= 0 && pw >= 0 && groups > 0 &&
        cin % groups == 0 && cout % groups == 0 && wcin == cin / groups))
    return -1;
  const int64_t vals[10] = {h, w, kh, kw, sh, sw, ph, pw, dh, dw};
  for (int i = 0; i < 10; ++i)
    if (vals[i] > INT32_MAX) return -2;
  if (dh * (kh - 1) > INT32_MAX || dw * (kw - 1) > INT32_MAX) return -2;
  if (!(h + 2 * ph >= dh * (kh - 1) + 1 && w + 2 * pw >= dw * (kw - 1) + 1)) return -3;
  const int64_t oh = (h + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
  const int64_t ow = (w + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
  if (!(oh > 0 && ow > 0)) return -4;
  if ((oh - 1) * sh + dh * (kh - 1) > INT32_MAX || (ow - 1) * sw + dw * (kw - 1) > INT32_MAX ||
      h - 1 + ph > INT32_MAX || w - 1 + pw > INT32_MAX)
    return -2;
  p->n = (uint32_t)n; p->cin = (uint32_t)cin; p->cout = (uint32_t)cout;
  p->h = (uint32_t)h; p->w = (uint32_t)w; p->kh = (uint32_t)kh; p->kw = (uint32_t)kw;
  p->oh = (uint32_t)oh; p->ow = (uint32_t)ow; p->sh = (uint32_t)sh; p->sw = (uint32_t)sw;
  p->ph = (uint32_t)ph; p->pw = (uint32_t)pw; p->dh = (uint32_t)dh; p->dw = (uint32_t)dw;
  p->groups = (uint32_t)groups;
  return 0;
}

/* View normaliser: gather a <=4-D strided/offset/broadcast view into a
 * contiguous buffer, address = offset + sum idx_d*stride_d.
 * csrc/shaders/conv2d_pack.comp:1-22, host side csrc/ops/convolution.cpp:62-99. */
void oracle_pack(const float* base, int64_t offset, const int64_t size[4],
                 const int64_t stride[4], float* dst) {
  const int64_t total = size[0] * size[1] * size[2] * size[3];
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < total; ++i) {
    int64_t r = i, addr = offset;
    for (int d = 3; d >= 0; --d) {
      addr += (r % size[d]) * stride[d];
      r /= size[d];
    }
    dst[i] = base[addr];
  }
}

/* ------------------------------------------------------------------------- */
/* Direct semantics: one output element per "thread", loop order of the      */
/* shader.  ACC is the accumulator type.                                     */
/* ------------------------------------------------------------------------- */
#define DEFINE_DIRECT(SUFFIX, ACC)                                                              \
  /* csrc/shaders/conv2d_forward.comp:11-43: sum starts at bias, loops c -> kh -> kw */         \
  void oracle_forward_direct##SUFFIX(const oracle_conv_params* p, const float* x,               \
                                     const float* wt, const float* bias, float* y) {            \
    const int64_t hw = (int64_t)p->oh * p->ow, total = (int64_t)p->n * p->cout * hw;            \
    const uint32_t cig = p->cin / p->groups, cog = p->cout / p->groups;                         \
    _Pragma("omp parallel for schedule(static)")                                                \
    for (int64_t idx = 0; idx < total; ++idx) {                                                 \
      const uint32_t ow = (uint32_t)(idx % p->ow), oh = (uint32_t)((idx / p->ow) % p->oh);      \
      const uint32_t oc = (uint32_t)((idx / hw) % p->cout);                                     \
      const uint32_t b = (uint32_t)(idx / ((int64_t)p->cout * hw));                             \
      const uint32_t first_in = (oc / cog) * cig;                                               \
      ACC sum = bias ? (ACC)bias[oc] : (ACC)0;                                                  \
      for (uint32_t c = 0; c < cig; ++c) {                                                      \
        const uint32_t ic = first_in + c;                                                       \
        for (uint32_t kh = 0; kh < p->kh; ++kh) {                                               \
          const int ih = (int)(oh * p->sh) - (int)p->ph + (int)(kh * p->dh);                    \
          if (ih < 0 || ih >= (int)p->h) continue;                                              \
          for (uint32_t kw = 0; kw < p->kw; ++kw) {                                             \
            const int iw = (int)(ow * p->sw) - (int)p->pw + (int)(kw * p->dw);                  \
            if (iw < 0 || iw >= (int)p->w) continue;                                            \
            const int64_t ox = (((int64_t)b * p->cin + ic) * p->h + ih) * p->w + iw;            \
            const int64_t owt = (((int64_t)oc * cig + c) * p->kh + kh) * p->kw + kw;            \
            sum += (ACC)x[ox] * (ACC)wt[owt];                                                   \
          }                                                                                     \
        }                                                                                       \
      }                                                                                         \
      y[idx] = (float)sum;                                                                      \
    }                                                                                           \
  }                                                                                             \
  /* csrc/shaders/conv2d_backward_input.comp:10-47: loops co -> kh -> kw, stride divisibility */\
  void oracle_dinput_direct##SUFFIX(const oracle_conv_params* p, const float* go,               \
                                    const float* wt, float* dx) {                               \
    const int64_t hw = (int64_t)p->h * p->w, total = (int64_t)p->n * p->cin * hw;               \
    const uint32_t cig = p->cin / p->groups, cog = p->cout / p->groups;                         \
    _Pragma("omp parallel for schedule(static)")                                                \
    for (int64_t idx = 0; idx < total; ++idx) {                                                 \
      const uint32_t iw = (uint32_t)(idx % p->w), ih = (uint32_t)((idx / p->w) % p->h);         \
      const uint32_t ic = (uint32_t)((idx / hw) % p->cin);                                      \
      const uint32_t b = (uint32_t)(idx / ((int64_t)p->cin * hw));                              \
      const uint32_t g = ic / cig, cg = ic % cig;                                               \
      ACC sum = (ACC)0;                                                                         \
      for (uint32_t co = 0; co < cog; ++co) {                                                   \
        const uint32_t oc = g * cog + co;                                                       \
        for (uint32_t kh = 0; kh < p->kh; ++kh) {                                               \
          const int ih0 = (int)ih + (int)p->ph - (int)(kh * p->dh);                             \
          if (ih0 < 0 || ih0 % (int)p->sh != 0) continue;                                       \
          const int out_h = ih0 / (int)p->sh;                                                   \
          if (out_h >= (int)p->oh) continue;                                                    \
          for (uint32_t kw = 0; kw < p->kw; ++kw) {                                             \
            const int iw0 = (int)iw + (int)p->pw - (int)(kw * p->dw);                           \
            if (iw0 < 0 || iw0 % (int)p->sw != 0) continue;                                     \
            const int out_w = iw0 / (int)p->sw;                                                 \
            if (out_w >= (int)p->ow) continue;                                                  \
            const int64_t og = (((int64_t)b * p->cout + oc) * p->oh + out_h) * p->ow + out_w;   \
            const int64_t owt = (((int64_t)oc * cig + cg) * p->kh + kh) * p->kw + kw;           \
            sum += (ACC)go[og] * (ACC)wt[owt];                                                  \
          }                                                                                     \
        }                                                                                       \
      }                                                                                         \
      dx[idx] = (float)sum;                                                                     \
    }                                                                                           \
  }                                                                                             \
  /* csrc/shaders/conv2d_backward_weight.comp:10-41: loops batch -> oh -> ow */                 \
  void oracle_dweight_direct##SUFFIX(const oracle_conv_params* p, const float* x,               \
                                     const float* go, float* dwt) {                             \
    const uint32_t cig = p->cin / p->groups, cog = p->cout / p->groups;                         \
    const int64_t total = (int64_t)p->cout * cig * p->kh * p->kw;                               \
    _Pragma("omp parallel for schedule(dynamic, 16)")                                           \
    for (int64_t idx = 0; idx < total; ++idx) {                                                 \
      const uint32_t kw = (uint32_t)(idx % p->kw), kh = (uint32_t)((idx / p->kw) % p->kh);      \
      const uint32_t c = (uint32_t)((idx / ((int64_t)p->kw * p->kh)) % cig);                    \
      const uint32_t oc = (uint32_t)(idx / ((int64_t)p->kw * p->kh * cig));                     \
      const uint32_t ic = (oc / cog) * cig + c;                                                 \
      ACC sum = (ACC)0;                                                                         \
      for (uint32_t b = 0; b < p->n; ++b)                                                       \
        for (uint32_t oh = 0; oh < p->oh; ++oh) {                                               \
          const int ih = (int)(oh * p->sh) - (int)p->ph + (int)(kh * p->dh);                    \
          if (ih < 0 || ih >= (int)p->h) continue;                                              \
          for (uint32_t ow = 0; ow < p->ow; ++ow) {                                             \
            const int iw = (int)(ow * p->sw) - (int)p->pw + (int)(kw * p->dw);                  \
            if (iw < 0 || iw >= (int)p->w) continue;                                            \
            const int64_t ox = (((int64_t)b * p->cin + ic) * p->h + ih) * p->w + iw;            \
            const int64_t og = (((int64_t)b * p->cout + oc) * p->oh + oh) * p->ow + ow;         \
            sum += (ACC)x[ox] * (ACC)go[og];                                                    \
          }                                                                                     \
        }                                                                                       \
      dwt[idx] = (float)sum;                                                                    \
    }                                                                                           \
  }                                                                                             \
  /* csrc/shaders/conv2d_backward_bias.comp:9-27: serial batch -> oh -> ow sum per channel */   \
  void oracle_dbias_direct##SUFFIX(const oracle_conv_params* p, const float* go, float* db) {   \
    const int64_t sp = (int64_t)p->oh * p->ow;                                                  \
    _Pragma("omp parallel for schedule(static)")                                                \
    for (int64_t oc = 0; oc < (int64_t)p->cout; ++oc) {                                         \
      ACC sum = (ACC)0;                                                                         \
      for (uint32_t b = 0; b < p->n; ++b)                                                       \
        for (int64_t i = 0; i < sp; ++i) sum += (ACC)go[((int64_t)b * p->cout + oc) * sp + i];  \
      db[oc] = (float)sum;                                                                      \
    }                                                                                           \
  }

DEFINE_DIRECT(, float)
DEFINE_DIRECT(_f64, double)

/* ------------------------------------------------------------------------- */
/* Tiled (implicit GEMM) orders                                              */
/* ------------------------------------------------------------------------- */

/* Forward implicit GEMM: k = (ci,ky,kx) ascending, padding taps contribute an
 * explicit 0.0f product, bias is added once at the end (value + bias[oc]).
 * csrc/shaders/conv2d_tiled_body.glsl:53-86 and :19-25. */
void oracle_forward_tiled(const oracle_conv_params* p, const float* x, const float* wt,
                          const float* bias, float* y) {
  const int64_t hw = (int64_t)p->oh * p->ow, total = (int64_t)p->n * p->cout * hw;
  const uint32_t cig = p->cin / p->groups, cog = p->cout / p->groups;
  const uint32_t taps = p->kh * p->kw, K = cig * taps;
#pragma omp parallel for schedule(static)
  for (int64_t idx = 0; idx < total; ++idx) {
    const uint32_t pos = (uint32_t)(idx % hw), oc = (uint32_t)((idx / hw) % p->cout);
    const uint32_t b = (uint32_t)(idx / ((int64_t)p->cout * hw));
    const uint32_t g = oc / cog;
    float acc = 0.0f;
    for (uint32_t k = 0; k < K; ++k) {
      const uint32_t inch = g * cig + k / taps, rem = k % taps;
      const int iy = (int)((pos / p->ow) * p->sh) - (int)p->ph + (int)((rem / p->kw) * p->dh);
      const int ix = (int)((pos % p->ow) * p->sw) - (int)p->pw + (int)((rem % p->kw) * p->dw);
      float v = 0.0f;
      if (iy >= 0 && iy < (int)p->h && ix >= 0 && ix < (int)p->w)
        v = x[(((int64_t)b * p->cin + inch) * p->h + iy) * p->w + ix];
      acc += wt[(int64_t)oc * K + k] * v;
    }
    y[idx] = acc + (bias ? bias[oc] : 0.0f);
  }
}

/* dInput implicit GEMM: k = (co,ky,kx) ascending,
 * csrc/shaders/conv2d_backward_input_tiled_body.glsl:49-93. */
void oracle_dinput_tiled(const oracle_conv_params* p, const float* go, const float* wt,
                         float* dx) {
  const int64_t hw = (int64_t)p->h * p->w, total = (int64_t)p->n * p->cin * hw;
  const uint32_t cig = p->cin / p->groups, cog = p->cout / p->groups;
  const uint32_t taps = p->kh * p->kw, K = cog * taps;
#pragma omp parallel for schedule(static)
  for (int64_t idx = 0; idx < total; ++idx) {
    const uint32_t pos = (uint32_t)(idx % hw), ic = (uint32_t)((idx / hw) % p->cin);
    const uint32_t b = (uint32_t)(idx / ((int64_t)p->cin * hw));
    const uint32_t g = ic / cig, c = ic % cig;
    float acc = 0.0f;
    for (uint32_t k = 0; k < K; ++k) {
      const uint32_t oc = g * cog + k / taps, rem = k % taps;
      const int yh = (int)(pos / p->w) + (int)p->ph - (int)((rem / p->kw) * p->dh);
      const int xw = (int)(pos % p->w) + (int)p->pw - (int)((rem % p->kw) * p->dw);
      float v = 0.0f;
      if (yh >= 0 && xw >= 0) {
        uint32_t oy = (uint32_t)yh, ox = (uint32_t)xw;
        int aligned = 1;
        if (p->sh != 1u || p->sw != 1u) {
          aligned = (oy % p->sh == 0u && ox % p->sw == 0u);
          oy /= p->sh; ox /= p->sw;
        }
        if (aligned && oy < p->oh && ox < p->ow)
          v = go[(((int64_t)b * p->cout + oc) * p->oh + oy) * p->ow + ox];
      }
      acc += wt[((int64_t)oc * cig + c) * taps + rem] * v;
    }
    dx[idx] = acc;
  }
}

/* Split-K plan for dWeight, csrc/ops/convolution.cpp:204-238.  `max_grid_z`
 * and `max_range` stand for the Vulkan device limits the reference clamps by
 * (maxComputeWorkGroupCount[2], maxStorageBufferRange).  Returns count (0 =
 * tiled split ineligible) and writes span/bytes. */
uint32_t oracle_weight_split_plan(const oracle_conv_params* p, uint64_t budget, uint32_t tile_k,
                                  uint64_t max_grid_z, uint64_t max_range, uint32_t* span_out,
                                  uint64_t* bytes_out) {
  const uint64_t positions = (uint64_t)p->n * p->oh * p->ow;
  const uint64_t default_span = ((256 + tile_k - 1) / tile_k) * (uint64_t)tile_k;
  if (positions <= default_span) { *span_out = (uint32_t)default_span; *bytes_out = 0; return 1; }
  const uint64_t weight_bytes =
      (uint64_t)p->cout * (p->cin / p->groups) * p->kh * p->kw * sizeof(float);
  uint64_t allowed = budget;
  if (max_range < allowed) allowed = max_range;
  if ((uint64_t)UINT32_MAX * sizeof(float) < allowed) allowed = (uint64_t)UINT32_MAX * sizeof(float);
  const uint64_t natural = (positions + default_span - 1) / default_span;
  uint64_t max_parts = 0;
  if (weight_bytes) {
    max_parts = natural;
    if (allowed / weight_bytes < max_parts) max_parts = allowed / weight_bytes;
    if (max_grid_z < max_parts) max_parts = max_grid_z;
  }
  if (max_parts < 2) { *span_out = 0; *bytes_out = 0; return 0; }
  uint64_t span = default_span;
  if (max_parts != natural) {
    const uint64_t per = (positions + max_parts - 1) / max_parts;
    span = ((per + tile_k - 1) / tile_k) * tile_k;
  }
  const uint64_t parts = (positions + span - 1) / span;
  *span_out = (uint32_t)span;
  *bytes_out = parts * weight_bytes;
  return (uint32_t)parts;
}

/* dWeight implicit GEMM with a spatial split: partial[s][oc][col] accumulates
 * positions [s*span, min((s+1)*span,total)) ascending (padding taps add 0.0f),
 * then dW = sum_s partial[s] with s ascending.
 * csrc/shaders/conv2d_backward_weight_tiled_body.glsl:42-70,
 * csrc/shaders/conv2d_backward_weight_finalize.comp:9-18.
 * `partial` must hold splits*numel(dW) floats, splits = ceil(total/span);
 * when splits == 1 the reference writes dW directly (same arithmetic). */
void oracle_dweight_split(const oracle_conv_params* p, const float* x, const float* go,
                          uint32_t span, float* partial, float* dwt) {
  const uint32_t cig = p->cin / p->groups, cog = p->cout / p->groups;
  const uint32_t taps = p->kh * p->kw, cols = cig * taps;
  const int64_t count = (int64_t)p->cout * cols;
  const uint32_t spatial = p->oh * p->ow, total = p->n * spatial;
  const uint32_t splits = 1 + (total - 1) / span;
#pragma omp parallel for schedule(dynamic, 16) collapse(2)
  for (uint32_t s = 0; s < splits; ++s)
    for (int64_t idx = 0; idx < count; ++idx) {
      const uint32_t oc = (uint32_t)(idx / cols), col = (uint32_t)(idx % cols);
      const uint32_t ic = (oc / cog) * cig + col / taps;
      const uint32_t ky = (col / p->kw) % p->kh, kx = col % p->kw;
      const uint32_t first = s * span;
      const uint32_t end = first + (span < total - first ? span : total - first);
      float acc = 0.0f;
      for (uint32_t k = first; k < end; ++k) {
        const uint32_t b = k / spatial, pos = k % spatial;
        const int iy = (int)((pos / p->ow) * p->sh) - (int)p->ph + (int)(ky * p->dh);
        const int ix = (int)((pos % p->ow) * p->sw) - (int)p->pw + (int)(kx * p->dw);
        float v = 0.0f;
        if (iy >= 0 && iy < (int)p->h && ix >= 0 && ix < (int)p->w)
          v = x[(((int64_t)b * p->cin + ic) * p->h + iy) * p->w + ix];
        acc += go[((int64_t)b * p->cout + oc) * spatial + pos] * v;
      }
      partial[(int64_t)s * count + idx] = acc;
    }
#pragma omp parallel for schedule(static)
  for (int64_t idx = 0; idx < count; ++idx) {
    float sum = 0.0f;
    for (uint32_t s = 0; s < splits; ++s) sum += partial[(int64_t)s * count + idx];
    dwt[idx] = sum;
  }
}

/* 128-lane strided partial sums followed by a 7-step halving tree.
 * csrc/shaders/conv2d_backward_weight_reduce.comp:23-37 */
static float tree128(float* lanes) {
  for (uint32_t stride = 64; stride > 0; stride /= 2)
    for (uint32_t lane = 0; lane < stride; ++lane) lanes[lane] += lanes[lane + stride];
  return lanes[0];
}

/* csrc/shaders/conv2d_backward_weight_reduce.comp:12-38 */
void oracle_dweight_reduce(const oracle_conv_params* p, const float* x, const float* go,
                           float* dwt) {
  const uint32_t cig = p->cin / p->groups, cog = p->cout / p->groups;
  const int64_t total = (int64_t)p->cout * cig * p->kh * p->kw;
  const uint32_t spatial = p->oh * p->ow;
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t idx = 0; idx < total; ++idx) {
    const uint32_t kx = (uint32_t)(idx % p->kw), ky = (uint32_t)((idx / p->kw) % p->kh);
    const uint32_t c = (uint32_t)((idx / ((int64_t)p->kw * p->kh)) % cig);
    const uint32_t oc = (uint32_t)(idx / ((int64_t)p->kw * p->kh * cig));
    const uint32_t ic = (oc / cog) * cig + c;
    float lanes[128];
    for (uint32_t lane = 0; lane < 128; ++lane) {
      float sum = 0.0f;
      for (uint32_t r = lane; r < p->n * spatial; r += 128) {
        const uint32_t b = r / spatial, pos = r % spatial;
        const int iy = (int)((pos / p->ow) * p->sh) - (int)p->ph + (int)(ky * p->dh);
        const int ix = (int)((pos % p->ow) * p->sw) - (int)p->pw + (int)(kx * p->dw);
        if (iy >= 0 && iy < (int)p->h && ix >= 0 && ix < (int)p->w)
          sum += x[(((int64_t)b * p->cin + ic) * p->h + iy) * p->w + ix] *
                 go[((int64_t)b * p->cout + oc) * spatial + pos];
      }
      lanes[lane] = sum;
    }
    dwt[idx] = tree128(lanes);
  }
}

/* csrc/shaders/conv2d_backward_bias_reduce.comp:9-24 */
void oracle_dbias_reduce(const oracle_conv_params* p, const float* go, float* db) {
  const uint32_t spatial = p->oh * p->ow;
#pragma omp parallel for schedule(static)
  for (int64_t oc = 0; oc < (int64_t)p->cout; ++oc) {
    float lanes[128];
    for (uint32_t lane = 0; lane < 128; ++lane) {
      float sum = 0.0f;
      for (uint32_t r = lane; r < p->n * spatial; r += 128)
        sum += go[((int64_t)(r / spatial) * p->cout + oc) * spatial + r % spatial];
      lanes[lane] = sum;
    }
    db[oc] = tree128(lanes);
  }
}

/* Depthwise with channel multiplier (groups == cin): ic = oc/(cout/cin), loops
 * ky -> kx from bias.  csrc/shaders/conv2d_depthwise.comp:14-41 */
void oracle_forward_depthwise(const oracle_conv_params* p, const float* x, const float* wt,
                              const float* bias, float* y) {
  const int64_t sp = (int64_t)p->oh * p->ow, total = (int64_t)p->n * p->cout * sp;
#pragma omp parallel for schedule(static)
  for (int64_t id = 0; id < total; ++id) {
    const uint32_t pos = (uint32_t)(id % sp), oc = (uint32_t)((id / sp) % p->cout);
    const uint32_t b = (uint32_t)(id / (sp * p->cout)), ic = oc / (p->cout / p->cin);
    const uint32_t oy = pos / p->ow, ox = pos % p->ow;
    float v = bias ? bias[oc] : 0.0f;
    for (uint32_t ky = 0; ky < p->kh; ++ky) {
      const int iy = (int)(oy * p->sh) - (int)p->ph + (int)(ky * p->dh);
      if (iy < 0 || iy >= (int)p->h) continue;
      for (uint32_t kx = 0; kx < p->kw; ++kx) {
        const int ix = (int)(ox * p->sw) - (int)p->pw + (int)(kx * p->dw);
        if (ix < 0 || ix >= (int)p->w) continue;
        v += x[(((int64_t)b * p->cin + ic) * p->h + iy) * p->w + ix] *
             wt[((int64_t)oc * p->kh + ky) * p->kw + kx];
      }
    }
    y[id] = v;
  }
}

/* ------------------------------------------------------------------------- */
/* Winograd F(2x2,3x3) forward, three stages                                 */
/* ------------------------------------------------------------------------- */

/* U = G g G^T packed [16][cout][cin/g]. csrc/shaders/conv2d_winograd_weights.comp:11-29 */
static void winograd_f2_weights(const oracle_conv_params* p, const float* wt, float* tw) {
  const uint32_t ci = p->cin / p->groups;
  const int64_t count = (int64_t)p->cout * ci;
  for (int64_t idx = 0; idx < count; ++idx) {
    float g[3][3], z[4][3];
    for (int r = 0; r < 3; ++r) for (int c = 0; c < 3; ++c) g[r][c] = wt[idx * 9 + r * 3 + c];
    for (int c = 0; c < 3; ++c) {
      z[0][c] = g[0][c];
      z[1][c] = 0.5f * (g[0][c] + g[1][c] + g[2][c]);
      z[2][c] = 0.5f * (g[0][c] - g[1][c] + g[2][c]);
      z[3][c] = g[2][c];
    }
    for (int r = 0; r < 4; ++r) {
      tw[(r * 4 + 0) * count + idx] = z[r][0];
      tw[(r * 4 + 1) * count + idx] = 0.5f * (z[r][0] + z[r][1] + z[r][2]);
      tw[(r * 4 + 2) * count + idx] = 0.5f * (z[r][0] - z[r][1] + z[r][2]);
      tw[(r * 4 + 3) * count + idx] = z[r][2];
    }
  }
}

/* V = B^T d B packed [16][cin][tiles], zero padded. conv2d_winograd_input.comp:11-38 */
static void winograd_f2_input(const oracle_conv_params* p, const float* x, float* ti) {
  const uint32_t tile_w = (p->ow + 1) / 2, tile_h = (p->oh + 1) / 2;
  const uint32_t per_image = tile_w * tile_h;
  const int64_t tiles = (int64_t)p->n * per_image, stride = (int64_t)p->cin * tiles;
#pragma omp parallel for schedule(static)
  for (int64_t idx = 0; idx < stride; ++idx) {
    const uint32_t channel = (uint32_t)(idx / tiles), tile = (uint32_t)(idx % tiles);
    const uint32_t b = tile / per_image, pos = tile % per_image;
    const int y0 = (int)((pos / tile_w) * 2) - (int)p->ph, x0 = (int)((pos % tile_w) * 2) - (int)p->pw;
    float d[4][4], z[4][4];
    for (int r = 0; r < 4; ++r) for (int c = 0; c < 4; ++c) {
      const int iy = y0 + r, ix = x0 + c;
      d[r][c] = (iy >= 0 && iy < (int)p->h && ix >= 0 && ix < (int)p->w)
                    ? x[(((int64_t)b * p->cin + channel) * p->h + iy) * p->w + ix] : 0.0f;
    }
    for (int c = 0; c < 4; ++c) {
      z[0][c] = d[0][c] - d[2][c];
      z[1][c] = d[1][c] + d[2][c];
      z[2][c] = d[2][c] - d[1][c];
      z[3][c] = d[1][c] - d[3][c];
    }
    for (int r = 0; r < 4; ++r) {
      ti[(r * 4 + 0) * stride + channel * tiles + tile] = z[r][0] - z[r][2];
      ti[(r * 4 + 1) * stride + channel * tiles + tile] = z[r][1] + z[r][2];
      ti[(r * 4 + 2) * stride + channel * tiles + tile] = z[r][2] - z[r][1];
      ti[(r * 4 + 3) * stride + channel * tiles + tile] = z[r][1] - z[r][3];
    }
  }
}

/* 16 plane GEMMs over ci ascending + fused A^T m A + bias, edge-guarded stores.
 * csrc/shaders/conv2d_winograd_gemm_output.comp:17-64; three-stage launcher
 * csrc/ops/convolution.cpp:285-335.  Requires 3x3, stride 1, dilation 1. */
int oracle_forward_winograd_f2(const oracle_conv_params* p, const float* x, const float* wt,
                               const float* bias, float* y) {
  if (p->kh != 3 || p->kw != 3 || p->sh != 1 || p->sw != 1 || p->dh != 1 || p->dw != 1) return -1;
  const uint32_t ci = p->cin / p->groups, co = p->cout / p->groups;
  const uint32_t tile_w = (p->ow + 1) / 2, tile_h = (p->oh + 1) / 2;
  const uint32_t per_image = tile_w * tile_h;
  const int64_t tiles = (int64_t)p->n * per_image;
  const int64_t wcount = (int64_t)p->cout * ci, xcount = (int64_t)p->cin * tiles;
  float* tw = (float*)malloc(sizeof(float) * 16 * wcount);
  float* ti = (float*)malloc(sizeof(float) * 16 * xcount);
  if (!tw || !ti) { free(tw); free(ti); return -2; }
  winograd_f2_weights(p, wt, tw);
  winograd_f2_input(p, x, ti);
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t oc = 0; oc < (int64_t)p->cout; ++oc)
    for (int64_t tile = 0; tile < tiles; ++tile) {
      const uint32_t g = (uint32_t)oc / co;
      float accum[16];
      for (int t = 0; t < 16; ++t) accum[t] = 0.0f;
      for (uint32_t k = 0; k < ci; ++k)
        for (int t = 0; t < 16; ++t)
          accum[t] += tw[t * wcount + oc * ci + k] * ti[t * xcount + ((int64_t)g * ci + k) * tiles + tile];
      float r0[4], r1[4];
      for (int c = 0; c < 4; ++c) {
        r0[c] = accum[c] + accum[4 + c] + accum[8 + c];
        r1[c] = accum[4 + c] - accum[8 + c] - accum[12 + c];
      }
      const float b = bias ? bias[oc] : 0.0f;
      const float v00 = r0[0] + r0[1] + r0[2] + b, v01 = r0[1] - r0[2] - r0[3] + b;
      const float v10 = r1[0] + r1[1] + r1[2] + b, v11 = r1[1] - r1[2] - r1[3] + b;
      const uint32_t bt = (uint32_t)(tile / per_image), pos = (uint32_t)(tile % per_image);
      const uint32_t oy = (pos / tile_w) * 2, ox = (pos % tile_w) * 2;
      float* out = y + ((int64_t)bt * p->cout + oc) * p->oh * p->ow;
      if (oy < p->oh && ox < p->ow) out[oy * p->ow + ox] = v00;
      if (oy < p->oh && ox + 1 < p->ow) out[oy * p->ow + ox + 1] = v01;
      if (oy + 1 < p->oh && ox < p->ow) out[(oy + 1) * p->ow + ox] = v10;
      if (oy + 1 < p->oh && ox + 1 < p->ow) out[(oy + 1) * p->ow + ox + 1] = v11;
    }
  free(tw); free(ti);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Strided GEMM with the fused addmm epilogue                                */
/* ------------------------------------------------------------------------- */

/* C[M,N] = alpha * sum_k A[m*sa0+k*sa1]*B[k*sb0+n*sb1] + (beta==0 ? 0 : beta*bias[n]),
 * k ascending, C contiguous.  csrc/shaders/matmul_strided.comp:1-65 and
 * matmul_strided_bias.comp:33-68 (epilogue :66); host csrc/ops/mm.cpp:244-343,835-879.
 * bias may be NULL (plain mm: alpha=1, beta=0). */
void oracle_gemm(int64_t M, int64_t N, int64_t K, const float* A, int64_t sa0, int64_t sa1,
                 const float* B, int64_t sb0, int64_t sb1, const float* bias, float alpha,
                 float beta, float* C) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      float sum = 0.0f;
      for (int64_t k = 0; k < K; ++k) sum += A[m * sa0 + k * sa1] * B[k * sb0 + n * sb1];
      C[m * N + n] = bias ? alpha * sum + (beta == 0.0f ? 0.0f : beta * bias[n]) : sum;
    }
}

void oracle_gemm_f64(int64_t M, int64_t N, int64_t K, const float* A, int64_t sa0, int64_t sa1,
                     const float* B, int64_t sb0, int64_t sb1, const float* bias, float alpha,
                     float beta, float* C) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      double sum = 0.0;
      for (int64_t k = 0; k < K; ++k)
        sum += (double)A[m * sa0 + k * sa1] * (double)B[k * sb0 + n * sb1];
      C[m * N + n] = (float)(bias ? (double)alpha * sum + (beta == 0.0f ? 0.0 : (double)beta * bias[n]) : sum);
    }
}
