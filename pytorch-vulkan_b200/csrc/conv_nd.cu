// Generic N-d convolution (1 to 3 spatial dimensions, ordinary and transposed, FP32 and int64 forward): one thread
// per output element, contiguous operands.  This is the branch the reference's convolution entry point takes for
// everything that is not a plain FP32 Conv2D (csrc/ops/convolution_nd.cpp:51-74,
// shaders convolution_nd.comp / convolution_nd_int64.comp, also one invocation per output element).  The 2-D and
// 1-D FP32 cases never come here: they run the Conv2D kernels; what remains is 3-D convolution and integer tensors.
//
//   ordinary     y[n, co, o]  = b[co] + sum_{ci in group, k} x[n, ci, o*s - p + k*d] * w[co, ci_local, k]
//   transposed   y[n, co, o]  = b[co] + sum_{ci in group, k : (o + p - k*d) = i*s} x[n, ci, i] * w[ci, co_local, k]
// and the three gradients of either (mode 1: dx, 2: dw, 3: db), each again one thread per result element.
#include "common.cuh"

namespace b200 {
namespace cnd {

struct Nd {
  long long n, cin, cout, groups;
  int in[3], out[3], k[3], s[3], p[3], d[3];   // depth, height, width (missing leading dimensions are 1)
  int transposed;
};

__device__ __forceinline__ long long vol(const int (&v)[3]) { return (long long)v[0] * v[1] * v[2]; }

// position of the operand that pairs with result position `o` under tap `k`:
//   gather  (ordinary forward, transposed dx):  i = o*s - p + k*d, valid if inside
//   scatter (transposed forward, ordinary dx):  i = (o + p - k*d) / s, valid if divisible and inside
__device__ __forceinline__ bool pair_pos(const Nd& g, bool scatter, const int (&o)[3], const int (&k)[3], const int (&lim)[3], int (&i)[3]) {
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    int v;
    if (scatter) {
      v = o[a] + g.p[a] - k[a] * g.d[a];
      if (v < 0 || v % g.s[a] != 0) return false;
      v /= g.s[a];
    } else {
      v = o[a] * g.s[a] - g.p[a] + k[a] * g.d[a];
      if (v < 0) return false;
    }
    if (v >= lim[a]) return false;
    i[a] = v;
  }
  return true;
}

// mode 0: forward (y from x, w, bias).  mode 1: dx from grad, w.  T = float or long long (mode 0 only).
template <typename T>
__global__ void __launch_bounds__(256) convnd_map_kernel(Nd g, int mode, const T* __restrict__ src, const T* __restrict__ w,
                                                         const T* __restrict__ bias, T* __restrict__ dst, long long total) {
  const long long idx = blockIdx.x * 256ll + threadIdx.x;
  if (idx >= total) return;
  // the result lives on the output grid (mode 0) or on the input grid (mode 1)
  const bool on_out = mode == 0;
  const int (&rs)[3] = on_out ? g.out : g.in;     // extent of the result
  const int (&ss)[3] = on_out ? g.in : g.out;     // extent of the operand it reads
  const long long rc = on_out ? g.cout : g.cin, sc = on_out ? g.cin : g.cout;
  long long r = idx;
  int o[3];
  o[2] = (int)(r % rs[2]); r /= rs[2];
  o[1] = (int)(r % rs[1]); r /= rs[1];
  o[0] = (int)(r % rs[0]); r /= rs[0];
  const long long c = r % rc, n = r / rc;
  const long long rcg = rc / g.groups, scg = sc / g.groups, grp = c / rcg, cl = c % rcg;
  // ordinary forward and transposed dx gather; transposed forward and ordinary dx scatter
  const bool scatter = (mode == 0) == (g.transposed != 0);
  const long long kvol = vol(g.k);
  T acc = (mode == 0 && bias) ? bias[c] : T(0);
  for (long long c2l = 0; c2l < scg; ++c2l) {
    const long long c2 = grp * scg + c2l;
    const T* plane = src + (n * sc + c2) * vol(ss);
    // weight layout: ordinary [cout][cin/g][k], transposed [cin][cout/g][k]; (co, ci) in terms of (c, c2):
    // the result channel is cout in mode 0 and cin in mode 1
    const long long co = on_out ? c : c2, col = on_out ? cl : c2l, ci = on_out ? c2 : c, cil = on_out ? c2l : cl;
    const T* wk = g.transposed ? w + (ci * (g.cout / g.groups) + col) * kvol : w + (co * (g.cin / g.groups) + cil) * kvol;
    int k[3], i[3];
    for (k[0] = 0; k[0] < g.k[0]; ++k[0])
      for (k[1] = 0; k[1] < g.k[1]; ++k[1])
        for (k[2] = 0; k[2] < g.k[2]; ++k[2])
          if (pair_pos(g, scatter, o, k, ss, i))
            acc += plane[((long long)i[0] * ss[1] + i[1]) * ss[2] + i[2]] * wk[((long long)k[0] * g.k[1] + k[1]) * g.k[2] + k[2]];
  }
  dst[idx] = acc;
}

// mode 2: dw[., ., k] = sum over samples and positions of grad * x.  One thread per weight element.
__global__ void __launch_bounds__(256) convnd_dw_kernel(Nd g, const float* __restrict__ grad, const float* __restrict__ x,
                                                        float* __restrict__ dw, long long total) {
  const long long idx = blockIdx.x * 256ll + threadIdx.x;
  if (idx >= total) return;
  long long r = idx;
  int k[3];
  k[2] = (int)(r % g.k[2]); r /= g.k[2];
  k[1] = (int)(r % g.k[1]); r /= g.k[1];
  k[0] = (int)(r % g.k[0]); r /= g.k[0];
  const long long cig = g.cin / g.groups, cog = g.cout / g.groups;
  long long co, ci;
  if (g.transposed) { const long long col = r % cog; ci = r / cog; co = (ci / cig) * cog + col; }
  else { const long long cil = r % cig; co = r / cig; ci = (co / cog) * cig + cil; }
  float acc = 0.f;
  for (long long n = 0; n < g.n; ++n) {
    const float* gp = grad + (n * g.cout + co) * vol(g.out);
    const float* xp = x + (n * g.cin + ci) * vol(g.in);
    int o[3], i[3];
    // ordinary: grad lives on the output grid o, x at o*s - p + k*d.  transposed: x on the input grid i, grad at
    // i*s - p + k*d.  Either way: walk the grid that is indexed directly, gather from the other.
    const int (&walk)[3] = g.transposed ? g.in : g.out;
    const int (&other)[3] = g.transposed ? g.out : g.in;
    const float* pw = g.transposed ? xp : gp;
    const float* po = g.transposed ? gp : xp;
    for (o[0] = 0; o[0] < walk[0]; ++o[0])
      for (o[1] = 0; o[1] < walk[1]; ++o[1])
        for (o[2] = 0; o[2] < walk[2]; ++o[2])
          if (pair_pos(g, false, o, k, other, i))
            acc += pw[((long long)o[0] * walk[1] + o[1]) * walk[2] + o[2]] * po[((long long)i[0] * other[1] + i[1]) * other[2] + i[2]];
  }
  dw[idx] = acc;
}

// mode 3: db[co] = sum grad[:, co, ...].  One warp per channel, lanes stride over the elements, fixed-order tree.
__global__ void __launch_bounds__(256) convnd_db_kernel(Nd g, const float* __restrict__ grad, float* __restrict__ db) {
  const long long co = blockIdx.x * 8ll + (threadIdx.x >> 5);
  if (co >= g.cout) return;
  const int lane = threadIdx.x & 31;
  const long long v = vol(g.out);
  float acc = 0.f;
  for (long long n = 0; n < g.n; ++n) {
    const float* p = grad + (n * g.cout + co) * v;
    for (long long e = lane; e < v; e += 32) acc += p[e];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) db[co] = acc;
}

static Nd to_nd(const b200_convnd_params& p) {
  Nd g{};
  g.n = p.n; g.cin = p.cin; g.cout = p.cout; g.groups = p.groups; g.transposed = p.transposed;
  for (int a = 0; a < 3; ++a) {
    g.in[a] = (int)p.in[a]; g.out[a] = (int)p.out[a]; g.k[a] = (int)p.k[a];
    g.s[a] = (int)p.stride[a]; g.p[a] = (int)p.pad[a]; g.d[a] = (int)p.dilation[a];
  }
  return g;
}

}  // namespace cnd
}  // namespace b200

using namespace b200;

extern "C" {

int b200_convnd_geometry(b200_convnd_params* out, int rank, int64_t n, int64_t cin, const int64_t* in_sizes, int64_t w0,
                         int64_t w1, const int64_t* kernel, const int64_t* stride, const int64_t* pad, const int64_t* dilation,
                         const int64_t* output_pad, int transposed, int64_t groups) {
  if (!out || !in_sizes || !kernel || !stride || !pad || !dilation || !output_pad) return fail(B200_EINVAL, "convolution: null argument");
  if (rank < 1 || rank > 3) return fail(B200_EINVAL, "convolution: expected matching rank 3, 4 or 5 tensors");
  if (!(groups > 0 && cin > 0 && cin % groups == 0)) return fail(B200_EINVAL, "convolution: invalid groups/input channels");
  if (w0 <= 0 || w1 <= 0) return fail(B200_EINVAL, "convolution: empty weight dimension");
  const int64_t cout = transposed ? w1 * groups : w0;
  if (!(cout % groups == 0 && (transposed ? w0 == cin : w1 * groups == cin)))
    return fail(B200_EINVAL, "convolution: weight/channel/group mismatch");
  b200_convnd_params g{};
  g.rank = rank; g.n = n; g.cin = cin; g.cout = cout; g.groups = groups; g.transposed = transposed ? 1 : 0;
  for (int a = 0; a < 3; ++a) { g.in[a] = g.out[a] = g.k[a] = g.stride[a] = g.dilation[a] = 1; g.pad[a] = 0; }
  for (int a = 0; a < rank; ++a) {
    const int d = 3 - rank + a;
    const int64_t in = in_sizes[a], k = kernel[a], s = stride[a], p = pad[a], di = dilation[a], op = output_pad[a];
    if (k <= 0) return fail(B200_EINVAL, "convolution: empty weight dimension");
    if (!(in > 0 && s > 0 && di > 0 && p >= 0 && op >= 0)) return fail(B200_EINVAL, "convolution: invalid spatial parameters");
    if (!(transposed ? (op < s || op < di) : op == 0)) return fail(B200_EINVAL, "convolution: invalid output padding");
    if (!(in <= INT32_MAX && k <= INT32_MAX && s <= INT32_MAX && p <= INT32_MAX / 2 && di <= INT32_MAX && (k - 1) <= INT32_MAX / di &&
          (in - 1) <= INT32_MAX / s))
      return fail(B200_ERANGE, "convolution: spatial addressing exceeds int32");
    const int64_t effective = (k - 1) * di + 1;
    const int64_t o = transposed ? (in - 1) * s - 2 * p + effective + op : (in + 2 * p - effective) / s + 1;
    if (!((transposed || in + 2 * p >= effective) && o > 0 && o <= INT32_MAX && o * s + effective + p <= INT32_MAX))
      return fail(B200_EINVAL, "convolution: invalid or oversized output shape");
    g.in[d] = in; g.out[d] = o; g.k[d] = k; g.stride[d] = s; g.pad[d] = p; g.dilation[d] = di;
  }
  *out = g;
  return B200_OK;
}

int b200_convnd_forward(const b200_convnd_params* p, const void* x, const void* w, const void* bias, void* y, int is_int64,
                        void* stream) {
  if (!p) return fail(B200_EINVAL, "convolution: null parameters");
  if (int rc = ensure_init()) return rc;
  const cnd::Nd g = cnd::to_nd(*p);
  const long long total = p->n * p->cout * p->out[0] * p->out[1] * p->out[2];
  if (total == 0) return B200_OK;
  if (!x || !w || !y) return fail(B200_EINVAL, "convolution: null tensor");
  const unsigned blocks = (unsigned)div_up64(total, 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (is_int64)
    cnd::convnd_map_kernel<long long><<<blocks, 256, 0, st>>>(g, 0, (const long long*)x, (const long long*)w, (const long long*)bias,
                                                             (long long*)y, total);
  else
    cnd::convnd_map_kernel<float><<<blocks, 256, 0, st>>>(g, 0, (const float*)x, (const float*)w, (const float*)bias, (float*)y, total);
  count_launch();
  note_kernel(is_int64 ? "convnd_forward_int64" : "convnd_forward");
  return launch_check("convnd_map_kernel");
}

int b200_convnd_backward(const b200_convnd_params* p, const float* grad, const float* x, const float* w, float* dx, float* dw,
                         float* db, void* stream) {
  if (!p) return fail(B200_EINVAL, "convolution: null parameters");
  if (int rc = ensure_init()) return rc;
  const cnd::Nd g = cnd::to_nd(*p);
  cudaStream_t st = (cudaStream_t)stream;
  const long long in_total = p->n * p->cin * p->in[0] * p->in[1] * p->in[2];
  const long long w_total = (p->transposed ? p->cin * (p->cout / p->groups) : p->cout * (p->cin / p->groups)) * p->k[0] * p->k[1] * p->k[2];
  const long long out_total = p->n * p->cout * p->out[0] * p->out[1] * p->out[2];
  if ((dx || dw || db) && out_total && !grad) return fail(B200_EINVAL, "convolution backward: null gradient");
  if (dx && in_total) {
    if (!w) return fail(B200_EINVAL, "convolution backward: null weight");
    cnd::convnd_map_kernel<float><<<(unsigned)div_up64(in_total, 256), 256, 0, st>>>(g, 1, grad, w, nullptr, dx, in_total);
    count_launch();
    if (int rc = launch_check("convnd_map_kernel")) return rc;
  }
  if (dw && w_total) {
    if (!x && in_total) return fail(B200_EINVAL, "convolution backward: null input");
    cnd::convnd_dw_kernel<<<(unsigned)div_up64(w_total, 256), 256, 0, st>>>(g, grad, x, dw, w_total);
    count_launch();
    if (int rc = launch_check("convnd_dw_kernel")) return rc;
  }
  if (db && p->cout) {
    cnd::convnd_db_kernel<<<(unsigned)div_up64(p->cout, 8), 256, 0, st>>>(g, grad, db);
    count_launch();
    if (int rc = launch_check("convnd_db_kernel")) return rc;
  }
  note_kernel("convnd_backward");
  return B200_OK;
}

}  // extern "C"
