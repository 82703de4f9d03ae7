// Scaled dot-product attention, forward and backward, for contiguous FP32 [batch, tokens, dim]
// operands.  Replaces attention_forward / attention_backward of the reference
// (csrc/ops/attention.cpp:16-34) and its sdpa_training shader, dropout included (the same counter-based stream).
//
// The products run on the GEMM kernels of this library (b200_bmm: tcgen05 from 128x64x32, CUDA
// cores below); the score matrix is materialised in the caller's workspace, so this is the
// composed form of attention, not a single fused pass:
//   forward   S = Q K^T;  P = softmax(S * scale + mask) row by row, in place, with the
//             log-sum-exp kept per row;  O = P V
//   backward  P again from S and the saved log-sum-exp;  dP = dO V^T;
//             dS = P (dP w - rowsum(dO O)) * scale in place (w: dropout weights);  dV = (P w)^T dO;  dQ = dS K;  dK = dS^T Q
// The two elementwise kernels here are bound by HBM traffic over the [tokens, tokens] matrices.
// Masking as in the shader (sdpa_training.comp:16): causal hides keys j > i; a mask of the scores' shape, either
// additive FP32 or one byte per score where zero hides the key (a bool tensor); a row with every key hidden has
// log-sum-exp -inf and probability 0.  The backward pass can also return the gradient of the additive mask,
// dM = P (dP - rowsum(dO O)), the unscaled score gradient (sdpa_training.comp:38,40 `aux[index]=ds`).
#include <cmath>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Block-wide reduction of one value per thread; every thread gets the result.
template <bool MAX>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  v = MAX ? warp_max(v) : warp_add(v);
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  v = lane < kThreads / 32 ? scratch[lane] : (MAX ? -INFINITY : 0.f);
  return MAX ? warp_max(v) : warp_add(v);
}

// One row of the mask: additive floats, or bytes of which zero hides the key; both null = no mask.
struct MaskRow {
  const float* f;
  const unsigned char* b;
  __device__ __forceinline__ float at(int j) const {
    if (f) return __ldg(f + j);
    if (b) return __ldg(b + j) ? 0.f : -INFINITY;
    return 0.f;
  }
  // four consecutive entries from index 4*q; the caller has checked the 16-byte (float) / 4-byte (byte) alignment
  __device__ __forceinline__ float4 at4(int q) const {
    if (f) return __ldg(reinterpret_cast<const float4*>(f) + q);
    if (b) {
      const uchar4 m = __ldg(reinterpret_cast<const uchar4*>(b) + q);
      return make_float4(m.x ? 0.f : -INFINITY, m.y ? 0.f : -INFINITY, m.z ? 0.f : -INFINITY, m.w ? 0.f : -INFINITY);
    }
    return make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __device__ __forceinline__ bool aligned() const { return (reinterpret_cast<uintptr_t>(f) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 3) == 0; }
};
__device__ __forceinline__ MaskRow mask_row(const void* mask, int mask_type, long long row, int tk) {
  MaskRow m{nullptr, nullptr};
  if (mask && mask_type == B200_MASK_ADDITIVE) m.f = static_cast<const float*>(mask) + row * tk;
  if (mask && mask_type == B200_MASK_BYTES) m.b = static_cast<const unsigned char*>(mask) + row * tk;
  return m;
}

__device__ __forceinline__ float masked_score(float s, float scale, const MaskRow& m, int i, int j, int causal) {
  if (causal && j > i) return -INFINITY;
  return s * scale + m.at(j);
}

// ---- dropout: the reference's counter-based stream (csrc/shaders/philox.glsl; sdpa_training.comp:17) ------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3") keyed by the 64-bit seed; the counter
// is the 64-bit offset reserved for the call plus the element's block (four elements per block, one output word
// each).  An element is kept when its uniform in [0, 1) (top 24 bits of the word) is at least the dropout probability,
// and kept probabilities are scaled by 1 / (1 - p).
struct DropState {
  float p, keep_scale;   // dropout probability; 1 / (1 - p) (0 when p == 1)
  uint2 seed, offset;
};
__device__ __forceinline__ uint4 philox4x32_10(uint2 key, uint4 c) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ key.x, lo1, hi0 ^ c.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return c;
}
__device__ __forceinline__ uint4 drop_words(const DropState& d, uint32_t block) {
  const uint32_t low = d.offset.x + block;
  return philox4x32_10(d.seed, make_uint4(low, d.offset.y + (low < d.offset.x ? 1u : 0u), 0u, 0u));
}
__device__ __forceinline__ float keep_weight(const DropState& d, uint32_t word) {
  return (float)(word >> 8) * 0.000000059604644775390625f >= d.p ? d.keep_scale : 0.f;
}
// weight of element `index` (0 when dropped)
__device__ __forceinline__ float drop_weight(const DropState& d, uint32_t index) {
  if (d.p == 0.f) return 1.f;
  if (d.p >= 1.f) return 0.f;
  const uint4 r = drop_words(d, index >> 2);
  const uint32_t w = (index & 3u) == 0 ? r.x : (index & 3u) == 1 ? r.y : (index & 3u) == 2 ? r.z : r.w;
  return keep_weight(d, w);
}
// weights of the four elements of block `block` (index = 4 * block + i)
__device__ __forceinline__ float4 drop_weight4(const DropState& d, uint32_t block) {
  if (d.p == 0.f) return make_float4(1.f, 1.f, 1.f, 1.f);
  if (d.p >= 1.f) return make_float4(0.f, 0.f, 0.f, 0.f);
  const uint4 r = drop_words(d, block);
  return make_float4(keep_weight(d, r.x), keep_weight(d, r.y), keep_weight(d, r.z), keep_weight(d, r.w));
}

// One CTA per score row: s[j] <- softmax_j(s[j] * scale + mask), lse[row] <- log sum exp.
__global__ void __launch_bounds__(kThreads) softmax_rows_kernel(float* __restrict__ scores, const void* __restrict__ mask, int mask_type, int tq,
                                                                 int tk, float scale, int causal, float* __restrict__ lse,
                                                                 DropState drop) {
  __shared__ float scratch[kThreads / 32];
  const long long row = blockIdx.x;
  const int i = (int)(row % tq);
  float* s = scores + row * tk;
  const MaskRow mrow = mask_row(mask, mask_type, row, tk);
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < tk; j += kThreads) mx = fmaxf(mx, masked_score(s[j], scale, mrow, i, j, causal));
  mx = block_reduce<true>(mx, scratch);
  float sum = 0.f;
  if (mx > -INFINITY)
    for (int j = threadIdx.x; j < tk; j += kThreads) sum += expf(masked_score(s[j], scale, mrow, i, j, causal) - mx);
  sum = block_reduce<false>(sum, scratch);
  const float logsum = sum > 0.f ? mx + logf(sum) : -INFINITY;
  if (threadIdx.x == 0) lse[row] = logsum;
  const bool dead = !(logsum > -INFINITY);
  for (int j = threadIdx.x; j < tk; j += kThreads)
    s[j] = dead ? 0.f : expf(masked_score(s[j], scale, mrow, i, j, causal) - logsum) * drop_weight(drop, (uint32_t)(row * tk + j));
}

// The same for rows of at most 4096 keys that are whole 16-byte groups: the row is read once into
// registers (four groups of four per thread), reduced there and written once.
__global__ void __launch_bounds__(kThreads) softmax_rows_resident_kernel(float* __restrict__ scores, const void* __restrict__ mask,
                                                                          int mask_type, int tq, int tk, float scale, int causal,
                                                                          float* __restrict__ lse, DropState drop) {
  __shared__ float scratch[kThreads / 32];
  const long long row = blockIdx.x;
  const int i = (int)(row % tq), quads = tk >> 2;
  float4* s4 = reinterpret_cast<float4*>(scores + row * tk);
  const MaskRow mrow = mask_row(mask, mask_type, row, tk);
  float v[16];
  float mx = -INFINITY;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int q = threadIdx.x + u * kThreads;
    float4 a = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    if (q < quads) {
      a = s4[q];
      const float4 m = mrow.at4(q);
      const int j = 4 * q;
      a.x = (causal && j > i) ? -INFINITY : a.x * scale + m.x;
      a.y = (causal && j + 1 > i) ? -INFINITY : a.y * scale + m.y;
      a.z = (causal && j + 2 > i) ? -INFINITY : a.z * scale + m.z;
      a.w = (causal && j + 3 > i) ? -INFINITY : a.w * scale + m.w;
    }
    v[4 * u] = a.x, v[4 * u + 1] = a.y, v[4 * u + 2] = a.z, v[4 * u + 3] = a.w;
    mx = fmaxf(fmaxf(mx, fmaxf(a.x, a.y)), fmaxf(a.z, a.w));
  }
  mx = block_reduce<true>(mx, scratch);
  float sum = 0.f;
  if (mx > -INFINITY) {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      v[e] = expf(v[e] - mx);  // exp(-inf) = 0 for hidden keys and for the slots beyond the row
      sum += v[e];
    }
  }
  sum = block_reduce<false>(sum, scratch);
  const bool dead = !(sum > 0.f);
  if (threadIdx.x == 0) lse[row] = dead ? -INFINITY : mx + logf(sum);
  const float inv = dead ? 0.f : 1.f / sum;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int q = threadIdx.x + u * kThreads;
    if (q < quads) {
      // tk is a multiple of 4 here, so the four elements are one Philox block
      const float4 w = drop_weight4(drop, (uint32_t)((row * tk) >> 2) + (uint32_t)q);
      s4[q] = dead ? make_float4(0.f, 0.f, 0.f, 0.f)   // (the row's values are still -inf: no arithmetic on them)
                   : make_float4(v[4 * u] * inv * w.x, v[4 * u + 1] * inv * w.y, v[4 * u + 2] * inv * w.z, v[4 * u + 3] * inv * w.w);
    }
  }
}

// Backward, first elementwise step: s[j] <- P[j] = exp(s[j] * scale + mask - lse[row]).
__global__ void __launch_bounds__(kThreads) probabilities_kernel(float* __restrict__ scores, const void* __restrict__ mask, int mask_type, int tq,
                                                                  int tk, float scale, int causal, const float* __restrict__ lse) {
  const long long row = blockIdx.x;
  const int i = (int)(row % tq);
  float* s = scores + row * tk;
  const MaskRow mrow = mask_row(mask, mask_type, row, tk);
  const float logsum = __ldg(lse + row);
  const bool dead = !(logsum > -INFINITY);
  if ((tk & 3) == 0 && (reinterpret_cast<uintptr_t>(s) & 15) == 0 && mrow.aligned()) {
    float4* s4 = reinterpret_cast<float4*>(s);
    for (int q = threadIdx.x; q < (tk >> 2); q += kThreads) {
      const float4 a = s4[q], m = mrow.at4(q);
      const int j = 4 * q;
      float4 r;
      r.x = (dead || (causal && j > i)) ? 0.f : expf(a.x * scale + m.x - logsum);
      r.y = (dead || (causal && j + 1 > i)) ? 0.f : expf(a.y * scale + m.y - logsum);
      r.z = (dead || (causal && j + 2 > i)) ? 0.f : expf(a.z * scale + m.z - logsum);
      r.w = (dead || (causal && j + 3 > i)) ? 0.f : expf(a.w * scale + m.w - logsum);
      s4[q] = r;
    }
    return;
  }
  for (int j = threadIdx.x; j < tk; j += kThreads)
    s[j] = dead ? 0.f : expf(masked_score(s[j], scale, mrow, i, j, causal) - logsum);
}

// Backward, second step: dp[j] <- dS[j] = P[j] * (dp[j] * w[j] - delta) * scale with delta = sum_e dO[e] O[e]
// of the row and w the dropout weight (sdpa_training.comp:38); dmask[j] <- the same without the scale when the mask
// gradient is wanted; with dropout p[j] <- P[j] * w[j], which is what dV = (P w)^T dO contracts afterwards.
__global__ void __launch_bounds__(kThreads) score_gradient_kernel(float* __restrict__ dp, float* __restrict__ p,
                                                                   const float* __restrict__ grad, const float* __restrict__ out, int tk,
                                                                   int dv, float scale, float* __restrict__ dmask, DropState drop) {
  __shared__ float scratch[kThreads / 32];
  const long long row = blockIdx.x;
  float delta = 0.f;
  for (int e = threadIdx.x; e < dv; e += kThreads) delta = fmaf(__ldg(grad + row * dv + e), __ldg(out + row * dv + e), delta);
  delta = block_reduce<false>(delta, scratch);
  float* d = dp + row * tk;
  float* pr = p + row * tk;
  float* dm = dmask ? dmask + row * tk : nullptr;
  const bool dropping = drop.p != 0.f;
  if ((tk & 3) == 0 && ((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(pr) | reinterpret_cast<uintptr_t>(dm)) & 15) == 0) {
    float4* d4 = reinterpret_cast<float4*>(d);
    float4* dm4 = reinterpret_cast<float4*>(dm);
    float4* p4 = reinterpret_cast<float4*>(pr);
    for (int q = threadIdx.x; q < (tk >> 2); q += kThreads) {
      const float4 a = d4[q], b = p4[q];
      const float4 w = drop_weight4(drop, (uint32_t)((row * tk) >> 2) + (uint32_t)q);
      const float4 ds = make_float4(b.x * (a.x * w.x - delta), b.y * (a.y * w.y - delta), b.z * (a.z * w.z - delta), b.w * (a.w * w.w - delta));
      if (dm4) dm4[q] = ds;
      d4[q] = make_float4(ds.x * scale, ds.y * scale, ds.z * scale, ds.w * scale);
      if (dropping) p4[q] = make_float4(b.x * w.x, b.y * w.y, b.z * w.z, b.w * w.w);
    }
    return;
  }
  for (int j = threadIdx.x; j < tk; j += kThreads) {
    const float w = drop_weight(drop, (uint32_t)(row * tk + j));
    const float pj = pr[j], ds = pj * (d[j] * w - delta);
    if (dm) dm[j] = ds;
    d[j] = ds * scale;
    if (dropping) pr[j] = pj * w;
  }
}

__global__ void fill_kernel(float* p, float value, long long n) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) p[i] = value;
}

struct AttentionShape {
  int64_t batch, tq, tk, d, dv;
  size_t score_bytes;
};

int make_shape(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, AttentionShape* out) {
  if (batch < 0 || tq < 0 || tk < 0 || d < 0 || dv < 0) return fail(B200_EINVAL, "attention dimensions mismatch");
  if (tk > INT32_MAX || tq > INT32_MAX || dv > INT32_MAX || (tk > 0 && batch * tq > (int64_t)UINT32_MAX / tk))
    return fail(B200_ERANGE, "attention score indexing exceeds uint32");
  *out = {batch, tq, tk, d, dv, ((size_t)(batch * tq * tk) * sizeof(float) + 255) & ~(size_t)255};
  return B200_OK;
}

int make_drop(float dropout, const uint32_t* rng, DropState* d) {
  if (!(dropout >= 0.f && dropout <= 1.f)) return fail(B200_EINVAL, "invalid attention dropout");
  *d = DropState{dropout, dropout < 1.f ? 1.f / (1.f - dropout) : 0.f, make_uint2(0u, 0u), make_uint2(0u, 0u)};
  if (dropout > 0.f && dropout < 1.f) {
    if (!rng) return fail(B200_EINVAL, "attention dropout needs the four words of the random stream (seed, offset)");
    d->seed = make_uint2(rng[0], rng[1]);
    d->offset = make_uint2(rng[2], rng[3]);
  }
  return B200_OK;
}

int check_mask(const void* mask, int mask_type) {
  if (mask_type != B200_MASK_NONE && mask_type != B200_MASK_ADDITIVE && mask_type != B200_MASK_BYTES)
    return fail(B200_EINVAL, "attention mask shape/dtype mismatch");
  if ((mask_type != B200_MASK_NONE) != (mask != nullptr)) return fail(B200_EINVAL, "attention mask shape/dtype mismatch");
  return B200_OK;
}

// -inf -> 0 in place (rows with every key hidden)
__global__ void __launch_bounds__(kThreads) lse_finite_kernel(float* __restrict__ lse, long long count) {
  const long long i = blockIdx.x * (long long)kThreads + threadIdx.x;
  if (i < count && lse[i] == -INFINITY) lse[i] = 0.f;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_attention_workspace(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, int backward) {
  AttentionShape sh;
  if (make_shape(batch, tq, tk, d, dv, &sh)) return 0;
  return sh.score_bytes * (backward ? 2 : 1);
}

int b200_attention_forward(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, const float* q, const float* k,
                           const float* v, const void* mask, int mask_type, int causal, float scale, float dropout,
                           const uint32_t* rng, float* out, float* lse, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = ensure_init()) return rc;
  AttentionShape sh;
  if (int rc = make_shape(batch, tq, tk, d, dv, &sh)) return rc;
  if (int rc = check_mask(mask, mask_type)) return rc;
  DropState drop;
  if (int rc = make_drop(dropout, rng, &drop)) return rc;
  const int64_t rows = batch * tq;
  if (rows == 0) return B200_OK;
  if (!q || !out || !lse || (tk > 0 && (!k || !v))) return fail(B200_EINVAL, "attention: null tensor");
  cudaStream_t st = (cudaStream_t)stream;
  if (tk == 0) {  // no keys at all: zero output, log-sum-exp of an empty set (attention.cpp:20)
    if (dv) B200_CUDA(cudaMemsetAsync(out, 0, (size_t)rows * dv * sizeof(float), st));
    fill_kernel<<<(unsigned)((rows + kThreads - 1) / kThreads), kThreads, 0, st>>>(lse, -INFINITY, rows);
    count_launch();
    return launch_check("fill_kernel");
  }
  if (!workspace || workspace_bytes < sh.score_bytes) return fail(B200_EWORKSPACE, "attention: workspace smaller than b200_attention_workspace()");
  float* scores = (float*)workspace;
  // S[b] = Q[b] K[b]^T: the right-hand matrix is K read with its strides swapped
  if (int rc = b200_bmm(batch, tq, tk, d, q, tq * d, d, 1, k, tk * d, 1, d, scores, B200_ALGO_AUTO, stream)) return rc;
  const uintptr_t mask_align = mask_type == B200_MASK_BYTES ? 3 : 15;
  const bool resident = tk % 4 == 0 && tk <= 16 * kThreads && (reinterpret_cast<uintptr_t>(scores) & 15) == 0 &&
                        (reinterpret_cast<uintptr_t>(mask) & mask_align) == 0;
  if (resident) softmax_rows_resident_kernel<<<(unsigned)rows, kThreads, 0, st>>>(scores, mask, mask_type, (int)tq, (int)tk, scale, causal, lse, drop);
  else softmax_rows_kernel<<<(unsigned)rows, kThreads, 0, st>>>(scores, mask, mask_type, (int)tq, (int)tk, scale, causal, lse, drop);
  count_launch();
  if (int rc = launch_check("softmax_rows_kernel")) return rc;
  if (dv == 0) return B200_OK;
  const int rc = b200_bmm(batch, tq, dv, tk, scores, tq * tk, tk, 1, v, tk * dv, dv, 1, out, B200_ALGO_AUTO, stream);
  note_kernel("attention_forward: bmm + softmax_rows + bmm");
  return rc;
}

int b200_attention_lse_finite(float* lse, int64_t count, void* stream) {
  if (int rc = ensure_init()) return rc;
  if (count < 0 || (count > 0 && !lse)) return fail(B200_EINVAL, "attention: invalid log-sum-exp buffer");
  if (count == 0) return B200_OK;
  lse_finite_kernel<<<(unsigned)((count + kThreads - 1) / kThreads), kThreads, 0, (cudaStream_t)stream>>>(lse, count);
  count_launch();
  return launch_check("lse_finite_kernel");
}

int b200_attention_backward(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, const float* grad, const float* q,
                            const float* k, const float* v, const void* mask, int mask_type, const float* out, const float* lse,
                            int causal, float scale, float dropout, const uint32_t* rng, float* dq, float* dk, float* dvalue,
                            float* dmask, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = ensure_init()) return rc;
  AttentionShape sh;
  if (int rc = make_shape(batch, tq, tk, d, dv, &sh)) return rc;
  if (int rc = check_mask(mask, mask_type)) return rc;
  DropState drop;
  if (int rc = make_drop(dropout, rng, &drop)) return rc;
  if (!dq || !dk || !dvalue) return fail(B200_EINVAL, "attention backward: null gradient");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows = batch * tq;
  if (rows == 0 || tk == 0 || d == 0 || dv == 0) {  // nothing flows: all gradients are zero (attention.cpp:28)
    if (batch * tq * d) B200_CUDA(cudaMemsetAsync(dq, 0, (size_t)(batch * tq * d) * sizeof(float), st));
    if (batch * tk * d) B200_CUDA(cudaMemsetAsync(dk, 0, (size_t)(batch * tk * d) * sizeof(float), st));
    if (batch * tk * dv) B200_CUDA(cudaMemsetAsync(dvalue, 0, (size_t)(batch * tk * dv) * sizeof(float), st));
    if (dmask && rows * tk) B200_CUDA(cudaMemsetAsync(dmask, 0, (size_t)(rows * tk) * sizeof(float), st));
    return B200_OK;
  }
  if (!grad || !q || !k || !v || !out || !lse) return fail(B200_EINVAL, "attention backward: null tensor");
  if (!workspace || workspace_bytes < 2 * sh.score_bytes)
    return fail(B200_EWORKSPACE, "attention: workspace smaller than b200_attention_workspace()");
  float* p = (float*)workspace;
  float* dp = (float*)((char*)workspace + sh.score_bytes);
  if (int rc = b200_bmm(batch, tq, tk, d, q, tq * d, d, 1, k, tk * d, 1, d, p, B200_ALGO_AUTO, stream)) return rc;
  probabilities_kernel<<<(unsigned)rows, kThreads, 0, st>>>(p, mask, mask_type, (int)tq, (int)tk, scale, causal, lse);
  count_launch();
  if (int rc = launch_check("probabilities_kernel")) return rc;
  // dP[b] = dO[b] V[b]^T
  if (int rc = b200_bmm(batch, tq, tk, dv, grad, tq * dv, dv, 1, v, tk * dv, 1, dv, dp, B200_ALGO_AUTO, stream)) return rc;
  // dS in place of dP; with dropout P becomes P w for the product below
  score_gradient_kernel<<<(unsigned)rows, kThreads, 0, st>>>(dp, p, grad, out, (int)tk, (int)dv, scale, dmask, drop);
  count_launch();
  if (int rc = launch_check("score_gradient_kernel")) return rc;
  // dV[b] = (P w)[b]^T dO[b]
  if (int rc = b200_bmm(batch, tk, dv, tq, p, tq * tk, 1, tk, grad, tq * dv, dv, 1, dvalue, B200_ALGO_AUTO, stream)) return rc;
  // dQ[b] = dS[b] K[b];  dK[b] = dS[b]^T Q[b]
  if (int rc = b200_bmm(batch, tq, d, tk, dp, tq * tk, tk, 1, k, tk * d, d, 1, dq, B200_ALGO_AUTO, stream)) return rc;
  const int rc = b200_bmm(batch, tk, d, tq, dp, tq * tk, 1, tk, q, tq * d, d, 1, dk, B200_ALGO_AUTO, stream);
  note_kernel("attention_backward: bmm x5 + probabilities + score_gradient");
  return rc;
}

}  // extern "C"
