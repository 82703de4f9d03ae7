/*
 * b200conv.h - C ABI of the B200 (sm_100a) FP32 Conv2D / GEMM library.
 *
 * Plain C: pointers, sizes and POD structs only.  This is the boundary a host
 * extension binds to; the PyTorch PrivateUse1 extension shipped next to it
 * (csrc/torch_backend) and the ctypes binding (b200conv.py) call nothing else.
 *
 * The reference backend has no C plug-in interface of its own: its operators
 * are C++ functions registered with the PyTorch dispatcher that record Vulkan
 * compute dispatches.  Each entry point below therefore cites the reference
 * function whose device work it replaces (paths are inside the reference tree).
 *
 * Conventions
 *  - every function returns 0 on success or a negative B200_E* code; the text
 *    of the most recent failure on the calling thread is b200_last_error().
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *    All compute entry points are asynchronous with respect to the host.
 *  - tensors are FP32.  Inputs are described by b200_view4 (device pointer to
 *    element [0,0,0,0] plus four element strides, which may be zero, negative
 *    or non-monotone), so NCHW, channels-last, sliced, offset, transposed and
 *    broadcast views are consumed in place; outputs are contiguous NCHW, as in
 *    the reference (csrc/ops/convolution.cpp:662,685,689,693).
 *  - there is no CPU fallback: with no usable device every call fails.
 */
#ifndef B200CONV_H
#define B200CONV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_EINVAL (-1)      /* invalid shapes or parameters */
#define B200_ECUDA (-2)       /* a CUDA runtime/driver call failed */
#define B200_EWORKSPACE (-3)  /* workspace too small / forced candidate exceeds the budget */
#define B200_EUNSUPPORTED (-4)/* forced candidate not applicable to this geometry */
#define B200_ENOMEM (-5)
#define B200_ERANGE (-6)      /* int32 coordinate / uint32 element-count guards */
#define B200_EDEVICE (-7)     /* a device-side bounded wait gave up (status word set) */

/* The 16 push constants of the reference's ConvParams, same order
 * (csrc/ops/convolution.cpp:45-52). */
typedef struct {
  int32_t n, cin, cout, h, w, kh, kw, oh, ow;
  int32_t sh, sw, ph, pw, dh, dw, groups;
} b200_conv_params;

typedef struct {
  const float* ptr;   /* device address of element [0,0,0,0] (storage offset already applied) */
  int64_t stride[4];  /* element strides of the logical [N,C,H,W] / [Cout,Cin/g,kh,kw] view */
} b200_view4;

/* Phases and candidates: ConvPhase / ConvKind of csrc/ops/convolution.cpp:161-187. */
enum { B200_PHASE_FORWARD = 0, B200_PHASE_DINPUT = 1, B200_PHASE_DWEIGHT = 2, B200_PHASE_DBIAS = 3 };
enum {
  B200_ALGO_AUTO = 0,    /* heuristic (replaces `heuristic`, convolution.cpp:423-482) */
  B200_ALGO_DIRECT = 1,  /* one thread per output, loop order of the direct shaders (exact FP32 FMA) */
  B200_ALGO_TILED = 2,   /* CUDA-core FP32 implicit GEMM, any geometry / strides */
  B200_ALGO_TC = 3,      /* tcgen05 implicit GEMM, split-precision FP32 (TF32 hi*hi + cross terms) with FP32 accumulation in TMEM */
  B200_ALGO_WINOGRAD = 4 /* Winograd F(4x4,3x3) forward and dInput for 3x3 stride-1 dilation-1 filters (replaces winograd_f2) */
};

/* ---- runtime: replaces VulkanContext / VulkanAllocator --------------------------------- */

/* Select the device and create the library state.  Idempotent.
 * Replaces VulkanContext::instance() device pick, csrc/vulkan_context.cpp:59-83. */
int b200_init(int device_ordinal);
const char* b200_last_error(void);
/* csrc/torch_vulkan.cpp:181-183 (device_name) */
const char* b200_device_name(void);
int b200_device_sm_count(void);

/* Stream-ordered caching allocator: a block freed on a stream can be handed out
 * again on that stream at once, and on another stream after the free point has
 * been reached.  Replaces VulkanAllocator::allocate / free-list reuse,
 * csrc/vulkan_allocator.cpp:33-47,123-154. */
int b200_malloc(void** ptr, size_t bytes, void* stream);
int b200_free(void* ptr, void* stream);
int b200_empty_cache(void);
/* out[0..3] = bytes in use, bytes cached, cudaMalloc calls, cache hits */
int b200_mem_stats(uint64_t out[4]);
/* pinned host memory for staged transfers */
int b200_host_alloc(void** ptr, size_t bytes);
int b200_host_free(void* ptr);

enum { B200_H2D = 1, B200_D2H = 2, B200_D2D = 3 };
/* Asynchronous on `stream`; replaces the upload/download recording of
 * csrc/vulkan_context.cpp:98-112,172-211 and csrc/ops/device_copy.cpp. */
int b200_memcpy(void* dst, const void* src, size_t bytes, int kind, void* stream);
int b200_memset(void* dst, int value, size_t bytes, void* stream);
/* dst (contiguous, numel elements of elem_bytes = 1,2,4 or 8) <- strided view;
 * replaces conv2d_pack.comp / native_pack (csrc/ops/convolution.cpp:62-99) for the
 * copy_/contiguous plumbing.  Convolution itself never packs. */
int b200_gather_strided(void* dst, const void* src, int ndim, const int64_t* sizes,
                        const int64_t* strides, int elem_bytes, void* stream);
/* strided dst <- contiguous src (copy_ into a view) */
int b200_scatter_strided(void* dst, const void* src, int ndim, const int64_t* sizes,
                         const int64_t* strides, int elem_bytes, void* stream);

/* strided dst += contiguous src (FP32; the view must not alias itself): partial results accumulated into a slice of a
 * larger tensor (the depth taps of a 3-D dInput).  No counterpart in the reference. */
int b200_scatter_add_strided(float* dst, const float* src, int ndim, const int64_t* sizes, const int64_t* strides, void* stream);

/* dst (contiguous over the dimensions that are kept, in their order) <- sum of the FP32 strided view over the
 * dimensions with reduce[i] != 0.  The reduction the autograd graph of a broadcast operand needs (expand's backward,
 * `sum_to_size`): a broadcast attention mask, grouped-query key / value heads.  Stands for the reference's reduction
 * operator on this one signature (sum_dim, csrc/ops/reduce.cpp:24-35); one warp per result. */
int b200_sum_strided(float* dst, const float* src, int ndim, const int64_t* sizes, const int64_t* strides,
                     const unsigned char* reduce, void* stream);

/* Streams and events: replaces the single in-order queue and event sequences of
 * csrc/torch_vulkan.cpp:34-103 and csrc/vulkan_context.cpp:493-523. */
int b200_stream_create(void** stream);
int b200_stream_destroy(void* stream);
int b200_stream_sync(void* stream);
int b200_stream_query(void* stream); /* 1 = idle, 0 = busy, <0 = error */
int b200_device_sync(void);
int b200_event_create(void** event, int enable_timing);
int b200_event_destroy(void* event);
int b200_event_record(void* event, void* stream);
int b200_event_sync(void* event);
int b200_event_query(void* event);   /* 1 = complete, 0 = pending */
int b200_stream_wait_event(void* stream, void* event);
int b200_event_elapsed_ms(void* first, void* second, float* ms);

/* ---- convolution ----------------------------------------------------------------------- */

/* Validate a geometry and derive OH/OW: convolution_params, csrc/ops/convolution.cpp:101-156,
 * plus the element-count guards of dispatch (:559-560).  `wcin` is weight.size(1). */
int b200_conv2d_geometry(b200_conv_params* out, int64_t n, int64_t cin, int64_t cout, int64_t h,
                         int64_t w, int64_t wcin, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                         int64_t ph, int64_t pw, int64_t dh, int64_t dw, int64_t groups);

/* Candidate actually used for (geometry, phase) when `algo` is requested
 * (AUTO resolves through the heuristic); <0 if the forced candidate is not applicable.
 * Replaces applicable/candidates/heuristic, csrc/ops/convolution.cpp:357-482. */
int b200_conv2d_select(const b200_conv_params* p, int phase, int algo, size_t workspace_bytes);
/* Which kernel a forward / dInput call of the tcgen05 candidate runs for this activation view (x for
 * forward, dy for dInput; only the strides are read, the pointer is not dereferenced):
 * 0 = strip kernel; 1 = per-tap gather kernel (views that span 2^31 elements or more, reduction
 * channels in whole blocks of 32); 2 = CUDA-core implicit GEMM (such a view with a ragged channel
 * count, which the gather kernel would truncate); 3 = transposed strip kernel (filter on the M side, 65 or
 * more output channels per group; 64-bit view offsets).  <0 if the candidate does not take the geometry.
 * Part of execute_candidate's role, csrc/ops/convolution.cpp:483-520 (kernel choice per memory class). */
int b200_conv2d_tc_route(const b200_conv_params* p, int phase, b200_view4 act);
/* Scratch bytes the selected candidate wants (0 = none).  For dWeight this is the
 * split-K partial buffer of weight_split_plan, csrc/ops/convolution.cpp:204-238;
 * a smaller non-zero budget yields fewer, longer splits. */
size_t b200_conv2d_workspace(const b200_conv_params* p, int phase, int algo, size_t budget_bytes);

/* y = conv(x, w) + bias.  Replaces convolution_overrideable's dispatch
 * (csrc/ops/convolution.cpp:641-665) and the conv2d_forward, conv2d_tiled_<tile>,
 * conv2d_depthwise and conv2d_winograd_<stage> shaders.  bias may be NULL (the reference binds
 * a shared zero buffer, :660).  y: contiguous [n,cout,oh,ow]. */
int b200_conv2d_forward(const b200_conv_params* p, b200_view4 x, b200_view4 w, const float* bias,
                        int64_t bias_stride, float* y, void* workspace, size_t workspace_bytes,
                        int algo, void* stream);
/* y = act(conv(x, w) + bias + residual), optionally written channels-last.  No single counterpart in
 * the reference: it fuses the convolution with the add.Tensor / relu the reference registers as
 * separate operators (csrc/ops/mm.cpp:1094-1097) and that follow it in ResNet / U-Net blocks.
 * residual: view of the result's logical shape [n,cout,oh,ow] (any strides), ptr NULL = none.
 * relu: 0 or 1.  y_channels_last = 0: y contiguous [n,cout,oh,ow]; 1: y contiguous [n,oh,ow,cout],
 * available when the tcgen05 strip kernel takes the geometry (else B200_EUNSUPPORTED, "incompatible").
 * With the strip kernel everything happens in its epilogue; other candidates run the plain forward
 * followed by one elementwise pass.  Workspace and algo as for b200_conv2d_forward. */
int b200_conv2d_forward_fused(const b200_conv_params* p, b200_view4 x, b200_view4 w, const float* bias,
                              int64_t bias_stride, b200_view4 residual, int relu, float* y, int y_channels_last,
                              void* workspace, size_t workspace_bytes, int algo, void* stream);
/* dx = conv_transpose(dy, w).  Replaces dispatch(Input), csrc/ops/convolution.cpp:684-687 and
 * the conv2d_backward_input shaders.  dx: contiguous [n,cin,h,w]. */
int b200_conv2d_dinput(const b200_conv_params* p, b200_view4 dy, b200_view4 w, float* dx,
                       void* workspace, size_t workspace_bytes, int algo, void* stream);
/* y = conv_transpose2d(x, w) + bias: the transposed ("fractionally strided") convolution, which is
 * the input gradient of an ordinary convolution.  `p` describes THAT convolution: p->n samples,
 * (p->cin, p->h, p->w) are the channels and extent of the RESULT y, (p->cout, p->oh, p->ow) those of
 * x, and w is [p->cout, p->cin / groups, kh, kw], the layout PyTorch gives a transposed convolution's
 * weight.  An output_padding is expressed through p->h / p->w (b200_conv2d_geometry must map them
 * back to x's extent).  bias: p->cin values or NULL.  y: contiguous [n, cin, h, w].
 * Replaces the transposed branch of convolution_nd (csrc/ops/convolution_nd.cpp:46-56, shader
 * convolution_nd.comp), to which the reference's convolution entry point delegates
 * (csrc/ops/convolution.cpp:647).  Its gradients need no entry points of their own: with g the
 * gradient of y, dx = b200_conv2d_forward(p, g, w), dw = b200_conv2d_dweight(p, g as x, x as dy),
 * and db = b200_conv2d_dbias over g. */
int b200_conv_transpose2d_forward(const b200_conv_params* p, b200_view4 x, b200_view4 w, const float* bias,
                                  int64_t bias_stride, float* y, void* workspace, size_t workspace_bytes, int algo,
                                  void* stream);
/* dw = dy (*) x summed over batch and positions.  Replaces dispatch(Weight), :688-691,
 * the conv2d_backward_weight shaders (direct, reduce, tiled, finalize).  The split-K partials are summed in
 * ascending split order (no float atomics), so results are run-to-run identical.
 * dw: contiguous [cout,cin/g,kh,kw]. */
int b200_conv2d_dweight(const b200_conv_params* p, b200_view4 x, b200_view4 dy, float* dw,
                        void* workspace, size_t workspace_bytes, int algo, void* stream);
/* db[co] = sum dy.  Replaces dispatch(Bias), :692-695, conv2d_backward_bias{,_reduce}.
 * workspace may be NULL (then a single pass per channel is used). */
int b200_conv2d_dbias(const b200_conv_params* p, b200_view4 dy, float* db, void* workspace,
                      size_t workspace_bytes, void* stream);

/* dWeight for callers that cannot allocate device memory (no counterpart in the reference).
 * Same result as b200_conv2d_dweight with the CUDA-core split-K kernel, but the split-K scratch
 * is a fixed B200_STATIC_SCRATCH_BYTES array inside the library's device image, so the call
 * performs no cudaMalloc/cudaFree and takes no workspace argument.  Meant for hosts whose
 * device memory is entirely owned by their own pool, or whose hot loop cannot tolerate the
 * implicit synchronisation of an allocation.  Requirements and limits:
 *  - b200_init must have been called before (initialisation allocates; this call does not);
 *  - fails with B200_EWORKSPACE when 2 * numel(dw) * 4 bytes exceed B200_STATIC_SCRATCH_BYTES;
 *  - the array is shared by all calls and occupies device memory on every GPU that loads the
 *    library until process exit; calls whose kernels may overlap on the GPU (different streams)
 *    race on it and must be ordered by the caller; nothing needs clearing between calls;
 *  - the first call on a device resolves the array's address and should be made outside any
 *    stream capture. */
#define B200_STATIC_SCRATCH_BYTES (16u << 20)
int b200_conv2d_dweight_static(const b200_conv_params* p, b200_view4 x, b200_view4 dy, float* dw,
                               void* stream);

/* ---- generic N-d convolution (3-D and integer tensors) ------------------------------------ */

/* Geometry of a convolution with 1 to 3 spatial dimensions, ordinary or transposed.  Arrays hold
 * depth, height, width; a lower rank fills the trailing entries and leaves the leading ones at
 * extent 1 / stride 1 / padding 0.  Mirrors the reference's `geometry()` parameter block
 * (csrc/ops/convolution_nd.cpp:7-43). */
typedef struct b200_convnd_params {
  int32_t rank, transposed;
  int64_t n, cin, cout, groups;
  int64_t in[3], out[3], k[3], stride[3], pad[3], dilation[3];
} b200_convnd_params;

/* Validates and fills `out`.  `in_sizes`, `kernel`, `stride`, `pad`, `dilation`, `output_pad` have
 * `rank` entries; w0, w1 are the first two weight extents ([cout][cin/groups] ordinary,
 * [cin][cout/groups] transposed).  Same checks and messages as csrc/ops/convolution_nd.cpp:13-40. */
int b200_convnd_geometry(b200_convnd_params* out, int rank, int64_t n, int64_t cin,
                         const int64_t* in_sizes, int64_t w0, int64_t w1, const int64_t* kernel,
                         const int64_t* stride, const int64_t* pad, const int64_t* dilation,
                         const int64_t* output_pad, int transposed, int64_t groups);

/* y = conv(x, w) + bias on contiguous tensors; FP32 (is_int64 == 0) or int64 with wrapping
 * arithmetic (is_int64 != 0; csrc/ops/convolution_nd.cpp:57-61, shader convolution_nd_int64).  bias may be
 * NULL.  One thread per output element, like shader mode 0 (csrc/ops/convolution_nd.cpp:45-49,62) -- except FP32 calls
 * over three spatial dimensions of 2^24 multiply-adds or more, which are decomposed over the depth taps into calls of the
 * 2-D kernels (tcgen05 from 16 channels per group; scratch comes from b200_malloc on `stream`). */
int b200_convnd_forward(const b200_convnd_params* p, const void* x, const void* w,
                        const void* bias, void* y, int is_int64, void* stream);

/* FP32 gradients on contiguous tensors; a NULL result pointer skips that gradient (shader modes
 * 1 dInput, 2 dWeight, 3 dBias; csrc/ops/convolution_nd.cpp:65-74).  Wide 3-D calls run the 2-D tcgen05 kernels per
 * depth tap as in the forward call. */
int b200_convnd_backward(const b200_convnd_params* p, const float* grad, const float* x,
                         const float* w, float* dx, float* dw, float* db, void* stream);

/* ---- GEMM (nn.Linear neighbours of the conv path) -------------------------------------- */

/* C[M,N] (contiguous) = alpha * A*B + (beta == 0 ? 0 : beta * bias[n]); A, B arbitrary 2-D
 * element strides; bias NULL = plain mm.  Replaces mm_impl (csrc/ops/mm.cpp:244-343) and
 * addmm_bias_vulkan (:835-879) with matmul_strided{,_reg}{,_bias}.comp. */
int b200_gemm(int64_t M, int64_t N, int64_t K, const float* A, int64_t sa0, int64_t sa1,
              const float* B, int64_t sb0, int64_t sb1, const float* bias, float alpha, float beta,
              float* C, int algo, void* stream);

/* ---- BatchNorm (the normalisation either side of a convolution) --------------------------- */

/* Memory layout of the FP32 tensors of a batch-norm call.  The logical shape is [n, c, s] with s the
 * product of the trailing dimensions; the reference first packs every input to the contiguous form
 * (csrc/ops/batch_norm.cpp:30, `packed(input)`), here a channels-last tensor is consumed as it is. */
enum {
  B200_BN_PLANAR = 0,      /* contiguous [n][c][s] (NCHW and its 1-D/3-D relatives) */
  B200_BN_INTERLEAVED = 1  /* contiguous [n][s][c] (channels-last); y / dx are written the same way */
};

/* Bytes of workspace the two calls below need for this shape (0 on invalid shapes).  The workspace
 * holds per-channel coefficients and the partial reductions; it must be 16-byte aligned. */
size_t b200_batch_norm_workspace(int64_t n, int64_t c, int64_t s, int layout);

/* y = (x - mean) * inv * weight + bias per channel.  Replaces batch_norm (csrc/ops/batch_norm.cpp:21-83)
 * with the shaders batch_norm_forward.comp (training, and evaluation of small tensors) and
 * batch_norm_eval.comp.
 *  - training != 0: mean and biased variance over the n*s values of each channel; save_mean[c] and
 *    save_inv[c] = 1/sqrt(var + eps) (0 when var == 0 and eps == 0) are written (contiguous);
 *    running_mean / running_var, when not NULL, are updated in place with `momentum`, the variance
 *    with the unbiased estimate (NaN for n*s == 1, as in the reference).
 *  - training == 0: running_mean and running_var are required and read only; save_* are not touched.
 *  weight, bias, running_* are channel vectors with an element stride each (NULL = absent).
 *  Fails with B200_ERANGE above INT32_MAX elements (the reference stops at UINT32_MAX, :19). */
int b200_batch_norm_forward(int64_t n, int64_t c, int64_t s, int layout, const float* x, const float* weight,
                            int64_t weight_stride, const float* bias, int64_t bias_stride, float* running_mean,
                            int64_t running_mean_stride, float* running_var, int64_t running_var_stride, int training,
                            float momentum, float eps, float* y, float* save_mean, float* save_inv, void* workspace,
                            size_t workspace_bytes, void* stream);

/* The call above followed by `+ residual` (a tensor of x's shape and layout, NULL = none) and a
 * ReLU (relu != 0) in the same pass that writes y: the add.Tensor / relu pair that follows a BatchNorm
 * in a residual block (csrc/ops/mm.cpp:1094-1097 registers them as separate elementwise operators;
 * no fused counterpart exists in the reference).  save_mean / save_inv and the running statistics
 * are those of the plain call. */
int b200_batch_norm_forward_fused(int64_t n, int64_t c, int64_t s, int layout, const float* x, const float* weight,
                                  int64_t weight_stride, const float* bias, int64_t bias_stride, float* running_mean,
                                  int64_t running_mean_stride, float* running_var, int64_t running_var_stride, int training,
                                  float momentum, float eps, const float* residual, int relu, float* y, float* save_mean,
                                  float* save_inv, void* workspace, size_t workspace_bytes, void* stream);

/* Gradients of the call above.  Replaces batch_norm_backward (csrc/ops/batch_norm.cpp:84-113) and
 * batch_norm_backward.comp.  dx, dw, db: NULL = not wanted (the reference's output mask).
 *  - training != 0: mean / inv_or_var are save_mean / save_inv of the forward call;
 *    db = sum g, dw = sum (x - mean) g * inv, dx = (g - db/m - (x - mean) * dw * inv / m) * inv * weight.
 *    With two values per channel the algebraic form of batch_norm_backward.comp:24-37 is used.
 *  - training == 0: mean / inv_or_var are the running mean and variance; dx = g * weight / sqrt(var + eps). */
int b200_batch_norm_backward(int64_t n, int64_t c, int64_t s, int layout, const float* grad, const float* x,
                             const float* weight, int64_t weight_stride, const float* mean, int64_t mean_stride,
                             const float* inv_or_var, int64_t inv_stride, int training, float eps, float* dx, float* dw,
                             float* db, void* workspace, size_t workspace_bytes, void* stream);

/* ---- GroupNorm ---------------------------------------------------------------------------------- */

/* All tensors contiguous FP32: x, y, grad, dx [n][c][hw]; weight, bias, dw, db [c]; mean, rstd
 * [n][groups] (the reference packs every operand first, csrc/ops/group_norm.cpp:97-99,134-135).
 * Bytes of workspace the backward call needs when dw or db is asked for (0 on invalid shapes). */
size_t b200_group_norm_workspace(int64_t n, int64_t c, int64_t hw, int64_t groups);

/* y = (x - mean) * rstd * weight + bias with mean / rstd = 1/sqrt(var + eps) over each (sample,
 * group) block of c/groups * hw values; mean and rstd are written.  weight / bias NULL = absent.
 * Replaces forward (csrc/ops/group_norm.cpp:76-109) and group_norm_forward.comp.
 * More than 4096 channels per group: B200_EUNSUPPORTED. */
int b200_group_norm_forward(int64_t n, int64_t c, int64_t hw, int64_t groups, const float* x, const float* weight,
                            const float* bias, float eps, float* y, float* mean, float* rstd, void* stream);

/* dx, dw (weight gradient), db (bias gradient); NULL = not wanted.  Replaces backward
 * (csrc/ops/group_norm.cpp:111-155) with group_norm_backward_input.comp and
 * group_norm_backward_affine.comp; one pass over x and grad feeds all three results. */
int b200_group_norm_backward(int64_t n, int64_t c, int64_t hw, int64_t groups, const float* grad, const float* x,
                             const float* mean, const float* rstd, const float* weight, float* dx, float* dw, float* db,
                             void* workspace, size_t workspace_bytes, void* stream);

/* C[b] (contiguous [batch, M, N]) = A[b] * B[b]; A and B arbitrary 3-D element strides (a zero batch
 * stride broadcasts one matrix).  Replaces bmm_impl (csrc/ops/bmm.cpp:16-68, shader bmm_strided.comp).
 * K == 0 gives zeros, as there (:50-54).  From 64 rows, 16 columns and a contraction of 16 every
 * batch runs in ONE launch of the tcgen05 GEMM kernel (the batch rides on its group dimension); a
 * right-hand matrix shared by all batches with left-hand rows at one stride folds into a single
 * product; smaller shapes are one b200_gemm per batch. */
int b200_bmm(int64_t batch, int64_t M, int64_t N, int64_t K, const float* A, int64_t sa_b, int64_t sa0, int64_t sa1,
             const float* B, int64_t sb_b, int64_t sb0, int64_t sb1, float* C, int algo, void* stream);

/* ---- scaled dot-product attention ---------------------------------------------------------------- */

/* Kinds of attention mask (masktype of csrc/ops/attention.cpp:12): none; additive FP32; one byte per
 * score where zero hides the key (the storage of a bool tensor). */
enum { B200_MASK_NONE = 0, B200_MASK_ADDITIVE = 1, B200_MASK_BYTES = 2 };

/* q [batch, tq, d], k [batch, tk, d], v [batch, tk, dv], out / grad [batch, tq, dv], lse [batch, tq],
 * mask NULL (mask_type B200_MASK_NONE) or [batch, tq, tk] of the stated kind; all contiguous (the
 * reference packs them, csrc/ops/attention.cpp:21,29).  causal != 0 hides keys j > i.
 * dropout in [0, 1]: probability of dropping a (query, key) probability; kept ones are scaled by 1 / (1 - dropout).
 * For 0 < dropout < 1, rng points to four host words {seed low, seed high, offset low, offset high}: the
 * Philox4x32-10 stream of the reference (csrc/shaders/philox.glsl; state layout of VulkanGenerator::reserve,
 * csrc/vulkan_generator.cpp:17-20), element (row, key) drawing word (row * tk + key) % 4 of block
 * offset + (row * tk + key) / 4.  The backward call must get the same dropout and rng as its forward call.
 * Workspace: the score matrix (forward) or two of them (backward != 0). */
size_t b200_attention_workspace(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, int backward);

/* out = softmax(q k^T * scale + mask) v and the per-row log-sum-exp.  Replaces attention_forward
 * (csrc/ops/attention.cpp:16-23, shader sdpa_training.comp mode 0).  Composed from b200_bmm and one
 * row-softmax kernel; the scores are materialised in the workspace. */
int b200_attention_forward(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, const float* q, const float* k,
                           const float* v, const void* mask, int mask_type, int causal, float scale, float dropout,
                           const uint32_t* rng, float* out, float* lse, void* workspace, size_t workspace_bytes, void* stream);

/* Replaces -inf by 0 in a log-sum-exp buffer, in place: what the reference's operator
 * _scaled_dot_product_flash_attention_for_cpu returns for rows with every key hidden
 * (csrc/ops/attention.cpp, cpu_flash_forward_native: at::where(isneginf(lse), 0, lse)).
 * b200_attention_backward accepts either form: a hidden key's score is -inf, so its probability is 0. */
int b200_attention_lse_finite(float* lse, int64_t count, void* stream);

/* dq, dk, dvalue from the output gradient, the saved output and log-sum-exp, and, when dmask is not
 * NULL, the gradient of an additive mask [batch, tq, tk]: P (dP - rowsum(dO O)), the score gradient
 * before the scale.  Replaces attention_backward (csrc/ops/attention.cpp:24-34, sdpa_training.comp
 * modes 1 and 2, whose mode 1 writes the same `dm`). */
int b200_attention_backward(int64_t batch, int64_t tq, int64_t tk, int64_t d, int64_t dv, const float* grad, const float* q,
                            const float* k, const float* v, const void* mask, int mask_type, const float* out, const float* lse,
                            int causal, float scale, float dropout, const uint32_t* rng, float* dq, float* dk, float* dvalue,
                            float* dmask, void* workspace, size_t workspace_bytes, void* stream);

/* ---- data-parallel exchange (batch sharded over GPUs, one process per GPU) ------------------------ */

/* These entry points have no counterpart in the reference, which is single-device
 * (csrc/torch_vulkan.cpp:105-107: deviceCount() == 1).  Forward and dInput are local to a rank; the
 * weight and bias gradients of a layer are summed over ranks with one all-reduce (NCCL over NVLink),
 * which the caller may issue on a second stream so that it runs under the next layer's kernels.
 * NCCL is bound at run time (dlopen): a process that never calls these loads no communication library.
 *
 * b200_comm_unique_id: rank 0 fills 128 opaque bytes and hands them to every rank by its own means.
 * b200_comm_init: every rank calls it with the same id after b200_init; returns once all nranks have
 *   joined, or fails with B200_ECUDA after the timeout (default 60 s, b200_comm_set_timeout_ms) with the
 *   half-built communicator aborted, so a rank that never joins cannot hang the others.
 * b200_allreduce_sum_f32: in-place sum of `count` floats over all ranks, asynchronous on `stream`.
 * b200_comm_destroy: releases the communicator (idempotent).  b200_comm_rank / _size: -1 / 0 before init. */
int b200_comm_unique_id(void* out128);
int b200_comm_set_timeout_ms(int timeout_ms);
int b200_comm_init(int rank, int nranks, const void* unique_id128);
int b200_comm_rank(void);
int b200_comm_size(void);
int b200_allreduce_sum_f32(float* buf, size_t count, void* stream);
int b200_comm_destroy(void);

/* Device-side health word.  The tcgen05 kernels bound every wait on an mbarrier; a wait that
 * gives up records (code << 24 | CTA index) here, frees its tensor memory and returns, so the
 * context stays usable.  *status = 0 means no wait ever gave up.  Synchronises the device.
 * (No counterpart in the reference: Vulkan fences time out on the host, csrc/vulkan_context.cpp:493-499.) */
int b200_device_status(int* status, int clear);

/* ---- statistics ------------------------------------------------------------------------ */

/* Number of kernels this library has launched since load (all streams). */
uint64_t b200_launch_count(void);
/* Name of the kernel family the last conv/gemm call on this thread launched
 * (e.g. "tc_igemm_fwd", "simt_igemm_dweight+finalize"). */
const char* b200_last_kernel(void);

#ifdef __cplusplus
}
#endif
#endif /* B200CONV_H */
