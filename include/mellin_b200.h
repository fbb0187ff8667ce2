/* mellin_b200 -- C ABI of the B200 (sm_100a) Mellin / linear correlation and
 * convolution kernels.
 *
 * Every entry point takes plain device pointers, 64-bit extents and a CUDA
 * stream (passed as void*; a cudaStream_t is a pointer).  Nothing here
 * depends on PyTorch.  All calls are asynchronous with respect to the host:
 * they enqueue work on `stream` and return.  The caller owns every buffer.
 * One exception: the FIRST call of a geometry (kernel / signal / output extents
 * on the Mellin axis with s, d, p, u) on a device builds its index table on the
 * host, allocates device memory for it and uploads it with a synchronous copy,
 * so that call blocks, allocates, and cannot be part of a stream capture.  The
 * tables (a few KB to a few MB each) are kept per device until
 * mellin_clear_tables(); nothing evicts them, so a caller that feeds a 1-D
 * Mellin operator signals of ever-changing length should call it now and then.
 * The operator-level entry points without a workspace argument also keep one
 * scratch arena per (device, stream), grown on demand and freed by the same call.
 *
 * Return value: MELLIN_OK (0) or one of the error codes below; a
 * human-readable description of the most recent failure on the calling thread
 * is available from mellin_last_error().  Kernels never trap; a failed launch
 * is reported through the return code.
 *
 * Notation (as in the reference, sdrobert/cnn-mellin): f = kernel / weight,
 * g = signal / input, h = result.  "x" is the Mellin axis (dim 2), "y" the
 * linear axis (dim 3, contiguous).  With P = p + 1 the taps that contribute are
 * the integer solutions of
 *     Mellin correlation:  (hx + s)(fx + d) = P (gx + u)
 *     Mellin convolution:  P (hx + s)       = (fx + d)(gx + u)
 *     linear correlation:  s hy + d fy - p  = u gy
 *     linear convolution:  s hy - d fy + p  = u gy
 * with 0 <= g < ng.
 */
#ifndef MELLIN_B200_H_
#define MELLIN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MELLIN_OK = 0,
  MELLIN_ERR_BAD_ARGUMENT = 1, /* null pointer, negative extent, zero divisor ... */
  MELLIN_ERR_LAUNCH = 2,       /* CUDA reported an error for an allocation, copy or launch */
  MELLIN_ERR_WORKSPACE = 3,    /* workspace missing or smaller than the *_workspace_bytes() answer */
  MELLIN_ERR_UNSUPPORTED = 4   /* extent beyond what the kernels index (2^31 - 1 per tensor axis product) */
};

/* Version of this ABI (major * 100 + minor). */
int mellin_abi_version(void);

/* Description of the last error raised on the calling thread ("" if none). */
const char *mellin_last_error(void);

/* ---- output sizes ---------------------------------------------------------
 * Replace the constexpr functions of the reference at
 * ext/include/cdrobert/mellin/mconv.h:452-672 (Python twins mconv.py:73-118).
 * "valid": every tap reads inside the signal; "support": at least one tap can.
 */
int64_t mellin_mconv_valid_size(int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u);
int64_t mellin_mconv_support_size(int64_t nf, int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u);
int64_t mellin_mcorr_valid_size(int64_t nf, int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u);
int64_t mellin_mcorr_support_size(int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u);
int64_t mellin_lconv_valid_size(int64_t ng, int64_t s, int64_t p, int64_t u);
int64_t mellin_lconv_support_size(int64_t nf, int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u);
int64_t mellin_lcorr_valid_size(int64_t nf, int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u);
int64_t mellin_lcorr_support_size(int64_t ng, int64_t s, int64_t p, int64_t u);

/* ---- operator-level entry points (accumulate into h) -----------------------
 * Drop-in for the reference's device entry points MConv1DCuda, MCorr1DCuda,
 * MConvLConvCuda and MCorrLCorrCuda
 * (ext/include/cdrobert/mellin/mconv_cuda.cuh:23-71, launchers :962-1052):
 * same argument order and meaning.  h must be allocated and initialised by
 * the caller (bias or zero); results are ADDED to it.  A non-zero
 * transposed_* flag says the operand's two leading extents are swapped in
 * memory: f is (c_in, c_out, ...), g is (c_in, batch, ...), h is
 * (c_out, batch, ...).
 */
#define MELLIN_DECL_OP1D(name, T)                                                    \
  int name(const T *f, const T *g, int64_t c_out, int64_t c_in, int64_t batch,        \
           int64_t nf, int64_t ng, int64_t nh, int64_t s, int64_t d, int64_t p,       \
           int64_t u, int transposed_f, int transposed_g, int transposed_h, T *h,    \
           void *stream)
#define MELLIN_DECL_OP2D(name, T)                                                    \
  int name(const T *f, const T *g, int64_t c_out, int64_t c_in, int64_t batch,        \
           int64_t nfx, int64_t nfy, int64_t ngx, int64_t ngy, int64_t nhx,           \
           int64_t nhy, int64_t sx, int64_t sy, int64_t dx, int64_t dy, int64_t px,   \
           int64_t py, int64_t ux, int64_t uy, int transposed_f, int transposed_g,   \
           int transposed_h, T *h, void *stream)

MELLIN_DECL_OP1D(mellin_mconv1d_f32, float);    /* mconv_cuda.cuh:23-33   */
MELLIN_DECL_OP1D(mellin_mconv1d_f64, double);
MELLIN_DECL_OP1D(mellin_mcorr1d_f32, float);    /* mconv_cuda.cuh:35-45   */
MELLIN_DECL_OP1D(mellin_mcorr1d_f64, double);
MELLIN_DECL_OP2D(mellin_mconvlconv_f32, float); /* mconv_cuda.cuh:47-58   */
MELLIN_DECL_OP2D(mellin_mconvlconv_f64, double);
MELLIN_DECL_OP2D(mellin_mcorrlcorr_f32, float); /* mconv_cuda.cuh:60-71   */
MELLIN_DECL_OP2D(mellin_mcorrlcorr_f64, double);

/* ---- column operators (every output element is written) --------------------
 * Drop-in for Snd2ColCuda, Col2SndCuda, Spec2ColCuda, Col2SpecCuda
 * (mconv_cuda.cuh:73-121, launchers :1054-1151).
 *   snd2col : g (batch, c_in, ng)            -> gg (batch, c_in, nf, ngg)
 *   col2snd : gg                             -> g    (adjoint: gather-sum)
 *   spec2col: g (batch, c_in, ngx, ngy)      -> gg (batch, c_in, nfx, nfy, nggx, nggy)
 *   col2spec: gg                             -> g
 */
#define MELLIN_DECL_COL1D(name, T, in, out)                                          \
  int name(const T *in, int64_t c_in, int64_t batch, int64_t nf, int64_t ng,          \
           int64_t ngg, int64_t s, int64_t d, int64_t p, int64_t u,                   \
           int transposed_g, int transposed_gg, T *out, void *stream)
#define MELLIN_DECL_COL2D(name, T, in, out)                                          \
  int name(const T *in, int64_t c_in, int64_t batch, int64_t nfx, int64_t nfy,        \
           int64_t ngx, int64_t ngy, int64_t nggx, int64_t nggy, int64_t sx,          \
           int64_t sy, int64_t dx, int64_t dy, int64_t px, int64_t py, int64_t ux,    \
           int64_t uy, int transposed_g, int transposed_gg, T *out, void *stream)

MELLIN_DECL_COL1D(mellin_snd2col_f32, float, g, gg);   /* mconv_cuda.cuh:73-83   */
MELLIN_DECL_COL1D(mellin_snd2col_f64, double, g, gg);
MELLIN_DECL_COL1D(mellin_col2snd_f32, float, gg, g);   /* mconv_cuda.cuh:85-95   */
MELLIN_DECL_COL1D(mellin_col2snd_f64, double, gg, g);
MELLIN_DECL_COL2D(mellin_spec2col_f32, float, g, gg);  /* mconv_cuda.cuh:97-108  */
MELLIN_DECL_COL2D(mellin_spec2col_f64, double, g, gg);
MELLIN_DECL_COL2D(mellin_col2spec_f32, float, gg, g);  /* mconv_cuda.cuh:110-121 */
MELLIN_DECL_COL2D(mellin_col2spec_f64, double, gg, g);

/* ---- layer-level entry points ----------------------------------------------
 * One call per tensor a correlation layer produces; they replace what the
 * reference composes in its torch binding out of the operators above:
 *   forward     = BuildOutput (bias broadcast / zero fill) followed by
 *                 mcorrlcorr (ext/torch.cpp:88-101, ext/torch_cuda.cu:144-177);
 *   grad_input  = mconvlconv(weight^T, grad_out, (s,d,p,u) <- (u,s,p,d))^T
 *                 (ext/torch.cpp:282-290);
 *   grad_weight = mcorrlcorr(input^T, grad_out^T, (s,d,p,u) <- (d,s,p,u))^T and
 *                 grad_bias = grad_out.sum over batch and positions
 *                 (ext/torch.cpp:292-300).
 * All tensors are contiguous, untransposed:
 *   x (batch, c_in, ngx, ngy), w (c_out, c_in, nfx, nfy), bias (c_out) or NULL,
 *   y / grad_y (batch, c_out, nhx, nhy).
 * Outputs are WRITTEN (no pre-initialisation needed).  The 1-D Mellin layer
 * is the case nfy = ngy = nhy = 1, sy = dy = uy = 1, py = 0.
 */
#define MELLIN_LAYER_GEOMETRY                                                        \
  int64_t batch, int64_t c_in, int64_t c_out, int64_t nfx, int64_t nfy, int64_t ngx,  \
  int64_t ngy, int64_t nhx, int64_t nhy, int64_t sx, int64_t sy, int64_t dx,          \
  int64_t dy, int64_t px, int64_t py, int64_t ux, int64_t uy

/* Scratch for the tensor-core path of forward / grad_input (packed hi/lo weight
 * copies; 37 KB for a 3->64 channel 8x3 kernel).  0 means the geometry is served
 * by the CUDA-core kernels and needs none. */
size_t mellin_mcorrlcorr_forward_workspace_bytes(MELLIN_LAYER_GEOMETRY);
size_t mellin_mcorrlcorr_grad_input_workspace_bytes(MELLIN_LAYER_GEOMETRY);

/* workspace: at least the *_workspace_bytes() answer, 16-byte aligned, clobbered.
 * With a NULL or smaller workspace the call still succeeds on the CUDA-core
 * kernels (float64 always uses them). */
int mellin_mcorrlcorr_forward_f32(const float *x, const float *w, const float *bias,
                                  MELLIN_LAYER_GEOMETRY, float *y, void *workspace,
                                  size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_forward_f64(const double *x, const double *w, const double *bias,
                                  MELLIN_LAYER_GEOMETRY, double *y, void *workspace,
                                  size_t workspace_bytes, void *stream);

/* forward with the step the reference's models apply around every layer fused
 * in (models.py:386-390 length masks, :424-434 ReLU; no single reference
 * function): y[n, :, :, oy] = oy < lens[n] ? act(bias + corr) : 0, act = ReLU
 * when relu != 0, identity otherwise.  lens: device array of `batch` int32
 * lengths along the linear axis (NULL: no mask).  On the tensor-core path the
 * mask and the activation cost nothing and tiles past an utterance's end are
 * not computed; elsewhere they are one more pass over y. */
int mellin_mcorrlcorr_forward_masked_f32(const float *x, const float *w, const float *bias, const int *lens,
                                         int relu, MELLIN_LAYER_GEOMETRY, float *y, void *workspace,
                                         size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_forward_masked_f64(const double *x, const double *w, const double *bias, const int *lens,
                                         int relu, MELLIN_LAYER_GEOMETRY, double *y, void *workspace,
                                         size_t workspace_bytes, void *stream);

/* The same with the models' dropout fused in as well (models.py:424-434 apply conv -> nonlinearity -> dropout):
 * y = dropout(mask * act(bias + mcorrlcorr(x, w))) for a training step.  An element is dropped when a hash of
 * (dropout_seed, its offset in y) falls below dropout_p * 2^32 and is scaled by 1 / (1 - dropout_p) otherwise;
 * every kernel that can write y uses the same hash, so the mask depends on the seed only.  dropout_p = 0 is
 * mellin_mcorrlcorr_forward_masked_*; lens may be NULL.  No reference counterpart (three operators there). */
int mellin_mcorrlcorr_forward_fused_f32(const float *x, const float *w, const float *bias, const int *lens, int relu,
                                        double dropout_p, uint32_t dropout_seed, MELLIN_LAYER_GEOMETRY, float *y,
                                        void *workspace, size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_forward_fused_f64(const double *x, const double *w, const double *bias, const int *lens,
                                        int relu, double dropout_p, uint32_t dropout_seed, MELLIN_LAYER_GEOMETRY,
                                        double *y, void *workspace, size_t workspace_bytes, void *stream);

/* Backward of that epilogue in one pass over the layer's OUTPUT: grad_pre[i] = y[i] > 0 ? grad_y[i] * scale : 0
 * (with ReLU an element of y is positive exactly where it passed the activation, the mask and the dropout);
 * scale = 1 / (1 - dropout_p).  grad_pre is what the masked grad-input / grad-weight entry points take. */
int mellin_relu_dropout_backward_f32(const float *grad_y, const float *y, double scale, float *grad_pre, int64_t count,
                                     void *stream);
int mellin_relu_dropout_backward_f64(const double *grad_y, const double *y, double scale, double *grad_pre,
                                     int64_t count, void *stream);

/* grad_input for a grad_y that is zero from position lens[n] on (the gradient of
 * a masked layer): the same result as mellin_mcorrlcorr_grad_input_*, but the
 * tensor-core path does not compute the tiles that can only hold zeros. */
int mellin_mcorrlcorr_grad_input_masked_f32(const float *w, const float *grad_y, const int *lens,
                                            MELLIN_LAYER_GEOMETRY, float *grad_x, void *workspace,
                                            size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_grad_input_masked_f64(const double *w, const double *grad_y, const int *lens,
                                            MELLIN_LAYER_GEOMETRY, double *grad_x, void *workspace,
                                            size_t workspace_bytes, void *stream);

int mellin_mcorrlcorr_grad_input_f32(const float *w, const float *grad_y,
                                     MELLIN_LAYER_GEOMETRY, float *grad_x, void *workspace,
                                     size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_grad_input_f64(const double *w, const double *grad_y,
                                     MELLIN_LAYER_GEOMETRY, double *grad_x, void *workspace,
                                     size_t workspace_bytes, void *stream);

/* Scratch the grad-weight kernel needs for its per-block partial sums (they
 * are combined by a second, deterministic pass -- no floating-point atomics).
 * The answer depends on the geometry and on the current device. */
size_t mellin_mcorrlcorr_grad_weight_workspace_bytes(MELLIN_LAYER_GEOMETRY);

/* grad_b may be NULL.  workspace must hold at least
 * mellin_mcorrlcorr_grad_weight_workspace_bytes(...) bytes, 256-byte aligned;
 * it may be NULL only if that answer is 0.  Its contents are clobbered. */
/* grad_weight for a grad_y that is zero from position lens[n] on: the same
 * result as mellin_mcorrlcorr_grad_weight_*; the tensor-core kernel stops each
 * utterance's reduction at its length. */
int mellin_mcorrlcorr_grad_weight_masked_f32(const float *x, const float *grad_y, const int *lens,
                                             MELLIN_LAYER_GEOMETRY, float *grad_w, float *grad_b,
                                             void *workspace, size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_grad_weight_masked_f64(const double *x, const double *grad_y, const int *lens,
                                             MELLIN_LAYER_GEOMETRY, double *grad_w, double *grad_b,
                                             void *workspace, size_t workspace_bytes, void *stream);

int mellin_mcorrlcorr_grad_weight_f32(const float *x, const float *grad_y,
                                      MELLIN_LAYER_GEOMETRY, float *grad_w, float *grad_b,
                                      void *workspace, size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_grad_weight_f64(const double *x, const double *grad_y,
                                      MELLIN_LAYER_GEOMETRY, double *grad_w, double *grad_b,
                                      void *workspace, size_t workspace_bytes, void *stream);

/* No counterpart in the reference: grad_weight (+ grad_b) for callers that may
 * not allocate device memory -- inside a stream capture, under a framework that
 * forbids allocation in backward, in a plugin with a fixed arena.  Scratch and
 * index tables live in a fixed 8.25 MiB array inside the library image (held by
 * every GPU that loads the library); nothing is allocated, by this call or for
 * it.  Geometries whose partial sums exceed 8 MiB are rejected
 * (MELLIN_ERR_WORKSPACE).  The first call on a device resolves the array's
 * address: make it before any stream capture.  All calls share the array, so
 * calls that overlap on the GPU race; serialise them.  Results are identical to
 * mellin_mcorrlcorr_grad_weight_f32. */
int mellin_mcorrlcorr_grad_weight_noalloc_f32(const float *x, const float *grad_y, MELLIN_LAYER_GEOMETRY,
                                              float *grad_w, float *grad_b, void *stream);

/* ---- float16 ------------------------------------------------------------------ */

/* Layer-level entry points on float16 tensors (`const void *` = device pointers to IEEE half values), as the
 * reference's CUDA binding dispatches Half into its kernels (ext/torch_cuda.cu:62) with a float32 accumulator
 * (mconv_cuda.cuh:135-139): operands are widened into the workspace, the float32 kernels run on them, results are
 * rounded to float16 once.  Because every float16 value is exact in TF32, the tensor-core kernels issue one MMA per
 * product here instead of the three of their float32 hi/lo split.  The workspace (256-byte aligned) must hold
 * mellin_mcorrlcorr_*_workspace_bytes_f16(...) bytes: float32 copies of the tensors plus the operator's scratch. */
size_t mellin_mcorrlcorr_forward_workspace_bytes_f16(MELLIN_LAYER_GEOMETRY);
size_t mellin_mcorrlcorr_grad_input_workspace_bytes_f16(MELLIN_LAYER_GEOMETRY);
size_t mellin_mcorrlcorr_grad_weight_workspace_bytes_f16(MELLIN_LAYER_GEOMETRY);
int mellin_mcorrlcorr_forward_f16(const void *x, const void *w, const void *bias, MELLIN_LAYER_GEOMETRY, void *y,
                                  void *workspace, size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_grad_input_f16(const void *w, const void *grad_y, MELLIN_LAYER_GEOMETRY, void *grad_x,
                                     void *workspace, size_t workspace_bytes, void *stream);
int mellin_mcorrlcorr_grad_weight_f16(const void *x, const void *grad_y, MELLIN_LAYER_GEOMETRY, void *grad_w,
                                      void *grad_b, void *workspace, size_t workspace_bytes, void *stream);

/* ---- the elementwise layers in front of the first Mellin layer ----------------
 * Replace layers.py:8-21 (dilation_lift / DilationLift) and layers.py:100-101 (LogCompression.forward) of the
 * reference, which models.py:413-417 applies one after the other, by ONE pass over the tensor:
 *     y[o, t, i] = (t + 1)^tau * log(eps + |x[o, t, i]|)
 * on a contiguous tensor viewed as [outer][len][inner] with `len` the lifted axis.  tau and eps are DEVICE scalars
 * (the layers' parameters); either may be NULL, which leaves that step out (tau NULL: log compression alone; eps
 * NULL: the lift alone).  With log_domain != 0 they hold log(tau) / log(eps), as the reference's modules store
 * them (log_tau, log_eps), and the parameter gradients are those of the logarithms.
 *
 * Backward: grad_x as above, grad_tau / grad_eps (device scalars, either may be NULL) summed in a fixed order,
 * so that two runs give the same bits.  workspace: mellin_lift_compress_workspace_bytes() bytes, 8-byte aligned. */
size_t mellin_lift_compress_workspace_bytes(void);
int mellin_lift_compress_f32(const float *x, const float *tau, const float *eps, int log_domain, int64_t outer,
                             int64_t len, int64_t inner, float *y, void *stream);
int mellin_lift_compress_f64(const double *x, const double *tau, const double *eps, int log_domain, int64_t outer,
                             int64_t len, int64_t inner, double *y, void *stream);
int mellin_lift_compress_backward_f32(const float *x, const float *grad_y, const float *tau, const float *eps,
                                      int log_domain, int64_t outer, int64_t len, int64_t inner, float *grad_x,
                                      float *grad_tau, float *grad_eps, void *workspace, size_t workspace_bytes,
                                      void *stream);
int mellin_lift_compress_backward_f64(const double *x, const double *grad_y, const double *tau, const double *eps,
                                      int log_domain, int64_t outer, int64_t len, int64_t inner, double *grad_x,
                                      double *grad_tau, double *grad_eps, void *workspace, size_t workspace_bytes,
                                      void *stream);

/* ---- diagnostics ------------------------------------------------------------ */

/* Number of kernels this library has launched from the calling process since
 * it was loaded (all threads, all devices). */
int64_t mellin_launch_count(void);

/* Enable (1, default) or disable (0) the tcgen05 tensor-core kernels process-wide;
 * returns the previous setting.  Disabled, every operator runs on CUDA cores. */
int mellin_set_tensor_cores(int enable);

/* The first-layer operators launch their helper kernels (weight operands before, plane sum / reduction after the
 * main kernel) programmatically dependent: a kernel's set-up runs under the kernel before it in the stream.  This
 * switches that off (0) or on (non-zero) process-wide and returns the previous setting; off, every launch is an
 * ordinary one.  The environment variable MELLIN_DEPENDENT_LAUNCH=0, read on first use, does the same.  No
 * reference counterpart. */
int mellin_set_dependent_launch(int enable);

/* Every kernel that waits on a barrier (the tensor-core kernels and the
 * row-streaming first-layer kernels) bounds the wait; if one ever gives up it
 * records a non-zero code on the device instead of hanging, and the results of
 * that launch are incomplete.  This call synchronises the current device,
 * stores the first code recorded since the last query in *code (0 = healthy;
 * 1..99 tensor-core forward / grad-input, 100.. tensor-core weight gradient,
 * 200.. row-streaming weight gradient, 300.. row-streaming grad-input by
 * output row, 400.. tensor-core grad-input by source row, 500.. tensor-core
 * first-layer forward, 600.. tensor-core first-layer weight gradient) and
 * clears it. */
int mellin_device_status(int *code);

/* Self-test of the bounded waits: launches one thread that waits, with a limit
 * of 1000 polls, on a barrier nothing ever arms.  The kernel must return by
 * itself and leave mellin_device_status() reporting 202.  No reference
 * counterpart (the reference's kernels never wait). */
int mellin_selftest_unarmed_wait(void *stream);

/* Measurement aid: runs `blocks` blocks of 256 threads, each thread `iters`
 * iterations of 128 packed FP32 multiply-adds on registers, and returns the
 * number of multiply-adds performed (-1 on bad arguments); `out` receives
 * blocks * 256 floats.  Timed by the caller, it gives the FP32 CUDA-core
 * ceiling of the device.  No reference counterpart. */
int64_t mellin_selftest_fma_rate(float *out, int64_t blocks, int64_t iters, void *stream);

/* Drop every cached index table of the current device (frees device memory). */
int mellin_clear_tables(void);

/* Host-only: build the Mellin index map the kernels consume, for inspection
 * and validation (no GPU needed).  relation: 0 = correlation, 1 = convolution.
 * order: 0 = rows are hx, entries (fx, gx); 1 = rows are gx, entries (fx, hx);
 * 2 = rows are fx, entries (hx | flags, gx) where bit 29 marks the entry that
 * owns its hx row for the bias sum and bit 30 an hx row no tap reaches.
 * row_ptr receives rows + 1 ints; entries receives up to `capacity` (a, b)
 * pairs.  Returns the number of entries of the full table, or -1 on bad
 * arguments.  Either output pointer may be NULL to query sizes. */
int64_t mellin_index_map_build(int relation, int order, int64_t nf, int64_t ng, int64_t nh, int64_t s,
                               int64_t d, int64_t p, int64_t u, int32_t *row_ptr, int32_t *entries,
                               int64_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* MELLIN_B200_H_ */
