// extern "C" surface of the library: argument validation, translation of the
// reference's operator vocabulary (f, g, h, transposition flags, s/d/p/u) into
// the kernels' problem descriptions, table look-up, launch.
#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <type_traits>

#include "../../include/mellin_b200.h"
#include <cuda_fp16.h>

#include "mellin_internal.h"
#include "tuning_hooks.h"

namespace mellin {
int tc_read_prof(long long *out);
int tc_gradw_read_prof(long long *out);
const std::string &last_error();
int64_t launch_count();
}  // namespace mellin

using namespace mellin;

namespace {

constexpr int64_t kMaxExtent = (1LL << 29) - 1;

int64_t floordiv(int64_t a, int64_t b) {
  int64_t q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}
int64_t nonneg(int64_t v) { return v > 0 ? v : 0; }

struct Geometry2D {
  int64_t c_out, c_in, batch, nfx, nfy, ngx, ngy, nhx, nhy, sx, sy, dx, dy, px, py, ux, uy;
};

// Common checks.  Mellin axis: p >= 0 (P = p + 1 is a divisor).  Linear axis:
// the quantity that ends up as the exact divisor must be >= 1.
int check_geometry(const char *who, const Geometry2D &q, int64_t linear_divisor) {
  const int64_t extents[] = {q.c_out, q.c_in, q.batch, q.nfx, q.nfy, q.ngx, q.ngy, q.nhx, q.nhy};
  for (int64_t e : extents) {
    if (e < 0) return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": negative extent");
    if (e > kMaxExtent) return fail(MELLIN_ERR_UNSUPPORTED, std::string(who) + ": extent above 2^29 - 1");
  }
  const int64_t params[] = {q.sx, q.sy, q.dx, q.dy, q.px, q.py, q.ux, q.uy};
  for (int64_t e : params)
    if (e > kMaxExtent || e < -kMaxExtent)
      return fail(MELLIN_ERR_UNSUPPORTED, std::string(who) + ": parameter magnitude above 2^29 - 1");
  if (q.px < 0) return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": Mellin p must be >= 0");
  if (linear_divisor < 1)
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": linear-axis divisor must be >= 1");
  return MELLIN_OK;
}

// out = oy < lens[n] ? act(out) : 0 on a dense (N, A, nox, noy) tensor: the fused
// epilogue as a separate pass, for the paths that do not carry it themselves
template <typename T>
__global__ void mask_relu_kernel(T *__restrict__ out, const int *__restrict__ lens, int len_scale, int len_offset,
                                 int relu, unsigned drop_threshold, unsigned drop_seed, float drop_scale,
                                 long long total, long long per_utterance, int noy) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(i / per_utterance), oy = (int)(i % noy);
    T v = out[i];
    if (relu && v < T(0)) v = T(0);
    if (lens != nullptr && oy >= lens[n] * len_scale + len_offset) v = T(0);
    if (drop_threshold != 0u)
      v = dropout_hash(drop_seed, (unsigned long long)i) < drop_threshold ? T(0) : v * T(drop_scale);
    out[i] = v;
  }
}

// grad_pre[i] = y[i] > 0 ? grad[i] * scale : 0: the backward of relu + mask + dropout in one pass, read off the
// layer's own output (an element is positive exactly where it passed all three)
template <typename T>
__global__ void relu_dropout_backward_kernel(const T *__restrict__ grad, const T *__restrict__ y, T scale,
                                             T *__restrict__ out, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = y[i] > T(0) ? grad[i] * scale : T(0);
}
template <typename T>
int launch_relu_dropout_backward(const T *grad, const T *y, double scale, T *out, int64_t total, void *stream) {
  if (total <= 0) return MELLIN_OK;
  if (grad == nullptr || y == nullptr || out == nullptr) return fail(MELLIN_ERR_BAD_ARGUMENT, "relu_dropout_backward: null pointer");
  const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 32);
  relu_dropout_backward_kernel<T><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(grad, y, (T)scale, out, total);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("relu_dropout_backward_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

template <typename T>
int launch_mask_relu(const DirectProblem<T> &p, cudaStream_t stream) {
  const long long per_utterance = (long long)p.A * p.nox * p.noy, total = per_utterance * p.N;
  if (total == 0) return MELLIN_OK;
  const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
  mask_relu_kernel<T><<<blocks, 256, 0, stream>>>(p.out, p.lens, p.len_scale, p.len_offset, p.relu, p.drop_threshold,
                                                  p.drop_seed, p.drop_scale, total, per_utterance, p.noy);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("mask_relu_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

// tensor cores when enabled, covered and given scratch; CUDA cores otherwise
int dispatch_direct(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (p.lens != nullptr || p.relu || p.drop_threshold) {
    // fused length mask / ReLU / dropout: the tensor-core kernel that carries it, else the plain operator and one more pass
    if (p.B <= 4 && p.A >= 16 && !p.accumulate && tensor_cores_enabled() && workspace != nullptr) {
      const int rc = launch_tc_few_in(p, workspace, workspace_bytes, stream);
      if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
    }
    if (p.lens != nullptr && !p.accumulate && tensor_cores_enabled() && workspace != nullptr && p.A > 4) {
      const size_t need = direct_tc_workspace_bytes_masked(p);
      if (need > 0 && workspace_bytes >= need) {
        const int rc = launch_direct_tc_masked(p, workspace, workspace_bytes, stream);
        if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
      }
    }
    if (p.B <= 4 && p.A >= 8 && !p.accumulate) {
      // first layers without the tensor cores: the row kernel carries the epilogue too
      const int rc = launch_few_in_rows(p, stream);
      if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
    }
    DirectProblem<float> plain = p;
    plain.lens = nullptr, plain.relu = 0, plain.drop_threshold = 0;
    const int rc = dispatch_direct(plain, workspace, workspace_bytes, stream);
    return rc ? rc : launch_mask_relu(p, stream);
  }
  if (p.B <= 4 && p.A >= 16 && !p.accumulate && tensor_cores_enabled() && workspace != nullptr) {
    // a handful of input channels (a first layer): taps folded into the reduction, operand A in tensor memory,
    // output tiles written by TMA stores
    const int rc = launch_tc_few_in(p, workspace, workspace_bytes, stream);
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
  }
  if (p.A <= 4) {
    // a handful of output channels: by source row on the tensor cores (each row of the reduced tensor
    // fetched once, partial planes in the workspace) when covered, else the row-streaming CUDA-core kernel
    int rc = (p.accumulate || !tensor_cores_enabled()) ? MELLIN_ERR_UNSUPPORTED
                                                       : launch_tc_scatter(p, workspace, workspace_bytes, stream);
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
    rc = launch_direct_rows(p, workspace, workspace_bytes, stream);
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
  }
  if (!p.accumulate && tensor_cores_enabled() && workspace != nullptr) {
    if (p.noy == 1) {
      // wide 1-D Mellin operator: the batch becomes the linear axis
      const int rc = launch_direct_batch_inner(p, workspace, workspace_bytes, stream);
      if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
    }
    if (p.niy % 4 != 0) {
      // rows whose pitch the TMA loads cannot address: a zero-padded copy first
      const int rc = launch_direct_repitched(p, workspace, workspace_bytes, stream);
      if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
    }
    const size_t need = direct_tc_workspace_bytes(p);
    if (need > 0 && workspace_bytes >= need) {
      const int rc = launch_direct_tc(p, workspace, workspace_bytes, stream);
      if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
    }
  }
  if (p.B <= 4 && p.A >= 8) {
    // a handful of reduced channels (a first layer's forward) without the tensor cores: the row kernel
    // (152 us at the benchmark layer against 121 us for the tcgen05 kernel and 220 us for the tile kernel)
    const int rc = launch_few_in_rows(p, stream);
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
  }
  return launch_direct<float>(p, stream);
}
// out[n, a, :] += tmp[n, a, :] for a dense tmp and an `out` with arbitrary (n, a) strides
__global__ void add_into_kernel(const float *__restrict__ tmp, float *__restrict__ out, long long plane, int A,
                                long long out_sn, long long out_sa, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long na = i / plane, r = i - na * plane;
    const long long n = na / A, a = na - n * A;
    out[n * out_sn + a * out_sa + r] += tmp[i];
  }
}

int add_into(const float *tmp, float *out, long long plane, int A, long long n_count, long long out_sn, long long out_sa,
             cudaStream_t stream) {
  const long long total = n_count * A * plane;
  if (total <= 0) return MELLIN_OK;
  const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 32);
  add_into_kernel<<<blocks, 256, 0, stream>>>(tmp, out, plane, A, out_sn, out_sa, total);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("add_into_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

// Operator-level calls accumulate into their output and bring no workspace (the reference's
// signatures have none).  Where a tensor-core kernel covers the problem it is run into
// library-owned scratch and the result added to the output: two more passes over the
// output, against per-output kernels that are orders of magnitude slower at wide channels.
int dispatch_accumulating(const DirectProblem<float> &p, cudaStream_t stream) {
  if (!p.accumulate || !tensor_cores_enabled() || p.A <= 4 || p.B < 16) return MELLIN_ERR_UNSUPPORTED;
  DirectProblem<float> q = p;
  q.accumulate = false, q.bias = nullptr, q.lens = nullptr, q.relu = 0;
  const long long plane = (long long)p.nox * p.noy;
  q.out_sa = plane, q.out_sn = plane * p.A;
  const size_t ws = std::max(std::max(direct_tc_workspace_bytes(q), direct_batch_inner_workspace_bytes(q)),
                             direct_repitch_workspace_bytes(q));
  if (ws == 0) return MELLIN_ERR_UNSUPPORTED;
  const size_t out_bytes = ((size_t)p.N * p.A * plane * sizeof(float) + 255) / 256 * 256;
  unsigned char *arena = static_cast<unsigned char *>(scratch_arena(out_bytes + ws + 256, stream));
  if (arena == nullptr) return MELLIN_ERR_UNSUPPORTED;  // no memory for the scratch: the slow kernels need none
  q.out = reinterpret_cast<float *>(arena);
  int rc = dispatch_direct(q, arena + out_bytes, ws + 256, stream);
  if (rc) return rc;
  return add_into(q.out, p.out, plane, p.A, p.N, p.out_sn, p.out_sa, stream);
}
int dispatch_accumulating(const DirectProblem<double> &, cudaStream_t) { return MELLIN_ERR_UNSUPPORTED; }

int dispatch_direct(const DirectProblem<double> &p, void *, size_t, cudaStream_t stream) {
  DirectProblem<double> plain = p;
  plain.drop_threshold = 0;
  const int rc = launch_direct<double>(plain, stream);
  return (rc || (p.lens == nullptr && !p.relu && !p.drop_threshold)) ? rc : launch_mask_relu(p, stream);
}

// ---- polyphase forms of linear stride / dilation 2 -------------------------------------
// The tensor-core kernels take linear stride 1 and dilation 1.  A layer-level operator
// whose linear axis has (stride, dilation) = (1, 2), (2, 1) or (2, 2) and no padding is
// rewritten, exactly, as a stride-1 dilation-1 operator on de-interleaved tensors:
//   (1, 2)  y[2m + q] = sum_k W[k] x[2(m + k) + q]: the two phases of x are two utterances
//           whose outputs interleave into y (batch 2N, half the length);
//   (2, 2)  y[h] = sum_k W[k] x[2(h + k)]: only the even phase of x is read;
//   (2, 1)  y[h] = sum_j W[2j] x[2(h + j)] + sum_j W[2j + 1] x[2(h + j) + 1]: the phases of
//           x become extra input channels and the kernel splits into its even and odd taps.
// The copies are two passes over tensors the operator reads once; the products and the
// set of terms of every sum are those of the definition.
struct Polyphase {
  int mode = 0;  // 1: (1, 2), 2: (2, 1), 3: (2, 2)
  Geometry2D inner;
  int64_t Lp = 0, Hp = 0, Kp = 0;  // half lengths of input rows, output rows, kernel taps
};

size_t round256(size_t b) { return (b + 255) / 256 * 256; }

bool plan_polyphase(const Geometry2D &q, Polyphase &P) {
  if (!tensor_cores_enabled() || q.uy != 1 || q.py != 0) return false;
  if (q.sy == 1 && q.dy == 2) P.mode = 1;
  else if (q.sy == 2 && q.dy == 1) P.mode = 2;
  else if (q.sy == 2 && q.dy == 2) P.mode = 3;
  else return false;
  // only where the stride-1 form then runs on the tensor cores
  if (q.c_in < 16 || q.c_out < 32 || q.ngy < 64 || q.nhy < 16 || q.nfy < 2 || q.batch < 1) return false;
  P.Lp = (q.ngy + 1) / 2, P.Hp = (q.nhy + 1) / 2, P.Kp = (q.nfy + 1) / 2;
  P.inner = q;
  P.inner.sy = 1, P.inner.dy = 1, P.inner.ngy = P.Lp;
  if (P.mode == 1) P.inner.batch = 2 * q.batch, P.inner.nhy = P.Hp;
  if (P.mode == 2) P.inner.c_in = 2 * q.c_in, P.inner.nfy = P.Kp;
  return true;
}

// dst[((o * phases + t) * inner + r) * Lp + m] = src[(o * inner + r) * L + 2 m + t]  (0 past the row's end)
__global__ void deinterleave_kernel(const float *__restrict__ src, long long outer, long long inner, int L, int Lp,
                                    int phases, float *__restrict__ dst) {
  const long long total = outer * phases * inner * Lp;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i % Lp);
    long long r = i / Lp;
    const long long ri = r % inner;
    r /= inner;
    const int t = (int)(r % phases);
    const long long o = r / phases;
    const int x = 2 * m + t;
    dst[i] = x < L ? src[(o * inner + ri) * L + x] : 0.f;
  }
}
// dst[(o * inner + r) * L + x] = x odd and phases == 1 ? 0 : src[((o * phases + x % 2) * inner + r) * Lp + x / 2]
__global__ void interleave_kernel(const float *__restrict__ src, long long outer, long long inner, int L, int Lp,
                                  int phases, float *__restrict__ dst) {
  const long long total = outer * inner * L;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(i % L);
    const long long r = i / L;
    const long long ri = r % inner, o = r / inner;
    const int t = x & 1;
    dst[i] = t < phases ? src[((o * phases + t) * inner + ri) * Lp + (x >> 1)] : 0.f;
  }
}
int copy_launch(bool split, const float *src, int64_t outer, int64_t inner, int64_t L, int64_t Lp, int phases, float *dst,
                cudaStream_t stream) {
  const long long total = split ? outer * phases * inner * Lp : outer * inner * L;
  if (total <= 0) return MELLIN_OK;
  const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 32);
  if (split) deinterleave_kernel<<<blocks, 256, 0, stream>>>(src, outer, inner, (int)L, (int)Lp, phases, dst);
  else interleave_kernel<<<blocks, 256, 0, stream>>>(src, outer, inner, (int)L, (int)Lp, phases, dst);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("polyphase copy: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

size_t direct_workspace_query(const Geometry2D &q, bool input_gradient);
size_t gradw_workspace_query(const Geometry2D &q);
int add_into(const float *tmp, float *out, long long plane, int A, long long n_count, long long out_sn, long long out_sa,
             cudaStream_t stream);

// scratch of the polyphase forms: copies first, then the inner operator's own scratch
struct PolyBuffers {
  size_t in_copy = 0, out_copy = 0, w_copy = 0, inner = 0;
  size_t total() const { return in_copy + out_copy + w_copy + inner; }
};
PolyBuffers polyphase_buffers(const Geometry2D &q, const Polyphase &P, int op /*0 fwd, 1 grad-input, 2 grad-weight*/) {
  PolyBuffers b;
  const Geometry2D &i = P.inner;
  const size_t x_inner = round256((size_t)i.batch * i.c_in * i.ngx * i.ngy * sizeof(float));
  const size_t y_inner = round256((size_t)i.batch * i.c_out * i.nhx * i.nhy * sizeof(float));
  const size_t w_inner = round256((size_t)i.c_out * i.c_in * i.nfx * i.nfy * sizeof(float));
  if (op == 0) {
    b.in_copy = x_inner;
    b.out_copy = P.mode == 1 ? y_inner : 0;
    b.w_copy = P.mode == 2 ? w_inner : 0;
    b.inner = direct_workspace_query(i, false);
  } else if (op == 1) {
    b.in_copy = P.mode == 1 ? y_inner : 0;  // de-interleaved grad_y
    b.out_copy = x_inner;                   // grad_x of the inner problem
    b.w_copy = P.mode == 2 ? w_inner : 0;
    b.inner = direct_workspace_query(i, true);
  } else {
    b.in_copy = x_inner + (P.mode == 1 ? y_inner : 0);
    b.out_copy = P.mode == 2 ? w_inner : 0;  // grad_w of the inner problem
    b.inner = gradw_workspace_query(i);
  }
  b.inner = round256(b.inner);
  return b;
}

template <typename T>
int op2d(const char *who, Relation rel, const T *f, const T *g, const Geometry2D &q, int tf, int tg, int th,
         T *h, const T *bias, bool accumulate, void *workspace, size_t workspace_bytes, void *stream,
         const int *lens = nullptr, int relu = 0, double dropout_p = 0.0, unsigned dropout_seed = 0, int exact = 0) {
  if (!(dropout_p >= 0.0 && dropout_p < 1.0))
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": dropout probability must be in [0, 1)");
  int rc = check_geometry(who, q, q.uy);
  if (rc) return rc;
  const int64_t out_elems = q.batch * q.c_out * q.nhx * q.nhy;
  if (out_elems == 0) return MELLIN_OK;
  if (h == nullptr) return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null output");
  const bool has_terms = q.c_in > 0 && q.nfx > 0 && q.nfy > 0 && q.ngx > 0 && q.ngy > 0;
  if (has_terms && (f == nullptr || g == nullptr))
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null operand");
  if constexpr (std::is_same<T, float>::value) {
    Polyphase P;
    if (rel == Relation::Corr && accumulate && workspace == nullptr && !tf && !tg && has_terms && plan_polyphase(q, P)) {
      // operator-level call of a strided / dilated linear operator: the polyphase form into library scratch, then h += it
      const size_t out_bytes = round256((size_t)out_elems * sizeof(float));
      const size_t ws = polyphase_buffers(q, P, 0).total();
      unsigned char *arena = static_cast<unsigned char *>(scratch_arena(out_bytes + ws + 256, static_cast<cudaStream_t>(stream)));
      if (arena != nullptr) {
        float *tmp = reinterpret_cast<float *>(arena);
        rc = op2d<float>(who, rel, f, g, q, 0, 0, 0, tmp, nullptr, false, arena + out_bytes, ws + 256, stream);
        if (rc) return rc;
        const int64_t hp = q.nhx * q.nhy;
        return add_into(tmp, h, hp, (int)q.c_out, q.batch, th ? hp : q.c_out * hp, th ? q.batch * hp : hp,
                        static_cast<cudaStream_t>(stream));
      }
    }
    if (rel == Relation::Corr && !accumulate && !tf && !tg && !th && has_terms && lens == nullptr && !relu &&
        workspace != nullptr && reinterpret_cast<uintptr_t>(workspace) % 256 == 0 && plan_polyphase(q, P)) {
      const PolyBuffers b = polyphase_buffers(q, P, 0);
      if (workspace_bytes >= b.total()) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        unsigned char *base = static_cast<unsigned char *>(workspace);
        float *xc = reinterpret_cast<float *>(base), *yc = reinterpret_cast<float *>(base + b.in_copy);
        float *wc = reinterpret_cast<float *>(base + b.in_copy + b.out_copy);
        void *inner_ws = base + b.in_copy + b.out_copy + b.w_copy;
        const int64_t rows_x = q.c_in * q.ngx;
        if (P.mode == 1) rc = copy_launch(true, g, 1, q.batch * rows_x, q.ngy, P.Lp, 2, xc, st);
        else if (P.mode == 2) rc = copy_launch(true, g, q.batch, rows_x, q.ngy, P.Lp, 2, xc, st);
        else rc = copy_launch(true, g, 1, q.batch * rows_x, q.ngy, P.Lp, 1, xc, st);
        if (rc) return rc;
        const float *w_in = f;
        if (P.mode == 2) {
          rc = copy_launch(true, f, q.c_out, q.c_in * q.nfx, q.nfy, P.Kp, 2, wc, st);
          if (rc) return rc;
          w_in = wc;
        }
        float *y_out = P.mode == 1 ? yc : h;
        rc = op2d<float>(who, rel, w_in, xc, P.inner, 0, 0, 0, y_out, bias, false, inner_ws, b.inner, stream);
        if (rc || P.mode != 1) return rc;
        return copy_launch(false, yc, 1, q.batch * q.c_out * q.nhx, q.nhy, P.Hp, 2, h, st);
      }
    }
  }
  DirectProblem<T> p;
  rc = get_device_table(IndexMapKey{rel, SortBy::H, has_terms ? q.nfx : 0, q.ngx, q.nhx, q.sx, q.dx, q.px, q.ux},
                        &p.table);
  if (rc) return rc;
  const int64_t gplane = q.ngx * q.ngy, fplane = q.nfx * q.nfy, hplane = q.nhx * q.nhy;
  p.in = g, p.w = f, p.bias = bias, p.out = h;
  p.N = (int)q.batch, p.A = (int)q.c_out, p.B = has_terms ? (int)q.c_in : 0;
  p.nkx = (int)q.nfx, p.nky = (int)q.nfy, p.nix = (int)q.ngx, p.niy = (int)q.ngy;
  p.nox = (int)q.nhx, p.noy = (int)q.nhy;
  p.in_sn = tg ? gplane : q.c_in * gplane;
  p.in_sb = tg ? q.batch * gplane : gplane;
  p.w_sa = tf ? fplane : q.c_in * fplane;
  p.w_sb = tf ? q.c_out * fplane : fplane;
  p.out_sn = th ? hplane : q.c_out * hplane;
  p.out_sa = th ? q.batch * hplane : hplane;
  p.Ay = (int)q.sy;
  p.By = rel == Relation::Corr ? (int)q.dy : -(int)q.dy;
  p.Cy = rel == Relation::Corr ? -(int)q.py : (int)q.py;
  p.Dy = (int)q.uy;
  p.accumulate = accumulate;
  p.lens = lens, p.relu = relu;
  p.exact_tf32 = exact;
  if (dropout_p > 0.0) {
    p.drop_threshold = (unsigned)std::min<double>(dropout_p * 4294967296.0, 4294967295.0);
    p.drop_seed = dropout_seed;
    p.drop_scale = (float)(1.0 / (1.0 - dropout_p));
  }
  if constexpr (std::is_same<T, float>::value) {
    if (has_terms && p.A <= 4 && !accumulate && workspace != nullptr) {
      rc = get_device_table(IndexMapKey{rel, SortBy::G, q.nfx, q.ngx, q.nhx, q.sx, q.dx, q.px, q.ux}, &p.table_by_in);
      if (rc) return rc;
    }
  }
  if (accumulate && workspace == nullptr) {
    rc = dispatch_accumulating(p, static_cast<cudaStream_t>(stream));
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
  }
  return dispatch_direct(p, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

template <typename T>
int grad_input(const char *who, const T *w, const T *go, const Geometry2D &q, T *gx, void *workspace,
               size_t workspace_bytes, void *stream, const int *lens = nullptr, int exact = 0) {
  int rc = check_geometry(who, q, q.sy);
  if (rc) return rc;
  if (q.batch * q.c_in * q.ngx * q.ngy == 0) return MELLIN_OK;
  if (gx == nullptr) return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null output");
  const bool has_terms = q.c_out > 0 && q.nfx > 0 && q.nfy > 0 && q.nhx > 0 && q.nhy > 0;
  if (has_terms && (w == nullptr || go == nullptr))
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null operand");
  if constexpr (std::is_same<T, float>::value) {
    Polyphase P;
    if (has_terms && lens == nullptr && workspace != nullptr && reinterpret_cast<uintptr_t>(workspace) % 256 == 0 &&
        plan_polyphase(q, P)) {
      const PolyBuffers b = polyphase_buffers(q, P, 1);
      if (workspace_bytes >= b.total()) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        unsigned char *base = static_cast<unsigned char *>(workspace);
        float *goc = reinterpret_cast<float *>(base), *gxc = reinterpret_cast<float *>(base + b.in_copy);
        float *wc = reinterpret_cast<float *>(base + b.in_copy + b.out_copy);
        void *inner_ws = base + b.in_copy + b.out_copy + b.w_copy;
        const float *go_in = go, *w_in = w;
        if (P.mode == 1) {
          rc = copy_launch(true, go, 1, q.batch * q.c_out * q.nhx, q.nhy, P.Hp, 2, goc, st);
          if (rc) return rc;
          go_in = goc;
        }
        if (P.mode == 2) {
          rc = copy_launch(true, w, q.c_out, q.c_in * q.nfx, q.nfy, P.Kp, 2, wc, st);
          if (rc) return rc;
          w_in = wc;
        }
        rc = grad_input<float>(who, w_in, go_in, P.inner, gxc, inner_ws, b.inner, stream);
        if (rc) return rc;
        const int64_t rows_x = q.c_in * q.ngx;
        if (P.mode == 2) return copy_launch(false, gxc, q.batch, rows_x, q.ngy, P.Lp, 2, gx, st);
        return copy_launch(false, gxc, 1, q.batch * rows_x, q.ngy, P.Lp, P.mode == 1 ? 2 : 1, gx, st);
      }
    }
  }
  DirectProblem<T> p;
  rc = get_device_table(
      IndexMapKey{Relation::Corr, SortBy::G, has_terms ? q.nfx : 0, q.ngx, q.nhx, q.sx, q.dx, q.px, q.ux}, &p.table);
  if (rc) return rc;
  const int64_t gplane = q.ngx * q.ngy, fplane = q.nfx * q.nfy, hplane = q.nhx * q.nhy;
  p.in = go, p.w = w, p.bias = nullptr, p.out = gx;
  p.N = (int)q.batch, p.A = (int)q.c_in, p.B = has_terms ? (int)q.c_out : 0;
  p.nkx = (int)q.nfx, p.nky = (int)q.nfy, p.nix = (int)q.nhx, p.niy = (int)q.nhy;
  p.nox = (int)q.ngx, p.noy = (int)q.ngy;
  p.in_sn = q.c_out * hplane, p.in_sb = hplane;
  p.w_sa = fplane, p.w_sb = q.c_in * fplane;  // W[a = ci, b = co] = w[co, ci]
  p.out_sn = q.c_in * gplane, p.out_sa = gplane;
  // s hy + d fy - p = u gy   =>   hy = (u gy - d fy + p) / s
  p.Ay = (int)q.uy, p.By = -(int)q.dy, p.Cy = (int)q.py, p.Dy = (int)q.sy;
  p.accumulate = false;
  p.exact_tf32 = exact;
  if constexpr (std::is_same<T, float>::value) {
    if (has_terms && p.A <= 4 && workspace != nullptr) {
      rc = get_device_table(IndexMapKey{Relation::Corr, SortBy::H, q.nfx, q.ngx, q.nhx, q.sx, q.dx, q.px, q.ux},
                            &p.table_by_in);
      if (rc) return rc;
    }
  }
  if (lens != nullptr && q.uy == 1 && p.A > 4) {
    // grad_y is zero from position lens[n] on, so grad_x is zero from this position on: the last
    // input position any output below lens[n] reads is s (len - 1) - p + d (nfy - 1)
    p.lens = lens, p.len_scale = (int)q.sy;
    p.len_offset = (int)(-q.sy - q.py + q.dy * (q.nfy > 0 ? q.nfy - 1 : 0) + 1);
  }
  return dispatch_direct(p, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

template <typename T>
int make_gradw_problem(const char *who, const Geometry2D &q, GradWProblem<T> *p, bool need_table) {
  int rc = check_geometry(who, q, q.uy);
  if (rc) return rc;
  p->N = (int)q.batch, p->A = (int)q.c_out, p->B = (int)q.c_in;
  p->nkx = (int)q.nfx, p->nky = (int)q.nfy, p->nix = (int)q.ngx, p->niy = (int)q.ngy;
  p->nox = (int)q.nhx, p->noy = (int)q.nhy;
  p->Ay = (int)q.sy, p->By = (int)q.dy, p->Cy = -(int)q.py, p->Dy = (int)q.uy;
  if (need_table) {
    rc = get_device_table(IndexMapKey{Relation::Corr, SortBy::F, q.nfx, q.ngx, q.nhx, q.sx, q.dx, q.px, q.ux},
                          &p->table);
    if (rc) return rc;
    rc = get_device_table(IndexMapKey{Relation::Corr, SortBy::H, q.nfx, q.ngx, q.nhx, q.sx, q.dx, q.px, q.ux},
                          &p->table_h);
  }
  return rc;
}

template <typename T>
int grad_weight(const char *who, const T *x, const T *go, const Geometry2D &q, T *gw, T *gb, void *workspace,
                size_t workspace_bytes, void *stream, const int *lens = nullptr, int exact = 0) {
  GradWProblem<T> p;
  int rc = make_gradw_problem(who, q, &p, true);
  if (rc) return rc;
  const int64_t gw_elems = q.c_out * q.c_in * q.nfx * q.nfy;
  if (gw_elems > 0 && gw == nullptr) return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null grad_w");
  const bool has_terms = q.batch > 0 && q.nhx > 0 && q.nhy > 0;
  if (has_terms && gw_elems > 0 && (x == nullptr || go == nullptr))
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null operand");
  if (gb != nullptr && has_terms && go == nullptr)
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null grad_y");
  if constexpr (std::is_same<T, float>::value) {
    Polyphase P;
    if (has_terms && gw_elems > 0 && lens == nullptr && workspace != nullptr &&
        reinterpret_cast<uintptr_t>(workspace) % 256 == 0 && plan_polyphase(q, P)) {
      const PolyBuffers b = polyphase_buffers(q, P, 2);
      if (workspace_bytes >= b.total()) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        unsigned char *base = static_cast<unsigned char *>(workspace);
        const Geometry2D &i = P.inner;
        const size_t x_inner = round256((size_t)i.batch * i.c_in * i.ngx * i.ngy * sizeof(float));
        float *xc = reinterpret_cast<float *>(base), *goc = reinterpret_cast<float *>(base + x_inner);
        float *gwc = reinterpret_cast<float *>(base + b.in_copy);
        void *inner_ws = base + b.in_copy + b.out_copy;
        const int64_t rows_x = q.c_in * q.ngx;
        if (P.mode == 2) rc = copy_launch(true, x, q.batch, rows_x, q.ngy, P.Lp, 2, xc, st);
        else rc = copy_launch(true, x, 1, q.batch * rows_x, q.ngy, P.Lp, P.mode == 1 ? 2 : 1, xc, st);
        if (rc) return rc;
        const float *go_in = go;
        if (P.mode == 1) {
          rc = copy_launch(true, go, 1, q.batch * q.c_out * q.nhx, q.nhy, P.Hp, 2, goc, st);
          if (rc) return rc;
          go_in = goc;
        }
        rc = grad_weight<float>(who, xc, go_in, P.inner, P.mode == 2 ? gwc : gw, gb, inner_ws, b.inner, stream);
        if (rc || P.mode != 2) return rc;
        return copy_launch(false, gwc, q.c_out, q.c_in * q.nfx, q.nfy, P.Kp, 2, gw, st);
      }
    }
  }
  p.in = x, p.go = go, p.gw = gw, p.gb = gb;
  p.exact_tf32 = exact;
  p.lens = q.nhy > 1 ? lens : nullptr;
  if (gw_elems == 0 && (gb == nullptr || q.c_out == 0)) return MELLIN_OK;
  return launch_gradw<T>(p, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

template <typename T>
int col_op(const char *who, bool gather, const T *src, T *dst, int64_t c_in, int64_t batch, int64_t nfx,
           int64_t nfy, int64_t ngx, int64_t ngy, int64_t nggx, int64_t nggy, int64_t sx, int64_t sy, int64_t dx,
           int64_t dy, int64_t px, int64_t py, int64_t ux, int64_t uy, int tg, int tgg, void *stream) {
  Geometry2D q{0, c_in, batch, nfx, nfy, ngx, ngy, nggx, nggy, sx, sy, dx, dy, px, py, ux, uy};
  // gather divides by u on the linear axis, the adjoint by s
  int rc = check_geometry(who, q, gather ? uy : sy);
  if (rc) return rc;
  const int64_t out_elems = gather ? batch * c_in * nfx * nfy * nggx * nggy : batch * c_in * ngx * ngy;
  if (out_elems == 0) return MELLIN_OK;
  const int64_t in_elems = gather ? batch * c_in * ngx * ngy : batch * c_in * nfx * nfy * nggx * nggy;
  if (dst == nullptr || (in_elems > 0 && src == nullptr))
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null pointer");
  ColProblem<T> p;
  p.src = src, p.dst = dst, p.N = (int)batch, p.C = (int)c_in;
  p.nfx = (int)nfx, p.nfy = (int)nfy, p.ngx = (int)ngx, p.ngy = (int)ngy, p.nggx = (int)nggx, p.nggy = (int)nggy;
  p.sx = (int)sx, p.sy = (int)sy, p.dx = (int)dx, p.dy = (int)dy, p.px = (int)px, p.py = (int)py;
  p.ux = (int)ux, p.uy = (int)uy;
  p.transposed_g = tg != 0, p.transposed_gg = tgg != 0;
  return gather ? launch_spec2col<T>(p, static_cast<cudaStream_t>(stream))
                : launch_col2spec<T>(p, static_cast<cudaStream_t>(stream));
}

// ---- float16 entry points -------------------------------------------------------------
// The reference's kernels take Half tensors and accumulate them in float32 (mconv_cuda.cuh:135-139).
// Here float16 operands are widened into scratch, the float32 kernels run on them, and the result
// is rounded back.  Every float16 value is exact in TF32, so the tensor-core kernels skip the two
// compensation products of their hi/lo split: one MMA per product instead of three.
__global__ void widen_kernel(const __half *__restrict__ src, float *__restrict__ dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __half2float(src[i]);
}
__global__ void narrow_kernel(const float *__restrict__ src, __half *__restrict__ dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2half_rn(src[i]);
}
int convert_launch(bool widen, const void *src, void *dst, long long n, cudaStream_t stream) {
  if (n <= 0 || src == nullptr) return MELLIN_OK;
  const int blocks = (int)std::min<long long>((n + 255) / 256, (long long)sm_count() * 32);
  if (widen) widen_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __half *>(src), static_cast<float *>(dst), n);
  else narrow_kernel<<<blocks, 256, 0, stream>>>(static_cast<const float *>(src), static_cast<__half *>(dst), n);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("float16 conversion: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

struct HalfBuffers {
  size_t x = 0, w = 0, b = 0, y = 0, inner = 0;  // float32 copies of the four tensors, then the operator's own scratch
  size_t total() const { return x + w + b + y + inner; }
};
HalfBuffers half_buffers(const Geometry2D &q, int op /*0 fwd, 1 grad-input, 2 grad-weight*/) {
  HalfBuffers h;
  h.x = round256((size_t)q.batch * q.c_in * q.ngx * q.ngy * sizeof(float));
  h.w = round256((size_t)q.c_out * q.c_in * q.nfx * q.nfy * sizeof(float));
  h.b = round256((size_t)q.c_out * sizeof(float));
  h.y = round256((size_t)q.batch * q.c_out * q.nhx * q.nhy * sizeof(float));
  h.inner = round256(op == 2 ? gradw_workspace_query(q) : direct_workspace_query(q, op == 1));
  return h;
}
int half_check(const char *who, const Geometry2D &q, const HalfBuffers &h, void *workspace, size_t workspace_bytes) {
  const int rc = check_geometry(who, q, q.uy);
  if (rc) return rc;
  if (workspace == nullptr || workspace_bytes < h.total() || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(MELLIN_ERR_WORKSPACE, std::string(who) + ": needs " + std::to_string(h.total()) +
                                          " bytes of 256-byte aligned workspace, got " + std::to_string(workspace_bytes));
  return MELLIN_OK;
}

}  // namespace

extern "C" {

int mellin_abi_version(void) { return 100; }
const char *mellin_last_error(void) { return last_error().c_str(); }
int64_t mellin_launch_count(void) { return launch_count(); }
int mellin_clear_tables(void) { return clear_device_tables(); }

int64_t mellin_mconv_valid_size(int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u) {
  return nonneg(floordiv(d * (ng + u - 1), p + 1) - s + 1);
}
int64_t mellin_mconv_support_size(int64_t nf, int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u) {
  return nonneg(floordiv((nf + d - 1) * (ng + u - 1), p + 1) - s + 1);
}
int64_t mellin_mcorr_valid_size(int64_t nf, int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u) {
  return nonneg(floordiv((ng + u - 1) * (p + 1), nf + d - 1) - s + 1);
}
int64_t mellin_mcorr_support_size(int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u) {
  return nonneg(floordiv((ng + u - 1) * (p + 1), d) - s + 1);
}
int64_t mellin_lconv_valid_size(int64_t ng, int64_t s, int64_t p, int64_t u) {
  return nonneg(floordiv(u * (ng - 1) - p, s) + 1);
}
int64_t mellin_lconv_support_size(int64_t nf, int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u) {
  return nonneg(floordiv(u * (ng - 1) + d * (nf - 1) - p, s) + 1);
}
int64_t mellin_lcorr_valid_size(int64_t nf, int64_t ng, int64_t s, int64_t d, int64_t p, int64_t u) {
  return nonneg(floordiv(u * (ng - 1) - d * (nf - 1) + p, s) + 1);
}
int64_t mellin_lcorr_support_size(int64_t ng, int64_t s, int64_t p, int64_t u) {
  return nonneg(floordiv(u * (ng - 1) + p, s) + 1);
}

#define GEOM_FROM_OP2D \
  Geometry2D { c_out, c_in, batch, nfx, nfy, ngx, ngy, nhx, nhy, sx, sy, dx, dy, px, py, ux, uy }
#define GEOM_FROM_OP1D \
  Geometry2D { c_out, c_in, batch, nf, 1, ng, 1, nh, 1, s, 1, d, 1, p, 0, u, 1 }
#define GEOM_FROM_LAYER \
  Geometry2D { c_out, c_in, batch, nfx, nfy, ngx, ngy, nhx, nhy, sx, sy, dx, dy, px, py, ux, uy }

#define DEFINE_OPS(T, sfx)                                                                            \
  MELLIN_DECL_OP1D(mellin_mconv1d_##sfx, T) {                                                         \
    return op2d<T>("mconv1d", Relation::Conv, f, g, GEOM_FROM_OP1D, transposed_f, transposed_g,       \
                   transposed_h, h, nullptr, true, nullptr, 0, stream);                                           \
  }                                                                                                   \
  MELLIN_DECL_OP1D(mellin_mcorr1d_##sfx, T) {                                                         \
    return op2d<T>("mcorr1d", Relation::Corr, f, g, GEOM_FROM_OP1D, transposed_f, transposed_g,       \
                   transposed_h, h, nullptr, true, nullptr, 0, stream);                                           \
  }                                                                                                   \
  MELLIN_DECL_OP2D(mellin_mconvlconv_##sfx, T) {                                                      \
    return op2d<T>("mconvlconv", Relation::Conv, f, g, GEOM_FROM_OP2D, transposed_f, transposed_g,    \
                   transposed_h, h, nullptr, true, nullptr, 0, stream);                                           \
  }                                                                                                   \
  MELLIN_DECL_OP2D(mellin_mcorrlcorr_##sfx, T) {                                                      \
    return op2d<T>("mcorrlcorr", Relation::Corr, f, g, GEOM_FROM_OP2D, transposed_f, transposed_g,    \
                   transposed_h, h, nullptr, true, nullptr, 0, stream);                                           \
  }                                                                                                   \
  MELLIN_DECL_COL1D(mellin_snd2col_##sfx, T, g, gg) {                                                 \
    return col_op<T>("snd2col", true, g, gg, c_in, batch, nf, 1, ng, 1, ngg, 1, s, 1, d, 1, p, 0, u,  \
                     1, transposed_g, transposed_gg, stream);                                         \
  }                                                                                                   \
  MELLIN_DECL_COL1D(mellin_col2snd_##sfx, T, gg, g) {                                                 \
    return col_op<T>("col2snd", false, gg, g, c_in, batch, nf, 1, ng, 1, ngg, 1, s, 1, d, 1, p, 0, u, \
                     1, transposed_g, transposed_gg, stream);                                         \
  }                                                                                                   \
  MELLIN_DECL_COL2D(mellin_spec2col_##sfx, T, g, gg) {                                                \
    return col_op<T>("spec2col", true, g, gg, c_in, batch, nfx, nfy, ngx, ngy, nggx, nggy, sx, sy,    \
                     dx, dy, px, py, ux, uy, transposed_g, transposed_gg, stream);                    \
  }                                                                                                   \
  MELLIN_DECL_COL2D(mellin_col2spec_##sfx, T, gg, g) {                                                \
    return col_op<T>("col2spec", false, gg, g, c_in, batch, nfx, nfy, ngx, ngy, nggx, nggy, sx, sy,   \
                     dx, dy, px, py, ux, uy, transposed_g, transposed_gg, stream);                    \
  }                                                                                                   \
  int mellin_mcorrlcorr_forward_##sfx(const T *x, const T *w, const T *bias, MELLIN_LAYER_GEOMETRY,   \
                                      T *y, void *workspace, size_t workspace_bytes, void *stream) {  \
    return op2d<T>("mcorrlcorr_forward", Relation::Corr, w, x, GEOM_FROM_LAYER, 0, 0, 0, y, bias,     \
                   false, workspace, workspace_bytes, stream);                                        \
  }                                                                                                   \
  int mellin_mcorrlcorr_forward_masked_##sfx(const T *x, const T *w, const T *bias, const int *lens,   \
                                             int relu, MELLIN_LAYER_GEOMETRY, T *y, void *workspace,  \
                                             size_t workspace_bytes, void *stream) {                  \
    return op2d<T>("mcorrlcorr_forward_masked", Relation::Corr, w, x, GEOM_FROM_LAYER, 0, 0, 0, y,    \
                   bias, false, workspace, workspace_bytes, stream, lens, relu ? 1 : 0);              \
  }                                                                                                   \
  int mellin_mcorrlcorr_forward_fused_##sfx(const T *x, const T *w, const T *bias, const int *lens,    \
                                            int relu, double dropout_p, uint32_t dropout_seed,        \
                                            MELLIN_LAYER_GEOMETRY, T *y, void *workspace,             \
                                            size_t workspace_bytes, void *stream) {                   \
    return op2d<T>("mcorrlcorr_forward_fused", Relation::Corr, w, x, GEOM_FROM_LAYER, 0, 0, 0, y,     \
                   bias, false, workspace, workspace_bytes, stream, lens, relu ? 1 : 0, dropout_p,    \
                   dropout_seed);                                                                     \
  }                                                                                                   \
  int mellin_relu_dropout_backward_##sfx(const T *grad_y, const T *y, double scale, T *grad_pre,      \
                                         int64_t count, void *stream) {                               \
    return launch_relu_dropout_backward<T>(grad_y, y, scale, grad_pre, count, stream);                \
  }                                                                                                   \
  int mellin_mcorrlcorr_grad_input_##sfx(const T *w, const T *grad_y, MELLIN_LAYER_GEOMETRY,          \
                                         T *grad_x, void *workspace, size_t workspace_bytes,          \
                                         void *stream) {                                              \
    return grad_input<T>("mcorrlcorr_grad_input", w, grad_y, GEOM_FROM_LAYER, grad_x, workspace,      \
                         workspace_bytes, stream);                                                    \
  }                                                                                                   \
  int mellin_mcorrlcorr_grad_input_masked_##sfx(const T *w, const T *grad_y, const int *lens,        \
                                                MELLIN_LAYER_GEOMETRY, T *grad_x, void *workspace,    \
                                                size_t workspace_bytes, void *stream) {               \
    return grad_input<T>("mcorrlcorr_grad_input_masked", w, grad_y, GEOM_FROM_LAYER, grad_x,          \
                         workspace, workspace_bytes, stream, lens);                                   \
  }                                                                                                   \
  int mellin_mcorrlcorr_grad_weight_##sfx(const T *x, const T *grad_y, MELLIN_LAYER_GEOMETRY,         \
                                          T *grad_w, T *grad_b, void *workspace,                      \
                                          size_t workspace_bytes, void *stream) {                     \
    return grad_weight<T>("mcorrlcorr_grad_weight", x, grad_y, GEOM_FROM_LAYER, grad_w, grad_b,       \
                          workspace, workspace_bytes, stream);                                        \
  }                                                                                                   \
  int mellin_mcorrlcorr_grad_weight_masked_##sfx(const T *x, const T *grad_y, const int *lens,        \
                                                 MELLIN_LAYER_GEOMETRY, T *grad_w, T *grad_b,         \
                                                 void *workspace, size_t workspace_bytes,             \
                                                 void *stream) {                                      \
    return grad_weight<T>("mcorrlcorr_grad_weight_masked", x, grad_y, GEOM_FROM_LAYER, grad_w,        \
                          grad_b, workspace, workspace_bytes, stream, lens);                          \
  }

DEFINE_OPS(float, f32)
DEFINE_OPS(double, f64)

#ifdef MELLIN_TUNING_HOOKS
int mellin_tc_profile(long long *out) { return mellin::tc_read_prof(out); }
int mellin_tc_gradw_profile(long long *out) { return mellin::tc_gradw_read_prof(out); }
#endif
int mellin_set_tensor_cores(int enable) { return set_tensor_cores(enable); }
int mellin_set_dependent_launch(int enable) { return set_dependent_launch(enable); }
int mellin_device_status(int *code) {
  if (code == nullptr) return fail(MELLIN_ERR_BAD_ARGUMENT, "device_status: null pointer");
  int rc = tc_take_error(code);
  if (rc) return rc;
  int gw_code = 0;
  rc = tc_gradw_take_error(&gw_code);
  if (rc) return rc;
  if (*code == 0 && gw_code != 0) *code = 100 + gw_code;
  int rows_code = 0;
  rc = gradw_rows_take_error(&rows_code);
  if (rc) return rc;
  if (*code == 0 && rows_code != 0) *code = 200 + rows_code;
  rows_code = 0;
  rc = direct_rows_take_error(&rows_code);
  if (rc == MELLIN_OK && *code == 0 && rows_code != 0) *code = 300 + rows_code;
  if (rc) return rc;
  rc = tc_scatter_take_error(&rows_code);
  if (rc == MELLIN_OK && *code == 0 && rows_code != 0) *code = 400 + rows_code;
  if (rc) return rc;
  rc = tc_few_in_take_error(&rows_code);
  if (rc == MELLIN_OK && *code == 0 && rows_code != 0) *code = 500 + rows_code;
  if (rc) return rc;
  rc = tc_gradw_few_in_take_error(&rows_code);
  if (rc == MELLIN_OK && *code == 0 && rows_code != 0) *code = 600 + rows_code;
  return rc;
}
int mellin_selftest_unarmed_wait(void *stream) { return launch_unarmed_wait(static_cast<cudaStream_t>(stream)); }

// Workspace queries plan with the extents only (tables are not needed: the
// longest table row is bounded by the kernel extent along the Mellin axis).
}  // extern "C"
namespace {
size_t direct_workspace_query(const Geometry2D &q, bool input_gradient) {
  if (check_geometry("workspace_bytes", q, input_gradient ? q.sy : q.uy)) return 0;
  {
    Polyphase P;
    if (plan_polyphase(q, P)) return polyphase_buffers(q, P, input_gradient ? 1 : 0).total();
  }
  DirectProblem<float> p;
  p.N = (int)q.batch;
  p.A = input_gradient ? (int)q.c_in : (int)q.c_out;
  p.B = input_gradient ? (int)q.c_out : (int)q.c_in;
  p.nkx = (int)q.nfx, p.nky = (int)q.nfy;
  p.nix = input_gradient ? (int)q.nhx : (int)q.ngx, p.niy = input_gradient ? (int)q.nhy : (int)q.ngy;
  p.nox = input_gradient ? (int)q.ngx : (int)q.nhx, p.noy = input_gradient ? (int)q.ngy : (int)q.nhy;
  p.Ay = input_gradient ? (int)q.uy : (int)q.sy;
  p.By = input_gradient ? -(int)q.dy : (int)q.dy;
  p.Cy = input_gradient ? (int)q.py : -(int)q.py;
  p.Dy = input_gradient ? (int)q.sy : (int)q.uy;
  p.table.max_row = (int)q.nfx;  // upper bound: one entry per kernel tap
  size_t rows = p.A <= 4 ? direct_rows_workspace_bytes(p) : 0;
  if ((p.A <= 4 || p.B <= 4) && q.nfx <= 16 && q.nfx > 0) {
    // the first-layer tensor-core kernels size their scratch by the number of table entries: count them
    const int64_t triples = (int64_t)enumerate_triples(Relation::Corr, q.nfx, q.ngx, q.nhx, q.sx, q.dx, q.px, q.ux).size();
    if (p.A <= 4) {
      p.table_by_in.num_entries = triples;
      p.table_by_in.max_row = (int)q.nfx;
      rows = std::max(rows, tc_scatter_workspace_bytes(p));
    }
    if (p.B <= 4) {
      p.table.num_entries = triples;
      DirectProblem<float> dense = p;  // the query describes dense, aligned tensors
      dense.in_sb = (long long)p.nix * p.niy, dense.in_sn = (long long)p.B * p.nix * p.niy;
      dense.out_sa = (long long)p.nox * p.noy, dense.out_sn = (long long)p.A * p.nox * p.noy;
      rows = std::max(rows, tc_few_in_workspace_bytes(dense));
    }
  }
  // the query describes dense tensors
  p.in_sb = (long long)p.nix * p.niy, p.in_sn = (long long)p.B * p.nix * p.niy;
  return std::max(std::max(rows, direct_tc_workspace_bytes(p)),
                  std::max(direct_batch_inner_workspace_bytes(p), direct_repitch_workspace_bytes(p)));
}
size_t gradw_workspace_query(const Geometry2D &q) {
  {
    Polyphase P;
    if (check_geometry("grad_weight_workspace_bytes", q, q.uy) == MELLIN_OK && plan_polyphase(q, P))
      return polyphase_buffers(q, P, 2).total();
  }
  GradWProblem<float> p;
  if (make_gradw_problem<float>("grad_weight_workspace_bytes", q, &p, false)) return 0;
  // planning only looks at extents, parameters and pointer alignment; probe
  // with an aligned dummy so that the answer is an upper bound for any buffer
  p.go = reinterpret_cast<const float *>(uintptr_t(256));
  return gradw_workspace_bytes<float>(p);
}
}  // namespace
extern "C" {
size_t mellin_mcorrlcorr_forward_workspace_bytes(MELLIN_LAYER_GEOMETRY) {
  return direct_workspace_query(GEOM_FROM_LAYER, false);
}
size_t mellin_mcorrlcorr_grad_input_workspace_bytes(MELLIN_LAYER_GEOMETRY) {
  return direct_workspace_query(GEOM_FROM_LAYER, true);
}

int64_t mellin_index_map_build(int relation, int order, int64_t nf, int64_t ng, int64_t nh, int64_t s,
                               int64_t d, int64_t p, int64_t u, int32_t *row_ptr, int32_t *entries,
                               int64_t capacity) {
  if (relation < 0 || relation > 1 || order < 0 || order > 2) {
    fail(MELLIN_ERR_BAD_ARGUMENT, "index_map_build: relation must be 0/1 and order 0/1/2");
    return -1;
  }
  IndexMap m;
  try {
    m = build_index_map(IndexMapKey{static_cast<Relation>(relation), static_cast<SortBy>(order), nf, ng, nh, s, d, p, u});
  } catch (const std::exception &e) {
    fail(MELLIN_ERR_BAD_ARGUMENT, e.what());
    return -1;
  }
  if (row_ptr != nullptr)
    for (size_t i = 0; i < m.row_ptr.size(); ++i) row_ptr[i] = m.row_ptr[i];
  if (entries != nullptr)
    for (size_t i = 0; i < m.entries.size() && static_cast<int64_t>(i) < capacity; ++i) {
      entries[2 * i] = m.entries[i].a;
      entries[2 * i + 1] = m.entries[i].b;
    }
  return static_cast<int64_t>(m.entries.size());
}

size_t mellin_mcorrlcorr_grad_weight_workspace_bytes(MELLIN_LAYER_GEOMETRY) {
  return gradw_workspace_query(GEOM_FROM_LAYER);
}

size_t mellin_mcorrlcorr_forward_workspace_bytes_f16(MELLIN_LAYER_GEOMETRY) { return half_buffers(GEOM_FROM_LAYER, 0).total(); }
size_t mellin_mcorrlcorr_grad_input_workspace_bytes_f16(MELLIN_LAYER_GEOMETRY) { return half_buffers(GEOM_FROM_LAYER, 1).total(); }
size_t mellin_mcorrlcorr_grad_weight_workspace_bytes_f16(MELLIN_LAYER_GEOMETRY) { return half_buffers(GEOM_FROM_LAYER, 2).total(); }

int mellin_mcorrlcorr_forward_f16(const void *x, const void *w, const void *bias, MELLIN_LAYER_GEOMETRY, void *y,
                                  void *workspace, size_t workspace_bytes, void *stream) {
  const Geometry2D q = GEOM_FROM_LAYER;
  const HalfBuffers h = half_buffers(q, 0);
  int rc = half_check("mcorrlcorr_forward_f16", q, h, workspace, workspace_bytes);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char *base = static_cast<unsigned char *>(workspace);
  float *x32 = reinterpret_cast<float *>(base), *w32 = reinterpret_cast<float *>(base + h.x);
  float *b32 = reinterpret_cast<float *>(base + h.x + h.w), *y32 = reinterpret_cast<float *>(base + h.x + h.w + h.b);
  if ((rc = convert_launch(true, x, x32, q.batch * q.c_in * q.ngx * q.ngy, st))) return rc;
  if ((rc = convert_launch(true, w, w32, q.c_out * q.c_in * q.nfx * q.nfy, st))) return rc;
  if ((rc = convert_launch(true, bias, b32, q.c_out, st))) return rc;
  rc = op2d<float>("mcorrlcorr_forward_f16", Relation::Corr, w32, x32, q, 0, 0, 0, y32, bias ? b32 : nullptr, false,
                   base + h.x + h.w + h.b + h.y, h.inner, stream, nullptr, 0, 0.0, 0, /*exact=*/1);
  if (rc) return rc;
  return convert_launch(false, y32, y, q.batch * q.c_out * q.nhx * q.nhy, st);
}

int mellin_mcorrlcorr_grad_input_f16(const void *w, const void *grad_y, MELLIN_LAYER_GEOMETRY, void *grad_x,
                                     void *workspace, size_t workspace_bytes, void *stream) {
  const Geometry2D q = GEOM_FROM_LAYER;
  const HalfBuffers h = half_buffers(q, 1);
  int rc = half_check("mcorrlcorr_grad_input_f16", q, h, workspace, workspace_bytes);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char *base = static_cast<unsigned char *>(workspace);
  float *x32 = reinterpret_cast<float *>(base), *w32 = reinterpret_cast<float *>(base + h.x);
  float *y32 = reinterpret_cast<float *>(base + h.x + h.w + h.b);
  if ((rc = convert_launch(true, w, w32, q.c_out * q.c_in * q.nfx * q.nfy, st))) return rc;
  if ((rc = convert_launch(true, grad_y, y32, q.batch * q.c_out * q.nhx * q.nhy, st))) return rc;
  rc = grad_input<float>("mcorrlcorr_grad_input_f16", w32, y32, q, x32, base + h.x + h.w + h.b + h.y, h.inner, stream,
                         nullptr, /*exact=*/1);
  if (rc) return rc;
  return convert_launch(false, x32, grad_x, q.batch * q.c_in * q.ngx * q.ngy, st);
}

int mellin_mcorrlcorr_grad_weight_f16(const void *x, const void *grad_y, MELLIN_LAYER_GEOMETRY, void *grad_w,
                                      void *grad_b, void *workspace, size_t workspace_bytes, void *stream) {
  const Geometry2D q = GEOM_FROM_LAYER;
  const HalfBuffers h = half_buffers(q, 2);
  int rc = half_check("mcorrlcorr_grad_weight_f16", q, h, workspace, workspace_bytes);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char *base = static_cast<unsigned char *>(workspace);
  float *x32 = reinterpret_cast<float *>(base), *w32 = reinterpret_cast<float *>(base + h.x);
  float *b32 = reinterpret_cast<float *>(base + h.x + h.w), *y32 = reinterpret_cast<float *>(base + h.x + h.w + h.b);
  if ((rc = convert_launch(true, x, x32, q.batch * q.c_in * q.ngx * q.ngy, st))) return rc;
  if ((rc = convert_launch(true, grad_y, y32, q.batch * q.c_out * q.nhx * q.nhy, st))) return rc;
  rc = grad_weight<float>("mcorrlcorr_grad_weight_f16", x32, y32, q, w32, grad_b ? b32 : nullptr,
                          base + h.x + h.w + h.b + h.y, h.inner, stream, nullptr, /*exact=*/1);
  if (rc) return rc;
  if ((rc = convert_launch(false, w32, grad_w, q.c_out * q.c_in * q.nfx * q.nfy, st))) return rc;
  return grad_b ? convert_launch(false, b32, grad_b, q.c_out, st) : MELLIN_OK;
}

}  // extern "C"
