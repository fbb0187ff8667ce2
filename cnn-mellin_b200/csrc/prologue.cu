// The two elementwise layers in front of the first Mellin layer, as one pass over the tensor:
//
//   c[i] = log(eps + |x[i]|)          (log compression, layers.py:100-101 of the reference)
//   y[i] = (t + 1)^tau * c[i]         (dilation lift along one axis, layers.py:8-21; t = index along that axis)
//
// and their backward as one pass (grad_x and the block sums of the two parameter gradients) followed by a
// fixed-order sum of the block sums.  The reference runs abs, add, log, arange, pow, mul as separate torch
// kernels (six passes over the tensor forward, more backward).  The tensor is viewed as [outer][len][inner],
// contiguous, with `len` the lifted axis.  Either step can be left out (null parameter pointer).
//
// The parameters are DEVICE scalars (the layers' learnable log_tau / log_eps): nothing is read back to the host.
// With log_domain != 0 they hold log(tau) / log(eps), as the reference's modules store them, and the parameter
// gradients are taken with respect to those logarithms.
//
// HBM-bound: 8 bytes per element forward (read x, write y), 12 backward (read x and grad_y, write grad_x).
// The weights (t + 1)^tau are built once per block in shared memory (pow is ~100 instructions; a table entry
// is one shared load), 16-byte accesses where `inner` is a multiple of 4.
#include <algorithm>
#include <cmath>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"

namespace mellin {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxBlocks = 4096;        // also fixes the size of the backward's block sums
constexpr int kTableBytes = 40 * 1024;  // weights kept in shared memory up to this size

template <typename T>
struct Params {
  T tau, eps;
  bool lift, compress;
};

template <typename T>
__device__ __forceinline__ Params<T> load_params(const T *tau, const T *eps, int log_domain) {
  Params<T> q;
  q.lift = tau != nullptr, q.compress = eps != nullptr;
  q.tau = q.lift ? (log_domain ? exp(*tau) : *tau) : T(0);
  q.eps = q.compress ? (log_domain ? exp(*eps) : *eps) : T(0);
  return q;
}

// weights of the lifted axis into shared memory (or nothing when the axis is longer than the table)
template <typename T>
__device__ __forceinline__ void build_table(T *table, long long len, bool in_smem, const Params<T> &q) {
  if (in_smem && q.lift)
    for (long long t = threadIdx.x; t < len; t += blockDim.x) table[t] = pow(T(t + 1), q.tau);
  __syncthreads();
}
template <typename T>
__device__ __forceinline__ T weight(const T *table, long long t, bool in_smem, const Params<T> &q) {
  if (!q.lift) return T(1);
  return in_smem ? table[t] : pow(T(t + 1), q.tau);
}

template <typename T>
__device__ __forceinline__ T compressed(T x, const Params<T> &q) {
  return q.compress ? log(q.eps + fabs(x)) : x;
}

// position along the lifted axis of element i; I is a 32-bit type for tensors below 2^31 elements (a 64-bit
// division costs about as much as the rest of an element's work)
template <typename I>
__device__ __forceinline__ long long axis_index(long long i, long long inner, long long len) {
  return (long long)(((I)i / (I)inner) % (I)len);
}

template <typename T, int VEC, typename I>
__global__ void __launch_bounds__(kThreads)
lift_compress_kernel(const T *__restrict__ x, T *__restrict__ y, const T *__restrict__ tau_p,
                     const T *__restrict__ eps_p, int log_domain, long long total, long long len, long long inner,
                     int table_in_smem) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T *table = reinterpret_cast<T *>(smem_raw);
  const Params<T> q = load_params(tau_p, eps_p, log_domain);
  build_table(table, len, table_in_smem != 0, q);
  const long long groups = total / VEC, step = (long long)gridDim.x * blockDim.x;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups; g += step) {
    const long long i = g * VEC;
    if constexpr (VEC == 4) {  // inner is a multiple of 4: the four elements share t
      const T w = weight(table, axis_index<I>(i, inner, len), table_in_smem != 0, q);
      const float4 v = *reinterpret_cast<const float4 *>(x + i);
      float4 o;
      o.x = w * compressed((T)v.x, q), o.y = w * compressed((T)v.y, q);
      o.z = w * compressed((T)v.z, q), o.w = w * compressed((T)v.w, q);
      *reinterpret_cast<float4 *>(y + i) = o;
    } else {
      y[i] = weight(table, axis_index<I>(i, inner, len), table_in_smem != 0, q) * compressed(x[i], q);
    }
  }
}

// one element of the backward: grad_x, and the terms of the two parameter sums
//   y = w c, w = (t+1)^tau, c = log(eps + |x|)
//   d y / d tau = y log(t+1);  d y / d eps = w / (eps + |x|);  d y / d x = w sign(x) / (eps + |x|)
template <typename T>
__device__ __forceinline__ T backward_element(T x, T gy, T w, T log_t1, const Params<T> &q, T &sum_tau, T &sum_eps) {
  const T gc = gy * w;
  T gx = gc;
  if (q.compress) {
    const T inv = T(1) / (q.eps + fabs(x));
    sum_eps += gc * inv;
    gx = x > T(0) ? gc * inv : (x < T(0) ? -gc * inv : T(0));
  }
  if (q.lift) sum_tau += gc * compressed(x, q) * log_t1;
  return gx;
}

template <typename T, int VEC, typename I>
__global__ void __launch_bounds__(kThreads)
lift_compress_backward_kernel(const T *__restrict__ x, const T *__restrict__ grad_y, T *__restrict__ grad_x,
                              const T *__restrict__ tau_p, const T *__restrict__ eps_p, int log_domain,
                              long long total, long long len, long long inner, int table_in_smem,
                              double *__restrict__ block_sums) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T *table = reinterpret_cast<T *>(smem_raw);
  __shared__ double warp_sums[2][kThreads / 32];
  const Params<T> q = load_params(tau_p, eps_p, log_domain);
  build_table(table, len, table_in_smem != 0, q);
  // a thread adds its own few hundred terms in T (double-precision adds per element would cost more than the
  // rest of the element's work); across threads and blocks the sums are carried in double
  T thread_tau = T(0), thread_eps = T(0);
  const long long groups = total / VEC, step = (long long)gridDim.x * blockDim.x;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups; g += step) {
    const long long i = g * VEC, t = axis_index<I>(i, inner, len);
    const T w = weight(table, t, table_in_smem != 0, q);
    const T log_t1 = q.lift ? log(T(t + 1)) : T(0);
    if constexpr (VEC == 4) {
      const float4 v = *reinterpret_cast<const float4 *>(x + i);
      const float4 gy = *reinterpret_cast<const float4 *>(grad_y + i);
      float4 o;
      o.x = backward_element((T)v.x, (T)gy.x, w, log_t1, q, thread_tau, thread_eps);
      o.y = backward_element((T)v.y, (T)gy.y, w, log_t1, q, thread_tau, thread_eps);
      o.z = backward_element((T)v.z, (T)gy.z, w, log_t1, q, thread_tau, thread_eps);
      o.w = backward_element((T)v.w, (T)gy.w, w, log_t1, q, thread_tau, thread_eps);
      *reinterpret_cast<float4 *>(grad_x + i) = o;
    } else {
      grad_x[i] = backward_element(x[i], grad_y[i], w, log_t1, q, thread_tau, thread_eps);
    }
  }
  // block sums in a fixed order: lanes by shuffle tree, warps one after the other
  double sum_tau = (double)thread_tau, sum_eps = (double)thread_eps;
  for (int off = 16; off > 0; off >>= 1) {
    sum_tau += __shfl_down_sync(0xffffffffu, sum_tau, off);
    sum_eps += __shfl_down_sync(0xffffffffu, sum_eps, off);
  }
  if ((threadIdx.x & 31) == 0) warp_sums[0][threadIdx.x >> 5] = sum_tau, warp_sums[1][threadIdx.x >> 5] = sum_eps;
  __syncthreads();
  if (threadIdx.x < 2) {
    double s = 0.0;
    for (int wi = 0; wi < kThreads / 32; ++wi) s += warp_sums[threadIdx.x][wi];
    block_sums[2 * blockIdx.x + threadIdx.x] = s;
  }
}

// grad_tau / grad_eps = the block sums added in block order by one warp (lane l takes blocks l, l + 32, ...),
// times tau / eps when the parameters are held as logarithms
template <typename T>
__global__ void lift_compress_finish_kernel(const double *__restrict__ block_sums, int blocks,
                                            const T *__restrict__ tau_p, const T *__restrict__ eps_p, int log_domain,
                                            T *__restrict__ grad_tau, T *__restrict__ grad_eps) {
  double s0 = 0.0, s1 = 0.0;
  for (int b = threadIdx.x; b < blocks; b += 32) s0 += block_sums[2 * b], s1 += block_sums[2 * b + 1];
  for (int off = 16; off > 0; off >>= 1) {
    s0 += __shfl_down_sync(0xffffffffu, s0, off);
    s1 += __shfl_down_sync(0xffffffffu, s1, off);
  }
  if (threadIdx.x == 0) {
    const Params<T> q = load_params(tau_p, eps_p, log_domain);
    if (grad_tau != nullptr) *grad_tau = q.lift ? (T)(log_domain ? s0 * (double)q.tau : s0) : T(0);
    if (grad_eps != nullptr) *grad_eps = q.compress ? (T)(log_domain ? s1 * (double)q.eps : s1) : T(0);
  }
}

// Blocks of `kernel` that one SM holds at a time.  The kernels walk the tensor in grid-sized strides, so the grid
// must be what the device holds at once: a grid of 8 blocks per SM under a kernel that fits 6 runs as 1.33 waves.
template <typename K>
int resident_blocks(K kernel, size_t smem) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem) != cudaSuccess || per_sm < 1) {
    (void)cudaGetLastError();
    per_sm = 1;
  }
  return per_sm;
}

struct Plan {
  long long total;
  int blocks, vec, table_in_smem, wide_index;
  size_t smem;
};

template <typename T>
int make_plan(const char *who, int64_t outer, int64_t len, int64_t inner, const void *a, const void *b, const void *c,
              bool three_tensors, Plan *plan) {
  if (outer < 0 || len < 0 || inner < 0) return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": negative extent");
  const long double prod = (long double)outer * (long double)len * (long double)inner;
  if (prod > 9.0e18L) return fail(MELLIN_ERR_UNSUPPORTED, std::string(who) + ": more than 2^63 elements");
  plan->total = (long long)outer * len * inner;
  if (plan->total == 0) return MELLIN_OK;
  if (a == nullptr || b == nullptr || (c == nullptr && three_tensors))
    return fail(MELLIN_ERR_BAD_ARGUMENT, std::string(who) + ": null pointer");
  auto aligned = [](const void *p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  plan->vec = (sizeof(T) == 4 && inner % 4 == 0 && aligned(a) && aligned(b) && aligned(c)) ? 4 : 1;
  plan->wide_index = plan->total >= (1LL << 31) ? 1 : 0;
  plan->table_in_smem = (size_t)len * sizeof(T) <= (size_t)kTableBytes ? 1 : 0;
  plan->smem = plan->table_in_smem ? (size_t)len * sizeof(T) : 0;
  const long long groups = plan->total / plan->vec, per_block = (long long)kThreads * 4;
  plan->blocks = (int)std::max<long long>(1, std::min<long long>((groups + per_block - 1) / per_block, kMaxBlocks));
  return MELLIN_OK;
}

template <typename T>
int launch_forward(const T *x, const T *tau, const T *eps, int log_domain, int64_t outer, int64_t len, int64_t inner,
                   T *y, void *stream) {
  Plan plan{};
  const int rc = make_plan<T>("lift_compress", outer, len, inner, x, y, nullptr, false, &plan);
  if (rc != MELLIN_OK || plan.total == 0) return rc;
  auto st = static_cast<cudaStream_t>(stream);
  auto go = [&](auto kernel) {
    plan.blocks = std::min(plan.blocks, sm_count() * resident_blocks(kernel, plan.smem));
    kernel<<<plan.blocks, kThreads, plan.smem, st>>>(x, y, tau, eps, log_domain, plan.total, len, inner,
                                                     plan.table_in_smem);
  };
  if constexpr (sizeof(T) == 4) {
    if (plan.vec == 4 && !plan.wide_index) go(lift_compress_kernel<T, 4, unsigned>);
    else if (plan.vec == 4) go(lift_compress_kernel<T, 4, long long>);
  }
  if (plan.vec == 1 && !plan.wide_index) go(lift_compress_kernel<T, 1, unsigned>);
  else if (plan.vec == 1) go(lift_compress_kernel<T, 1, long long>);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("lift_compress_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

template <typename T>
int launch_backward(const T *x, const T *grad_y, const T *tau, const T *eps, int log_domain, int64_t outer,
                    int64_t len, int64_t inner, T *grad_x, T *grad_tau, T *grad_eps, void *workspace,
                    size_t workspace_bytes, void *stream) {
  Plan plan{};
  const int rc = make_plan<T>("backward of lift_compress", outer, len, inner, x, grad_y, grad_x, true, &plan);
  if (rc != MELLIN_OK) return rc;
  auto st = static_cast<cudaStream_t>(stream);
  if (workspace == nullptr || workspace_bytes < mellin_lift_compress_workspace_bytes())
    return fail(MELLIN_ERR_WORKSPACE, "backward of lift_compress: workspace smaller than mellin_lift_compress_workspace_bytes()");
  if ((reinterpret_cast<uintptr_t>(workspace) & 7u) != 0)
    return fail(MELLIN_ERR_WORKSPACE, "backward of lift_compress: workspace must be 8-byte aligned");
  double *block_sums = static_cast<double *>(workspace);
  if (plan.total > 0) {
    auto go = [&](auto kernel) {
      plan.blocks = std::min(plan.blocks, sm_count() * resident_blocks(kernel, plan.smem));
      kernel<<<plan.blocks, kThreads, plan.smem, st>>>(x, grad_y, grad_x, tau, eps, log_domain, plan.total, len, inner,
                                                       plan.table_in_smem, block_sums);
    };
    if constexpr (sizeof(T) == 4) {
      if (plan.vec == 4 && !plan.wide_index) go(lift_compress_backward_kernel<T, 4, unsigned>);
      else if (plan.vec == 4) go(lift_compress_backward_kernel<T, 4, long long>);
    }
    if (plan.vec == 1 && !plan.wide_index) go(lift_compress_backward_kernel<T, 1, unsigned>);
    else if (plan.vec == 1) go(lift_compress_backward_kernel<T, 1, long long>);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
      return fail(MELLIN_ERR_LAUNCH, std::string("lift_compress_backward_kernel: ") + cudaGetErrorString(err));
    count_launch();
  }
  if (grad_tau != nullptr || grad_eps != nullptr) {
    lift_compress_finish_kernel<T><<<1, 32, 0, st>>>(block_sums, plan.total > 0 ? plan.blocks : 0, tau, eps, log_domain,
                                                     grad_tau, grad_eps);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
      return fail(MELLIN_ERR_LAUNCH, std::string("lift_compress_finish_kernel: ") + cudaGetErrorString(err));
    count_launch();
  }
  return MELLIN_OK;
}

}  // namespace
}  // namespace mellin

using namespace mellin;

extern "C" {

size_t mellin_lift_compress_workspace_bytes(void) { return (size_t)kMaxBlocks * 2 * sizeof(double); }

int mellin_lift_compress_f32(const float *x, const float *tau, const float *eps, int log_domain, int64_t outer,
                             int64_t len, int64_t inner, float *y, void *stream) {
  return launch_forward<float>(x, tau, eps, log_domain, outer, len, inner, y, stream);
}
int mellin_lift_compress_f64(const double *x, const double *tau, const double *eps, int log_domain, int64_t outer,
                             int64_t len, int64_t inner, double *y, void *stream) {
  return launch_forward<double>(x, tau, eps, log_domain, outer, len, inner, y, stream);
}
int mellin_lift_compress_backward_f32(const float *x, const float *grad_y, const float *tau, const float *eps,
                                      int log_domain, int64_t outer, int64_t len, int64_t inner, float *grad_x,
                                      float *grad_tau, float *grad_eps, void *workspace, size_t workspace_bytes,
                                      void *stream) {
  return launch_backward<float>(x, grad_y, tau, eps, log_domain, outer, len, inner, grad_x, grad_tau, grad_eps,
                                workspace, workspace_bytes, stream);
}
int mellin_lift_compress_backward_f64(const double *x, const double *grad_y, const double *tau, const double *eps,
                                      int log_domain, int64_t outer, int64_t len, int64_t inner, double *grad_x,
                                      double *grad_tau, double *grad_eps, void *workspace, size_t workspace_bytes,
                                      void *stream) {
  return launch_backward<double>(x, grad_y, tau, eps, log_domain, outer, len, inner, grad_x, grad_tau, grad_eps,
                                 workspace, workspace_bytes, stream);
}

}  // extern "C"
