// Internal declarations shared by the C-ABI layer and the kernel launchers.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "index_map.h"

namespace mellin {

// ---- error reporting ---------------------------------------------------------
void set_error(const std::string &msg);
int fail(int code, const std::string &msg);  // records msg, returns code
void count_launch(int n = 1);

// Programmatic dependent launch can be switched off (environment variable MELLIN_DEPENDENT_LAUNCH=0, read once,
// or mellin_set_dependent_launch): the kernels' waits then return at once and every launch is an ordinary one.
bool dependent_launch_enabled();
int set_dependent_launch(int enable);

// Launches `kernel` so that it may begin while the kernel before it in the stream still runs (programmatic
// dependent launch): its blocks are scheduled as that kernel's blocks make room, run their prologue, and wait
// in tc::grid_dependency_wait() for that kernel to complete.  Only for kernels that make that call.
template <typename... KernelArgs, typename... Args>
cudaError_t launch_after_predecessor(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;  // without it: an ordinary launch
  return cudaLaunchKernelEx(&cfg, kernel, KernelArgs(args)...);
}

// ---- device-resident index maps ------------------------------------------------
struct DeviceTable {
  const int32_t *row_ptr = nullptr;
  const int2 *entries = nullptr;
  const int32_t *order = nullptr;
  int32_t rows = 0;
  int32_t max_row = 0;
  int64_t triples = 0;
  int64_t num_entries = 0;
};

// Looks the table up in the per-device cache, building and uploading it on
// first use (one cudaMalloc + one synchronous cudaMemcpy: a set-up cost paid
// once per geometry per device).  Returns a status code.
int get_device_table(const IndexMapKey &key, DeviceTable *out);
int clear_device_tables();
// library-owned scratch of the operator-level entry points (table_cache.cu); nullptr when it cannot be had
void *scratch_arena(size_t bytes, cudaStream_t stream);
int sm_count();  // of the current device (cached)

// ---- problem descriptions ------------------------------------------------------
//
// Every multi-channel operator on the path is an instance of
//
//   out[n, a, ox, oy] (+)= sum_b sum_{(kx, ix) in row ox of the Mellin table}
//                        sum_ky W[a, b, kx, ky] * in[n, b, ix, iy(oy, ky)]
//   iy(oy, ky) = (Ay * oy + By * ky + Cy) / Dy   (exact, 0 <= iy < niy)
//
// with arbitrary (n, channel) strides so that the reference's transposition
// flags and the weight-transposed grad-input form need no copies.
template <typename T>
struct DirectProblem {
  const T *in = nullptr;
  const T *w = nullptr;
  const T *bias = nullptr;  // used when !accumulate; may be null
  T *out = nullptr;
  DeviceTable table;  // rows = ox, entries (kx, ix)
  // The same triples by SOURCE row (rows = ix, entries (kx, ox)); optional: filled in for problems
  // with a handful of output channels, which tc_scatter.cu walks by source row.
  DeviceTable table_by_in;
  int N = 0, A = 0, B = 0;
  int nkx = 0, nky = 0, nix = 0, niy = 0, nox = 0, noy = 0;
  long long in_sn = 0, in_sb = 0;    // element strides of in[n], in[.., b]
  long long w_sa = 0, w_sb = 0;      // element strides of W[a], W[.., b]; (kx, ky) plane is dense
  long long out_sn = 0, out_sa = 0;  // element strides of out[n], out[.., a]
  int Ay = 1, By = 1, Cy = 0, Dy = 1;
  bool accumulate = false;
  // fused epilogue (layer-level forward only): out = (oy < lens[n]) ? act(value) : 0
  const int *lens = nullptr;  // device array of N lengths along the linear axis, or null
  int len_scale = 1, len_offset = 0;  // the bound used is lens[n] * len_scale + len_offset
  int relu = 0;
  // fused dropout (training): an output element is zeroed when dropout_hash(seed, its offset in `out`) falls below
  // drop_threshold (= p * 2^32; 0 switches dropout off) and scaled by drop_scale = 1 / (1 - p) otherwise
  unsigned drop_threshold = 0, drop_seed = 0;
  float drop_scale = 1.f;
  // Both operands hold values that are exact in TF32 (e.g. widened float16): the tensor-core kernels then skip the
  // two error-compensation products of their hi/lo split (the lo parts are all zero) -- one MMA per product, not three.
  int exact_tf32 = 0;
};

// Stateless per-element random number of the fused dropout: a 32-bit avalanche hash of (seed, element offset).
// Every kernel that can write a layer's output uses this one function, so the mask does not depend on the kernel.
__host__ __device__ __forceinline__ unsigned dropout_hash(unsigned seed, unsigned long long offset) {
  unsigned h = (unsigned)offset * 0x9E3779B1u ^ seed ^ ((unsigned)(offset >> 32) * 0x85EBCA77u);
  h ^= h >> 16;
  h *= 0x85EBCA6Bu;
  h ^= h >> 13;
  h *= 0xC2B2AE35u;
  h ^= h >> 16;
  return h;
}

// Weight gradient of a correlation layer:
//   gw[a, b, kx, ky] = sum_n sum_{(ox, ix) in row kx} sum_oy
//                      go[n, a, ox, oy] * in[n, b, ix, (Ay*oy + By*ky + Cy)/Dy]
//   gb[a]            = sum_{n, ox, oy} go[n, a, ox, oy]
// All tensors dense and untransposed.
template <typename T>
struct GradWProblem {
  const T *in = nullptr;   // (N, B, nix, niy)
  const T *go = nullptr;   // (N, A, nox, noy)
  T *gw = nullptr;         // (A, B, nkx, nky)
  T *gb = nullptr;         // (A) or null
  DeviceTable table;       // rows = kx, entries (ox | flags, ix)
  DeviceTable table_h;     // the same triples by output row: rows = ox, entries (kx, ix)
  const int *lens = nullptr;  // optional: grad_y is zero from position lens[n] on (device array of N)
  int N = 0, A = 0, B = 0;
  int nkx = 0, nky = 0, nix = 0, niy = 0, nox = 0, noy = 0;
  int Ay = 1, By = 1, Cy = 0, Dy = 1;
  int exact_tf32 = 0;  // as in DirectProblem
};

// gather / scatter between a signal and its column form
template <typename T>
struct ColProblem {
  const T *src = nullptr;
  T *dst = nullptr;
  int N = 0, C = 0;
  int nfx = 0, nfy = 0, ngx = 0, ngy = 0, nggx = 0, nggy = 0;
  int sx = 1, sy = 1, dx = 1, dy = 1, px = 0, py = 0, ux = 1, uy = 1;
  bool transposed_g = false, transposed_gg = false;
};

template <typename T> int launch_direct(const DirectProblem<T> &p, cudaStream_t stream);
// tensor-core path (tc_direct.cu): scratch for the packed hi/lo weights, launch
// (MELLIN_ERR_UNSUPPORTED when the problem is outside its coverage), and the
// device-side timeout flag
// few-input-channel forward kernel (few_in_rows.cu), carries the fused mask / ReLU epilogue;
// MELLIN_ERR_UNSUPPORTED when not covered
int launch_few_in_rows(const DirectProblem<float> &p, cudaStream_t stream);
// few-output-channel kernel (direct_rows.cu); MELLIN_ERR_UNSUPPORTED when not covered
size_t direct_rows_workspace_bytes(const DirectProblem<float> &p);
int launch_direct_rows(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
size_t direct_tc_workspace_bytes(const DirectProblem<float> &p);
int launch_direct_tc(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
int tc_take_error(int *code);
int direct_rows_take_error(int *code);
// few-input-channel forward on tensor cores (tc_few_in.cu)
size_t tc_few_in_workspace_bytes(const DirectProblem<float> &p);
int launch_tc_few_in(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
int tc_few_in_take_error(int *code);
// few-output-channel operator walked by source row on tensor cores (tc_scatter.cu); needs p.table_by_in
size_t tc_scatter_workspace_bytes(const DirectProblem<float> &p);
int launch_tc_scatter(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
int tc_scatter_take_error(int *code);
int gradw_rows_take_error(int *code);
int launch_unarmed_wait(cudaStream_t stream);  // self-test of the bounded waits (gradw_rows.cu)
// tensor-core forward with the fused length mask / ReLU epilogue (tc_direct_masked.cu)
size_t direct_tc_workspace_bytes_masked(const DirectProblem<float> &p);
int launch_direct_tc_masked(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
// tensor-core weight gradient for wide layers (tc_gradw.cu): floats of partial
// sums (0 when not covered), launch, and the device-side timeout flag
size_t gradw_tc_workspace_floats(const GradWProblem<float> &p, size_t *bias_offset);
int launch_gradw_tc(const GradWProblem<float> &p, float *part_w, float *part_b, cudaStream_t stream);
int tc_gradw_take_error(int *code);
// 1-D Mellin operators through the tensor-core kernels, the batch standing in
// for the linear axis (batch_inner.cu); 0 bytes / MELLIN_ERR_UNSUPPORTED when not covered
size_t direct_batch_inner_workspace_bytes(const DirectProblem<float> &p);
int launch_direct_batch_inner(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes,
                              cudaStream_t stream);
size_t gradw_batch_inner_workspace_bytes(const GradWProblem<float> &p);
int launch_gradw_batch_inner(const GradWProblem<float> &p, void *workspace, size_t workspace_bytes,
                             cudaStream_t stream);
// tensor-core weight gradient for linear extents that are not multiples of 4: zero-padded copies first
size_t gradw_repitch_workspace_bytes(const GradWProblem<float> &p);
int launch_gradw_repitched(const GradWProblem<float> &p, void *workspace, size_t workspace_bytes,
                           cudaStream_t stream);
size_t direct_repitch_workspace_bytes(const DirectProblem<float> &p);
int launch_direct_repitched(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes,
                            cudaStream_t stream);
bool tensor_cores_enabled();
int set_tensor_cores(int enable);
template <typename T> size_t gradw_workspace_bytes(const GradWProblem<T> &p);
template <typename T>
int launch_gradw(const GradWProblem<T> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
// few-input-channel weight gradient on tensor cores (tc_gradw_few_in.cu): scratch in floats (0 = not covered),
// partial sums and their reduction
size_t tc_gradw_few_in_workspace_floats(const GradWProblem<float> &p);
int launch_tc_gradw_few_in(const GradWProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
int tc_gradw_few_in_take_error(int *code);
// few-input-channel weight gradient (gradw_rows.cu): partial-sum scratch in floats
// (0 = not covered) and the launch that fills it
size_t gradw_rows_workspace_floats(const GradWProblem<float> &p, size_t *bias_offset);
int launch_gradw_rows(const GradWProblem<float> &p, float *part_w, float *part_b, int *slices, cudaStream_t stream);
template <typename T> int launch_spec2col(const ColProblem<T> &p, cudaStream_t stream);
template <typename T> int launch_col2spec(const ColProblem<T> &p, cudaStream_t stream);

}  // namespace mellin
