// 1-D Mellin operators (singleton linear axis) on the tensor-core kernels.
//
// The 2-D kernels want a long contiguous "linear" axis; a 1-D Mellin signal has
// none, but every utterance of the batch is gathered with the same index map, so
// the batch can play that part: x[n, c, ix] is transposed to x'[c, ix, n] and the
// operator becomes a 2-D one over a single "utterance" whose linear axis has N
// positions and one tap.  The Mellin table, the weights and the bias are
// unchanged; the result comes back through the inverse transposition (the
// weight gradient needs none).  Two extra passes over the activations buy the
// tcgen05 kernels for an operator that is otherwise a per-output gather.
//
// Also here: re-pitching.  The TMA loads of the tensor-core kernels need row
// pitches that are multiples of 16 bytes; signals whose linear extent is not a
// multiple of 4 are first copied into zero-padded rows (the padding contributes
// nothing: zeros beyond the signal are what the operators read there anyway).
#include <algorithm>
#include <string>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"

namespace mellin {

namespace {

constexpr int kTile = 32;

// dst[(c * L + x) * Np + n] = n < N ? src[n * sn + c * sc + x] : 0   (Np >= N: the padded batch)
__global__ void to_batch_inner_kernel(const float *__restrict__ src, long long sn, long long sc, int N, int Np, int C,
                                      int L, float *__restrict__ dst) {
  __shared__ float tile[kTile][kTile + 1];
  const int c = blockIdx.z;
  const int x0 = blockIdx.x * kTile, n0 = blockIdx.y * kTile;
  for (int j = threadIdx.y; j < kTile; j += blockDim.y) {
    const int n = n0 + j, x = x0 + threadIdx.x;
    tile[j][threadIdx.x] = (n < N && x < L) ? src[n * sn + c * sc + x] : 0.f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < kTile; j += blockDim.y) {
    const int x = x0 + j, n = n0 + threadIdx.x;
    if (x < L && n < Np) dst[((long long)c * L + x) * Np + n] = tile[threadIdx.x][j];
  }
}

// dst[n * dn + c * dc + x] = src[(c * L + x) * Np + n]
__global__ void from_batch_inner_kernel(const float *__restrict__ src, int N, int Np, int C, int L,
                                        float *__restrict__ dst, long long dn, long long dc) {
  __shared__ float tile[kTile][kTile + 1];
  const int c = blockIdx.z;
  const int x0 = blockIdx.x * kTile, n0 = blockIdx.y * kTile;
  for (int j = threadIdx.y; j < kTile; j += blockDim.y) {
    const int x = x0 + j, n = n0 + threadIdx.x;
    tile[j][threadIdx.x] = (x < L && n < N) ? src[((long long)c * L + x) * Np + n] : 0.f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < kTile; j += blockDim.y) {
    const int n = n0 + j, x = x0 + threadIdx.x;
    if (n < N && x < L) dst[n * dn + c * dc + x] = tile[threadIdx.x][j];
  }
}

// dst[r * pitch + i] = i < len ? src[r * len + i] : 0
__global__ void repitch_kernel(const float *__restrict__ src, long long rows, int len, int pitch,
                               float *__restrict__ dst) {
  const long long total = rows * pitch;
  for (long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x; j < total;
       j += (long long)gridDim.x * blockDim.x) {
    const long long r = j / pitch;
    const int i = (int)(j - r * pitch);
    dst[j] = i < len ? src[r * len + i] : 0.f;
  }
}

int check(const char *what) {
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string(what) + ": " + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

// the batch padded to what the tensor-core kernels need of a linear axis: at least 16 positions, a multiple of 4
int padded_batch(int N) { return std::max(16, (N + 3) / 4 * 4); }

int to_batch_inner(const float *src, long long sn, long long sc, int N, int C, int L, float *dst, cudaStream_t s) {
  if (C > 65535) return MELLIN_ERR_UNSUPPORTED;
  const int Np = padded_batch(N);
  const dim3 grid((L + kTile - 1) / kTile, (Np + kTile - 1) / kTile, C);
  to_batch_inner_kernel<<<grid, dim3(kTile, 8), 0, s>>>(src, sn, sc, N, Np, C, L, dst);
  return check("to_batch_inner_kernel");
}

int from_batch_inner(const float *src, int N, int C, int L, float *dst, long long dn, long long dc, cudaStream_t s) {
  if (C > 65535) return MELLIN_ERR_UNSUPPORTED;
  const dim3 grid((L + kTile - 1) / kTile, (N + kTile - 1) / kTile, C);
  from_batch_inner_kernel<<<grid, dim3(kTile, 8), 0, s>>>(src, N, padded_batch(N), C, L, dst, dn, dc);
  return check("from_batch_inner_kernel");
}

size_t round256(size_t bytes) { return (bytes + 255) / 256 * 256; }

int repitch(const float *src, long long rows, int len, int pitch, float *dst, cudaStream_t s) {
  const long long total = rows * pitch;
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 32);
  repitch_kernel<<<blocks, 256, 0, s>>>(src, rows, len, pitch, dst);
  return check("repitch_kernel");
}

GradWProblem<float> padded_gradw(const GradWProblem<float> &p) {
  GradWProblem<float> q = p;
  q.niy = (p.niy + 3) / 4 * 4;
  q.noy = (p.noy + 3) / 4 * 4;
  return q;
}

// wide 1-D Mellin operators with a batch that can stand in for the linear axis
bool eligible(int N, int A, int B, int nky, int niy, int noy, int Ay, int Cy, int Dy) {
  return tensor_cores_enabled() && niy == 1 && noy == 1 && nky == 1 && Ay == 1 && Cy == 0 && Dy == 1 && N >= 2 &&
         A >= 32 && B >= 16 && A <= 65535 && B <= 65535;
}

DirectProblem<float> inner_direct(const DirectProblem<float> &p, const float *xt, float *yt) {
  DirectProblem<float> q = p;
  q.in = xt, q.out = yt;
  const int Np = padded_batch(p.N);
  q.N = 1, q.niy = Np, q.noy = Np;
  q.in_sn = (long long)p.B * p.nix * Np, q.in_sb = (long long)p.nix * Np;
  q.out_sn = (long long)p.A * p.nox * Np, q.out_sa = (long long)p.nox * Np;
  q.Ay = 1, q.By = 1, q.Cy = 0, q.Dy = 1;
  return q;
}

GradWProblem<float> inner_gradw(const GradWProblem<float> &p, const float *xt, const float *got) {
  GradWProblem<float> q = p;
  q.in = xt, q.go = got;
  q.lens = nullptr;  // the linear axis is the batch here
  q.N = 1, q.niy = padded_batch(p.N), q.noy = padded_batch(p.N);
  q.Ay = 1, q.By = 1, q.Cy = 0, q.Dy = 1;
  return q;
}

}  // namespace

size_t direct_batch_inner_workspace_bytes(const DirectProblem<float> &p) {
  if (p.accumulate || !eligible(p.N, p.A, p.B, p.nky, p.niy, p.noy, p.Ay, p.Cy, p.Dy)) return 0;
  const size_t xt = round256((size_t)p.B * p.nix * padded_batch(p.N) * sizeof(float));
  const size_t yt = round256((size_t)p.A * p.nox * padded_batch(p.N) * sizeof(float));
  const size_t tc = direct_tc_workspace_bytes(inner_direct(p, nullptr, nullptr));
  return tc ? xt + yt + tc : 0;
}

int launch_direct_batch_inner(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes,
                              cudaStream_t stream) {
  const size_t need = direct_batch_inner_workspace_bytes(p);
  if (need == 0 || workspace == nullptr || workspace_bytes < need ||
      reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return MELLIN_ERR_UNSUPPORTED;
  unsigned char *base = static_cast<unsigned char *>(workspace);
  const size_t xt_bytes = round256((size_t)p.B * p.nix * padded_batch(p.N) * sizeof(float));
  const size_t yt_bytes = round256((size_t)p.A * p.nox * padded_batch(p.N) * sizeof(float));
  float *xt = reinterpret_cast<float *>(base);
  float *yt = reinterpret_cast<float *>(base + xt_bytes);
  int rc = to_batch_inner(p.in, p.in_sn, p.in_sb, p.N, p.B, p.nix, xt, stream);
  if (rc) return rc;
  rc = launch_direct_tc(inner_direct(p, xt, yt), base + xt_bytes + yt_bytes, workspace_bytes - xt_bytes - yt_bytes,
                        stream);
  if (rc) return rc;
  return from_batch_inner(yt, p.N, p.A, p.nox, p.out, p.out_sn, p.out_sa, stream);
}

size_t gradw_batch_inner_workspace_bytes(const GradWProblem<float> &p) {
  if (!eligible(p.N, p.A, p.B, p.nky, p.niy, p.noy, p.Ay, p.Cy, p.Dy)) return 0;
  const size_t xt = round256((size_t)p.B * p.nix * padded_batch(p.N) * sizeof(float));
  const size_t got = round256((size_t)p.A * p.nox * padded_batch(p.N) * sizeof(float));
  const size_t tc = gradw_tc_workspace_floats(inner_gradw(p, nullptr, nullptr), nullptr) * sizeof(float);
  return tc ? xt + got + round256(tc) : 0;
}

int launch_gradw_batch_inner(const GradWProblem<float> &p, void *workspace, size_t workspace_bytes,
                             cudaStream_t stream) {
  const size_t need = gradw_batch_inner_workspace_bytes(p);
  if (need == 0 || workspace == nullptr || workspace_bytes < need ||
      reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return MELLIN_ERR_UNSUPPORTED;
  unsigned char *base = static_cast<unsigned char *>(workspace);
  const size_t xt_bytes = round256((size_t)p.B * p.nix * padded_batch(p.N) * sizeof(float));
  const size_t got_bytes = round256((size_t)p.A * p.nox * padded_batch(p.N) * sizeof(float));
  float *xt = reinterpret_cast<float *>(base);
  float *got = reinterpret_cast<float *>(base + xt_bytes);
  int rc = to_batch_inner(p.in, (long long)p.B * p.nix, p.nix, p.N, p.B, p.nix, xt, stream);
  if (rc) return rc;
  rc = to_batch_inner(p.go, (long long)p.A * p.nox, p.nox, p.N, p.A, p.nox, got, stream);
  if (rc) return rc;
  const GradWProblem<float> q = inner_gradw(p, xt, got);
  size_t bias_off = 0;
  gradw_tc_workspace_floats(q, &bias_off);
  float *pw = reinterpret_cast<float *>(base + xt_bytes + got_bytes);
  return launch_gradw_tc(q, pw, p.gb != nullptr ? pw + bias_off : nullptr, stream);
}

size_t gradw_repitch_workspace_bytes(const GradWProblem<float> &p) {
  if (!tensor_cores_enabled() || (p.niy % 4 == 0 && p.noy % 4 == 0) || p.niy < 1 || p.noy < 1) return 0;
  const GradWProblem<float> q = padded_gradw(p);
  const size_t tc = gradw_tc_workspace_floats(q, nullptr) * sizeof(float);
  if (tc == 0) return 0;
  const size_t xp = p.niy % 4 ? round256((size_t)p.N * p.B * p.nix * q.niy * sizeof(float)) : 0;
  const size_t gop = p.noy % 4 ? round256((size_t)p.N * p.A * p.nox * q.noy * sizeof(float)) : 0;
  return xp + gop + round256(tc);
}

// the tensor-core weight gradient on zero-padded copies of the misaligned operands
int launch_gradw_repitched(const GradWProblem<float> &p, void *workspace, size_t workspace_bytes,
                           cudaStream_t stream) {
  const size_t need = gradw_repitch_workspace_bytes(p);
  if (need == 0 || workspace == nullptr || workspace_bytes < need ||
      reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return MELLIN_ERR_UNSUPPORTED;
  GradWProblem<float> q = padded_gradw(p);
  unsigned char *base = static_cast<unsigned char *>(workspace);
  if (p.niy % 4) {
    float *xp = reinterpret_cast<float *>(base);
    const int rc = repitch(p.in, (long long)p.N * p.B * p.nix, p.niy, q.niy, xp, stream);
    if (rc) return rc;
    q.in = xp;
    base += round256((size_t)p.N * p.B * p.nix * q.niy * sizeof(float));
  }
  if (p.noy % 4) {
    float *gop = reinterpret_cast<float *>(base);
    const int rc = repitch(p.go, (long long)p.N * p.A * p.nox, p.noy, q.noy, gop, stream);
    if (rc) return rc;
    q.go = gop;
    base += round256((size_t)p.N * p.A * p.nox * q.noy * sizeof(float));
  }
  size_t bias_off = 0;
  gradw_tc_workspace_floats(q, &bias_off);
  float *pw = reinterpret_cast<float *>(base);
  return launch_gradw_tc(q, pw, p.gb != nullptr ? pw + bias_off : nullptr, stream);
}

namespace {

bool dense_input(const DirectProblem<float> &p) {
  return p.in_sb == (long long)p.nix * p.niy && p.in_sn == (long long)p.B * p.nix * p.niy;
}

DirectProblem<float> padded_direct(const DirectProblem<float> &p, const float *xp) {
  DirectProblem<float> q = p;
  q.in = xp;
  q.niy = (p.niy + 3) / 4 * 4;
  q.in_sb = (long long)p.nix * q.niy;
  q.in_sn = (long long)p.B * p.nix * q.niy;
  return q;
}

}  // namespace

size_t direct_repitch_workspace_bytes(const DirectProblem<float> &p) {
  if (!tensor_cores_enabled() || p.accumulate || p.niy % 4 == 0 || p.niy < 1 || p.A <= 4) return 0;
  const size_t tc = direct_tc_workspace_bytes(padded_direct(p, nullptr));
  if (tc == 0) return 0;
  return round256((size_t)p.N * p.B * p.nix * ((p.niy + 3) / 4 * 4) * sizeof(float)) + tc;
}

// forward / grad-input on tensor cores for inputs whose linear extent is not a multiple of 4
int launch_direct_repitched(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes,
                            cudaStream_t stream) {
  const size_t need = direct_repitch_workspace_bytes(p);
  if (need == 0 || !dense_input(p) || workspace == nullptr || workspace_bytes < need ||
      reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return MELLIN_ERR_UNSUPPORTED;
  const int pitch = (p.niy + 3) / 4 * 4;
  float *xp = static_cast<float *>(workspace);
  const size_t xp_bytes = round256((size_t)p.N * p.B * p.nix * pitch * sizeof(float));
  const int rc = repitch(p.in, (long long)p.N * p.B * p.nix, p.niy, pitch, xp, stream);
  if (rc) return rc;
  return launch_direct_tc(padded_direct(p, xp), static_cast<unsigned char *>(workspace) + xp_bytes,
                          workspace_bytes - xp_bytes, stream);
}

}  // namespace mellin
