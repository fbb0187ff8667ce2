// CUDA kernels (sm_100a) for the Mellin / linear correlation family and their
// host-side launch planning.
//
// Kernel inventory
//   direct_tile_kernel    forward, grad-input and the operator-level entry
//                         points when the linear axis is long and its index
//                         map is affine (divisor 1): input rows selected by
//                         the Mellin table are staged in shared memory as
//                         contiguous segments of the linear axis, the weight
//                         slab next to them, and every thread keeps an
//                         RA x (RYG*4) register tile.
//   gradw_tile_kernel     weight (+ bias) gradient: a warp's lanes split the
//                         linear axis, each thread keeps an RM x RN x NKY
//                         register tile, lanes are combined with warp
//                         shuffles, blocks write partial sums that a second
//                         deterministic pass adds up (no float atomics).
//   direct_generic_kernel / gradw_generic_kernel / bias_generic_kernel
//                         any element type, any divisor, any extent: one
//                         thread (warp) per output element walking the same
//                         tables.  They serve float64 (gradient checks), the
//                         1-D Mellin operators and non-affine linear maps.
//   spec2col_kernel / col2spec_kernel
//                         gather to / adjoint gather from column form.
#include <algorithm>
#include <cstdio>
#include <string>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"

namespace mellin {

namespace {

constexpr int kMaxThreads = 256;

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int round_up(int a, int b) { return ceil_div(a, b) * b; }

int check_launch(const char *what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return fail(MELLIN_ERR_LAUNCH, std::string(what) + ": " + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

// ============================================================================
// generic kernels
// ============================================================================

template <typename T>
__global__ void direct_generic_kernel(const DirectProblem<T> p, const long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int oy = (int)(i % p.noy);
    long long r = i / p.noy;
    const int ox = (int)(r % p.nox);
    r /= p.nox;
    const int a = (int)(r % p.A);
    const int n = (int)(r / p.A);
    const T *in_n = p.in + n * p.in_sn;
    const T *w_a = p.w + a * p.w_sa;
    T acc = 0;
    const int e1 = p.table.row_ptr[ox + 1];
    for (int e = p.table.row_ptr[ox]; e < e1; ++e) {
      const int2 en = p.table.entries[e];
      for (int ky = 0; ky < p.nky; ++ky) {
        const int num = p.Ay * oy + p.By * ky + p.Cy;
        if (num % p.Dy) continue;
        const int iy = num / p.Dy;
        if (iy < 0 || iy >= p.niy) continue;
        const T *wp = w_a + en.x * p.nky + ky;
        const T *ip = in_n + (long long)en.y * p.niy + iy;
        for (int b = 0; b < p.B; ++b) acc += wp[b * p.w_sb] * ip[b * p.in_sb];
      }
    }
    T *o = p.out + n * p.out_sn + a * p.out_sa + (long long)ox * p.noy + oy;
    const T init = p.accumulate ? *o : (p.bias != nullptr ? p.bias[a] : T(0));
    *o = init + acc;
  }
}

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// one warp per weight element
template <typename T>
__global__ void gradw_generic_kernel(const GradWProblem<T> p, const long long total) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = warp0; i < total; i += nwarps) {
    const int ky = (int)(i % p.nky);
    long long r = i / p.nky;
    const int kx = (int)(r % p.nkx);
    r /= p.nkx;
    const int b = (int)(r % p.B);
    const int a = (int)(r / p.B);
    T acc = 0;
    const int e0 = p.table.row_ptr[kx], e1 = p.table.row_ptr[kx + 1];
    for (int n = 0; n < p.N; ++n) {
      for (int e = e0; e < e1; ++e) {
        const int2 en = p.table.entries[e];
        if (en.x & kFlagBiasOnly) continue;
        const int ox = en.x & kIndexMask;
        const T *go = p.go + (((long long)n * p.A + a) * p.nox + ox) * p.noy;
        const T *in = p.in + (((long long)n * p.B + b) * p.nix + en.y) * p.niy;
        for (int oy = lane; oy < p.noy; oy += 32) {
          const int num = p.Ay * oy + p.By * ky + p.Cy;
          if (num % p.Dy) continue;
          const int iy = num / p.Dy;
          if (iy < 0 || iy >= p.niy) continue;
          acc += go[oy] * in[iy];
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) p.gw[i] = acc;
  }
}

// one warp per output channel
template <typename T>
__global__ void bias_generic_kernel(const T *go, T *gb, int N, int A, long long plane) {
  const int lane = threadIdx.x & 31;
  const int a = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5);
  if (a >= A) return;
  T acc = 0;
  for (int n = 0; n < N; ++n) {
    const T *src = go + ((long long)n * A + a) * plane;
    for (long long i = lane; i < plane; i += 32) acc += src[i];
  }
  acc = warp_sum(acc);
  if (lane == 0) gb[a] = acc;
}

// ============================================================================
// direct tile kernel (float)
// ============================================================================

struct DirectTiling {
  int TA = 0;          // output channels per block
  int TB = 0;          // reduced channels staged per chunk
  int KS = 1;          // thread groups splitting the reduced channels
  int ty_threads = 0;  // threads along the linear axis
  int y_tiles = 0, a_tiles = 0;
  int XW = 0;          // staged row width (floats)
  int MP = 0;          // longest Mellin table row
  int pair_bytes = 0;
  int vec_store = 0;
  int threads = 0;
  size_t smem = 0;
};

// RA  : output channels per thread
// RYG : groups of 4 consecutive linear-axis positions per thread
// NKY : linear taps when the map is "unit" (Ay = 1, |By| = 1); 0 selects the
//       run-time path for any Ay, By, nky
template <int RA, int RYG, int NKY>
__global__ void __launch_bounds__(kMaxThreads)
direct_tile_kernel(const DirectProblem<float> p, const DirectTiling t) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int2 *pair_s = reinterpret_cast<int2 *>(smem_raw);
  float *Xs = reinterpret_cast<float *>(smem_raw + t.pair_bytes);
  float *Ws = Xs + t.TB * t.MP * t.XW;

  int bid = blockIdx.x;
  const int at = bid % t.a_tiles;
  bid /= t.a_tiles;
  const int yt = bid % t.y_tiles;
  bid /= t.y_tiles;
  const int ox = bid % p.nox;
  const int n = bid / p.nox;

  const int TY = t.ty_threads * 4 * RYG;
  const int y0 = yt * TY, a0 = at * t.TA;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  const int agroups = t.TA / RA;
  const int group_threads = t.ty_threads * agroups;
  const int ty = tid % t.ty_threads;
  const int ta = (tid / t.ty_threads) % agroups;
  const int ks = tid / group_threads;
  const bool active = ks < t.KS;
  const int nky = NKY > 0 ? NKY : p.nky;
  const int absBy = p.By < 0 ? -p.By : p.By;

  const int e0 = p.table.row_ptr[ox];
  const int np = p.table.row_ptr[ox + 1] - e0;
  for (int i = tid; i < np; i += blockDim.x) pair_s[i] = p.table.entries[e0 + i];

  // shared column c of a staged row holds input position ws + c
  const int ws = p.Ay * y0 + p.Cy + min(0, p.By * (nky - 1));

  float acc[RA][RYG][4];
#pragma unroll
  for (int r = 0; r < RA; ++r)
#pragma unroll
    for (int g = 0; g < RYG; ++g)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[r][g][j] = 0.f;

  for (int b0 = 0; b0 < p.B; b0 += t.TB) {
    const int tb = min(t.TB, p.B - b0);
    const int nrows = tb * np;
    __syncthreads();
    for (int row = warp; row < nrows; row += nwarps) {
      const int bb = row / np, pp = row - bb * np;
      const int2 pr = pair_s[pp];
      const float *src = p.in + n * p.in_sn + (b0 + bb) * p.in_sb + (long long)pr.y * p.niy;
      float *dst = Xs + (bb * t.MP + pp) * t.XW;
      for (int c = lane; c < t.XW; c += 32) {
        const int iy = ws + c;
        dst[c] = (iy >= 0 && iy < p.niy) ? __ldg(src + iy) : 0.f;
      }
      // weights of this (channel, tap row): slot tt holds the tap whose input
      // offset is tt * |By| above the window start, so the inner loop never
      // needs the sign of By
      const float *wsrc = p.w + (b0 + bb) * p.w_sb + pr.x * nky;
      float *wdst = Ws + (bb * t.MP + pp) * nky * t.TA;
      for (int e = lane; e < nky * t.TA; e += 32) {
        const int tt = e / t.TA, aa = e - tt * t.TA;
        const int ky = p.By < 0 ? nky - 1 - tt : tt;
        const int a = a0 + aa;
        wdst[e] = a < p.A ? __ldg(wsrc + a * p.w_sa + ky) : 0.f;
      }
    }
    __syncthreads();
    if (!active) continue;
    for (int bb = ks; bb < tb; bb += t.KS) {
      for (int pp = 0; pp < np; ++pp) {
        const float *xrow = Xs + (bb * t.MP + pp) * t.XW;
        const float *wrow = Ws + (bb * t.MP + pp) * nky * t.TA + ta * RA;
        if (NKY > 0) {
          float xw[RYG][8];
#pragma unroll
          for (int g = 0; g < RYG; ++g) {
            const float4 *q = reinterpret_cast<const float4 *>(xrow + (g * t.ty_threads + ty) * 4);
            const float4 v0 = q[0];
            xw[g][0] = v0.x, xw[g][1] = v0.y, xw[g][2] = v0.z, xw[g][3] = v0.w;
            if (NKY > 1) {
              const float4 v1 = q[1];
              xw[g][4] = v1.x, xw[g][5] = v1.y, xw[g][6] = v1.z, xw[g][7] = v1.w;
            }
          }
#pragma unroll
          for (int tt = 0; tt < (NKY > 0 ? NKY : 1); ++tt) {
            float wv[RA];
#pragma unroll
            for (int r4 = 0; r4 < RA / 4; ++r4) {
              const float4 v = *reinterpret_cast<const float4 *>(wrow + tt * t.TA + 4 * r4);
              wv[4 * r4] = v.x, wv[4 * r4 + 1] = v.y, wv[4 * r4 + 2] = v.z, wv[4 * r4 + 3] = v.w;
            }
#pragma unroll
            for (int r = 0; r < RA; ++r)
#pragma unroll
              for (int g = 0; g < RYG; ++g)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[r][g][j] = fmaf(wv[r], xw[g][j + tt], acc[r][g][j]);
          }
        } else {
          for (int tt = 0; tt < nky; ++tt) {
            float wv[RA];
#pragma unroll
            for (int r4 = 0; r4 < RA / 4; ++r4) {
              const float4 v = *reinterpret_cast<const float4 *>(wrow + tt * t.TA + 4 * r4);
              wv[4 * r4] = v.x, wv[4 * r4 + 1] = v.y, wv[4 * r4 + 2] = v.z, wv[4 * r4 + 3] = v.w;
            }
#pragma unroll
            for (int g = 0; g < RYG; ++g)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float xv = xrow[p.Ay * ((g * t.ty_threads + ty) * 4 + j) + absBy * tt];
#pragma unroll
                for (int r = 0; r < RA; ++r) acc[r][g][j] = fmaf(wv[r], xv, acc[r][g][j]);
              }
          }
        }
      }
    }
  }

  if (t.KS > 1) {
    // combine the channel-split groups through shared memory, value-major so
    // that consecutive threads touch consecutive words
    __syncthreads();
    float *red = Xs;
    const int slot = ta * t.ty_threads + ty;
    if (active && ks > 0) {
      float *dst = red + (ks - 1) * (RA * RYG * 4) * group_threads + slot;
#pragma unroll
      for (int r = 0; r < RA; ++r)
#pragma unroll
        for (int g = 0; g < RYG; ++g)
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[((r * RYG + g) * 4 + j) * group_threads] = acc[r][g][j];
    }
    __syncthreads();
    if (active && ks == 0) {
      for (int k = 1; k < t.KS; ++k) {
        const float *src = red + (k - 1) * (RA * RYG * 4) * group_threads + slot;
#pragma unroll
        for (int r = 0; r < RA; ++r)
#pragma unroll
          for (int g = 0; g < RYG; ++g)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[r][g][j] += src[((r * RYG + g) * 4 + j) * group_threads];
      }
    }
  }

  if (!active || ks != 0) return;
#pragma unroll
  for (int r = 0; r < RA; ++r) {
    const int a = a0 + ta * RA + r;
    if (a >= p.A) continue;
    const float bias = (!p.accumulate && p.bias != nullptr) ? __ldg(p.bias + a) : 0.f;
    float *orow = p.out + n * p.out_sn + a * p.out_sa + (long long)ox * p.noy;
#pragma unroll
    for (int g = 0; g < RYG; ++g) {
      const int y = y0 + (g * t.ty_threads + ty) * 4;
      if (t.vec_store && y + 3 < p.noy) {
        float4 v = make_float4(acc[r][g][0], acc[r][g][1], acc[r][g][2], acc[r][g][3]);
        float4 *o = reinterpret_cast<float4 *>(orow + y);
        if (p.accumulate) {
          const float4 old = *o;
          v.x += old.x, v.y += old.y, v.z += old.z, v.w += old.w;
        } else {
          v.x += bias, v.y += bias, v.z += bias, v.w += bias;
        }
        *o = v;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (y + j < p.noy) orow[y + j] = (p.accumulate ? orow[y + j] : bias) + acc[r][g][j];
      }
    }
  }
}

bool plan_direct(const DirectProblem<float> &p, DirectTiling &t, int &RA, int &RYG, int &NKY) {
  if (p.Dy != 1 || p.noy < 16 || p.nky < 1 || p.nox < 1) return false;
  RA = p.A <= 4 ? 4 : 8;
  t.TA = RA == 4 ? 4 : std::min(64, round_up(p.A, 8));
  const int agroups = t.TA / RA;
  RYG = agroups >= 4 ? 1 : 2;
  const int quads = ceil_div(p.noy, 4 * RYG);
  const int max_ty = std::max(1, std::min(32, kMaxThreads / agroups));
  t.y_tiles = ceil_div(quads, max_ty);
  t.ty_threads = ceil_div(quads, t.y_tiles);
  t.a_tiles = ceil_div(p.A, t.TA);
  const int group_threads = t.ty_threads * agroups;
  t.KS = 1;
  while (t.KS * 2 * group_threads <= kMaxThreads && t.KS * 2 <= std::min(8, p.B)) t.KS *= 2;
  t.threads = std::min(kMaxThreads, round_up(group_threads * t.KS, 32));
  const bool unit = p.Ay == 1 && (p.nky == 1 || p.By == 1 || p.By == -1) && p.nky <= 5;
  NKY = unit ? p.nky : 0;
  const int absBy = p.By < 0 ? -p.By : p.By;
  const int TY = t.ty_threads * 4 * RYG;
  t.XW = round_up(p.Ay * (TY - 1) + absBy * (p.nky - 1) + 1, 4) + 4;
  t.MP = std::max(1, (int)p.table.max_row);
  t.pair_bytes = round_up(t.MP * (int)sizeof(int2), 16);
  const size_t per_b = (size_t)t.MP * (t.XW + (size_t)p.nky * t.TA) * sizeof(float);
  const size_t budget = 56 * 1024;
  int tb = (int)std::min<size_t>(p.B, std::max<size_t>(1, budget / per_b));
  tb = std::max(t.KS, tb / t.KS * t.KS);
  t.TB = tb;
  size_t tile_bytes = per_b * t.TB;
  const size_t red_bytes = (size_t)(t.KS - 1) * group_threads * RA * RYG * 4 * sizeof(float);
  tile_bytes = std::max(tile_bytes, red_bytes);
  t.smem = t.pair_bytes + tile_bytes;
  if (t.smem > 200 * 1024) return false;
  const bool aligned = (reinterpret_cast<uintptr_t>(p.out) % 16 == 0) && p.noy % 4 == 0 &&
                       p.out_sn % 4 == 0 && p.out_sa % 4 == 0;
  t.vec_store = aligned ? 1 : 0;
  return true;
}

template <int RA, int RYG, int NKY>
int launch_direct_tile(const DirectProblem<float> &p, const DirectTiling &t, cudaStream_t stream) {
  auto kernel = direct_tile_kernel<RA, RYG, NKY>;
  if (t.smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem);
    if (err != cudaSuccess)
      return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  }
  const long long blocks = (long long)p.N * p.nox * t.y_tiles * t.a_tiles;
  if (blocks <= 0) return MELLIN_OK;
  if (blocks > 0x7fffffffLL) return fail(MELLIN_ERR_UNSUPPORTED, "too many blocks for the tile kernel");
  kernel<<<(unsigned)blocks, t.threads, t.smem, stream>>>(p, t);
  return check_launch("direct_tile_kernel");
}

template <int RA, int RYG>
int dispatch_direct_nky(const DirectProblem<float> &p, const DirectTiling &t, int NKY, cudaStream_t stream) {
  switch (NKY) {
    case 1: return launch_direct_tile<RA, RYG, 1>(p, t, stream);
    case 2: return launch_direct_tile<RA, RYG, 2>(p, t, stream);
    case 3: return launch_direct_tile<RA, RYG, 3>(p, t, stream);
    case 4: return launch_direct_tile<RA, RYG, 4>(p, t, stream);
    case 5: return launch_direct_tile<RA, RYG, 5>(p, t, stream);
    default: return launch_direct_tile<RA, RYG, 0>(p, t, stream);
  }
}

template <typename T>
int launch_direct_generic(const DirectProblem<T> &p, cudaStream_t stream) {
  const long long total = (long long)p.N * p.A * p.nox * p.noy;
  if (total <= 0) return MELLIN_OK;
  const int threads = 128;
  const long long blocks = std::min<long long>((total + threads - 1) / threads, (long long)sm_count() * 64);
  direct_generic_kernel<T><<<(unsigned)blocks, threads, 0, stream>>>(p, total);
  return check_launch("direct_generic_kernel");
}

// ============================================================================
// weight-gradient tile kernel (float)
// ============================================================================

struct GradWTiling {
  int TM = 0, TN = 0;        // output / input channels per block
  int warps_a = 0, warps_b = 0;
  int TKQ = 0;               // quads (4 positions) of the linear axis per tile
  int TKW = 0;               // staged input row width
  int y_tiles = 0, items = 0;  // items = N * y_tiles
  int Z = 0;                 // blocks splitting the items
  int a_tiles = 0, b_tiles = 0;
  int vec_go = 0;
  size_t smem = 0;
};

template <int RM, int RN, int NKY>
__global__ void __launch_bounds__(kMaxThreads)
gradw_tile_kernel(const GradWProblem<float> p, const GradWTiling t, float *__restrict__ part_w,
                  float *__restrict__ part_b) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int TK = 4 * t.TKQ;
  float *GOs = reinterpret_cast<float *>(smem_raw);
  float *INs = GOs + t.TM * TK;

  int bid = blockIdx.x;
  const int z = bid % t.Z;
  bid /= t.Z;
  const int bt = bid % t.b_tiles;
  bid /= t.b_tiles;
  const int at = bid % t.a_tiles;
  const int krow = bid / t.a_tiles;          // position in the heaviest-first order
  const int kx = p.table.order[krow];
  const int e0 = p.table.row_ptr[kx];
  const int ne = p.table.row_ptr[kx + 1] - e0;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  const int wa = warp % t.warps_a, wb = warp / t.warps_a;
  const bool want_bias = part_b != nullptr && bt == 0;
  const bool bias_warp = want_bias && wb == 0;
  const int ws_off = p.Cy + min(0, p.By * (NKY - 1));  // Ay == 1 here

  float acc[RM][RN][NKY];
  float bsum[RM];
#pragma unroll
  for (int r = 0; r < RM; ++r) {
    bsum[r] = 0.f;
#pragma unroll
    for (int c = 0; c < RN; ++c)
#pragma unroll
      for (int k = 0; k < NKY; ++k) acc[r][c][k] = 0.f;
  }

  for (int item = z; item < t.items; item += t.Z) {
    const int n = item / t.y_tiles;
    const int y0 = (item - n * t.y_tiles) * TK;
    for (int e = 0; e < ne; ++e) {
      const int2 en = p.table.entries[e0 + e];
      const bool only_bias = (en.x & kFlagBiasOnly) != 0;
      const bool owner = (en.x & kFlagBiasOwner) != 0;
      if (only_bias && !want_bias) continue;
      const int ox = en.x & kIndexMask;
      __syncthreads();
      for (int row = warp; row < t.TM; row += nwarps) {
        const int a = at * t.TM + row;
        float *dst = GOs + row * TK;
        const float *src = p.go + (((long long)n * p.A + a) * p.nox + ox) * p.noy;
        if (t.vec_go) {
          for (int q = lane; q < t.TKQ; q += 32) {
            const int y = y0 + 4 * q;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a < p.A && y < p.noy) v = __ldg(reinterpret_cast<const float4 *>(src + y));
            *reinterpret_cast<float4 *>(dst + 4 * q) = v;
          }
        } else {
          for (int c = lane; c < TK; c += 32) {
            const int y = y0 + c;
            dst[c] = (a < p.A && y < p.noy) ? __ldg(src + y) : 0.f;
          }
        }
      }
      if (!only_bias) {
        const int ws = y0 + ws_off;
        for (int row = warp; row < t.TN; row += nwarps) {
          const int b = bt * t.TN + row;
          float *dst = INs + row * t.TKW;
          const float *src = p.in + (((long long)n * p.B + b) * p.nix + en.y) * p.niy;
          for (int c = lane; c < t.TKW; c += 32) {
            const int iy = ws + c;
            dst[c] = (b < p.B && iy >= 0 && iy < p.niy) ? __ldg(src + iy) : 0.f;
          }
        }
      }
      __syncthreads();
      for (int q = lane; q < t.TKQ; q += 32) {
        float4 g4[RM];
#pragma unroll
        for (int r = 0; r < RM; ++r)
          g4[r] = *reinterpret_cast<const float4 *>(GOs + (wa * RM + r) * TK + 4 * q);
        if (bias_warp && owner) {
#pragma unroll
          for (int r = 0; r < RM; ++r) bsum[r] += (g4[r].x + g4[r].y) + (g4[r].z + g4[r].w);
        }
        if (only_bias) continue;
#pragma unroll
        for (int c = 0; c < RN; ++c) {
          float xw[8];
          const float4 *xp = reinterpret_cast<const float4 *>(INs + (wb * RN + c) * t.TKW + 4 * q);
          const float4 v0 = xp[0];
          xw[0] = v0.x, xw[1] = v0.y, xw[2] = v0.z, xw[3] = v0.w;
          if (NKY > 1) {
            const float4 v1 = xp[1];
            xw[4] = v1.x, xw[5] = v1.y, xw[6] = v1.z, xw[7] = v1.w;
          }
#pragma unroll
          for (int r = 0; r < RM; ++r)
#pragma unroll
            for (int k = 0; k < NKY; ++k) {
              float s = acc[r][c][k];
              s = fmaf(g4[r].x, xw[k], s);
              s = fmaf(g4[r].y, xw[k + 1], s);
              s = fmaf(g4[r].z, xw[k + 2], s);
              s = fmaf(g4[r].w, xw[k + 3], s);
              acc[r][c][k] = s;
            }
        }
      }
    }
  }

  // lanes hold disjoint slices of the linear axis: butterfly-sum them, then
  // spread the stores over the lanes
  const long long gw_elems = (long long)p.A * p.B * p.nkx * p.nky;
  float *pw = part_w + (long long)z * gw_elems;
#pragma unroll
  for (int r = 0; r < RM; ++r)
#pragma unroll
    for (int c = 0; c < RN; ++c)
#pragma unroll
      for (int k = 0; k < NKY; ++k) {
        const float s = warp_sum(acc[r][c][k]);
        const int idx = (r * RN + c) * NKY + k;
        if (lane == (idx & 31)) {
          const int a = at * t.TM + wa * RM + r;
          const int b = bt * t.TN + wb * RN + c;
          const int ky = p.By < 0 ? NKY - 1 - k : k;
          if (a < p.A && b < p.B && wb < t.warps_b)
            pw[(((long long)a * p.B + b) * p.nkx + kx) * p.nky + ky] = s;
        }
      }
  if (bias_warp) {
#pragma unroll
    for (int r = 0; r < RM; ++r) {
      const float s = warp_sum(bsum[r]);
      const int a = at * t.TM + wa * RM + r;
      if (lane == r && a < p.A) part_b[((long long)krow * t.Z + z) * p.A + a] = s;
    }
  }
}

// out[i] = sum over slices of part[slice][i].  A block owns 32 outputs; its 8
// warps split the slices and are combined in a fixed order through shared
// memory, so the result does not depend on scheduling.
template <typename T>
__global__ void reduce_partials_kernel(const T *__restrict__ part, T *__restrict__ out, long long count,
                                       int slices, long long slice_stride) {
  __shared__ T red[8][33];
  const int lane = threadIdx.x & 31, zs = threadIdx.x >> 5;
  const long long i = blockIdx.x * 32LL + lane;
  T s = 0;
  if (i < count)
    for (int z = zs; z < slices; z += 8) s += part[z * slice_stride + i];
  red[zs][lane] = s;
  __syncthreads();
  if (zs == 0 && i < count) {
    T t = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][lane];
    out[i] = t;
  }
}

// The same for the weight sums and the bias sums of one launch together: blocks [0, w_blocks) own weights,
// the rest own bias entries.  Four running sums per thread keep the loads independent.
template <typename T>
__global__ void reduce_partials_pair_kernel(const T *__restrict__ part_w, T *__restrict__ out_w, long long count_w,
                                            const T *__restrict__ part_b, T *__restrict__ out_b, long long count_b,
                                            int slices, long long w_blocks) {
  __shared__ T red[8][33];
  const int lane = threadIdx.x & 31, zs = threadIdx.x >> 5;
  const bool weights = (long long)blockIdx.x < w_blocks;
  const T *__restrict__ part = weights ? part_w : part_b;
  const long long count = weights ? count_w : count_b;
  const long long i = (weights ? blockIdx.x : blockIdx.x - w_blocks) * 32LL + lane;
  T s0 = 0, s1 = 0, s2 = 0, s3 = 0;
  if (i < count) {
    int z = zs;
    for (; z + 24 < slices; z += 32) {
      s0 += part[z * count + i];
      s1 += part[(z + 8) * count + i];
      s2 += part[(z + 16) * count + i];
      s3 += part[(z + 24) * count + i];
    }
    for (; z < slices; z += 8) s0 += part[z * count + i];
  }
  red[zs][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (zs == 0 && i < count) {
    T t = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][lane];
    (weights ? out_w : out_b)[i] = t;
  }
}

bool plan_gradw(const GradWProblem<float> &p, GradWTiling &t, int &RM, int &RN) {
  if (p.Dy != 1 || p.Ay != 1 || p.noy < 16) return false;
  if (!(p.nky >= 1 && p.nky <= 5)) return false;
  if (p.nky > 1 && p.By != 1 && p.By != -1) return false;
  RM = p.A <= 4 ? 4 : 8;
  RN = std::min(4, p.B);
  if (RM * RN * p.nky > 96) RN = std::max(1, 96 / (RM * p.nky));
  t.warps_a = std::min(8, ceil_div(p.A, RM));
  t.warps_b = std::max(1, std::min(8 / t.warps_a, ceil_div(p.B, RN)));
  t.TM = t.warps_a * RM;
  t.TN = t.warps_b * RN;
  t.a_tiles = ceil_div(p.A, t.TM);
  t.b_tiles = ceil_div(p.B, t.TN);
  const int quads = ceil_div(p.noy, 4);
  t.y_tiles = ceil_div(quads, 32);
  t.TKQ = ceil_div(quads, t.y_tiles);
  t.TKW = 4 * t.TKQ + 8;
  t.items = p.N * t.y_tiles;
  const long long column_blocks = (long long)p.nkx * t.a_tiles * t.b_tiles;
  const long long want = 4LL * sm_count();
  t.Z = (int)std::max<long long>(1, std::min<long long>(t.items, (want + column_blocks - 1) / column_blocks));
  t.smem = ((size_t)t.TM * 4 * t.TKQ + (size_t)t.TN * t.TKW) * sizeof(float);
  t.vec_go = (reinterpret_cast<uintptr_t>(p.go) % 16 == 0 && p.noy % 4 == 0) ? 1 : 0;
  return t.smem <= 200 * 1024;
}

template <int RM, int RN, int NKY>
int launch_gradw_tile(const GradWProblem<float> &p, const GradWTiling &t, float *part_w, float *part_b,
                      cudaStream_t stream) {
  auto kernel = gradw_tile_kernel<RM, RN, NKY>;
  if (t.smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem);
    if (err != cudaSuccess)
      return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  }
  const long long blocks = (long long)p.nkx * t.a_tiles * t.b_tiles * t.Z;
  const int threads = 32 * t.warps_a * t.warps_b;
  kernel<<<(unsigned)blocks, threads, t.smem, stream>>>(p, t, part_w, part_b);
  return check_launch("gradw_tile_kernel");
}

template <int RM, int RN>
int dispatch_gradw_nky(const GradWProblem<float> &p, const GradWTiling &t, float *pw, float *pb, cudaStream_t s) {
  switch (p.nky) {
    case 1: return launch_gradw_tile<RM, RN, 1>(p, t, pw, pb, s);
    case 2: return launch_gradw_tile<RM, RN, 2>(p, t, pw, pb, s);
    case 3: return launch_gradw_tile<RM, RN, 3>(p, t, pw, pb, s);
    case 4: return launch_gradw_tile<RM, RN, 4>(p, t, pw, pb, s);
    default: return launch_gradw_tile<RM, RN, 5>(p, t, pw, pb, s);
  }
}

template <int RM>
int dispatch_gradw_rn(const GradWProblem<float> &p, const GradWTiling &t, int RN, float *pw, float *pb,
                      cudaStream_t s) {
  switch (RN) {
    case 1: return dispatch_gradw_nky<RM, 1>(p, t, pw, pb, s);
    case 2: return dispatch_gradw_nky<RM, 2>(p, t, pw, pb, s);
    case 3: return dispatch_gradw_nky<RM, 3>(p, t, pw, pb, s);
    default: return dispatch_gradw_nky<RM, 4>(p, t, pw, pb, s);
  }
}

size_t gradw_partial_floats(const GradWProblem<float> &p, const GradWTiling &t, size_t *bias_offset) {
  const size_t gw = (size_t)p.A * p.B * p.nkx * p.nky;
  size_t w_part = (size_t)t.Z * gw;
  w_part = (w_part + 63) / 64 * 64;
  if (bias_offset) *bias_offset = w_part;
  return w_part + (size_t)p.nkx * t.Z * p.A;
}

template <typename T>
int launch_gradw_generic(const GradWProblem<T> &p, cudaStream_t stream) {
  const long long total = (long long)p.A * p.B * p.nkx * p.nky;
  if (total > 0) {
    const int threads = 128;
    const long long blocks = std::min<long long>((total * 32 + threads - 1) / threads, (long long)sm_count() * 32);
    gradw_generic_kernel<T><<<(unsigned)blocks, threads, 0, stream>>>(p, total);
    int rc = check_launch("gradw_generic_kernel");
    if (rc) return rc;
  }
  if (p.gb != nullptr && p.A > 0) {
    const int threads = 128;
    const int blocks = ceil_div(p.A * 32, threads);
    bias_generic_kernel<T><<<blocks, threads, 0, stream>>>(p.go, p.gb, p.N, p.A, (long long)p.nox * p.noy);
    return check_launch("bias_generic_kernel");
  }
  return MELLIN_OK;
}

// ============================================================================
// column kernels
// ============================================================================

template <typename T>
__global__ void spec2col_kernel(const ColProblem<T> p, const long long total) {
  const int P = p.px + 1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ggy = (int)(i % p.nggy);
    long long r = i / p.nggy;
    const int ggx = (int)(r % p.nggx);
    r /= p.nggx;
    const int fy = (int)(r % p.nfy);
    r /= p.nfy;
    const int fx = (int)(r % p.nfx);
    r /= p.nfx;
    const int c = p.transposed_gg ? (int)(r / p.N) : (int)(r % p.C);
    const int n = p.transposed_gg ? (int)(r % p.N) : (int)(r / p.C);
    T val = 0;
    const long long numx = (long long)(p.sx + ggx) * (fx + p.dx);
    const int numy = p.sy * ggy + p.dy * fy - p.py;
    if (numx % P == 0 && numy % p.uy == 0) {
      const long long gx = numx / P - p.ux;
      const int gy = numy / p.uy;
      if (gx >= 0 && gx < p.ngx && gy >= 0 && gy < p.ngy) {
        const long long plane = p.transposed_g ? (long long)c * p.N + n : (long long)n * p.C + c;
        val = p.src[(plane * p.ngx + gx) * p.ngy + gy];
      }
    }
    p.dst[i] = val;
  }
}

template <typename T>
__global__ void col2spec_kernel(const ColProblem<T> p, const long long total) {
  const int P = p.px + 1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int gy = (int)(i % p.ngy);
    long long r = i / p.ngy;
    const int gx = (int)(r % p.ngx);
    r /= p.ngx;
    const int c = p.transposed_g ? (int)(r / p.N) : (int)(r % p.C);
    const int n = p.transposed_g ? (int)(r % p.N) : (int)(r / p.C);
    const long long plane = p.transposed_gg ? (long long)c * p.N + n : (long long)n * p.C + c;
    const T *src = p.src + plane * p.nfx * p.nfy * p.nggx * p.nggy;
    const long long numx = (long long)P * (gx + p.ux);
    T acc = 0;
    for (int fx = 0; fx < p.nfx; ++fx) {
      const int den = fx + p.dx;
      if (den == 0 || numx % den) continue;
      const long long ggx = numx / den - p.sx;
      if (ggx < 0 || ggx >= p.nggx) continue;
      for (int fy = 0; fy < p.nfy; ++fy) {
        const int numy = p.uy * gy - p.dy * fy + p.py;
        if (numy % p.sy) continue;
        const int ggy = numy / p.sy;
        if (ggy < 0 || ggy >= p.nggy) continue;
        acc += src[(((long long)fx * p.nfy + fy) * p.nggx + ggx) * p.nggy + ggy];
      }
    }
    p.dst[i] = acc;
  }
}

}  // namespace

// ============================================================================
// launchers
// ============================================================================

template <>
int launch_direct<float>(const DirectProblem<float> &p, cudaStream_t stream) {
  DirectTiling t;
  int RA = 0, RYG = 0, NKY = 0;
  if (!plan_direct(p, t, RA, RYG, NKY)) return launch_direct_generic<float>(p, stream);
  if (RA == 4) {
    return RYG == 1 ? dispatch_direct_nky<4, 1>(p, t, NKY, stream) : dispatch_direct_nky<4, 2>(p, t, NKY, stream);
  }
  return RYG == 1 ? dispatch_direct_nky<8, 1>(p, t, NKY, stream) : dispatch_direct_nky<8, 2>(p, t, NKY, stream);
}

template <>
int launch_direct<double>(const DirectProblem<double> &p, cudaStream_t stream) {
  return launch_direct_generic<double>(p, stream);
}

template <>
size_t gradw_workspace_bytes<float>(const GradWProblem<float> &p) {
  const size_t rows = std::max(std::max(std::max(gradw_rows_workspace_floats(p, nullptr), tc_gradw_few_in_workspace_floats(p)),
                                        gradw_tc_workspace_floats(p, nullptr)) * sizeof(float),
                               std::max(gradw_batch_inner_workspace_bytes(p), gradw_repitch_workspace_bytes(p)));
  GradWTiling t;
  int RM = 0, RN = 0;
  if (!plan_gradw(p, t, RM, RN)) return rows;
  return std::max(rows, gradw_partial_floats(p, t, nullptr) * sizeof(float));
}

template <>
size_t gradw_workspace_bytes<double>(const GradWProblem<double> &) {
  return 0;
}

template <>
int launch_gradw<float>(const GradWProblem<float> &p, void *workspace, size_t workspace_bytes,
                        cudaStream_t stream) {
  const long long gw_count = (long long)p.A * p.B * p.nkx * p.nky;
  if (tensor_cores_enabled() && p.B <= 4) {
    // layers with few input channels, on the tensor cores: grad_y read once, operand A in tensor memory
    const int rc = launch_tc_gradw_few_in(p, workspace, workspace_bytes, stream);
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
  }
  {
    // layers with few input channels: the kernel that reads grad_y once
    size_t rows_bias_off = 0;
    const size_t rows_need = gradw_rows_workspace_floats(p, &rows_bias_off) * sizeof(float);
    if (rows_need > 0 && p.table_h.row_ptr != nullptr) {
      if (workspace == nullptr || workspace_bytes < rows_need)
        return fail(MELLIN_ERR_WORKSPACE, "grad_weight workspace too small: need " + std::to_string(rows_need) +
                                              " bytes, got " + std::to_string(workspace_bytes));
      float *pw = static_cast<float *>(workspace);
      float *pb = p.gb != nullptr ? pw + rows_bias_off : nullptr;
      int slices = 0;
      int rc = launch_gradw_rows(p, pw, pb, &slices, stream);
      if (rc != MELLIN_ERR_UNSUPPORTED) {
        if (rc) return rc;
        const long long w_blocks = (gw_count + 31) / 32, b_blocks = p.gb != nullptr ? ceil_div(p.A, 32) : 0;
        reduce_partials_pair_kernel<float><<<(unsigned)(w_blocks + b_blocks), 256, 0, stream>>>(
            pw, p.gw, gw_count, pb, p.gb, p.A, slices, w_blocks);
        return check_launch("reduce_partials_pair_kernel");
      }
    }
  }
  if (tensor_cores_enabled() && p.noy == 1) {
    // wide 1-D Mellin operator: the batch becomes the linear axis
    const int rc = launch_gradw_batch_inner(p, workspace, workspace_bytes, stream);
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
  }
  if (tensor_cores_enabled() && (p.noy % 4 != 0 || p.niy % 4 != 0)) {
    const int rc = launch_gradw_repitched(p, workspace, workspace_bytes, stream);
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
  }
  if (tensor_cores_enabled()) {
    // wide layers: positions are the reduction axis of a tensor-core GEMM
    size_t tc_bias_off = 0;
    const size_t tc_need = gradw_tc_workspace_floats(p, &tc_bias_off) * sizeof(float);
    if (tc_need > 0 && workspace != nullptr && workspace_bytes >= tc_need) {
      float *pw = static_cast<float *>(workspace);
      float *pb = p.gb != nullptr ? pw + tc_bias_off : nullptr;
      const int rc = launch_gradw_tc(p, pw, pb, stream);
      if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
    }
  }
  GradWTiling t;
  int RM = 0, RN = 0;
  if (!plan_gradw(p, t, RM, RN)) return launch_gradw_generic<float>(p, stream);
  size_t bias_off = 0;
  const size_t need = gradw_partial_floats(p, t, &bias_off) * sizeof(float);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(MELLIN_ERR_WORKSPACE, "grad_weight workspace too small: need " + std::to_string(need) +
                                          " bytes, got " + std::to_string(workspace_bytes));
  float *part_w = static_cast<float *>(workspace);
  float *part_b = p.gb != nullptr ? part_w + bias_off : nullptr;
  int rc = RM == 4 ? dispatch_gradw_rn<4>(p, t, RN, part_w, part_b, stream)
                   : dispatch_gradw_rn<8>(p, t, RN, part_w, part_b, stream);
  if (rc) return rc;
  const long long gw_elems = (long long)p.A * p.B * p.nkx * p.nky;
  reduce_partials_kernel<float><<<(unsigned)((gw_elems + 31) / 32), 256, 0, stream>>>(part_w, p.gw, gw_elems, t.Z,
                                                                                     gw_elems);
  rc = check_launch("reduce_partials_kernel");
  if (rc) return rc;
  if (p.gb != nullptr) {
    reduce_partials_kernel<float><<<(unsigned)ceil_div(p.A, 32), 256, 0, stream>>>(part_b, p.gb, p.A,
                                                                                   p.nkx * t.Z, p.A);
    rc = check_launch("reduce_partials_kernel(bias)");
  }
  return rc;
}

template <>
int launch_gradw<double>(const GradWProblem<double> &p, void *, size_t, cudaStream_t stream) {
  return launch_gradw_generic<double>(p, stream);
}

template <typename T>
int launch_spec2col(const ColProblem<T> &p, cudaStream_t stream) {
  const long long total = (long long)p.N * p.C * p.nfx * p.nfy * p.nggx * p.nggy;
  if (total <= 0) return MELLIN_OK;
  const int threads = 256;
  const long long blocks = std::min<long long>((total + threads - 1) / threads, (long long)sm_count() * 32);
  spec2col_kernel<T><<<(unsigned)blocks, threads, 0, stream>>>(p, total);
  return check_launch("spec2col_kernel");
}

template <typename T>
int launch_col2spec(const ColProblem<T> &p, cudaStream_t stream) {
  const long long total = (long long)p.N * p.C * p.ngx * p.ngy;
  if (total <= 0) return MELLIN_OK;
  const int threads = 256;
  const long long blocks = std::min<long long>((total + threads - 1) / threads, (long long)sm_count() * 32);
  col2spec_kernel<T><<<(unsigned)blocks, threads, 0, stream>>>(p, total);
  return check_launch("col2spec_kernel");
}

template int launch_spec2col<float>(const ColProblem<float> &, cudaStream_t);
template int launch_spec2col<double>(const ColProblem<double> &, cudaStream_t);
template int launch_col2spec<float>(const ColProblem<float> &, cudaStream_t);
template int launch_col2spec<double>(const ColProblem<double> &, cudaStream_t);

}  // namespace mellin
