// "Direct" operator for FEW OUTPUT CHANNELS (at most 4) and many reduced
// channels -- the input gradient of a first layer (3 feature maps receive the
// gradient of 64..128), or a forward pass onto a handful of channels:
//
//   out[n, a, ox, oy] = init + sum_{(kx, ix) in row ox} sum_b sum_ky
//                       W[a, b, kx, ky] * in[n, b, ix, oy + By * ky + Cy]
//
// The work is a long reduction over (table entry, b) of rows of `in`; the
// output tile is tiny.  A block owns (n, ox, 256 positions).  Each of its 8
// warps takes every 8th reduced channel and streams "its" rows through a
// private 4-deep cp.async ring -- there is no block-wide barrier in the main
// loop -- while the whole weight set sits in shared memory and is read with
// broadcast loads.  A lane keeps A x 8 running sums (8 consecutive positions);
// the eight warps' partial sums are combined through shared memory at the end.
#include <algorithm>
#include <string>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"

namespace mellin {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRY = 8;                 // positions per lane
constexpr int kTY = 32 * kRY;          // positions per block
constexpr int kRowFloats = kTY + 12;   // staged row: tile + taps (<= 4) + alignment lead (<= 3), multiple of 4
constexpr int kStages = 4;

struct RowsPlan {
  int y_tiles = 0;
  int ws0 = 0;     // first input position of tile 0 relative to its first output position
  int WP = 0;      // floats per (kx, b) weight record: A * NKY rounded up to 4
  int vec_store = 0;
  size_t smem = 0;
};

__device__ __forceinline__ void cp16(void *dst, const void *src, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the destination is zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int A, int NKY>
__global__ void __launch_bounds__(kThreads) direct_rows_kernel(const DirectProblem<float> p, const RowsPlan t) {
  constexpr int AN = A * NKY;
  constexpr int WP = (AN + 3) / 4 * 4;
  constexpr int kWin = kRY + NKY - 1;
  extern __shared__ __align__(16) float smem[];
  float *Ws = smem;                                         // [nkx][B][WP]
  float *ring = smem + (size_t)p.nkx * p.B * WP;            // [warp][stage][kRowFloats]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int bid = blockIdx.x;
  const int yt = bid % t.y_tiles;
  bid /= t.y_tiles;
  const int ox = bid % p.nox;
  const int n = bid / p.nox;
  const int y0 = yt * kTY;

  // ---- weights: record (kx, b) holds W[a, b, kx, .] for all a, taps in increasing input offset
  for (int i = tid; i < p.nkx * p.B * WP; i += kThreads) {
    const int e = i % WP;
    const int rec = i / WP;
    const int b = rec % p.B, kx = rec / p.B;
    float v = 0.f;
    if (e < AN) {
      const int a = e / NKY, k = e % NKY;
      const int ky = p.By < 0 ? NKY - 1 - k : k;
      v = __ldg(p.w + a * p.w_sa + b * p.w_sb + (long long)kx * NKY + ky);
    }
    Ws[i] = v;
  }
  __syncthreads();

  const int e0 = p.table.row_ptr[ox];
  const int np = p.table.row_ptr[ox + 1] - e0;
  const int ws = y0 + t.ws0;
  const int start = ws & ~3;  // 16-byte aligned copy origin (two's complement: floors negatives too)
  const int lead = ws - start;
  float *my_ring = ring + (size_t)warp * kStages * kRowFloats;
  const int per_entry = (p.B - warp + kWarps - 1) / kWarps;  // reduced channels this warp takes per entry
  const int items = per_entry > 0 ? np * per_entry : 0;

  auto issue = [&](int item, int stage) {
    if (item < items) {
      const int pp = item / per_entry;
      const int b = warp + kWarps * (item - pp * per_entry);
      const int ix = p.table.entries[e0 + pp].y;
      const float *row = p.in + n * p.in_sn + b * p.in_sb + (long long)ix * p.niy;
      float *dst = my_ring + stage * kRowFloats;
      for (int c = lane; c < kRowFloats / 4; c += 32) {
        const int iy = start + 4 * c;
        const bool valid = iy >= 0 && iy < p.niy;  // niy and start are multiples of 4: a chunk is in or out as a whole
        cp16(dst + 4 * c, valid ? row + iy : p.in, valid);
      }
    }
    cp_commit();
  };

  float acc[A][kRY];
#pragma unroll
  for (int a = 0; a < A; ++a)
#pragma unroll
    for (int j = 0; j < kRY; ++j) acc[a][j] = 0.f;

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(s, s);
  for (int item = 0; item < items; ++item) {
    issue(item + kStages - 1, (item + kStages - 1) % kStages);
    cp_wait<kStages - 1>();
    __syncwarp();
    const int pp = item / per_entry;
    const int b = warp + kWarps * (item - pp * per_entry);
    const int kx = p.table.entries[e0 + pp].x;
    const float *row = my_ring + (item % kStages) * kRowFloats + lead + kRY * lane;
    float xw[kWin];
#pragma unroll
    for (int j = 0; j < kWin; ++j) xw[j] = row[j];
    const float4 *wrec = reinterpret_cast<const float4 *>(Ws + (size_t)(kx * p.B + b) * WP);
    float wv[WP];
#pragma unroll
    for (int i = 0; i < WP / 4; ++i) {
      const float4 v = wrec[i];
      wv[4 * i] = v.x, wv[4 * i + 1] = v.y, wv[4 * i + 2] = v.z, wv[4 * i + 3] = v.w;
    }
#pragma unroll
    for (int a = 0; a < A; ++a)
#pragma unroll
      for (int k = 0; k < NKY; ++k)
#pragma unroll
        for (int j = 0; j < kRY; ++j) acc[a][j] = fmaf(wv[a * NKY + k], xw[j + k], acc[a][j]);
    __syncwarp();
  }
  cp_wait<0>();
  __syncthreads();

  // ---- combine the warps: red[warp][a][position] -----------------------------------
  float *red = ring;
#pragma unroll
  for (int a = 0; a < A; ++a) {
    float4 *dst = reinterpret_cast<float4 *>(red + ((size_t)warp * A + a) * kTY + kRY * lane);
    dst[0] = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    dst[1] = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
  }
  __syncthreads();
  for (int o = tid; o < A * (kTY / 4); o += kThreads) {
    const int a = o / (kTY / 4), pos = 4 * (o % (kTY / 4));
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float4 v = *reinterpret_cast<const float4 *>(red + ((size_t)w * A + a) * kTY + pos);
      s.x += v.x, s.y += v.y, s.z += v.z, s.w += v.w;
    }
    const int y = y0 + pos;
    if (y >= p.noy) continue;
    float *out = p.out + n * p.out_sn + a * p.out_sa + (long long)ox * p.noy + y;
    const float bias = (!p.accumulate && p.bias != nullptr) ? __ldg(p.bias + a) : 0.f;
    if (t.vec_store && y + 3 < p.noy) {
      float4 *o4 = reinterpret_cast<float4 *>(out);
      if (p.accumulate) {
        const float4 old = *o4;
        s.x += old.x, s.y += old.y, s.z += old.z, s.w += old.w;
      } else {
        s.x += bias, s.y += bias, s.z += bias, s.w += bias;
      }
      *o4 = s;
    } else {
      const float v[4] = {s.x, s.y, s.z, s.w};
      for (int j = 0; j < 4; ++j)
        if (y + j < p.noy) out[j] = (p.accumulate ? out[j] : bias) + v[j];
    }
  }
}

bool plan_rows(const DirectProblem<float> &p, RowsPlan &t) {
  if (p.Dy != 1 || p.Ay != 1) return false;
  if (p.A < 1 || p.A > 4 || p.nky < 1 || p.nky > 3 || p.B < 8) return false;
  if (p.nky > 1 && p.By != 1 && p.By != -1) return false;
  if (p.noy < 64 || p.nox < 1 || p.N < 1 || p.nkx < 1) return false;
  // rows are copied in 16-byte chunks
  if (p.niy % 4 != 0 || reinterpret_cast<uintptr_t>(p.in) % 16 != 0 || p.in_sn % 4 != 0 || p.in_sb % 4 != 0)
    return false;
  t.y_tiles = (p.noy + kTY - 1) / kTY;
  if ((long long)p.N * p.nox * t.y_tiles >= (1LL << 31)) return false;
  t.ws0 = p.Cy + std::min(0, p.By * (p.nky - 1));
  t.WP = (p.A * p.nky + 3) / 4 * 4;
  const size_t w_floats = (size_t)p.nkx * p.B * t.WP;
  const size_t ring_floats = (size_t)kWarps * kStages * kRowFloats;
  const size_t red_floats = (size_t)kWarps * p.A * kTY;
  t.smem = (w_floats + std::max(ring_floats, red_floats)) * sizeof(float);
  if (t.smem > 100 * 1024) return false;
  t.vec_store = (reinterpret_cast<uintptr_t>(p.out) % 16 == 0 && p.noy % 4 == 0 && p.out_sn % 4 == 0 &&
                 p.out_sa % 4 == 0)
                    ? 1
                    : 0;
  return true;
}

template <int A>
int dispatch_nky(const DirectProblem<float> &p, const RowsPlan &t, cudaStream_t stream) {
  void (*kernel)(DirectProblem<float>, RowsPlan) = nullptr;
  switch (p.nky) {
    case 1: kernel = direct_rows_kernel<A, 1>; break;
    case 2: kernel = direct_rows_kernel<A, 2>; break;
    default: kernel = direct_rows_kernel<A, 3>; break;
  }
  if (t.smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem);
    if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  }
  const unsigned blocks = (unsigned)((long long)p.N * p.nox * t.y_tiles);
  kernel<<<blocks, kThreads, t.smem, stream>>>(p, t);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("direct_rows_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

}  // namespace

// MELLIN_ERR_UNSUPPORTED when the problem is outside this kernel's coverage.
int launch_direct_rows(const DirectProblem<float> &p, cudaStream_t stream) {
  RowsPlan t;
  if (!plan_rows(p, t)) return MELLIN_ERR_UNSUPPORTED;
  switch (p.A) {
    case 1: return dispatch_nky<1>(p, t, stream);
    case 2: return dispatch_nky<2>(p, t, stream);
    case 3: return dispatch_nky<3>(p, t, stream);
    default: return dispatch_nky<4>(p, t, stream);
  }
}

}  // namespace mellin
