// "Direct" operator for FEW OUTPUT CHANNELS (at most 4) and many reduced
// channels -- the input gradient of a first layer (3 feature maps receive the
// gradient of 64..128), or a forward pass onto a handful of channels:
//
//   out[n, a, ox, oy] = init + sum_{(kx, ix) in row ox} sum_b sum_ky
//                       W[a, b, kx, ky] * in[n, b, ix, oy + By * ky + Cy]
//
// The work is a long reduction over (table entry, b) of rows of `in`; the
// output tile is tiny.  A block owns (n, ox, 240 positions).  Each of its 8
// warps takes every 8th group of 4 reduced channels and streams "its" rows through a
// private ring filled by TMA box loads of 4 rows each (one lane issues, an mbarrier
// per slot signals arrival; positions outside the signal are zero-filled by the
// copy engine) -- there is no block-wide barrier in the main loop -- while the
// whole weight set sits in shared memory and is read with broadcast loads.
// A lane keeps A x 8 running sums (8 consecutive positions);
// the eight warps' partial sums are combined through shared memory at the end.
#include <cuda.h>

#include <algorithm>
#include <string>

#include "../../include/mellin_b200.h"

#include "mellin_internal.h"
#include "tc_ptx.cuh"

namespace mellin {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRY = 8;                 // positions per lane: two groups of 4 consecutive ones, 128 apart
constexpr int kTY = 240;               // output positions per block (a staged row must fit a 256-element TMA box)
constexpr int kRowFloats = 256;        // staged row: 240 positions + taps (<= 4) + tile shift (<= 3), rounded to the box
constexpr int kGroup = 4;              // consecutive reduced channels fetched by one TMA box
constexpr int kSlotFloats = kGroup * kRowFloats;
constexpr int kStages = 2;
constexpr int kRedPitch = 256;
constexpr uint32_t kWaitLimit = 1u << 20;

// First bounded wait that gave up since the last query (0 = none):
// 1 = the weight records never arrived, 2 = a ring slot's rows never arrived.
__device__ int g_direct_rows_error = 0;

struct RowsPlan {
  int y_tiles = 0;
  int ws0 = 0;     // first input position of tile 0 relative to its first output position
  int shift = 0;   // tiles start at output position yt * 240 - shift, which makes (tile start + ws0) a multiple of 4
  int WP = 0;      // floats per (kx, b) weight record: A * NKY rounded up to 4
  int vec_store = 0;
  int w_floats = 0;        // weight records in shared memory, rounded up to 128 bytes
  const float *w_packed = nullptr;  // records pre-packed in global memory (nullptr: gather in the kernel)
  size_t smem = 0;
};

template <int A, int NKY>
__global__ void __launch_bounds__(kThreads)
direct_rows_kernel(const DirectProblem<float> p, const RowsPlan t, const __grid_constant__ CUtensorMap in_map) {
  constexpr int AN = A * NKY;
  constexpr int WP = (AN + 3) / 4 * 4;
  constexpr int kWin = kRY + NKY - 1;
  extern __shared__ __align__(128) float smem[];
  float *Ws = smem;                                         // [nkx][B][WP]
  float *ring = smem + t.w_floats;                          // [warp][stage][kSlotFloats]
  __shared__ uint64_t slot_full[kWarps][kStages];
  __shared__ uint64_t w_full;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int bid = blockIdx.x;
  const int yt = bid % t.y_tiles;
  bid /= t.y_tiles;
  const int ox = bid % p.nox;
  const int n = bid / p.nox;
  const int y0 = yt * kTY - t.shift;  // may be negative for the first tile: those outputs are masked
  const bool second_window = y0 + 128 < p.noy;  // outputs y0 + 128 .. of this tile exist

  if (tid == 0) {
    for (int w = 0; w < kWarps; ++w)
      for (int st = 0; st < kStages; ++st) tc::mbar_init(&slot_full[w][st], 1);
    tc::mbar_init(&w_full, 1);
    tc::fence_mbar_init();
  }
  __syncthreads();
  // ---- weights: record (kx, b) holds W[a, b, kx, .] for all a, taps in increasing input offset
  if (t.w_packed != nullptr) {
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)(p.nkx * p.B * WP) * 4u;
      tc::mbar_arrive_expect_tx(&w_full, bytes);
      tc::bulk_load(Ws, t.w_packed, bytes, &w_full);
    }
  } else {
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
  }

  const int e0 = p.table.row_ptr[ox];
  const int np = p.table.row_ptr[ox + 1] - e0;
  const int start = y0 + t.ws0;  // first staged input position: a multiple of 4 by construction
  float *my_ring = ring + (size_t)warp * kStages * kSlotFloats;
  const int groups = (p.B + kGroup - 1) / kGroup;
  const int per_entry = (groups - warp + kWarps - 1) / kWarps;  // channel groups this warp takes per entry
  const int items = per_entry > 0 ? np * per_entry : 0;

  // issue side: item -> (entry ipp, k-th channel of this warp), advanced incrementally
  int ipp = 0, ik = 0, iix = np > 0 ? p.table.entries[e0].y : 0;
  auto issue = [&](int item) {
    if (item < items && lane == 0) {
      const int stage = item % kStages;
      tc::fence_proxy_async();  // the slot's previous contents were read through the generic proxy
      tc::mbar_arrive_expect_tx(&slot_full[warp][stage], (uint32_t)kSlotFloats * 4u);
      tc::tma_load_4d(my_ring + stage * kSlotFloats, &in_map, start, iix, n, kGroup * (warp + kWarps * ik),
                      &slot_full[warp][stage]);
    }
    if (++ik == per_entry) {
      ik = 0;
      ++ipp;
      if (ipp < np) iix = p.table.entries[e0 + ipp].y;
    }
  };

  float acc[A][kRY];
#pragma unroll
  for (int a = 0; a < A; ++a)
#pragma unroll
    for (int j = 0; j < kRY; ++j) acc[a][j] = 0.f;

#pragma unroll
  for (int st = 0; st < kStages - 1; ++st) issue(st);
  bool weights_ok = true;  // warp-uniform
  if (t.w_packed != nullptr) {
    const bool ok = tc::mbar_wait(&w_full, 0, kWaitLimit);
    if (!__all_sync(0xffffffffu, ok)) {  // never spin forever: flag the failure, leave the outputs unwritten
      if (lane == 0) atomicCAS(&g_direct_rows_error, 0, 1);
      weights_ok = false;
    }
  }
  int cpp = 0, ck = 0, ckx = np > 0 ? p.table.entries[e0].x : 0;
  for (int item = 0; weights_ok && item < items; ++item) {
    issue(item + kStages - 1);
    const bool ok = tc::mbar_wait(&slot_full[warp][item % kStages], (uint32_t)((item / kStages) & 1), kWaitLimit);
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0) atomicCAS(&g_direct_rows_error, 0, 2);
      // the copy issued for the next item may still be in flight into this warp's ring
      if (item + 1 < items) tc::mbar_wait(&slot_full[warp][(item + 1) % kStages], (uint32_t)(((item + 1) / kStages) & 1), kWaitLimit);
      break;
    }
    const int b0 = kGroup * (warp + kWarps * ck);
#pragma unroll
    for (int r = 0; r < kGroup; ++r) {
      if (b0 + r >= p.B) break;  // channels past the last were zero-filled by the copy; they have no weights
      const float *row = my_ring + (item % kStages) * kSlotFloats + r * kRowFloats + 4 * lane;
      // two windows: positions 4*lane .. +3 and 128 + 4*lane .. +3, each followed by NKY - 1 more values
      float xw[2][8];
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const float4 v0 = *reinterpret_cast<const float4 *>(row + 128 * g);
        xw[g][0] = v0.x, xw[g][1] = v0.y, xw[g][2] = v0.z, xw[g][3] = v0.w;
        if (NKY > 1) {
          const float2 v1 = *reinterpret_cast<const float2 *>(row + 128 * g + 4);
          xw[g][4] = v1.x, xw[g][5] = v1.y;
        }
      }
      const float4 *wrec = reinterpret_cast<const float4 *>(Ws + (size_t)(ckx * p.B + b0 + r) * WP);
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
          for (int j = 0; j < 4; ++j) acc[a][j] = fmaf(wv[a * NKY + k], xw[0][j + k], acc[a][j]);
      if (second_window) {  // block-uniform: false only where the last tile's second half lies past the signal
#pragma unroll
        for (int a = 0; a < A; ++a)
#pragma unroll
          for (int k = 0; k < NKY; ++k)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[a][4 + j] = fmaf(wv[a * NKY + k], xw[1][j + k], acc[a][4 + j]);
      }
    }
    __syncwarp();
    if (++ck == per_entry) {
      ck = 0;
      ++cpp;
      if (cpp < np) ckx = p.table.entries[e0 + cpp].x;
    }
  }
  __syncthreads();

  // ---- combine the warps: red[warp][a][position] -----------------------------------
  float *red = ring;
#pragma unroll
  for (int a = 0; a < A; ++a) {
    float *dst = red + ((size_t)warp * A + a) * kRedPitch + 4 * lane;
    *reinterpret_cast<float4 *>(dst) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    *reinterpret_cast<float4 *>(dst + 128) = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
  }
  __syncthreads();
  for (int o = tid; o < A * (kTY / 4); o += kThreads) {
    const int a = o / (kTY / 4), pos = 4 * (o % (kTY / 4));
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float4 v = *reinterpret_cast<const float4 *>(red + ((size_t)w * A + a) * kRedPitch + pos);
      s.x += v.x, s.y += v.y, s.z += v.z, s.w += v.w;
    }
    const int y = y0 + pos;
    if (y >= p.noy || y + 3 < 0) continue;
    float *out = p.out + n * p.out_sn + a * p.out_sa + (long long)ox * p.noy + y;
    const float bias = (!p.accumulate && p.bias != nullptr) ? __ldg(p.bias + a) : 0.f;
    if (t.vec_store && y >= 0 && y + 3 < p.noy) {
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
        if (y + j >= 0 && y + j < p.noy) out[j] = (p.accumulate ? out[j] : bias) + v[j];
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
  t.ws0 = p.Cy + std::min(0, p.By * (p.nky - 1));
  t.shift = ((t.ws0 % 4) + 4) % 4;  // (-shift + ws0) is then a multiple of 4
  t.y_tiles = (p.noy + t.shift + kTY - 1) / kTY;
  if ((long long)p.N * p.nox * t.y_tiles >= (1LL << 31)) return false;
  t.WP = (p.A * p.nky + 3) / 4 * 4;
  const size_t w_floats = ((size_t)p.nkx * p.B * t.WP + 31) / 32 * 32;
  t.w_floats = (int)w_floats;
  const size_t ring_floats = (size_t)kWarps * kStages * kSlotFloats;
  const size_t red_floats = (size_t)kWarps * p.A * kRedPitch;
  t.smem = (w_floats + std::max(ring_floats, red_floats)) * sizeof(float) + 128;  // + slack to align the base
  if (t.smem > 100 * 1024) return false;
  t.vec_store = (t.shift == 0 && reinterpret_cast<uintptr_t>(p.out) % 16 == 0 && p.noy % 4 == 0 &&
                 p.out_sn % 4 == 0 && p.out_sa % 4 == 0)
                    ? 1
                    : 0;
  return true;
}

// weight records in the kernel's shared-memory layout: [kx][b][WP], entry a * nky + k
// holds W[a, b, kx, ky(k)] with taps in increasing input offset
__global__ void pack_rows_weights_kernel(const float *__restrict__ w, long long w_sa, long long w_sb, int A, int B,
                                         int nkx, int nky, int WP, int By, float *__restrict__ out) {
  const int total = nkx * B * WP;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int e = i % WP, rec = i / WP;
    const int b = rec % B, kx = rec / B;
    float v = 0.f;
    if (e < A * nky) {
      const int a = e / nky, k = e % nky;
      const int ky = By < 0 ? nky - 1 - k : k;
      v = w[a * w_sa + b * w_sb + (long long)kx * nky + ky];
    }
    out[i] = v;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn encode = nullptr;
  if (encode == nullptr) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  return encode;
}

template <int A>
int dispatch_nky(const DirectProblem<float> &p, const RowsPlan &t, const CUtensorMap &in_map, cudaStream_t stream) {
  void (*kernel)(DirectProblem<float>, RowsPlan, const CUtensorMap) = nullptr;
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
  kernel<<<blocks, kThreads, t.smem, stream>>>(p, t, in_map);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("direct_rows_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

}  // namespace

// Reads and clears this kernel's timeout flag of the current device (synchronises it).
int direct_rows_take_error(int *code) {
  int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(code, g_direct_rows_error, sizeof(int));
  if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_direct_rows_error, &zero, sizeof(int));
  return err == cudaSuccess ? MELLIN_OK : fail(MELLIN_ERR_LAUNCH, std::string("device status: ") + cudaGetErrorString(err));
}

// scratch for the pre-packed weight records (0 = problem not covered by this kernel)
size_t direct_rows_workspace_bytes(const DirectProblem<float> &p) {
  RowsPlan t;
  if (!plan_rows(p, t)) return 0;
  return (size_t)p.nkx * p.B * t.WP * sizeof(float);
}

// MELLIN_ERR_UNSUPPORTED when the problem is outside this kernel's coverage.
// With too little (or no) workspace the weights are gathered inside the kernel.
int launch_direct_rows(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  RowsPlan t;
  if (!plan_rows(p, t)) return MELLIN_ERR_UNSUPPORTED;
  EncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr) return MELLIN_ERR_UNSUPPORTED;
  CUtensorMap in_map;
  {
    // the reduced tensor as (position, Mellin row, batch, channel) with its real strides;
    // a box is one staged row for each of 4 consecutive channels
    const cuuint64_t dims[4] = {(cuuint64_t)p.niy, (cuuint64_t)p.nix, (cuuint64_t)p.N, (cuuint64_t)p.B};
    const cuuint64_t strides[3] = {(cuuint64_t)p.niy * sizeof(float), (cuuint64_t)p.in_sn * sizeof(float),
                                   (cuuint64_t)p.in_sb * sizeof(float)};
    const cuuint32_t box[4] = {(cuuint32_t)kRowFloats, 1u, 1u, (cuuint32_t)kGroup};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    if (encode(&in_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(p.in), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return MELLIN_ERR_UNSUPPORTED;
  }
  const size_t need = (size_t)p.nkx * p.B * t.WP * sizeof(float);
  if (workspace != nullptr && workspace_bytes >= need && reinterpret_cast<uintptr_t>(workspace) % 16 == 0) {
    float *packed = static_cast<float *>(workspace);
    const int total = p.nkx * p.B * t.WP;
    pack_rows_weights_kernel<<<(total + 255) / 256, 256, 0, stream>>>(p.w, p.w_sa, p.w_sb, p.A, p.B, p.nkx, p.nky, t.WP,
                                                                      p.By, packed);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
      return fail(MELLIN_ERR_LAUNCH, std::string("pack_rows_weights_kernel: ") + cudaGetErrorString(err));
    count_launch();
    t.w_packed = packed;
  }
  switch (p.A) {
    case 1: return dispatch_nky<1>(p, t, in_map, stream);
    case 2: return dispatch_nky<2>(p, t, in_map, stream);
    case 3: return dispatch_nky<3>(p, t, in_map, stream);
    default: return dispatch_nky<4>(p, t, in_map, stream);
  }
}

}  // namespace mellin
