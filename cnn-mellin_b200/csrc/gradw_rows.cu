// Weight (+ bias) gradient for layers with few input channels (the first layer
// of a stack: 3 feature maps in, 64..128 out), where the operation is bound by
// reading the output gradient once from HBM.
//
//   gw[a, b, kx, ky] = sum_{n, ox, oy} go[n, a, ox, oy] * x[n, b, ix(ox, kx), oy + By*ky + Cy]
//   gb[a]            = sum_{n, ox, oy} go[n, a, ox, oy]
//
// Work decomposition.  A tile is (n, ox, 128 positions oy).  Its 64 x 128 slab of
// `go` is fetched ONCE (16-byte cp.async, three stages in flight) and used for
// every Mellin tap kx that row ox takes part in; the few input rows those taps
// read ride along in the same stage.  A thread owns one output channel and a
// quarter of the positions and keeps the full [kx][b][ky] set of running sums
// in registers -- which is what limits this kernel to nkx <= 8 and
// b * nky <= 12.  A block walks many tiles, so its partial sums leave registers
// once, at the end; a second pass adds the per-block partials in a fixed order
// (no floating-point atomics: results are bit-reproducible).
#include <algorithm>
#include <string>

#include "../../include/mellin_b200.h"
#include <cuda.h>

#include "mellin_internal.h"
#include "tc_ptx.cuh"

namespace mellin {

namespace {

constexpr int kThreads = 256;
constexpr int kTA = 64;             // output channels per block
constexpr int kTK = 128;            // positions per tile
constexpr int kGoPitch = kTK + 4;   // floats; 4 extra keep 16-byte rows and spread banks
constexpr int kXPitch = kTK + 8;    // floats per staged input row (window + taps)
constexpr int kMaxKx = 8;
constexpr int kStages = 2;

struct RowsTiling {
  int y_tiles = 0, a_tiles = 0;
  long long tiles = 0;
  int Z = 0;  // blocks along the tile axis
  int ws0 = 0;  // first input position of tile 0 relative to its first output position
  size_t smem = 0;
};

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the destination is zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst, const void *src, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  const int bytes = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int B, int NKY>
__global__ void __launch_bounds__(kThreads, 2)
gradw_rows_kernel(const GradWProblem<float> p, const RowsTiling t, float *__restrict__ part_w,
                  float *__restrict__ part_b) {
  constexpr int BN = B * NKY;
  constexpr int kStageFloats = kTA * kGoPitch + kMaxKx * B * kXPitch;
  extern __shared__ __align__(16) float smem[];

  const int tid = threadIdx.x;
  const int co_l = tid & (kTA - 1), q = tid >> 6;  // channel, position slice
  const int a0 = blockIdx.y * kTA;
  const int z = blockIdx.x;

  float acc[kMaxKx][BN];
  float bsum = 0.f;
#pragma unroll
  for (int k = 0; k < kMaxKx; ++k)
#pragma unroll
    for (int i = 0; i < BN; ++i) acc[k][i] = 0.f;

  // ---- stage loader: every thread issues its share of one tile's copies -------
  const int warp = tid >> 5, lane = tid & 31;
  const long long go_plane = (long long)p.nox * p.noy;  // one (n, a) plane of grad_y
  auto load_tile = [&](long long tile, int stage) {
    if (tile < t.tiles) {
      const int tl = (int)tile;
      const int yt = tl % t.y_tiles;
      const int r = tl / t.y_tiles;
      const int ox = r % p.nox, n = r / p.nox;
      const int y0 = yt * kTK;
      float *gos = smem + stage * kStageFloats;
      float *xs = gos + kTA * kGoPitch;
      // output-gradient slab: a warp copies a row of 32 chunks of 16 bytes
      {
        const int y = y0 + 4 * lane;
        const float *base = p.go + ((long long)n * p.A + a0) * go_plane + (long long)ox * p.noy + y;
#pragma unroll
        for (int k = 0; k < kTA / 8; ++k) {
          const int row = warp + 8 * k;
          const bool valid = a0 + row < p.A && y < p.noy;
          cp_async16(gos + row * kGoPitch + 4 * lane, valid ? base + row * go_plane : p.go, valid);
        }
      }
      // input rows of the taps of this ox: slot = kx, one row per input channel
      const int e0 = p.table_h.row_ptr[ox];
      const int np = p.table_h.row_ptr[ox + 1] - e0;
      const int ws = y0 + t.ws0;
      for (int rb = warp; rb < np * B; rb += kThreads / 32) {
        const int b = rb % B, pp = rb / B;
        const int2 e = p.table_h.entries[e0 + pp];
        const float *row = p.in + (((long long)n * p.B + b) * p.nix + e.y) * p.niy;
        float *dst = xs + (e.x * B + b) * kXPitch;
        for (int c = lane; c < kXPitch; c += 32) {
          const int iy = ws + c;
          const bool valid = iy >= 0 && iy < p.niy;
          cp_async4(dst + c, valid ? row + iy : p.in, valid);
        }
      }
    }
    cp_async_commit();
  };

  long long tile = z;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) load_tile(tile + (long long)s * t.Z, s);

  for (int it = 0; tile < t.tiles; tile += t.Z, ++it) {
    load_tile(tile + (long long)(kStages - 1) * t.Z, (it + kStages - 1) % kStages);
    cp_async_wait<kStages - 1>();
    __syncthreads();

    const int ox = ((int)tile / t.y_tiles) % p.nox;
    const int e0 = p.table_h.row_ptr[ox];
    const int np = p.table_h.row_ptr[ox + 1] - e0;
    unsigned mask = 0;
    for (int pp = 0; pp < np; ++pp) mask |= 1u << p.table_h.entries[e0 + pp].x;

    const float *gos = smem + (it % kStages) * kStageFloats + co_l * kGoPitch;
    const float *xs = smem + (it % kStages) * kStageFloats + kTA * kGoPitch;
    // The four position slices interleave in steps of 8 positions, so that a
    // ragged last tile (800 = 6 * 128 + 32) costs only the steps that hold data.
    const int valid = p.noy - ((int)tile % t.y_tiles) * kTK;
#pragma unroll 1
    for (int yo = 8 * q; yo < kTK && yo < valid; yo += 32) {
      const float4 ga = *reinterpret_cast<const float4 *>(gos + yo);
      const float4 gb4 = *reinterpret_cast<const float4 *>(gos + yo + 4);
      const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb4.x, gb4.y, gb4.z, gb4.w};
      bsum += ((g[0] + g[1]) + (g[2] + g[3])) + ((g[4] + g[5]) + (g[6] + g[7]));
#pragma unroll
      for (int kx = 0; kx < kMaxKx; ++kx) {
        if (!((mask >> kx) & 1u)) continue;
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const float4 *xp = reinterpret_cast<const float4 *>(xs + (kx * B + b) * kXPitch + yo);
          const float4 x0 = xp[0], x1 = xp[1];
          float xw[12];
          xw[0] = x0.x, xw[1] = x0.y, xw[2] = x0.z, xw[3] = x0.w, xw[4] = x1.x, xw[5] = x1.y, xw[6] = x1.z, xw[7] = x1.w;
          if (NKY > 1) {
            const float4 x2 = xp[2];
            xw[8] = x2.x, xw[9] = x2.y, xw[10] = x2.z, xw[11] = x2.w;
          }
#pragma unroll
          for (int k = 0; k < NKY; ++k) {
            float s = acc[kx][b * NKY + k];
#pragma unroll
            for (int j = 0; j < 8; ++j) s = fmaf(g[j], xw[j + k], s);
            acc[kx][b * NKY + k] = s;
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- combine the four position slices and write this block's partial sums ----
  float *red = smem;  // [4][64][BN]
  const long long gw_elems = (long long)p.A * p.B * p.nkx * p.nky;
  float *pw = part_w + (long long)z * gw_elems;
  for (int kx = 0; kx < p.nkx && kx < kMaxKx; ++kx) {
    // static register indexing: select the kx-th row with an unrolled compare
    float mine[BN];
#pragma unroll
    for (int i = 0; i < BN; ++i) mine[i] = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxKx; ++k)
      if (k == kx) {
#pragma unroll
        for (int i = 0; i < BN; ++i) mine[i] = acc[k][i];
      }
#pragma unroll
    for (int i = 0; i < BN; ++i) red[(q * kTA + co_l) * BN + i] = mine[i];
    __syncthreads();
    if (q == 0) {
      const int a = a0 + co_l;
      if (a < p.A) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const float s = (red[co_l * BN + i] + red[(kTA + co_l) * BN + i]) +
                          (red[(2 * kTA + co_l) * BN + i] + red[(3 * kTA + co_l) * BN + i]);
          const int b = i / NKY, k = i % NKY;
          const int ky = p.By < 0 ? NKY - 1 - k : k;  // slot k holds the tap whose input offset is k
          pw[(((long long)a * p.B + b) * p.nkx + kx) * p.nky + ky] = s;
        }
      }
    }
    __syncthreads();
  }
  if (part_b != nullptr) {
    red[q * kTA + co_l] = bsum;
    __syncthreads();
    const int a = a0 + co_l;
    if (q == 0 && a < p.A)
      part_b[(long long)z * p.A + a] = (red[co_l] + red[kTA + co_l]) + (red[2 * kTA + co_l] + red[3 * kTA + co_l]);
  }
}

// ---- the same kernel fed by TMA ---------------------------------------------------
// One thread issues a tile's copies (one 64 x 132 box of grad_y, one box of
// B x 136 positions per table entry) and everybody else only waits on the
// stage's mbarrier: the per-thread address arithmetic of the cp.async version
// was a quarter of its non-FMA instructions.  TMA boxes start at multiples of 4
// positions, so an input window begins LEAD positions into its row
// (LEAD = (Cy + min(0, By (nky - 1))) mod 4, a constant of the layer).
constexpr int kSlotAlign = 128;
__host__ __device__ constexpr int x_slot_floats(int b) { return (b * kXPitch * 4 + kSlotAlign - 1) / kSlotAlign * kSlotAlign / 4; }

struct TileMeta {
  unsigned mask;  // Mellin taps present in this tile's row
  int valid;      // positions of the tile that lie inside the signal
};

// First bounded wait that gave up since the last query (0 = none): 1 = a stage's
// copies never completed, 2 = the self-test's unarmed barrier (expected there).
__device__ int g_rows_error = 0;
constexpr uint32_t kWaitLimit = 1u << 22;

template <int B, int NKY, int LEAD>
__global__ void __launch_bounds__(kThreads, 2)
gradw_rows_tma_kernel(const GradWProblem<float> p, const RowsTiling t, float *__restrict__ part_w,
                      float *__restrict__ part_b, const __grid_constant__ CUtensorMap go_map,
                      const __grid_constant__ CUtensorMap x_map) {
  constexpr int BN = B * NKY;
  constexpr int kSlot = x_slot_floats(B);
  constexpr int kStageFloats = kTA * kGoPitch + kMaxKx * kSlot;
  constexpr int kStep = 16;  // positions per inner step
  constexpr int kWin = (LEAD + kStep + NKY - 1 + 3) / 4;  // float4 loads per window
  extern __shared__ __align__(1024) float tile_smem[];
  float *smem = tile_smem;
  __shared__ uint64_t full[kStages];
  __shared__ TileMeta meta[kStages];
  __shared__ volatile int abort_word;

  const int tid = threadIdx.x;
  const int co_l = tid & (kTA - 1), q = tid >> 6;
  const int a0 = blockIdx.y * kTA;
  const int z = blockIdx.x;

  float acc[kMaxKx][BN];
  float bsum = 0.f;
#pragma unroll
  for (int k = 0; k < kMaxKx; ++k)
#pragma unroll
    for (int i = 0; i < BN; ++i) acc[k][i] = 0.f;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) tc::mbar_init(&full[s], 1);
    abort_word = 0;
    tc::fence_mbar_init();
  }
  __syncthreads();

  // Thread 0 publishes a tile's mask / extent in meta[stage] BEFORE it arrives on
  // the stage's barrier: the arrive releases those writes, a waiter's successful
  // try_wait acquires them.  (Written after the arrive they raced with the
  // waiters -- a warp that saw the copies complete while thread 0 was still
  // between its last copy and the two stores read the previous tile's mask and
  // summed the wrong taps; seen on the first launch over fresh tensors.)
  auto issue = [&](long long tile, int stage) {  // thread 0 only
    if (tile >= t.tiles) return;
    const int tl = (int)tile;
    const int yt = tl % t.y_tiles;
    const int r = tl / t.y_tiles;
    const int ox = r % p.nox, n = r / p.nox;
    const int y0 = yt * kTK;
    float *gos = smem + stage * kStageFloats;
    float *xs = gos + kTA * kGoPitch;
    const int e0 = p.table_h.row_ptr[ox];
    const int np = min(p.table_h.row_ptr[ox + 1] - e0, kMaxKx);
    int2 ent[kMaxKx];
    unsigned mask = 0;
#pragma unroll
    for (int pp = 0; pp < kMaxKx; ++pp) {
      ent[pp] = pp < np ? p.table_h.entries[e0 + pp] : make_int2(0, 0);
      if (pp < np) mask |= 1u << ent[pp].x;
    }
    meta[stage].mask = mask;
    meta[stage].valid = p.noy - y0;
    tc::mbar_arrive_expect_tx(&full[stage], (uint32_t)((kTA * kGoPitch + np * B * kXPitch) * sizeof(float)));
    tc::tma_load_4d(gos, &go_map, y0, ox, a0, n, &full[stage]);
    const int x0 = y0 + t.ws0 - LEAD;  // a multiple of 4
#pragma unroll
    for (int pp = 0; pp < kMaxKx; ++pp)
      if (pp < np) tc::tma_load_4d(xs + ent[pp].x * kSlot, &x_map, x0, ent[pp].y, 0, n, &full[stage]);
  };

  long long tile = z;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(tile + (long long)s * t.Z, s);
  }

  int it = 0;
  for (; tile < t.tiles; tile += t.Z, ++it) {
    const int stage = it % kStages;
    if (tid == 0) issue(tile + (long long)(kStages - 1) * t.Z, (it + kStages - 1) % kStages);
    // A wait that gives up raises the device flag and the block-wide abort word;
    // the thread skips the tile but still reaches the barrier below, after which
    // every thread sees the word and leaves the loop together.
    const bool arrived = tc::mbar_wait(&full[stage], (uint32_t)((it / kStages) & 1), kWaitLimit);
    if (!arrived) {
      atomicCAS(&g_rows_error, 0, 1);
      abort_word = 1;
    } else {
      const unsigned mask = meta[stage].mask;
      const int valid = meta[stage].valid;

      const float *gos = smem + stage * kStageFloats + co_l * kGoPitch;
      const float *xs = smem + stage * kStageFloats + kTA * kGoPitch;
#pragma unroll 1
      for (int yo = kStep * q; yo < kTK && yo < valid; yo += 4 * kStep) {
        float g[kStep];
#pragma unroll
        for (int i = 0; i < kStep / 4; ++i) {
          const float4 v = *reinterpret_cast<const float4 *>(gos + yo + 4 * i);
          g[4 * i] = v.x, g[4 * i + 1] = v.y, g[4 * i + 2] = v.z, g[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int i = 0; i < kStep; i += 4) bsum += (g[i] + g[i + 1]) + (g[i + 2] + g[i + 3]);
#pragma unroll
        for (int kx = 0; kx < kMaxKx; ++kx) {
          if (!((mask >> kx) & 1u)) continue;
#pragma unroll
          for (int b = 0; b < B; ++b) {
            const float4 *xp = reinterpret_cast<const float4 *>(xs + kx * kSlot + b * kXPitch + yo);
            float xw[4 * kWin];
#pragma unroll
            for (int i = 0; i < kWin; ++i) {
              const float4 v = xp[i];
              xw[4 * i] = v.x, xw[4 * i + 1] = v.y, xw[4 * i + 2] = v.z, xw[4 * i + 3] = v.w;
            }
#pragma unroll
            for (int k = 0; k < NKY; ++k) {
              float s = acc[kx][b * NKY + k];
#pragma unroll
              for (int j = 0; j < kStep; ++j) s = fmaf(g[j], xw[LEAD + j + k], s);
              acc[kx][b * NKY + k] = s;
            }
          }
        }
      }
    }
    // this stage is refilled by the copy engine after the barrier: order the reads before it
    tc::fence_proxy_async();
    __syncthreads();
    if (abort_word) break;  // block-uniform: written before the barrier, read after it
  }
  if (abort_word) {
    // copies issued for the next tile may still be in flight into this block's
    // shared memory: give them a bounded time to land before the block exits
    if (tid == 0 && tile + t.Z < t.tiles) tc::mbar_wait(&full[(it + 1) % kStages], (uint32_t)(((it + 1) / kStages) & 1), kWaitLimit);
    __syncthreads();
  }
  __syncthreads();

  // ---- combine the four position slices and write this block's partial sums ----
  float *red = smem;  // [4][64][BN]
  const long long gw_elems = (long long)p.A * p.B * p.nkx * p.nky;
  float *pw = part_w + (long long)z * gw_elems;
  for (int kx = 0; kx < p.nkx && kx < kMaxKx; ++kx) {
    float mine[BN];
#pragma unroll
    for (int i = 0; i < BN; ++i) mine[i] = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxKx; ++k)
      if (k == kx) {
#pragma unroll
        for (int i = 0; i < BN; ++i) mine[i] = acc[k][i];
      }
#pragma unroll
    for (int i = 0; i < BN; ++i) red[(q * kTA + co_l) * BN + i] = mine[i];
    __syncthreads();
    if (q == 0) {
      const int a = a0 + co_l;
      if (a < p.A) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const float s = (red[co_l * BN + i] + red[(kTA + co_l) * BN + i]) +
                          (red[(2 * kTA + co_l) * BN + i] + red[(3 * kTA + co_l) * BN + i]);
          const int b = i / NKY, k = i % NKY;
          const int ky = p.By < 0 ? NKY - 1 - k : k;
          pw[(((long long)a * p.B + b) * p.nkx + kx) * p.nky + ky] = s;
        }
      }
    }
    __syncthreads();
  }
  if (part_b != nullptr) {
    red[q * kTA + co_l] = bsum;
    __syncthreads();
    const int a = a0 + co_l;
    if (q == 0 && a < p.A)
      part_b[(long long)z * p.A + a] = (red[co_l] + red[kTA + co_l]) + (red[2 * kTA + co_l] + red[3 * kTA + co_l]);
  }
}

bool plan_rows(const GradWProblem<float> &p, RowsTiling &t) {
  if (p.Dy != 1 || p.Ay != 1) return false;
  if (p.nkx < 1 || p.nkx > kMaxKx || p.B < 1 || p.B > 4 || p.nky < 1 || p.nky > 3) return false;
  if (p.nky > 1 && p.By != 1 && p.By != -1) return false;
  if (p.noy < 32 || p.noy % 4 != 0 || p.A < 1 || p.N < 1 || p.nox < 1) return false;
  if (reinterpret_cast<uintptr_t>(p.go) % 16 != 0) return false;
  t.y_tiles = (p.noy + kTK - 1) / kTK;
  t.a_tiles = (p.A + kTA - 1) / kTA;
  t.tiles = (long long)p.N * p.nox * t.y_tiles;
  if (t.tiles >= (1LL << 31)) return false;
  t.ws0 = p.Cy + std::min(0, p.By * (p.nky - 1));
  t.Z = (int)std::min<long long>(t.tiles, std::max(1, 2 * sm_count() / t.a_tiles));
  t.smem = (size_t)kStages * (kTA * kGoPitch + kMaxKx * p.B * kXPitch) * sizeof(float);
  return t.smem <= 200 * 1024;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// (position, Mellin row, channel, utterance) view of a dense activation tensor
bool make_map(CUtensorMap *map, const float *base, int inner, int rows, int chans, int batch, int box_inner,
              int box_chans) {
  static EncodeTiledFn encode = nullptr;
  if (encode == nullptr) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return false;
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)chans, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)inner * 4, (cuuint64_t)inner * rows * 4, (cuuint64_t)inner * rows * chans * 4};
  const cuuint32_t box[4] = {(cuuint32_t)box_inner, 1u, (cuuint32_t)box_chans, 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int B, int NKY>
int launch_rows_tma(const GradWProblem<float> &p, const RowsTiling &t, float *pw, float *pb, cudaStream_t stream) {
  // TMA needs 16-byte aligned bases and row pitches
  if (p.niy % 4 != 0 || p.noy % 4 != 0 || reinterpret_cast<uintptr_t>(p.in) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(p.go) % 16 != 0)
    return MELLIN_ERR_UNSUPPORTED;
  CUtensorMap go_map, x_map;
  if (!make_map(&go_map, p.go, p.noy, p.nox, p.A, p.N, kGoPitch, kTA) ||
      !make_map(&x_map, p.in, p.niy, p.nix, p.B, p.N, kXPitch, B))
    return MELLIN_ERR_UNSUPPORTED;
  void (*kernel)(GradWProblem<float>, RowsTiling, float *, float *, const CUtensorMap, const CUtensorMap) = nullptr;
  switch (((t.ws0 % 4) + 4) % 4) {
    case 0: kernel = gradw_rows_tma_kernel<B, NKY, 0>; break;
    case 1: kernel = gradw_rows_tma_kernel<B, NKY, 1>; break;
    case 2: kernel = gradw_rows_tma_kernel<B, NKY, 2>; break;
    default: kernel = gradw_rows_tma_kernel<B, NKY, 3>; break;
  }
  const size_t smem = (size_t)kStages * (kTA * kGoPitch + kMaxKx * x_slot_floats(B)) * sizeof(float);
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  kernel<<<dim3(t.Z, t.a_tiles), kThreads, smem, stream>>>(p, t, pw, pb, go_map, x_map);
  err = cudaGetLastError();
  if (err != cudaSuccess)
    return fail(MELLIN_ERR_LAUNCH, std::string("gradw_rows_tma_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

template <int B>
int dispatch_rows_nky(const GradWProblem<float> &p, const RowsTiling &t, float *pw, float *pb, cudaStream_t stream) {
  {
    int rc = MELLIN_ERR_UNSUPPORTED;
    switch (p.nky) {
      case 1: rc = launch_rows_tma<B, 1>(p, t, pw, pb, stream); break;
      case 2: rc = launch_rows_tma<B, 2>(p, t, pw, pb, stream); break;
      default: rc = launch_rows_tma<B, 3>(p, t, pw, pb, stream); break;
    }
    if (rc != MELLIN_ERR_UNSUPPORTED) return rc;
  }
  void (*kernel)(GradWProblem<float>, RowsTiling, float *, float *) = nullptr;
  switch (p.nky) {
    case 1: kernel = gradw_rows_kernel<B, 1>; break;
    case 2: kernel = gradw_rows_kernel<B, 2>; break;
    default: kernel = gradw_rows_kernel<B, 3>; break;
  }
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  kernel<<<dim3(t.Z, t.a_tiles), kThreads, t.smem, stream>>>(p, t, pw, pb);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("gradw_rows_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

}  // namespace

size_t gradw_rows_workspace_floats(const GradWProblem<float> &p, size_t *bias_offset) {
  RowsTiling t;
  if (!plan_rows(p, t)) return 0;
  size_t w_part = (size_t)t.Z * p.A * p.B * p.nkx * p.nky;
  w_part = (w_part + 63) / 64 * 64;
  if (bias_offset) *bias_offset = w_part;
  return w_part + (size_t)t.Z * p.A;
}

// Launches the kernel that fills the per-block partial sums; *slices receives
// their number.  MELLIN_ERR_UNSUPPORTED when the problem is outside its coverage.
int launch_gradw_rows(const GradWProblem<float> &p, float *part_w, float *part_b, int *slices, cudaStream_t stream) {
  RowsTiling t;
  if (!plan_rows(p, t)) return MELLIN_ERR_UNSUPPORTED;
  *slices = t.Z;
  switch (p.B) {
    case 1: return dispatch_rows_nky<1>(p, t, part_w, part_b, stream);
    case 2: return dispatch_rows_nky<2>(p, t, part_w, part_b, stream);
    case 3: return dispatch_rows_nky<3>(p, t, part_w, part_b, stream);
    default: return dispatch_rows_nky<4>(p, t, part_w, part_b, stream);
  }
}

// Reads and clears the row kernels' timeout flag of the current device (synchronises it).
int gradw_rows_take_error(int *code) {
  int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(code, g_rows_error, sizeof(int));
  if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_rows_error, &zero, sizeof(int));
  return err == cudaSuccess ? MELLIN_OK : fail(MELLIN_ERR_LAUNCH, std::string("device status: ") + cudaGetErrorString(err));
}

namespace {
// One thread waits, with a limit of 1000 polls, on a barrier that nothing arms,
// and must come back with the flag raised instead of hanging.
__global__ void unarmed_wait_kernel() {
  __shared__ uint64_t bar;
  tc::mbar_init(&bar, 1);
  tc::fence_mbar_init();
  if (!tc::mbar_wait(&bar, 0, 1000u)) atomicCAS(&g_rows_error, 0, 2);
}
}  // namespace

int launch_unarmed_wait(cudaStream_t stream) {
  unarmed_wait_kernel<<<1, 1, 0, stream>>>();
  const cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? MELLIN_OK : fail(MELLIN_ERR_LAUNCH, std::string("unarmed_wait_kernel: ") + cudaGetErrorString(err));
}

}  // namespace mellin
