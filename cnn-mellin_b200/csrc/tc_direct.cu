// Tensor-core (tcgen05, sm_100a) kernel for the "direct" operator family:
//
//   out[n, a, ox, oy] = bias[a] + sum_{(kx, ix) in row ox} sum_b sum_ky
//                       W[a, b, kx, ky] * in[n, b, ix, oy + By * ky + Cy]
//
// i.e. the forward pass of a Mellin x linear layer and its input gradient when
// the linear axis has unit stride.  It is an implicit GEMM per output row:
//
//   M = 128 consecutive positions oy          (TMEM lanes)
//   N = output channels, padded to 16..256    (TMEM columns)
//   K = "rows" r = (table entry, b): one gathered input row in[n, b, ix, :]
//       per r, times the nky linear taps
//
// Shared-memory operand layout.  A (activations) is K-major with no swizzle:
// 16-byte chunk c holds rows 4c..4c+3 for one position, positions are 16 bytes
// apart.  Because consecutive positions are uniformly strided, the operand for
// linear tap t is the same buffer with its descriptor start address advanced by
// t * |By| positions: the taps cost no extra staging (descriptor-shift implicit
// GEMM).  B (weights) is K-major as well: for each (tap, group of 8 rows) two
// slabs of [channel][4 rows].  Rows are grouped per table entry with the
// channel count b padded to a multiple of 4, so that a 16-byte chunk never
// straddles two entries.
//
// FP32 accuracy on TF32 tensor cores: every operand is split as x = hi + lo
// with hi exactly representable in TF32 (low 13 mantissa bits cleared) and
// lo = x - hi (exact in FP32); three MMAs hi*hi + lo*hi + hi*lo accumulate in
// FP32 in TMEM.  The dropped lo*lo term and the rounding of lo to TF32 are
// O(2^-22) relative.  The tensor core's FP32 accumulator rounds toward zero on
// every MMA, a one-sided error that grows linearly with the number of chained
// MMAs; chains are therefore kept short: each K-block (at most 96 MMAs) is
// accumulated in TMEM from zero, then added by the epilogue warps into FP32
// registers with round-to-nearest (two-level accumulation).
//
// Warp roles (13 warps): 0-3 epilogue (TMEM -> registers -> global, one warp per
// 32 TMEM lanes), 4-11 producers (gather + split activations, copy packed
// weights), 12 MMA issuer.  A ring of shared-memory stages and two TMEM
// accumulators are handed around with mbarriers; every wait is bounded and a
// timeout raises a device-side error flag instead of hanging.
#include <algorithm>
#include <string>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"
#include "tc_ptx.cuh"

namespace mellin {

namespace {

constexpr int kEpilogueWarps = 4;
constexpr int kProducerWarps = 8;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kThreads = (kEpilogueWarps + kProducerWarps + 1) * 32;
constexpr int kTileM = 128;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr int kMaxStages = 4;

__device__ int g_tc_error = 0;  // first timeout code seen by any block since the last query

struct TcParams {
  const float *in;
  const float *bias;
  float *out;
  const float *w_hi;  // packed [kx][tap][b / 4][NP][b % 4]
  const float *w_lo;
  const int32_t *row_ptr;
  const int2 *entries;
  int N, A, B;
  int Bp;        // B rounded up to a multiple of 4: rows per table entry
  int nky, niy, nox, noy, nix;
  long long in_sn, in_sb, out_sn, out_sa;
  int By, Cy;
  int NP;        // padded output channels (multiple of 16)
  int a_tiles;   // tiles over output channels when A > 256
  int RW;        // staged positions per row (multiple of 8)
  int KB;        // rows per stage (multiple of 8)
  int stages;
  int y_tiles;
  long long tiles;
  int tmem_cols;
  uint32_t a_stage_bytes, w_stage_bytes;  // per hi or lo part
};

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// ---- weight packing ---------------------------------------------------------------
// W[a, b, kx, ky] (arbitrary a / b strides) -> hi and lo parts laid out
// [kx][tap][b / 4][NP_total][b % 4]: 16-byte chunks of 4 consecutive reduced
// channels for one output channel, tap slots in increasing input-offset order,
// output channels beyond A and reduced channels beyond B zero-filled.
__global__ void pack_weights_kernel(const float *__restrict__ w, long long w_sa, long long w_sb, int A, int B, int nkx,
                                    int nky, int NP_total, int By, float *__restrict__ hi, float *__restrict__ lo) {
  const int B4 = (B + 3) / 4;
  const long long total = (long long)nkx * nky * B4 * NP_total * 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int bl = (int)(i & 3);
    long long r = i >> 2;
    const int a = (int)(r % NP_total);
    r /= NP_total;
    const int b = (int)(r % B4) * 4 + bl;
    r /= B4;
    const int t = (int)(r % nky);
    const int kx = (int)(r / nky);
    const int ky = By < 0 ? nky - 1 - t : t;
    float v = 0.f;
    if (a < A && b < B) v = w[a * w_sa + b * w_sb + (long long)kx * nky + ky];
    const float h = tf32_hi(v);
    hi[i] = h;
    lo[i] = v - h;
  }
}

// ---- shared-memory carve-up -----------------------------------------------------------
struct TcControl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t dfull[2];
  uint64_t dempty[2];
  uint32_t tmem_base;
  int abort;
};
constexpr int kMaxKB = 64;
struct TcRowTable {
  long long in_off[kMaxKB];  // element offset of the gathered input row, -1 for padding rows
  int w_off[kMaxKB / 4];     // float4 offset of the packed weight chunk (tap 0, channel 0) of every 4 rows, -1 = padding
};
constexpr uint32_t kControlBytes = 1024 + kMaxStages * 1024;  // control block, then one row table per stage

__device__ __forceinline__ void raise_timeout(TcControl *ctl, int code) {
  atomicCAS(&g_tc_error, 0, code);
  ctl->abort = 1;
}

__device__ __forceinline__ void producer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory"); }

// NPC: padded output channels / 16 (the epilogue keeps 16 * NPC running sums per thread)
template <int NPC>
__global__ void __launch_bounds__(kThreads, 1) tc_direct_kernel(const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  TcControl *ctl = reinterpret_cast<TcControl *>(smem);
  TcRowTable *tables = reinterpret_cast<TcRowTable *>(smem + 1024);
  unsigned char *stage_base = smem + kControlBytes;
  const uint32_t stage_bytes = 2 * (p.a_stage_bytes + p.w_stage_bytes);
  volatile int *abort_flag = &ctl->abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int absBy = p.By < 0 ? -p.By : p.By;
  const int JB = p.KB >> 3;
  const int NPtot = p.NP * p.a_tiles;
  const int B4 = p.Bp >> 2;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      tc::mbar_init(&ctl->full[s], kProducerThreads);
      tc::mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(&ctl->dfull[a], 1);
      tc::mbar_init(&ctl->dempty[a], kEpilogueWarps * 32);
    }
    ctl->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == kEpilogueWarps + kProducerWarps) {
    tc::tmem_alloc(&ctl->tmem_base, (uint32_t)p.tmem_cols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < kEpilogueWarps) {
    // =========================== epilogue ===========================
    long long g = 0;  // K-blocks (accumulation intervals) consumed so far
    for (long long tile = blockIdx.x; tile < p.tiles; tile += gridDim.x) {
      // tcgen05.ld is warp-collective: keep every exit decision warp-uniform
      if (__any_sync(0xffffffffu, *abort_flag)) break;
      long long T = tile;
      const int at = (int)(T % p.a_tiles);
      T /= p.a_tiles;
      const int yt = (int)(T % p.y_tiles);
      T /= p.y_tiles;
      const int ox = (int)(T % p.nox);
      const int n = (int)(T / p.nox);
      const int np = p.row_ptr[ox + 1] - p.row_ptr[ox];
      const int Kr = np * p.Bp;
      const int oy = yt * kTileM + warp * 32 + lane;
      const int a0 = at * p.NP;
      float sum[NPC][16];
#pragma unroll
      for (int c = 0; c < NPC; ++c)
#pragma unroll
        for (int i = 0; i < 16; ++i) sum[c][i] = 0.f;
      bool failed = false;
      for (int k0 = 0; k0 < Kr; k0 += p.KB, ++g) {
        const int acc = (int)(g & 1);
        const bool ok = tc::mbar_wait(&ctl->dfull[acc], (uint32_t)((g >> 1) & 1), kSpinLimit);
        if (!__all_sync(0xffffffffu, ok)) {
          raise_timeout(ctl, 3);
          failed = true;
          break;
        }
        tc::tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < NPC; ++c) {
          uint32_t v[16];
          tc::tmem_ld16(tmem_base + (uint32_t)(acc * p.NP + 16 * c) + ((uint32_t)(warp * 32) << 16), v);
          tc::tmem_ld_wait();
          if (c == NPC - 1) {
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&ctl->dempty[acc]);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) sum[c][i] += __uint_as_float(v[i]);
        }
      }
      if (failed) break;
      if (oy < p.noy) {
        float *orow = p.out + n * p.out_sn + (long long)ox * p.noy + oy;
#pragma unroll
        for (int c = 0; c < NPC; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int a = a0 + 16 * c + i;
            if (a < p.A) {
              const float b = p.bias != nullptr ? __ldg(p.bias + a) : 0.f;
              orow[a * p.out_sa] = sum[c][i] + b;
            }
          }
      }
    }
  } else if (warp < kEpilogueWarps + kProducerWarps) {
    // =========================== producers ===========================
    const int ptid = tid - kEpilogueWarps * 32;
    long long it = 0;  // stage uses so far
    for (long long tile = blockIdx.x; tile < p.tiles && !*abort_flag; tile += gridDim.x) {
      long long T = tile;
      const int at = (int)(T % p.a_tiles);
      T /= p.a_tiles;
      const int yt = (int)(T % p.y_tiles);
      T /= p.y_tiles;
      const int ox = (int)(T % p.nox);
      const int n = (int)(T / p.nox);
      const int e0 = p.row_ptr[ox];
      const int np = p.row_ptr[ox + 1] - e0;
      const int Kr = np * p.Bp;
      const int ws = yt * kTileM + p.Cy + min(0, p.By * (p.nky - 1));
      bool failed = false;
      for (int k0 = 0; k0 < Kr; k0 += p.KB, ++it) {
        const int s = (int)(it % p.stages);
        const uint32_t use = (uint32_t)(it / p.stages);
        if (!tc::mbar_wait(&ctl->empty[s], (use & 1) ^ 1, kSpinLimit)) {
          raise_timeout(ctl, 1);
          failed = true;
          break;
        }
        TcRowTable *tab = tables + s;
        const int rows_here = min(p.KB, Kr - k0);
        const int rows_pad = (rows_here + 7) & ~7;
        if (ptid < p.KB) {
          long long in_off = -1;
          int w_off = -1;
          if (ptid < rows_here) {
            const int r = k0 + ptid;
            const int pp = r / p.Bp, b = r - pp * p.Bp;
            const int2 e = p.entries[e0 + pp];
            if (b < p.B) in_off = n * p.in_sn + b * p.in_sb + (long long)e.y * p.niy;
            w_off = (e.x * p.nky * B4 + (b >> 2)) * NPtot + at * p.NP;
          }
          tab->in_off[ptid] = in_off;
          if ((ptid & 3) == 0) tab->w_off[ptid >> 2] = w_off;
        }
        producer_sync();
        unsigned char *st = stage_base + (size_t)s * stage_bytes;
        float4 *a_hi = reinterpret_cast<float4 *>(st);
        float4 *a_lo = reinterpret_cast<float4 *>(st + p.a_stage_bytes);
        float4 *w_hi = reinterpret_cast<float4 *>(st + 2 * p.a_stage_bytes);
        float4 *w_lo = reinterpret_cast<float4 *>(st + 2 * p.a_stage_bytes + p.w_stage_bytes);
        // activations: item = (chunk of 4 rows, position)
        const int a_items = (rows_pad >> 2) * p.RW;
        for (int idx = ptid; idx < a_items; idx += kProducerThreads) {
          const int c = idx / p.RW, rho = idx - c * p.RW;
          const int iy = ws + rho;
          const bool in_range = iy >= 0 && iy < p.niy;
          float x[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const long long off = tab->in_off[4 * c + i];
            x[i] = (in_range && off >= 0) ? __ldg(p.in + off + iy) : 0.f;
          }
          float4 h, l;
          h.x = tf32_hi(x[0]), h.y = tf32_hi(x[1]), h.z = tf32_hi(x[2]), h.w = tf32_hi(x[3]);
          l.x = x[0] - h.x, l.y = x[1] - h.y, l.z = x[2] - h.z, l.w = x[3] - h.w;
          a_hi[c * p.RW + rho] = h;
          a_lo[c * p.RW + rho] = l;
        }
        // weights: item = (tap, chunk of 4 rows, output channel); consecutive
        // threads copy consecutive 16-byte chunks
        const int chunks_here = rows_pad >> 2;
        const int w_items = p.nky * chunks_here * p.NP;
        const float4 *src_hi = reinterpret_cast<const float4 *>(p.w_hi);
        const float4 *src_lo = reinterpret_cast<const float4 *>(p.w_lo);
        for (int idx = ptid; idx < w_items; idx += kProducerThreads) {
          const int nn = idx % p.NP;
          int rest = idx / p.NP;
          const int c = rest % chunks_here, t = rest / chunks_here;
          const int woff = tab->w_off[c];
          float4 h = make_float4(0.f, 0.f, 0.f, 0.f), l = h;
          if (woff >= 0) {
            const long long src = (long long)woff + (long long)t * B4 * NPtot + nn;
            h = __ldg(src_hi + src);
            l = __ldg(src_lo + src);
          }
          const int dst = (t * JB + (c >> 1)) * (2 * p.NP) + (c & 1) * p.NP + nn;
          w_hi[dst] = h;
          w_lo[dst] = l;
        }
        tc::fence_proxy_async();
        tc::mbar_arrive(&ctl->full[s]);
      }
      if (failed) break;
    }
  } else {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      const uint32_t idesc = tc::idesc_tf32(kTileM, p.NP);
      const uint32_t a_lbo = (uint32_t)p.RW * 16u;
      const uint32_t b_lbo = (uint32_t)p.NP * 16u;
      long long it = 0;  // K-blocks issued so far: stage = it % stages, accumulator = it & 1
      bool failed = false;
      for (long long tile = blockIdx.x; tile < p.tiles && !*abort_flag && !failed; tile += gridDim.x) {
        long long T = tile / p.a_tiles / p.y_tiles;
        const int ox = (int)(T % p.nox);
        const int np = p.row_ptr[ox + 1] - p.row_ptr[ox];
        const int Kr = np * p.Bp;
        for (int k0 = 0; k0 < Kr; k0 += p.KB, ++it) {
          const int s = (int)(it % p.stages);
          const uint32_t use = (uint32_t)(it / p.stages);
          const int acc = (int)(it & 1);
          if (!tc::mbar_wait(&ctl->full[s], use & 1, kSpinLimit)) {
            raise_timeout(ctl, 4);
            failed = true;
            break;
          }
          if (!tc::mbar_wait(&ctl->dempty[acc], (uint32_t)(((it >> 1) & 1) ^ 1), kSpinLimit)) {
            raise_timeout(ctl, 2);
            failed = true;
            break;
          }
          tc::tc_fence_after_sync();
          const uint32_t d_addr = tmem_base + (uint32_t)(acc * p.NP);
          const uint32_t st = tc::smem_u32(stage_base + (size_t)s * stage_bytes);
          const uint32_t a_hi = st, a_lo = st + p.a_stage_bytes;
          const uint32_t w_hi = st + 2 * p.a_stage_bytes, w_lo = w_hi + p.w_stage_bytes;
          const int jb_here = (min(p.KB, Kr - k0) + 7) >> 3;
          uint32_t accumulate = 0;
          for (int j = 0; j < jb_here; ++j) {
            for (int t = 0; t < p.nky; ++t) {
              const uint32_t a_off = (uint32_t)(2 * j) * a_lbo + (uint32_t)(t * absBy) * 16u;
              const uint32_t b_off = (uint32_t)((t * JB + j) * 2 * p.NP) * 16u;
              const uint64_t da_hi = tc::smem_desc(a_hi + a_off, a_lbo, 128u);
              const uint64_t da_lo = tc::smem_desc(a_lo + a_off, a_lbo, 128u);
              const uint64_t db_hi = tc::smem_desc(w_hi + b_off, b_lbo, 128u);
              const uint64_t db_lo = tc::smem_desc(w_lo + b_off, b_lbo, 128u);
              tc::mma_tf32(d_addr, da_lo, db_hi, idesc, accumulate);
              tc::mma_tf32(d_addr, da_hi, db_lo, idesc, 1u);
              tc::mma_tf32(d_addr, da_hi, db_hi, idesc, 1u);
              accumulate = 1u;
            }
          }
          tc::tc_commit(&ctl->empty[s]);
          tc::tc_commit(&ctl->dfull[acc]);
        }
      }
    }
    __syncwarp();
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == kEpilogueWarps + kProducerWarps) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

}  // namespace

// ---- host side ---------------------------------------------------------------------------

namespace {

struct TcPlan {
  TcParams params;
  size_t smem = 0;
  size_t pack_floats = 0;  // per hi / lo array
  int grid = 0;
};

bool plan_tc_direct(const DirectProblem<float> &p, TcPlan &plan) {
  if (p.Dy != 1 || p.Ay != 1) return false;
  if (p.A < 1 || p.B < 1 || p.nky < 1 || p.nkx < 1 || p.noy < 32 || p.nox < 1 || p.N < 1) return false;
  if (p.table.max_row < 1) return false;
  const int absBy = p.By < 0 ? -p.By : p.By;
  const long long halo = (long long)absBy * (p.nky - 1);
  if (halo > 128) return false;
  TcParams &q = plan.params;
  q.in = p.in, q.bias = p.accumulate ? nullptr : p.bias, q.out = p.out;
  q.row_ptr = p.table.row_ptr, q.entries = p.table.entries;
  q.N = p.N, q.A = p.A, q.B = p.B, q.Bp = (p.B + 3) / 4 * 4, q.nky = p.nky, q.niy = p.niy, q.nox = p.nox, q.noy = p.noy, q.nix = p.nix;
  q.in_sn = p.in_sn, q.in_sb = p.in_sb, q.out_sn = p.out_sn, q.out_sa = p.out_sa;
  q.By = p.By, q.Cy = p.Cy;
  const int a16 = (p.A + 15) / 16 * 16;
  q.a_tiles = (a16 + 127) / 128;  // the epilogue keeps NP running sums per thread: NP <= 128
  q.NP = ((a16 + q.a_tiles - 1) / q.a_tiles + 15) / 16 * 16;
  q.RW = (int)((kTileM + halo + 7) / 8 * 8);
  q.y_tiles = (p.noy + kTileM - 1) / kTileM;
  q.tiles = (long long)p.N * p.nox * q.y_tiles * q.a_tiles;
  int cols = 32;
  while (cols < 2 * q.NP) cols *= 2;
  q.tmem_cols = cols;
  // rows per stage: as many as fit a budget, at most what the longest table row needs
  const long long max_rows = ((long long)p.table.max_row * q.Bp + 7) / 8 * 8;
  const size_t per_row = 8u * q.RW + 8u * (size_t)p.nky * q.NP;  // bytes of A (hi+lo) and W (hi+lo) per row
  const size_t budget = 200 * 1024;
  int stages = 3;
  long long kb = (long long)(budget / stages / per_row) / 8 * 8;
  if (kb < 8) {
    stages = 2;
    kb = (long long)(budget / stages / per_row) / 8 * 8;
  }
  if (kb < 8) return false;
  kb = std::min<long long>(std::min<long long>(kb, max_rows), kMaxKB);
  // at most 96 chained MMAs (3 per tap per 8 rows) per K-block, see the note on accumulation above
  kb = std::min<long long>(kb, std::max<long long>(8, 96 / (3 * p.nky) * 8));
  q.KB = (int)kb;
  q.stages = stages;
  q.a_stage_bytes = (uint32_t)(q.KB / 4 * q.RW * 16);
  q.w_stage_bytes = (uint32_t)(p.nky * (q.KB / 8) * q.NP * 32);
  plan.smem = kControlBytes + (size_t)stages * 2 * (q.a_stage_bytes + q.w_stage_bytes);
  // one block per SM: keep shared memory above half of the SM so that the
  // TMEM request of a co-resident block can never wait for columns
  plan.smem = std::max<size_t>(plan.smem, 116 * 1024);
  if (plan.smem > 227 * 1024) return false;
  plan.pack_floats = (size_t)p.nkx * p.nky * q.Bp * q.NP * q.a_tiles;
  plan.grid = (int)std::min<long long>(q.tiles, sm_count());
  return true;
}

}  // namespace

size_t direct_tc_workspace_bytes(const DirectProblem<float> &p) {
  TcPlan plan;
  if (!plan_tc_direct(p, plan)) return 0;
  return 2 * ((plan.pack_floats * sizeof(float) + 255) / 256 * 256);
}

// Returns MELLIN_ERR_UNSUPPORTED (without recording an error message) when the
// problem is outside what this kernel covers; the caller then uses the CUDA-core path.
int launch_direct_tc(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  TcPlan plan;
  if (!plan_tc_direct(p, plan)) return MELLIN_ERR_UNSUPPORTED;
  const size_t part = (plan.pack_floats * sizeof(float) + 255) / 256 * 256;
  if (workspace == nullptr || workspace_bytes < 2 * part || reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
    return fail(MELLIN_ERR_WORKSPACE, "workspace too small or misaligned: need " + std::to_string(2 * part) +
                                          " bytes (16-byte aligned), got " + std::to_string(workspace_bytes));
  float *w_hi = static_cast<float *>(workspace);
  float *w_lo = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + part);
  {
    const int threads = 256;
    const long long total = (long long)plan.pack_floats;
    const int blocks = (int)std::min<long long>((total + threads - 1) / threads, 4096);
    pack_weights_kernel<<<blocks, threads, 0, stream>>>(p.w, p.w_sa, p.w_sb, p.A, p.B, p.nkx, p.nky,
                                                        plan.params.NP * plan.params.a_tiles, p.By, w_hi, w_lo);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("pack_weights_kernel: ") + cudaGetErrorString(err));
    count_launch();
  }
  plan.params.w_hi = w_hi;
  plan.params.w_lo = w_lo;
  void (*kernel)(TcParams) = nullptr;
  switch (plan.params.NP / 16) {
    case 1: kernel = tc_direct_kernel<1>; break;
    case 2: kernel = tc_direct_kernel<2>; break;
    case 3: kernel = tc_direct_kernel<3>; break;
    case 4: kernel = tc_direct_kernel<4>; break;
    case 5: kernel = tc_direct_kernel<5>; break;
    case 6: kernel = tc_direct_kernel<6>; break;
    case 7: kernel = tc_direct_kernel<7>; break;
    default: kernel = tc_direct_kernel<8>; break;
  }
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  kernel<<<plan.grid, kThreads, plan.smem, stream>>>(plan.params);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("tc_direct_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

// Reads and clears the device-side timeout flag of the current device
// (synchronises the device).
int tc_take_error(int *code) {
  int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(code, g_tc_error, sizeof(int));
  if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("device status: ") + cudaGetErrorString(err));
  return MELLIN_OK;
}

}  // namespace mellin
