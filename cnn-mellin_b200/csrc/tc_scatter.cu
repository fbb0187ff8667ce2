// Few OUTPUT channels (at most 4), many reduced channels, on tensor cores (tcgen05,
// sm_100a), walked BY SOURCE ROW -- the input gradient of a first layer (3 feature
// maps receive the gradient of 64..256 channels):
//
//   out[n, a, ox, oy] = init + sum_{(kx, ix) in row ox} sum_b sum_ky
//                       W[a, b, kx, ky] * in[n, b, ix, oy + By * ky + Cy]
//
// Walked by output row, every row of `in` is fetched once per table entry that names it
// (2.6 times on average for an 8-tap Mellin kernel over 41 rows) and the work is a long
// thin reduction that CUDA cores issue one FMA at a time.  Here an item is (n, SOURCE row
// ix, 128 staged positions) and ONE GEMM serves every table entry (kx, ox) of the row:
//
//   D[position, (entry, a, tap)] = sum_b in[n, b, ix, start + position] * W[a, b, kx(entry), ky(tap)]
//   M = 128 positions (TMEM lanes), N = entries x A x taps columns (<= 96), K = reduced channels
//
// The linear taps are not gathered: tap k of output position q is column (.., k) of row
// q + k, so the epilogue adds nky rows of D that lie k lanes apart (warp shuffles: the four
// lane quadrants hold overlapping runs of positions, so no sum crosses a warp) and a tile
// emits 128 - 4 (nky - 1) outputs.  The sums of an entry are its
// "partial plane" (n, entry, a, position); a second, tiny kernel adds the planes of every
// output row in table order (deterministic: no atomics on floats anywhere).
//
// `in` arrives by 4-D TMA boxes of 32 channels x 128 positions (zero-filled outside the
// signal).  Operand A lives in TENSOR MEMORY: 8 converter warps read a box (position =
// TMEM lane, so a warp reads 32 consecutive positions of one channel: no bank conflicts),
// split it into TF32 hi / lo parts and write them with tcgen05.st, 16 channels per thread --
// shared memory carries the raw box once in and once out, instead of seven times for an
// operand staged there.  The B operand (the weights of the row's entries, hi / lo, already
// in operand layout) is prepared once per launch by a small kernel and fetched per stage
// with one bulk copy; 3 MMAs (lo*hi, hi*lo, hi*hi) per 8 channels keep FP32 accuracy;
// accumulators are double-buffered in TMEM so that the epilogue of one item runs under the
// MMAs of the next.  15 warps: 4 epilogue, 8 converter, 1 MMA issuer, 2 copy
// issuers; persistent blocks take items round-robin (all items cost the same: the kernel is
// bound by the one pass over `in`).  Every wait is bounded and reports through a device word.
#include <cuda.h>

#include <algorithm>
#include <string>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"
#include "tc_ptx.cuh"

namespace mellin {

namespace {

constexpr int kEpilogueWarps = 4;
constexpr int kConvertWarps = 8;
constexpr int kConvertThreads = kConvertWarps * 32;
constexpr int kMmaWarp = kEpilogueWarps + kConvertWarps;
constexpr int kCopyWarp = kMmaWarp + 1;    // boxes of `in`
constexpr int kCopyBWarp = kCopyWarp + 1;  // B operands (their ring is shallower: a loader of its own, so that
                                           // the boxes of `in` can run the whole raw ring ahead)
constexpr int kThreads = (kCopyBWarp + 1) * 32;
constexpr int kTM = 128;          // staged positions per item
constexpr int kKB = 32;           // reduced channels per stage
constexpr int kRawStages = 8;     // 128 KB of copies in flight per SM
constexpr int kOpStages = 4;      // operand A sets in tensor memory
constexpr int kBStages = 3;
constexpr int kMaxCols = 96;      // entries x A x taps
constexpr int kMaxEntries = 16;   // per table row, either order
constexpr uint32_t kRawBytes = kKB * kTM * 4;            // 16 KB
constexpr uint32_t kBufCols = 128;                       // TMEM columns of one accumulator tile; two items in flight
constexpr uint32_t kACol0 = 2 * kBufCols;                // first TMEM column of the operand A ring
constexpr uint32_t kAStageCols = 2 * kKB;                // hi then lo: 32 columns each
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr int kMaxRows = 384;     // source rows (their offsets are kept in shared memory)
constexpr int kHeaderBytes = 2048;

struct Control {
  uint64_t raw_full[kRawStages], raw_empty[kRawStages], a_full[kOpStages], a_empty[kOpStages];
  uint64_t b_full[kBStages], b_empty[kBStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort;
  int rp[kMaxRows + 1];  // the by-source-row table's row offsets
};
static_assert(sizeof(Control) <= kHeaderBytes, "Control must fit the header");

// First bounded wait that gave up since the last query (0 = none): 1 converters, 2 MMA issuer
// (operands), 3 MMA issuer (accumulator buffer), 4 epilogue, 5 copy issuer (boxes), 6 copy issuer (B operands).
__device__ int g_tc_scatter_error = 0;

#ifdef MELLIN_TUNING_HOOKS
// per-role wait / work cycles of block 0: 0 epilogue, 1 converter, 2 MMA issuer, 3 copy issuer
__device__ long long g_ts_prof[16];
#define PROF_BEGIN() long long prof_t0 = clock64(), prof_wait = 0, prof_t1 = 0
#define PROF_WAIT_START() prof_t1 = clock64()
#define PROF_WAIT_END() prof_wait += clock64() - prof_t1
#define PROF_END(slot)                                           \
  if (blockIdx.x == 0 && lane == 0) {                            \
    g_ts_prof[2 * (slot)] = prof_wait;                           \
    g_ts_prof[2 * (slot) + 1] = clock64() - prof_t0 - prof_wait; \
  }
#else
#define PROF_BEGIN()
#define PROF_WAIT_START()
#define PROF_WAIT_END()
#define PROF_END(slot)
#endif

struct TsParams {
  const int32_t *row_ptr_in;   // by source row: rows = ix, entries (kx, ox)
  const int2 *entries_in;
  const int32_t *row_ptr_out;  // by output row: rows = ox, entries (kx, ix)
  const int2 *entries_out;
  const float *w;
  const float *bias;
  float *out;
  float *b_pack;               // [ix][k-block][hi | lo][4-channel chunk][column][4]
  float *planes;               // [n][entry][a][plane]
  int *plane_of;               // for every entry of the by-output-row table: the entry of the by-source-row table (= plane)
  long long w_sa, w_sb, out_sn, out_sa;
  long long entries;           // table entries = planes per (n, a)
  int N, A, B, nkx, nky, nix, nox, noy, By;
  int AN;                      // A * nky: columns per entry
  int T;                       // outputs per item
  int y_tiles, shift, ws0, plane;
  int kblocks;                 // stages per item
  int n_max_pad;               // widest GEMM of the launch (columns, multiple of 16)
  int total;                   // items
  int accumulate;
  uint32_t b_stage_bytes;      // 256 * n_max_pad
};

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ void raise_timeout(Control *ctl, int code) {
  atomicCAS(&g_tc_scatter_error, 0, code);
  ctl->abort = 1;
}

// Items (n, y tile, ix) in round-robin order over the blocks, rows varying fastest; advanced without divisions.
struct ItemIter {
  int id, ix, yt, n;
  int step_ix, step_yt, step_n;
  __device__ __forceinline__ ItemIter(const TsParams &p) {
    id = blockIdx.x;
    ix = id % p.nix;
    const int r = id / p.nix;
    yt = r % p.y_tiles, n = r / p.y_tiles;
    const int g = gridDim.x;
    step_ix = g % p.nix;
    const int gr = g / p.nix;
    step_yt = gr % p.y_tiles, step_n = gr / p.y_tiles;
  }
  __device__ __forceinline__ void next(const TsParams &p) {
    id += gridDim.x;
    ix += step_ix;
    yt += step_yt;
    n += step_n;
    if (ix >= p.nix) ix -= p.nix, ++yt;
    if (yt >= p.y_tiles) yt -= p.y_tiles, ++n;
  }
};
__device__ __forceinline__ int pad16(int v) { return (v + 15) & ~15; }

// The B operand of every source row: column (entry, a, tap) of row ix holds W[a, b, kx(entry), ky(tap)]
// (taps in increasing input offset), split into TF32 hi / lo parts, in the K-major operand layout of a
// GEMM with pad16(columns) columns; unused columns and channels past the last are zero.  Grid: (chunks of
// 256 elements, source row x k-block); one more row of blocks (blockIdx.y = nix * kblocks) finds, for every
// entry of the by-output-row table, the partial plane that holds its sums.
__global__ void __launch_bounds__(256) pack_scatter_b_kernel(const TsParams p) {
  tc::launch_dependents();  // the main kernel may set itself up meanwhile; it waits for this grid before reading
  if ((int)blockIdx.y == p.nix * p.kblocks) {
    const int total = p.row_ptr_out[p.nox];
    for (int e = blockIdx.x * 256 + threadIdx.x; e < total; e += gridDim.x * 256) {
      const int2 t = p.entries_out[e];  // (kx, ix)
      int found = 0;
      for (int j = p.row_ptr_in[t.y]; j < p.row_ptr_in[t.y + 1]; ++j)
        if (p.entries_in[j].x == t.x) found = j;
      p.plane_of[e] = found;
    }
    return;
  }
  const int ix = blockIdx.y / p.kblocks, kb = blockIdx.y % p.kblocks;
  const int e0 = p.row_ptr_in[ix];
  const int cols = (p.row_ptr_in[ix + 1] - e0) * p.AN;
  const int n_pad = pad16(cols);
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= 64 * n_pad) return;  // also rows without entries
  const int part = j / (32 * n_pad), r1 = j % (32 * n_pad);
  const int c = r1 / (4 * n_pad), r2 = r1 % (4 * n_pad);
  const int col = r2 >> 2, b = kb * kKB + 4 * c + (r2 & 3);
  float v = 0.f;
  if (col < cols && b < p.B) {
    const int e = col / p.AN, a = (col % p.AN) / p.nky, k = col % p.nky;
    const int ky = p.By < 0 ? p.nky - 1 - k : k;
    const int kx = p.entries_in[e0 + e].x;
    const float w = p.w[a * p.w_sa + b * p.w_sb + (long long)kx * p.nky + ky];
    const float hi = tf32_hi(w);
    v = part ? w - hi : hi;
  }
  p.b_pack[(size_t)blockIdx.y * 64 * p.n_max_pad + j] = v;
}

template <int NKY>
__global__ void __launch_bounds__(kThreads, 1)
tc_scatter_kernel(const TsParams p, const __grid_constant__ CUtensorMap in_map) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Control *ctl = reinterpret_cast<Control *>(smem);
  unsigned char *raw_base = smem + kHeaderBytes;
  unsigned char *b_base = raw_base + kRawStages * kRawBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // TMEM lane 32 w + i holds staged position (32 - halo) w + i: the quadrants overlap by the taps' reach, so
  // that every output of a quadrant finds its NKY rows inside the quadrant (the epilogue needs no exchange
  // between warps); a tile emits 4 (32 - halo) outputs.
  constexpr int kHalo = NKY - 1;
  constexpr int kQuadOut = 32 - kHalo;

  for (int i = tid; i <= p.nix; i += kThreads) ctl->rp[i] = p.row_ptr_in[i];
  if (tid == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      tc::mbar_init(&ctl->raw_full[s], 1);
      tc::mbar_init(&ctl->raw_empty[s], kConvertThreads);
    }
    for (int s = 0; s < kOpStages; ++s) {
      tc::mbar_init(&ctl->a_full[s], kConvertThreads);
      tc::mbar_init(&ctl->a_empty[s], 1);
    }
    for (int s = 0; s < kBStages; ++s) {
      tc::mbar_init(&ctl->b_full[s], 1);
      tc::mbar_init(&ctl->b_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      tc::mbar_init(&ctl->acc_full[s], 1);
      tc::mbar_init(&ctl->acc_empty[s], kEpilogueWarps * 32);
    }
    ctl->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tc::tmem_alloc(&ctl->tmem_base, kTmemCols);  // two accumulator tiles, then the operand A ring
    tc::tmem_relinquish();
  }
  tc::launch_dependents();      // the plane sum may be scheduled; it waits for this grid before reading
  tc::grid_dependency_wait();   // the weight operands and the plane index come from the kernel before
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const int *rp = ctl->rp;

  if (warp < kEpilogueWarps) {
    // ===================== epilogue: TMEM -> sums over the taps (lane shuffles) -> partial planes =====================
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int q = kQuadOut * warp + lane;  // tile-local output position of this lane
    const bool emits = lane < kQuadOut;
    int j = 0;
    PROF_BEGIN();
#ifdef MELLIN_TUNING_HOOKS
    long long prof_ld = 0, prof_sum = 0;
#endif
    for (ItemIter it(p); it.id < p.total; it.next(p)) {
      const int e0 = rp[it.ix];
      const int nea = (rp[it.ix + 1] - e0) * p.A;  // (entry, a) pairs: NKY columns each
      if (nea == 0) continue;
      const int buf = j & 1;
      PROF_WAIT_START();
      const bool ok = tc::mbar_wait(&ctl->acc_full[buf], (uint32_t)((j >> 1) & 1), kSpinLimit);
      PROF_WAIT_END();
      if (!__all_sync(0xffffffffu, ok)) {
        raise_timeout(ctl, 4);
        break;
      }
      tc::tc_fence_after_sync();
      const int pos = it.yt * p.T + q;  // plane position; position 0 = output position -shift
      const bool store = emits && pos < p.noy + p.shift;
      float *dst = p.planes + ((size_t)it.n * p.entries + e0) * p.A * p.plane + pos;
      const uint32_t acc = tmem_base + lane_base + (uint32_t)buf * kBufCols;
      for (int c0 = 0; c0 < nea; c0 += 16) {
        // 16 (entry, a) pairs = 16 NKY consecutive columns
        uint32_t v[NKY][16];
#ifdef MELLIN_TUNING_HOOKS
        const long long ld_t0 = clock64();
#endif
#pragma unroll
        for (int t = 0; t < NKY; ++t) tc::tmem_ld16(acc + (uint32_t)(c0 * NKY + 16 * t), v[t]);
        tc::tmem_ld_wait();
#ifdef MELLIN_TUNING_HOOKS
        prof_ld += clock64() - ld_t0;
#endif
        if (c0 + 16 >= nea) {
          // last read of this tile: the MMAs of the item after next may overwrite it
          tc::tc_fence_before_sync();
          tc::mbar_arrive(&ctl->acc_empty[buf]);
        }
        // all the shuffles first, in converged code; the stores (lane-dependent) after them
        float sums[16];
        const int left = nea - c0;  // warp-uniform
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (8 * half < left) {  // the second eight pairs only where the row has them
#pragma unroll
            for (int jj = 8 * half; jj < 8 * half + 8; ++jj) {
              sums[jj] = __uint_as_float(v[(jj * NKY) / 16][(jj * NKY) % 16]);
#pragma unroll
              for (int k = 1; k < NKY; ++k)
                sums[jj] += __shfl_down_sync(0xffffffffu, __uint_as_float(v[(jj * NKY + k) / 16][(jj * NKY + k) % 16]), k);
            }
          }
        }
        if (store) {
          float *d = dst + (size_t)c0 * p.plane;
#pragma unroll
          for (int jj = 0; jj < 16; ++jj)
            if (jj < left) d[(size_t)jj * p.plane] = sums[jj];
        }
#ifdef MELLIN_TUNING_HOOKS
        prof_sum += clock64() - ld_t0;
#endif
      }
      ++j;
    }
    if (warp == 0) { PROF_END(0); }
#ifdef MELLIN_TUNING_HOOKS
    if (blockIdx.x == 0 && tid == 0) g_ts_prof[14] = prof_ld, g_ts_prof[15] = prof_sum;
#endif
  } else if (warp < kMmaWarp) {
    // ===================== converters: raw [channel][position] -> hi / lo rows of operand A in TMEM =====================
    const int cw = warp - kEpilogueWarps;
    const int quad = cw & 3, half = cw >> 2;  // TMEM lane quadrant (= warp index mod 4), 16-channel half of the stage
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const int pos = kQuadOut * quad + lane;
    int st = 0;
    bool failed = false;
    PROF_BEGIN();
    for (ItemIter it(p); it.id < p.total && !failed; it.next(p)) {
      if (rp[it.ix + 1] == rp[it.ix]) continue;
      for (int kb = 0; kb < p.kblocks; ++kb, ++st) {
        const int r = st % kRawStages, s = st % kOpStages;
        PROF_WAIT_START();
        const bool ok = tc::mbar_wait(&ctl->raw_full[r], (uint32_t)((st / kRawStages) & 1), kSpinLimit) &&
                        tc::mbar_wait(&ctl->a_empty[s], (uint32_t)(((st / kOpStages) & 1) ^ 1), kSpinLimit);
        PROF_WAIT_END();
        if (!__all_sync(0xffffffffu, ok)) {
          raise_timeout(ctl, 1);
          failed = true;
          break;
        }
        tc::tc_fence_after_sync();
        const float *raw = reinterpret_cast<const float *>(raw_base + (size_t)r * kRawBytes) + (16 * half) * kTM + pos;
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float v = raw[i * kTM];
          const float h = tf32_hi(v);
          hi[i] = __float_as_uint(h), lo[i] = __float_as_uint(v - h);
        }
        const uint32_t col = kACol0 + (uint32_t)s * kAStageCols + 16u * half;
        tc::tmem_st16(tmem_base + lane_base + col, hi);
        tc::tmem_st16(tmem_base + lane_base + col + kKB, lo);
        tc::tmem_st_wait();
        tc::tc_fence_before_sync();
        // the proxy fence orders this thread's reads of the raw slot before the copy engine's next write into it
        tc::fence_proxy_async();
        tc::mbar_arrive(&ctl->raw_empty[r]);
        tc::mbar_arrive(&ctl->a_full[s]);
      }
    }
    if (warp == kEpilogueWarps) { PROF_END(1); }
  } else if (warp == kCopyWarp) {
    // ===================== copy issuer: boxes of `in` =====================
    if (lane == 0) {
      int st = 0;
      bool failed = false;
      PROF_BEGIN();
      for (ItemIter it(p); it.id < p.total && !failed; it.next(p)) {
        if (rp[it.ix + 1] == rp[it.ix]) continue;
        const int start = it.yt * p.T - p.shift + p.ws0;  // a multiple of 4
        for (int kb = 0; kb < p.kblocks; ++kb, ++st) {
          const int r = st % kRawStages;
          PROF_WAIT_START();
          const bool ok = tc::mbar_wait(&ctl->raw_empty[r], (uint32_t)(((st / kRawStages) & 1) ^ 1), kSpinLimit);
          PROF_WAIT_END();
          if (!ok) {
            raise_timeout(ctl, 5);
            failed = true;
            break;
          }
          tc::mbar_arrive_expect_tx(&ctl->raw_full[r], kRawBytes);
          tc::tma_load_4d(raw_base + (size_t)r * kRawBytes, &in_map, start, it.ix, it.n, kb * kKB, &ctl->raw_full[r]);
        }
      }
      PROF_END(3);
    }
    __syncwarp();
  } else if (warp == kCopyBWarp) {
    // ===================== copy issuer: B operands =====================
    if (lane == 0) {
      int st = 0;
      bool failed = false;
      for (ItemIter it(p); it.id < p.total && !failed; it.next(p)) {
        const int cols = (rp[it.ix + 1] - rp[it.ix]) * p.AN;
        if (cols == 0) continue;
        const uint32_t b_bytes = 256u * (uint32_t)pad16(cols);
        const float *b_src = p.b_pack + (size_t)it.ix * p.kblocks * 64 * p.n_max_pad;
        for (int kb = 0; kb < p.kblocks; ++kb, ++st) {
          const int s = st % kBStages;
          if (!tc::mbar_wait(&ctl->b_empty[s], (uint32_t)(((st / kBStages) & 1) ^ 1), kSpinLimit)) {
            raise_timeout(ctl, 6);
            failed = true;
            break;
          }
          tc::mbar_arrive_expect_tx(&ctl->b_full[s], b_bytes);
          tc::bulk_load(b_base + (size_t)s * p.b_stage_bytes, b_src + (size_t)kb * 64 * p.n_max_pad, b_bytes,
                        &ctl->b_full[s]);
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer =====================
    // The whole warp walks the items; one elected lane issues.  Everything an MMA names is computed from
    // warp-uniform values (what comes from shared memory is broadcast from lane 0 to say so).
    {
      const uint32_t tmem0 = tc::uniform(tmem_base);
      // B descriptors: the start address (16-byte units) and the chunk pitch share the low word, the 128-byte
      // pitch of the 8-column groups and the version bit sit in the high word
      const uint32_t b0 = tc::smem_u32(b_base) >> 4;
      const uint64_t desc_hi_word = tc::smem_desc(0u, 0u, 128u);
      int st = 0, j = 0;
      bool failed = false;
      PROF_BEGIN();
#ifdef MELLIN_TUNING_HOOKS
      long long prof_acc = 0;
#endif
      for (ItemIter it(p); it.id < p.total && !failed; it.next(p)) {
        const int cols = (int)tc::uniform((uint32_t)(rp[it.ix + 1] - rp[it.ix])) * p.AN;
        if (cols == 0) continue;
        const int n_pad = pad16(cols);
        const uint32_t idesc = tc::idesc_tf32(kTM, n_pad);
        const uint32_t b_chunk = (uint32_t)n_pad;       // 16-byte units per 4-channel chunk of B
        const uint32_t lbo_bits = (b_chunk & 0x3FFFu) << 16;
        const int buf = j & 1;
        PROF_WAIT_START();
        const bool acc_ok = tc::mbar_wait(&ctl->acc_empty[buf], (uint32_t)(((j >> 1) & 1) ^ 1), kSpinLimit);
        PROF_WAIT_END();
#ifdef MELLIN_TUNING_HOOKS
        prof_acc += clock64() - prof_t1;
#endif
        if (!__all_sync(0xffffffffu, acc_ok)) {
          if (lane == 0) raise_timeout(ctl, 3);
          failed = true;
          break;
        }
        const uint32_t d0 = tmem0 + (uint32_t)buf * kBufCols;
        uint32_t fresh = 0;  // 0: the next MMA overwrites the accumulators
        for (int kb = 0; kb < p.kblocks; ++kb, ++st) {
          const int s = st % kOpStages, sb = st % kBStages;
          PROF_WAIT_START();
          const bool ok = tc::mbar_wait(&ctl->a_full[s], (uint32_t)((st / kOpStages) & 1), kSpinLimit) &&
                          tc::mbar_wait(&ctl->b_full[sb], (uint32_t)((st / kBStages) & 1), kSpinLimit);
          PROF_WAIT_END();
          if (!__all_sync(0xffffffffu, ok)) {
            if (lane == 0) raise_timeout(ctl, 2);
            failed = true;
            break;
          }
          tc::tc_fence_after_sync();
          const uint32_t a_hi = tmem0 + kACol0 + (uint32_t)s * kAStageCols, a_lo = a_hi + kKB;
          const uint32_t b_hi = b0 + (uint32_t)sb * (p.b_stage_bytes >> 4), b_lo = b_hi + 8u * b_chunk;
          if (tc::elect_one()) {
#pragma unroll
            for (int ks = 0; ks < kKB / 8; ++ks) {
              const uint32_t bo = (uint32_t)ks * 2u * b_chunk;
              const uint64_t db_hi = desc_hi_word | (uint64_t)(((b_hi + bo) & 0x3FFFu) | lbo_bits);
              const uint64_t db_lo = desc_hi_word | (uint64_t)(((b_lo + bo) & 0x3FFFu) | lbo_bits);
              // the three products of the hi/lo split, smallest first
              tc::mma_tf32_a_tmem(d0, a_lo + 8u * ks, db_hi, idesc, fresh);
              tc::mma_tf32_a_tmem(d0, a_hi + 8u * ks, db_lo, idesc, 1u);
              tc::mma_tf32_a_tmem(d0, a_hi + 8u * ks, db_hi, idesc, 1u);
              fresh = 1u;
            }
            tc::tc_commit(&ctl->a_empty[s]);
            tc::tc_commit(&ctl->b_empty[sb]);
            if (kb == p.kblocks - 1) tc::tc_commit(&ctl->acc_full[buf]);
          }
          fresh = 1u;
          __syncwarp();
        }
        if (failed) break;
        ++j;
      }
      PROF_END(2);
#ifdef MELLIN_TUNING_HOOKS
      if (blockIdx.x == 0 && lane == 0) g_ts_prof[12] = prof_acc, g_ts_prof[13] = j;
#endif
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// out[n, a, ox, oy] = init + sum of the planes of row ox's entries, in table order.
// A block owns (n, ox, a); a thread takes groups of 4 consecutive positions, so that up to
// 4 x entries independent loads are in flight per thread (the planes were written a moment
// ago: most of them are still in L2).
__global__ void __launch_bounds__(128)
gather_planes_kernel(const TsParams p, int vec_store) {
  __shared__ int pid[kMaxEntries];
  int bid = blockIdx.x;
  const int a = bid % p.A;
  bid /= p.A;
  const int ox = bid % p.nox, n = bid / p.nox;
  const int e0 = p.row_ptr_out[ox];
  const int np = min(p.row_ptr_out[ox + 1] - e0, kMaxEntries);
  tc::grid_dependency_wait();  // the planes (and, before them, the plane index) come from the kernels before
  if ((int)threadIdx.x < np) pid[threadIdx.x] = p.plane_of[e0 + threadIdx.x];
  __syncthreads();
  const float *__restrict__ base = p.planes + ((size_t)n * p.entries * p.A + a) * p.plane + p.shift;
  const size_t entry_pitch = (size_t)p.A * p.plane;
  float *out_row = p.out + n * p.out_sn + a * p.out_sa + (long long)ox * p.noy;
  const float bias = (!p.accumulate && p.bias != nullptr) ? __ldg(p.bias + a) : 0.f;
  for (int oy = 4 * threadIdx.x; oy < p.noy; oy += 4 * 128) {
    float *out = out_row + oy;
    float v[4] = {bias, bias, bias, bias};
    if (vec_store && oy + 3 < p.noy) {
      if (p.accumulate) {
        const float4 old = *reinterpret_cast<const float4 *>(out);
        v[0] = old.x, v[1] = old.y, v[2] = old.z, v[3] = old.w;
      }
      for (int e = 0; e < np; ++e) {
        const float *src = base + (size_t)pid[e] * entry_pitch + oy;
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += __ldcg(src + j);
      }
      *reinterpret_cast<float4 *>(out) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      for (int j = 0; j < 4 && oy + j < p.noy; ++j) {
        float sum = p.accumulate ? out[j] : bias;
        for (int e = 0; e < np; ++e) sum += __ldcg(base + (size_t)pid[e] * entry_pitch + oy + j);
        out[j] = sum;
      }
    }
  }
}

size_t round256(size_t v) { return (v + 255) / 256 * 256; }

struct TsPlan {
  TsParams params;
  size_t smem = 0, b_pack_bytes = 0, planes_bytes = 0, index_bytes = 0;
  size_t total() const { return b_pack_bytes + planes_bytes + index_bytes; }
  int blocks = 0;
};

// Needs p.table_by_in.num_entries and .max_row (an upper bound will do for a workspace query).
bool plan_tc_scatter(const DirectProblem<float> &p, TsPlan &plan) {
  if (p.Dy != 1 || p.Ay != 1 || p.accumulate) return false;
  if (p.A < 1 || p.A > 4 || p.nky < 1 || p.nky > 3 || p.B < 16 || p.B > 256) return false;
  if (p.nky > 1 && p.By != 1 && p.By != -1) return false;
  if (p.nkx < 1 || p.noy < 64 || p.nox < 1 || p.N < 1 || p.nix < 1 || p.nix > kMaxRows) return false;
  if (p.table_by_in.num_entries < 1 || p.table_by_in.max_row < 1 || p.table_by_in.max_row > kMaxEntries) return false;
  if (p.table.max_row > kMaxEntries) return false;
  if (p.table_by_in.row_ptr != nullptr && p.table_by_in.rows != p.nix) return false;
  const int AN = p.A * p.nky;
  if (AN * p.table_by_in.max_row > kMaxCols) return false;
  // rows are copied in 16-byte chunks
  if (p.niy % 4 != 0 || reinterpret_cast<uintptr_t>(p.in) % 16 != 0 || p.in_sn % 4 != 0 || p.in_sb % 4 != 0)
    return false;
  TsParams &q = plan.params;
  q.row_ptr_in = p.table_by_in.row_ptr, q.entries_in = p.table_by_in.entries;
  q.row_ptr_out = p.table.row_ptr, q.entries_out = p.table.entries;
  q.w = p.w, q.bias = p.bias, q.out = p.out;
  q.w_sa = p.w_sa, q.w_sb = p.w_sb, q.out_sn = p.out_sn, q.out_sa = p.out_sa;
  q.entries = p.table_by_in.num_entries;
  q.N = p.N, q.A = p.A, q.B = p.B, q.nkx = p.nkx, q.nky = p.nky, q.nix = p.nix, q.nox = p.nox, q.noy = p.noy, q.By = p.By;
  q.AN = AN;
  q.T = kTM - 4 * (p.nky - 1);  // four lane quadrants, each short of the taps' reach
  q.ws0 = p.Cy + std::min(0, p.By * (p.nky - 1));
  q.shift = ((q.ws0 % 4) + 4) % 4;
  q.y_tiles = (p.noy + q.shift + q.T - 1) / q.T;
  q.plane = q.y_tiles * q.T;
  q.kblocks = (p.B + kKB - 1) / kKB;
  q.n_max_pad = (AN * p.table_by_in.max_row + 15) / 16 * 16;
  const long long total = (long long)p.N * p.nix * q.y_tiles;
  if (total >= (1LL << 30)) return false;
  q.total = (int)total;
  q.accumulate = 0;
  q.b_stage_bytes = 256u * (uint32_t)q.n_max_pad;
  plan.smem = kHeaderBytes + (size_t)kRawStages * kRawBytes + (size_t)kBStages * q.b_stage_bytes;
  plan.smem = std::max<size_t>(plan.smem, 116 * 1024);  // one block per SM
  if (plan.smem > 227 * 1024) return false;
  plan.b_pack_bytes = round256((size_t)p.nix * q.kblocks * 64 * q.n_max_pad * sizeof(float));
  plan.planes_bytes = round256((size_t)p.N * q.entries * p.A * q.plane * sizeof(float));
  plan.index_bytes = round256((size_t)q.entries * sizeof(int));
  plan.blocks = (int)std::min<long long>(sm_count(), total);
  return true;
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

}  // namespace

// Reads and clears this kernel's timeout flag of the current device (synchronises it).
int tc_scatter_take_error(int *code) {
  int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(code, g_tc_scatter_error, sizeof(int));
  if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_tc_scatter_error, &zero, sizeof(int));
  return err == cudaSuccess ? MELLIN_OK : fail(MELLIN_ERR_LAUNCH, std::string("device status: ") + cudaGetErrorString(err));
}

#ifdef MELLIN_TUNING_HOOKS
extern "C" int mellin_tc_scatter_profile(long long *out) {
  return cudaMemcpyFromSymbol(out, g_ts_prof, 16 * sizeof(long long)) == cudaSuccess ? 0 : 2;
}
#endif

// scratch for the B operands and the partial planes (0 = problem not covered by this kernel);
// needs p.table_by_in.num_entries and .max_row
size_t tc_scatter_workspace_bytes(const DirectProblem<float> &p) {
  TsPlan plan;
  if (!plan_tc_scatter(p, plan)) return 0;
  return plan.total();
}

// MELLIN_ERR_UNSUPPORTED when the problem is outside this kernel's coverage or the workspace too small.
int launch_tc_scatter(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  TsPlan plan;
  if (p.table_by_in.row_ptr == nullptr || p.table.row_ptr == nullptr || !plan_tc_scatter(p, plan))
    return MELLIN_ERR_UNSUPPORTED;
  if (workspace == nullptr || workspace_bytes < plan.total() ||
      reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return MELLIN_ERR_UNSUPPORTED;
  EncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr) return MELLIN_ERR_UNSUPPORTED;
  CUtensorMap in_map;
  {
    // the reduced tensor as (position, Mellin row, batch, channel) with its real strides;
    // a box is 128 positions of each of 32 consecutive channels
    const cuuint64_t dims[4] = {(cuuint64_t)p.niy, (cuuint64_t)p.nix, (cuuint64_t)p.N, (cuuint64_t)p.B};
    const cuuint64_t strides[3] = {(cuuint64_t)p.niy * sizeof(float), (cuuint64_t)p.in_sn * sizeof(float),
                                   (cuuint64_t)p.in_sb * sizeof(float)};
    const cuuint32_t box[4] = {(cuuint32_t)kTM, 1u, 1u, (cuuint32_t)kKB};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    if (encode(&in_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(p.in), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return MELLIN_ERR_UNSUPPORTED;
  }
  TsParams &q = plan.params;
  unsigned char *base = static_cast<unsigned char *>(workspace);
  q.b_pack = reinterpret_cast<float *>(base);
  q.planes = reinterpret_cast<float *>(base + plan.b_pack_bytes);
  q.plane_of = reinterpret_cast<int *>(base + plan.b_pack_bytes + plan.planes_bytes);
  pack_scatter_b_kernel<<<dim3((unsigned)((64 * q.n_max_pad + 255) / 256), (unsigned)(p.nix * q.kblocks + 1)), 256, 0, stream>>>(q);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("pack_scatter_b_kernel: ") + cudaGetErrorString(err));
  count_launch();
  auto kernel = p.nky == 1 ? tc_scatter_kernel<1> : p.nky == 2 ? tc_scatter_kernel<2> : tc_scatter_kernel<3>;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  err = launch_after_predecessor(kernel, dim3(plan.blocks), dim3(kThreads), plan.smem, stream, q, in_map);
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("tc_scatter_kernel: ") + cudaGetErrorString(err));
  count_launch();
  const int vec_store =
      (reinterpret_cast<uintptr_t>(p.out) % 16 == 0 && p.noy % 4 == 0 && p.out_sn % 4 == 0 && p.out_sa % 4 == 0) ? 1 : 0;
  err = launch_after_predecessor(gather_planes_kernel, dim3((unsigned)(p.N * p.nox * p.A)), dim3(128), 0, stream, q, vec_store);
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("gather_planes_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

}  // namespace mellin
