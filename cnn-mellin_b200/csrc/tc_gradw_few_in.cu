// Weight (+ bias) gradient of a layer with FEW INPUT channels (at most 4) on tensor cores
// (tcgen05, sm_100a) -- the first layer of a model (3 feature maps in, up to 64 x tiles out):
//
//   gw[a, b, kx, ky] = sum_n sum_{ox : (kx, ix) in row ox} sum_oy
//                      go[n, a, ox, oy] * x[n, b, ix, oy + By * ky + Cy]
//   gb[a]            = sum_{n, ox, oy} go[n, a, ox, oy]
//
// The big operand is grad_y and it is read ONCE: an item is (output row ox, channel tile,
// n, 128 positions), and one GEMM serves every table entry (kx, ix) of row ox at a time,
//
//   D[a, (entry, b, tap)] += sum_oy go[a, oy] * x[b, ix(entry), oy + tap]        (K = positions)
//
// with the 128 positions of an item taken as TWO halves of 64 stacked along M, so that an
// MMA has 128 rows: row (h, a) is channel a over the positions of half h, column
// (h', entry, b, tap) the shifted input row over the positions of half h'; the blocks h = h'
// are the sums wanted (the other two are computed and ignored -- the tensor pipe idles
// anyway, the MMA count is what costs).
//
//   A : grad_y, in TENSOR MEMORY.  One 4-D TMA box per item (64 channels x 132 positions,
//       zero-filled outside the tensor); converter warps split it into TF32 hi / lo parts
//       and write them with tcgen05.st (lane = (half, channel), columns = positions) while
//       summing what they convert for the bias gradient.
//   B : the shifted input rows, K-major in shared memory, built by the same warps from a
//       few small boxes of x (one per table entry), hi / lo.
//   3 MMAs (lo*hi, hi*lo, hi*hi) per 8 positions, issued by one elected lane of a converged warp.
//   The tensor core's accumulator rounds toward zero at every MMA, so sums are kept in two
//   levels, both in TMEM: level 1 takes at most 96 chained MMAs; the epilogue warps then add
//   it into level 2 with ordinary FP32 adds (tcgen05.ld / st).
//
// Items are ordered by (ox, channel tile) and every block takes one contiguous run of them,
// so a block meets at most a few different (ox, channel tile) "segments"; at the end of a
// segment its level-2 sums go to a partial buffer, and a second kernel adds the partials of
// every weight in a fixed order (no floating-point atomics: results are bit-reproducible).
// 15 warps: 4 epilogue, 4 + 4 converter (grad_y / x), 1 MMA issuer, 2 copy issuers.  Every wait is bounded
// and reports through a device word.
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
constexpr int kCopyWarp = kMmaWarp + 1;    // boxes of grad_y
constexpr int kCopyXWarp = kCopyWarp + 1;  // boxes of x
constexpr int kThreads = (kCopyXWarp + 1) * 32;
constexpr int kTP = 128;           // positions per item
constexpr int kHalf = 64;          // ... in two halves stacked along M
constexpr int kSK = 32;            // positions of each half per stage (4 k-steps): two stages per item
constexpr int kStagesPerItem = kHalf / kSK;
constexpr int kCo = 64;            // output channels per item
constexpr int kGoRow = 132;        // staged positions per grad_y row: a pitch that keeps 16-byte column reads free of bank conflicts
constexpr uint32_t kGoBytes = kCo * kGoRow * 4;  // 33792
constexpr int kGoStages = 3;
constexpr int kXRow = 136;         // staged positions per x row: 128 + lead (<= 3) + taps - 1 (<= 2), rounded to 16 bytes
constexpr int kBoxChannels = 4;
constexpr int kMaxEntries = 8;     // per output row
constexpr uint32_t kXEntryBytes = kBoxChannels * kXRow * 4;  // 2176
constexpr uint32_t kXBytes = kMaxEntries * kXEntryBytes;
constexpr int kXStages = 2;
constexpr int kMaxK1 = 80;         // entries x B x taps of a row, rounded to 16: columns of one half
constexpr int kOpStages = 3;       // operand A sets in tensor memory (64 columns each: hi, lo)
constexpr int kBStages = 2;
constexpr int kPromote = 8;        // stages per level-1 interval: 8 x 12 = 96 chained MMAs
constexpr uint32_t kL1Col = 0, kL2Col = 2 * kMaxK1, kACol0 = 4 * kMaxK1;  // 160 + 160 + 3 x 64 = 512 columns
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxTable = 640;
constexpr int kMaxRows = 256;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr int kHeaderBytes = 8192;

struct Control {
  uint64_t go_full[kGoStages], go_empty[kGoStages], x_full[kXStages], x_empty[kXStages];
  uint64_t a_full[kOpStages], a_empty[kOpStages], b_full[kBStages], b_empty[kBStages];
  uint64_t l1_full, l1_empty;
  uint32_t tmem_base;
  int abort;
  int first, last;        // this block's run of items
  int rp[kMaxRows + 1];   // the by-output-row table's row offsets
  int2 ent[kMaxTable];    // its entries (kx, ix)
};
static_assert(sizeof(Control) <= kHeaderBytes, "Control must fit the header");

// First bounded wait that gave up since the last query (0 = none): 1 converters, 2 MMA issuer (operands),
// 3 MMA issuer (level-1 sums), 4 epilogue, 5 copy issuer (grad_y), 6 copy issuer (x).
__device__ int g_tc_gwfi_error = 0;

#ifdef MELLIN_TUNING_HOOKS
// per-role wait / work cycles of block 0: 0 epilogue, 1 converter, 2 MMA issuer, 3 copy issuer (grad_y)
__device__ long long g_gf_prof[16];
#define PROF_BEGIN() long long prof_t0 = clock64(), prof_wait = 0, prof_t1 = 0
#define PROF_WAIT_START() prof_t1 = clock64()
#define PROF_WAIT_END() prof_wait += clock64() - prof_t1
#define PROF_END(slot)                                           \
  if (blockIdx.x == 0 && lane == 0) {                            \
    g_gf_prof[2 * (slot)] = prof_wait;                           \
    g_gf_prof[2 * (slot) + 1] = clock64() - prof_t0 - prof_wait; \
  }
#else
#define PROF_BEGIN()
#define PROF_WAIT_START()
#define PROF_WAIT_END()
#define PROF_END(slot)
#endif

struct GfParams {
  const int32_t *row_ptr;  // rows = ox, entries (kx, ix)
  const int2 *entries;
  float *part_w;           // [block][segment][half][column (kMaxK1)][channel (64)]
  float *part_b;           // [block][channel tile][half][channel (64)]
  float *gw, *gb;
  int N, A, B, nkx, nky, nox, noy, By;
  int BK;                  // B * nky: columns per entry
  int y_tiles, a_tiles;
  int lead, ws0;           // x box start = tile start + ws0 - lead (a multiple of 4); tap t of position oy reads staged oy + t + lead
  int per_segment;         // items of one (ox, channel tile): N * y_tiles
  int total;               // items
  int seg_max;             // segments a block can meet
  int num_entries;
  int k1p_max;             // widest half of the launch (columns, multiple of 16)
  uint32_t b_stage_bytes;  // 2 parts x 8 chunks x (2 k1p_max + 1) rows x 16 bytes
};

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ void raise_timeout(Control *ctl, int code) {
  atomicCAS(&g_tc_gwfi_error, 0, code);
  ctl->abort = 1;
}
__device__ __forceinline__ int pad16(int v) { return (v + 15) & ~15; }

// Blocks take contiguous runs of the (ox, channel tile, n, y tile) order, cut so that every run costs about the
// same: an item of a row with E table entries is weighted 7 + E (the work that does not depend on the entries --
// converting grad_y -- against the rows of B to build and the width of the MMAs).  first_item(b) is the first item
// of block b's run, first_item(nblocks) the number of items: a pure function of the table, so that the kernel and
// the reduction agree on it.
constexpr int kItemWeight = 7;
__device__ int first_item(const GfParams &p, const int *row_ptr, int b, int nblocks) {
  const int nseg = p.nox * p.a_tiles;
  long long total_weight = 0;
  for (int seg = 0; seg < nseg; ++seg) {
    const int ox = seg / p.a_tiles;
    total_weight += (long long)p.per_segment * (kItemWeight + row_ptr[ox + 1] - row_ptr[ox]);
  }
  const long long target = total_weight * b / nblocks;
  long long acc = 0;
  for (int seg = 0; seg < nseg; ++seg) {
    const int ox = seg / p.a_tiles;
    const int w = kItemWeight + row_ptr[ox + 1] - row_ptr[ox];
    const long long ws = (long long)p.per_segment * w;
    if (acc + ws > target) return seg * p.per_segment + (int)((target - acc + w - 1) / w);
    acc += ws;
  }
  return p.total;
}

struct Item {
  int seg, ox, at, n, yt;  // seg = ox * a_tiles + at
};
__device__ __forceinline__ Item decode(const GfParams &p, int i) {
  Item it;
  it.seg = i / p.per_segment;
  const int r = i - it.seg * p.per_segment;
  it.ox = it.seg / p.a_tiles, it.at = it.seg - it.ox * p.a_tiles;
  it.n = r / p.y_tiles, it.yt = r - it.n * p.y_tiles;
  return it;
}

template <int NB, int NKY>
__global__ void __launch_bounds__(kThreads, 1)
tc_gradw_few_in_kernel(const GfParams p, const __grid_constant__ CUtensorMap go_map, const __grid_constant__ CUtensorMap x_map) {
  constexpr int BK = NB * NKY;
  extern __shared__ __align__(1024) unsigned char smem[];
  Control *ctl = reinterpret_cast<Control *>(smem);
  unsigned char *go_base = smem + kHeaderBytes;
  unsigned char *x_base = go_base + kGoStages * kGoBytes;
  unsigned char *b_base = x_base + kXStages * kXBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int i = tid; i <= p.nox; i += kThreads) ctl->rp[i] = p.row_ptr[i];
  for (int i = tid; i < p.num_entries; i += kThreads) ctl->ent[i] = p.entries[i];
  // rows of B past a half's real columns are never written again: give them a finite value once
  for (uint32_t i = tid; i < kBStages * p.b_stage_bytes / 16; i += kThreads)
    reinterpret_cast<float4 *>(b_base)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (tid == 0) {
    for (int s = 0; s < kGoStages; ++s) {
      tc::mbar_init(&ctl->go_full[s], 1);
      tc::mbar_init(&ctl->go_empty[s], kConvertThreads / 2);
    }
    for (int s = 0; s < kXStages; ++s) {
      tc::mbar_init(&ctl->x_full[s], 1);
      tc::mbar_init(&ctl->x_empty[s], kConvertThreads / 2);
    }
    for (int s = 0; s < kOpStages; ++s) {
      tc::mbar_init(&ctl->a_full[s], kConvertThreads / 2);
      tc::mbar_init(&ctl->a_empty[s], 1);
    }
    for (int s = 0; s < kBStages; ++s) {
      tc::mbar_init(&ctl->b_full[s], kConvertThreads / 2);
      tc::mbar_init(&ctl->b_empty[s], 1);
    }
    tc::mbar_init(&ctl->l1_full, 1);
    tc::mbar_init(&ctl->l1_empty, kEpilogueWarps * 32);
    ctl->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tc::tmem_alloc(&ctl->tmem_base, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::launch_dependents();  // the reduction may be scheduled; it waits for this grid before reading the partial sums
  tc::fence_proxy_async();  // the zero fill above, before the tensor core reads those rows
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  if (tid < 2) (tid == 0 ? ctl->first : ctl->last) = first_item(p, ctl->rp, blockIdx.x + tid, gridDim.x);
  __syncthreads();
  const uint32_t tmem_base = ctl->tmem_base;
  const int *rp = ctl->rp;
  const int first = ctl->first, last = ctl->last;
  const int seg_first = first < last ? first / p.per_segment : 0;

  if (warp < kEpilogueWarps) {
    // ===================== epilogue: level-1 -> level-2 promotion; partial sums at the end of a segment =====================
    // lane (h, a): only the columns of half h are sums that are wanted
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int h = warp >> 1, a = 32 * (warp & 1) + lane;
    int iv = 0;  // level-1 intervals seen
    bool failed = false;
    PROF_BEGIN();
    for (int i = first; i < last && !failed;) {
      const Item it = decode(p, i);
      const int seg_end = min(last, (it.seg + 1) * p.per_segment);
      const int k1 = (rp[it.ox + 1] - rp[it.ox]) * BK;
      if (k1 == 0) {
        i = seg_end;
        continue;
      }
      const int k1p = pad16(k1);
      const int stages = (seg_end - i) * kStagesPerItem;
      const int intervals = (stages + kPromote - 1) / kPromote;
      const uint32_t l1 = tmem_base + lane_base + kL1Col + (uint32_t)(h * k1p);
      const uint32_t l2 = tmem_base + lane_base + kL2Col + (uint32_t)(h * k1p);
      for (int q = 0; q < intervals && !failed; ++q, ++iv) {
        PROF_WAIT_START();
        const bool ok = tc::mbar_wait(&ctl->l1_full, (uint32_t)(iv & 1), kSpinLimit);
        PROF_WAIT_END();
        if (!__all_sync(0xffffffffu, ok)) {
          raise_timeout(ctl, 4);
          failed = true;
          break;
        }
        tc::tc_fence_after_sync();
        for (int g = 0; 16 * g < k1p; ++g) {
          uint32_t va[16], vb[16];
          tc::tmem_ld16(l1 + (uint32_t)(16 * g), va);
          if (q > 0) tc::tmem_ld16(l2 + (uint32_t)(16 * g), vb);
          tc::tmem_ld_wait();
          if (q > 0) {
#pragma unroll
            for (int c = 0; c < 16; ++c) va[c] = __float_as_uint(__uint_as_float(va[c]) + __uint_as_float(vb[c]));
          }
          if (q + 1 < intervals) {
            tc::tmem_st16(l2 + (uint32_t)(16 * g), va);
          } else {
            // the segment's sums: partial[block][segment][h][column][channel]
            float *dst = p.part_w + ((((size_t)blockIdx.x * p.seg_max + (it.seg - seg_first)) * 2 + h) * kMaxK1 + 16 * g) * kCo + a;
#pragma unroll
            for (int c = 0; c < 16; ++c)
              if (16 * g + c < k1) dst[c * kCo] = __uint_as_float(va[c]);
          }
        }
        tc::tmem_st_wait();
        tc::tc_fence_before_sync();
        tc::mbar_arrive(&ctl->l1_empty);
      }
      i = seg_end;
    }
    if (warp == 0) { PROF_END(0); }
  } else if (warp < kMmaWarp) {
    // ===================== converters: warps 0-3 grad_y -> operand A in TMEM; warps 4-7 x -> operand B =====================
    const int cw = warp - kEpilogueWarps;
    if (cw < 4) {
      // ---- grad_y: the 32 positions of a stage of this lane's (half, channel) row -> TMEM, hi / lo; bias sum ----
      const int quad = cw;  // TMEM lane quadrant (= warp index mod 4)
      const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
      const int h = quad >> 1, a = 32 * (quad & 1) + lane;
      int sg = 0, sa = 0;  // items seen (grad_y ring), stages of items with entries (A ring)
      float bsum = 0.f, btile[4] = {0.f, 0.f, 0.f, 0.f};  // this segment's sum; the block's sums per channel tile
      bool failed = false;
      PROF_BEGIN();
      for (int i = first; i < last && !failed;) {
        const Item seg_it = decode(p, i);
        const int seg_end = min(last, (seg_it.seg + 1) * p.per_segment);
        const bool has_terms = rp[seg_it.ox + 1] > rp[seg_it.ox];
        for (; i < seg_end && !failed; ++i, ++sg) {
          const int rg = sg % kGoStages;
          PROF_WAIT_START();
          const bool ok = tc::mbar_wait(&ctl->go_full[rg], (uint32_t)((sg / kGoStages) & 1), kSpinLimit);
          PROF_WAIT_END();
          if (!__all_sync(0xffffffffu, ok)) {
            raise_timeout(ctl, 1);
            failed = true;
            break;
          }
          const float *go_raw = reinterpret_cast<const float *>(go_base + (size_t)rg * kGoBytes) + a * kGoRow + kHalf * h;
          for (int s = 0; s < kStagesPerItem; ++s) {
            float v[kSK];
#pragma unroll
            for (int c = 0; c < kSK / 4; ++c) {
              const float4 t4 = *reinterpret_cast<const float4 *>(go_raw + kSK * s + 4 * c);
              v[4 * c] = t4.x, v[4 * c + 1] = t4.y, v[4 * c + 2] = t4.z, v[4 * c + 3] = t4.w;
            }
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < kSK; ++c) part += v[c];
            bsum += part;
            if (!has_terms) continue;  // a row no tap reads: it only counts for the bias
            const int so = sa % kOpStages;
            PROF_WAIT_START();
            const bool ok2 = tc::mbar_wait(&ctl->a_empty[so], (uint32_t)(((sa / kOpStages) & 1) ^ 1), kSpinLimit);
            PROF_WAIT_END();
            if (!__all_sync(0xffffffffu, ok2)) {
              raise_timeout(ctl, 1);
              failed = true;
              break;
            }
            tc::tc_fence_after_sync();
            const uint32_t col = tmem_base + lane_base + kACol0 + (uint32_t)so * (2 * kSK);
#pragma unroll
            for (int g = 0; g < kSK / 16; ++g) {
              uint32_t hi[16], lo[16];
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                const float hh = tf32_hi(v[16 * g + c]);
                hi[c] = __float_as_uint(hh), lo[c] = __float_as_uint(v[16 * g + c] - hh);
              }
              tc::tmem_st16(col + 16u * g, hi);
              tc::tmem_st16(col + kSK + 16u * g, lo);
            }
            tc::tmem_st_wait();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&ctl->a_full[so]);
            ++sa;
          }
          // this thread's reads of the raw slot are done (the proxy fence orders them before the copy engine's next write)
          tc::fence_proxy_async();
          tc::mbar_arrive(&ctl->go_empty[rg]);
        }
#pragma unroll
        for (int t4 = 0; t4 < 4; ++t4)
          if (seg_it.at == t4) btile[t4] += bsum;
        bsum = 0.f;
      }
      if (p.part_b != nullptr) {
        // bias partials of the block: [block][channel tile][h][channel]
#pragma unroll
        for (int t4 = 0; t4 < 4; ++t4)
          if (t4 < p.a_tiles) p.part_b[(((size_t)blockIdx.x * p.a_tiles + t4) * 2 + h) * kCo + a] = btile[t4];
      }
      if (cw == 0) { PROF_END(1); }
    } else {
      // ---- x: rows (half, entry, channel, tap) x 8 chunks of 4 positions -> K-major operand B, hi / lo ----
      // thread = (chunk, half, one of 8 row lanes); it reads the 12 staged values around its 4 positions once
      // and writes one row per tap.  Chunks are (n_pad + 1) rows apart: the eight chunk lanes of a warp then
      // store into different banks.
      const int btid = tid - (kEpilogueWarps + 4) * 32;  // 0..127
      const int c = btid & 7, hh = (btid >> 3) & 1;
      const bool lead_bit0 = (p.lead & 1) != 0, lead_bit1 = (p.lead & 2) != 0;
      int sx = 0, sa = 0;  // items with entries seen (x ring), their stages (B ring)
      bool failed = false;
      PROF_BEGIN();
      for (int i = first; i < last && !failed;) {
        const Item seg_it = decode(p, i);
        const int seg_end = min(last, (seg_it.seg + 1) * p.per_segment);
        const int ne = rp[seg_it.ox + 1] - rp[seg_it.ox];
        if (ne == 0) {
          i = seg_end;
          continue;
        }
        const int k1p = pad16(ne * BK);
        const int pitch = 2 * k1p + 1;
        for (; i < seg_end && !failed; ++i, ++sx) {
          const int rx = sx % kXStages;
          PROF_WAIT_START();
          const bool ok = tc::mbar_wait(&ctl->x_full[rx], (uint32_t)((sx / kXStages) & 1), kSpinLimit);
          PROF_WAIT_END();
          if (!__all_sync(0xffffffffu, ok)) {
            raise_timeout(ctl, 1);
            failed = true;
            break;
          }
          const float *x_box = reinterpret_cast<const float *>(x_base + (size_t)rx * kXBytes);
          for (int s = 0; s < kStagesPerItem; ++s, ++sa) {
            const int sb = sa % kBStages;
            PROF_WAIT_START();
            const bool ok2 = tc::mbar_wait(&ctl->b_empty[sb], (uint32_t)(((sa / kBStages) & 1) ^ 1), kSpinLimit);
            PROF_WAIT_END();
            if (!__all_sync(0xffffffffu, ok2)) {
              raise_timeout(ctl, 1);
              failed = true;
              break;
            }
            float4 *b_hi = reinterpret_cast<float4 *>(b_base + (size_t)sb * p.b_stage_bytes);
            float4 *b_lo = b_hi + 8 * pitch;
            for (int rb = btid >> 4; rb < ne * NB; rb += 8) {
              const int e = rb / NB, bb = rb - e * NB;
              const float4 *src = reinterpret_cast<const float4 *>(x_box + (e * kBoxChannels + bb) * kXRow + kHalf * hh + kSK * s + 4 * c);
              const float4 q0 = src[0], q1 = src[1], q2 = src[2];
              const float v12[12] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w};
              float w[4 + NKY - 1];
              // the window starts `lead` floats into the aligned reads (selects, no branches)
#pragma unroll
              for (int j = 0; j < 4 + NKY - 1; ++j) {
                const float lo01 = lead_bit0 ? v12[j + 1] : v12[j], hi23 = lead_bit0 ? v12[j + 3] : v12[j + 2];
                w[j] = lead_bit1 ? hi23 : lo01;
              }
              float4 *dh = b_hi + c * pitch + hh * k1p + rb * NKY, *dl = b_lo + c * pitch + hh * k1p + rb * NKY;
#pragma unroll
              for (int t = 0; t < NKY; ++t) {
                float4 vh, vl;
                vh.x = tf32_hi(w[t]), vh.y = tf32_hi(w[t + 1]), vh.z = tf32_hi(w[t + 2]), vh.w = tf32_hi(w[t + 3]);
                vl.x = w[t] - vh.x, vl.y = w[t + 1] - vh.y, vl.z = w[t + 2] - vh.z, vl.w = w[t + 3] - vh.w;
                dh[t] = vh;
                dl[t] = vl;
              }
            }
            tc::fence_proxy_async();  // operand B was written through the generic proxy; the tensor core reads it through the async one
            tc::mbar_arrive(&ctl->b_full[sb]);
          }
          // (the same fence ordered this thread's reads of the raw slot before the copy engine's next write)
          tc::mbar_arrive(&ctl->x_empty[rx]);
        }
      }
      if (cw == 4) { PROF_END(4); }
    }
  } else if (warp == kCopyWarp) {
    // ===================== copy issuer: one box of grad_y per item =====================
    if (lane == 0) {
      int sg = 0;
      PROF_BEGIN();
      for (int i = first; i < last; ++i, ++sg) {
        const Item it = decode(p, i);
        const int r = sg % kGoStages;
        PROF_WAIT_START();
        const bool empty_ok = tc::mbar_wait(&ctl->go_empty[r], (uint32_t)(((sg / kGoStages) & 1) ^ 1), kSpinLimit);
        PROF_WAIT_END();
        if (!empty_ok) {
          raise_timeout(ctl, 5);
          break;
        }
        tc::mbar_arrive_expect_tx(&ctl->go_full[r], kGoBytes);
        tc::tma_load_4d(go_base + (size_t)r * kGoBytes, &go_map, it.yt * kTP, it.ox, it.n, it.at * kCo, &ctl->go_full[r]);
      }
      PROF_END(3);
    }
    __syncwarp();
  } else if (warp == kCopyXWarp) {
    // ===================== copy issuer: one box of x per table entry =====================
    if (lane == 0) {
      int sx = 0;  // items with entries: the others use no slot of this ring
      for (int i = first; i < last; ++i) {
        const Item it = decode(p, i);
        const int e0 = rp[it.ox], ne = rp[it.ox + 1] - e0;
        if (ne == 0) continue;
        const int r = sx % kXStages;
        if (!tc::mbar_wait(&ctl->x_empty[r], (uint32_t)(((sx / kXStages) & 1) ^ 1), kSpinLimit)) {
          raise_timeout(ctl, 6);
          break;
        }
        const int start = it.yt * kTP + p.ws0 - p.lead;  // a multiple of 4
        unsigned char *dst = x_base + (size_t)r * kXBytes;
        tc::mbar_arrive_expect_tx(&ctl->x_full[r], (uint32_t)ne * kXEntryBytes);
        for (int e = 0; e < ne; ++e)
          tc::tma_load_4d(dst + (size_t)e * kXEntryBytes, &x_map, start, ctl->ent[e0 + e].y, it.n, 0, &ctl->x_full[r]);
        ++sx;
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer =====================
    // The whole warp walks the items; one elected lane issues.  Everything an MMA names is computed from
    // warp-uniform values (what comes from shared memory is broadcast from lane 0 to say so).
    const uint32_t tmem0 = tc::uniform(tmem_base);
    const uint32_t b0 = tc::smem_u32(b_base) >> 4;
    const uint64_t desc_hi_word = tc::smem_desc(0u, 0u, 128u);
    int sa = 0, iv = 0;
    bool failed = false;
    PROF_BEGIN();
    for (int i = first; i < last && !failed;) {
      const Item it = decode(p, i);
      const int seg_end = min(last, (it.seg + 1) * p.per_segment);
      const int k1 = (int)tc::uniform((uint32_t)(rp[it.ox + 1] - rp[it.ox])) * BK;
      if (k1 == 0) {
        i = seg_end;
        continue;
      }
      const int n_pad = 2 * pad16(k1);
      const uint32_t idesc = tc::idesc_tf32(2 * kCo, n_pad);
      const uint32_t pitch = (uint32_t)n_pad + 1u;  // rows of 16 bytes between the 4-position chunks of B
      const uint32_t lbo_bits = (pitch & 0x3FFFu) << 16;
      const int stages = (seg_end - i) * kStagesPerItem;
      for (int s = 0; s < stages && !failed; ++s, ++sa) {
        const int so = sa % kOpStages, sb = sa % kBStages;
        PROF_WAIT_START();
        bool ok = tc::mbar_wait(&ctl->a_full[so], (uint32_t)((sa / kOpStages) & 1), kSpinLimit) &&
                  tc::mbar_wait(&ctl->b_full[sb], (uint32_t)((sa / kBStages) & 1), kSpinLimit);
        const bool opens = s % kPromote == 0;
        // a new level-1 interval: the epilogue must have drained the previous one
        if (opens) ok = ok && tc::mbar_wait(&ctl->l1_empty, (uint32_t)((iv & 1) ^ 1), kSpinLimit);
        PROF_WAIT_END();
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) raise_timeout(ctl, opens ? 3 : 2);
          failed = true;
          break;
        }
        tc::tc_fence_after_sync();
        const bool closes = (s + 1) % kPromote == 0 || s + 1 == stages;
        const uint32_t a_hi = tmem0 + kACol0 + (uint32_t)so * (2 * kSK), a_lo = a_hi + kSK;
        const uint32_t b_hi = b0 + (uint32_t)sb * (p.b_stage_bytes >> 4), b_lo = b_hi + 8u * pitch;
        if (tc::elect_one()) {
          uint32_t fresh = opens ? 0u : 1u;  // 0: the next MMA overwrites the level-1 sums
#pragma unroll
          for (int ks = 0; ks < kSK / 8; ++ks) {
            const uint32_t bo = (uint32_t)ks * 2u * pitch;
            const uint64_t db_hi = desc_hi_word | (uint64_t)(((b_hi + bo) & 0x3FFFu) | lbo_bits);
            const uint64_t db_lo = desc_hi_word | (uint64_t)(((b_lo + bo) & 0x3FFFu) | lbo_bits);
            // the three products of the hi/lo split, smallest first
            tc::mma_tf32_a_tmem(tmem0 + kL1Col, a_lo + 8u * ks, db_hi, idesc, fresh);
            tc::mma_tf32_a_tmem(tmem0 + kL1Col, a_hi + 8u * ks, db_lo, idesc, 1u);
            tc::mma_tf32_a_tmem(tmem0 + kL1Col, a_hi + 8u * ks, db_hi, idesc, 1u);
            fresh = 1u;
          }
          tc::tc_commit(&ctl->a_empty[so]);
          tc::tc_commit(&ctl->b_empty[sb]);
          if (closes) tc::tc_commit(&ctl->l1_full);
        }
        if (closes) ++iv;
        __syncwarp();
      }
      i = seg_end;
    }
    PROF_END(2);
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// gw[a, b, kx, ky] = sum, in a fixed order, of the partials of every (block, segment) whose output row has an
// entry for tap kx; gb[a] = sum of all bias partials.  A block owns one (b, kx, ky, channel tile) -- or, past
// those, the bias of one channel tile: 64 threads along the channels (the partials are channel-contiguous),
// sixteen groups that split the output rows (the blocks) and are combined in a fixed order through shared memory.
constexpr int kReduceGroups = 16;
__global__ void __launch_bounds__(kReduceGroups * kCo) tc_gradw_few_in_reduce_kernel(const GfParams p, int nblocks) {
  __shared__ float red[kReduceGroups][kCo];
  __shared__ int first_s[256];  // first item of every block's run (nblocks + 1 values)
  __shared__ int rp_s[kMaxRows + 1];
  __shared__ int kx_s[kMaxTable];
  for (int i = threadIdx.x; i <= p.nox; i += blockDim.x) rp_s[i] = p.row_ptr[i];
  for (int i = threadIdx.x; i < p.num_entries; i += blockDim.x) kx_s[i] = p.entries[i].x;
  __syncthreads();
  for (int b = threadIdx.x; b <= nblocks; b += blockDim.x) first_s[b] = first_item(p, rp_s, b, nblocks);
  tc::grid_dependency_wait();  // the partial sums come from the kernel before
  __syncthreads();
  const int al = threadIdx.x & (kCo - 1), grp = threadIdx.x >> 6;
  const int weight_blocks = p.B * p.nkx * p.nky * p.a_tiles;
  float sum = 0.f;
  int a, out_index = -1;
  if ((int)blockIdx.x < weight_blocks) {
    int r = blockIdx.x;
    const int at = r % p.a_tiles;
    r /= p.a_tiles;
    const int ky = r % p.nky, kx = (r / p.nky) % p.nkx, b = r / (p.nky * p.nkx);
    a = at * kCo + al;
    const int t = p.By < 0 ? p.nky - 1 - ky : ky;  // taps are kept in increasing input offset
    for (int ox = grp; ox < p.nox; ox += kReduceGroups) {
      const int e0 = rp_s[ox], ne = rp_s[ox + 1] - e0;
      int e = -1;
      for (int j = 0; j < ne; ++j)
        if (kx_s[e0 + j] == kx) e = j;
      if (e < 0) continue;
      const int col = (e * p.B + b) * p.nky + t;
      const int seg = ox * p.a_tiles + at;
      // the blocks whose run of items meets this segment, eight at a time (their loads in flight together)
      const int i0 = seg * p.per_segment, i1 = i0 + p.per_segment;
      int blk = (int)((long long)i0 * nblocks / p.total);  // a guess; the runs are cut by weight, not by count
      while (blk > 0 && first_s[blk] > i0) --blk;
      while (blk + 1 < nblocks && first_s[blk + 1] <= i0) ++blk;
      while (blk < nblocks && first_s[blk] < i1) {
        float v[8][2];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int bu = blk + u;
          const bool valid = bu < nblocks && first_s[bu] < i1 && first_s[bu + 1] > i0 && first_s[bu + 1] > first_s[bu];
          v[u][0] = v[u][1] = 0.f;
          if (valid) {
            const int sidx = seg - first_s[bu] / p.per_segment;
            const float *src = p.part_w + ((((size_t)bu * p.seg_max + sidx) * 2) * kMaxK1 + col) * kCo + al;
            v[u][0] = __ldcg(src), v[u][1] = __ldcg(src + (size_t)kMaxK1 * kCo);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) sum += v[u][0] + v[u][1];
        blk += 8;
      }
    }
    if (a < p.A) out_index = ((a * p.B + b) * p.nkx + kx) * p.nky + ky;
  } else {
    const int at = blockIdx.x - weight_blocks;
    a = at * kCo + al;
    for (int blk0 = grp; blk0 < nblocks; blk0 += 4 * kReduceGroups) {
      float v[4][2];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int blk = blk0 + u * kReduceGroups;
        v[u][0] = v[u][1] = 0.f;
        if (blk < nblocks && first_s[blk + 1] > first_s[blk]) {
          const float *src = p.part_b + (((size_t)blk * p.a_tiles + at) * 2) * kCo + al;
          v[u][0] = __ldcg(src), v[u][1] = __ldcg(src + kCo);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) sum += v[u][0] + v[u][1];
    }
  }
  red[grp][al] = sum;
  __syncthreads();
  if (grp == 0) {
    float total = 0.f;
#pragma unroll
    for (int g = 0; g < kReduceGroups; ++g) total += red[g][al];
    if ((int)blockIdx.x < weight_blocks) {
      if (out_index >= 0) p.gw[out_index] = total;
    } else if (a < p.A) {
      p.gb[a] = total;
    }
  }
}

struct GfPlan {
  GfParams params;
  size_t smem = 0, part_w_floats = 0, part_b_floats = 0;
  int blocks = 0;
};

bool plan_tc_gradw_few_in(const GradWProblem<float> &p, GfPlan &plan) {
  if (p.Dy != 1 || p.Ay != 1) return false;
  if (p.B < 1 || p.B > kBoxChannels || p.A < 16 || p.A > 4 * kCo || p.nky < 1 || p.nky > 3) return false;
  if (p.nky > 1 && p.By != 1 && p.By != -1) return false;
  if (p.nkx < 1 || p.noy < 64 || p.nox < 1 || p.nox > kMaxRows || p.N < 1 || p.nix < 1) return false;
  const int max_row = p.table_h.row_ptr != nullptr ? p.table_h.max_row : std::min(p.nkx, kMaxEntries + 1);
  if (max_row < 1 || max_row > kMaxEntries) return false;
  const int BK = p.B * p.nky;
  if ((BK * max_row + 15) / 16 * 16 > kMaxK1) return false;
  if (p.table_h.row_ptr != nullptr && p.table_h.num_entries > kMaxTable) return false;
  // rows are copied in 16-byte chunks
  if (p.niy % 4 != 0 || p.noy % 4 != 0 || reinterpret_cast<uintptr_t>(p.in) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(p.go) % 16 != 0)
    return false;
  GfParams &q = plan.params;
  q.row_ptr = p.table_h.row_ptr, q.entries = p.table_h.entries;
  q.gw = p.gw, q.gb = p.gb;
  q.N = p.N, q.A = p.A, q.B = p.B, q.nkx = p.nkx, q.nky = p.nky, q.nox = p.nox, q.noy = p.noy, q.By = p.By;
  q.BK = BK;
  q.y_tiles = (p.noy + kTP - 1) / kTP;
  q.a_tiles = (p.A + kCo - 1) / kCo;
  q.ws0 = p.Cy + std::min(0, p.By * (p.nky - 1));
  q.lead = ((q.ws0 % 4) + 4) % 4;
  q.per_segment = p.N * q.y_tiles;
  const long long total = (long long)p.nox * q.a_tiles * q.per_segment;
  if (total >= (1LL << 30)) return false;
  q.total = (int)total;
  q.num_entries = (int)p.table_h.num_entries;
  q.k1p_max = (BK * max_row + 15) / 16 * 16;
  q.b_stage_bytes = 2u * 8u * (uint32_t)(2 * q.k1p_max + 1) * 16u;
  plan.blocks = (int)std::min<long long>(std::min(sm_count(), 255), total);
  // a run weighs total_weight / blocks <= items * (kItemWeight + max_row) / blocks and an item at least kItemWeight
  const long long per_block = (total * (kItemWeight + max_row) / kItemWeight + plan.blocks - 1) / plan.blocks;
  q.seg_max = (int)(per_block / q.per_segment) + 2;
  plan.smem = kHeaderBytes + (size_t)kGoStages * kGoBytes + (size_t)kXStages * kXBytes + (size_t)kBStages * q.b_stage_bytes;
  if (plan.smem > 227 * 1024) return false;
  plan.smem = std::max<size_t>(plan.smem, 116 * 1024);  // one block per SM: it owns all of tensor memory
  plan.part_w_floats = (size_t)plan.blocks * q.seg_max * 2 * kMaxK1 * kCo;
  plan.part_b_floats = (size_t)plan.blocks * q.a_tiles * 2 * kCo;
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

// a dense (batch, channel, row, position) tensor as (position, row, batch, channel)
bool make_map(CUtensorMap *map, const float *base, int inner, int rows, int batch, int chans, int box_inner, int box_chans) {
  EncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batch, (cuuint64_t)chans};
  const cuuint64_t strides[3] = {(cuuint64_t)inner * 4, (cuuint64_t)inner * rows * chans * 4, (cuuint64_t)inner * rows * 4};
  const cuuint32_t box[4] = {(cuuint32_t)box_inner, 1u, 1u, (cuuint32_t)box_chans};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NB>
int launch_for_b(const GfPlan &plan, const CUtensorMap &go_map, const CUtensorMap &x_map, cudaStream_t stream) {
  const GfParams &q = plan.params;
  auto kernel = q.nky == 1   ? tc_gradw_few_in_kernel<NB, 1>
                : q.nky == 2 ? tc_gradw_few_in_kernel<NB, 2>
                             : tc_gradw_few_in_kernel<NB, 3>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  kernel<<<plan.blocks, kThreads, plan.smem, stream>>>(q, go_map, x_map);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("tc_gradw_few_in_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

}  // namespace

// Reads and clears this kernel's timeout flag of the current device (synchronises it).
int tc_gradw_few_in_take_error(int *code) {
  int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(code, g_tc_gwfi_error, sizeof(int));
  if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_tc_gwfi_error, &zero, sizeof(int));
  return err == cudaSuccess ? MELLIN_OK : fail(MELLIN_ERR_LAUNCH, std::string("device status: ") + cudaGetErrorString(err));
}

#ifdef MELLIN_TUNING_HOOKS
extern "C" int mellin_tc_gradw_few_in_profile(long long *out) {
  return cudaMemcpyFromSymbol(out, g_gf_prof, 16 * sizeof(long long)) == cudaSuccess ? 0 : 2;
}
#endif

// scratch for the partial sums in floats (0 = problem not covered by this kernel)
size_t tc_gradw_few_in_workspace_floats(const GradWProblem<float> &p) {
  GfPlan plan;
  if (!plan_tc_gradw_few_in(p, plan)) return 0;
  return plan.part_w_floats + plan.part_b_floats;
}

// Partial sums, then their reduction into p.gw (and p.gb).  MELLIN_ERR_UNSUPPORTED when the problem is
// outside this kernel's coverage or the workspace too small.
int launch_tc_gradw_few_in(const GradWProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  GfPlan plan;
  if (p.table_h.row_ptr == nullptr || !plan_tc_gradw_few_in(p, plan)) return MELLIN_ERR_UNSUPPORTED;
  if (workspace == nullptr || workspace_bytes < (plan.part_w_floats + plan.part_b_floats) * sizeof(float) ||
      reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
    return MELLIN_ERR_UNSUPPORTED;
  CUtensorMap go_map, x_map;
  if (!make_map(&go_map, p.go, p.noy, p.nox, p.N, p.A, kGoRow, kCo) ||
      !make_map(&x_map, p.in, p.niy, p.nix, p.N, p.B, kXRow, kBoxChannels))
    return MELLIN_ERR_UNSUPPORTED;
  GfParams &q = plan.params;
  q.part_w = static_cast<float *>(workspace);
  q.part_b = p.gb != nullptr ? q.part_w + plan.part_w_floats : nullptr;
  int rc;
  switch (p.B) {
    case 1: rc = launch_for_b<1>(plan, go_map, x_map, stream); break;
    case 2: rc = launch_for_b<2>(plan, go_map, x_map, stream); break;
    case 3: rc = launch_for_b<3>(plan, go_map, x_map, stream); break;
    default: rc = launch_for_b<4>(plan, go_map, x_map, stream); break;
  }
  if (rc) return rc;
  const int reduce_blocks = p.B * p.nkx * p.nky * q.a_tiles + (p.gb != nullptr ? q.a_tiles : 0);
  cudaError_t err = launch_after_predecessor(tc_gradw_few_in_reduce_kernel, dim3((unsigned)reduce_blocks),
                                             dim3(kReduceGroups * kCo), 0, stream, q, plan.blocks);
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess)
    return fail(MELLIN_ERR_LAUNCH, std::string("tc_gradw_few_in_reduce_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

}  // namespace mellin
