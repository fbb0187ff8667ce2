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
// Warp roles (14 warps): 0-3 epilogue (TMEM -> registers -> global, one warp per
// 32 TMEM lanes); 4-11 converters (raw rows in shared memory -> hi/lo operand
// layout); 12 MMA issuer; 13 copy issuer: every gathered input row of a K-block
// (4 rows = 4 consecutive channels of one table entry) is one 4-D TMA box load
// -- positions outside the signal and channels beyond the last are zero-filled
// by the copy engine -- and the packed weight chunks are bulk copies straight
// into operand layout.  The index table, the bias and all per-block constants
// live in shared memory.  A ring of shared-memory stages and two TMEM accumulators are handed
// around with mbarriers; every wait is bounded and a timeout raises a
// device-side error flag instead of hanging.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
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
constexpr int kCopyWarp = kMmaWarp + 1;
constexpr int kThreads = (kCopyWarp + 1) * 32;
constexpr int kTileM = 128;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr int kMaxStages = 4;
constexpr int kMaxKB = 64;          // rows per stage (16 chunks: one lane of the copy warp each)
constexpr int kMaxTableRows = 512;  // output rows (ox) whose table is cached in shared memory
constexpr int kMaxTableEntries = 1024;
constexpr int kMaxBias = 1024;      // output channels whose bias is cached in shared memory

__device__ int g_tc_error = 0;       // first timeout code seen by any block since the last query
__device__ long long g_tc_prof[16];  // per-role wait / work cycles of block 0 (written when profiling is on)

struct TcParams {
  const float *bias;
  float *out;
  const float *w_hi;  // packed [a tile][kx][tap][b / 4][NP][b % 4]
  const float *w_lo;
  const int32_t *row_ptr;
  const int2 *entries;
  const int32_t *order;  // table rows, most entries first
  int num_entries;
  int N, A, B;
  int Bp;        // B rounded up to a multiple of 4: rows per table entry
  int nkx, nky, nox, noy;
  long long out_sn, out_sa;
  int absBy;     // |By|: positions between consecutive taps
  int ws0;       // first input position of tile 0: Cy + min(0, By * (nky - 1))
  int NP;        // padded output channels per tile (multiple of 16, <= 128)
  int a_tiles;   // tiles over output channels
  int RW;        // staged positions per row (multiple of 8)
  int RWt;       // positions copied per raw row: RW + 4 (room for the 16-byte alignment lead)
  int raw_chunk_floats;  // pitch of a raw 4-row chunk in shared memory (128-byte aligned); its rows are RWt apart
  int KB;        // rows per stage (multiple of 8)
  int PI;        // stages per accumulation interval: PI * KB / 8 * 3 * TG <= 96 chained MMAs
  int TG, G;     // linear taps per stage and number of such tap groups: a block of KB rows is staged G times,
                 // each time with the weights of TG taps (weights of many taps do not fit a stage)
#ifdef MELLIN_MASKED
  const int *lens;  // per utterance: outputs at positions >= lens[n] * len_scale + len_offset are zero
  int len_scale, len_offset;
  int relu;
  unsigned drop_threshold, drop_seed;  // fused dropout (masked build): see DirectProblem
  float drop_scale;
#endif
  int table_in_smem;  // 1: row offsets, entries and row order are cached in shared memory
  int wide_box;  // 1: one TMA box brings all KB rows of a stage (they belong to one table entry)
  int kblock_pack;  // 1: weights packed stage by stage, [a tile][kx][b / KB][hi, lo][tap][(b % KB) / 4][NP][b % 4]
  int stages;
  int y_tiles;
  int tiles;
  int tmem_cols;
  uint32_t a_stage_bytes, w_stage_bytes;  // per hi or lo part
  uint32_t raw_stage_bytes;
  uint32_t w_pack_bytes;  // bytes of one packed weight array (hi or lo)
  uint32_t w_res_bytes;  // > 0: the whole packed weight set (hi, then lo) stays in shared memory for the
                         // life of the block and stages hold activations only
  int profile;
  int exact;  // operands are exact in TF32: no compensation MMAs
};

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// ---- weight packing ---------------------------------------------------------------
// W[a, b, kx, ky] (arbitrary a / b strides) -> hi and lo parts laid out
// [a tile][kx][tap][b / 4][NP][b % 4]: 16-byte chunks of 4 consecutive reduced
// channels for one output channel, tap slots in increasing input-offset order,
// output channels beyond A and reduced channels beyond B zero-filled.
__global__ void pack_weights_kernel(const float *__restrict__ w, long long w_sa, long long w_sb, int A, int B, int nkx,
                                    int nky, int NP, int a_tiles, int By, int KB, int TG, int G,
                                    float *__restrict__ hi, float *__restrict__ lo) {
  const int B4 = (B + 3) / 4;
  if (KB > 0) {
    // stage-by-stage layout: [a tile][kx][b / KB][tap group][hi, lo][tap in group][(b % KB) / 4][NP][b % 4] in `hi`
    const int blocks_b = B4 * 4 / KB, C = KB / 4;
    const long long total = (long long)a_tiles * nkx * blocks_b * G * 2 * TG * C * NP * 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
      const int bl = (int)(i & 3);
      long long r = i >> 2;
      int a = (int)(r % NP);
      r /= NP;
      const int c = (int)(r % C);
      r /= C;
      int t = (int)(r % TG);
      r /= TG;
      const int part = (int)(r & 1);
      r >>= 1;
      t += (int)(r % G) * TG;
      r /= G;
      const int b = ((int)(r % blocks_b) * C + c) * 4 + bl;
      r /= blocks_b;
      const int kx = (int)(r % nkx);
      a += (int)(r / nkx) * NP;
      const int ky = By < 0 ? nky - 1 - t : t;
      float v = 0.f;
      if (a < A && b < B && t < nky) v = w[a * w_sa + b * w_sb + (long long)kx * nky + ky];
      const float h = tf32_hi(v);
      hi[i] = part ? v - h : h;
    }
    return;
  }
  const long long total = (long long)a_tiles * nkx * nky * B4 * NP * 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int bl = (int)(i & 3);
    long long r = i >> 2;
    int a = (int)(r % NP);
    r /= NP;
    const int b = (int)(r % B4) * 4 + bl;
    r /= B4;
    const int t = (int)(r % nky);
    r /= nky;
    const int kx = (int)(r % nkx);
    a += (int)(r / nkx) * NP;
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
  uint64_t raw_full[kMaxStages];  // copies of a stage have landed
  uint64_t full[kMaxStages];      // operands of a stage are converted
  uint64_t empty[kMaxStages];     // the MMAs reading a stage have completed
  uint64_t dfull[2];
  uint64_t dempty[2];
  uint32_t tmem_base;
  int abort;
};
// control block | row_ptr | entries | bias | stages
constexpr uint32_t kRowPtrOffset = 256;
constexpr uint32_t kEntriesOffset = kRowPtrOffset + (kMaxTableRows + 1) * 4 + 12;  // 16-byte aligned
constexpr uint32_t kBiasOffset = kEntriesOffset + kMaxTableEntries * 8;
constexpr int kMaxKSteps = 1024;      // k-steps (8 rows) over all table rows, resident-weight mode
constexpr uint32_t kKOfsOffset = kBiasOffset + kMaxBias * 4;             // int[kMaxTableRows + 1]
constexpr uint32_t kKStepOffset = kKOfsOffset + (kMaxTableRows + 1) * 4 + 4;  // uint2[kMaxKSteps], 8-byte aligned
constexpr uint32_t kOrderOffset = kKStepOffset + kMaxKSteps * 8;  // int[kMaxTableRows]
#ifdef MELLIN_MASKED
constexpr int kMaxLens = 1024;  // utterances whose lengths are cached in shared memory
constexpr uint32_t kLensOffset = kOrderOffset + kMaxTableRows * 4;  // int[kMaxLens]
constexpr uint32_t kStageOffset = (kLensOffset + kMaxLens * 4 + 1023) / 1024 * 1024;
#else
constexpr uint32_t kStageOffset = (kOrderOffset + kMaxTableRows * 4 + 1023) / 1024 * 1024;
#endif

__device__ __forceinline__ void raise_timeout(TcControl *ctl, int code) {
  atomicCAS(&g_tc_error, 0, code);
  ctl->abort = 1;
}

// Tile coordinates of a block: tile = blockIdx.x + i * gridDim.x, decoded once
// and then advanced by the (decoded) grid stride with carries -- no divisions
// in the steady state.
// Tiles in heaviest-row-first order, ((rank, n), yt, at) with at fastest, dealt to the blocks in alternating
// direction (block b takes b, 2G-1-b, 2G+b, ...): the rows of the Mellin table
// differ several-fold in their number of entries, and this keeps the blocks'
// total work within about one tile of each other.  The tiles of one row are
// adjacent in the order, so blocks that run together share its weights in L2.
struct TileWalker {
  int n, ox, yt, at;  // current tile
  int rank;           // of its row in the heaviest-first order
  int tile;           // its place in the order; >= p.tiles when the block is done
  int step, step_after;          // tiles to the next round's tile, and from that one to the round after
  int dat, dyt, dn, drank;       // `step` as digits (at, yt, n, rank): next() adds with carries, no divisions
  int eat, eyt, en, erank;       // `step_after` as digits; the two swap every round
  const int *order_s;
#ifdef MELLIN_MASKED
  // With per-utterance lengths the (n, yt) digits as walked are a PLACE in a list of the row's (n, yt) pairs
  // that holds the pairs with data first and the pairs past their utterance's end (epilogue-only tiles) last:
  // in walk order the dead tiles fall on the blocks at random and leave them 11-14 % apart in work; with the
  // live tiles of a row contiguous the blocks end within 3-5 % of each other.
  int wn, wyt;
  const unsigned short *pairs;  // (n << 6 | yt) by place; nullptr: the digits are the tile
#define WALK_N wn
#define WALK_YT wyt
  __device__ __forceinline__ void resolve(const TcParams &p) {
    if (pairs != nullptr) {
      const unsigned v = pairs[wn * p.y_tiles + wyt];
      n = (int)(v >> 6), yt = (int)(v & 63u);
    } else {
      n = wn, yt = wyt;
    }
  }
#else
#define WALK_N n
#define WALK_YT yt
  __device__ __forceinline__ void resolve(const TcParams &) {}
#endif
  __device__ __forceinline__ static void digits(const TcParams &p, int t, int &a, int &y, int &nn, int &r) {
    a = t % p.a_tiles, t /= p.a_tiles;
    y = t % p.y_tiles, t /= p.y_tiles;
    nn = t % p.N;
    r = t / p.N;
  }
  __device__ __forceinline__ void init(const TcParams &p, const int *order_smem, const unsigned short *pairs_smem) {
    order_s = order_smem;
#ifdef MELLIN_MASKED
    pairs = pairs_smem;
#else
    (void)pairs_smem;
#endif
    tile = blockIdx.x;
    digits(p, tile, at, WALK_YT, WALK_N, rank);
    resolve(p);
    ox = rank < p.nox ? order_s[rank] : 0;
    step = 2 * (int)gridDim.x - 1 - 2 * (int)blockIdx.x;
    step_after = 2 * (int)blockIdx.x + 1;
    digits(p, step, dat, dyt, dn, drank);
    digits(p, step_after, eat, eyt, en, erank);
  }
  __device__ __forceinline__ void next(const TcParams &p) {
    tile += step;
    at += dat;
    int carry = at >= p.a_tiles;
    at -= carry ? p.a_tiles : 0;
    WALK_YT += dyt + carry;
    carry = WALK_YT >= p.y_tiles;
    WALK_YT -= carry ? p.y_tiles : 0;
    WALK_N += dn + carry;
    carry = WALK_N >= p.N;
    WALK_N -= carry ? p.N : 0;
    rank += drank + carry;
    resolve(p);
    ox = rank < p.nox ? order_s[rank] : 0;
    int t;
    t = step, step = step_after, step_after = t;
    t = dat, dat = eat, eat = t;
    t = dyt, dyt = eyt, eyt = t;
    t = dn, dn = en, en = t;
    t = drank, drank = erank, erank = t;
  }
};

#ifdef MELLIN_MASKED
// The list TileWalker::pairs: the (n, yt) pairs of one output row, those with yt * kTileM < lens_s[n] first, both
// groups in (n, yt) order.  Built by warp 0 behind the cached lengths (the list and the lengths share the
// kMaxLens * 4 bytes set aside for the lengths; a batch too large for that walks the tiles as they come).
// Every thread of the block calls this (it ends in a barrier); lens_s must be complete.
__device__ __forceinline__ const unsigned short *live_first_pairs(const TcParams &p, int *lens_s, int warp, int lane) {
  const int U = p.N * p.y_tiles;
  const bool fits = p.y_tiles <= 64 && p.N * 4 + U * 2 <= kMaxLens * 4;
  unsigned short *pairs = reinterpret_cast<unsigned short *>(lens_s + p.N);
  if (fits && warp == 0) {
    int live_total = 0;
    for (int base = 0; base < U; base += 32) {
      const int u = base + lane, n = u / p.y_tiles, yt = u - n * p.y_tiles;
      const bool live = u < U && yt * kTileM < lens_s[n < p.N ? n : 0];
      live_total += __popc(__ballot_sync(0xffffffffu, live));
    }
    int n_live = 0, n_dead = 0;
    const unsigned below = (1u << lane) - 1u;
    for (int base = 0; base < U; base += 32) {
      const int u = base + lane, n = u / p.y_tiles, yt = u - n * p.y_tiles;
      const bool in = u < U, live = in && yt * kTileM < lens_s[n < p.N ? n : 0];
      const unsigned m_live = __ballot_sync(0xffffffffu, live), m_dead = __ballot_sync(0xffffffffu, in && !live);
      const unsigned short v = (unsigned short)((n << 6) | yt);
      if (live) pairs[n_live + __popc(m_live & below)] = v;
      else if (in) pairs[live_total + n_dead + __popc(m_dead & below)] = v;
      n_live += __popc(m_live), n_dead += __popc(m_dead);
    }
  }
  __syncthreads();
  return fits ? pairs : nullptr;
}
#endif

// This file is compiled twice.  As itself it is the kernel for layers whose
// linear taps all fit one stage.  Included by tc_direct_taps.cu with
// MELLIN_TAP_GROUPS defined it becomes the variant that stages every block of
// rows once per group of TG taps (layers with many linear taps); every
// difference between the two is one of the macros below, so that the common
// kernel carries no code for the rare case (its single-thread issue loops are
// sensitive to it: the merged source cost the 3-channel layer 12 %).
#ifdef MELLIN_TAP_GROUPS
#define STAGE_LOOP(...) \
  for (int k0 = 0, tg = 0; k0 < Kr; (++tg == p.G ? (tg = 0, k0 += p.KB) : 0), ++it, __VA_ARGS__ RING_NEXT())
#define STAGES_IN_TILE ((Kr + p.KB - 1) / p.KB * p.G)  // epilogue: stages, counted one by one
#define STAGES_PER_PASS p.PI
#define TAP_GROUP tg
#define TAP_GROUPS p.G
#define TAPS_HERE min(p.TG, p.nky - tg * p.TG)
#define LAST_STAGE_OF_TILE (k0 + p.KB >= Kr && tg == p.G - 1)
#define TC_FN(name) name##_taps
#else
#define STAGE_LOOP(...) for (int k0 = 0; k0 < Kr; k0 += p.KB, ++it, __VA_ARGS__ RING_NEXT())
#define STAGES_IN_TILE Kr  // epilogue: rows, PI stages of KB rows per pass
#define STAGES_PER_PASS (p.KB * p.PI)
#define TAP_GROUP 0
#define TAP_GROUPS 1
#define TAPS_HERE p.nky
#define LAST_STAGE_OF_TILE (k0 + p.KB >= Kr)
#ifdef MELLIN_MASKED
#define TC_FN(name) name##_masked
#else
#define TC_FN(name) name
#endif
#endif

// A third build (tc_direct_masked.cu, MELLIN_MASKED) fuses what the reference's
// models do around a layer (models.py:386-390, 424-434): y = mask * relu(layer(x))
// with per-utterance lengths along the linear axis.  Tiles that start at or past
// an utterance's length are not computed at all (their outputs are zeros).
#ifdef MELLIN_MASKED
#define TILE_ROWS(rows) (tc_.yt * kTileM >= lens_s[tc_.n] ? 0 : (rows))
#define EPILOGUE_LEN                                          \
  const float keep = oy < lens_s[tc_.n] ? 1.f : 0.f;          \
  const float floor_ = p.relu ? 0.f : -3.0e38f;
#define STORE_VALUE(v)                                                                                           \
  (fmaxf((v), floor_) * keep *                                                                                   \
   ((p.drop_threshold != 0u && dropout_hash(p.drop_seed, (unsigned long long)(o - p.out)) < p.drop_threshold)    \
        ? 0.f                                                                                                    \
        : p.drop_scale))
#else
#define TILE_ROWS(rows) (rows)
#define EPILOGUE_LEN
#define STORE_VALUE(v) (v)
#endif

// position in the stage ring: slot and number of completed laps
#define RING_NEXT() (++ring_s == p.stages ? (ring_s = 0, ++ring_use) : 0u)

#define PROF_BEGIN() long long prof_t0 = clock64(), prof_wait = 0, prof_t1 = 0
#define PROF_WAIT_START() prof_t1 = clock64()
#define PROF_WAIT_END() prof_wait += clock64() - prof_t1
#define PROF_END(slot)                                           \
  if (blockIdx.x == 0 && lane == 0 && p.profile) {               \
    g_tc_prof[2 * (slot)] = prof_wait;                           \
    g_tc_prof[2 * (slot) + 1] = clock64() - prof_t0 - prof_wait; \
  }

// NPC: padded output channels per tile / 16 (the epilogue keeps 16 * NPC running sums per thread)
template <int NPC>
__global__ void __launch_bounds__(kThreads, 1)
tc_direct_kernel(const TcParams p, const __grid_constant__ CUtensorMap in_map,
                 const __grid_constant__ CUtensorMap in_map_wide) {
  extern __shared__ __align__(1024) unsigned char smem[];
  TcControl *ctl = reinterpret_cast<TcControl *>(smem);
  int *rowptr_s = reinterpret_cast<int *>(smem + kRowPtrOffset);
  int *order_s = reinterpret_cast<int *>(smem + kOrderOffset);
#ifdef MELLIN_MASKED
  int *lens_s = reinterpret_cast<int *>(smem + kLensOffset);
  for (int i = threadIdx.x; i < p.N; i += kThreads) lens_s[i] = p.lens[i] * p.len_scale + p.len_offset;
#endif
  int2 *ent_s = reinterpret_cast<int2 *>(smem + kEntriesOffset);
  float *bias_s = reinterpret_cast<float *>(smem + kBiasOffset);
  int *kofs_s = reinterpret_cast<int *>(smem + kKOfsOffset);        // first k-step of every table row
  uint2 *kstep_s = reinterpret_cast<uint2 *>(smem + kKStepOffset);  // (first weight chunk, distance to the second), 16-byte units
  unsigned char *w_res = smem + kStageOffset;  // resident weights: hi part, lo part
  unsigned char *stage_base = w_res + 2 * p.w_res_bytes;
  const uint32_t stage_bytes = 2 * (p.a_stage_bytes + p.w_stage_bytes) + p.raw_stage_bytes;
  volatile int *abort_flag = &ctl->abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int JB = p.KB >> 3;
  const int NPtot = p.NP * p.a_tiles;
  const int B4 = p.Bp >> 2;
  const int tile_chunks = p.nkx * p.nky * B4 * p.NP;  // 16-byte chunks of one output-channel tile's weights

  // ---- one-time set-up ------------------------------------------------------------
  // small tables are cached in shared memory, large ones are read in place
  const int *rowptr = p.table_in_smem ? rowptr_s : p.row_ptr;
  const int *order = p.table_in_smem ? order_s : p.order;
  const int2 *ent = p.table_in_smem ? ent_s : p.entries;
  if (p.table_in_smem) {
    for (int i = tid; i <= p.nox; i += kThreads) rowptr_s[i] = p.row_ptr[i];
    for (int i = tid; i < p.nox; i += kThreads) order_s[i] = p.order[i];
    for (int i = tid; i < p.num_entries; i += kThreads) ent_s[i] = p.entries[i];
  }
  for (int i = tid; i < NPtot; i += kThreads) bias_s[i] = (p.bias != nullptr && i < p.A) ? p.bias[i] : 0.f;
  {
    // weight chunks of padding rows are never copied: clear the stages once so
    // that they hold finite values (they meet zero activations)
    float4 *z = reinterpret_cast<float4 *>(stage_base);
    const int n16 = (int)((size_t)p.stages * stage_bytes / 16);
    for (int i = tid; i < n16; i += kThreads) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (p.w_res_bytes) {
    const int n16 = (int)(p.w_res_bytes / 16), have = (int)(p.w_pack_bytes / 16);
    const float4 *gh = reinterpret_cast<const float4 *>(p.w_hi), *gl = reinterpret_cast<const float4 *>(p.w_lo);
    float4 *sh = reinterpret_cast<float4 *>(w_res), *sl = reinterpret_cast<float4 *>(w_res + p.w_res_bytes);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = tid; i < n16; i += kThreads) {
      sh[i] = i < have ? __ldg(gh + i) : zero;
      sl[i] = i < have ? __ldg(gl + i) : zero;
    }
  }
  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      tc::mbar_init(&ctl->raw_full[s], 1);
      tc::mbar_init(&ctl->full[s], kConvertThreads);
      tc::mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(&ctl->dfull[a], 1);
      tc::mbar_init(&ctl->dempty[a], kEpilogueWarps * 32);
    }
    ctl->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tc::tmem_alloc(&ctl->tmem_base, (uint32_t)p.tmem_cols);
    tc::tmem_relinquish();
  }
  tc::fence_proxy_async();
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
#ifdef MELLIN_MASKED
  const unsigned short *tile_pairs = live_first_pairs(p, lens_s, warp, lane);
#else
  const unsigned short *tile_pairs = nullptr;
#endif
  if (p.w_res_bytes) {
    // weight chunk pair of every k-step of every table row (output-channel tile 0)
    if (tid == 0) {
      int o = 0;
      for (int ox = 0; ox <= p.nox; ++ox) {
        kofs_s[ox] = o;
        if (ox < p.nox) o += ((rowptr_s[ox + 1] - rowptr_s[ox]) * B4 + 1) >> 1;
      }
    }
    __syncthreads();
    for (int ox = warp; ox < p.nox; ox += kThreads / 32) {
      const int e0 = rowptr_s[ox];
      const int chunks = (rowptr_s[ox + 1] - e0) * B4;
      for (int j = lane; 2 * j < chunks; j += 32) {
        const int q0 = 2 * j, pp0 = q0 / B4, pp1 = (q0 + 1) / B4;
        const uint32_t c0 = (uint32_t)((ent_s[e0 + pp0].x * p.nky * B4 + (q0 - pp0 * B4)) * p.NP);
        uint32_t c1 = c0 + (uint32_t)p.NP;
        if (q0 + 1 < chunks) c1 = (uint32_t)((ent_s[e0 + pp1].x * p.nky * B4 + (q0 + 1 - pp1 * B4)) * p.NP);
        kstep_s[kofs_s[ox] + j] = make_uint2(c0, c1 - c0);
      }
    }
    __syncthreads();
  }

  if (warp < kEpilogueWarps) {
    // =========================== epilogue ===========================
    int g = 0;  // accumulation intervals consumed so far
    PROF_BEGIN();
    TileWalker tc_;
    for (tc_.init(p, order, tile_pairs); tc_.tile < p.tiles; tc_.next(p)) {
      // tcgen05.ld is warp-collective: keep every exit decision warp-uniform
      if (__any_sync(0xffffffffu, *abort_flag)) break;
      const int Kr = TILE_ROWS((rowptr[tc_.ox + 1] - rowptr[tc_.ox]) * p.Bp);
      const int oy = tc_.yt * kTileM + warp * 32 + lane;
      const int a0 = tc_.at * p.NP;
      float sum[NPC][16];
#pragma unroll
      for (int c = 0; c < NPC; ++c)
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
          const float4 b = *reinterpret_cast<const float4 *>(bias_s + a0 + 16 * c + 4 * i4);
          sum[c][4 * i4] = b.x, sum[c][4 * i4 + 1] = b.y, sum[c][4 * i4 + 2] = b.z, sum[c][4 * i4 + 3] = b.w;
        }
      bool failed = false;
      // one pass per accumulation interval: PI stages, each KB rows (of one tap group)
      for (int v0 = 0; v0 < STAGES_IN_TILE; v0 += STAGES_PER_PASS, ++g) {
        const int acc = g & 1;
        PROF_WAIT_START();
        const bool ok = tc::mbar_wait(&ctl->dfull[acc], (uint32_t)((g >> 1) & 1), kSpinLimit);
        PROF_WAIT_END();
        if (!__all_sync(0xffffffffu, ok)) {
          raise_timeout(ctl, 3);
          failed = true;
          break;
        }
        tc::tc_fence_after_sync();
        constexpr int kGroup = NPC < 4 ? NPC : 4;  // 16-column loads in flight together
#pragma unroll
        for (int c0 = 0; c0 < NPC; c0 += kGroup) {
          uint32_t v[kGroup][16];
#pragma unroll
          for (int c = 0; c < kGroup; ++c)
            if (c0 + c < NPC)
              tc::tmem_ld16(tmem_base + (uint32_t)(acc * p.NP + 16 * (c0 + c)) + ((uint32_t)(warp * 32) << 16), v[c]);
          tc::tmem_ld_wait();
          if (c0 + kGroup >= NPC) {
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&ctl->dempty[acc]);
          }
#pragma unroll
          for (int c = 0; c < kGroup; ++c)
            if (c0 + c < NPC)
#pragma unroll
              for (int i = 0; i < 16; ++i) sum[c0 + c][i] += __uint_as_float(v[c][i]);
        }
      }
      if (failed) break;
      if (oy < p.noy) {
        float *o = p.out + tc_.n * p.out_sn + a0 * p.out_sa + (long long)tc_.ox * p.noy + oy;
        const int a_left = p.A - a0;
        EPILOGUE_LEN
#pragma unroll
        for (int c = 0; c < NPC; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (16 * c + i < a_left) __stcs(o, STORE_VALUE(sum[c][i]));
            o += p.out_sa;
          }
      }
    }
    if (warp == 0) { PROF_END(0); }
  } else if (warp < kMmaWarp) {
    // =========================== converters ===========================
    const int pwarp = warp - kEpilogueWarps;
    int it = 0, ring_s = 0;
    uint32_t ring_use = 0;
    bool failed = false;
    PROF_BEGIN();
    TileWalker tc_;
    for (tc_.init(p, order, tile_pairs); tc_.tile < p.tiles && !*abort_flag && !failed; tc_.next(p)) {
      const int Kr = TILE_ROWS((rowptr[tc_.ox + 1] - rowptr[tc_.ox]) * p.Bp);
      const int lead = (tc_.yt * kTileM + p.ws0) & 3;  // the copy started at the 16-byte boundary below
      STAGE_LOOP() {
        const int s = ring_s;
        const uint32_t use = ring_use;
        PROF_WAIT_START();
        const bool okw = tc::mbar_wait(&ctl->raw_full[s], use & 1, kSpinLimit);
        PROF_WAIT_END();
        if (!okw) {
          raise_timeout(ctl, 1);
          failed = true;
          break;
        }
        unsigned char *st = stage_base + (size_t)s * stage_bytes;
        float4 *a_hi = reinterpret_cast<float4 *>(st);
        float4 *a_lo = reinterpret_cast<float4 *>(st + p.a_stage_bytes);
        const float *raw = reinterpret_cast<const float *>(st + 2 * (p.a_stage_bytes + p.w_stage_bytes));
        const int rows_here = min(p.KB, Kr - k0);
        const int chunks_loaded = (rows_here + 3) >> 2;
        const int chunks_total = ((rows_here + 7) >> 3) << 1;
        for (int c = pwarp; c < chunks_total; c += kConvertWarps) {
          float4 *dh = a_hi + c * p.RW, *dl = a_lo + c * p.RW;
          if (c < chunks_loaded) {
            const float *r0 = raw + (size_t)c * p.raw_chunk_floats + lead;
            for (int rho = lane; rho < p.RW; rho += 32) {
              const float x0 = r0[rho], x1 = r0[p.RWt + rho], x2 = r0[2 * p.RWt + rho], x3 = r0[3 * p.RWt + rho];
              float4 h, l;
              h.x = tf32_hi(x0), h.y = tf32_hi(x1), h.z = tf32_hi(x2), h.w = tf32_hi(x3);
              l.x = x0 - h.x, l.y = x1 - h.y, l.z = x2 - h.z, l.w = x3 - h.w;
              dh[rho] = h;
              dl[rho] = l;
            }
          } else {
            for (int rho = lane; rho < p.RW; rho += 32) {
              dh[rho] = make_float4(0.f, 0.f, 0.f, 0.f);
              dl[rho] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
        }
        tc::fence_proxy_async();
        tc::mbar_arrive(&ctl->full[s]);
      }
    }
    if (pwarp == 0) { PROF_END(1); }
  } else if (warp == kCopyWarp) {
    // =========================== copy issuer ===========================
    int it = 0, ring_s = 0;
    uint32_t ring_use = 0;
    bool failed = false;
    const float4 *src_hi = reinterpret_cast<const float4 *>(p.w_hi);
    const float4 *src_lo = reinterpret_cast<const float4 *>(p.w_lo);
    const uint32_t w_chunk_bytes = (uint32_t)p.NP * 16u;
    const uint32_t bytes_per_chunk =
        (uint32_t)p.RWt * 16u + (p.w_res_bytes ? 0u : 2u * (uint32_t)p.TG * w_chunk_bytes);
    PROF_BEGIN();
    TileWalker tc_;
    for (tc_.init(p, order, tile_pairs); tc_.tile < p.tiles && !failed; tc_.next(p)) {
      if (__any_sync(0xffffffffu, *abort_flag)) break;
      const int e0 = rowptr[tc_.ox];
      const int Kr = TILE_ROWS((rowptr[tc_.ox + 1] - e0) * p.Bp);
      const int ws = tc_.yt * kTileM + p.ws0;
      const int x0 = ws - (ws & 3);
      STAGE_LOOP() {
        const int s = ring_s;
        const uint32_t use = ring_use;
        PROF_WAIT_START();
        const bool ok = tc::mbar_wait(&ctl->empty[s], (use & 1) ^ 1, kSpinLimit);
        PROF_WAIT_END();
        if (!__all_sync(0xffffffffu, ok)) {
          raise_timeout(ctl, 5);
          failed = true;
          break;
        }
        unsigned char *st = stage_base + (size_t)s * stage_bytes;
        float4 *w_hi = reinterpret_cast<float4 *>(st + 2 * p.a_stage_bytes);
        float4 *w_lo = reinterpret_cast<float4 *>(st + 2 * p.a_stage_bytes + p.w_stage_bytes);
        float *raw = reinterpret_cast<float *>(st + 2 * (p.a_stage_bytes + p.w_stage_bytes));
        const int chunks_here = (min(p.KB, Kr - k0) + 3) >> 2;
        if (lane == 0) tc::mbar_arrive_expect_tx(&ctl->raw_full[s], (uint32_t)chunks_here * bytes_per_chunk);
        __syncwarp();
        // lane = chunk: 4 consecutive channels b0..b0+3 of one table entry.  The
        // chunks of one entry are consecutive in the packed weights and in the
        // stage, so the first lane of each run copies the whole run.
        const int r = k0 + 4 * lane;
        const int pp = lane < chunks_here ? r / p.Bp : -1 - lane;
        const int prev = __shfl_up_sync(0xffffffffu, pp, 1);
        const bool run_start = lane < chunks_here && (lane == 0 || prev != pp);
        const unsigned starts = __ballot_sync(0xffffffffu, run_start);
        if (lane < chunks_here) {
          const int b0 = r - pp * p.Bp;
          const int2 e = ent[e0 + pp];
          if (!p.wide_box) {
            tc::tma_load_4d(raw + (size_t)lane * p.raw_chunk_floats, &in_map, x0, e.y, tc_.n, b0, &ctl->raw_full[s]);
          } else if (lane == 0) {
            tc::tma_load_4d(raw, &in_map_wide, x0, e.y, tc_.n, b0, &ctl->raw_full[s]);
          }
          if (p.kblock_pack) {
            // the stage's weights (hi, then lo; every tap) are one contiguous run
            if (lane == 0) {
              const long long blk = ((long long)(tc_.at * p.nkx + e.x) * (p.Bp / p.KB) + b0 / p.KB) * TAP_GROUPS + TAP_GROUP;
              tc::bulk_load(w_hi, src_hi + blk * (2 * p.w_stage_bytes / 16), 2 * p.w_stage_bytes, &ctl->raw_full[s]);
            }
          } else if (run_start && !p.w_res_bytes) {
            const unsigned later = lane == 31 ? 0u : starts & ~((2u << lane) - 1u);
            const int run = (later ? __ffs(later) - 1 : chunks_here) - lane;
            long long src = (long long)tc_.at * tile_chunks + ((long long)(e.x * p.nky) * B4 + (b0 >> 2)) * p.NP;
            int dst = (lane >> 1) * (2 * p.NP) + (lane & 1) * p.NP;
            for (int t = 0; t < p.nky; ++t) {
              tc::bulk_load(w_hi + dst, src_hi + src, (uint32_t)run * w_chunk_bytes, &ctl->raw_full[s]);
              tc::bulk_load(w_lo + dst, src_lo + src, (uint32_t)run * w_chunk_bytes, &ctl->raw_full[s]);
              src += (long long)B4 * p.NP;
              dst += JB * 2 * p.NP;
            }
          }
        }
      }
    }
    PROF_END(3);
  } else if (warp == kMmaWarp) {
    // =========================== MMA issuer ===========================
    // The whole warp walks the tiles and one elected lane issues: addresses and descriptors computed by all
    // lanes from warp-uniform values (what is read from shared or global memory is broadcast from lane 0 to
    // say so) can live in the uniform registers the MMA reads them from.  Issued from inside an
    // `if (lane == 0)` region the same MMAs cost the issuing thread about twice as long.
    {
      const uint32_t tmem0 = tc::uniform(tmem_base);
      const uint32_t idesc = tc::idesc_tf32(kTileM, p.NP);
      const uint32_t a_lbo = (uint32_t)p.RW * 16u;
      const uint32_t b_lbo = (uint32_t)p.NP * 16u;
      int it = 0, ring_s = 0;  // K-blocks issued so far; slot in the stage ring
      uint32_t ring_use = 0;
      int g = 0;   // accumulation intervals started so far: accumulator = g & 1
      bool failed = false;
      PROF_BEGIN();
      TileWalker tc_;
      for (tc_.init(p, order, tile_pairs); tc_.tile < p.tiles && !tc::uniform((uint32_t)*abort_flag) && !failed; tc_.next(p)) {
        const int Kr = (int)tc::uniform((uint32_t)TILE_ROWS((rowptr[tc_.ox + 1] - rowptr[tc_.ox]) * p.Bp));
        uint32_t accumulate = 0;
        int left = 0;  // K-blocks left in the open accumulation interval
        int kb = 0;
        STAGE_LOOP(++kb,) {
          const int s = ring_s;
          const uint32_t use = ring_use;
          const bool opens = left == 0;  // first K-block of an accumulation interval
          if (opens) left = p.PI;
          --left;
          if (opens && kb) ++g;
          const int acc = g & 1;
          PROF_WAIT_START();
          // full[s] completes only after every converter has seen raw_full[s]
          const bool okf = tc::mbar_wait(&ctl->full[s], use & 1, kSpinLimit) &&
                           (!opens || tc::mbar_wait(&ctl->dempty[acc], (uint32_t)(((g >> 1) & 1) ^ 1), kSpinLimit));
          PROF_WAIT_END();
          if (opens) accumulate = 0;
          if (!__all_sync(0xffffffffu, okf)) {
            if (lane == 0) raise_timeout(ctl, 4);
            failed = true;
            break;
          }
          tc::tc_fence_after_sync();
          const uint32_t d_addr = tmem0 + (uint32_t)(acc * p.NP);
          const uint32_t st = tc::smem_u32(stage_base + (size_t)s * stage_bytes);
          // descriptors of (k-step 0, tap 0); the others differ only in the start-address field
          const uint64_t da_hi0 = tc::smem_desc(st, a_lbo, 128u);
          const uint64_t da_lo0 = tc::smem_desc(st + p.a_stage_bytes, a_lbo, 128u);
          const uint64_t db_hi0 = tc::smem_desc(st + 2 * p.a_stage_bytes, b_lbo, 128u);
          const uint64_t db_lo0 = tc::smem_desc(st + 2 * p.a_stage_bytes + p.w_stage_bytes, b_lbo, 128u);
          const int rows_here = min(p.KB, Kr - k0);
          const int jb_here = (rows_here + 7) >> 3;
          const bool commit_tile = left == 0 || LAST_STAGE_OF_TILE;
          if (p.w_res_bytes) {
            // resident weights: the two 16-byte K-chunks of a k-step are the chunks
            // of two consecutive (entry, channel group) rows; their distance goes
            // into the descriptor
            const uint32_t wr = tc::smem_u32(w_res) + tc::uniform((uint32_t)(tc_.at * tile_chunks)) * 16u;
            const uint32_t tap_stride = (uint32_t)(B4 * p.NP);  // 16-byte units between taps
            const uint2 *ks = kstep_s + kofs_s[tc_.ox] + (k0 >> 3);
            for (int j = 0; j < jb_here; ++j) {
              const uint2 k = ks[j];
              const uint64_t db_hi = tc::smem_desc(wr + tc::uniform(k.x) * 16u, tc::uniform(k.y) * 16u, 128u);
              const uint64_t db_lo = db_hi + (p.w_res_bytes >> 4);
              if (tc::elect_one()) {
                uint32_t a_off = (uint32_t)(2 * j * p.RW), b_off = 0;
                uint32_t accum = accumulate;
                for (int t = 0; t < p.nky; ++t) {
                  if (!p.exact) {
                    tc::mma_tf32(d_addr, da_lo0 + a_off, db_hi + b_off, idesc, accum);
                    tc::mma_tf32(d_addr, da_hi0 + a_off, db_lo + b_off, idesc, 1u);
                    accum = 1u;
                  }
                  tc::mma_tf32(d_addr, da_hi0 + a_off, db_hi + b_off, idesc, accum);
                  accum = 1u;
                  a_off += (uint32_t)p.absBy;
                  b_off += tap_stride;
                }
              }
              accumulate = 1u;
            }
            if (tc::elect_one()) {
              tc::tc_commit(&ctl->empty[s]);
              if (commit_tile) tc::tc_commit(&ctl->dfull[acc]);
            }
          } else {
            const int taps_here = TAPS_HERE;
            if (tc::elect_one()) {
              uint32_t accum = accumulate;
              for (int j = 0; j < jb_here; ++j) {
                uint32_t a_off = (uint32_t)(2 * j * p.RW + TAP_GROUP * p.TG * p.absBy);  // 16-byte units
                uint32_t b_off = (uint32_t)(j * 2 * p.NP);
                for (int t = 0; t < taps_here; ++t) {
                  if (!p.exact) {
                    tc::mma_tf32(d_addr, da_lo0 + a_off, db_hi0 + b_off, idesc, accum);
                    tc::mma_tf32(d_addr, da_hi0 + a_off, db_lo0 + b_off, idesc, 1u);
                    accum = 1u;
                  }
                  tc::mma_tf32(d_addr, da_hi0 + a_off, db_hi0 + b_off, idesc, accum);
                  accum = 1u;
                  a_off += (uint32_t)p.absBy;
                  b_off += (uint32_t)(JB * 2 * p.NP);
                }
              }
              tc::tc_commit(&ctl->empty[s]);
              if (commit_tile) tc::tc_commit(&ctl->dfull[acc]);
            }
            accumulate = 1u;
          }
          __syncwarp();
        }
        if (Kr > 0) ++g;
      }
      PROF_END(2);
    }
    __syncwarp();
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
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
  if (p.A < 1 || p.A > kMaxBias || p.B < 1 || p.nky < 1 || p.nkx < 1 || p.noy < 16 || p.nox < 1 || p.N < 1)
    return false;
  if (p.table.max_row < 1) return false;
  const int absBy = p.By < 0 ? -p.By : p.By;
  const long long halo = (long long)absBy * (p.nky - 1);
  if (halo > 120) return false;
  // the gathered rows are fetched with TMA: 16-byte aligned base and strides
  if (p.niy % 4 != 0 || reinterpret_cast<uintptr_t>(p.in) % 16 != 0 || p.in_sn % 4 != 0 || p.in_sb % 4 != 0)
    return false;
  TcParams &q = plan.params;
#ifdef MELLIN_MASKED
  if (p.lens == nullptr || p.N > kMaxLens) return false;
  q.lens = p.lens, q.relu = p.relu, q.len_scale = p.len_scale, q.len_offset = p.len_offset;
  q.drop_threshold = p.drop_threshold, q.drop_seed = p.drop_seed, q.drop_scale = p.drop_threshold ? p.drop_scale : 1.f;
#endif
  q.bias = p.accumulate ? nullptr : p.bias, q.out = p.out;
  q.exact = p.exact_tf32;
  q.table_in_smem = (p.nox <= kMaxTableRows && p.table.num_entries <= kMaxTableEntries) ? 1 : 0;
  q.row_ptr = p.table.row_ptr, q.entries = p.table.entries, q.order = p.table.order, q.num_entries = (int)p.table.num_entries;
  q.N = p.N, q.A = p.A, q.B = p.B, q.Bp = (p.B + 3) / 4 * 4, q.nkx = p.nkx, q.nky = p.nky, q.nox = p.nox, q.noy = p.noy;
  q.out_sn = p.out_sn, q.out_sa = p.out_sa;
  q.absBy = absBy;
  q.ws0 = p.Cy + std::min(0, p.By * (p.nky - 1));
  const int a16 = (p.A + 15) / 16 * 16;
  q.a_tiles = (a16 + 127) / 128;  // the epilogue keeps NP running sums per thread: NP <= 128
  q.NP = ((a16 + q.a_tiles - 1) / q.a_tiles + 15) / 16 * 16;
  q.RW = (int)((kTileM + halo + 7) / 8 * 8);
  q.RWt = q.RW + 4;
  q.raw_chunk_floats = (4 * q.RWt + 31) / 32 * 32;
  q.y_tiles = (p.noy + kTileM - 1) / kTileM;
  const long long tiles = (long long)p.N * p.nox * q.y_tiles * q.a_tiles;
  if (tiles >= (1LL << 30)) return false;
  q.tiles = (int)tiles;
  int cols = 32;
  while (cols < 2 * q.NP) cols *= 2;
  q.tmem_cols = cols;
  // rows per stage: as many as fit a budget, at most what the longest table row needs
  const long long max_rows = ((long long)p.table.max_row * q.Bp + 7) / 8 * 8;
  // small weight sets stay resident in shared memory for the whole block
  plan.pack_floats = (size_t)p.nkx * p.nky * q.Bp * q.NP * q.a_tiles;
  const size_t w_all = plan.pack_floats * sizeof(float) + 2048;  // + room for the dummy second chunk of an odd tail
  q.w_pack_bytes = (uint32_t)(plan.pack_floats * sizeof(float));
  const long long ksteps = (p.table.num_entries * (long long)(q.Bp / 4) + 1) / 2 + p.nox;  // upper bound
  q.w_res_bytes = (q.table_in_smem && 2 * w_all <= 72 * 1024 && ksteps <= kMaxKSteps)
                      ? (uint32_t)((w_all + 127) / 128 * 128)
                      : 0u;
#ifdef MELLIN_TAP_GROUPS
  // Streamed weights of many linear taps: a stage carries four of them, and every
  // block of rows is staged once per group of four.
  if (q.w_res_bytes || p.nky <= 5) return false;  // the single-group kernel covers these
  q.TG = 4;
#else
  q.TG = p.nky;
#endif
  q.G = (p.nky + q.TG - 1) / q.TG;
  plan.pack_floats = (size_t)p.nkx * q.G * q.TG * q.Bp * q.NP * q.a_tiles;
  // bytes per row: raw copy, A (hi+lo) and, unless resident, W (hi+lo)
  const size_t per_row =
      (size_t)q.raw_chunk_floats + 8u * q.RW + (q.w_res_bytes ? 0u : 8u * (size_t)q.TG * q.NP);
  const size_t budget = 227 * 1024 - kStageOffset - 1024 - 2 * (size_t)q.w_res_bytes;
  int stages = 3;
  long long kb = (long long)(budget / stages / per_row) / 8 * 8;
  if (kb < 8) {
    stages = 2;
    kb = (long long)(budget / stages / per_row) / 8 * 8;
  }
  if (kb < 8) return false;
  kb = std::min<long long>(std::min<long long>(kb, max_rows), kMaxKB);
  // at most 96 chained MMAs (3 per tap per 8 rows) per K-block, see the note on accumulation above
  kb = std::min<long long>(kb, std::max<long long>(8, 96 / (3 * q.TG) * 8));
  // a stage that stays inside one table entry can be fetched by one wide box and one weight copy
  if (q.Bp >= 8 && q.Bp % kb != 0)
    for (long long k = kb; k >= 8; k -= 8)
      if (q.Bp % k == 0) {
        kb = k;
        break;
      }
  q.KB = (int)kb;
  // short K-blocks leave room for a deeper ring
  while (stages < kMaxStages && (size_t)(stages + 1) * q.KB * per_row <= budget) ++stages;
  q.stages = stages;
  q.PI = std::max(1, 96 / (3 * q.TG * (q.KB / 8)));
  // when every stage lies inside one table entry, one wide box replaces its KB / 4
  // row copies; the chunks must then sit back to back: rows of RW + 8 positions
  q.wide_box = 0;
  q.kblock_pack = 0;
  if (q.KB >= 8 && q.Bp % q.KB == 0) {
    const int rwt = q.RW + 8;
    const size_t grown = (size_t)q.stages * q.KB * (size_t)(rwt - q.raw_chunk_floats / 4) * 4;
    const size_t now = kStageOffset + 2 * (size_t)q.w_res_bytes + (size_t)q.stages * q.KB * per_row;
    if (now + grown <= 227 * 1024) {
      q.wide_box = 1;
      q.RWt = rwt;
      q.raw_chunk_floats = 4 * rwt;
      q.kblock_pack = q.w_res_bytes ? 0 : 1;
    }
  }
  q.a_stage_bytes = (uint32_t)(q.KB / 4 * q.RW * 16);
  if (q.G > 1 && !q.kblock_pack) return false;  // tap groups exist in the stage-major weight layout only
  q.w_stage_bytes = q.w_res_bytes ? 0u : (uint32_t)(q.TG * (q.KB / 8) * q.NP * 32);
  q.raw_stage_bytes = (uint32_t)(q.KB / 4 * q.raw_chunk_floats * 4);
  plan.smem = kStageOffset + 2 * (size_t)q.w_res_bytes +
              (size_t)stages * (2 * (q.a_stage_bytes + q.w_stage_bytes) + q.raw_stage_bytes);
  // one block per SM: keep shared memory above half of the SM so that the
  // TMEM request of a co-resident block can never wait for columns
  plan.smem = std::max<size_t>(plan.smem, 116 * 1024);
  if (plan.smem > 227 * 1024) return false;
  plan.grid = (int)std::min<long long>(q.tiles, sm_count());
  q.profile = 0;
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

#if !defined(MELLIN_TAP_GROUPS) && !defined(MELLIN_MASKED)
#define MELLIN_BASE_BUILD 1
#endif
#ifdef MELLIN_BASE_BUILD
// the same kernel built for layers with many linear taps (tc_direct_taps.cu)
size_t direct_tc_workspace_bytes_taps(const DirectProblem<float> &p);
int launch_direct_tc_taps(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream);
int tc_take_error_taps(int *code);
int tc_take_error_masked(int *code);
#endif

size_t TC_FN(direct_tc_workspace_bytes)(const DirectProblem<float> &p) {
  TcPlan plan;
#ifdef MELLIN_BASE_BUILD
  if (p.nky > 5 && !plan_tc_direct(p, plan)) return direct_tc_workspace_bytes_taps(p);
#endif
  if (!plan_tc_direct(p, plan)) return 0;
  return 2 * ((plan.pack_floats * sizeof(float) + 255) / 256 * 256);
}

// Returns MELLIN_ERR_UNSUPPORTED (without recording an error message) when the
// problem is outside what this kernel covers; the caller then uses the CUDA-core path.
int TC_FN(launch_direct_tc)(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes,
                            cudaStream_t stream) {
  TcPlan plan;
#ifdef MELLIN_BASE_BUILD
  if (p.nky > 5 && !plan_tc_direct(p, plan)) return launch_direct_tc_taps(p, workspace, workspace_bytes, stream);
#endif
  if (!plan_tc_direct(p, plan) || p.table.order == nullptr) return MELLIN_ERR_UNSUPPORTED;
  const size_t part = (plan.pack_floats * sizeof(float) + 255) / 256 * 256;
  if (workspace == nullptr || workspace_bytes < 2 * part || reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
    return fail(MELLIN_ERR_WORKSPACE, "workspace too small or misaligned: need " + std::to_string(2 * part) +
                                          " bytes (16-byte aligned), got " + std::to_string(workspace_bytes));
  // the activations as a 4-D tensor (position, Mellin row, batch, channel) with their real strides
  CUtensorMap in_map, in_map_wide;
  {
    EncodeTiledFn encode = tensor_map_encoder();
    if (encode == nullptr) return fail(MELLIN_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[4] = {(cuuint64_t)p.niy, (cuuint64_t)p.nix, (cuuint64_t)p.N, (cuuint64_t)p.B};
    const cuuint64_t strides[3] = {(cuuint64_t)p.niy * sizeof(float), (cuuint64_t)p.in_sn * sizeof(float),
                                   (cuuint64_t)p.in_sb * sizeof(float)};
    const cuuint32_t box[4] = {(cuuint32_t)plan.params.RWt, 1u, 1u, 4u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUresult r = encode(&in_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(p.in), dims, strides, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return MELLIN_ERR_UNSUPPORTED;  // strides the copy engine cannot express
    in_map_wide = in_map;
    if (plan.params.wide_box) {
      const cuuint32_t wide[4] = {(cuuint32_t)plan.params.RWt, 1u, 1u, (cuuint32_t)plan.params.KB};
      const CUresult rw = encode(&in_map_wide, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(p.in), dims,
                                 strides, wide, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (rw != CUDA_SUCCESS) return MELLIN_ERR_UNSUPPORTED;
    }
  }
  float *w_hi = static_cast<float *>(workspace);
  float *w_lo = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + part);
  {
    const int threads = 256;
    const long long total = (long long)plan.pack_floats;
    const int blocks = (int)std::min<long long>((total + threads - 1) / threads, 4096);
    pack_weights_kernel<<<blocks, threads, 0, stream>>>(p.w, p.w_sa, p.w_sb, p.A, p.B, p.nkx, p.nky, plan.params.NP,
                                                        plan.params.a_tiles, p.By,
                                                        plan.params.kblock_pack ? plan.params.KB : 0, plan.params.TG,
                                                        plan.params.G, w_hi, w_lo);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("pack_weights_kernel: ") + cudaGetErrorString(err));
    count_launch();
  }
  plan.params.w_hi = w_hi;
  plan.params.w_lo = w_lo;
#ifdef MELLIN_TUNING_HOOKS
  const char *prof = getenv("MELLIN_TC_PROFILE");
#else
  const char *prof = nullptr;
#endif
  plan.params.profile = (prof != nullptr && prof[0] == '1') ? 1 : 0;
  void (*kernel)(TcParams, const CUtensorMap, const CUtensorMap) = nullptr;
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
  kernel<<<plan.grid, kThreads, plan.smem, stream>>>(plan.params, in_map, in_map_wide);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("tc_direct_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

int TC_FN(tc_read_prof)(long long *out) {
  return cudaMemcpyFromSymbol(out, g_tc_prof, 16 * sizeof(long long)) == cudaSuccess ? 0 : 2;
}

// Reads and clears the device-side timeout flag of the current device
// (synchronises the device).
int TC_FN(tc_take_error)(int *code) {
  int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(code, g_tc_error, sizeof(int));
  if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("device status: ") + cudaGetErrorString(err));
#ifdef MELLIN_BASE_BUILD
  int other = 0;
  int rc = tc_take_error_taps(&other);
  if (rc) return rc;
  if (*code == 0) *code = other;
  rc = tc_take_error_masked(&other);
  if (rc) return rc;
  if (*code == 0) *code = other;
#endif
  return MELLIN_OK;
}

}  // namespace mellin
