// Weight (+ bias) gradient on tensor cores (tcgen05, sm_100a) for layers with
// many channels on both sides:
//
//   gw[a, b, kx, ky] = sum_{n} sum_{(ox, ix) in row kx} sum_oy
//                      go[n, a, ox, oy] * x[n, b, ix, oy + By * ky + Cy]
//
// Per Mellin tap kx this is a GEMM whose reduction runs over positions:
//   M = 128 output channels a   (TMEM lanes)
//   N = 64 input channels b     (TMEM columns), one accumulator per linear tap
//   K = positions oy of every (utterance, table entry) of row kx
// Both operands are K-major (positions are contiguous in memory).  A stage holds
// 16 positions: one TMA box of grad_y (128 rows) and one of x (64 rows, a few
// positions wider); converter warps split them into TF32 hi/lo parts and write
// the x rows once per linear tap, shifted by the tap's offset.  Three MMAs
// (lo*hi, hi*lo, hi*hi) per 8 positions and tap keep FP32 accuracy.
//
// The reduction is thousands of MMAs long, and the tensor core's accumulator
// rounds toward zero at every MMA, so sums are kept in two levels, both in
// TMEM: level 1 takes at most 30 chained MMAs; the epilogue warps then add it
// into level 2 with ordinary round-to-nearest FP32 adds (tcgen05.ld / st).
//
// Work items are (utterance, entry, run of stages); the items of Mellin tap kx
// are dealt to Z[kx] blocks, Z[kx] in proportion to the tap's number of entries
// (every block computes the same split from the table's row offsets).  Blocks
// write partial sums; a second, fixed-order pass adds them (no floating-point
// atomics).  The bias
// gradient rides along: converter threads sum the grad_y values they convert
// (each grad_y row is owned by exactly one table entry).
#include <cuda.h>

#include <cstdlib>
#include <algorithm>
#include <string>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"
#include "tc_ptx.cuh"

namespace mellin {

namespace {

constexpr int kEpilogueWarps = 4;
constexpr int kConvertGroups = 2;  // groups of converter warps take alternate stages
constexpr int kGroupWarps = 8;
constexpr int kConvertWarps = kConvertGroups * kGroupWarps;
constexpr int kGroupThreads = kGroupWarps * 32;
constexpr int kMmaWarp = kEpilogueWarps + kConvertWarps;
constexpr int kCopyWarp = kMmaWarp + 1;
constexpr int kThreads = (kCopyWarp + 1) * 32;
constexpr int kTM = 128;       // output channels per block
constexpr int kNB = 64;        // input channels per block
constexpr int kKB = 16;        // positions per stage
constexpr int kRawStages = 6;   // TMA boxes in flight (at most): deep, to cover the copy latency
constexpr int kOpStages = 3;    // converted operand sets
constexpr int kPromote = 8;    // stages per level-1 interval: 2 k-steps x 3 MMAs x 8 = 48 chained MMAs
constexpr int kMaxRows = 64;   // Mellin taps
constexpr int kMaxTaps = 3;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr int kL2Col = 256;    // first TMEM column of the level-2 sums
// Operand slabs: one per 4-position chunk, rows 16 bytes apart.  32 bytes of
// padding between slabs spread the converters' 16-byte stores over all banks.
// An x slab holds the rows of every linear tap, (tap, b): the taps are extra
// columns of one MMA.
constexpr uint32_t kGoSlab = kTM * 16 + 32;
__host__ __device__ constexpr uint32_t x_slab(int nky) { return (uint32_t)(nky * kNB * 16 + 32); }

struct GwParams {
  const int32_t *row_ptr;  // by-kx table
  const int2 *entries;
  const int *lens;         // per utterance: grad_y is zero from this position on (null: no such promise)
  float *part_w;           // [slice][tap slot][B][A], slices of tap kx at prefix[kx] ...
  float *part_b;           // [slice][A] or null
  int N, A, B, nkx, nky, noy;
  int absBy, xs0;          // tap spacing; first x position of position block 0 for this launch's first tap slot
  int g0, nky_total;       // this launch covers tap slots g0 .. g0 + nky - 1 (ascending input offset) of nky_total
  int By;
  int RXW;                 // positions per raw x row
  int a_tiles, b_tiles;
  int target_slices;       // sum of Z[kx] aimed at
  int stages_per_row;      // ceil(noy / 16)
  int profile;
  int exact;               // operands are exact in TF32: no compensation MMAs
  int raw_stages;          // 3 .. kRawStages, as shared memory allows
  int chunks, chunk_stages;  // a row of positions is cut into `chunks` runs of at most `chunk_stages` stages
  uint32_t go_raw_bytes, x_raw_bytes, go_op_bytes, x_op_bytes;  // per stage; operand sizes per hi or lo part (x: per tap)
};

// Slices per Mellin tap: prefix[kx] .. prefix[kx + 1].  A pure function of the
// table's row offsets, so the blocks and the reduction pass agree on it.
__device__ void slice_prefix(const int32_t *row_ptr, int nkx, long long items_per_entry, int target, int *prefix) {
  const long long total = row_ptr[nkx] - row_ptr[0];
  int acc = 0;
  for (int k = 0; k < nkx; ++k) {
    prefix[k] = acc;
    const long long ne = row_ptr[k + 1] - row_ptr[k];
    long long zk = 0;
    if (ne > 0) {
      zk = ((long long)target * ne + total / 2) / total;
      zk = max(1LL, min(zk, ne * items_per_entry));
    }
    acc += (int)zk;
  }
  prefix[nkx] = acc;
}

constexpr int kHeaderBytes = 2048;  // Control, then the 128-byte aligned stages

struct Control {
  uint64_t raw_full[kRawStages], raw_empty[kRawStages], full[kOpStages], empty[kOpStages];
  uint64_t l1_full, l1_empty;
  uint32_t tmem_base;
  int abort;
  int prefix[kMaxRows + 1];
  float bias[kConvertGroups][kTM];
};

static_assert(sizeof(Control) <= kHeaderBytes, "Control must fit the header");

__device__ int g_gw_error = 0;
__device__ long long g_gw_prof[16];  // per-role wait / work cycles of block 0 (written when profiling is on)

#define PROF_BEGIN() long long prof_t0 = clock64(), prof_wait = 0, prof_t1 = 0
#define PROF_WAIT_START() \
  if (p.profile) prof_t1 = clock64()
#define PROF_WAIT_END() \
  if (p.profile) prof_wait += clock64() - prof_t1
#define PROF_END(slot)                                           \
  if (blockIdx.x == 0 && lane == 0 && p.profile) {               \
    g_gw_prof[2 * (slot)] = prof_wait;                           \
    g_gw_prof[2 * (slot) + 1] = clock64() - prof_t0 - prof_wait; \
  }

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ void raise_timeout(Control *ctl, int code) {
  atomicCAS(&g_gw_error, 0, code);
  ctl->abort = 1;
}

template <int NKY>
__global__ void __launch_bounds__(kThreads, 1)
tc_gradw_kernel(const GwParams p, const __grid_constant__ CUtensorMap go_map, const __grid_constant__ CUtensorMap x_map) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Control *ctl = reinterpret_cast<Control *>(smem);
  unsigned char *raw_base = smem + kHeaderBytes;
  constexpr uint32_t kXSlab = x_slab(NKY);
  const uint32_t op_bytes = 2 * p.go_op_bytes + 2 * p.x_op_bytes;
  const uint32_t raw_bytes = p.go_raw_bytes + p.x_raw_bytes;
  unsigned char *op_base = raw_base + (size_t)p.raw_stages * raw_bytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // block -> (slice, channel tiles); slice -> (tap kx, split index z of Z)
  const int bt = blockIdx.x % p.b_tiles;
  const int at = (blockIdx.x / p.b_tiles) % p.a_tiles;
  const int slice = blockIdx.x / (p.b_tiles * p.a_tiles);
  if (tid == 0) slice_prefix(p.row_ptr, p.nkx, (long long)p.N * p.chunks, p.target_slices, ctl->prefix);
  __syncthreads();
  if (slice >= ctl->prefix[p.nkx]) return;  // the grid is sized for the worst case of the rounding
  int kx = 0;
  while (slice >= ctl->prefix[kx + 1]) ++kx;
  const int z = slice - ctl->prefix[kx];
  const int Z = ctl->prefix[kx + 1] - ctl->prefix[kx];
  const int e0 = p.row_ptr[kx];
  const int ne = p.row_ptr[kx + 1] - e0;
  // item i = (n, entry, chunk) = (i / (ne chunks), e0 + (i / chunks) % ne, i % chunks); this block takes i = z, z + Z, ...
  const int items = p.N * ne * p.chunks;
  const bool want_bias = p.part_b != nullptr && bt == 0;
#define ITEM_ENTRY(i) (e0 + ((i) / p.chunks) % ne)
#define ITEM_FIRST_STAGE(i) (((i) % p.chunks) * p.chunk_stages)
// with per-utterance lengths (grad_y is zero from position lens[n] on) a row ends at its utterance's last stage
#define ITEM_ROW_STAGES(i) \
  (p.lens == nullptr ? p.stages_per_row : min(p.stages_per_row, (p.lens[(i) / (ne * p.chunks)] + kKB - 1) / kKB))
#define ITEM_END_STAGE(i) max(ITEM_FIRST_STAGE(i), min(ITEM_ROW_STAGES(i), ITEM_FIRST_STAGE(i) + p.chunk_stages))

  if (tid == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      tc::mbar_init(&ctl->raw_full[s], 1);
      tc::mbar_init(&ctl->raw_empty[s], kGroupThreads);
    }
    for (int s = 0; s < kOpStages; ++s) {
      tc::mbar_init(&ctl->full[s], kGroupThreads);
      tc::mbar_init(&ctl->empty[s], 1);
    }
    tc::mbar_init(&ctl->l1_full, 1);
    tc::mbar_init(&ctl->l1_empty, kEpilogueWarps * 32);
    ctl->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tc::tmem_alloc(&ctl->tmem_base, 512u);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  // number of stages that carry MMAs (entries flagged bias-only carry none)
  int mma_stages = 0;
  for (int i = z; i < items; i += Z)
    if (!(p.entries[ITEM_ENTRY(i)].x & kFlagBiasOnly)) mma_stages += ITEM_END_STAGE(i) - ITEM_FIRST_STAGE(i);
  const int intervals = (mma_stages + kPromote - 1) / kPromote;

  if (warp < kEpilogueWarps) {
    // ===================== epilogue: level-1 -> level-2 promotion, final write =====================
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    constexpr int groups = NKY * (kNB / 16);
    {
      uint32_t zero[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) zero[i] = 0u;
      for (int g = 0; g < groups; ++g) tc::tmem_st16(tmem_base + lane_base + (uint32_t)(kL2Col + 16 * g), zero);
      tc::tmem_st_wait();
    }
    bool failed = false;
    PROF_BEGIN();
    for (int iv = 0; iv < intervals && !failed; ++iv) {
      PROF_WAIT_START();
      const bool ok = tc::mbar_wait(&ctl->l1_full, (uint32_t)(iv & 1), kSpinLimit);
      PROF_WAIT_END();
      if (!__all_sync(0xffffffffu, ok)) {
        raise_timeout(ctl, 3);
        failed = true;
        break;
      }
      tc::tc_fence_after_sync();
      for (int g = 0; g < groups; ++g) {
        uint32_t a[16], b[16];
        tc::tmem_ld16(tmem_base + lane_base + (uint32_t)(16 * g), a);
        tc::tmem_ld16(tmem_base + lane_base + (uint32_t)(kL2Col + 16 * g), b);
        tc::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) b[i] = __float_as_uint(__uint_as_float(a[i]) + __uint_as_float(b[i]));
        tc::tmem_st16(tmem_base + lane_base + (uint32_t)(kL2Col + 16 * g), b);
      }
      tc::tmem_st_wait();
      tc::tc_fence_before_sync();
      tc::mbar_arrive(&ctl->l1_empty);
    }
    if (warp == 0) { PROF_END(0); }
    if (!failed) {
      // partial sums of this block: row a = lane (consecutive addresses), columns (tap slot, b)
      const int a = at * kTM + warp * 32 + lane;
      float *pw = p.part_w + (long long)slice * NKY * p.B * p.A;
      for (int g = 0; g < groups; ++g) {
        uint32_t v[16];
        tc::tmem_ld16(tmem_base + lane_base + (uint32_t)(kL2Col + 16 * g), v);
        tc::tmem_ld_wait();
        const int t = g / (kNB / 16);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int b = bt * kNB + (g % (kNB / 16)) * 16 + i;
          if (a < p.A && b < p.B) pw[((long long)t * p.B + b) * p.A + a] = __uint_as_float(v[i]);
        }
      }
    }
  } else if (warp < kMmaWarp) {
    // ===================== converters =====================
    const int group = (warp - kEpilogueWarps) / kGroupWarps;
    const int ctid = (tid - kEpilogueWarps * 32) % kGroupThreads;
    // grad_y items: (row, 4-position chunk); this thread: rows r0 and r0 + 64, chunk cg
    const int go_row = ctid >> 2, go_chunk = ctid & 3;
    // x items: (row, chunk): one per thread
    const int x_row = ctid >> 2, x_chunk = ctid & 3;
    float bsum[2] = {0.f, 0.f};
    int it = 0;
    bool failed = false;
    PROF_BEGIN();
    for (int i = z; i < items && !failed; i += Z) {
      const int flags = p.entries[ITEM_ENTRY(i)].x;
      const bool bias_only = (flags & kFlagBiasOnly) != 0;
      const bool add_bias = want_bias && (flags & kFlagBiasOwner) != 0;
      const int s_end = ITEM_END_STAGE(i);
      for (int sidx = ITEM_FIRST_STAGE(i); sidx < s_end; ++sidx, ++it) {
        if (it % kConvertGroups != group) continue;
        const int r = it % p.raw_stages, s = it % kOpStages;
        PROF_WAIT_START();
        const bool raw_ok = tc::mbar_wait(&ctl->raw_full[r], (uint32_t)((it / p.raw_stages) & 1), kSpinLimit) &&
                            tc::mbar_wait(&ctl->empty[s], (uint32_t)(((it / kOpStages) & 1) ^ 1), kSpinLimit);
        PROF_WAIT_END();
        if (!raw_ok) {
          raise_timeout(ctl, 1);
          failed = true;
          break;
        }
        const unsigned char *raw = raw_base + (size_t)r * raw_bytes;
        unsigned char *ops = op_base + (size_t)s * op_bytes;
        const float *raw_go = reinterpret_cast<const float *>(raw);
        const float *raw_x = reinterpret_cast<const float *>(raw + p.go_raw_bytes);
        float4 *go_hi = reinterpret_cast<float4 *>(ops);
        float4 *go_lo = reinterpret_cast<float4 *>(ops + p.go_op_bytes);
        unsigned char *x_ops = ops + 2 * p.go_op_bytes;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int row = go_row + 64 * k;
          const float4 v = *reinterpret_cast<const float4 *>(raw_go + row * kKB + 4 * go_chunk);
          if (add_bias) bsum[k] += (v.x + v.y) + (v.z + v.w);
          if (!bias_only) {
            float4 h, l;
            h.x = tf32_hi(v.x), h.y = tf32_hi(v.y), h.z = tf32_hi(v.z), h.w = tf32_hi(v.w);
            l.x = v.x - h.x, l.y = v.y - h.y, l.z = v.z - h.z, l.w = v.w - h.w;
            go_hi[go_chunk * (kGoSlab / 16) + row] = h;
            go_lo[go_chunk * (kGoSlab / 16) + row] = l;
          }
        }
        if (!bias_only) {
          const int xs = sidx * kKB + p.xs0;
          const int lead = xs & 3;
          const float *xr = raw_x + x_row * p.RXW + lead + 4 * x_chunk;
          float win[4 + NKY - 1];  // taps one position apart share a window
          if (p.absBy == 1) {
#pragma unroll
            for (int k = 0; k < 4 + NKY - 1; ++k) win[k] = xr[k];
          }
#pragma unroll
          for (int t = 0; t < NKY; ++t) {
            float v0, v1, v2, v3;
            if (p.absBy == 1) {
              v0 = win[t], v1 = win[t + 1], v2 = win[t + 2], v3 = win[t + 3];
            } else {
              const float *q = xr + t * p.absBy;
              v0 = q[0], v1 = q[1], v2 = q[2], v3 = q[3];
            }
            float4 h, l;
            h.x = tf32_hi(v0), h.y = tf32_hi(v1), h.z = tf32_hi(v2), h.w = tf32_hi(v3);
            l.x = v0 - h.x, l.y = v1 - h.y, l.z = v2 - h.z, l.w = v3 - h.w;
            float4 *x_hi = reinterpret_cast<float4 *>(x_ops);
            float4 *x_lo = reinterpret_cast<float4 *>(x_ops + p.x_op_bytes);
            x_hi[x_chunk * (kXSlab / 16) + t * kNB + x_row] = h;
            x_lo[x_chunk * (kXSlab / 16) + t * kNB + x_row] = l;
          }
        }
        // The proxy fence orders this thread's shared-memory accesses (its reads of
        // the raw slot as well as its operand writes) before what the copy engine
        // and the tensor core do once the two barriers below let them go on.
        tc::fence_proxy_async();
        tc::mbar_arrive(&ctl->raw_empty[r]);
        tc::mbar_arrive(&ctl->full[s]);
      }
    }
    if (warp == kEpilogueWarps) { PROF_END(1); }
    if (warp == kEpilogueWarps + kGroupWarps) { PROF_END(4); }
    if (want_bias) {
      // the four chunk threads of a row are adjacent lanes; each converter group
      // writes its own slot, added after the block-wide barrier below
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        float v = bsum[k];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if (go_chunk == 0) ctl->bias[group][go_row + 64 * k] = v;
      }
    }
  } else if (warp == kCopyWarp) {
    // ===================== copy issuer =====================
    if (lane == 0) {
      int it = 0;
      bool failed = false;
      PROF_BEGIN();
      for (int i = z; i < items && !failed; i += Z) {
        const int n = i / (ne * p.chunks);
        const int2 e = p.entries[ITEM_ENTRY(i)];
        const bool bias_only = (e.x & kFlagBiasOnly) != 0;
        const int ox = e.x & kIndexMask;
        const int s_end = ITEM_END_STAGE(i);
        for (int sidx = ITEM_FIRST_STAGE(i); sidx < s_end; ++sidx, ++it) {
          const int s = it % p.raw_stages;
          PROF_WAIT_START();
          const bool empty_ok = tc::mbar_wait(&ctl->raw_empty[s], (uint32_t)(((it / p.raw_stages) & 1) ^ 1), kSpinLimit);
          PROF_WAIT_END();
          if (!empty_ok) {
            raise_timeout(ctl, 5);
            failed = true;
            break;
          }
          unsigned char *st = raw_base + (size_t)s * raw_bytes;
          tc::mbar_arrive_expect_tx(&ctl->raw_full[s], p.go_raw_bytes + (bias_only ? 0u : p.x_raw_bytes));
          tc::tma_load_4d(st, &go_map, sidx * kKB, ox, at * kTM, n, &ctl->raw_full[s]);
          if (!bias_only) {
            const int xs = sidx * kKB + p.xs0;
            tc::tma_load_4d(st + p.go_raw_bytes, &x_map, xs - (xs & 3), e.y, bt * kNB, n, &ctl->raw_full[s]);
          }
        }
      }
      PROF_END(3);
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer =====================
    // The whole warp walks the items and one elected lane issues: addresses and descriptors computed by all
    // lanes from warp-uniform values (what is read from shared or global memory is broadcast from lane 0 to
    // say so) can live in the uniform registers the MMA reads them from.
    {
      const uint32_t tmem0 = tc::uniform(tmem_base);
      const int zu = (int)tc::uniform((uint32_t)z), Zu = (int)tc::uniform((uint32_t)Z);
      const int items_u = (int)tc::uniform((uint32_t)items), mma_stages_u = (int)tc::uniform((uint32_t)mma_stages);
      const uint32_t idesc = tc::idesc_tf32(kTM, NKY * kNB);  // the taps side by side in the columns
      // descriptors of stage 0; a stage's are these plus its offset
      const uint32_t ops0 = tc::smem_u32(op_base);
      const uint64_t dgo_hi = tc::smem_desc(ops0, kGoSlab, 128u);
      const uint64_t dgo_lo = tc::smem_desc(ops0 + p.go_op_bytes, kGoSlab, 128u);
      const uint64_t dx_hi = tc::smem_desc(ops0 + 2 * p.go_op_bytes, kXSlab, 128u);
      const uint64_t dx_lo = tc::smem_desc(ops0 + 2 * p.go_op_bytes + p.x_op_bytes, kXSlab, 128u);
      int it = 0, ms = 0;  // stages seen, stages with MMAs issued
      uint32_t fresh = 0;  // 0: the next MMA overwrites the level-1 accumulators
      bool failed = false;
      long long prof_l1 = 0;
      PROF_BEGIN();
      for (int i = zu; i < items_u && !failed; i += Zu) {
        const bool bias_only = tc::uniform((uint32_t)(p.entries[ITEM_ENTRY(i)].x & kFlagBiasOnly)) != 0;
        const int s_first = (int)tc::uniform((uint32_t)ITEM_FIRST_STAGE(i));
        const int s_end = (int)tc::uniform((uint32_t)ITEM_END_STAGE(i));
        for (int sidx = s_first; sidx < s_end; ++sidx, ++it) {
          const int s = it % kOpStages;
          PROF_WAIT_START();
          const bool full_ok = tc::mbar_wait(&ctl->full[s], (uint32_t)((it / kOpStages) & 1), kSpinLimit);
          PROF_WAIT_END();
          if (!__all_sync(0xffffffffu, full_ok)) {
            if (lane == 0) raise_timeout(ctl, 4);
            failed = true;
            break;
          }
          if (!bias_only) {
            if (ms % kPromote == 0) {
              // a new level-1 interval: the epilogue must have drained the previous one
              const int iv = ms / kPromote;
              const long long l1_t0 = p.profile ? clock64() : 0;
              const bool l1_ok = tc::mbar_wait(&ctl->l1_empty, (uint32_t)((iv & 1) ^ 1), kSpinLimit);
              if (p.profile) prof_l1 += clock64() - l1_t0;
              if (!__all_sync(0xffffffffu, l1_ok)) {
                if (lane == 0) raise_timeout(ctl, 2);
                failed = true;
                break;
              }
              fresh = 0;
            }
            tc::tc_fence_after_sync();
            const uint32_t soff = (uint32_t)s * (op_bytes >> 4);  // descriptor addresses count 16-byte units
            if (tc::elect_one()) {
              uint32_t fr = fresh;
#pragma unroll
              for (int ks = 0; ks < kKB / 8; ++ks) {
                // the three products of the hi/lo split
                const uint32_t ka = soff + (uint32_t)(ks * 2 * (kGoSlab / 16)), kb = soff + (uint32_t)(ks * 2 * (kXSlab / 16));
                if (!p.exact) {
                  tc::mma_tf32(tmem0, dgo_lo + ka, dx_hi + kb, idesc, fr);
                  tc::mma_tf32(tmem0, dgo_hi + ka, dx_lo + kb, idesc, 1u);
                  fr = 1u;
                }
                tc::mma_tf32(tmem0, dgo_hi + ka, dx_hi + kb, idesc, fr);
                fr = 1u;
              }
            }
            fresh = 1u;
            ++ms;
          }
          if (tc::elect_one()) {
            tc::tc_commit(&ctl->empty[s]);
            if (!bias_only && (ms % kPromote == 0 || ms == mma_stages_u)) tc::tc_commit(&ctl->l1_full);
          }
          __syncwarp();
        }
      }
      PROF_END(2);
      if (blockIdx.x == 0 && lane == 0 && p.profile) g_gw_prof[12] = prof_l1, g_gw_prof[13] = it;
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, 512u);
  }
  if (want_bias && tid < kTM && at * kTM + tid < p.A) {
    float v = 0.f;
#pragma unroll
    for (int g = 0; g < kConvertGroups; ++g) v += ctl->bias[g][tid];
    p.part_b[(long long)slice * p.A + at * kTM + tid] = v;
  }
#undef ITEM_ENTRY
#undef ITEM_FIRST_STAGE
#undef ITEM_END_STAGE
#undef ITEM_ROW_STAGES
}

// gw[a, b, kx, ky] = sum over the slices of tap kx; gb[a] = sum over all slices.
// A block owns 32 consecutive partial-sum addresses; its 8 warps split the
// slices and are combined in a fixed order.
__global__ void tc_gradw_reduce_kernel(const GwParams p, float *__restrict__ gw, float *__restrict__ gb,
                                       long long w_blocks) {
  __shared__ float red[8][33];
  __shared__ int prefix[kMaxRows + 1];
  if (threadIdx.x == 0) slice_prefix(p.row_ptr, p.nkx, (long long)p.N * p.chunks, p.target_slices, prefix);
  __syncthreads();
  const int lane = threadIdx.x & 31, zs = threadIdx.x >> 5;
  const long long per_tap = (long long)p.nky * p.B * p.A;
  float s = 0.f;
  long long out = -1;
  if ((long long)blockIdx.x < w_blocks) {
    const long long j = blockIdx.x * 32LL + lane;  // (kx, tap slot, b, a)
    if (j < per_tap * p.nkx) {
      const int kx = (int)(j / per_tap);
      const long long r = j % per_tap;
      const int a = (int)(r % p.A), b = (int)((r / p.A) % p.B), t = (int)(r / ((long long)p.A * p.B));
      const int slot = p.g0 + t;
      const int ky = p.By < 0 ? p.nky_total - 1 - slot : slot;
      out = (((long long)a * p.B + b) * p.nkx + kx) * p.nky_total + ky;
      for (int z = prefix[kx] + zs; z < prefix[kx + 1]; z += 8) s += p.part_w[z * per_tap + r];
    }
  } else {
    const long long a = ((long long)blockIdx.x - w_blocks) * 32LL + lane;
    if (a < p.A) {
      out = a;
      for (int z = zs; z < prefix[p.nkx]; z += 8) s += p.part_b[(long long)z * p.A + a];
    }
  }
  red[zs][lane] = s;
  __syncthreads();
  if (zs == 0 && out >= 0) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][lane];
    ((long long)blockIdx.x < w_blocks ? gw : gb)[out] = t;
  }
}

struct GwPlan {
  GwParams params;
  size_t smem = 0;
  int blocks = 0, max_slices = 0;
};

// Plans the launch for tap slots g0 .. g0 + nky - 1 (nky <= 3) of the problem's p.nky taps.
bool plan_tc_gradw(const GradWProblem<float> &p, int g0, int nky, GwPlan &plan) {
  if (p.Dy != 1 || p.Ay != 1) return false;
  if (p.A < 32 || p.B < 16 || nky < 1 || nky > kMaxTaps || g0 < 0 || g0 + nky > p.nky || p.nkx < 1 || p.nkx > kMaxRows || p.N < 1 || p.nox < 1 || p.noy < 16) return false;
  const int absBy = p.By < 0 ? -p.By : p.By;
  const int halo = absBy * (nky - 1);
  if (halo > 28) return false;
  // TMA: 16-byte aligned bases and strides
  if (p.noy % 4 != 0 || p.niy % 4 != 0 || reinterpret_cast<uintptr_t>(p.go) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(p.in) % 16 != 0)
    return false;
  GwParams &q = plan.params;
  q.profile = 0;
  q.row_ptr = p.table.row_ptr, q.entries = p.table.entries;
  q.lens = p.lens;
  q.N = p.N, q.A = p.A, q.B = p.B, q.nkx = p.nkx, q.nky = nky, q.noy = p.noy;
  q.g0 = g0, q.nky_total = p.nky;
  q.absBy = absBy, q.By = p.By;
  q.exact = p.exact_tf32;
  q.xs0 = p.Cy + std::min(0, p.By * (p.nky - 1)) + g0 * absBy;
  q.RXW = (kKB + halo + 3 + 3) / 4 * 4;
  q.a_tiles = (p.A + kTM - 1) / kTM;
  q.b_tiles = (p.B + kNB - 1) / kNB;
  q.stages_per_row = (p.noy + kKB - 1) / kKB;
  q.chunks = (q.stages_per_row + 2 * kPromote - 1) / (2 * kPromote);
  q.chunk_stages = (q.stages_per_row + q.chunks - 1) / q.chunks;
  const int tiles = q.a_tiles * q.b_tiles;
  q.target_slices = std::max(2 * p.nkx, (2 * sm_count() + tiles - 1) / tiles);
  q.go_raw_bytes = kTM * kKB * 4;
  q.x_raw_bytes = (uint32_t)((kNB * q.RXW * 4 + 127) / 128 * 128);
  q.go_op_bytes = (kKB / 4) * kGoSlab;
  q.x_op_bytes = (kKB / 4) * x_slab(nky);
  const size_t fixed = kHeaderBytes + (size_t)kOpStages * (2 * q.go_op_bytes + 2 * (size_t)q.x_op_bytes);
  q.raw_stages = kRawStages;
  while (q.raw_stages > 3 && fixed + (size_t)q.raw_stages * (q.go_raw_bytes + q.x_raw_bytes) > 227 * 1024) --q.raw_stages;
  plan.smem = fixed + (size_t)q.raw_stages * (q.go_raw_bytes + q.x_raw_bytes);
  plan.smem = std::max<size_t>(plan.smem, 116 * 1024);  // one block per SM: it owns all 512 TMEM columns
  if (plan.smem > 227 * 1024) return false;
  // sum of Z[kx] <= target + 2 nkx whatever the rounding does
  plan.max_slices = q.target_slices + 2 * p.nkx;
  plan.blocks = plan.max_slices * tiles;
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

bool make_map(CUtensorMap *map, const float *base, int inner, int rows, int chans, int batch, int box_inner,
              int box_chans) {
  EncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)chans, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)inner * 4, (cuuint64_t)inner * rows * 4, (cuuint64_t)inner * rows * chans * 4};
  const cuuint32_t box[4] = {(cuuint32_t)box_inner, 1u, (cuuint32_t)box_chans, 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

size_t gradw_tc_workspace_floats(const GradWProblem<float> &p, size_t *bias_offset) {
  GwPlan plan;
  const int nky = std::min(p.nky, kMaxTaps);  // more taps run as several launches over the same scratch
  if (!plan_tc_gradw(p, 0, nky, plan)) return 0;
  size_t w_part = (size_t)plan.max_slices * nky * p.B * p.A;
  w_part = (w_part + 63) / 64 * 64;
  if (bias_offset) *bias_offset = w_part;
  return w_part + (size_t)plan.max_slices * p.A;
}

// Partial sums, then their reduction into p.gw (and p.gb when part_b is given).
// More than three linear taps run as one launch pair per three taps.
// MELLIN_ERR_UNSUPPORTED when the problem is outside this kernel's coverage.
int launch_gradw_tc(const GradWProblem<float> &p, float *part_w, float *part_b, cudaStream_t stream) {
  if (p.table.row_ptr == nullptr) return MELLIN_ERR_UNSUPPORTED;
  {
    // every slice must be plannable before the first one is launched
    GwPlan probe;
    for (int g0 = 0; g0 < p.nky; g0 += kMaxTaps)
      if (!plan_tc_gradw(p, g0, std::min(kMaxTaps, p.nky - g0), probe)) return MELLIN_ERR_UNSUPPORTED;
  }
#ifdef MELLIN_TUNING_HOOKS
  const char *prof = getenv("MELLIN_TC_PROFILE");
#else
  const char *prof = nullptr;
#endif
  for (int g0 = 0; g0 < p.nky; g0 += kMaxTaps) {
    const int nky = std::min(kMaxTaps, p.nky - g0);
    GwPlan plan;
    plan_tc_gradw(p, g0, nky, plan);
    CUtensorMap go_map, x_map;
    if (!make_map(&go_map, p.go, p.noy, p.nox, p.A, p.N, kKB, kTM) ||
        !make_map(&x_map, p.in, p.niy, p.nix, p.B, p.N, plan.params.RXW, kNB))
      return g0 == 0 ? MELLIN_ERR_UNSUPPORTED : fail(MELLIN_ERR_LAUNCH, "tc_gradw: tensor map encoding failed");
    plan.params.part_w = part_w;
    plan.params.profile = (prof != nullptr && prof[0] == '1') ? 1 : 0;
    plan.params.part_b = g0 == 0 ? part_b : nullptr;  // the bias gradient rides on the first launch
    auto kernel = nky == 1 ? tc_gradw_kernel<1> : nky == 2 ? tc_gradw_kernel<2> : tc_gradw_kernel<3>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
    if (err != cudaSuccess)
      return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
    kernel<<<plan.blocks, kThreads, plan.smem, stream>>>(plan.params, go_map, x_map);
    err = cudaGetLastError();
    if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("tc_gradw_kernel: ") + cudaGetErrorString(err));
    count_launch();
    // one block per 32 partial-sum addresses of this slice's (kx, slot, b, a) space
    const long long w_blocks = ((long long)p.A * p.B * p.nkx * nky + 31) / 32;
    const long long b_blocks = plan.params.part_b != nullptr ? (p.A + 31) / 32 : 0;
    tc_gradw_reduce_kernel<<<(unsigned)(w_blocks + b_blocks), 256, 0, stream>>>(plan.params, p.gw, p.gb, w_blocks);
    err = cudaGetLastError();
    if (err != cudaSuccess)
      return fail(MELLIN_ERR_LAUNCH, std::string("tc_gradw_reduce_kernel: ") + cudaGetErrorString(err));
    count_launch();
  }
  return MELLIN_OK;
}

int tc_gradw_read_prof(long long *out) {
  return cudaMemcpyFromSymbol(out, g_gw_prof, 16 * sizeof(long long)) == cudaSuccess ? 0 : 2;
}

int tc_gradw_take_error(int *code) {
  int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(code, g_gw_error, sizeof(int));
  if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_gw_error, &zero, sizeof(int));
  return err == cudaSuccess ? MELLIN_OK : MELLIN_ERR_LAUNCH;
}

}  // namespace mellin
