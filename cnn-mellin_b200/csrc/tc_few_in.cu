// Forward of a layer with FEW INPUT channels (at most 4) and many output channels on
// tensor cores (tcgen05, sm_100a) -- the first layer of a model (3 feature maps in, 64..256 out):
//
//   out[n, a, ox, oy] = bias[a] + sum_{(kx, ix) in row ox} sum_b sum_ky
//                       W[a, b, kx, ky] * in[n, b, ix, oy + By * ky + Cy]
//
// The reduction is short (entries x channels x taps: 9..72 terms) and the output is the
// big tensor, so the kernel is organised around writing it once, well:
//
//   item  = (n, output row ox, 128 positions, 64 output channels)
//   GEMM  : D[position, a] = sum_k A[position, k] * B[a, k],  k = (entry, b, tap)
//           M = 128 positions (TMEM lanes), N = 64 channels, K = entries x B x taps (<= 96)
//   A     : lives in TENSOR MEMORY.  The input rows of the item's entries arrive by 4-D TMA boxes
//           (4 channels x 136 positions each, zero-filled outside the signal); converter warps
//           write, for every position, the K values it multiplies -- the taps are folded into K
//           here, as three reads one position apart -- split into TF32 hi / lo parts (tcgen05.st)
//   B     : the weights of row ox's entries in operand layout, hi / lo, prepared once per launch
//           by a small kernel, fetched per item with one bulk copy
//   MMAs  : 3 (lo*hi, hi*lo, hi*hi) per 8 terms of K, issued by one elected lane of a converged warp
//   bias  : one more term of K -- A holds the constant 1 there, B the bias -- so the epilogue adds nothing
//   fused : the models' length mask, ReLU and dropout (a hash of the element's offset) are applied on the way out;
//           tiles that start past their utterance's length are not computed at all (zeros are stored)
//   out   : the epilogue warps move the accumulator tile from TMEM to shared memory as
//           [channel][position] and ONE TMA store writes the 64 x 128 box (clipped at the tensor's
//           edges); two staging tiles, so a store runs under the next item's work
//
// 15 warps: 4 epilogue, 8 converter, 1 MMA issuer, 2 copy issuers; persistent blocks take items
// round-robin.  Every wait is bounded and reports through a device word.
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
constexpr int kCopyBWarp = kCopyWarp + 1;  // B operands
constexpr int kThreads = (kCopyBWarp + 1) * 32;
constexpr int kTM = 128;           // output positions per item
constexpr int kNP = 64;            // output channels per item
constexpr int kRawRow = 136;       // staged positions per row: 128 + lead (<= 3) + taps - 1 (<= 2), rounded to 16 bytes
constexpr int kBoxChannels = 4;
constexpr int kMaxEntries = 8;     // per output row: a raw stage holds that many boxes
constexpr int kMaxK = 96;          // entries x B x taps
constexpr int kMaxTable = 640;     // table entries kept in shared memory
constexpr int kMaxRows = 256;      // output rows (their offsets are kept in shared memory)
constexpr int kMaxA = 256;
constexpr uint32_t kRawEntryBytes = kBoxChannels * kRawRow * 4;  // 2176 = 17 x 128
constexpr uint32_t kRawBytes = kMaxEntries * kRawEntryBytes;
constexpr int kMaxRawStages = 4;
constexpr int kOpStages = 2;       // operand A sets in tensor memory
constexpr int kBStages = 2;
constexpr uint32_t kOutBytes = kNP * kTM * 4;  // one staging tile: 32 KB
constexpr uint32_t kACol0 = 2 * kNP;           // TMEM: two accumulator tiles, then the operand A ring
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr int kHeaderBytes = 8192;

struct Control {
  uint64_t raw_full[kMaxRawStages], raw_empty[kMaxRawStages], a_full[kOpStages], a_empty[kOpStages];
  uint64_t b_full[kBStages], b_empty[kBStages], acc_full[2], acc_empty[2], out_free[2], out_full[2];
  uint32_t tmem_base;
  int abort;
  int rp[kMaxRows + 1];   // the table's row offsets
  int2 ent[kMaxTable];    // its entries (kx, ix)
};
static_assert(sizeof(Control) <= kHeaderBytes, "Control must fit the header");

// First bounded wait that gave up since the last query (0 = none): 1 converters, 2 MMA issuer (operands),
// 3 MMA issuer (accumulator tile), 4 epilogue, 5 copy issuer (boxes), 6 copy issuer (B operands).
__device__ int g_tc_few_in_error = 0;

#ifdef MELLIN_TUNING_HOOKS
// per-role wait / work cycles of block 0: 0 epilogue, 1 converter, 2 MMA issuer, 3 copy issuer
__device__ long long g_fi_prof[16];
#define PROF_BEGIN() long long prof_t0 = clock64(), prof_wait = 0, prof_t1 = 0
#define PROF_WAIT_START() prof_t1 = clock64()
#define PROF_WAIT_END() prof_wait += clock64() - prof_t1
#define PROF_END(slot)                                           \
  if (blockIdx.x == 0 && lane == 0) {                            \
    g_fi_prof[2 * (slot)] = prof_wait;                           \
    g_fi_prof[2 * (slot) + 1] = clock64() - prof_t0 - prof_wait; \
  }
#else
#define PROF_BEGIN()
#define PROF_WAIT_START()
#define PROF_WAIT_END()
#define PROF_END(slot)
#endif

struct FiParams {
  const int32_t *row_ptr;  // rows = ox, entries (kx, ix)
  const int2 *entries;
  const float *w;
  const float *bias;
  float *b_pack;           // [ox][channel tile][hi | lo][4-term chunk][64 channels][4]
  long long w_sa, w_sb;
  int N, A, B, nkx, nky, nox, noy, By;
  int BK;                  // B * nky: terms per entry
  int y_tiles, a_tiles;
  int lead, ws0;           // box start = tile start + ws0 - lead (a multiple of 4); tap k of position m reads staged m + k + lead
  int k8_max, k16_max;     // longest reduction of the launch, rounded to 8 / 16
  int raw_stages;
  // fused epilogue: out = (oy < lens[n] * len_scale + len_offset) ? dropout(act(value)) : 0; tiles wholly past the
  // bound are not computed at all
  const int *lens;
  int len_scale, len_offset, relu;
  unsigned drop_threshold, drop_seed;
  float drop_scale;
  long long out_sn, out_sa;  // element strides of out (the dropout mask is a hash of the element's offset)
  int total;               // items
  int num_entries;
  uint32_t b_stage_bytes;  // 512 * k8_max
};

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ void raise_timeout(Control *ctl, int code) {
  atomicCAS(&g_tc_few_in_error, 0, code);
  ctl->abort = 1;
}
// first position of utterance n that the length mask zeroes (no mask: past every tile)
template <bool FUSED>
__device__ __forceinline__ int mask_bound(const FiParams &p, int n) {
  return (FUSED && p.lens != nullptr) ? p.lens[n] * p.len_scale + p.len_offset : 0x7fffffff;
}

// Items (n, y tile, channel tile, ox) in round-robin order over the blocks, rows varying fastest; advanced
// without divisions.
struct ItemIter {
  int id, ox, at, yt, n;
  int step_ox, step_at, step_yt, step_n;
  __device__ __forceinline__ static void digits(const FiParams &p, int t, int &o, int &a, int &y, int &nn) {
    o = t % p.nox, t /= p.nox;
    a = t % p.a_tiles, t /= p.a_tiles;
    y = t % p.y_tiles;
    nn = t / p.y_tiles;
  }
  __device__ __forceinline__ ItemIter(const FiParams &p) {
    id = blockIdx.x;
    digits(p, id, ox, at, yt, n);
    digits(p, (int)gridDim.x, step_ox, step_at, step_yt, step_n);
  }
  __device__ __forceinline__ void next(const FiParams &p) {
    id += gridDim.x;
    ox += step_ox, at += step_at, yt += step_yt, n += step_n;
    if (ox >= p.nox) ox -= p.nox, ++at;
    if (at >= p.a_tiles) at -= p.a_tiles, ++yt;
    if (yt >= p.y_tiles) yt -= p.y_tiles, ++n;
  }
};

// The B operand of every (output row, channel tile): row a of the tile, term (entry, b, tap) holds
// W[a, b, kx(entry), ky(tap)] (taps in increasing input offset), split into TF32 hi / lo parts, in the
// K-major operand layout (4-term chunks of 64 rows x 16 bytes); unused terms and channels are zero.
__global__ void __launch_bounds__(256) pack_few_in_b_kernel(const FiParams p) {
  tc::launch_dependents();  // the main kernel may set itself up meanwhile; it waits for this grid before reading
  const int ox = blockIdx.y / p.a_tiles, at = blockIdx.y % p.a_tiles;
  const int e0 = p.row_ptr[ox];
  const int K = (p.row_ptr[ox + 1] - e0) * p.BK;  // then one more term: the bias (A holds a 1 there)
  const int k8 = (K + 1 + 7) & ~7;
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= 2 * k8 * kNP) return;
  const int part = j / (k8 * kNP), r1 = j % (k8 * kNP);
  const int c = r1 / (4 * kNP), r2 = r1 % (4 * kNP);
  const int row = r2 >> 2, k = 4 * c + (r2 & 3);
  const int a = at * kNP + row;
  float v = 0.f;
  if (k <= K && a < p.A) {
    float w;
    if (k < K) {
      const int e = k / p.BK, r = k % p.BK;
      const int b = r / p.nky, t = r % p.nky;
      const int ky = p.By < 0 ? p.nky - 1 - t : t;
      const int kx = p.entries[e0 + e].x;
      w = p.w[a * p.w_sa + b * p.w_sb + (long long)kx * p.nky + ky];
    } else {
      w = p.bias != nullptr ? p.bias[a] : 0.f;
    }
    const float hi = tf32_hi(w);
    v = part ? w - hi : hi;
  }
  p.b_pack[(size_t)blockIdx.y * 2 * p.k8_max * kNP + j] = v;
}

// Terms 16 (2 u + HALF) .. + 15 of one position, u = 0, 1, ...: term k = (entry, channel, tap) reads the staged
// value (entry, channel, position + tap); term `ne * BK` (the one after the last entry's) is the constant 1 that
// multiplies the bias row of B; the terms after it are zero.  Every index is a compile-time constant, so a
// value costs one shared-memory load with an immediate offset.
template <int NB, int NKY, int HALF>
__device__ __forceinline__ void convert_chunks(const float *raw, int ne, uint32_t col0, uint32_t lo_offset) {
  constexpr int BK = NB * NKY;
#pragma unroll
  for (int u = 0; u < (kMaxK / 16 + 1) / 2; ++u) {
    const int cc = 2 * u + HALF;
    if (16 * cc <= ne * BK) {  // warp-uniform: the chunk holds a term (the last one is term ne * BK)
      uint32_t hi[16], lo[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int k = 16 * cc + i;
        const int e = k / BK, rr = k % BK;
        const int b = rr / NKY, t = rr % NKY;
        float v = 0.f;
        if (e < ne) v = raw[(e * kBoxChannels + b) * kRawRow + t];
        else if (rr == 0 && e == ne) v = 1.f;
        const float h = tf32_hi(v);
        hi[i] = __float_as_uint(h), lo[i] = __float_as_uint(v - h);
      }
      tc::tmem_st16(col0 + (uint32_t)(16 * cc), hi);
      tc::tmem_st16(col0 + lo_offset + (uint32_t)(16 * cc), lo);
    }
  }
}

template <int NB, int NKY, bool FUSED>
__global__ void __launch_bounds__(kThreads, 1)
tc_few_in_kernel(const FiParams p, const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map) {
  constexpr int BK = NB * NKY;
  extern __shared__ __align__(1024) unsigned char smem[];
  Control *ctl = reinterpret_cast<Control *>(smem);
  unsigned char *raw_base = smem + kHeaderBytes;
  unsigned char *b_base = raw_base + (size_t)p.raw_stages * kRawBytes;
  unsigned char *out_base = b_base + (size_t)kBStages * p.b_stage_bytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int i = tid; i <= p.nox; i += kThreads) ctl->rp[i] = p.row_ptr[i];
  for (int i = tid; i < p.num_entries; i += kThreads) ctl->ent[i] = p.entries[i];
  if (tid == 0) {
    for (int s = 0; s < kMaxRawStages; ++s) {
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
      tc::mbar_init(&ctl->out_free[s], 1);
      tc::mbar_init(&ctl->out_full[s], kEpilogueWarps * 32);
    }
    ctl->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tc::tmem_alloc(&ctl->tmem_base, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::grid_dependency_wait();  // the weight operands come from the kernel before
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const int *rp = ctl->rp;
  const uint32_t a_stage_cols = 2u * (uint32_t)p.k16_max;  // hi then lo

  if (warp < kEpilogueWarps) {
    // ===================== epilogue: TMEM -> [channel][position] staging tile -> one TMA store =====================
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int m = warp * 32 + lane;
    const float floor_ = p.relu ? 0.f : -3.0e38f;
    int j = 0, jt = 0;  // items; items that were computed (the others lie past their utterance's length: zeros)
    PROF_BEGIN();
    for (ItemIter it(p); it.id < p.total; it.next(p)) {
      const int buf = j & 1, acc = jt & 1;
      const uint32_t par = (uint32_t)((j >> 1) & 1);
      const int bound = mask_bound<FUSED>(p, it.n);
      const bool dead = it.yt * kTM >= bound;
      if (tid == 0) {
        tc::bulk_wait_group_read<1>();  // the store that read this staging tile two items ago has finished reading
        tc::mbar_arrive(&ctl->out_free[buf]);
      }
      PROF_WAIT_START();
      bool ok = tc::mbar_wait(&ctl->out_free[buf], par, kSpinLimit);
      if (!dead) ok = ok && tc::mbar_wait(&ctl->acc_full[acc], (uint32_t)((jt >> 1) & 1), kSpinLimit);
      PROF_WAIT_END();
      if (!__all_sync(0xffffffffu, ok)) {
        raise_timeout(ctl, 4);
        break;
      }
      float *stage = reinterpret_cast<float *>(out_base + (size_t)buf * kOutBytes) + m;
      if (dead) {
#pragma unroll
        for (int c = 0; c < kNP; ++c) stage[c * kTM] = 0.f;
      } else {
        tc::tc_fence_after_sync();
        uint32_t v[kNP / 16][16];
#pragma unroll
        for (int g = 0; g < kNP / 16; ++g) tc::tmem_ld16(tmem_base + lane_base + (uint32_t)(acc * kNP + 16 * g), v[g]);
        tc::tmem_ld_wait();
        // the tile is in registers: the MMAs of the item after next may overwrite it
        tc::tc_fence_before_sync();
        tc::mbar_arrive(&ctl->acc_empty[acc]);
        if (!FUSED) {
#pragma unroll
          for (int g = 0; g < kNP / 16; ++g)
#pragma unroll
            for (int i = 0; i < 16; ++i) stage[(16 * g + i) * kTM] = __uint_as_float(v[g][i]);
        } else {
          const int oy = it.yt * kTM + m;
          const float keep = oy < bound ? 1.f : 0.f;
          const unsigned long long off0 = (unsigned long long)(it.n * p.out_sn + (long long)(it.at * kNP) * p.out_sa +
                                                               (long long)it.ox * p.noy + oy);
#pragma unroll
          for (int g = 0; g < kNP / 16; ++g)
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float scale = (p.drop_threshold != 0u &&
                                   dropout_hash(p.drop_seed, off0 + (unsigned long long)((16 * g + i) * p.out_sa)) < p.drop_threshold)
                                      ? 0.f
                                      : p.drop_scale;
              stage[(16 * g + i) * kTM] = fmaxf(__uint_as_float(v[g][i]), floor_) * keep * scale;
            }
        }
      }
      tc::fence_proxy_async();  // the staging tile was written through the generic proxy; the store reads it through the async one
      tc::mbar_arrive(&ctl->out_full[buf]);
      if (tid == 0) {
        if (!tc::mbar_wait(&ctl->out_full[buf], par, kSpinLimit)) {
          raise_timeout(ctl, 4);
        } else {
          tc::tma_store_4d(&out_map, out_base + (size_t)buf * kOutBytes, it.yt * kTM, it.ox, it.n, it.at * kNP);
          tc::bulk_commit_group();
        }
      }
      __syncwarp();
      ++j;
      jt += dead ? 0 : 1;
    }
    if (warp == 1) { PROF_END(0); }
    if (tid == 0) tc::bulk_wait_group_all();
  } else if (warp < kMmaWarp) {
    // ===================== converters: staged rows -> the K terms of every position, hi / lo, in TMEM =====================
    const int cw = warp - kEpilogueWarps;
    const int quad = cw & 3;  // TMEM lane quadrant (= warp index mod 4); warps 0-3 take the even 16-term chunks, 4-7 the odd ones
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const int m = quad * 32 + lane;
    int st = 0;
    bool failed = false;
    PROF_BEGIN();
    for (ItemIter it(p); it.id < p.total && !failed; it.next(p)) {
      if (it.yt * kTM >= mask_bound<FUSED>(p, it.n)) continue;  // past the utterance's length: the epilogue writes zeros
      const int ne = rp[it.ox + 1] - rp[it.ox];
      const int r = st % p.raw_stages, s = st % kOpStages;
      PROF_WAIT_START();
      const bool ok = tc::mbar_wait(&ctl->raw_full[r], (uint32_t)((st / p.raw_stages) & 1), kSpinLimit) &&
                      tc::mbar_wait(&ctl->a_empty[s], (uint32_t)(((st / kOpStages) & 1) ^ 1), kSpinLimit);
      PROF_WAIT_END();
      if (!__all_sync(0xffffffffu, ok)) {
        raise_timeout(ctl, 1);
        failed = true;
        break;
      }
      tc::tc_fence_after_sync();
      const float *raw = reinterpret_cast<const float *>(raw_base + (size_t)r * kRawBytes) + m + p.lead;
      const uint32_t col0 = tmem_base + lane_base + kACol0 + (uint32_t)s * a_stage_cols;
      if (cw < 4)
        convert_chunks<NB, NKY, 0>(raw, ne, col0, (uint32_t)p.k16_max);
      else
        convert_chunks<NB, NKY, 1>(raw, ne, col0, (uint32_t)p.k16_max);
      tc::tmem_st_wait();
      tc::tc_fence_before_sync();
      // the proxy fence orders this thread's reads of the raw slot before the copy engine's next write into it
      tc::fence_proxy_async();
      tc::mbar_arrive(&ctl->raw_empty[r]);
      tc::mbar_arrive(&ctl->a_full[s]);
      ++st;
    }
    if (warp == kEpilogueWarps) { PROF_END(1); }
  } else if (warp == kCopyWarp) {
    // ===================== copy issuer: one box of `in` per table entry =====================
    if (lane == 0) {
      int st = 0;
      bool failed = false;
      PROF_BEGIN();
      for (ItemIter it(p); it.id < p.total && !failed; it.next(p)) {
        if (it.yt * kTM >= mask_bound<FUSED>(p, it.n)) continue;
        const int e0 = rp[it.ox], ne = rp[it.ox + 1] - e0;
        const int r = st % p.raw_stages;
        PROF_WAIT_START();
        const bool empty_ok = tc::mbar_wait(&ctl->raw_empty[r], (uint32_t)(((st / p.raw_stages) & 1) ^ 1), kSpinLimit);
        PROF_WAIT_END();
        if (!empty_ok) {
          raise_timeout(ctl, 5);
          failed = true;
          break;
        }
        const int start = it.yt * kTM + p.ws0 - p.lead;  // a multiple of 4
        unsigned char *dst = raw_base + (size_t)r * kRawBytes;
        tc::mbar_arrive_expect_tx(&ctl->raw_full[r], (uint32_t)ne * kRawEntryBytes);
        for (int e = 0; e < ne; ++e)
          tc::tma_load_4d(dst + (size_t)e * kRawEntryBytes, &in_map, start, ctl->ent[e0 + e].y, it.n, 0, &ctl->raw_full[r]);
        ++st;
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
        if (it.yt * kTM >= mask_bound<FUSED>(p, it.n)) continue;
        const int K = (rp[it.ox + 1] - rp[it.ox]) * BK + 1;  // + the bias term
        const int s = st % kBStages;
        if (!tc::mbar_wait(&ctl->b_empty[s], (uint32_t)(((st / kBStages) & 1) ^ 1), kSpinLimit)) {
          raise_timeout(ctl, 6);
          failed = true;
          break;
        }
        const uint32_t bytes = 512u * (uint32_t)((K + 7) & ~7);
        tc::mbar_arrive_expect_tx(&ctl->b_full[s], bytes);
        tc::bulk_load(b_base + (size_t)s * p.b_stage_bytes,
                      p.b_pack + ((size_t)it.ox * p.a_tiles + it.at) * 2 * p.k8_max * kNP, bytes, &ctl->b_full[s]);
        ++st;
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer =====================
    // The whole warp walks the items; one elected lane issues.  Everything an MMA names is computed from
    // warp-uniform values (what comes from shared memory is broadcast from lane 0 to say so).
    const uint32_t tmem0 = tc::uniform(tmem_base);
    const uint32_t b0 = tc::smem_u32(b_base) >> 4;
    // B descriptors: 4-term chunks of 64 rows x 16 bytes (pitch 64 units of 16 bytes), 8-row groups 128 bytes apart
    const uint64_t desc_fixed = tc::smem_desc(0u, (uint32_t)kNP * 16u, 128u);
    const uint32_t idesc = tc::idesc_tf32(kTM, kNP);
    int st = 0;
    bool failed = false;
    PROF_BEGIN();
    for (ItemIter it(p); it.id < p.total && !failed; it.next(p)) {
      if ((int)tc::uniform((uint32_t)(it.yt * kTM >= mask_bound<FUSED>(p, it.n)))) continue;
      const int K = (int)tc::uniform((uint32_t)(rp[it.ox + 1] - rp[it.ox])) * BK + 1;  // + the bias term
      const int ksteps = (K + 7) >> 3;
      const int buf = st & 1, s = st % kOpStages, sb = st % kBStages;
      PROF_WAIT_START();
      const bool ok = tc::mbar_wait(&ctl->acc_empty[buf], (uint32_t)(((st >> 1) & 1) ^ 1), kSpinLimit) &&
                      tc::mbar_wait(&ctl->a_full[s], (uint32_t)((st / kOpStages) & 1), kSpinLimit) &&
                      tc::mbar_wait(&ctl->b_full[sb], (uint32_t)((st / kBStages) & 1), kSpinLimit);
      PROF_WAIT_END();
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) raise_timeout(ctl, 2);
        failed = true;
        break;
      }
      tc::tc_fence_after_sync();
      const uint32_t d0 = tmem0 + (uint32_t)(buf * kNP);
      const uint32_t a_hi = tmem0 + kACol0 + (uint32_t)s * a_stage_cols, a_lo = a_hi + (uint32_t)p.k16_max;
      const uint32_t b_hi = b0 + (uint32_t)sb * (p.b_stage_bytes >> 4), b_lo = b_hi + (uint32_t)(2 * ksteps * kNP);
      if (tc::elect_one()) {
        uint32_t fresh = 0;  // 0: the next MMA overwrites the accumulators
        for (int ks = 0; ks < ksteps; ++ks) {
          const uint32_t bo = (uint32_t)(ks * 2 * kNP);
          const uint64_t db_hi = desc_fixed | (uint64_t)((b_hi + bo) & 0x3FFFu);
          const uint64_t db_lo = desc_fixed | (uint64_t)((b_lo + bo) & 0x3FFFu);
          // the three products of the hi/lo split, smallest first
          tc::mma_tf32_a_tmem(d0, a_lo + 8u * ks, db_hi, idesc, fresh);
          tc::mma_tf32_a_tmem(d0, a_hi + 8u * ks, db_lo, idesc, 1u);
          tc::mma_tf32_a_tmem(d0, a_hi + 8u * ks, db_hi, idesc, 1u);
          fresh = 1u;
        }
        tc::tc_commit(&ctl->a_empty[s]);
        tc::tc_commit(&ctl->b_empty[sb]);
        tc::tc_commit(&ctl->acc_full[buf]);
      }
      __syncwarp();
      ++st;
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

size_t round256(size_t v) { return (v + 255) / 256 * 256; }

struct FiPlan {
  FiParams params;
  size_t smem = 0, b_pack_bytes = 0;
  int blocks = 0;
};

// Needs p.table.num_entries and .max_row (upper bounds will do for a workspace query).
bool plan_tc_few_in(const DirectProblem<float> &p, FiPlan &plan) {
  if (p.Dy != 1 || p.Ay != 1 || p.accumulate) return false;
  if (p.B < 1 || p.B > kBoxChannels || p.A < 16 || p.A > kMaxA || p.nky < 1 || p.nky > 3) return false;
  if (p.nky > 1 && p.By != 1 && p.By != -1) return false;
  if (p.nkx < 1 || p.noy < 64 || p.nox < 1 || p.nox > kMaxRows || p.N < 1 || p.nix < 1) return false;
  if (p.table.max_row < 1 || p.table.max_row > kMaxEntries || p.table.num_entries > kMaxTable) return false;
  const int BK = p.B * p.nky;
  if (BK * p.table.max_row + 1 > kMaxK) return false;  // + the bias term
  // rows are copied in 16-byte chunks, the output is stored in 16-byte chunks
  if (p.niy % 4 != 0 || reinterpret_cast<uintptr_t>(p.in) % 16 != 0 || p.in_sn % 4 != 0 || p.in_sb % 4 != 0) return false;
  if (p.noy % 4 != 0 || reinterpret_cast<uintptr_t>(p.out) % 16 != 0 || p.out_sn % 4 != 0 || p.out_sa % 4 != 0) return false;
  FiParams &q = plan.params;
  q.row_ptr = p.table.row_ptr, q.entries = p.table.entries;
  q.w = p.w, q.bias = p.bias;
  q.w_sa = p.w_sa, q.w_sb = p.w_sb;
  q.N = p.N, q.A = p.A, q.B = p.B, q.nkx = p.nkx, q.nky = p.nky, q.nox = p.nox, q.noy = p.noy, q.By = p.By;
  q.BK = BK;
  q.y_tiles = (p.noy + kTM - 1) / kTM;
  q.a_tiles = (p.A + kNP - 1) / kNP;
  q.ws0 = p.Cy + std::min(0, p.By * (p.nky - 1));
  q.lead = ((q.ws0 % 4) + 4) % 4;
  const int kmax = BK * p.table.max_row + 1;
  q.k8_max = (kmax + 7) / 8 * 8, q.k16_max = (kmax + 15) / 16 * 16;
  if (kACol0 + kOpStages * 2 * q.k16_max > (int)kTmemCols) return false;
  const long long total = (long long)p.N * p.nox * q.y_tiles * q.a_tiles;
  if (total >= (1LL << 30)) return false;
  q.total = (int)total;
  q.num_entries = (int)p.table.num_entries;
  q.lens = p.lens, q.len_scale = p.len_scale, q.len_offset = p.len_offset, q.relu = p.relu;
  q.drop_threshold = p.drop_threshold, q.drop_seed = p.drop_seed, q.drop_scale = p.drop_scale;
  q.out_sn = p.out_sn, q.out_sa = p.out_sa;
  q.b_stage_bytes = 512u * (uint32_t)q.k8_max;
  for (q.raw_stages = kMaxRawStages; q.raw_stages >= 2; --q.raw_stages) {
    plan.smem = kHeaderBytes + (size_t)q.raw_stages * kRawBytes + (size_t)kBStages * q.b_stage_bytes + 2 * kOutBytes;
    if (plan.smem <= 227 * 1024) break;
  }
  if (q.raw_stages < 2) return false;
  plan.smem = std::max<size_t>(plan.smem, 116 * 1024);  // one block per SM: it owns all of tensor memory
  plan.b_pack_bytes = round256((size_t)p.nox * q.a_tiles * 2 * q.k8_max * kNP * sizeof(float));
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

// (position, Mellin row, batch, channel) with the tensor's real strides
bool make_map(CUtensorMap *map, const float *base, int inner, int rows, int batch, int chans, long long sn, long long sc,
              int box_inner, int box_chans) {
  EncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batch, (cuuint64_t)chans};
  const cuuint64_t strides[3] = {(cuuint64_t)inner * sizeof(float), (cuuint64_t)sn * sizeof(float),
                                 (cuuint64_t)sc * sizeof(float)};
  const cuuint32_t box[4] = {(cuuint32_t)box_inner, 1u, 1u, (cuuint32_t)box_chans};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NB>
int launch_for_b(const FiPlan &plan, const CUtensorMap &in_map, const CUtensorMap &out_map, cudaStream_t stream) {
  const FiParams &q = plan.params;
  const bool fused = q.lens != nullptr || q.relu || q.drop_threshold != 0u;
  auto kernel = fused ? (q.nky == 1   ? tc_few_in_kernel<NB, 1, true>
                         : q.nky == 2 ? tc_few_in_kernel<NB, 2, true>
                                      : tc_few_in_kernel<NB, 3, true>)
                      : (q.nky == 1   ? tc_few_in_kernel<NB, 1, false>
                         : q.nky == 2 ? tc_few_in_kernel<NB, 2, false>
                                      : tc_few_in_kernel<NB, 3, false>);
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  err = launch_after_predecessor(kernel, dim3(plan.blocks), dim3(kThreads), plan.smem, stream, q, in_map, out_map);
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("tc_few_in_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

}  // namespace

// Reads and clears this kernel's timeout flag of the current device (synchronises it).
int tc_few_in_take_error(int *code) {
  int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(code, g_tc_few_in_error, sizeof(int));
  if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_tc_few_in_error, &zero, sizeof(int));
  return err == cudaSuccess ? MELLIN_OK : fail(MELLIN_ERR_LAUNCH, std::string("device status: ") + cudaGetErrorString(err));
}

#ifdef MELLIN_TUNING_HOOKS
extern "C" int mellin_tc_few_in_profile(long long *out) {
  return cudaMemcpyFromSymbol(out, g_fi_prof, 16 * sizeof(long long)) == cudaSuccess ? 0 : 2;
}
#endif

// scratch for the B operands (0 = problem not covered by this kernel); needs p.table.num_entries and .max_row
size_t tc_few_in_workspace_bytes(const DirectProblem<float> &p) {
  FiPlan plan;
  if (!plan_tc_few_in(p, plan)) return 0;
  return plan.b_pack_bytes;
}

// MELLIN_ERR_UNSUPPORTED when the problem is outside this kernel's coverage or the workspace too small.
int launch_tc_few_in(const DirectProblem<float> &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  FiPlan plan;
  if (p.table.row_ptr == nullptr || !plan_tc_few_in(p, plan)) return MELLIN_ERR_UNSUPPORTED;
  if (workspace == nullptr || workspace_bytes < plan.b_pack_bytes || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return MELLIN_ERR_UNSUPPORTED;
  CUtensorMap in_map, out_map;
  if (!make_map(&in_map, p.in, p.niy, p.nix, p.N, p.B, p.in_sn, p.in_sb, kRawRow, kBoxChannels) ||
      !make_map(&out_map, p.out, p.noy, p.nox, p.N, p.A, p.out_sn, p.out_sa, kTM, kNP))
    return MELLIN_ERR_UNSUPPORTED;
  FiParams &q = plan.params;
  q.b_pack = static_cast<float *>(workspace);
  pack_few_in_b_kernel<<<dim3((unsigned)((2 * q.k8_max * kNP + 255) / 256), (unsigned)(p.nox * q.a_tiles)), 256, 0, stream>>>(q);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("pack_few_in_b_kernel: ") + cudaGetErrorString(err));
  count_launch();
  switch (p.B) {
    case 1: return launch_for_b<1>(plan, in_map, out_map, stream);
    case 2: return launch_for_b<2>(plan, in_map, out_map, stream);
    case 3: return launch_for_b<3>(plan, in_map, out_map, stream);
    default: return launch_for_b<4>(plan, in_map, out_map, stream);
  }
}

}  // namespace mellin
