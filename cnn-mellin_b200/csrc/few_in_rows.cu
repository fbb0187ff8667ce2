// "Direct" operator for FEW REDUCED CHANNELS (at most 4) and many output
// channels -- the forward pass of a first layer (3 feature maps in, 64..128
// out), which is bound by writing its output to HBM.  This is the CUDA-core
// engine for that layer: the tcgen05 kernel is the default and is faster
// (121 us against 152 us at batch 32, 41 x 800, 3 -> 64 channels); this one runs
// when the tensor cores are switched off or do not cover the problem:
//
//   out[n, a, ox, oy] = init + sum_{(kx, ix) in row ox} sum_b sum_ky
//                       W[a, b, kx, ky] * in[n, b, ix, oy + By * ky + Cy]
//
// Each output needs only ~24 multiply-adds, so the tensor cores have nothing to
// chew on (K is 3 channels x 3 taps x <= 8 rows); what matters is that the FP32
// pipe is starved neither by instruction issue nor by shared-memory bandwidth
// (128 bytes per clock per SM against 128 multiply-adds per clock: every float
// read from shared memory has to feed at least four of them).  A persistent
// block of 8 warps owns 64 output channels and walks tiles (n, ox, 256
// positions) utterance by utterance, heaviest table row first.  The few input
// rows of a tile are staged in shared memory with 16-byte cp.async copies one
// tile ahead; the block's weights stay in shared memory.  A lane keeps
// 8 channels x 8 positions of running sums: a 12-float input window serves
// 8 channels x 3 taps x 4 positions = 96 multiply-adds, a broadcast 16-byte
// weight load serves 4 channels x 8 positions, so FMAs are ~90 % of the issued
// instructions.  The linear taps are register shifts of the window; output
// rows are written with 16-byte stores.
#include <algorithm>
#include <string>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"

namespace mellin {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kCW = 8;                 // output channels per warp
constexpr int kTA = kWarps * kCW;      // output channels per block
constexpr int kTY = 256;               // positions per tile: two windows of 128
constexpr int kRowPitch = kTY + 12;    // floats staged per input row: 256 + taps + lead, padded to 16 bytes
constexpr int kMaxRows = 256;          // table rows / entries kept in shared memory
constexpr int kMaxEntries = 1024;
constexpr int kMaxKx = 8;              // entries of one table row

struct FewInPlan {
  int y_tiles = 0, a_tiles = 0;
  int ws0 = 0;    // first input position a tile reads, relative to its first output position
  int lead = 0;   // (tile start + ws0) mod 4: the window begins `lead` floats into its 16-byte chunk
  int tiles = 0;  // N * nox * y_tiles (per a-tile)
  int grid = 0;
  int w_floats = 0;
  size_t smem = 0;
};

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the destination is zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

struct Tile {
  int n, ox, y0, e0, np;
};

template <int NKY, int LEAD>
__global__ void __launch_bounds__(kThreads, 2)
few_in_rows_kernel(const DirectProblem<float> p, const FewInPlan t) {
  constexpr int kWin = (LEAD + 4 + NKY - 1 + 3) / 4;  // 16-byte chunks holding one 4-position window and its taps
  extern __shared__ __align__(16) float smem[];
  float *Ws = smem;                       // [kx][b][k][kTA]: the block's weights
  float *stage = smem + t.w_floats;       // [2][kMaxKx * B][kRowPitch]
  __shared__ int s_rowptr[kMaxRows + 1], s_order[kMaxRows];
  __shared__ int2 s_entries[kMaxEntries];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int at = blockIdx.x % t.a_tiles;       // this block's channel tile, fixed for its lifetime
  const int a0 = at * kTA;
  const int first = blockIdx.x / t.a_tiles, step = gridDim.x / t.a_tiles;

  for (int i = tid; i <= p.nox; i += kThreads) s_rowptr[i] = p.table.row_ptr[i];
  for (int i = tid; i < p.nox; i += kThreads) s_order[i] = p.table.order[i];
  for (int i = tid; i < (int)p.table.num_entries; i += kThreads) s_entries[i] = p.table.entries[i];
  // weights: Ws[((kx * B + b) * NKY + k) * kTA + a_local], taps in increasing input offset
  for (int i = tid; i < p.nkx * p.B * NKY * kTA; i += kThreads) {
    const int al = i % kTA;
    int r = i / kTA;
    const int k = r % NKY;
    r /= NKY;
    const int b = r % p.B, kx = r / p.B;
    const int ky = p.By < 0 ? NKY - 1 - k : k;
    const int a = a0 + al;
    Ws[i] = a < p.A ? __ldg(p.w + a * p.w_sa + b * p.w_sb + (long long)kx * NKY + ky) : 0.f;
  }
  __syncthreads();

  auto decode = [&](int tile) {
    const int per_n = p.nox * t.y_tiles;
    Tile c;
    c.n = tile / per_n;
    const int rem = tile - c.n * per_n;
    const int rr = rem / t.y_tiles;
    c.ox = s_order[rr];
    c.y0 = (rem - rr * t.y_tiles) * kTY;
    c.e0 = s_rowptr[c.ox];
    c.np = min(s_rowptr[c.ox + 1] - c.e0, kMaxKx);
    return c;
  };
  // stage the input rows of a tile: row (pp, b) holds positions [y0 + ws0 - LEAD, + kRowPitch)
  auto stage_tile = [&](int tile, int buf) {
    if (tile < t.tiles) {
      const Tile c = decode(tile);
      const int x0 = c.y0 + t.ws0 - LEAD;  // a multiple of 4
      const int chunks = kRowPitch / 4;
      const int total = c.np * p.B * chunks;
      float *dst = stage + (size_t)buf * kMaxKx * p.B * kRowPitch;
      for (int i = tid; i < total; i += kThreads) {
        const int ch = i % chunks, rb = i / chunks;
        const int b = rb % p.B, pp = rb / p.B;
        const int ix = s_entries[c.e0 + pp].y;
        const int iy = x0 + 4 * ch;
        const bool valid = iy >= 0 && iy + 3 < p.niy;  // rows are multiples of 4 long: a chunk is inside or outside
        const float *src = p.in + c.n * p.in_sn + b * p.in_sb + (long long)ix * p.niy + iy;
        cp_async16(dst + rb * kRowPitch + 4 * ch, valid ? src : p.in, valid);
      }
    }
    cp_async_commit();
  };

  float bias[kCW];
#pragma unroll
  for (int ch = 0; ch < kCW; ++ch) {
    const int a = a0 + kCW * warp + ch;
    bias[ch] = (!p.accumulate && p.bias != nullptr && a < p.A) ? __ldg(p.bias + a) : 0.f;
  }

  stage_tile(first, 0);
  int it = 0;
  for (int tile = first; tile < t.tiles; tile += step, ++it) {
    cp_async_wait_all();
    __syncthreads();  // this tile's rows have landed; every warp has left the buffer the next copies overwrite
    stage_tile(tile + step, (it + 1) & 1);
    const Tile c = decode(tile);
    int bound = p.noy;  // positions from `bound` on are written as zero (fused length mask)
    if (p.lens != nullptr) bound = min(p.noy, max(0, p.lens[c.n] * p.len_scale + p.len_offset));
    const bool dead = c.y0 >= bound;           // the whole tile lies past the utterance's end
    const bool second = c.y0 + 128 < p.noy;    // the tile's second window exists
    const bool second_live = c.y0 + 128 < bound;

    float acc[kCW][8];  // [channel][position]: window 0 = positions 0..3, window 1 = positions 4..7
#pragma unroll
    for (int ch = 0; ch < kCW; ++ch)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[ch][j] = bias[ch];

    if (!dead) {
      const float *rows = stage + (size_t)(it & 1) * kMaxKx * p.B * kRowPitch + 4 * lane;
      for (int pp = 0; pp < c.np; ++pp) {
        const int kx = s_entries[c.e0 + pp].x;
        for (int b = 0; b < p.B; ++b) {
          const float *row = rows + (pp * p.B + b) * kRowPitch;
          const float4 *wp = reinterpret_cast<const float4 *>(Ws + ((kx * p.B + b) * NKY) * kTA + kCW * warp);
          float xw[2][4 * kWin];
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            if (g == 1 && !second_live) break;  // tile-uniform
#pragma unroll
            for (int i = 0; i < kWin; ++i) {
              const float4 v = *reinterpret_cast<const float4 *>(row + 128 * g + 4 * i);
              xw[g][4 * i] = v.x, xw[g][4 * i + 1] = v.y, xw[g][4 * i + 2] = v.z, xw[g][4 * i + 3] = v.w;
            }
          }
#pragma unroll
          for (int k = 0; k < NKY; ++k) {
            // the eight channels' weights of this tap: two broadcast 16-byte loads
            const float4 wa = wp[k * (kTA / 4)], wb = wp[k * (kTA / 4) + 1];
            const float wv[kCW] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int ch = 0; ch < kCW; ++ch)
#pragma unroll
              for (int j = 0; j < 4; ++j) acc[ch][j] = fmaf(wv[ch], xw[0][LEAD + j + k], acc[ch][j]);
            if (second_live) {
#pragma unroll
              for (int ch = 0; ch < kCW; ++ch)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[ch][4 + j] = fmaf(wv[ch], xw[1][LEAD + j + k], acc[ch][4 + j]);
            }
          }
        }
      }
    }

    // ---- store: channel a0 + 8 * warp + ch, positions y0 + 128 * g + 4 * lane .. + 3 ----
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      if (g == 1 && !second) break;
      const int y = c.y0 + 128 * g + 4 * lane;
      if (y >= p.noy) continue;
#pragma unroll
      for (int ch = 0; ch < kCW; ++ch) {
        const int a = a0 + kCW * warp + ch;
        if (a >= p.A) break;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float val = acc[ch][4 * g + j];
          if (p.relu) val = fmaxf(val, 0.f);
          if (y + j >= bound) val = 0.f;
          v[j] = val;
        }
        float *out = p.out + c.n * p.out_sn + a * p.out_sa + (long long)c.ox * p.noy + y;
        if (p.drop_threshold != 0u) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[j] = dropout_hash(p.drop_seed, (unsigned long long)(out + j - p.out)) < p.drop_threshold ? 0.f : v[j] * p.drop_scale;
        }
        if (p.accumulate) {
          const float4 old = *reinterpret_cast<const float4 *>(out);
          v[0] += old.x, v[1] += old.y, v[2] += old.z, v[3] += old.w;
        }
        *reinterpret_cast<float4 *>(out) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
  }
  cp_async_wait_all();
}

bool plan_few_in(const DirectProblem<float> &p, FewInPlan &t) {
  if (p.Dy != 1 || p.Ay != 1) return false;
  if (p.B < 1 || p.B > 4 || p.A < 8 || p.nky < 1 || p.nky > 3 || p.nkx < 1 || p.nkx > kMaxKx) return false;
  if (p.nky > 1 && p.By != 1 && p.By != -1) return false;
  if (p.noy < 64 || p.noy % 4 != 0 || p.niy % 4 != 0 || p.nox < 1 || p.N < 1) return false;
  if (p.nox > kMaxRows || (long long)p.nox * p.nkx > kMaxEntries) return false;
  // 16-byte copies of the input rows, 16-byte stores of the output rows
  if (reinterpret_cast<uintptr_t>(p.in) % 16 != 0 || p.in_sn % 4 != 0 || p.in_sb % 4 != 0) return false;
  if (reinterpret_cast<uintptr_t>(p.out) % 16 != 0 || p.out_sn % 4 != 0 || p.out_sa % 4 != 0) return false;
  t.ws0 = p.Cy + std::min(0, p.By * (p.nky - 1));
  t.lead = ((t.ws0 % 4) + 4) % 4;
  if (t.lead + 4 + p.nky - 1 > 12) return false;
  t.y_tiles = (p.noy + kTY - 1) / kTY;
  t.a_tiles = (p.A + kTA - 1) / kTA;
  const long long tiles = (long long)p.N * p.nox * t.y_tiles;
  if (tiles >= (1LL << 30)) return false;
  t.tiles = (int)tiles;
  t.w_floats = (p.nkx * p.B * p.nky * kTA + 3) / 4 * 4;
  t.smem = ((size_t)t.w_floats + 2u * kMaxKx * p.B * kRowPitch) * sizeof(float);
  if (t.smem > 72 * 1024) return false;
  const long long want = (long long)sm_count() * 2 / t.a_tiles * t.a_tiles;
  t.grid = (int)std::max<long long>(t.a_tiles, std::min<long long>(want, tiles * t.a_tiles));
  t.grid = t.grid / t.a_tiles * t.a_tiles;
  return true;
}

template <int NKY>
int dispatch_lead(const DirectProblem<float> &p, const FewInPlan &t, cudaStream_t stream) {
  void (*kernel)(DirectProblem<float>, FewInPlan) = nullptr;
  switch (t.lead) {
    case 0: kernel = few_in_rows_kernel<NKY, 0>; break;
    case 1: kernel = few_in_rows_kernel<NKY, 1>; break;
    case 2: kernel = few_in_rows_kernel<NKY, 2>; break;
    default: kernel = few_in_rows_kernel<NKY, 3>; break;
  }
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem);
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(err));
  kernel<<<(unsigned)t.grid, kThreads, t.smem, stream>>>(p, t);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail(MELLIN_ERR_LAUNCH, std::string("few_in_rows_kernel: ") + cudaGetErrorString(err));
  count_launch();
  return MELLIN_OK;
}

}  // namespace

// MELLIN_ERR_UNSUPPORTED when the problem is outside this kernel's coverage.
int launch_few_in_rows(const DirectProblem<float> &p, cudaStream_t stream) {
  FewInPlan t;
  if (!plan_few_in(p, t) || p.table.order == nullptr) return MELLIN_ERR_UNSUPPORTED;
  switch (p.nky) {
    case 1: return dispatch_lead<1>(p, t, stream);
    case 2: return dispatch_lead<2>(p, t, stream);
    default: return dispatch_lead<3>(p, t, stream);
  }
}

}  // namespace mellin
