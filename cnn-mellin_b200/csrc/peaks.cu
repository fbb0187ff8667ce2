// Measurement aid: an FMA-bound micro-kernel whose rate is the FP32 CUDA-core
// ceiling that the CUDA-core kernels of this library are judged against.  Every
// thread runs 16 independent chains of packed FP32 multiply-adds (two per
// instruction on sm_100) with no memory traffic in the loop.
#include <string>

#include "../../include/mellin_b200.h"
#include "mellin_internal.h"

namespace mellin {
namespace {

constexpr int kChains = 16;
constexpr int kUnroll = 8;

__global__ void __launch_bounds__(256) fma_rate_kernel(float *__restrict__ out, int iters) {
  float2 acc[kChains];
#pragma unroll
  for (int i = 0; i < kChains; ++i) acc[i] = make_float2(threadIdx.x + i, blockIdx.x - i);
  const float2 a = make_float2(1.0001f, 0.9999f), b = make_float2(1e-6f, -1e-6f);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int i = 0; i < kChains; ++i) acc[i] = __ffma2_rn(acc[i], a, b);
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kChains; ++i) s += acc[i].x + acc[i].y;
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

}  // namespace
}  // namespace mellin

extern "C" int64_t mellin_selftest_fma_rate(float *out, int64_t blocks, int64_t iters, void *stream) {
  using namespace mellin;
  if (out == nullptr || blocks < 1 || iters < 1 || blocks > (1 << 20) || iters > (1 << 24)) {
    fail(MELLIN_ERR_BAD_ARGUMENT, "selftest_fma_rate: out must hold blocks * 256 floats; 1 <= blocks <= 2^20, 1 <= iters <= 2^24");
    return -1;
  }
  fma_rate_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, (int)iters);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    fail(MELLIN_ERR_LAUNCH, std::string("fma_rate_kernel: ") + cudaGetErrorString(err));
    return -1;
  }
  count_launch();
  return blocks * 256 * iters * kUnroll * kChains * 2;  // multiply-adds performed
}
