// Measurement helper, not on any product path: a register-resident chain of FP32 fused multiply-adds, used by the
// benchmark to measure the FP32-FMA rate of the device (the roofline denominator of the fp32 kernels, which run on
// the FMA pipe).  Every thread keeps 16 independent accumulators and performs `iters` rounds of 16 FMAs on them,
// either as scalar fma.rn.f32 or as packed fma.rn.f32x2; the result is stored only so that the chain stays live.
#include "kernels.cuh"

namespace elsa {
namespace {

template <bool PACKED>
__global__ void __launch_bounds__(256) fma_rate_kernel(float* __restrict__ sink, long long iters, float a, float b) {
  float2 acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = make_float2(threadIdx.x * 1e-3f + i, blockIdx.x * 1e-3f - i);
  const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
  for (long long it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (PACKED) {
        acc[i] = __ffma2_rn(acc[i], a2, b2);
      } else {
        acc[i].x = fmaf(acc[i].x, a, b);
        acc[i].y = fmaf(acc[i].y, a, b);
      }
    }
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += acc[i].x + acc[i].y;
  if (s == 123.456f) sink[0] = s;   // practically never true: keeps the chain from being optimised away
}

}  // namespace
}  // namespace elsa

// Launches `blocks` CTAs of 256 threads; the work is blocks * 256 * iters * 16 FMAs = twice that many FLOPs.
extern "C" int elsa_debug_fma_rate(float* sink, int blocks, int64_t iters, int packed, void* stream) {
  using namespace elsa;
  if (!sink || blocks < 1 || iters < 1) return ELSA_ERR_INVALID_ARGUMENT;
  auto st = static_cast<cudaStream_t>(stream);
  if (packed) fma_rate_kernel<true><<<blocks, 256, 0, st>>>(sink, iters, 0.999f, 1e-3f);
  else fma_rate_kernel<false><<<blocks, 256, 0, st>>>(sink, iters, 0.999f, 1e-3f);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}
