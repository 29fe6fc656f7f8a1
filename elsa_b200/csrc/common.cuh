// Shared helpers for the elsa_b200 kernels (device-side conversions, the monoid merge,
// launch-error bookkeeping).  No torch headers anywhere in csrc/: the library is plain CUDA.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include <atomic>

#include "../../include/elsa_b200.h"

namespace elsa {

constexpr float kLog2e = 1.4426950408889634f;

// ---- host-side error bookkeeping -------------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return ELSA_ERR_CUDA;
}

#define ELSA_CUDA_CHECK(expr)                          \
  do {                                                 \
    cudaError_t _e = (expr);                           \
    if (_e != cudaSuccess) return ::elsa::cuda_fail(_e); \
  } while (0)

// every kernel launch made by the library passes through ELSA_LAUNCH_CHECK: count them
extern std::atomic<long long> g_kernel_launches;

#define ELSA_LAUNCH_CHECK()                               \
  do {                                                    \
    ::elsa::g_kernel_launches.fetch_add(1, std::memory_order_relaxed); \
    cudaError_t _e = cudaPeekAtLastError();               \
    if (_e != cudaSuccess) {                              \
      (void)cudaGetLastError();                           \
      return ::elsa::cuda_fail(_e);                       \
    }                                                     \
  } while (0)

inline int dtype_size(int dt) { return dt == ELSA_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == ELSA_F32 || dt == ELSA_F16 || dt == ELSA_BF16; }
inline int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t align_up(int64_t a, int64_t b) { return cdiv64(a, b) * b; }

// ---- device-side element conversion -----------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// round-trip through T (the reference's "cast to the input dtype" rounding points)
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_f32<T>(from_f32<T>(x)); }

// Vector of 4 elements of T <-> float[4]; callers guarantee the alignment (4*sizeof(T)).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&o)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&o)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  }
};
template <> struct Vec4<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&o)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    float2 a = __half22float2(*reinterpret_cast<__half2*>(&t.x));
    float2 b = __half22float2(*reinterpret_cast<__half2*>(&t.y));
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
  }
  static __device__ __forceinline__ void store(__half* p, const float (&o)[4]) {
    __half2 a = __floats2half2_rn(o[0], o[1]);
    __half2 b = __floats2half2_rn(o[2], o[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&o)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.x));
    float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.y));
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&o)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(o[2], o[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  }
};

// exp2 with the guarantee exp2(-inf) == 0 (ex2.approx: 2 ulp, flushes denormals)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- the monoid -------------------------------------------------------------------------
// State (m, z, s[NV]); identity (-inf, 0, 0).  merge() folds `b` into the running state `a`:
//   m = max(m_a, m_b); alpha = z_a > 0 ? 2^(m_a - m) : 0; beta = z_b > 0 ? 2^(m_b - m) : 0
//   z = z_a*alpha + z_b*beta; s = s_a*alpha + s_b*beta; m = z > 0 ? m : -inf
template <int NV>
__device__ __forceinline__ void monoid_merge(float& m_a, float& z_a, float (&s_a)[NV],
                                             float m_b, float z_b, const float (&s_b)[NV]) {
  float m = fmaxf(m_a, m_b);
  float alpha = z_a > 0.f ? exp2f(m_a - m) : 0.f;
  float beta = z_b > 0.f ? exp2f(m_b - m) : 0.f;
  float z = z_a * alpha + z_b * beta;
#pragma unroll
  for (int i = 0; i < NV; ++i) s_a[i] = s_a[i] * alpha + s_b[i] * beta;
  z_a = z;
  m_a = z > 0.f ? m : -CUDART_INF_F;
}

}  // namespace elsa
