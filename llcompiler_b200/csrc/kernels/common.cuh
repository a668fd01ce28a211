// Shared device helpers for the sm_100a kernel library.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>

#include "../../../include/llc_cuda.h"
#include "../capi_common.h"

namespace llc {

constexpr int kNumSMs = 148;   // B200: 2 dies x 74 SMs

inline int cudaFail(cudaError_t e, const char* what) {
  return setError(LLC_ERR_CUDA, std::string("llc cuda: ") + what + ": " + cudaGetErrorString(e));
}
#define LLC_CUDA_CHECK(expr)                                   \
  do {                                                         \
    cudaError_t e__ = (expr);                                  \
    if (e__ != cudaSuccess) return llc::cudaFail(e__, #expr);  \
  } while (0)
#define LLC_LAUNCH_CHECK(name)                                     \
  do {                                                             \
    cudaError_t e__ = cudaGetLastError();                          \
    if (e__ != cudaSuccess) return llc::cudaFail(e__, name);       \
  } while (0)

// One-time set-up that CUDA keeps per device (function attributes such as the dynamic shared-memory opt-in): a bit
// per device ordinal.  Two threads that meet on a fresh device both run the set-up, which is idempotent.
struct DeviceOnce {
  std::atomic<unsigned long long> done{0};
  bool test(int dev) const { return dev >= 0 && dev < 64 && ((done.load(std::memory_order_acquire) >> dev) & 1ull); }
  void set(int dev) { if (dev >= 0 && dev < 64) done.fetch_or(1ull << dev, std::memory_order_release); }
};
inline int currentDevice() { int d = 0; return cudaGetDevice(&d) == cudaSuccess ? d : 0; }
// SM count of the current device (cached per ordinal).
inline int deviceSMs() {
  static std::atomic<int> cache[64];
  const int dev = currentDevice();
  if (dev < 0 || dev >= 64) return kNumSMs;
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  v = kNumSMs;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = kNumSMs;
  cache[dev].store(v, std::memory_order_relaxed);
  return v;
}

inline int dtypeBytes(int32_t dt) {
  switch (dt) {
    case LLC_INT8: case LLC_INT1: return 1;
    case LLC_INT16: case LLC_FLOAT16: case LLC_BFLOAT16: return 2;
    case LLC_INT32: case LLC_FLOAT32: return 4;
    default: return 8;
  }
}
inline bool isFloatOut(int32_t dt) { return dt == LLC_FLOAT32 || dt == LLC_BFLOAT16 || dt == LLC_FLOAT16 || dt == LLC_FLOAT64; }

// ---- scalar load/store with a run-time element type (uniform per launch) -------------------
__device__ __forceinline__ float loadAs(const void* p, int64_t i, int dt) {
  switch (dt) {
    case LLC_FLOAT32: return reinterpret_cast<const float*>(p)[i];
    case LLC_BFLOAT16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    case LLC_FLOAT16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case LLC_INT64: return (float)reinterpret_cast<const long long*>(p)[i];
    case LLC_INT32: return (float)reinterpret_cast<const int*>(p)[i];
    case LLC_INT16: return (float)reinterpret_cast<const short*>(p)[i];
    case LLC_INT8: return (float)reinterpret_cast<const signed char*>(p)[i];
    case LLC_INT1: return reinterpret_cast<const unsigned char*>(p)[i] ? 1.f : 0.f;
    case LLC_FLOAT64: return (float)reinterpret_cast<const double*>(p)[i];
  }
  return 0.f;
}
__device__ __forceinline__ void storeAs(void* p, int64_t i, int dt, float v) {
  switch (dt) {
    case LLC_FLOAT32: reinterpret_cast<float*>(p)[i] = v; break;
    case LLC_BFLOAT16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
    case LLC_FLOAT16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(v); break;
    case LLC_INT64: reinterpret_cast<long long*>(p)[i] = (long long)v; break;
    case LLC_INT32: reinterpret_cast<int*>(p)[i] = (int)v; break;
    case LLC_INT16: reinterpret_cast<short*>(p)[i] = (short)v; break;
    case LLC_INT8: reinterpret_cast<signed char*>(p)[i] = (signed char)v; break;
    case LLC_INT1: reinterpret_cast<unsigned char*>(p)[i] = v != 0.f ? 1 : 0; break;
    case LLC_FLOAT64: reinterpret_cast<double*>(p)[i] = (double)v; break;
  }
}

// ---- 4-wide vector access for the two storage types the hot kernels use --------------------
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw; raw.x = *reinterpret_cast<unsigned*>(&lo); raw.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};
template <typename T> __device__ __forceinline__ float toFloat(T v);
template <> __device__ __forceinline__ float toFloat<float>(float v) { return v; }
template <> __device__ __forceinline__ float toFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float geluErf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
// GELU with erf from Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7 on erf): one exp, one reciprocal
// and five FMAs instead of the ~30 instructions of erff.  Used where the epilogue of a large GEMM
// would otherwise be bound by the activation (BERT's 98304 x 3072 feed-forward).
__device__ __forceinline__ float geluFast(float x) {
  const float z = fabsf(x) * 0.70710678118654752f;
  const float t = __frcp_rn(fmaf(0.3275911f, z, 1.f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float erfAbs = 1.f - poly * t * __expf(-z * z);
  return 0.5f * x * (1.f + copysignf(erfAbs, x));
}
// GELU for results that are stored as bf16: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) with the
// hardware tanh.  It differs from the erf form by at most 5e-4 absolute, below half a bf16 ulp
// wherever the two differ at all, and costs 6 instructions per element.
__device__ __forceinline__ float geluTanhBf16(float x) {
  const float u = x * fmaf(0.0356774081f, x * x, 0.7978845608f);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float h = 0.5f * x;
  return fmaf(h, t, h);
}
__device__ __forceinline__ float applyAct(float v, int act) {
  if (act == LLC_ACT_RELU) return fmaxf(v, 0.f);
  if (act == LLC_ACT_GELU) return geluErf(v);
  return v;
}

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warpMin(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace llc
