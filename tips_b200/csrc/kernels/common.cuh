// Shared helpers of the sm_100a kernel library: error plumbing for the
// extern "C" launchers, dtype codes, vector load/store helpers.
//
// Every launcher returns 0 on success or a negative code and leaves a message
// retrievable with tipsk_last_error(); none of them allocates device memory
// unless its name says so, and all of them launch on the stream they are given.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace tipsk {

// Values match tips::Datatype on the host side.
enum DType : int32_t { kF32 = 0, kF64 = 1, kI32 = 2, kI64 = 3, kI8 = 4, kU8 = 5, kBF16 = 6, kF16 = 7 };

inline size_t DTypeSize(int32_t dt) {
  switch (dt) {
    case kF32: case kI32: return 4;
    case kF64: case kI64: return 8;
    case kI8: case kU8: return 1;
    case kBF16: case kF16: return 2;
    default: return 0;
  }
}

std::string& LastError();
int SetError(int code, const std::string& msg);

#define TIPSK_CUDA(expr)                                                                          \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess)                                                                        \
      return ::tipsk::SetError(-7, std::string(#expr) + ": " + cudaGetErrorString(_e));           \
  } while (0)

#define TIPSK_LAUNCH_CHECK()                                                                      \
  do {                                                                                            \
    cudaError_t _e = cudaGetLastError();                                                          \
    if (_e != cudaSuccess)                                                                        \
      return ::tipsk::SetError(-7, std::string("kernel launch failed: ") + cudaGetErrorString(_e)); \
  } while (0)

#define TIPSK_REQUIRE(cond, msg)                         \
  do {                                                   \
    if (!(cond)) return ::tipsk::SetError(-2, (msg));    \
  } while (0)

inline int CeilDiv(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

// Number of SMs of the current device (cached).
int NumSMs();

// ---- device-side conversions ------------------------------------------------
template <typename T>
__device__ __forceinline__ float ToFloat(T v);
template <>
__device__ __forceinline__ float ToFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ float ToFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float ToFloat<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T FromFloat(float v);
template <>
__device__ __forceinline__ float FromFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 FromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half FromFloat<__half>(float v) { return __float2half_rn(v); }

// 16-byte vector of T.
template <typename T>
struct alignas(16) Vec16 {
  static constexpr int kN = 16 / sizeof(T);
  T v[kN];
};

template <typename T>
__device__ __forceinline__ Vec16<T> LoadVec(const T* p) {
  return *reinterpret_cast<const Vec16<T>*>(p);
}
template <typename T>
__device__ __forceinline__ void StoreVec(T* p, const Vec16<T>& v) {
  *reinterpret_cast<Vec16<T>*>(p) = v;
}

__device__ __forceinline__ float WarpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float WarpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace tipsk
