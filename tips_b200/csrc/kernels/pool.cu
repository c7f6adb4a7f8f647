// 3x3 / stride 2 / pad 1 max pooling on NHWC activations (the ResNet stem pool), forward and backward.
//
// Forward: one thread per (output pixel, 8 channels): nine 16-byte loads, a running maximum that keeps the
// FIRST maximum in scan order (rows, then columns), one 16-byte store of the result and 8 bytes of argmax
// codes (0..8).  Backward: one thread per (input pixel, 8 channels) gathers from the at most four windows
// that contain the pixel the gradients whose argmax code points at it: no atomics, deterministic, and the
// input activation is not read again.
//
// The reference has no pooling (model math is TensorFlow's); this serves the ResNet-50 benchmark model.
#include <algorithm>

#include "kernels/common.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

template <typename T>
__global__ void __launch_bounds__(256)
MaxPoolFwdKernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ idx, int n, int h, int w, int c,
                 int ho, int wo) {
  constexpr int V = 8;
  const int cv = c / V;
  const int64_t total = static_cast<int64_t>(n) * ho * wo * cv;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(i % cv);
    int64_t pix  = i / cv;
    const int ow = static_cast<int>(pix % wo); pix /= wo;
    const int oh = static_cast<int>(pix % ho);
    const int in = static_cast<int>(pix / ho);
    float best[V];
    uint8_t arg[V];
#pragma unroll
    for (int j = 0; j < V; ++j) { best[j] = -INFINITY; arg[j] = 0; }
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int ih = oh * 2 - 1 + r;
      if (ih < 0 || ih >= h) continue;
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        const int iw = ow * 2 - 1 + s;
        if (iw < 0 || iw >= w) continue;
        const Vec16<T> v = LoadVec(x + ((static_cast<int64_t>(in) * h + ih) * w + iw) * c + cg * V);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float f = ToFloat(v.v[j]);
          if (f > best[j]) { best[j] = f; arg[j] = static_cast<uint8_t>(r * 3 + s); }
        }
      }
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = FromFloat<T>(best[j]);
    const int64_t opix = (static_cast<int64_t>(in) * ho + oh) * wo + ow;
    StoreVec(y + opix * c + cg * V, o);
    uint2 packed;
    packed.x = arg[0] | (arg[1] << 8) | (arg[2] << 16) | (arg[3] << 24);
    packed.y = arg[4] | (arg[5] << 8) | (arg[6] << 16) | (arg[7] << 24);
    *reinterpret_cast<uint2*>(idx + opix * c + cg * V) = packed;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
MaxPoolBwdKernel(const T* __restrict__ dy, const uint8_t* __restrict__ idx, T* __restrict__ dx, int n, int h, int w,
                 int c, int ho, int wo) {
  constexpr int V = 8;
  const int cv = c / V;
  const int64_t total = static_cast<int64_t>(n) * h * w * cv;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(i % cv);
    int64_t pix  = i / cv;
    const int iw = static_cast<int>(pix % w); pix /= w;
    const int ih = static_cast<int>(pix % h);
    const int in = static_cast<int>(pix / h);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    // windows oh with 2*oh - 1 <= ih <= 2*oh + 1
    const int oh_lo = ih / 2, oh_hi = (ih + 1) / 2;
    const int ow_lo = iw / 2, ow_hi = (iw + 1) / 2;
    for (int oh = oh_lo; oh <= oh_hi; ++oh) {
      if (oh >= ho) continue;
      const int r = ih - (oh * 2 - 1);
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        if (ow >= wo) continue;
        const int s = iw - (ow * 2 - 1);
        const uint32_t code = static_cast<uint32_t>(r * 3 + s);
        const int64_t opix  = (static_cast<int64_t>(in) * ho + oh) * wo + ow;
        const uint2 packed  = *reinterpret_cast<const uint2*>(idx + opix * c + cg * V);
        const Vec16<T> g    = LoadVec(dy + opix * c + cg * V);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const uint32_t a = ((j < 4 ? packed.x : packed.y) >> ((j & 3) * 8)) & 0xffu;
          if (a == code) acc[j] += ToFloat(g.v[j]);
        }
      }
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = FromFloat<T>(acc[j]);
    StoreVec(dx + ((static_cast<int64_t>(in) * h + ih) * w + iw) * c + cg * V, o);
  }
}

int GridFor(int64_t total) {
  const int64_t blocks = (total + 255) / 256;
  const int64_t cap    = static_cast<int64_t>(NumSMs()) * 16;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

// Global average pooling of an NHWC activation: y[n, c] = mean over the hw pixels; one thread per (image, 8
// channels), 16-byte loads down the pixel axis.  Backward spreads dy / hw over the pixels.
template <typename T>
__global__ void __launch_bounds__(256)
GlobalAvgPoolFwdKernel(const T* __restrict__ x, T* __restrict__ y, int n, int hw, int c) {
  constexpr int V = 16 / sizeof(T);
  const int cv = c / V;
  const int64_t total = static_cast<int64_t>(n) * cv;
  const float inv = 1.f / static_cast<float>(hw);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(i % cv);
    const int in = static_cast<int>(i / cv);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    const T* base = x + static_cast<int64_t>(in) * hw * c + cg * V;
    for (int p = 0; p < hw; ++p) {
      const Vec16<T> v = LoadVec(base + static_cast<int64_t>(p) * c);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += ToFloat(v.v[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = FromFloat<T>(acc[j] * inv);
    StoreVec(y + static_cast<int64_t>(in) * c + cg * V, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
GlobalAvgPoolBwdKernel(const T* __restrict__ dy, T* __restrict__ dx, int n, int hw, int c) {
  constexpr int V = 16 / sizeof(T);
  const int cv = c / V;
  const int64_t total = static_cast<int64_t>(n) * hw * cv;
  const float inv = 1.f / static_cast<float>(hw);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(i % cv);
    const int in = static_cast<int>(i / (static_cast<int64_t>(cv) * hw));
    const Vec16<T> g = LoadVec(dy + static_cast<int64_t>(in) * c + cg * V);
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = FromFloat<T>(ToFloat(g.v[j]) * inv);
    StoreVec(dx + i * V, o);
  }
}

}  // namespace
}  // namespace tipsk

using namespace tipsk;

extern "C" {

/* y[n, ho, wo, c] = max over 3x3 windows (stride 2, pad 1) of x[n, h, w, c]; idx (uint8, same shape as y) receives
 * the position 0..8 of the maximum inside its window.  dtype: 6 bf16 or 7 fp16; c must be a multiple of 8. */
int tipsk_maxpool3x3s2_fwd(const void* x, void* y, void* idx, int n, int h, int w, int c, int dtype, void* stream) {
  TIPSK_REQUIRE(c % 8 == 0, "maxpool: channel count must be a multiple of 8");
  TIPSK_REQUIRE(dtype == kBF16 || dtype == kF16, "maxpool: bf16 or fp16 only");
  const int ho = (h + 2 - 3) / 2 + 1, wo = (w + 2 - 3) / 2 + 1;
  const int64_t total = static_cast<int64_t>(n) * ho * wo * (c / 8);
  if (total == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    MaxPoolFwdKernel<__nv_bfloat16><<<GridFor(total), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                                  static_cast<__nv_bfloat16*>(y),
                                                                  static_cast<uint8_t*>(idx), n, h, w, c, ho, wo);
  else
    MaxPoolFwdKernel<__half><<<GridFor(total), 256, 0, s>>>(static_cast<const __half*>(x), static_cast<__half*>(y),
                                                            static_cast<uint8_t*>(idx), n, h, w, c, ho, wo);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_maxpool3x3s2_bwd(const void* dy, const void* idx, void* dx, int n, int h, int w, int c, int dtype,
                           void* stream) {
  TIPSK_REQUIRE(c % 8 == 0, "maxpool: channel count must be a multiple of 8");
  TIPSK_REQUIRE(dtype == kBF16 || dtype == kF16, "maxpool: bf16 or fp16 only");
  const int ho = (h + 2 - 3) / 2 + 1, wo = (w + 2 - 3) / 2 + 1;
  const int64_t total = static_cast<int64_t>(n) * h * w * (c / 8);
  if (total == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    MaxPoolBwdKernel<__nv_bfloat16><<<GridFor(total), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy),
                                                                  static_cast<const uint8_t*>(idx),
                                                                  static_cast<__nv_bfloat16*>(dx), n, h, w, c, ho, wo);
  else
    MaxPoolBwdKernel<__half><<<GridFor(total), 256, 0, s>>>(static_cast<const __half*>(dy),
                                                            static_cast<const uint8_t*>(idx), static_cast<__half*>(dx),
                                                            n, h, w, c, ho, wo);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* Global average pooling on NHWC: x [n, hw, c] -> y [n, c]; c a multiple of 8 (16-bit types) / 4 (fp32). */
int tipsk_global_avgpool_fwd(const void* x, void* y, int n, int hw, int c, int dtype, void* stream) {
  if (n <= 0 || hw <= 0 || c <= 0) return 0;
  const int v = 16 / static_cast<int>(DTypeSize(dtype));
  TIPSK_REQUIRE(dtype == kBF16 || dtype == kF16 || dtype == kF32, "avgpool: bf16, fp16 or fp32");
  TIPSK_REQUIRE(c % v == 0, "avgpool: the channel count must be a multiple of 16 bytes");
  const int64_t total = static_cast<int64_t>(n) * (c / v);
  const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, NumSMs() * 8));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    GlobalAvgPoolFwdKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                               static_cast<__nv_bfloat16*>(y), n, hw, c);
  else if (dtype == kF16)
    GlobalAvgPoolFwdKernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(x), static_cast<__half*>(y), n, hw, c);
  else
    GlobalAvgPoolFwdKernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(y), n, hw, c);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_global_avgpool_bwd(const void* dy, void* dx, int n, int hw, int c, int dtype, void* stream) {
  if (n <= 0 || hw <= 0 || c <= 0) return 0;
  const int v = 16 / static_cast<int>(DTypeSize(dtype));
  TIPSK_REQUIRE(dtype == kBF16 || dtype == kF16 || dtype == kF32, "avgpool: bf16, fp16 or fp32");
  TIPSK_REQUIRE(c % v == 0, "avgpool: the channel count must be a multiple of 16 bytes");
  const int64_t total = static_cast<int64_t>(n) * hw * (c / v);
  const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, NumSMs() * 8));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    GlobalAvgPoolBwdKernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy),
                                                               static_cast<__nv_bfloat16*>(dx), n, hw, c);
  else if (dtype == kF16)
    GlobalAvgPoolBwdKernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(dy), static_cast<__half*>(dx), n, hw, c);
  else
    GlobalAvgPoolBwdKernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(dy), static_cast<float*>(dx), n, hw, c);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
