// Pointwise epilogues and fused losses: bias + activation (ReLU / GELU) forward
// and backward with the bias gradient reduced in the same pass, binary
// cross-entropy with logits (loss and gradient in one read of the logits) and
// softmax cross-entropy (loss, count and gradient per row in one kernel).
// The reference leaves all of this to TensorFlow ops; here they are fused so
// that each activation tensor is touched once per direction.
#include "kernels/common.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

__device__ __forceinline__ float Act(float v, int act) {
  if (act == 1) return fmaxf(v, 0.f);
  if (act == 2) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  return v;
}
__device__ __forceinline__ float ActGrad(float v, int act) {
  if (act == 1) return v > 0.f ? 1.f : 0.f;
  if (act == 2) {
    // d/dv [v * Phi(v)] = Phi(v) + v * phi(v).  Phi through erf(z), z = v / sqrt(2), with the rational approximation
    // erf(z) = 1 - (a1 t + ... + a5 t^5) exp(-z^2), t = 1 / (1 + p z) (absolute error < 1.5e-7): exp(-z^2) is the
    // same exponential the density phi(v) needs, so the whole derivative costs one exp and one reciprocal.
    const float e  = __expf(-0.5f * v * v);
    const float z  = fabsf(v) * 0.70710678118654752f;
    const float t  = __frcp_rn(1.f + 0.3275911f * z);
    const float pl = t * (0.254829592f + t * (-0.284496736f + t * (1.421413741f + t * (-1.453152027f + t * 1.061405429f))));
    const float erf_abs = 1.f - pl * e;
    const float phi_cdf = 0.5f * (1.f + copysignf(erf_abs, v));
    return phi_cdf + v * 0.3989422804014327f * e;
  }
  return 1.f;
}

template <typename T>
__global__ void __launch_bounds__(256)
BiasActFwdKernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y, int64_t rows, int cols,
                 int act) {
  constexpr int N      = 16 / sizeof(T);
  const int vec_cols   = cols / N;
  const int64_t total  = rows * vec_cols;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int vc = static_cast<int>(i % vec_cols);
    Vec16<T> q = LoadVec(x + i * N), o;
    if (bias) {
      Vec16<T> b = LoadVec(bias + vc * N);
#pragma unroll
      for (int k = 0; k < N; ++k) o.v[k] = FromFloat<T>(Act(ToFloat<T>(q.v[k]) + ToFloat<T>(b.v[k]), act));
    } else {
#pragma unroll
      for (int k = 0; k < N; ++k) o.v[k] = FromFloat<T>(Act(ToFloat<T>(q.v[k]), act));
    }
    StoreVec(y + i * N, o);
  }
}

// block (32, 8): tx -> vector column, ty -> row lane; grid (col tiles, row partitions)
template <typename T>
__global__ void __launch_bounds__(256)
BiasActBwdKernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ dx,
                 float* __restrict__ dbias, int64_t rows, int cols, int act) {
  constexpr int N = 16 / sizeof(T);
  __shared__ float red[8][32][N + 1];
  const int vec_cols = cols / N;
  const int vc       = blockIdx.x * 32 + threadIdx.x;
  float acc[N];
#pragma unroll
  for (int k = 0; k < N; ++k) acc[k] = 0.f;
  if (vc < vec_cols) {
    float bv[N];
    if (bias) {
      Vec16<T> b = LoadVec(bias + vc * N);
#pragma unroll
      for (int k = 0; k < N; ++k) bv[k] = ToFloat<T>(b.v[k]);
    } else {
#pragma unroll
      for (int k = 0; k < N; ++k) bv[k] = 0.f;
    }
    for (int64_t r = static_cast<int64_t>(blockIdx.y) * 8 + threadIdx.y; r < rows;
         r += static_cast<int64_t>(gridDim.y) * 8) {
      const int64_t off = r * cols + static_cast<int64_t>(vc) * N;
      Vec16<T> d = LoadVec(dy + off), o;
      if (act != 0) {
        Vec16<T> q = LoadVec(x + off);
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const float g = ToFloat<T>(d.v[k]) * ActGrad(ToFloat<T>(q.v[k]) + bv[k], act);
          acc[k] += g;
          o.v[k] = FromFloat<T>(g);
        }
      } else {
#pragma unroll
        for (int k = 0; k < N; ++k) {
          acc[k] += ToFloat<T>(d.v[k]);
          o.v[k] = d.v[k];
        }
      }
      if (dx) StoreVec(dx + off, o);
    }
  }
  if (!dbias) return;
#pragma unroll
  for (int k = 0; k < N; ++k) red[threadIdx.y][threadIdx.x][k] = acc[k];
  __syncthreads();
  if (threadIdx.y == 0 && vc < vec_cols) {
#pragma unroll
    for (int k = 0; k < N; ++k) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s += red[j][threadIdx.x][k];
      atomicAdd(dbias + vc * N + k, s);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
SigmoidBceKernel(const T* __restrict__ z, const float* __restrict__ t, float* __restrict__ loss_sum,
                 T* __restrict__ dz, int64_t n, float scale) {
  __shared__ float warp_sums[8];
  float local = 0.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float zi = ToFloat<T>(z[i]), ti = t[i];
    local += fmaxf(zi, 0.f) - zi * ti + log1pf(__expf(-fabsf(zi)));
    if (dz) dz[i] = FromFloat<T>((1.f / (1.f + __expf(-zi)) - ti) * scale);
  }
  local = WarpSum(local);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x < 8) {
    float v = warp_sums[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffu, v, o);
    if (threadIdx.x == 0) atomicAdd(loss_sum, v);
  }
}

__device__ __forceinline__ float BlockReduce(float v, bool is_max, float* scratch) {
  v = is_max ? WarpMax(v) : WarpSum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
  return r;
}

template <typename T>
__global__ void __launch_bounds__(256)
SoftmaxXentKernel(const T* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ loss_sum,
                  float* __restrict__ count, T* __restrict__ dlogits, int64_t rows, int cols, int64_t ignore_index,
                  float scale) {
  __shared__ float scratch[8];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* row        = logits + r * cols;
    const int64_t label = labels[r];
    const bool ignored  = label == ignore_index || label < 0 || label >= cols;
    if (ignored) {
      if (dlogits)
        for (int c = threadIdx.x; c < cols; c += blockDim.x) dlogits[r * cols + c] = FromFloat<T>(0.f);
      continue;
    }
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) mx = fmaxf(mx, ToFloat<T>(row[c]));
    mx = BlockReduce(mx, true, scratch);
    float se = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) se += __expf(ToFloat<T>(row[c]) - mx);
    se = BlockReduce(se, false, scratch);
    const float lse = mx + logf(se);
    if (threadIdx.x == 0) {
      atomicAdd(loss_sum, lse - ToFloat<T>(row[label]));
      if (count) atomicAdd(count, 1.f);
    }
    if (dlogits) {
      const float inv = 1.f / se;
      for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float p = __expf(ToFloat<T>(row[c]) - mx) * inv;
        if (c == label) p -= 1.f;
        dlogits[r * cols + c] = FromFloat<T>(p * scale);
      }
    }
  }
}

}  // namespace
}  // namespace tipsk

using namespace tipsk;

#define EPI_DISPATCH(dtype, ...)                                        \
  if (dtype == kBF16) { using T = __nv_bfloat16; __VA_ARGS__; }         \
  else if (dtype == kF16) { using T = __half; __VA_ARGS__; }            \
  else if (dtype == kF32) { using T = float; __VA_ARGS__; }             \
  else return SetError(-2, "unsupported dtype");

extern "C" {

int tipsk_bias_act_fwd(const void* x, const void* bias, void* y, int64_t rows, int cols, int act, int dtype,
                       void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  TIPSK_REQUIRE(cols % (16 / (int)DTypeSize(dtype)) == 0, "bias_act: cols must be a multiple of 16 bytes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t vecs = rows * (cols / (16 / (int)DTypeSize(dtype)));
  int grid = CeilDiv(vecs, 256);
  if (grid > NumSMs() * 8) grid = NumSMs() * 8;
  EPI_DISPATCH(dtype, {
    BiasActFwdKernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(bias), static_cast<T*>(y),
                                             rows, cols, act);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_bias_act_bwd(const void* dy, const void* x, const void* bias, void* dx, float* dbias, int64_t rows, int cols,
                       int act, int dtype, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const int n = 16 / (int)DTypeSize(dtype);
  TIPSK_REQUIRE(cols % n == 0, "bias_act: cols must be a multiple of 16 bytes");
  TIPSK_REQUIRE(act == 0 || x, "bias_act backward needs the pre-activation input");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dbias) TIPSK_CUDA(cudaMemsetAsync(dbias, 0, sizeof(float) * cols, s));
  const int col_tiles = CeilDiv(cols / n, 32);
  int parts = CeilDiv(NumSMs() * 4, col_tiles);
  int maxp  = CeilDiv(rows, 8 * 4);
  if (parts > maxp) parts = maxp;
  if (parts < 1) parts = 1;
  dim3 grid(col_tiles, parts), block(32, 8);
  EPI_DISPATCH(dtype, {
    BiasActBwdKernel<T><<<grid, block, 0, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x),
                                               static_cast<const T*>(bias), static_cast<T*>(dx), dbias, rows, cols, act);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_sigmoid_bce(const void* logits, const float* targets, float* loss_sum, void* dlogits, int64_t n,
                      float grad_scale, int dtype, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int grid = CeilDiv(n, 256);
  if (grid > NumSMs() * 4) grid = NumSMs() * 4;
  EPI_DISPATCH(dtype, {
    SigmoidBceKernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(logits), targets, loss_sum, static_cast<T*>(dlogits),
                                             n, grad_scale);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_softmax_xent(const void* logits, const int64_t* labels, float* loss_sum, float* count, void* dlogits,
                       int64_t rows, int cols, int64_t ignore_index, float grad_scale, int dtype, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int grid = rows < NumSMs() * 8 ? static_cast<int>(rows) : NumSMs() * 8;
  EPI_DISPATCH(dtype, {
    SoftmaxXentKernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(logits), labels, loss_sum, count,
                                              static_cast<T*>(dlogits), rows, cols, ignore_index, grad_scale);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
