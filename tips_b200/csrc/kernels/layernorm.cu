// Layer normalisation over the last dimension of a row-major [rows, cols]
// matrix, forward and backward.  One warp owns a row: it reads the row once in
// 16-byte vectors, keeps it in registers, and produces mean / rstd / output (or
// dx) without a second trip to HBM.  In the backward pass each warp also
// accumulates dgamma / dbeta for its lane's columns over all the rows it
// visits; blocks write one partial row each and a small second kernel sums
// them.  The reference has no model math; this serves the BERT-shaped encoder.
#include "kernels/common.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

constexpr int kWarpsPerBlock = 4;

template <typename T>
struct VecOf {
  static constexpr int kN = 16 / sizeof(T);
};

// VPL = 16-byte vectors per lane; handles cols <= 32 * VPL * kN, cols % kN == 0.
template <typename T, int VPL, bool kResidual>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
LnFwdKernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
            float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t rows, int cols, float eps,
            const T* __restrict__ residual, T* __restrict__ sum_out) {
  // With `residual` the row normalised is x + residual (rounded to T, as a separate add kernel would leave it),
  // and that sum is also written to `sum_out` for the backward pass.
  constexpr int N = VecOf<T>::kN;
  const int lane  = threadIdx.x & 31;
  const int warp  = threadIdx.x >> 5;
  const int nvec  = cols / N;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp; r < rows;
       r += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
    const T* xr = x + r * cols;
    float v[VPL][N];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        Vec16<T> q = LoadVec(xr + vi * N);
        if constexpr (kResidual) {
          const Vec16<T> rr = LoadVec(residual + r * cols + vi * N);
#pragma unroll
          for (int i = 0; i < N; ++i) q.v[i] = FromFloat<T>(ToFloat<T>(q.v[i]) + ToFloat<T>(rr.v[i]));
          StoreVec(sum_out + r * cols + vi * N, q);
        }
#pragma unroll
        for (int i = 0; i < N; ++i) {
          v[k][i] = ToFloat<T>(q.v[i]);
          sum += v[k][i];
        }
      }
    }
    const float mean = WarpSum(sum) / cols;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
#pragma unroll
        for (int i = 0; i < N; ++i) {
          const float d = v[k][i] - mean;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(WarpSum(sq) / cols + eps);
    if (lane == 0) {
      mean_out[r] = mean;
      rstd_out[r] = rstd;
    }
    T* yr = y + r * cols;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        Vec16<T> g = LoadVec(gamma + vi * N), b = LoadVec(beta + vi * N), o;
#pragma unroll
        for (int i = 0; i < N; ++i)
          o.v[i] = FromFloat<T>((v[k][i] - mean) * rstd * ToFloat<T>(g.v[i]) + ToFloat<T>(b.v[i]));
        StoreVec(yr + vi * N, o);
      }
    }
  }
}

template <typename T, int VPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
LnBwdKernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
            const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
            float* __restrict__ dgamma_partial, float* __restrict__ dbeta_partial, int64_t rows, int cols) {
  constexpr int N = VecOf<T>::kN;
  extern __shared__ float smem[];  // [kWarpsPerBlock][2][cols]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = cols / N;
  float dg[VPL][N], db[VPL][N], gm[VPL][N];
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int vi = lane + k * 32;
    Vec16<T> g;
    if (vi < nvec) g = LoadVec(gamma + vi * N);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      dg[k][i] = db[k][i] = 0.f;
      gm[k][i] = vi < nvec ? ToFloat<T>(g.v[i]) : 0.f;
    }
  }
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp; r < rows;
       r += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
    const float mu = mean[r], rs = rstd[r];
    float xh[VPL][N], dyv[VPL][N];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        Vec16<T> qx = LoadVec(x + r * cols + vi * N), qd = LoadVec(dy + r * cols + vi * N);
#pragma unroll
        for (int i = 0; i < N; ++i) {
          xh[k][i]  = (ToFloat<T>(qx.v[i]) - mu) * rs;
          dyv[k][i] = ToFloat<T>(qd.v[i]);
          const float dyg = dyv[k][i] * gm[k][i];
          s1 += dyg;
          s2 += dyg * xh[k][i];
          dg[k][i] += dyv[k][i] * xh[k][i];
          db[k][i] += dyv[k][i];
        }
      }
    }
    s1 = WarpSum(s1) / cols;
    s2 = WarpSum(s2) / cols;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int vi = lane + k * 32;
      if (vi < nvec) {
        Vec16<T> o;
#pragma unroll
        for (int i = 0; i < N; ++i) o.v[i] = FromFloat<T>(rs * (dyv[k][i] * gm[k][i] - s1 - xh[k][i] * s2));
        StoreVec(dx + r * cols + vi * N, o);
      }
    }
  }
  // block-level reduction of the per-warp column sums
  float* sg = smem + warp * 2 * cols;
  float* sb = sg + cols;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int vi = lane + k * 32;
    if (vi < nvec) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        sg[vi * N + i] = dg[k][i];
        sb[vi * N + i] = db[k][i];
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsPerBlock; ++w) {
      a += smem[w * 2 * cols + c];
      b += smem[w * 2 * cols + cols + c];
    }
    dgamma_partial[static_cast<int64_t>(blockIdx.x) * cols + c] = a;
    dbeta_partial[static_cast<int64_t>(blockIdx.x) * cols + c]  = b;
  }
}

// Backward with one BLOCK per row: each thread owns 8 consecutive columns (one 16-byte vector), so the per-column
// dgamma / dbeta accumulators are 16 registers instead of 64 and many more rows are in flight per SM than with a
// warp per row.  The two row sums go through shared memory (one barrier per row, double-buffered).
template <typename T>
__global__ void __launch_bounds__(1024)
LnBwdBlockRowKernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                    const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                    float* __restrict__ dgamma_partial, float* __restrict__ dbeta_partial, int64_t rows, int cols) {
  constexpr int N = 8;
  __shared__ float red[2][2][32];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = blockDim.x >> 5;
  float gm[N], dg[N], db[N];
  {
    const Vec16<T> g = LoadVec(gamma + t * N);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      gm[i] = ToFloat<T>(g.v[i]);
      dg[i] = db[i] = 0.f;
    }
  }
  const float inv_cols = 1.f / static_cast<float>(cols);
  int it = 0;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x, ++it) {
    const float mu = mean[r], rs = rstd[r];
    const Vec16<T> qx = LoadVec(x + r * cols + t * N), qd = LoadVec(dy + r * cols + t * N);
    float xh[N], dyg[N];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      xh[i] = (ToFloat<T>(qx.v[i]) - mu) * rs;
      const float d = ToFloat<T>(qd.v[i]);
      dyg[i] = d * gm[i];
      s1 += dyg[i];
      s2 += dyg[i] * xh[i];
      dg[i] += d * xh[i];
      db[i] += d;
    }
    s1 = WarpSum(s1);
    s2 = WarpSum(s2);
    const int p = it & 1;
    if (lane == 0) {
      red[p][0][warp] = s1;
      red[p][1][warp] = s2;
    }
    __syncthreads();
    s1 = s2 = 0.f;
    for (int w = 0; w < nwarps; ++w) {
      s1 += red[p][0][w];
      s2 += red[p][1][w];
    }
    s1 *= inv_cols;
    s2 *= inv_cols;
    Vec16<T> o;
#pragma unroll
    for (int i = 0; i < N; ++i) o.v[i] = FromFloat<T>(rs * (dyg[i] - s1 - xh[i] * s2));
    StoreVec(dx + r * cols + t * N, o);
  }
  float* pg = dgamma_partial + static_cast<int64_t>(blockIdx.x) * cols + t * N;
  float* pb = dbeta_partial + static_cast<int64_t>(blockIdx.x) * cols + t * N;
#pragma unroll
  for (int i = 0; i < N; ++i) {
    pg[i] = dg[i];
    pb[i] = db[i];
  }
}

// Column sums of the per-block partial gradients. Block (32, 32): tx = column, ty strides over the partial rows.
template <typename T>
__global__ void __launch_bounds__(1024)
LnReducePartialsKernel(const float* __restrict__ pg, const float* __restrict__ pb, int partial_rows, int cols,
                       T* __restrict__ dgamma, T* __restrict__ dbeta) {
  __shared__ float ra[32][33], rb[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float a = 0.f, b = 0.f;
  if (c < cols) {
    for (int p = threadIdx.y; p < partial_rows; p += 32) {
      a += pg[static_cast<int64_t>(p) * cols + c];
      b += pb[static_cast<int64_t>(p) * cols + c];
    }
  }
  ra[threadIdx.y][threadIdx.x] = a;
  rb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      sa += ra[j][threadIdx.x];
      sb += rb[j][threadIdx.x];
    }
    dgamma[c] = FromFloat<T>(sa);
    dbeta[c]  = FromFloat<T>(sb);
  }
}

int LnGrid(int64_t rows) {
  int64_t blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  int64_t cap    = static_cast<int64_t>(NumSMs()) * 8;
  return static_cast<int>(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

}  // namespace
}  // namespace tipsk

using namespace tipsk;

#define LN_DISPATCH(dtype, cols, ...)                                                        \
  {                                                                                          \
    if (dtype == kBF16) { using T = __nv_bfloat16; LN_VPL(cols, __VA_ARGS__) }               \
    else if (dtype == kF16) { using T = __half; LN_VPL(cols, __VA_ARGS__) }                  \
    else if (dtype == kF32) { using T = float; LN_VPL(cols, __VA_ARGS__) }                   \
    else return SetError(-2, "layer norm: unsupported dtype");                               \
  }
#define LN_VPL(cols, ...)                                                                    \
  {                                                                                          \
    const int per_lane = ((cols) / VecOf<T>::kN + 31) / 32;                                  \
    if (per_lane <= 1) { constexpr int VPL = 1; __VA_ARGS__; }                               \
    else if (per_lane <= 2) { constexpr int VPL = 2; __VA_ARGS__; }                          \
    else if (per_lane <= 4) { constexpr int VPL = 4; __VA_ARGS__; }                          \
    else if (per_lane <= 8) { constexpr int VPL = 8; __VA_ARGS__; }                          \
    else return SetError(-2, "layer norm: rows longer than 8 vectors per lane are not supported"); \
  }

extern "C" {

int tipsk_ln_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int64_t rows,
                 int cols, float eps, int dtype, void* stream) {
  if (rows <= 0) return 0;
  TIPSK_REQUIRE(cols > 0 && cols % (16 / (int)DTypeSize(dtype)) == 0, "layer norm: cols must be a multiple of 16 bytes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LN_DISPATCH(dtype, cols, {
    LnFwdKernel<T, VPL, false><<<LnGrid(rows), kWarpsPerBlock * 32, 0, s>>>(
        static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<T*>(y), mean,
        rstd, rows, cols, eps, nullptr, nullptr);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* y = LN(x + residual); the sum (rounded to the activation dtype) is written to sum_out for the backward pass. */
int tipsk_ln_fwd_residual(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                          void* sum_out, float* mean, float* rstd, int64_t rows, int cols, float eps, int dtype,
                          void* stream) {
  if (rows <= 0) return 0;
  TIPSK_REQUIRE(cols > 0 && cols % (16 / (int)DTypeSize(dtype)) == 0, "layer norm: cols must be a multiple of 16 bytes");
  TIPSK_REQUIRE(residual != nullptr && sum_out != nullptr, "layer norm: residual and sum_out are required");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LN_DISPATCH(dtype, cols, {
    LnFwdKernel<T, VPL, true><<<LnGrid(rows), kWarpsPerBlock * 32, 0, s>>>(
        static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<T*>(y), mean,
        rstd, rows, cols, eps, static_cast<const T*>(residual), static_cast<T*>(sum_out));
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_ln_bwd_partials(int64_t rows, int cols) {
  (void)cols;
  return LnGrid(rows);
}

int tipsk_ln_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                 float* dgamma_partial, float* dbeta_partial, int partial_rows, int64_t rows, int cols, int dtype,
                 void* stream) {
  if (rows <= 0) return 0;
  TIPSK_REQUIRE(cols > 0 && cols % (16 / (int)DTypeSize(dtype)) == 0, "layer norm: cols must be a multiple of 16 bytes");
  TIPSK_REQUIRE(partial_rows == LnGrid(rows), "layer norm backward: wrong number of partial rows");
  cudaStream_t s    = static_cast<cudaStream_t>(stream);
  if (dtype != kF32 && cols % 256 == 0 && cols / 8 <= 1024) {  // one block of cols/8 threads per row
    if (dtype == kBF16)
      LnBwdBlockRowKernel<__nv_bfloat16><<<partial_rows, cols / 8, 0, s>>>(
          static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
          static_cast<const __nv_bfloat16*>(gamma), mean, rstd, static_cast<__nv_bfloat16*>(dx), dgamma_partial,
          dbeta_partial, rows, cols);
    else
      LnBwdBlockRowKernel<__half><<<partial_rows, cols / 8, 0, s>>>(
          static_cast<const __half*>(dy), static_cast<const __half*>(x), static_cast<const __half*>(gamma), mean, rstd,
          static_cast<__half*>(dx), dgamma_partial, dbeta_partial, rows, cols);
    TIPSK_LAUNCH_CHECK();
    return 0;
  }
  const size_t smem = sizeof(float) * kWarpsPerBlock * 2 * cols;
  TIPSK_REQUIRE(smem <= 48 * 1024, "layer norm backward: row too long for the shared-memory reduction");
  LN_DISPATCH(dtype, cols, {
    LnBwdKernel<T, VPL><<<partial_rows, kWarpsPerBlock * 32, smem, s>>>(
        static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(gamma), mean, rstd,
        static_cast<T*>(dx), dgamma_partial, dbeta_partial, rows, cols);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_ln_reduce_partials(const float* dgamma_partial, const float* dbeta_partial, int partial_rows, int cols,
                             void* dgamma, void* dbeta, int dtype, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = CeilDiv(cols, 32);
  const dim3 block(32, 32);
  if (dtype == kBF16)
    LnReducePartialsKernel<__nv_bfloat16><<<grid, block, 0, s>>>(dgamma_partial, dbeta_partial, partial_rows, cols,
                                                               static_cast<__nv_bfloat16*>(dgamma),
                                                               static_cast<__nv_bfloat16*>(dbeta));
  else if (dtype == kF16)
    LnReducePartialsKernel<__half><<<grid, block, 0, s>>>(dgamma_partial, dbeta_partial, partial_rows, cols,
                                                        static_cast<__half*>(dgamma), static_cast<__half*>(dbeta));
  else if (dtype == kF32)
    LnReducePartialsKernel<float><<<grid, block, 0, s>>>(dgamma_partial, dbeta_partial, partial_rows, cols,
                                                       static_cast<float*>(dgamma), static_cast<float*>(dbeta));
  else
    return SetError(-2, "layer norm: unsupported dtype");
  TIPSK_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
