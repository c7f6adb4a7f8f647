// Batch normalisation (channels-last) and layer normalisation, forward and
// backward, with the neighbouring pointwise work fused in: the BN forward adds
// the residual branch and applies ReLU while it writes the output, and the BN
// backward applies the ReLU mask and emits the residual gradient while it reads
// dy.  The reference delegates all model math to TensorFlow ops; these kernels
// exist because normalisation layers are HBM-bound and every extra pass over
// the activations costs as much as the layer itself.
//
// Layout: activations are a row-major [M, C] matrix (M = N*H*W for NHWC batch
// norm, rows x cols for layer norm), 16-byte vectors along C.
#include "kernels/common.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {
namespace {

// ------------------------------------------------------------------ batch norm

template <typename T, int V>
struct alignas(sizeof(T) * V) VecT {
  T v[V];
};

template <typename T, int V>
__device__ __forceinline__ void LoadV(const T* p, float (&out)[V]) {
  VecT<T, V> q = *reinterpret_cast<const VecT<T, V>*>(p);
#pragma unroll
  for (int i = 0; i < V; ++i) out[i] = ToFloat<T>(q.v[i]);
}
template <typename T, int V>
__device__ __forceinline__ void StoreV(T* p, const float (&in)[V]) {
  VecT<T, V> q;
#pragma unroll
  for (int i = 0; i < V; ++i) q.v[i] = FromFloat<T>(in[i]);
  *reinterpret_cast<VecT<T, V>*>(p) = q;
}

struct BnGeom {
  int tx, ty;      // block = tx * ty threads; tx vector-columns, ty rows
  int col_tiles;   // grid.x
  int partials;    // grid.y of the reduction kernels and of the backward apply kernel (3 blocks per SM, 2 waves)
  int fwd_rows;    // grid.y of the forward apply kernel (4 blocks per SM, 2 waves)
};

BnGeom BnGeometry(int64_t m, int c, int v) {
  BnGeom g;
  int vec_cols = c / v;
  g.tx = 1;
  while (g.tx * 2 <= vec_cols && g.tx < 32 && vec_cols % (g.tx * 2) == 0) g.tx *= 2;
  g.ty        = 256 / g.tx;
  g.col_tiles = vec_cols / g.tx;
  // Whole waves: the kernels are grid-stride loops over the rows, and a last partial wave costs a full one.
  int64_t maxp = (m + g.ty * 4 - 1) / (g.ty * 4);
  int64_t want = (static_cast<int64_t>(NumSMs()) * 6 + g.col_tiles - 1) / g.col_tiles;
  if (want > maxp) want = maxp;
  if (want < 1) want = 1;
  if (want > 1024) want = 1024;
  g.partials = static_cast<int>(want);
  int64_t fwd = (static_cast<int64_t>(NumSMs()) * 8 + g.col_tiles - 1) / g.col_tiles;
  if (fwd > maxp) fwd = maxp;
  if (fwd < 1) fwd = 1;
  g.fwd_rows = static_cast<int>(fwd);
  return g;
}

// Partial column sums of a and a*b-like quantities.
// kBwd = false: s0 = sum x, s1 = sum x^2
// kBwd = true : s0 = sum dyr, s1 = sum dyr * xhat, with dyr = relu-masked dy
// kMask (backward only): how the ReLU mask is obtained: 0 from the forward output y, 1 recomputed from x,
// 2 from the bit mask the forward pass wrote (one byte per 8 channels; needs V == 8).
template <typename T, int V, bool kBwd, int kMask = 0>
__global__ void __launch_bounds__(256, 3)
BnReduceKernel(const T* __restrict__ a, const T* __restrict__ x, const T* __restrict__ y,
               const float* __restrict__ mean, const float* __restrict__ invstd, float* __restrict__ ws, int64_t m,
               int c, int relu, const float* __restrict__ gamma = nullptr, const float* __restrict__ beta = nullptr,
               const uint8_t* __restrict__ relu_mask = nullptr) {
  // relu with y == nullptr: the mask is recomputed from x exactly as the forward pass computed its output
  // (x * scale + shift > 0), which saves reading the forward output; needs gamma and beta.
  extern __shared__ float smem[];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int TX = blockDim.x, TY = blockDim.y;
  const int col = (blockIdx.x * TX + tx) * V;
  float s0[V], s1[V], mu[V], is[V], sc[V], sh[V];
#pragma unroll
  for (int i = 0; i < V; ++i) s0[i] = s1[i] = sc[i] = sh[i] = 0.f;
  constexpr bool recompute = kBwd && kMask == 1;
  if (kBwd) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      mu[i] = mean[col + i];
      is[i] = invstd[col + i];
      if (recompute) {
        sc[i] = gamma[col + i] * is[i];
        sh[i] = beta[col + i] - mu[i] * sc[i];
      }
    }
  }
#pragma unroll 4
  for (int64_t r = static_cast<int64_t>(blockIdx.y) * TY + ty; r < m; r += static_cast<int64_t>(gridDim.y) * TY) {
    float av[V];
    LoadV<T, V>(a + r * c + col, av);
    if (kBwd) {
      float xv[V];
      LoadV<T, V>(x + r * c + col, xv);
      if (recompute) {
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (xv[i] * sc[i] + sh[i] <= 0.f) av[i] = 0.f;
      } else if (kMask == 2) {
        const uint32_t bits = relu_mask[(r * c + col) >> 3];
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (!((bits >> i) & 1u)) av[i] = 0.f;
      } else if (relu) {
        float yv[V];
        LoadV<T, V>(y + r * c + col, yv);
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (yv[i] <= 0.f) av[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < V; ++i) {
        s0[i] += av[i];
        s1[i] += av[i] * (xv[i] - mu[i]) * is[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        s0[i] += av[i];
        s1[i] += av[i] * av[i];
      }
    }
  }
  // reduce over ty through shared memory: layout [ty][tx][2V]
  float* mine = smem + (ty * TX + tx) * 2 * V;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    mine[i]     = s0[i];
    mine[V + i] = s1[i];
  }
  __syncthreads();
  for (int h = TY / 2; h > 0; h >>= 1) {
    if (ty < h) {
      float* other = smem + ((ty + h) * TX + tx) * 2 * V;
#pragma unroll
      for (int i = 0; i < 2 * V; ++i) mine[i] += other[i];
    }
    __syncthreads();
  }
  if (ty == 0) {
    float* out = ws + static_cast<int64_t>(blockIdx.y) * 2 * c;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      out[col + i]     = mine[i];
      out[c + col + i] = mine[V + i];
    }
  }
}

// Sums the partial rows of the workspace for this thread's V channels. The
// threads of a block that share a column (same tx) split the partial rows
// between them and combine through shared memory ([ty][tx][2V] floats).
template <int V>
__device__ __forceinline__ void BlockCombine(const float* __restrict__ ws, int partials, int c, int col, float* smem,
                                             float (&s0)[V], float (&s1)[V]) {
  // The partial rows were summed by BnFinalizeKernel into the row after the last partial row.
  (void)smem;
  const float* total = ws + static_cast<int64_t>(partials) * 2 * c;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    s0[i] = total[col + i];
    s1[i] = total[c + col + i];
  }
}

// Sums the partial rows column-wise into row `partials` of the workspace. Block (32, 32): tx = column,
// ty = lane over the partial rows; consecutive threads read consecutive floats.
constexpr int kFinalizeRows = 32;
__global__ void __launch_bounds__(32 * kFinalizeRows) BnFinalizeKernel(float* __restrict__ ws, int partials, int c) {
  __shared__ float red[kFinalizeRows][33];
  const int col = blockIdx.x * 32 + threadIdx.x;  // 0 .. 2c-1 (sums and second sums side by side)
  float acc = 0.f;
  if (col < 2 * c)
    for (int p = threadIdx.y; p < partials; p += kFinalizeRows) acc += ws[static_cast<int64_t>(p) * 2 * c + col];
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < 2 * c) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kFinalizeRows; ++j) s += red[j][threadIdx.x];
    ws[static_cast<int64_t>(partials) * 2 * c + col] = s;
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256)
BnApplyKernel(const T* __restrict__ x, const T* __restrict__ residual, T* __restrict__ y,
              const float* __restrict__ gamma, const float* __restrict__ beta, float* running_mean, float* running_var,
              float* save_mean, float* save_invstd, const float* __restrict__ ws, int partials, int64_t m, int c,
              float eps, float momentum, int relu, int training, uint8_t* __restrict__ relu_mask = nullptr) {
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int TX = blockDim.x, TY = blockDim.y;
  const int col = (blockIdx.x * TX + tx) * V;
  extern __shared__ float smem[];
  float scale[V], shift[V], t0[V], t1[V];
  if (training) BlockCombine<V>(ws, partials, c, col, smem, t0, t1);
#pragma unroll
  for (int i = 0; i < V; ++i) {
    float mean, invstd;
    if (training) {
      mean      = t0[i] / static_cast<float>(m);
      float var = fmaxf(t1[i] / static_cast<float>(m) - mean * mean, 0.f);
      invstd    = rsqrtf(var + eps);
      if (blockIdx.y == 0 && ty == 0) {
        save_mean[col + i]   = mean;
        save_invstd[col + i] = invstd;
        if (running_mean) {
          float unbiased       = m > 1 ? var * static_cast<float>(m) / static_cast<float>(m - 1) : var;
          running_mean[col + i] = (1.f - momentum) * running_mean[col + i] + momentum * mean;
          running_var[col + i]  = (1.f - momentum) * running_var[col + i] + momentum * unbiased;
        }
      }
    } else {
      mean   = running_mean[col + i];
      invstd = rsqrtf(running_var[col + i] + eps);
    }
    scale[i] = gamma[col + i] * invstd;
    shift[i] = beta[col + i] - mean * scale[i];
  }
#pragma unroll 4
  for (int64_t r = static_cast<int64_t>(blockIdx.y) * TY + ty; r < m; r += static_cast<int64_t>(gridDim.y) * TY) {
    float xv[V];
    LoadV<T, V>(x + r * c + col, xv);
    if (residual) {
      float rv[V];
      LoadV<T, V>(residual + r * c + col, rv);
#pragma unroll
      for (int i = 0; i < V; ++i) xv[i] = xv[i] * scale[i] + shift[i] + rv[i];
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) xv[i] = xv[i] * scale[i] + shift[i];
    }
    if (relu) {
      if (V == 8 && relu_mask != nullptr) {  // one bit per element for the backward pass, instead of y
        uint32_t bits = 0;
#pragma unroll
        for (int i = 0; i < V; ++i) bits |= (xv[i] > 0.f ? 1u : 0u) << i;
        relu_mask[(r * c + col) >> 3] = static_cast<uint8_t>(bits);
      }
#pragma unroll
      for (int i = 0; i < V; ++i) xv[i] = fmaxf(xv[i], 0.f);
    }
    StoreV<T, V>(y + r * c + col, xv);
  }
}

template <typename T, int V, int kMask = 0>
__global__ void __launch_bounds__(256, 3)
BnBwdApplyKernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ y,
                 const float* __restrict__ gamma, const float* __restrict__ mean, const float* __restrict__ invstd,
                 T* __restrict__ dx, T* __restrict__ dres, float* dgamma, float* dbeta, const float* __restrict__ ws,
                 int partials, int64_t m, int c, int relu, const float* __restrict__ beta = nullptr,
                 const uint8_t* __restrict__ relu_mask = nullptr) {
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int TX = blockDim.x, TY = blockDim.y;
  const int col = (blockIdx.x * TX + tx) * V;
  extern __shared__ float smem[];
  float mu[V], is[V], k0[V], k1[V], gs[V], t0[V], t1[V], sh[V];
  const float inv_m = 1.f / static_cast<float>(m);
  constexpr bool recompute = kMask == 1;  // mask from x, as in the reduction kernel
  BlockCombine<V>(ws, partials, c, col, smem, t0, t1);
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const float s0 = t0[i], s1 = t1[i];
    if (blockIdx.y == 0 && ty == 0) {
      dbeta[col + i]  = s0;
      dgamma[col + i] = s1;
    }
    mu[i] = mean[col + i];
    is[i] = invstd[col + i];
    gs[i] = gamma[col + i] * is[i];
    sh[i] = recompute ? beta[col + i] - mu[i] * gs[i] : 0.f;
    k0[i] = s0 * inv_m;
    k1[i] = s1 * inv_m;
  }
#pragma unroll 4
  for (int64_t r = static_cast<int64_t>(blockIdx.y) * TY + ty; r < m; r += static_cast<int64_t>(gridDim.y) * TY) {
    float dv[V], xv[V];
    LoadV<T, V>(dy + r * c + col, dv);
    LoadV<T, V>(x + r * c + col, xv);
    if (recompute) {
#pragma unroll
      for (int i = 0; i < V; ++i)
        if (xv[i] * gs[i] + sh[i] <= 0.f) dv[i] = 0.f;
    } else if (kMask == 2) {
      const uint32_t bits = relu_mask[(r * c + col) >> 3];
#pragma unroll
      for (int i = 0; i < V; ++i)
        if (!((bits >> i) & 1u)) dv[i] = 0.f;
    } else if (relu) {
      float yv[V];
      LoadV<T, V>(y + r * c + col, yv);
#pragma unroll
      for (int i = 0; i < V; ++i)
        if (yv[i] <= 0.f) dv[i] = 0.f;
    }
    if (dres) StoreV<T, V>(dres + r * c + col, dv);
#pragma unroll
    for (int i = 0; i < V; ++i) dv[i] = gs[i] * (dv[i] - k0[i] - (xv[i] - mu[i]) * is[i] * k1[i]);
    StoreV<T, V>(dx + r * c + col, dv);
  }
}

int BnVec(int dtype, int c) {
  int v = dtype == kF32 ? 4 : 8;
  while (v > 1 && c % v != 0) v /= 2;
  return v;
}

#define BN_DISPATCH(dtype, c, ...)                                                    \
  {                                                                                   \
    const int v_ = BnVec(dtype, c);                                                   \
    if (dtype == kBF16) {                                                             \
      using T = __nv_bfloat16;                                                        \
      if (v_ == 8) { constexpr int V = 8; __VA_ARGS__; }                              \
      else if (v_ == 4) { constexpr int V = 4; __VA_ARGS__; }                         \
      else if (v_ == 2) { constexpr int V = 2; __VA_ARGS__; }                         \
      else { constexpr int V = 1; __VA_ARGS__; }                                      \
    } else if (dtype == kF16) {                                                       \
      using T = __half;                                                               \
      if (v_ == 8) { constexpr int V = 8; __VA_ARGS__; }                              \
      else if (v_ == 4) { constexpr int V = 4; __VA_ARGS__; }                         \
      else if (v_ == 2) { constexpr int V = 2; __VA_ARGS__; }                         \
      else { constexpr int V = 1; __VA_ARGS__; }                                      \
    } else if (dtype == kF32) {                                                       \
      using T = float;                                                                \
      if (v_ == 4) { constexpr int V = 4; __VA_ARGS__; }                              \
      else if (v_ == 2) { constexpr int V = 2; __VA_ARGS__; }                         \
      else { constexpr int V = 1; __VA_ARGS__; }                                      \
    } else {                                                                          \
      return SetError(-2, "batch norm: unsupported dtype");                           \
    }                                                                                 \
  }

}  // namespace
}  // namespace tipsk

using namespace tipsk;

extern "C" {

int tipsk_bn_partials(int64_t m, int c) {
  // Upper bound over the vector widths the dispatcher may choose.
  int best = 1;
  for (int v = 1; v <= 8; v *= 2)
    if (c % v == 0) {
      int p = BnGeometry(m, c, v).partials;
      if (p > best) best = p;
    }
  return best + 1;  // one more row: the column sums of the partial rows
}

int tipsk_bn_fwd_train(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                       float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                       float* workspace, int64_t m, int c, float eps, float momentum, int relu, int dtype,
                       void* stream) {
  TIPSK_REQUIRE(m > 0 && c > 0, "batch norm: empty input");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  BN_DISPATCH(dtype, c, {
    BnGeom g = BnGeometry(m, c, V);
    dim3 block(g.tx, g.ty), grid(g.col_tiles, g.partials);
    size_t smem = sizeof(float) * 256 * 2 * V;
    BnReduceKernel<T, V, false><<<grid, block, smem, s>>>(static_cast<const T*>(x), nullptr, nullptr, nullptr, nullptr,
                                                          workspace, m, c, 0);
    BnFinalizeKernel<<<CeilDiv(2 * c, 32), dim3(32, kFinalizeRows), 0, s>>>(workspace, g.partials, c);
    BnApplyKernel<T, V><<<dim3(g.col_tiles, g.fwd_rows), block, sizeof(float) * 256 * 2 * V, s>>>(static_cast<const T*>(x), static_cast<const T*>(residual),
                                               static_cast<T*>(y), gamma, beta, running_mean, running_var, save_mean,
                                               save_invstd, workspace, g.partials, m, c, eps, momentum, relu, 1);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* Training forward when the per-channel sum and sum of squares of x are already known (`stats` = fp32 [2, C]:
 * sums, then sums of squares; the convolution epilogue produces them): only the apply pass runs. */
int tipsk_bn_fwd_train_stats(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                             float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                             const float* stats, int64_t m, int c, float eps, float momentum, int relu, int dtype,
                             void* stream) {
  TIPSK_REQUIRE(m > 0 && c > 0, "batch norm: empty input");
  TIPSK_REQUIRE(stats != nullptr, "batch norm: statistics buffer is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  BN_DISPATCH(dtype, c, {
    BnGeom g = BnGeometry(m, c, V);
    dim3 block(g.tx, g.ty), grid(g.col_tiles, g.partials);
    BnApplyKernel<T, V><<<dim3(g.col_tiles, g.fwd_rows), block, sizeof(float) * 256 * 2 * V, s>>>(static_cast<const T*>(x), static_cast<const T*>(residual),
                                               static_cast<T*>(y), gamma, beta, running_mean, running_var, save_mean,
                                               save_invstd, stats, 0, m, c, eps, momentum, relu, 1);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_bn_fwd_eval(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                      const float* running_mean, const float* running_var, int64_t m, int c, float eps, int relu,
                      int dtype, void* stream) {
  TIPSK_REQUIRE(m > 0 && c > 0, "batch norm: empty input");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  BN_DISPATCH(dtype, c, {
    BnGeom g = BnGeometry(m, c, V);
    dim3 block(g.tx, g.ty), grid(g.col_tiles, g.partials);
    BnApplyKernel<T, V><<<dim3(g.col_tiles, g.fwd_rows), block, sizeof(float) * 256 * 2 * V, s>>>(static_cast<const T*>(x), static_cast<const T*>(residual),
                                               static_cast<T*>(y), gamma, beta, const_cast<float*>(running_mean),
                                               const_cast<float*>(running_var), nullptr, nullptr, nullptr, 0, m, c,
                                               eps, 0.f, relu, 0);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_bn_bwd(const void* dy, const void* x, const void* y, const float* gamma, const float* save_mean,
                 const float* save_invstd, void* dx, void* dresidual, float* dgamma, float* dbeta, float* workspace,
                 int64_t m, int c, int relu, int dtype, void* stream) {
  TIPSK_REQUIRE(m > 0 && c > 0, "batch norm: empty input");
  TIPSK_REQUIRE(!relu || y, "batch norm backward with ReLU needs the forward output");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  BN_DISPATCH(dtype, c, {
    BnGeom g = BnGeometry(m, c, V);
    dim3 block(g.tx, g.ty), grid(g.col_tiles, g.partials);
    size_t smem = sizeof(float) * 256 * 2 * V;
    BnReduceKernel<T, V, true><<<grid, block, smem, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x),
                                                         static_cast<const T*>(y), save_mean, save_invstd, workspace, m,
                                                         c, relu);
    BnFinalizeKernel<<<CeilDiv(2 * c, 32), dim3(32, kFinalizeRows), 0, s>>>(workspace, g.partials, c);
    BnBwdApplyKernel<T, V><<<grid, block, smem, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x),
                                                  static_cast<const T*>(y), gamma, save_mean, save_invstd,
                                                  static_cast<T*>(dx), static_cast<T*>(dresidual), dgamma, dbeta,
                                                  workspace, g.partials, m, c, relu);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* Training forward that also writes the ReLU bit mask (uint8 [M * C / 8]; needs C % 8 == 0 and a 16-bit dtype) for
 * tipsk_bn_bwd_bitmask.  `stats` (fp32 [2, C]) may be null: then the statistics are reduced here into `workspace`. */
int tipsk_bn_fwd_train_mask(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                            float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                            float* workspace, const float* stats, void* relu_mask, int64_t m, int c, float eps,
                            float momentum, int relu, int dtype, void* stream) {
  TIPSK_REQUIRE(m > 0 && c > 0, "batch norm: empty input");
  TIPSK_REQUIRE(stats != nullptr || workspace != nullptr, "batch norm: statistics or a workspace are required");
  TIPSK_REQUIRE(relu_mask == nullptr || (c % 8 == 0 && dtype != kF32), "batch norm: the bit mask needs C % 8 == 0");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  BN_DISPATCH(dtype, c, {
    BnGeom g = BnGeometry(m, c, V);
    dim3 block(g.tx, g.ty), grid(g.col_tiles, g.partials);
    size_t smem = sizeof(float) * 256 * 2 * V;
    if (stats == nullptr) {
      BnReduceKernel<T, V, false><<<grid, block, smem, s>>>(static_cast<const T*>(x), nullptr, nullptr, nullptr, nullptr,
                                                            workspace, m, c, 0);
      BnFinalizeKernel<<<CeilDiv(2 * c, 32), dim3(32, kFinalizeRows), 0, s>>>(workspace, g.partials, c);
    }
    BnApplyKernel<T, V><<<dim3(g.col_tiles, g.fwd_rows), block, smem, s>>>(static_cast<const T*>(x), static_cast<const T*>(residual),
                                                  static_cast<T*>(y), gamma, beta, running_mean, running_var, save_mean,
                                                  save_invstd, stats ? stats : workspace, stats ? 0 : g.partials, m, c,
                                                  eps, momentum, relu, 1, static_cast<uint8_t*>(relu_mask));
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* Backward of BN (+ residual) + ReLU with the mask taken from the bit mask of tipsk_bn_fwd_train_mask. */
int tipsk_bn_bwd_bitmask(const void* dy, const void* x, const void* relu_mask, const float* gamma,
                         const float* save_mean, const float* save_invstd, void* dx, void* dresidual, float* dgamma,
                         float* dbeta, float* workspace, int64_t m, int c, int dtype, void* stream) {
  TIPSK_REQUIRE(m > 0 && c > 0, "batch norm: empty input");
  TIPSK_REQUIRE(relu_mask != nullptr && c % 8 == 0 && dtype != kF32, "batch norm: bit mask missing or C % 8 != 0");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  BN_DISPATCH(dtype, c, {
    BnGeom g = BnGeometry(m, c, V);
    dim3 block(g.tx, g.ty), grid(g.col_tiles, g.partials);
    size_t smem = sizeof(float) * 256 * 2 * V;
    BnReduceKernel<T, V, true, 2><<<grid, block, smem, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x), nullptr,
                                                            save_mean, save_invstd, workspace, m, c, 1, nullptr, nullptr,
                                                            static_cast<const uint8_t*>(relu_mask));
    BnFinalizeKernel<<<CeilDiv(2 * c, 32), dim3(32, kFinalizeRows), 0, s>>>(workspace, g.partials, c);
    BnBwdApplyKernel<T, V, 2><<<grid, block, smem, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x), nullptr, gamma,
                                                     save_mean, save_invstd, static_cast<T*>(dx),
                                                     static_cast<T*>(dresidual), dgamma, dbeta, workspace, g.partials, m,
                                                     c, 1, nullptr, static_cast<const uint8_t*>(relu_mask));
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* Backward of BN + ReLU (no residual) that rebuilds the ReLU mask from x, gamma, beta and the saved statistics
 * instead of reading the forward output: one activation read fewer in each of its two passes. */
int tipsk_bn_bwd_relu_recompute(const void* dy, const void* x, const float* gamma, const float* beta,
                                const float* save_mean, const float* save_invstd, void* dx, float* dgamma, float* dbeta,
                                float* workspace, int64_t m, int c, int dtype, void* stream) {
  TIPSK_REQUIRE(m > 0 && c > 0, "batch norm: empty input");
  TIPSK_REQUIRE(beta != nullptr && gamma != nullptr, "batch norm backward: gamma and beta are required");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  BN_DISPATCH(dtype, c, {
    BnGeom g = BnGeometry(m, c, V);
    dim3 block(g.tx, g.ty), grid(g.col_tiles, g.partials);
    size_t smem = sizeof(float) * 256 * 2 * V;
    BnReduceKernel<T, V, true, 1><<<grid, block, smem, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x),
                                                               nullptr, save_mean, save_invstd, workspace, m, c, 1,
                                                               gamma, beta);
    BnFinalizeKernel<<<CeilDiv(2 * c, 32), dim3(32, kFinalizeRows), 0, s>>>(workspace, g.partials, c);
    BnBwdApplyKernel<T, V, 1><<<grid, block, smem, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x), nullptr,
                                                        gamma, save_mean, save_invstd, static_cast<T*>(dx), nullptr,
                                                        dgamma, dbeta, workspace, g.partials, m, c, 1, beta);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Batch-norm forward for callers that cannot allocate: the partial-sum scratch is a fixed array in
// the device image of this library.  See kernels/tips_noalloc.h for the contract.
#include <mutex>

#include "kernels/tips_noalloc.h"

namespace {

static __device__ __align__(256) float g_bn_noalloc_scratch[TIPSK_BN_NOALLOC_SCRATCH_FLOATS];

constexpr int kNoAllocMaxDevices = 64;
float* g_bn_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
std::mutex g_bn_noalloc_mu;

// Device address of the scratch array on the current device.  In host code the array's name is only a
// stand-in for the symbol; the address a kernel can use comes from cudaGetSymbolAddress.
int BnNoAllocScratch(float** out) {
  int dev = 0;
  TIPSK_CUDA(cudaGetDevice(&dev));
  TIPSK_REQUIRE(dev >= 0 && dev < kNoAllocMaxDevices, "bn_noalloc: device index out of range");
  std::lock_guard<std::mutex> lock(g_bn_noalloc_mu);
  if (!g_bn_noalloc_ptr[dev]) {
    float* ptr = nullptr;
    TIPSK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_bn_noalloc_scratch));
    TIPSK_REQUIRE(ptr != nullptr, "bn_noalloc: the scratch symbol has no device address");
    g_bn_noalloc_ptr[dev] = ptr;
  }
  *out = g_bn_noalloc_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int tipsk_bn_fwd_train_noalloc(const void* x, const void* residual, void* y, const float* gamma,
                                          const float* beta, float* running_mean, float* running_var,
                                          float* save_mean, float* save_invstd, int64_t m, int c, float eps,
                                          float momentum, int relu, int dtype, void* stream) {
  TIPSK_REQUIRE(m > 0 && c > 0, "bn_noalloc: empty input");
  const int64_t need = 2ll * c * tipsk_bn_partials(m, c);
  if (need > TIPSK_BN_NOALLOC_SCRATCH_FLOATS)
    return SetError(-2, "bn_noalloc: needs " + std::to_string(need) + " scratch floats, the built-in array holds " +
                            std::to_string(TIPSK_BN_NOALLOC_SCRATCH_FLOATS) + "; use tipsk_bn_fwd_train with a workspace");
  float* scratch = nullptr;
  int rc = BnNoAllocScratch(&scratch);
  if (rc) return rc;
  return tipsk_bn_fwd_train(x, residual, y, gamma, beta, running_mean, running_var, save_mean, save_invstd, scratch, m,
                            c, eps, momentum, relu, dtype, stream);
}
