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
    const int64_t step = static_cast<int64_t>(gridDim.y) * 8;
    for (int64_t r = static_cast<int64_t>(blockIdx.y) * 8 + threadIdx.y; r < rows; r += 2 * step) {
      // two rows in flight per thread
      const int64_t off[2] = {r * cols + static_cast<int64_t>(vc) * N, (r + step) * cols + static_cast<int64_t>(vc) * N};
      const bool have[2]   = {true, r + step < rows};
      Vec16<T> d[2], q[2];
#pragma unroll
      for (int u = 0; u < 2; ++u)
        if (have[u]) {
          d[u] = LoadVec(dy + off[u]);
          if (act != 0) q[u] = LoadVec(x + off[u]);
        }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (!have[u]) continue;
        Vec16<T> o;
        if (act != 0) {
#pragma unroll
          for (int k = 0; k < N; ++k) {
            const float g = ToFloat<T>(d[u].v[k]) * ActGrad(ToFloat<T>(q[u].v[k]) + bv[k], act);
            acc[k] += g;
            o.v[k] = FromFloat<T>(g);
          }
        } else {
#pragma unroll
          for (int k = 0; k < N; ++k) {
            acc[k] += ToFloat<T>(d[u].v[k]);
            o.v[k] = d[u].v[k];
          }
        }
        if (dx) StoreVec(dx + off[u], o);
      }
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

// Output layer with one unit fused with its loss: z_i = x_i . w + b, loss = sum_i BCE(z_i, t_i), and
// dz_i = (sigmoid(z_i) - t_i) * scale kept for the backward pass.  A GEMM with one output column wastes a
// 128-wide tensor-core tile on it; this is a streaming dot product per row (one warp per row, 16-byte loads).
template <typename T>
__global__ void __launch_bounds__(256)
DotSigmoidBceFwdKernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                       const float* __restrict__ t, float* __restrict__ loss_sum, float* __restrict__ dz,
                       float* __restrict__ logits, int64_t rows, int k, int64_t ldx, float scale) {
  constexpr int N = 16 / sizeof(T);
  __shared__ float warp_sums[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float b  = bias ? ToFloat<T>(bias[0]) : 0.f;
  float local    = 0.f;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + warp; r < rows; r += static_cast<int64_t>(gridDim.x) * 8) {
    const T* row = x + r * ldx;
    float acc    = 0.f;
    for (int c = lane * N; c < k; c += 32 * N) {
      const Vec16<T> xv = LoadVec(row + c), wv = LoadVec(w + c);
#pragma unroll
      for (int j = 0; j < N; ++j) acc += ToFloat<T>(xv.v[j]) * ToFloat<T>(wv.v[j]);
    }
    acc = WarpSum(acc);
    if (lane == 0) {
      const float z = acc + b, ti = t[r];
      local += fmaxf(z, 0.f) - z * ti + log1pf(__expf(-fabsf(z)));
      dz[r] = (1.f / (1.f + __expf(-z)) - ti) * scale;
      if (logits) logits[r] = z;
    }
  }
  if (lane == 0) warp_sums[warp] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) v += warp_sums[j];
    atomicAdd(loss_sum, v * scale);
  }
}

// Backward of the same layer: g_i = dz_i * dloss; dx_i = g_i * w; dw = sum_i g_i * x_i; db = sum_i g_i.
// A block owns a run of rows and 32 * N columns per pass; its warps keep the dw partial sums of their rows in
// registers, the block adds them up in shared memory and issues one atomic per column.
template <typename T>
__global__ void __launch_bounds__(256)
DotSigmoidBceBwdKernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ dz,
                       const float* __restrict__ dloss, T* __restrict__ dx, float* __restrict__ dw,
                       float* __restrict__ db, int64_t rows, int k, int64_t ldx, int64_t rows_per_block) {
  constexpr int N = 16 / sizeof(T);
  __shared__ float red[8][32 * N + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float up = dloss ? *dloss : 1.f;
  const int64_t r0 = static_cast<int64_t>(blockIdx.x) * rows_per_block;
  const int64_t r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  for (int c0 = 0; c0 < k; c0 += 32 * N) {
    const int c       = c0 + lane * N;
    const bool active = c < k;
    Vec16<T> wv;
    if (active) wv = LoadVec(w + c);
    float acc[N];
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = 0.f;
    float gsum = 0.f;
    for (int64_t r = r0 + warp; r < r1; r += 8) {
      const float g = dz[r] * up;
      gsum += g;
      if (active) {
        const Vec16<T> xv = LoadVec(x + r * ldx + c);
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < N; ++j) {
          acc[j] += g * ToFloat<T>(xv.v[j]);
          o.v[j] = FromFloat<T>(g * ToFloat<T>(wv.v[j]));
        }
        StoreVec(dx + r * k + c, o);
      }
    }
#pragma unroll
    for (int j = 0; j < N; ++j) red[warp][lane * N + j] = acc[j];
    __syncthreads();
    for (int col = threadIdx.x; col < 32 * N; col += blockDim.x) {
      if (c0 + col >= k) continue;
      float v = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v += red[j][col];
      atomicAdd(dw + c0 + col, v);
    }
    if (c0 == 0 && db && lane == 0) atomicAdd(db, gsum);
    __syncthreads();
  }
}

// Input embedding of a transformer encoder: x[t, :] = tok[ids[t], :] + pos[t mod seq, :] + typ[:], one warp per
// token, 16-byte vectors.  Backward: the token-table gradient is a scatter-add of the rows of dx (packed bf16x2 /
// fp32 atomics into a zeroed table-sized buffer; a token id repeats a few times per batch at most), the position
// gradient sums dx over the batch in fp32 (one thread per (position, 8 columns), no atomics), the type gradient
// is the column sum of the position gradient.
template <typename T>
__global__ void __launch_bounds__(256)
EmbedSumFwdKernel(const int64_t* __restrict__ ids, const T* __restrict__ tok, const T* __restrict__ pos,
                  const T* __restrict__ typ, T* __restrict__ x, int64_t tokens, int seq, int hidden, int64_t vocab) {
  constexpr int N = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t warp  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarp = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t t = warp; t < tokens; t += nwarp) {
    int64_t id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    const T* a = tok + id * hidden;
    const T* b = pos + static_cast<int64_t>(t % seq) * hidden;
    for (int c = lane * N; c < hidden; c += 32 * N) {
      const Vec16<T> va = LoadVec(a + c), vb = LoadVec(b + c), vc = LoadVec(typ + c);
      Vec16<T> o;
#pragma unroll
      for (int j = 0; j < N; ++j) o.v[j] = FromFloat<T>(ToFloat<T>(va.v[j]) + ToFloat<T>(vb.v[j]) + ToFloat<T>(vc.v[j]));
      StoreVec(x + t * hidden + c, o);
    }
  }
}

template <typename T>
__device__ __forceinline__ void AtomicAddPair(T* addr, T a, T b);
template <>
__device__ __forceinline__ void AtomicAddPair<float>(float* addr, float a, float b) {
  atomicAdd(addr, a);
  atomicAdd(addr + 1, b);
}
template <>
__device__ __forceinline__ void AtomicAddPair<__nv_bfloat16>(__nv_bfloat16* addr, __nv_bfloat16 a, __nv_bfloat16 b) {
  atomicAdd(reinterpret_cast<__nv_bfloat162*>(addr), __halves2bfloat162(a, b));
}
template <>
__device__ __forceinline__ void AtomicAddPair<__half>(__half* addr, __half a, __half b) {
  atomicAdd(reinterpret_cast<__half2*>(addr), __halves2half2(a, b));
}

template <typename T>
__global__ void __launch_bounds__(256)
EmbedTokBwdKernel(const int64_t* __restrict__ ids, const T* __restrict__ dx, T* __restrict__ dtok, int64_t tokens,
                  int hidden, int64_t vocab) {
  constexpr int N = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t warp  = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarp = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t t = warp; t < tokens; t += nwarp) {
    const int64_t id = ids[t];
    if (id < 0 || id >= vocab) continue;
    T* row = dtok + id * hidden;
    for (int c = lane * N; c < hidden; c += 32 * N) {
      const Vec16<T> g = LoadVec(dx + t * hidden + c);
#pragma unroll
      for (int j = 0; j < N; j += 2) AtomicAddPair<T>(row + c + j, g.v[j], g.v[j + 1]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
EmbedPosBwdKernel(const T* __restrict__ dx, T* __restrict__ dpos, int64_t batch, int seq, int hidden) {
  constexpr int N = 16 / sizeof(T);
  const int cv = hidden / N;
  const int64_t total = static_cast<int64_t>(seq) * cv;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % cv) * N;
    const int s = static_cast<int>(i / cv);
    float acc[N];
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = 0.f;
    for (int64_t b = 0; b < batch; ++b) {
      const Vec16<T> g = LoadVec(dx + (b * seq + s) * hidden + c);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] += ToFloat<T>(g.v[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < N; ++j) o.v[j] = FromFloat<T>(acc[j]);
    StoreVec(dpos + static_cast<int64_t>(s) * hidden + c, o);
  }
}

// dtyp[c] = sum over the positions of dpos[s, c] (fp32 accumulation), one thread per column.
template <typename T>
__global__ void __launch_bounds__(256)
EmbedTypBwdKernel(const T* __restrict__ dpos, T* __restrict__ dtyp, int seq, int hidden) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= hidden) return;
  float acc = 0.f;
  for (int s = 0; s < seq; ++s) acc += ToFloat<T>(dpos[static_cast<int64_t>(s) * hidden + c]);
  dtyp[c] = FromFloat<T>(acc);
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
  // about four blocks per SM, but at least 8 row iterations per thread: every partition ends in one atomic per
  // column, and a short tensor cut into hundreds of partitions spends its time in those
  int parts = CeilDiv(NumSMs() * 4, col_tiles);
  int maxp  = CeilDiv(rows, 8 * 8);
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

/* One-unit output layer fused with its loss.  x: [rows, k] with pitch ldx, w: [k], bias: [1] or null, targets:
 * [rows] fp32.  loss_sum (fp32 scalar, zeroed here) receives scale * sum of the per-row binary cross-entropies,
 * dz [rows] fp32 the gradient of that sum with respect to the logits, logits (optional, [rows] fp32) the logits. */
int tipsk_dot_sigmoid_bce_fwd(const void* x, const void* w, const void* bias, const float* targets, float* loss_sum,
                              float* dz, float* logits, int64_t rows, int k, int64_t ldx, float scale, int dtype,
                              void* stream) {
  if (rows <= 0) return 0;
  const int n = 16 / (int)DTypeSize(dtype);
  TIPSK_REQUIRE(k % n == 0 && ldx % n == 0, "dot_sigmoid_bce: k and the row pitch must be multiples of 16 bytes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TIPSK_CUDA(cudaMemsetAsync(loss_sum, 0, sizeof(float), s));
  int grid = CeilDiv(rows, 8);
  if (grid > NumSMs() * 8) grid = NumSMs() * 8;
  EPI_DISPATCH(dtype, {
    DotSigmoidBceFwdKernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(w),
                                                   static_cast<const T*>(bias), targets, loss_sum, dz, logits, rows, k,
                                                   ldx, scale);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* dx: [rows, k] (contiguous) = dz * dloss * w; dw: [k] fp32 and db: [1] fp32 (may be null), both zeroed here;
 * dloss: device scalar (null = 1). */
int tipsk_dot_sigmoid_bce_bwd(const void* x, const void* w, const float* dz, const float* dloss, void* dx, float* dw,
                              float* db, int64_t rows, int k, int64_t ldx, int dtype, void* stream) {
  if (rows <= 0) return 0;
  const int n = 16 / (int)DTypeSize(dtype);
  TIPSK_REQUIRE(k % n == 0 && ldx % n == 0, "dot_sigmoid_bce: k and the row pitch must be multiples of 16 bytes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TIPSK_CUDA(cudaMemsetAsync(dw, 0, sizeof(float) * k, s));
  if (db) TIPSK_CUDA(cudaMemsetAsync(db, 0, sizeof(float), s));
  int blocks = NumSMs() * 2;
  int64_t rpb = (rows + blocks - 1) / blocks;
  rpb         = (rpb + 7) / 8 * 8;
  blocks      = CeilDiv(rows, rpb);
  EPI_DISPATCH(dtype, {
    DotSigmoidBceBwdKernel<T><<<blocks, 256, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(w), dz, dloss,
                                                     static_cast<T*>(dx), dw, db, rows, k, ldx, rpb);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* x[t] = tok[ids[t]] + pos[t mod seq] + typ for t < tokens (ids laid out [batch, seq]); hidden a multiple of 16
 * bytes; ids outside [0, vocab) read row 0 and get no gradient. */
int tipsk_embed_sum_fwd(const int64_t* ids, const void* tok, const void* pos, const void* typ, void* x, int64_t tokens,
                        int seq, int hidden, int64_t vocab, int dtype, void* stream) {
  if (tokens <= 0) return 0;
  TIPSK_REQUIRE(hidden % (16 / (int)DTypeSize(dtype)) == 0 && seq >= 1, "embed: hidden must be a multiple of 16 bytes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int grid = CeilDiv(tokens, 8);
  if (grid > NumSMs() * 8) grid = NumSMs() * 8;
  EPI_DISPATCH(dtype, {
    EmbedSumFwdKernel<T><<<grid, 256, 0, s>>>(ids, static_cast<const T*>(tok), static_cast<const T*>(pos),
                                              static_cast<const T*>(typ), static_cast<T*>(x), tokens, seq, hidden, vocab);
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* dtok [vocab, hidden] (zeroed here), dpos [seq, hidden], dtyp [hidden]; tokens = batch * seq. */
int tipsk_embed_sum_bwd(const int64_t* ids, const void* dx, void* dtok, void* dpos, void* dtyp, int64_t tokens, int seq,
                        int hidden, int64_t vocab, int dtype, void* stream) {
  if (tokens <= 0) return 0;
  const int n = 16 / (int)DTypeSize(dtype);
  TIPSK_REQUIRE(hidden % n == 0 && seq >= 1 && tokens % seq == 0, "embed: hidden must be a multiple of 16 bytes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TIPSK_CUDA(cudaMemsetAsync(dtok, 0, static_cast<size_t>(vocab) * hidden * DTypeSize(dtype), s));
  int grid = CeilDiv(tokens, 8);
  if (grid > NumSMs() * 8) grid = NumSMs() * 8;
  const int64_t pos_items = static_cast<int64_t>(seq) * (hidden / n);
  int pgrid = CeilDiv(pos_items, 256);
  if (pgrid > NumSMs() * 8) pgrid = NumSMs() * 8;
  EPI_DISPATCH(dtype, {
    EmbedTokBwdKernel<T><<<grid, 256, 0, s>>>(ids, static_cast<const T*>(dx), static_cast<T*>(dtok), tokens, hidden, vocab);
    EmbedPosBwdKernel<T><<<pgrid, 256, 0, s>>>(static_cast<const T*>(dx), static_cast<T*>(dpos), tokens / seq, seq, hidden);
    EmbedTypBwdKernel<T><<<CeilDiv(hidden, 256), 256, 0, s>>>(static_cast<const T*>(dpos), static_cast<T*>(dtyp), seq, hidden);
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
