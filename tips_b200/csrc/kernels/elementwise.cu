// HBM-bound elementwise kernels: fused optimizers (SGD-momentum, Adam/AdamW) on
// flat parameter slabs and on tensor lists, gradient pack / unpack between
// tensor lists and a flat fusion bucket (with scale, cast and accumulate), and
// scale+cast.
//
// The reference has none of these: its only math kernel is the elementwise
// Vec::Mul loop used by the server-side update (tips/core/common/vec.h:194-216)
// and gradient accumulation / averaging are TensorFlow ops
// (tips/tensorflow/gradient_aggregation_eager.py:74, gradient_aggregation.py:166-173).
// Here one launch covers a whole bucket: every element is read once and written
// once, in 16-byte vectors, so the kernels run at HBM speed.
#include "kernels/common.cuh"
#include "kernels/optim_rules.cuh"
#include "kernels/tips_kernels.h"

namespace tipsk {

std::string& LastError() {
  static thread_local std::string err;
  return err;
}
int SetError(int code, const std::string& msg) {
  LastError() = msg;
  return code;
}
int NumSMs() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

namespace {

constexpr int kThreads = 256;

template <typename T>
struct alignas(sizeof(T) * 4) Quad {  // four consecutive elements of T
  T v[4];
};

template <typename T>
__device__ __forceinline__ void Load4(const T* p, float (&out)[4]) {
  Quad<T> q = *reinterpret_cast<const Quad<T>*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = ToFloat<T>(q.v[i]);
}
template <typename T>
__device__ __forceinline__ void Store4(T* p, const float (&in)[4]) {
  Quad<T> q;
#pragma unroll
  for (int i = 0; i < 4; ++i) q.v[i] = FromFloat<T>(in[i]);
  *reinterpret_cast<Quad<T>*>(p) = q;
}

template <typename G, typename P16>
__global__ void __launch_bounds__(kThreads)
SgdFlatKernel(float* __restrict__ p32, P16* __restrict__ p16, const G* __restrict__ g, float* __restrict__ m,
              int64_t n, SgdParams a) {
  const int64_t nvec   = n / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float pv[4], gv[4], mv[4];
    Load4(p32 + i * 4, pv);
    Load4(g + i * 4, gv);
    if (a.momentum != 0.f && !a.first_step) Load4(m + i * 4, mv);
#pragma unroll
    for (int k = 0; k < 4; ++k) SgdUpdate(pv[k], mv[k], gv[k], a);
    Store4(p32 + i * 4, pv);
    if (a.momentum != 0.f) Store4(m + i * 4, mv);
    if (p16) Store4(p16 + i * 4, pv);
  }
  // tail
  const int64_t t = nvec * 4 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t < n) {
    float p = p32[t], mm = (a.momentum != 0.f && !a.first_step) ? m[t] : 0.f;
    SgdUpdate(p, mm, ToFloat<G>(g[t]), a);
    p32[t] = p;
    if (a.momentum != 0.f) m[t] = mm;
    if (p16) p16[t] = FromFloat<P16>(p);
  }
}

template <typename G, typename P16>
__global__ void __launch_bounds__(kThreads)
AdamFlatKernel(float* __restrict__ p32, P16* __restrict__ p16, const G* __restrict__ g, float* __restrict__ m,
               float* __restrict__ v, int64_t n, AdamParams a) {
  if (a.step_dev) {
    const float step = static_cast<float>(*a.step_dev);
    a.bias1 = 1.f - powf(a.beta1, step);
    a.bias2 = 1.f - powf(a.beta2, step);
  }
  const int64_t nvec   = n / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float pv[4], gv[4], mv[4], vv[4];
    Load4(p32 + i * 4, pv);
    Load4(g + i * 4, gv);
    Load4(m + i * 4, mv);
    Load4(v + i * 4, vv);
#pragma unroll
    for (int k = 0; k < 4; ++k) AdamUpdate(pv[k], mv[k], vv[k], gv[k], a);
    Store4(p32 + i * 4, pv);
    Store4(m + i * 4, mv);
    Store4(v + i * 4, vv);
    if (p16) Store4(p16 + i * 4, pv);
  }
  const int64_t t = nvec * 4 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t < n) {
    float p = p32[t], mm = m[t], vv = v[t];
    AdamUpdate(p, mm, vv, ToFloat<G>(g[t]), a);
    p32[t] = p;
    m[t]   = mm;
    v[t]   = vv;
    if (p16) p16[t] = FromFloat<P16>(p);
  }
}

int FlatGrid(int64_t n) {
  int64_t blocks = (n / 4 + kThreads - 1) / kThreads;
  int64_t cap    = static_cast<int64_t>(NumSMs()) * 8;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

// ---- pack / unpack ------------------------------------------------------------

constexpr int kMaxList = 96;
struct ListArgs {
  const void* ptr[kMaxList];
  int64_t offset[kMaxList];  // element offset inside the flat buffer
  int64_t numel[kMaxList];
};

// mode 0: flat = scale * src ; mode 1: flat += scale * src ; mode 2: dst = scale * flat (unpack)
template <typename S, typename D, int kMode>
__global__ void __launch_bounds__(kThreads) PackKernel(ListArgs args, void* flat_v, float scale) {
  const int t       = blockIdx.y;
  const int64_t n   = args.numel[t];
  const int64_t off = args.offset[t];
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (kMode == 2) {
    const S* flat = static_cast<const S*>(flat_v) + off;
    D* dst        = static_cast<D*>(const_cast<void*>(args.ptr[t]));
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
      dst[i] = FromFloat<D>(ToFloat<S>(flat[i]) * scale);
  } else {
    const S* src = static_cast<const S*>(args.ptr[t]);
    D* flat      = static_cast<D*>(flat_v) + off;
    const bool aligned = ((reinterpret_cast<uintptr_t>(src) % (4 * sizeof(S))) == 0) &&
                         ((reinterpret_cast<uintptr_t>(flat) % (4 * sizeof(D))) == 0);
    if (aligned) {
      const int64_t nvec = n / 4;
      for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        float s[4];
        Load4(src + i * 4, s);
        if (kMode == 1) {
          float d[4];
          Load4(flat + i * 4, d);
#pragma unroll
          for (int k = 0; k < 4; ++k) s[k] = d[k] + s[k] * scale;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) s[k] *= scale;
        }
        Store4(flat + i * 4, s);
      }
      const int64_t i = nvec * 4 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
      if (i < n) {
        float s = ToFloat<S>(src[i]) * scale;
        if (kMode == 1) s += ToFloat<D>(flat[i]);
        flat[i] = FromFloat<D>(s);
      }
    } else {
      for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float s = ToFloat<S>(src[i]) * scale;
        if (kMode == 1) s += ToFloat<D>(flat[i]);
        flat[i] = FromFloat<D>(s);
      }
    }
  }
}

template <typename S, typename D>
int LaunchPack(int mode, const void* const* ptrs, const int64_t* offsets, const int64_t* numels, int n, void* flat,
               float scale, cudaStream_t stream) {
  for (int base = 0; base < n; base += kMaxList) {
    ListArgs a;
    int cnt         = n - base < kMaxList ? n - base : kMaxList;
    int64_t largest = 1;
    for (int i = 0; i < cnt; ++i) {
      a.ptr[i]    = ptrs[base + i];
      a.offset[i] = offsets[base + i];
      a.numel[i]  = numels[base + i];
      if (numels[base + i] > largest) largest = numels[base + i];
    }
    int gx = CeilDiv(largest, kThreads * 4 * 4);
    if (gx > 64) gx = 64;
    if (gx < 1) gx = 1;
    dim3 grid(gx, cnt);
    if (mode == 0)
      PackKernel<S, D, 0><<<grid, kThreads, 0, stream>>>(a, flat, scale);
    else if (mode == 1)
      PackKernel<S, D, 1><<<grid, kThreads, 0, stream>>>(a, flat, scale);
    else
      PackKernel<S, D, 2><<<grid, kThreads, 0, stream>>>(a, flat, scale);
    TIPSK_LAUNCH_CHECK();
  }
  return 0;
}

template <typename S, typename D>
__global__ void __launch_bounds__(kThreads) ScaleCastKernel(const S* __restrict__ src, D* __restrict__ dst, int64_t n,
                                                            float scale) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = FromFloat<D>(ToFloat<S>(src[i]) * scale);
}

// Strided copy of a 4-D tensor whose innermost rows are contiguous: dst[i0, i1, i2, :] = src[i0, i1, i2, :] with
// independent element strides for the three outer axes on both sides; rows move as 16-byte vectors.  Used to
// re-lay attention tensors ([b, heads, s, d] <-> [b, s, 3, heads, d]) in one pass at copy bandwidth.
struct Copy4dParams {
  int64_t n0, n1, n2;
  int row_vecs;  // 16-byte vectors per row
  int64_t ss[3], ds[3];  // strides in 16-byte vectors
};

__global__ void __launch_bounds__(256) Copy4dKernel(const uint4* __restrict__ src, uint4* __restrict__ dst, Copy4dParams p) {
  const int64_t total = p.n0 * p.n1 * p.n2 * p.row_vecs;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int v      = static_cast<int>(i % p.row_vecs);
    int64_t r        = i / p.row_vecs;
    const int64_t i2 = r % p.n2; r /= p.n2;
    const int64_t i1 = r % p.n1;
    const int64_t i0 = r / p.n1;
    dst[i0 * p.ds[0] + i1 * p.ds[1] + i2 * p.ds[2] + v] = src[i0 * p.ss[0] + i1 * p.ss[1] + i2 * p.ss[2] + v];
  }
}

}  // namespace
}  // namespace tipsk

using namespace tipsk;

#define TIPSK_DISPATCH_FLOAT(dt, T, ...)                                  \
  switch (dt) {                                                           \
    case kF32: { using T = float; __VA_ARGS__; } break;                   \
    case kBF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;          \
    case kF16: { using T = __half; __VA_ARGS__; } break;                  \
    default: return SetError(-2, "unsupported floating dtype");           \
  }

extern "C" {

const char* tipsk_last_error(void) { return LastError().c_str(); }

int tipsk_sgd_momentum_flat(float* p32, void* p16, int p16_dtype, const void* grad, int grad_dtype, float* momentum_buf,
                            int64_t n, float lr, float momentum, float dampening, float weight_decay, int nesterov,
                            float grad_scale, int first_step, void* stream) {
  if (n <= 0) return 0;
  TIPSK_REQUIRE(p32 && grad, "sgd: null pointer");
  TIPSK_REQUIRE(momentum == 0.f || momentum_buf, "sgd: momentum buffer missing");
  SgdParams a{lr, momentum, dampening, weight_decay, grad_scale, nesterov, first_step};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = FlatGrid(n);
  TIPSK_DISPATCH_FLOAT(grad_dtype, G, {
    if (!p16 || p16_dtype == kBF16)
      SgdFlatKernel<G, __nv_bfloat16><<<grid, kThreads, 0, s>>>(p32, static_cast<__nv_bfloat16*>(p16),
                                                                 static_cast<const G*>(grad), momentum_buf, n, a);
    else if (p16_dtype == kF16)
      SgdFlatKernel<G, __half><<<grid, kThreads, 0, s>>>(p32, static_cast<__half*>(p16), static_cast<const G*>(grad),
                                                         momentum_buf, n, a);
    else
      return SetError(-2, "sgd: low-precision copy must be bf16 or fp16");
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_adam_flat(float* p32, void* p16, int p16_dtype, const void* grad, int grad_dtype, float* exp_avg,
                    float* exp_avg_sq, int64_t n, float lr, float beta1, float beta2, float eps, float weight_decay,
                    int64_t step, float grad_scale, int decoupled, void* stream) {
  return tipsk_adam_flat_devstep(p32, p16, p16_dtype, grad, grad_dtype, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps,
                                 weight_decay, step, nullptr, grad_scale, decoupled, stream);
}

/* Same, but when step_dev is non-null the step count (>= 1) is read from that device int64 by the kernel, so a
 * captured graph can be replayed with a changing step. */
int tipsk_adam_flat_devstep(float* p32, void* p16, int p16_dtype, const void* grad, int grad_dtype, float* exp_avg,
                            float* exp_avg_sq, int64_t n, float lr, float beta1, float beta2, float eps,
                            float weight_decay, int64_t step, const int64_t* step_dev, float grad_scale, int decoupled,
                            void* stream) {
  if (n <= 0) return 0;
  TIPSK_REQUIRE(p32 && grad && exp_avg && exp_avg_sq, "adam: null pointer");
  TIPSK_REQUIRE(step >= 1 || step_dev, "adam: step counts from 1");
  AdamParams a{lr, beta1, beta2, eps, weight_decay, grad_scale,
               1.f - powf(beta1, static_cast<float>(step)), 1.f - powf(beta2, static_cast<float>(step)), decoupled,
               step_dev};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = FlatGrid(n);
  TIPSK_DISPATCH_FLOAT(grad_dtype, G, {
    if (!p16 || p16_dtype == kBF16)
      AdamFlatKernel<G, __nv_bfloat16><<<grid, kThreads, 0, s>>>(p32, static_cast<__nv_bfloat16*>(p16),
                                                                  static_cast<const G*>(grad), exp_avg, exp_avg_sq, n, a);
    else if (p16_dtype == kF16)
      AdamFlatKernel<G, __half><<<grid, kThreads, 0, s>>>(p32, static_cast<__half*>(p16), static_cast<const G*>(grad),
                                                          exp_avg, exp_avg_sq, n, a);
    else
      return SetError(-2, "adam: low-precision copy must be bf16 or fp16");
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

int tipsk_pack(const void* const* srcs, const int64_t* offsets, const int64_t* numels, int ntensors, int src_dtype,
               void* flat, int flat_dtype, float scale, int accumulate, void* stream) {
  if (ntensors <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TIPSK_DISPATCH_FLOAT(src_dtype, S, {
    TIPSK_DISPATCH_FLOAT(flat_dtype, D, {
      int rc = LaunchPack<S, D>(accumulate ? 1 : 0, srcs, offsets, numels, ntensors, flat, scale, s);
      if (rc) return rc;
    });
  });
  return 0;
}

int tipsk_unpack(const void* flat, int flat_dtype, void* const* dsts, const int64_t* offsets, const int64_t* numels,
                 int ntensors, int dst_dtype, float scale, void* stream) {
  if (ntensors <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TIPSK_DISPATCH_FLOAT(flat_dtype, S, {
    TIPSK_DISPATCH_FLOAT(dst_dtype, D, {
      int rc = LaunchPack<S, D>(2, reinterpret_cast<const void* const*>(dsts), offsets, numels, ntensors,
                                const_cast<void*>(flat), scale, s);
      if (rc) return rc;
    });
  });
  return 0;
}

int tipsk_scale_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, float scale, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int grid       = CeilDiv(n, kThreads * 4);
  if (grid > NumSMs() * 8) grid = NumSMs() * 8;
  TIPSK_DISPATCH_FLOAT(src_dtype, S, {
    TIPSK_DISPATCH_FLOAT(dst_dtype, D, {
      ScaleCastKernel<S, D><<<grid, kThreads, 0, s>>>(static_cast<const S*>(src), static_cast<D*>(dst), n, scale);
    });
  });
  TIPSK_LAUNCH_CHECK();
  return 0;
}

/* dst[i0, i1, i2, 0:row_bytes] = src[i0, i1, i2, 0:row_bytes]; strides in BYTES for the three outer axes; rows,
 * strides and both base pointers must be multiples of 16 bytes.  The iteration order follows dst (i2 fastest). */
int tipsk_copy4d(const void* src, void* dst, int64_t n0, int64_t n1, int64_t n2, int64_t row_bytes,
                 const int64_t* src_strides, const int64_t* dst_strides, void* stream) {
  if (n0 <= 0 || n1 <= 0 || n2 <= 0 || row_bytes <= 0) return 0;
  TIPSK_REQUIRE(row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(dst) % 16 == 0,
                "copy4d: rows and base pointers must be multiples of 16 bytes");
  Copy4dParams p;
  p.n0 = n0; p.n1 = n1; p.n2 = n2;
  p.row_vecs = static_cast<int>(row_bytes / 16);
  for (int i = 0; i < 3; ++i) {
    TIPSK_REQUIRE(src_strides[i] % 16 == 0 && dst_strides[i] % 16 == 0, "copy4d: strides must be multiples of 16 bytes");
    p.ss[i] = src_strides[i] / 16;
    p.ds[i] = dst_strides[i] / 16;
  }
  const int64_t total = n0 * n1 * n2 * p.row_vecs;
  int64_t grid = (total + 255) / 256;
  if (grid > static_cast<int64_t>(NumSMs()) * 16) grid = static_cast<int64_t>(NumSMs()) * 16;
  Copy4dKernel<<<static_cast<int>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), p);
  TIPSK_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
