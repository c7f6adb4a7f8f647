// Per-element update rules of the fused optimizers, shared by the flat-slab
// kernels (elementwise.cu) and by the allreduce kernel that applies the update
// to the slice of the parameters a rank owns (comm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tipsk {

struct SgdParams {
  float lr, momentum, dampening, wd, grad_scale;
  int nesterov, first_step;
};

// torch.optim.SGD: coupled weight decay, momentum buffer seeded with the first gradient.
__device__ __forceinline__ void SgdUpdate(float& p, float& m, float g, const SgdParams& a) {
  g = g * a.grad_scale + a.wd * p;
  if (a.momentum != 0.f) {
    m = a.first_step ? g : a.momentum * m + (1.f - a.dampening) * g;
    g = a.nesterov ? g + a.momentum * m : m;
  }
  p -= a.lr * g;
}

struct AdamParams {
  float lr, beta1, beta2, eps, wd, grad_scale, bias1, bias2;  // bias = 1 - beta^step
  int decoupled;
  const int64_t* step_dev;  // when set, the step count is read on the device (CUDA-graph replays)
};

__device__ __forceinline__ void AdamUpdate(float& p, float& m, float& v, float g, const AdamParams& a) {
  g *= a.grad_scale;
  if (!a.decoupled) g += a.wd * p;
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float mhat  = m / a.bias1;
  const float denom = sqrtf(v / a.bias2) + a.eps;
  if (a.decoupled) p *= (1.f - a.lr * a.wd);
  p -= a.lr * mhat / denom;
}

}  // namespace tipsk
