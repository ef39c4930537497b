// Scalar definitions of the PoM non-linearities, shared by every kernel so the
// fused epilogues and the stand-alone operators agree bit for bit.
//
//   act(x)        = clamp(leaky_relu(x, 0.01), -0.1, 6)        (reference pom/pom.py:27-28)
//   poly(a)       = sum_{i<K} coeff[i] * a^(i+1)               (reference pom/pom.py:83-88)
//   hardsigmoid z = min(max(z + 3, 0), 6) / 6                  (reference pom/pom.py:207)
//
// Derivatives follow PyTorch autograd on the reference expressions:
// leaky_relu' is 1 for x > 0 else 0.01 (so 0.01 at exactly 0); clamp' is 1 on
// the closed interval [-0.1, 6] of the leaky output; hardsigmoid' is 1/6 on the
// open interval (-3, 3).
#pragma once
#include <cuda_runtime.h>

namespace pomk {

constexpr int kMaxDegree = 16;

__device__ __forceinline__ float pom_act(float x) { return x > 0.f ? fminf(x, 6.f) : fmaxf(0.01f * x, -0.1f); }

__device__ __forceinline__ float pom_act_grad(float x) {
  if (x > 0.f) return x <= 6.f ? 1.f : 0.f;
  return (0.01f * x >= -0.1f) ? 0.01f : 0.f;
}

// Running-power evaluation in the same order as the reference (power i+1 is
// power i times a; terms are summed in increasing degree).
__device__ __forceinline__ float pom_poly(float a, const float* __restrict__ c, int K) {
  float p = a;
  float acc = c[0] * p;
  for (int i = 1; i < K; ++i) {
    p *= a;
    acc = fmaf(c[i], p, acc);
  }
  return acc;
}

// d poly / d a = sum_i (i+1) * coeff[i] * a^i
__device__ __forceinline__ float pom_poly_grad(float a, const float* __restrict__ c, int K) {
  float p = 1.f;
  float acc = c[0];
  for (int i = 1; i < K; ++i) {
    p *= a;
    acc = fmaf(static_cast<float>(i + 1) * c[i], p, acc);
  }
  return acc;
}

__device__ __forceinline__ float pom_hardsigmoid(float z) { return fminf(fmaxf(z + 3.f, 0.f), 6.f) * (1.f / 6.f); }

__device__ __forceinline__ float pom_hardsigmoid_grad(float z) { return (z > -3.f && z < 3.f) ? (1.f / 6.f) : 0.f; }

}  // namespace pomk
