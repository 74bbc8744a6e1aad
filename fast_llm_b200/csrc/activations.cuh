// Scalar activation functions and their derivatives, shared by the elementwise and convolution kernels.
#pragma once
#include "common.cuh"

namespace {
// Activations.  type: 0 identity, 1 silu, 2 gelu(tanh), 3 relu, 4 squared relu, 5 sigmoid, 6 gelu(erf)
__device__ __forceinline__ float act_fwd(float x, int type) {
  switch (type) {
    case 1: return x / (1.f + __expf(-x));
    case 2: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case 3: return fmaxf(x, 0.f);
    case 4: { const float r = fmaxf(x, 0.f); return r * r; }
    case 5: return 1.f / (1.f + __expf(-x));
    case 6: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    default: return x;
  }
}
__device__ __forceinline__ float act_grad(float x, int type) {
  switch (type) {
    case 1: { const float s = 1.f / (1.f + __expf(-x)); return s * (1.f + x * (1.f - s)); }
    case 2: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      const float t = tanhf(u);
      const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
      return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
    }
    case 3: return x > 0.f ? 1.f : 0.f;
    case 4: return x > 0.f ? 2.f * x : 0.f;
    case 5: { const float s = 1.f / (1.f + __expf(-x)); return s * (1.f - s); }
    case 6: return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
    default: return 1.f;
  }
}

}  // namespace
