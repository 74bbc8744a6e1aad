// Optimizer kernels over flat fp32 shards: deterministic sum of squares (gradient norm), clip coefficient computed on
// the device (no host round trip), and fused AdamW that also writes the bf16 copy of the updated weights.
#include "common.cuh"
#include "no_alloc.h"
#include <mutex>

namespace {
using namespace flb;
constexpr int kThreads = 256;
constexpr int kSumsqBlocks = 1024;

__global__ void __launch_bounds__(kThreads)
sumsq_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float scratch[32];
  float s = 0.f;
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec; i += (long long)gridDim.x * kThreads) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = (nvec << 2) + threadIdx.x; i < n; i += kThreads) s += x[i] * x[i];
  const float t = block_sum(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

__global__ void __launch_bounds__(kThreads)
sumsq_final_kernel(const float* __restrict__ partial, int parts, float* __restrict__ out, int accumulate) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < parts; i += kThreads) s += partial[i];
  const float t = block_sum(s, scratch);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + t : t;
}

// coeff = extra_scale * min(1, max_norm / (norm + 1e-6)); norm = sqrt(normsq) * extra_scale
__global__ void clip_coeff_kernel(const float* __restrict__ normsq, float max_norm, float extra_scale,
                                  float* __restrict__ coeff_out, float* __restrict__ norm_out) {
  const float norm = sqrtf(normsq[0]) * extra_scale;
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (norm + 1e-6f));
  coeff_out[0] = c * extra_scale;
  if (norm_out) norm_out[0] = norm;
}

__global__ void __launch_bounds__(kThreads)
adamw_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             __nv_bfloat16* __restrict__ w_lp, long long n, float lr, float beta1, float beta2, float eps, float wd,
             float inv_bc1, float inv_bc2, float gscale, const float* __restrict__ gscale_ptr,
             const int* __restrict__ noop_flag) {
  if (noop_flag && *noop_flag) return;
  const float sc = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec; i += (long long)gridDim.x * kThreads) {
    float4 wv = reinterpret_cast<float4*>(w)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* wp = &wv.x; const float* gp = &gv.x; float* mp = &mv.x; float* vp = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gp[j] * sc;
      mp[j] = beta1 * mp[j] + (1.f - beta1) * gj;
      vp[j] = beta2 * vp[j] + (1.f - beta2) * gj * gj;
      const float upd = (mp[j] * inv_bc1) / (sqrtf(vp[j] * inv_bc2) + eps) + wd * wp[j];
      wp[j] -= lr * upd;
    }
    reinterpret_cast<float4*>(w)[i] = wv;
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (w_lp) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y), hi = __floats2bfloat162_rn(wv.z, wv.w);
      reinterpret_cast<uint2*>(w_lp)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
  if (blockIdx.x == 0) {
    for (long long i = (nvec << 2) + threadIdx.x; i < n; i += kThreads) {
      const float gj = g[i] * sc;
      m[i] = beta1 * m[i] + (1.f - beta1) * gj;
      v[i] = beta2 * v[i] + (1.f - beta2) * gj * gj;
      const float upd = (m[i] * inv_bc1) / (sqrtf(v[i] * inv_bc2) + eps) + wd * w[i];
      w[i] -= lr * upd;
      if (w_lp) w_lp[i] = f2bf(w[i]);
    }
  }
}

}  // namespace

FLB_API int flb_sumsq_scratch_floats() { return kSumsqBlocks; }

// out[0] (+)= sum(x^2); `partial` is caller-provided scratch of flb_sumsq_scratch_floats() floats.
FLB_API int flb_sumsq(const float* x, long long n, float* partial, float* out, int accumulate, cudaStream_t stream) {
  if (n < 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return FLB_ERR_SHAPE;
  sumsq_partial_kernel<<<kSumsqBlocks, kThreads, 0, stream>>>(x, n, partial);
  FLB_CHECK_LAUNCH();
  sumsq_final_kernel<<<1, kThreads, 0, stream>>>(partial, kSumsqBlocks, out, accumulate);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// out[0] (+)= sum of `parts` floats (one block, fixed order: deterministic).  Finishes norms whose per-block partial sums
// were produced by other kernels (the fused gradient reduction writes them while it reduces).
FLB_API int flb_sum_partials(const float* partial, int parts, float* out, int accumulate, cudaStream_t stream) {
  if (parts <= 0) return FLB_ERR_SHAPE;
  sumsq_final_kernel<<<1, kThreads, 0, stream>>>(partial, parts, out, accumulate);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_clip_coeff(const float* normsq, float max_norm, float extra_scale, float* coeff_out, float* norm_out,
                           cudaStream_t stream) {
  clip_coeff_kernel<<<1, 1, 0, stream>>>(normsq, max_norm, extra_scale, coeff_out, norm_out);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// Decoupled-weight-decay Adam on n contiguous fp32 elements; w_lp (bf16, may be null) receives the rounded weights.
// step >= 1 is used for bias correction.  The gradient is multiplied by gscale * (*gscale_ptr if non-null).
FLB_API int flb_adamw(float* w, const float* g, float* m, float* v, void* w_lp, long long n, float lr, float beta1,
                      float beta2, float eps, float wd, int step, float gscale, const float* gscale_ptr,
                      const int* noop_flag, cudaStream_t stream) {
  if (n <= 0) return FLB_OK;
  const uintptr_t al = reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                       reinterpret_cast<uintptr_t>(v);
  if ((al & 15) || (w_lp && (reinterpret_cast<uintptr_t>(w_lp) & 7))) return FLB_ERR_SHAPE;
  const float inv_bc1 = 1.f / (1.f - powf(beta1, (float)step));
  const float inv_bc2 = 1.f / (1.f - powf(beta2, (float)step));
  long long blocks = ((n >> 2) + kThreads - 1) / kThreads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  adamw_kernel<<<(int)blocks, kThreads, 0, stream>>>(w, g, m, v, (__nv_bfloat16*)w_lp, n, lr, beta1, beta2, eps, wd,
                                                      inv_bc1, inv_bc2, gscale, gscale_ptr, noop_flag);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// ------------------------------------------------------------------------------------------------
// Variant of flb_sumsq for callers that cannot allocate: the per-block partial sums live in a scratch array that is
// part of the library image instead of a caller-provided buffer.  See no_alloc.h for the contract.
// ------------------------------------------------------------------------------------------------
static_assert(FLB_NO_ALLOC_SCRATCH_FLOATS == kSumsqBlocks, "built-in scratch must hold one partial per block");
static __device__ __align__(256) float g_sumsq_scratch[FLB_NO_ALLOC_SCRATCH_FLOATS];

namespace {
// In host code `g_sumsq_scratch` is only a handle for the symbol, not a device address: resolve the real address once
// per device (with that device current) and hand the kernels that pointer.
int no_alloc_scratch(float** out) {
  static float* addresses[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return flb_record_cuda_error(e);
  if (dev < 0 || dev >= 64) return FLB_ERR_SHAPE;
  std::lock_guard<std::mutex> lock(mu);
  if (addresses[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_sumsq_scratch);
    if (e != cudaSuccess) return flb_record_cuda_error(e);
    addresses[dev] = static_cast<float*>(p);
  }
  *out = addresses[dev];
  return FLB_OK;
}
}  // namespace

FLB_API int flb_sumsq_no_alloc(const float* x, long long n, float* out, int accumulate, cudaStream_t stream) {
  if (n < 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return FLB_ERR_SHAPE;
  if (n > FLB_NO_ALLOC_MAX_ELEMENTS) return FLB_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int st = no_alloc_scratch(&scratch);
  if (st != FLB_OK) return st;
  // Every block writes its own slot before the final kernel reads any, so stale contents of earlier calls are harmless.
  sumsq_partial_kernel<<<kSumsqBlocks, kThreads, 0, stream>>>(x, n, scratch);
  FLB_CHECK_LAUNCH();
  sumsq_final_kernel<<<1, kThreads, 0, stream>>>(scratch, kSumsqBlocks, out, accumulate);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
