// Dispatch / combine of a dropless mixture-of-experts layer.
//
// `rows[t * k + j]` is the row, in the expert-sorted padded row space, that holds token t for its j-th expert.
//   flb_moe_dispatch    out[rows[t, j]] = x[t] * (scale ? scale[t, j] : 1)      (padding rows are left untouched: zero them first)
//   flb_moe_combine     out[t] = sum_j scores[t, j] * y[rows[t, j]]             (fp32 accumulation, no atomics: a token gathers)
//   flb_moe_score_grad  dscores[t, j] = <y[rows[t, j]], dout[t]>
// Dispatch is also the backward of combine (with the scores as scale) and combine the backward of dispatch (with unit
// scores).  One warp per token, 16-byte accesses.  Replaces `copy_dense_to_sparse`, `copy_sparse_to_dense` and
// `copy_sparse_to_dense_grad_score` of `fast_llm/functional/triton/sparse_copy.py:28-200`.
#include "common.cuh"

namespace {
using namespace flb;
constexpr int kWarpsPerBlock = 8;

__global__ void moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ scale,
                                    __nv_bfloat16* __restrict__ out, int tokens, int k, int hidden) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(x + (long long)t * hidden);
  for (int j = 0; j < k; ++j) {
    const int row = rows[t * k + j];
    const float s = scale ? scale[t * k + j] : 1.f;
    bf16x8* dst = reinterpret_cast<bf16x8*>(out + (long long)row * hidden);
    for (int v = lane; v < hidden / 8; v += 32) {
      if (scale) {
        float f[8];
        unpack8(src[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= s;
        dst[v] = pack8(f);
      } else {
        dst[v] = src[v];
      }
    }
  }
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ rows, const float* __restrict__ scores,
                                   __nv_bfloat16* __restrict__ out, int tokens, int k, int hidden) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (t >= tokens) return;
  for (int v = lane; v < hidden / 8; v += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const float s = scores ? scores[t * k + j] : 1.f;
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(y + (long long)rows[t * k + j] * hidden)[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += s * f[i];
    }
    reinterpret_cast<bf16x8*>(out + (long long)t * hidden)[v] = pack8(acc);
  }
}

__global__ void moe_score_grad_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ rows, const __nv_bfloat16* __restrict__ dout,
                                      float* __restrict__ dscores, int tokens, int k, int hidden) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const bf16x8* g = reinterpret_cast<const bf16x8*>(dout + (long long)t * hidden);
  for (int j = 0; j < k; ++j) {
    const bf16x8* src = reinterpret_cast<const bf16x8*>(y + (long long)rows[t * k + j] * hidden);
    float acc = 0.f;
    for (int v = lane; v < hidden / 8; v += 32) {
      float a[8], b[8];
      unpack8(src[v], a);
      unpack8(g[v], b);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += a[i] * b[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) dscores[t * k + j] = acc;
  }
}

int check(int tokens, int k, int hidden) { return (tokens < 0 || k <= 0 || hidden <= 0 || hidden % 8) ? FLB_ERR_SHAPE : FLB_OK; }
}  // namespace

FLB_API int flb_moe_dispatch(const void* x, const int* rows, const float* scale, void* out, int tokens, int k, int hidden, cudaStream_t stream) {
  if (int st = check(tokens, k, hidden)) return st;
  if (tokens == 0) return FLB_OK;
  moe_dispatch_kernel<<<(tokens + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, stream>>>(
      (const __nv_bfloat16*)x, rows, scale, (__nv_bfloat16*)out, tokens, k, hidden);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_moe_combine(const void* y, const int* rows, const float* scores, void* out, int tokens, int k, int hidden, cudaStream_t stream) {
  if (int st = check(tokens, k, hidden)) return st;
  if (tokens == 0) return FLB_OK;
  moe_combine_kernel<<<(tokens + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, stream>>>(
      (const __nv_bfloat16*)y, rows, scores, (__nv_bfloat16*)out, tokens, k, hidden);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_moe_score_grad(const void* y, const int* rows, const void* dout, float* dscores, int tokens, int k, int hidden,
                               cudaStream_t stream) {
  if (int st = check(tokens, k, hidden)) return st;
  if (tokens == 0) return FLB_OK;
  moe_score_grad_kernel<<<(tokens + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, stream>>>(
      (const __nv_bfloat16*)y, rows, (const __nv_bfloat16*)dout, dscores, tokens, k, hidden);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
