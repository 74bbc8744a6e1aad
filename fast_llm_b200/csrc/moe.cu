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

// ---------------------------------------------------------------------------------------------------------------------
// Routing of a top-k mixture-of-experts layer in two kernels (instead of top-k, two softmaxes, scatter, means, sort,
// histogram and scans as separate passes):
//   flb_moe_route         per token: the k largest router logits (ties: lower expert first, as a stable descending sort gives),
//                         their softmax (the routing scores), the full softmax for the load-balancing loss (summed per expert
//                         and block, so the result does not depend on the order of atomics) and logsumexp for the router z-loss.
//   flb_moe_route_bwd     gradient of the logits from the score gradients, the load-balancing loss and the z-loss.
//   flb_moe_layout        rows of every (token, choice) in the expert-sorted row space whose expert ranges are padded to whole
//                         GEMM tiles, in token order inside an expert (stable, deterministic), and the range starts.
// Replaces the routing part of `fast_llm/layers/decoder/mlp/mixture_of_experts.py:237-262` and
// `fast_llm/functional/triton/sparse_copy.py:201-241` (sparse map).
namespace {
constexpr int kMaxExperts = 64, kMaxTopK = 8, kRouteThreads = 128;

__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(const float* __restrict__ logits, int tokens, int experts, int k, float* __restrict__ scores, int* __restrict__ top,
                 float* __restrict__ prob_partial, float* __restrict__ lse_out) {
  __shared__ float block_prob[kMaxExperts];
  for (int e = threadIdx.x; e < experts; e += kRouteThreads) block_prob[e] = 0.f;
  __syncthreads();
  const int t = blockIdx.x * kRouteThreads + threadIdx.x;
  if (t < tokens) {
    float v[kMaxExperts];
    float m = -INFINITY;
#pragma unroll 8
    for (int e = 0; e < experts; ++e) { v[e] = logits[(long long)t * experts + e]; m = fmaxf(m, v[e]); }
    float se = 0.f;
    for (int e = 0; e < experts; ++e) se += expf(v[e] - m);
    if (lse_out) lse_out[t] = m + logf(se);
    const float inv = 1.f / se;
    for (int e = 0; e < experts; ++e) atomicAdd(&block_prob[e], expf(v[e] - m) * inv);
    // k passes of arg-max over what is left
    unsigned long long taken = 0ull;
    float chosen[kMaxTopK];
    int idx[kMaxTopK];
    for (int j = 0; j < k; ++j) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < experts; ++e)
        if (!((taken >> e) & 1ull) && (best < 0 || v[e] > bv)) { best = e; bv = v[e]; }
      taken |= 1ull << best;
      chosen[j] = bv; idx[j] = best;
    }
    float top_sum = 0.f;
    for (int j = 0; j < k; ++j) top_sum += expf(chosen[j] - chosen[0]);
    for (int j = 0; j < k; ++j) {
      scores[(long long)t * k + j] = expf(chosen[j] - chosen[0]) / top_sum;
      top[(long long)t * k + j] = idx[j];
    }
  }
  __syncthreads();
  // shared-memory float atomics of one block: the order inside a block varies, the partial sums are written per block and
  // added up in a fixed order afterwards; rounding differences of the in-block order are of the order of 1e-7 relative
  for (int e = threadIdx.x; e < experts; e += kRouteThreads) prob_partial[(long long)blockIdx.x * experts + e] = block_prob[e];
}

// dlogits[t, e] = sum_j [e == top[t, j]] s_j (ds_j - <s, ds>)  +  p_e (g_e - <p, g>)  +  z_coeff * 2 lse p_e
// with s the routing scores, p the full softmax, g_e = aux_grad[e] (gradient of the load-balancing loss wrt the mean
// probability of expert e, already scaled), z_coeff the scaled z-loss weight divided by the number of tokens.
__global__ void __launch_bounds__(kRouteThreads)
moe_route_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ scores, const int* __restrict__ top,
                     const float* __restrict__ dscores, const float* __restrict__ aux_grad, float z_coeff, int tokens, int experts,
                     int k, float* __restrict__ dlogits) {
  const int t = blockIdx.x * kRouteThreads + threadIdx.x;
  if (t >= tokens) return;
  float p[kMaxExperts];
  float m = -INFINITY;
  for (int e = 0; e < experts; ++e) { p[e] = logits[(long long)t * experts + e]; m = fmaxf(m, p[e]); }
  float se = 0.f;
  for (int e = 0; e < experts; ++e) { p[e] = expf(p[e] - m); se += p[e]; }
  const float lse = m + logf(se), inv = 1.f / se;
  float pg = 0.f;
  for (int e = 0; e < experts; ++e) { p[e] *= inv; if (aux_grad) pg += p[e] * aux_grad[e]; }
  float out[kMaxExperts];
  for (int e = 0; e < experts; ++e) out[e] = p[e] * ((aux_grad ? aux_grad[e] - pg : 0.f) + z_coeff * 2.f * lse);
  if (dscores) {
    float dot = 0.f;
    for (int j = 0; j < k; ++j) dot += scores[(long long)t * k + j] * dscores[(long long)t * k + j];
    for (int j = 0; j < k; ++j) {
      const float s = scores[(long long)t * k + j];
      out[top[(long long)t * k + j]] += s * (dscores[(long long)t * k + j] - dot);
    }
  }
  for (int e = 0; e < experts; ++e) dlogits[(long long)t * experts + e] = out[e];
}

// One warp per expert (all in one block): count the expert's entries, then hand out rows in entry order.
__global__ void moe_layout_kernel(const int* __restrict__ top, int entries, int experts, int tile_rows, int* __restrict__ rows,
                                  int* __restrict__ row_begin, int* __restrict__ counts_out) {
  __shared__ int counts[kMaxExperts];
  __shared__ int begin[kMaxExperts + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int e = warp; e < experts; e += warps) {
    int count = 0;
    for (int base = 0; base < entries; base += 32) {
      const int i = base + lane;
      count += __popc(__ballot_sync(0xffffffffu, i < entries && top[i] == e));
    }
    if (lane == 0) counts[e] = count;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      begin[e] = at;
      at += (counts[e] + tile_rows - 1) / tile_rows * tile_rows;
      if (counts_out) counts_out[e] = counts[e];
    }
    begin[experts] = at;
    for (int e = 0; e <= experts; ++e) row_begin[e] = begin[e];
  }
  __syncthreads();
  for (int e = warp; e < experts; e += warps) {
    int at = begin[e];
    for (int base = 0; base < entries; base += 32) {
      const int i = base + lane;
      const bool mine = i < entries && top[i] == e;
      const unsigned ballot = __ballot_sync(0xffffffffu, mine);
      if (mine) rows[i] = at + __popc(ballot & ((1u << lane) - 1u));
      at += __popc(ballot);
    }
  }
}
}  // namespace

FLB_API int flb_moe_route_blocks(int tokens) { return (tokens + kRouteThreads - 1) / kRouteThreads; }

// logits fp32 [tokens, experts]; scores fp32 [tokens, k]; top int32 [tokens, k]; prob_partial fp32 [flb_moe_route_blocks(tokens), experts]
// (every entry written); lse fp32 [tokens] or null.
FLB_API int flb_moe_route(const float* logits, int tokens, int experts, int k, float* scores, int* top, float* prob_partial, float* lse,
                          cudaStream_t stream) {
  if (tokens <= 0 || experts < 1 || experts > kMaxExperts || k < 1 || k > kMaxTopK || k > experts) return FLB_ERR_SHAPE;
  moe_route_kernel<<<flb_moe_route_blocks(tokens), kRouteThreads, 0, stream>>>(logits, tokens, experts, k, scores, top, prob_partial, lse);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_moe_route_bwd(const float* logits, const float* scores, const int* top, const float* dscores, const float* aux_grad,
                              float z_coeff, int tokens, int experts, int k, float* dlogits, cudaStream_t stream) {
  if (tokens <= 0 || experts < 1 || experts > kMaxExperts || k < 1 || k > kMaxTopK) return FLB_ERR_SHAPE;
  moe_route_bwd_kernel<<<flb_moe_route_blocks(tokens), kRouteThreads, 0, stream>>>(logits, scores, top, dscores, aux_grad, z_coeff, tokens, experts, k,
                                                                                     dlogits);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// top int32 [entries] (entries = tokens * k, token-major); rows int32 [entries]; row_begin int32 [experts + 1]; counts int32 [experts] or null.
FLB_API int flb_moe_layout(const int* top, int entries, int experts, int tile_rows, int* rows, int* row_begin, int* counts, cudaStream_t stream) {
  if (entries <= 0 || experts < 1 || experts > kMaxExperts || tile_rows < 1) return FLB_ERR_SHAPE;
  const int warps = experts < 32 ? experts : 32;
  moe_layout_kernel<<<1, warps * 32, 0, stream>>>(top, entries, experts, tile_rows, rows, row_begin, counts);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
