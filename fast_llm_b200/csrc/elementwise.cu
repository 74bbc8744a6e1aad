// Memory-bound elementwise kernels: rotary embedding, MLP activations (gated / plain), pointwise
// copy-cast / fill / add / scale, bias + residual add, embedding gather / scatter-add.
// All use 16-byte accesses and grid-stride loops sized to a multiple of the SM count.
#include "common.cuh"
#include "activations.cuh"

namespace {
using namespace flb;

int grid_for(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = 148ll * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

// ------------------------------------------------------------------------------------------------
// Rotary embedding, in place, "half" layout: element i pairs with i + rot_dim/2 inside each head.
// x: [tokens, row_stride]; heads [0, n_heads) at column h*head_dim.  table: [max_pos, rot_dim] fp32 holding
// cos in [0, rot_dim/2) and sin in [rot_dim/2, rot_dim).  conj=1 applies the inverse rotation (backward).
// ------------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ table,
                            const int* __restrict__ positions, long long tokens, long long row_stride, int n_heads,
                            int head_dim, int rot_dim, int conj) {
  const int half = rot_dim >> 1;
  const int vec_per_head = half >> 3;  // 8 pairs per work item
  const long long per_token = (long long)n_heads * vec_per_head;
  const long long total = tokens * per_token;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / per_token;
    const int r = (int)(idx - t * per_token);
    const int h = r / vec_per_head;
    const int i0 = (r - h * vec_per_head) * 8;
    const int pos = positions ? positions[t] : (int)t;
    const float* tab = table + (long long)pos * rot_dim;
    __nv_bfloat16* p = x + t * row_stride + (long long)h * head_dim + i0;
    float a[8], b[8], c[8], s[8];
    unpack8(*reinterpret_cast<const bf16x8*>(p), a);
    unpack8(*reinterpret_cast<const bf16x8*>(p + half), b);
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(tab + i0);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(tab + i0 + 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(tab + half + i0);
    *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(tab + half + i0 + 4);
    float o1[8], o2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = conj ? -s[j] : s[j];
      o1[j] = a[j] * c[j] - b[j] * sj;
      o2[j] = b[j] * c[j] + a[j] * sj;
    }
    *reinterpret_cast<bf16x8*>(p) = pack8(o1);
    *reinterpret_cast<bf16x8*>(p + half) = pack8(o2);
  }
}

// Activations: act_fwd / act_grad in activations.cuh
// in: [rows, (gated?2:1)*n] (gate columns first, then up columns); out: [rows, n]
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long rows,
                               int n, int gated, int type) {
  const int nvec = n >> 3;
  const long long total = rows * nvec;
  const long long in_stride = gated ? 2ll * n : n;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / nvec;
    const int c = (int)(idx - r * nvec) * 8;
    float g[8], o[8];
    unpack8(*reinterpret_cast<const bf16x8*>(in + r * in_stride + c), g);
    if (gated) {
      float u[8];
      unpack8(*reinterpret_cast<const bf16x8*>(in + r * in_stride + n + c), u);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], type) * u[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], type);
    }
    *reinterpret_cast<bf16x8*>(out + r * n + c) = pack8(o);
  }
}

// grad_in: [rows, (gated?2:1)*n]; optionally recomputes the forward output into out_recompute.
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ grad_out, const __nv_bfloat16* __restrict__ in,
                               __nv_bfloat16* __restrict__ grad_in, __nv_bfloat16* __restrict__ out_recompute,
                               long long rows, int n, int gated, int type) {
  const int nvec = n >> 3;
  const long long total = rows * nvec;
  const long long in_stride = gated ? 2ll * n : n;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / nvec;
    const int c = (int)(idx - r * nvec) * 8;
    float g[8], go[8], dg[8];
    unpack8(*reinterpret_cast<const bf16x8*>(in + r * in_stride + c), g);
    unpack8(*reinterpret_cast<const bf16x8*>(grad_out + r * n + c), go);
    if (gated) {
      float u[8], du[8], o[8];
      unpack8(*reinterpret_cast<const bf16x8*>(in + r * in_stride + n + c), u);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = act_fwd(g[j], type);
        dg[j] = go[j] * u[j] * act_grad(g[j], type);
        du[j] = go[j] * a;
        o[j] = a * u[j];
      }
      *reinterpret_cast<bf16x8*>(grad_in + r * in_stride + c) = pack8(dg);
      *reinterpret_cast<bf16x8*>(grad_in + r * in_stride + n + c) = pack8(du);
      if (out_recompute) *reinterpret_cast<bf16x8*>(out_recompute + r * n + c) = pack8(o);
    } else {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dg[j] = go[j] * act_grad(g[j], type);
        o[j] = act_fwd(g[j], type);
      }
      *reinterpret_cast<bf16x8*>(grad_in + r * in_stride + c) = pack8(dg);
      if (out_recompute) *reinterpret_cast<bf16x8*>(out_recompute + r * n + c) = pack8(o);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Pointwise: dtype codes 0 = fp32, 1 = bf16
// ------------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float ld(const T* p, long long i);
template <> __device__ __forceinline__ float ld<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return bf2f(p[i]); }
template <typename T> __device__ __forceinline__ void st(T* p, long long i, float v);
template <> __device__ __forceinline__ void st<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = f2bf(v); }

// out = alpha * a (+ beta * b)
template <typename TA, typename TB, typename TO>
__global__ void axpby_kernel(const TA* __restrict__ a, const TB* __restrict__ b, TO* __restrict__ out, long long n,
                             float alpha, float beta) {
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (i + j < n) {
        float v = alpha * ld<TA>(a, i + j);
        if (b) v += beta * ld<TB>(b, i + j);
        st<TO>(out, i + j, v);
      }
    }
  }
}

template <typename T>
__global__ void fill_kernel(T* __restrict__ out, long long n, float value) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    st<T>(out, i, value);
}

// out[r, :] = x[r, :] + bias[:] (+ residual[r, :]), bf16, cols % 8 == 0
__global__ void bias_residual_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias,
                                     const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                                     long long rows, int cols, float scale) {
  const int nvec = cols >> 3;
  const long long total = rows * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % nvec) * 8;
    float v[8];
    unpack8(*reinterpret_cast<const bf16x8*>(x + idx * 8), v);
    if (bias) {
      float b[8];
      unpack8(*reinterpret_cast<const bf16x8*>(bias + c), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= scale;
    if (residual) {
      float r[8];
      unpack8(*reinterpret_cast<const bf16x8*>(residual + idx * 8), r);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += r[j];
    }
    *reinterpret_cast<bf16x8*>(out + idx * 8) = pack8(v);
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding: out[t] = W[id - vocab_begin] * scale (zero when the id is outside [vocab_begin, vocab_end))
// ------------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, long long tokens, int hidden,
                                     long long vocab_begin, long long vocab_end, float scale) {
  const int nvec = hidden >> 3;
  const long long total = tokens * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c = (int)(idx - t * nvec) * 8;
    const long long id = ids[t];
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (id >= vocab_begin && id < vocab_end) {
      unpack8(*reinterpret_cast<const bf16x8*>(w + (id - vocab_begin) * hidden + c), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= scale;
    }
    *reinterpret_cast<bf16x8*>(out + t * hidden + c) = pack8(v);
  }
}

// grad_w[id - vocab_begin] += grad_out[t] * scale   (fp32 atomics; grad_w fp32)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ grad_out,
                                     float* __restrict__ grad_w, long long tokens, int hidden, long long vocab_begin,
                                     long long vocab_end, float scale) {
  const int nvec = hidden >> 3;
  const long long total = tokens * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c = (int)(idx - t * nvec) * 8;
    const long long id = ids[t];
    if (id < vocab_begin || id >= vocab_end) continue;
    float v[8];
    unpack8(*reinterpret_cast<const bf16x8*>(grad_out + t * hidden + c), v);
    float* dst = grad_w + (id - vocab_begin) * hidden + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, v[j] * scale);
  }
}

}  // namespace

FLB_API int flb_rope(void* x, const float* table, const int* positions, long long tokens, long long row_stride,
                     int n_heads, int head_dim, int rot_dim, int conj, cudaStream_t stream) {
  if (rot_dim % 16 || rot_dim > head_dim || row_stride % 8 || head_dim % 8) return FLB_ERR_SHAPE;
  const long long total = tokens * n_heads * (rot_dim / 16);
  if (total == 0) return FLB_OK;
  rope_kernel<<<grid_for(total, 256), 256, 0, stream>>>((__nv_bfloat16*)x, table, positions, tokens, row_stride,
                                                         n_heads, head_dim, rot_dim, conj);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_act_fwd(const void* in, void* out, long long rows, int n, int gated, int type, cudaStream_t stream) {
  if (n % 8) return FLB_ERR_SHAPE;
  const long long total = rows * (n / 8);
  if (total == 0) return FLB_OK;
  act_fwd_kernel<<<grid_for(total, 256), 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, rows, n, gated, type);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_act_bwd(const void* grad_out, const void* in, void* grad_in, void* out_recompute, long long rows, int n,
                        int gated, int type, cudaStream_t stream) {
  if (n % 8) return FLB_ERR_SHAPE;
  const long long total = rows * (n / 8);
  if (total == 0) return FLB_OK;
  act_bwd_kernel<<<grid_for(total, 256), 256, 0, stream>>>((const __nv_bfloat16*)grad_out, (const __nv_bfloat16*)in,
                                                            (__nv_bfloat16*)grad_in, (__nv_bfloat16*)out_recompute,
                                                            rows, n, gated, type);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// out = alpha*a + beta*b (b may be null).  dtype codes: 0 fp32, 1 bf16.
FLB_API int flb_axpby(const void* a, int a_dtype, const void* b, int b_dtype, void* out, int out_dtype, long long n,
                      float alpha, float beta, cudaStream_t stream) {
  if (n <= 0) return FLB_OK;
  const int g = grid_for((n + 3) / 4, 256);
#define FLB_AX(TA, TB, TO) axpby_kernel<TA, TB, TO><<<g, 256, 0, stream>>>((const TA*)a, (const TB*)b, (TO*)out, n, alpha, beta)
  const int code = a_dtype * 4 + b_dtype * 2 + out_dtype;
  switch (code) {
    case 0: FLB_AX(float, float, float); break;
    case 1: FLB_AX(float, float, __nv_bfloat16); break;
    case 2: FLB_AX(float, __nv_bfloat16, float); break;
    case 3: FLB_AX(float, __nv_bfloat16, __nv_bfloat16); break;
    case 4: FLB_AX(__nv_bfloat16, float, float); break;
    case 5: FLB_AX(__nv_bfloat16, float, __nv_bfloat16); break;
    case 6: FLB_AX(__nv_bfloat16, __nv_bfloat16, float); break;
    case 7: FLB_AX(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); break;
    default: return FLB_ERR_SHAPE;
  }
#undef FLB_AX
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_fill(void* out, int dtype, long long n, float value, cudaStream_t stream) {
  if (n <= 0) return FLB_OK;
  const int g = grid_for(n, 256);
  if (dtype == 0) fill_kernel<float><<<g, 256, 0, stream>>>((float*)out, n, value);
  else fill_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>((__nv_bfloat16*)out, n, value);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_bias_residual(const void* x, const void* bias, const void* residual, void* out, long long rows,
                              int cols, float scale, cudaStream_t stream) {
  if (cols % 8) return FLB_ERR_SHAPE;
  const long long total = rows * (cols / 8);
  if (total == 0) return FLB_OK;
  bias_residual_kernel<<<grid_for(total, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)bias,
                                                                  (const __nv_bfloat16*)residual, (__nv_bfloat16*)out,
                                                                  rows, cols, scale);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_embedding_fwd(const long long* ids, const void* w, void* out, long long tokens, int hidden,
                              long long vocab_begin, long long vocab_end, float scale, cudaStream_t stream) {
  if (hidden % 8) return FLB_ERR_SHAPE;
  const long long total = tokens * (hidden / 8);
  if (total == 0) return FLB_OK;
  embedding_fwd_kernel<<<grid_for(total, 256), 256, 0, stream>>>(ids, (const __nv_bfloat16*)w, (__nv_bfloat16*)out,
                                                                  tokens, hidden, vocab_begin, vocab_end, scale);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_embedding_bwd(const long long* ids, const void* grad_out, float* grad_w, long long tokens, int hidden,
                              long long vocab_begin, long long vocab_end, float scale, cudaStream_t stream) {
  if (hidden % 8) return FLB_ERR_SHAPE;
  const long long total = tokens * (hidden / 8);
  if (total == 0) return FLB_OK;
  embedding_bwd_kernel<<<grid_for(total, 256), 256, 0, stream>>>(ids, (const __nv_bfloat16*)grad_out, grad_w, tokens,
                                                                  hidden, vocab_begin, vocab_end, scale);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
