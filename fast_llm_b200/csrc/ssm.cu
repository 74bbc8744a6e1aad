// State-space building blocks over packed documents ([tokens, channels] row-major, channels contiguous):
//
//   flb_causal_conv1d_fwd / _bwd   depthwise causal convolution (kernel width <= 8) with fused bias and activation; a token
//                                  never sees tokens of another document (`doc_index`).
//   flb_selective_scan_fwd / _bwd  Mamba selective scan  h_t = exp(dt_t A) h_{t-1} + dt_t B_t x_t,  y_t = <C_t, h_t> + D x_t,
//                                  y_t *= silu(z_t), with dt_t = softplus(dt_raw_t + dt_bias).  The sequence is cut into
//                                  chunks that are scanned in parallel from a zero state; a second kernel chains the chunk
//                                  summaries (decay product, end state) in order; a third re-scans every chunk from its
//                                  true start state and emits y.  The backward pass runs the same three phases in
//                                  reverse on the adjoint recurrence, recomputing the states of a chunk from its saved
//                                  start state.  One thread owns one (channel, state index) pair; the `state` lanes of a
//                                  channel sit in one warp and reduce <C, h> with shuffles.
//
// These replace the external `causal_conv1d_fn` and `selective_scan_fn` kernels the reference calls
// (`fast_llm/layers/common/linear/convolution.py:15-68`, `fast_llm/layers/ssm/mamba.py:183-236`).
#include "activations.cuh"

namespace {
using namespace flb;

// ----------------------------------------------------------------------------------------------------------------------
// causal conv1d
// ----------------------------------------------------------------------------------------------------------------------
constexpr int kMaxWidth = 8;

// thread = (token, 8 channels)
__global__ void conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                  const int* __restrict__ doc, __nv_bfloat16* __restrict__ out, long long tokens, int channels, int width,
                                  int act) {
  const int nvec = channels >> 3;
  const long long total = tokens * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c0 = (int)(idx - t * nvec) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = bias ? bias[c0 + i] : 0.f;
    const int my_doc = doc ? doc[t] : 0;
    for (int j = 0; j < width; ++j) {
      const long long s = t - (width - 1 - j);
      if (s < 0 || (doc && doc[s] != my_doc)) continue;
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(x + s * channels + c0), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i] * w[(c0 + i) * width + j];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = act_fwd(acc[i], act);
    *reinterpret_cast<bf16x8*>(out + t * channels + c0) = pack8(acc);
  }
}

// dpre[t] = dout[t] * act'(pre[t]) is recomputed where needed.  dx[t] = sum_j w[j] dpre[t + (width - 1 - j)].
__device__ __forceinline__ void conv_pre(const __nv_bfloat16* x, const float* w, const float* bias, const int* doc, long long t, int c0,
                                         int channels, int width, float* pre) {
#pragma unroll
  for (int i = 0; i < 8; ++i) pre[i] = bias ? bias[c0 + i] : 0.f;
  const int my_doc = doc ? doc[t] : 0;
  for (int j = 0; j < width; ++j) {
    const long long s = t - (width - 1 - j);
    if (s < 0 || (doc && doc[s] != my_doc)) continue;
    float f[8];
    unpack8(*reinterpret_cast<const bf16x8*>(x + s * channels + c0), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) pre[i] += f[i] * w[(c0 + i) * width + j];
  }
}

__global__ void conv1d_dpre_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                   const int* __restrict__ doc, const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dpre,
                                   long long tokens, int channels, int width, int act) {
  const int nvec = channels >> 3;
  const long long total = tokens * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c0 = (int)(idx - t * nvec) * 8;
    float pre[8], g[8];
    conv_pre(x, w, bias, doc, t, c0, channels, width, pre);
    unpack8(*reinterpret_cast<const bf16x8*>(dout + t * channels + c0), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] *= act_grad(pre[i], act);
    *reinterpret_cast<bf16x8*>(dpre + t * channels + c0) = pack8(g);
  }
}

__global__ void conv1d_dx_kernel(const __nv_bfloat16* __restrict__ dpre, const float* __restrict__ w, const int* __restrict__ doc,
                                 __nv_bfloat16* __restrict__ dx, long long tokens, int channels, int width) {
  const int nvec = channels >> 3;
  const long long total = tokens * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c0 = (int)(idx - t * nvec) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const int my_doc = doc ? doc[t] : 0;
    for (int j = 0; j < width; ++j) {
      const long long s = t + (width - 1 - j);
      if (s >= tokens || (doc && doc[s] != my_doc)) continue;
      float g[8];
      unpack8(*reinterpret_cast<const bf16x8*>(dpre + s * channels + c0), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += g[i] * w[(c0 + i) * width + j];
    }
    *reinterpret_cast<bf16x8*>(dx + t * channels + c0) = pack8(acc);
  }
}

// partial[block, c, j] = sum over the block's tokens of dpre[t, c] x[t - (width-1-j), c]; partial[block, c, width] = sum dpre.
// grid (token blocks, channel blocks of 128); thread = channel; deterministic (the host sums the blocks in order).
__global__ void conv1d_dw_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dpre, const int* __restrict__ doc,
                                 float* __restrict__ partial, long long tokens, int channels, int width, int tokens_per_block) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const long long t0 = (long long)blockIdx.x * tokens_per_block;
  const long long t1 = min(t0 + tokens_per_block, tokens);
  float acc[kMaxWidth + 1];
#pragma unroll
  for (int j = 0; j <= kMaxWidth; ++j) acc[j] = 0.f;
  for (long long t = t0; t < t1; ++t) {
    const float g = bf2f(dpre[t * channels + c]);
    acc[kMaxWidth] += g;
    const int my_doc = doc ? doc[t] : 0;
#pragma unroll
    for (int j = 0; j < kMaxWidth; ++j) {
      if (j >= width) break;
      const long long s = t - (width - 1 - j);
      if (s < 0 || (doc && doc[s] != my_doc)) continue;
      acc[j] += g * bf2f(x[s * channels + c]);
    }
  }
  float* dst = partial + ((long long)blockIdx.x * channels + c) * (width + 1);
  for (int j = 0; j < width; ++j) dst[j] = acc[j];
  dst[width] = acc[kMaxWidth];
}

int grid_1d(long long items, int threads) {
  long long blocks = (items + threads - 1) / threads;
  return (int)(blocks > 148ll * 16 ? 148ll * 16 : (blocks < 1 ? 1 : blocks));
}
}  // namespace

// x, out: [tokens, channels] bf16; w: [channels, width] fp32; bias: [channels] fp32 or null; doc: [tokens] int32 or null.
FLB_API int flb_causal_conv1d_fwd(const void* x, const float* w, const float* bias, const int* doc, void* out, long long tokens, int channels,
                                  int width, int act, cudaStream_t stream) {
  if (channels % 8 || width <= 0 || width > kMaxWidth || tokens < 0) return FLB_ERR_SHAPE;
  if (tokens == 0) return FLB_OK;
  conv1d_fwd_kernel<<<grid_1d(tokens * (channels / 8), 256), 256, 0, stream>>>((const __nv_bfloat16*)x, w, bias, doc, (__nv_bfloat16*)out, tokens,
                                                                                channels, width, act);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_causal_conv1d_partial_blocks(long long tokens, int tokens_per_block) { return (int)((tokens + tokens_per_block - 1) / tokens_per_block); }

// dpre: scratch [tokens, channels] bf16; partial: [blocks, channels, width + 1] fp32 with blocks = ceil(tokens / tokens_per_block).
FLB_API int flb_causal_conv1d_bwd(const void* x, const float* w, const float* bias, const int* doc, const void* dout, void* dpre, void* dx,
                                  float* partial, long long tokens, int channels, int width, int act, int tokens_per_block, cudaStream_t stream) {
  if (channels % 8 || width <= 0 || width > kMaxWidth || tokens < 0 || tokens_per_block <= 0) return FLB_ERR_SHAPE;
  if (tokens == 0) return FLB_OK;
  const int grid = grid_1d(tokens * (channels / 8), 256);
  conv1d_dpre_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, w, bias, doc, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dpre, tokens,
                                               channels, width, act);
  FLB_CHECK_LAUNCH();
  conv1d_dx_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dpre, w, doc, (__nv_bfloat16*)dx, tokens, channels, width);
  FLB_CHECK_LAUNCH();
  dim3 dw_grid((unsigned)((tokens + tokens_per_block - 1) / tokens_per_block), (unsigned)((channels + 127) / 128));
  conv1d_dw_kernel<<<dw_grid, 128, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dpre, doc, partial, tokens, channels, width,
                                                tokens_per_block);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// ----------------------------------------------------------------------------------------------------------------------
// selective scan
// ----------------------------------------------------------------------------------------------------------------------
namespace {
constexpr int kScanThreads = 128;
constexpr int kChunk = 64;  // tokens per chunk (also the number of states a thread keeps in registers in the backward)

struct ScanArgs {
  const __nv_bfloat16* x;       // [T, D]
  const __nv_bfloat16* dt;      // [T, D] raw step (before bias and softplus)
  const float* a;               // [D, N] (negative)
  const __nv_bfloat16* b;       // [T, Gb, N]
  const __nv_bfloat16* c;       // [T, Gc, N]
  const float* skip;            // [D]
  const __nv_bfloat16* z;       // [T, D] or null
  const float* dt_bias;         // [D] or null
  const unsigned char* start;   // [T] 1 where a document starts, or null
  long long tokens;
  int channels, state, groups_b, groups_c, chunks;
};

__device__ __forceinline__ float softplus(float v) { return v > 20.f ? v : log1pf(__expf(v)); }
__device__ __forceinline__ float sigmoidf(float v) { return 1.f / (1.f + __expf(-v)); }

struct Lane {
  int d, n, gb, gc;
  bool valid;
};
__device__ __forceinline__ Lane lane_of(const ScanArgs& p) {
  Lane l;
  const int per_block = kScanThreads / p.state;
  l.n = threadIdx.x % p.state;
  l.d = blockIdx.x * per_block + threadIdx.x / p.state;
  l.valid = l.d < p.channels;
  const int dd = l.valid ? l.d : 0;
  l.gb = dd / (p.channels / p.groups_b);
  l.gc = dd / (p.channels / p.groups_c);
  l.d = dd;
  return l;
}

// Phase 1: scan the chunk from a zero state; chunk_state[chunk, d, n] = end state, chunk_decay[chunk, d, n] = product of decays.
__global__ void scan_chunk_summary_kernel(const ScanArgs p, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
  const Lane l = lane_of(p);
  const int chunk = blockIdx.y;
  const long long t0 = (long long)chunk * kChunk, t1 = min(t0 + kChunk, p.tokens);
  const float a = p.a[l.d * p.state + l.n];
  const float bias = p.dt_bias ? p.dt_bias[l.d] : 0.f;
  float h = 0.f, decay = 1.f;
  for (long long t = t0; t < t1; ++t) {
    const float dt = softplus(bf2f(p.dt[t * p.channels + l.d]) + bias);
    const float da = (p.start && p.start[t]) ? 0.f : __expf(dt * a);
    const float write = dt * bf2f(p.x[t * p.channels + l.d]) * bf2f(p.b[(t * p.groups_b + l.gb) * p.state + l.n]);
    h = da * h + write;
    decay *= da;
  }
  if (l.valid) {
    const long long idx = ((long long)chunk * p.channels + l.d) * p.state + l.n;
    chunk_state[idx] = h;
    chunk_decay[idx] = decay;
  }
}

// Phase 2: chain the summaries in order.  chunk_state is overwritten by the state at the START of every chunk.
__global__ void scan_chain_kernel(float* __restrict__ chunk_state, const float* __restrict__ chunk_decay, int chunks, long long per_chunk) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= per_chunk) return;
  float h = 0.f;
  for (int c = 0; c < chunks; ++c) {
    const long long idx = c * per_chunk + i;
    const float end = chunk_decay[idx] * h + chunk_state[idx];
    chunk_state[idx] = h;
    h = end;
  }
}

// Phase 3: re-scan from the true start state and emit y.
__global__ void scan_output_kernel(const ScanArgs p, const float* __restrict__ chunk_start, __nv_bfloat16* __restrict__ y) {
  const Lane l = lane_of(p);
  const int chunk = blockIdx.y;
  const long long t0 = (long long)chunk * kChunk, t1 = min(t0 + kChunk, p.tokens);
  const float a = p.a[l.d * p.state + l.n];
  const float bias = p.dt_bias ? p.dt_bias[l.d] : 0.f;
  const float skip = p.skip[l.d];
  float h = chunk_start[((long long)chunk * p.channels + l.d) * p.state + l.n];
  for (long long t = t0; t < t1; ++t) {
    const float dt = softplus(bf2f(p.dt[t * p.channels + l.d]) + bias);
    const float xv = bf2f(p.x[t * p.channels + l.d]);
    const float da = (p.start && p.start[t]) ? 0.f : __expf(dt * a);
    h = da * h + dt * xv * bf2f(p.b[(t * p.groups_b + l.gb) * p.state + l.n]);
    float acc = h * bf2f(p.c[(t * p.groups_c + l.gc) * p.state + l.n]);
    for (int o = p.state >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (l.n == 0 && l.valid) {
      float out = acc + skip * xv;
      if (p.z) {
        const float zv = bf2f(p.z[t * p.channels + l.d]);
        out *= zv * sigmoidf(zv);
      }
      y[t * p.channels + l.d] = f2bf(out);
    }
  }
}

struct ScanGrads {
  const __nv_bfloat16* dy;  // [T, D]
  __nv_bfloat16* dx;        // [T, D]
  __nv_bfloat16* ddt;       // [T, D]
  __nv_bfloat16* dz;        // [T, D] or null
  float* db;                // [T, Gb, N] fp32, zero-initialised (atomic adds)
  float* dc;                // [T, Gc, N] fp32, zero-initialised
  float* da_partial;        // [chunks, D, N]
  float* dskip_partial;     // [chunks, D]
  float* dbias_partial;     // [chunks, D]
};

// Backward phase 1: adjoint reaching the start of the chunk when nothing flows in from later chunks.
__global__ void scan_bwd_summary_kernel(const ScanArgs p, const ScanGrads g, float* __restrict__ chunk_adjoint) {
  const Lane l = lane_of(p);
  const int chunk = blockIdx.y;
  const long long t0 = (long long)chunk * kChunk, t1 = min(t0 + kChunk, p.tokens);
  const float a = p.a[l.d * p.state + l.n];
  const float bias = p.dt_bias ? p.dt_bias[l.d] : 0.f;
  float adj = 0.f;
  for (long long t = t1 - 1; t >= t0; --t) {
    float gy = bf2f(g.dy[t * p.channels + l.d]);
    if (p.z) {
      const float zv = bf2f(p.z[t * p.channels + l.d]);
      gy *= zv * sigmoidf(zv);
    }
    adj += gy * bf2f(p.c[(t * p.groups_c + l.gc) * p.state + l.n]);
    const float dt = softplus(bf2f(p.dt[t * p.channels + l.d]) + bias);
    adj *= (p.start && p.start[t]) ? 0.f : __expf(dt * a);  // adjoint of the state BEFORE token t
  }
  if (l.valid) chunk_adjoint[((long long)chunk * p.channels + l.d) * p.state + l.n] = adj;
}

// Backward phase 2: chunk_adjoint becomes the adjoint of the state at the END of every chunk (what later chunks send back).
__global__ void scan_bwd_chain_kernel(float* __restrict__ chunk_adjoint, const float* __restrict__ chunk_decay, int chunks, long long per_chunk) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= per_chunk) return;
  float incoming = 0.f;  // adjoint of the end state of the chunk being visited
  for (int c = chunks - 1; c >= 0; --c) {
    const long long idx = c * per_chunk + i;
    const float at_start = chunk_adjoint[idx] + chunk_decay[idx] * incoming;
    chunk_adjoint[idx] = incoming;
    incoming = at_start;
  }
}

// Backward phase 3: recompute the chunk's states from its start state, then walk back.
__global__ void scan_bwd_kernel(const ScanArgs p, const ScanGrads g, const float* __restrict__ chunk_start, const float* __restrict__ chunk_adjoint) {
  const Lane l = lane_of(p);
  const int chunk = blockIdx.y;
  const long long t0 = (long long)chunk * kChunk, t1 = min(t0 + kChunk, p.tokens);
  const int len = (int)(t1 - t0);
  const float a = p.a[l.d * p.state + l.n];
  const float bias = p.dt_bias ? p.dt_bias[l.d] : 0.f;
  const float skip = p.skip[l.d];
  const long long sidx = ((long long)chunk * p.channels + l.d) * p.state + l.n;
  float states[kChunk + 1];  // states[i] = state before token t0 + i
  states[0] = chunk_start[sidx];
#pragma unroll
  for (int i = 0; i < kChunk; ++i) {
    if (i < len) {
      const long long t = t0 + i;
      const float dt = softplus(bf2f(p.dt[t * p.channels + l.d]) + bias);
      const float da = (p.start && p.start[t]) ? 0.f : __expf(dt * a);
      states[i + 1] = da * states[i] + dt * bf2f(p.x[t * p.channels + l.d]) * bf2f(p.b[(t * p.groups_b + l.gb) * p.state + l.n]);
    } else {
      states[i + 1] = states[i];
    }
  }
  float adj = chunk_adjoint[sidx];  // adjoint of the state after the chunk's last token
  float grad_a = 0.f, grad_skip = 0.f, grad_bias = 0.f;
#pragma unroll
  for (int i = kChunk - 1; i >= 0; --i) {
    if (i >= len) continue;
    const long long t = t0 + i;
    const long long td = t * p.channels + l.d;
    const float raw = bf2f(p.dt[td]) + bias;
    const float dt = softplus(raw);
    const float xv = bf2f(p.x[td]);
    const float bv = bf2f(p.b[(t * p.groups_b + l.gb) * p.state + l.n]);
    const float cv = bf2f(p.c[(t * p.groups_c + l.gc) * p.state + l.n]);
    const bool is_start = p.start && p.start[t];
    const float da = is_start ? 0.f : __expf(dt * a);
    float gy = bf2f(g.dy[td]);
    float zv = 0.f, gate = 1.f;
    if (p.z) {
      zv = bf2f(p.z[td]);
      gate = zv * sigmoidf(zv);
    }
    const float gyraw = gy * gate;
    // y_raw = <c, h_t> + skip x
    float dot = states[i + 1] * cv;
    for (int o = p.state >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    adj += gyraw * cv;                       // adjoint of h_t
    const float grad_c = gyraw * states[i + 1];
    // h_t = da h_{t-1} + dt x b
    const float grad_da = adj * states[i];   // zero decay at a document start carries no gradient (da is a constant 0 there)
    const float grad_write = adj;
    float grad_dt = (is_start ? 0.f : grad_da * da * a) + grad_write * xv * bv;
    float grad_x = grad_write * dt * bv;
    const float grad_b = grad_write * dt * xv;
    grad_a += is_start ? 0.f : grad_da * da * dt;
    adj *= da;                               // adjoint of h_{t-1}
    for (int o = p.state >> 1; o > 0; o >>= 1) {
      grad_dt += __shfl_xor_sync(0xffffffffu, grad_dt, o);
      grad_x += __shfl_xor_sync(0xffffffffu, grad_x, o);
    }
    if (l.valid) {
      atomicAdd(g.db + (t * p.groups_b + l.gb) * p.state + l.n, grad_b);
      atomicAdd(g.dc + (t * p.groups_c + l.gc) * p.state + l.n, grad_c);
      if (l.n == 0) {
        const float yraw = dot + skip * xv;
        grad_x += gyraw * skip;
        const float grad_raw = grad_dt * sigmoidf(raw);
        g.dx[td] = f2bf(grad_x);
        g.ddt[td] = f2bf(grad_raw);
        if (g.dz) {
          const float s = sigmoidf(zv);
          g.dz[td] = f2bf(gy * yraw * s * (1.f + zv * (1.f - s)));
        }
        grad_skip += gyraw * xv;
        grad_bias += grad_raw;
      }
    }
  }
  if (l.valid) {
    g.da_partial[sidx] = grad_a;
    if (l.n == 0) {
      g.dskip_partial[(long long)chunk * p.channels + l.d] = grad_skip;
      g.dbias_partial[(long long)chunk * p.channels + l.d] = grad_bias;
    }
  }
}

int scan_check(const ScanArgs& p) {
  if (p.state < 1 || p.state > 32 || (p.state & (p.state - 1)) || p.channels <= 0 || p.groups_b <= 0 || p.groups_c <= 0) return FLB_ERR_SHAPE;
  if (p.channels % p.groups_b || p.channels % p.groups_c || p.channels % (kScanThreads / p.state)) return FLB_ERR_SHAPE;
  return FLB_OK;
}
}  // namespace

FLB_API int flb_selective_scan_chunks(long long tokens) { return (int)((tokens + kChunk - 1) / kChunk); }

// chunk_state, chunk_decay: scratch [chunks, D, N] fp32 (chunk_state ends up holding the state at the start of every chunk and
// chunk_decay the decay product of every chunk: keep both for the backward pass).
FLB_API int flb_selective_scan_fwd(const void* x, const void* dt, const float* a, const void* b, const void* c, const float* skip, const void* z,
                                   const float* dt_bias, const unsigned char* start, long long tokens, int channels, int state, int groups_b,
                                   int groups_c, float* chunk_state, float* chunk_decay, void* y, cudaStream_t stream) {
  ScanArgs p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)dt, a, (const __nv_bfloat16*)b, (const __nv_bfloat16*)c, skip, (const __nv_bfloat16*)z,
             dt_bias, start, tokens, channels, state, groups_b, groups_c, flb_selective_scan_chunks(tokens)};
  if (int st = scan_check(p)) return st;
  if (tokens == 0) return FLB_OK;
  dim3 grid((unsigned)(channels / (kScanThreads / state)), (unsigned)p.chunks);
  scan_chunk_summary_kernel<<<grid, kScanThreads, 0, stream>>>(p, chunk_state, chunk_decay);
  FLB_CHECK_LAUNCH();
  const long long per_chunk = (long long)channels * state;
  scan_chain_kernel<<<(unsigned)((per_chunk + 255) / 256), 256, 0, stream>>>(chunk_state, chunk_decay, p.chunks, per_chunk);
  FLB_CHECK_LAUNCH();
  scan_output_kernel<<<grid, kScanThreads, 0, stream>>>(p, chunk_state, (__nv_bfloat16*)y);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// chunk_start / chunk_decay: as left by the forward call.  chunk_adjoint: scratch [chunks, D, N].  db, dc must be zero on entry.
FLB_API int flb_selective_scan_bwd(const void* x, const void* dt, const float* a, const void* b, const void* c, const float* skip, const void* z,
                                   const float* dt_bias, const unsigned char* start, long long tokens, int channels, int state, int groups_b,
                                   int groups_c, const float* chunk_start, const float* chunk_decay, float* chunk_adjoint, const void* dy, void* dx,
                                   void* ddt, void* dz, float* db, float* dc, float* da_partial, float* dskip_partial, float* dbias_partial,
                                   cudaStream_t stream) {
  ScanArgs p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)dt, a, (const __nv_bfloat16*)b, (const __nv_bfloat16*)c, skip, (const __nv_bfloat16*)z,
             dt_bias, start, tokens, channels, state, groups_b, groups_c, flb_selective_scan_chunks(tokens)};
  if (int st = scan_check(p)) return st;
  if (tokens == 0) return FLB_OK;
  ScanGrads g{(const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, (__nv_bfloat16*)ddt, (__nv_bfloat16*)dz, db, dc, da_partial, dskip_partial, dbias_partial};
  dim3 grid((unsigned)(channels / (kScanThreads / state)), (unsigned)p.chunks);
  scan_bwd_summary_kernel<<<grid, kScanThreads, 0, stream>>>(p, g, chunk_adjoint);
  FLB_CHECK_LAUNCH();
  const long long per_chunk = (long long)channels * state;
  scan_bwd_chain_kernel<<<(unsigned)((per_chunk + 255) / 256), 256, 0, stream>>>(chunk_adjoint, chunk_decay, p.chunks, per_chunk);
  FLB_CHECK_LAUNCH();
  scan_bwd_kernel<<<grid, kScanThreads, 0, stream>>>(p, g, chunk_start, chunk_adjoint);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
