// State-space building blocks over packed documents ([tokens, channels] row-major, channels contiguous):
//
//   flb_causal_conv1d_fwd / _bwd   depthwise causal convolution (kernel width <= 8) with fused bias and activation; a token
//                                  never sees tokens of another document (`doc_index`).
//   flb_selective_scan_fwd / _bwd  Mamba selective scan  h_t = exp(dt_t A) h_{t-1} + dt_t B_t x_t,  y_t = <C_t, h_t> + D x_t,
//                                  y_t *= silu(z_t), with dt_t = softplus(dt_raw_t + dt_bias).  One thread owns one channel
//                                  and keeps its `state` values in registers, so x / dt / z loads are coalesced across the
//                                  block and <C_t, h_t> needs no shuffles.  The sequence is cut into 64-token chunks that
//                                  are scanned in parallel from a zero state; a second kernel chains the chunk summaries
//                                  (decay product, end state) in order; a third re-scans every chunk from its true start
//                                  state and emits y.  The backward pass chains the adjoint the same way in reverse, then
//                                  walks every chunk backwards in sub-chunks whose states are recomputed from checkpoints
//                                  (written by a re-run of the third forward kernel, not kept between forward and
//                                  backward).  Gradients of B and C, which are shared by the channels of a group, are
//                                  transposed through shared memory and summed in a fixed order.
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
constexpr int kConvThreads = 128;

struct Row8 {
  float f[8];
  int doc;  // -1: no such token
};

__device__ __forceinline__ Row8 load_row(const __nv_bfloat16* base, const int* doc, long long t, long long tokens, int channels, int c0) {
  Row8 r;
  if (t >= 0 && t < tokens) {
    unpack8(*reinterpret_cast<const bf16x8*>(base + t * channels + c0), r.f);
    r.doc = doc ? doc[t] : 0;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) r.f[i] = 0.f;
    r.doc = -1;
  }
  return r;
}

// One thread owns 8 adjacent channels (their taps live in registers) and walks a segment of tokens, keeping the previous
// W - 1 rows in registers so that every row of x is read once.
// BACKWARD false: out = act(conv(x)).  BACKWARD true: out = dpre = dout * act'(conv(x)), and the segment's contribution to the
// weight / bias gradient goes to partial[segment, channel, 0..W-1 | W].
template <int W, bool BACKWARD>
__global__ void __launch_bounds__(kConvThreads) conv1d_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                              const float* __restrict__ bias, const int* __restrict__ doc,
                                                              const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ out,
                                                              float* __restrict__ partial, long long tokens, int channels, int act, int segment) {
  const int vec = blockIdx.x * kConvThreads + threadIdx.x;
  if (vec >= (channels >> 3)) return;
  const int c0 = vec * 8;
  float taps[W][8], offset[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    offset[i] = bias ? bias[c0 + i] : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) taps[j][i] = w[(c0 + i) * W + j];
  }
  const long long t0 = (long long)blockIdx.y * segment, t1 = min(t0 + segment, tokens);
  constexpr int H = W > 1 ? W - 1 : 1;
  Row8 hist[H];  // hist[k] = row t - (W - 1) + k
#pragma unroll
  for (int k = 0; k < W - 1; ++k) hist[k] = load_row(x, doc, t0 - (W - 1) + k, tokens, channels, c0);
  float sums[W + 1][8];
  if (BACKWARD) {
#pragma unroll
    for (int j = 0; j <= W; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) sums[j][i] = 0.f;
  }
#pragma unroll 4
  for (long long t = t0; t < t1; ++t) {
    const Row8 row = load_row(x, doc, t, tokens, channels, c0);
    float pre[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) pre[i] = offset[i] + taps[W - 1][i] * row.f[i];
#pragma unroll
    for (int k = 0; k < W - 1; ++k) {
      const float same = hist[k].doc == row.doc ? 1.f : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) pre[i] += same * taps[k][i] * hist[k].f[i];
    }
    if (!BACKWARD) {
#pragma unroll
      for (int i = 0; i < 8; ++i) pre[i] = act_fwd(pre[i], act);
      *reinterpret_cast<bf16x8*>(out + t * channels + c0) = pack8(pre);
    } else {
      float g[8];
      unpack8(*reinterpret_cast<const bf16x8*>(dout + t * channels + c0), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        g[i] *= act_grad(pre[i], act);
        sums[W][i] += g[i];
        sums[W - 1][i] += g[i] * row.f[i];
      }
#pragma unroll
      for (int k = 0; k < W - 1; ++k) {
        const float same = hist[k].doc == row.doc ? 1.f : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sums[k][i] += same * g[i] * hist[k].f[i];
      }
      *reinterpret_cast<bf16x8*>(out + t * channels + c0) = pack8(g);
    }
#pragma unroll
    for (int k = 0; k + 1 < W - 1; ++k) hist[k] = hist[k + 1];
    if (W > 1) hist[H - 1] = row;
  }
  if (BACKWARD) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j <= W; ++j) partial[((long long)blockIdx.y * channels + c0 + i) * (W + 1) + j] = sums[j][i];
  }
}

// dx[t] = sum_j w[j] dpre[t + (W - 1 - j)] over the tokens of the same document; the next W - 1 rows are kept in registers.
template <int W>
__global__ void __launch_bounds__(kConvThreads) conv1d_dx_kernel(const __nv_bfloat16* __restrict__ dpre, const float* __restrict__ w,
                                                                 const int* __restrict__ doc, __nv_bfloat16* __restrict__ dx, long long tokens,
                                                                 int channels, int segment) {
  const int vec = blockIdx.x * kConvThreads + threadIdx.x;
  if (vec >= (channels >> 3)) return;
  const int c0 = vec * 8;
  float taps[W][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < W; ++j) taps[j][i] = w[(c0 + i) * W + j];
  const long long t0 = (long long)blockIdx.y * segment, t1 = min(t0 + segment, tokens);
  constexpr int H = W > 1 ? W - 1 : 1;
  Row8 current = load_row(dpre, doc, t0, tokens, channels, c0);
  Row8 next[H];  // next[k] = row t + 1 + k
#pragma unroll
  for (int k = 0; k < W - 1; ++k) next[k] = load_row(dpre, doc, t0 + 1 + k, tokens, channels, c0);
#pragma unroll 4
  for (long long t = t0; t < t1; ++t) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = taps[W - 1][i] * current.f[i];
#pragma unroll
    for (int k = 0; k < W - 1; ++k) {
      const float same = next[k].doc == current.doc ? 1.f : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += same * taps[W - 2 - k][i] * next[k].f[i];
    }
    *reinterpret_cast<bf16x8*>(dx + t * channels + c0) = pack8(acc);
    if (W > 1) {
      current = next[0];
#pragma unroll
      for (int k = 0; k + 1 < W - 1; ++k) next[k] = next[k + 1];
      next[H - 1] = load_row(dpre, doc, t + W, tokens, channels, c0);
    } else {
      current = load_row(dpre, doc, t + 1, tokens, channels, c0);
    }
  }
}

constexpr int kConvSegment = 32;  // tokens per thread in the forward and dx kernels

template <int W>
int conv_forward(const __nv_bfloat16* x, const float* w, const float* bias, const int* doc, __nv_bfloat16* out, long long tokens, int channels, int act,
                 cudaStream_t stream) {
  dim3 grid((unsigned)(((channels >> 3) + kConvThreads - 1) / kConvThreads), (unsigned)((tokens + kConvSegment - 1) / kConvSegment));
  conv1d_kernel<W, false><<<grid, kConvThreads, 0, stream>>>(x, w, bias, doc, nullptr, out, nullptr, tokens, channels, act, kConvSegment);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

template <int W>
int conv_backward(const __nv_bfloat16* x, const float* w, const float* bias, const int* doc, const __nv_bfloat16* dout, __nv_bfloat16* dpre,
                  __nv_bfloat16* dx, float* partial, long long tokens, int channels, int act, int tokens_per_block, cudaStream_t stream) {
  const unsigned vec_blocks = (unsigned)(((channels >> 3) + kConvThreads - 1) / kConvThreads);
  dim3 grid(vec_blocks, (unsigned)((tokens + tokens_per_block - 1) / tokens_per_block));
  conv1d_kernel<W, true><<<grid, kConvThreads, 0, stream>>>(x, w, bias, doc, dout, dpre, partial, tokens, channels, act, tokens_per_block);
  FLB_CHECK_LAUNCH();
  dim3 dx_grid(vec_blocks, (unsigned)((tokens + kConvSegment - 1) / kConvSegment));
  conv1d_dx_kernel<W><<<dx_grid, kConvThreads, 0, stream>>>(dpre, w, doc, dx, tokens, channels, kConvSegment);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

#define FLB_CONV_WIDTHS(CALL) \
  switch (width) {            \
    case 1: return CALL(1);   \
    case 2: return CALL(2);   \
    case 3: return CALL(3);   \
    case 4: return CALL(4);   \
    case 5: return CALL(5);   \
    case 6: return CALL(6);   \
    case 7: return CALL(7);   \
    default: return CALL(8);  \
  }
}  // namespace

// x, out: [tokens, channels] bf16; w: [channels, width] fp32; bias: [channels] fp32 or null; doc: [tokens] int32 (>= 0) or null.
FLB_API int flb_causal_conv1d_fwd(const void* x, const float* w, const float* bias, const int* doc, void* out, long long tokens, int channels,
                                  int width, int act, cudaStream_t stream) {
  if (channels % 8 || width <= 0 || width > kMaxWidth || tokens < 0) return FLB_ERR_SHAPE;
  if (tokens == 0) return FLB_OK;
#define FLB_CONV_FWD(W) conv_forward<W>((const __nv_bfloat16*)x, w, bias, doc, (__nv_bfloat16*)out, tokens, channels, act, stream)
  FLB_CONV_WIDTHS(FLB_CONV_FWD)
#undef FLB_CONV_FWD
}

FLB_API int flb_causal_conv1d_partial_blocks(long long tokens, int tokens_per_block) { return (int)((tokens + tokens_per_block - 1) / tokens_per_block); }

// dpre: scratch [tokens, channels] bf16; partial: [blocks, channels, width + 1] fp32 with blocks = ceil(tokens / tokens_per_block).
FLB_API int flb_causal_conv1d_bwd(const void* x, const float* w, const float* bias, const int* doc, const void* dout, void* dpre, void* dx,
                                  float* partial, long long tokens, int channels, int width, int act, int tokens_per_block, cudaStream_t stream) {
  if (channels % 8 || width <= 0 || width > kMaxWidth || tokens < 0 || tokens_per_block <= 0) return FLB_ERR_SHAPE;
  if (tokens == 0) return FLB_OK;
#define FLB_CONV_BWD(W)                                                                                                                     \
  conv_backward<W>((const __nv_bfloat16*)x, w, bias, doc, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dpre, (__nv_bfloat16*)dx, partial, tokens, \
                   channels, act, tokens_per_block, stream)
  FLB_CONV_WIDTHS(FLB_CONV_BWD)
#undef FLB_CONV_BWD
}

// ----------------------------------------------------------------------------------------------------------------------
// selective scan
// ----------------------------------------------------------------------------------------------------------------------
namespace {
constexpr int kScanThreads = 128;  // channels per block
constexpr int kChunk = 64;         // tokens per chunk
constexpr float kLog2e = 1.4426950408889634f;

// Tokens per backward sub-chunk: the thread keeps sub x state values of recomputed states in registers.
__host__ __device__ constexpr int scan_sub(int state) { return state >= 8 ? 64 / state : 8; }

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
  int channels, groups_b, groups_c, chunks;
};

// log(1 + e^v); below -15 the sum rounds to 1 and the series' first term e^v is exact to fp32.
__device__ __forceinline__ float softplus(float v) {
  const float e = __expf(v);
  return v > 20.f ? v : (v < -15.f ? e : __logf(1.f + e));
}
__device__ __forceinline__ float sigmoidf(float v) { return 1.f / (1.f + __expf(-v)); }

template <int N>
__device__ __forceinline__ void load_state_vec(const __nv_bfloat16* p, float (&out)[N]) {
  if constexpr (N >= 8) {
#pragma unroll
    for (int k = 0; k < N / 8; ++k) unpack8(*reinterpret_cast<const bf16x8*>(p + 8 * k), out + 8 * k);
  } else {
#pragma unroll
    for (int k = 0; k < N / 2; ++k) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + 2 * k));
      out[2 * k] = f.x;
      out[2 * k + 1] = f.y;
    }
  }
}

// Per-thread constants of one channel.  Threads past the last channel work on channel 0 and never store.
template <int N>
struct Channel {
  int d;
  bool valid;
  float a[N], a2[N];  // a and a * log2(e)
  float bias, skip;
  const __nv_bfloat16 *b, *c;  // this channel's group inside a token's B / C row
  long long b_stride, c_stride;
  __device__ __forceinline__ Channel(const ScanArgs& p) {
    const int raw = blockIdx.x * kScanThreads + threadIdx.x;
    valid = raw < p.channels;
    d = valid ? raw : 0;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      a[n] = p.a[(long long)d * N + n];
      a2[n] = a[n] * kLog2e;
    }
    bias = p.dt_bias ? p.dt_bias[d] : 0.f;
    skip = p.skip[d];
    b = p.b + (d / (p.channels / p.groups_b)) * N;
    c = p.c + (d / (p.channels / p.groups_c)) * N;
    b_stride = (long long)p.groups_b * N;
    c_stride = (long long)p.groups_c * N;
  }
};

// Scratch layouts: [chunk or checkpoint][state index][channel], so the block's accesses are coalesced.
__device__ __forceinline__ long long scratch_index(long long slot, int n, int states, int channels, int d) {
  return (slot * states + n) * channels + d;
}

// Phase 1: scan the chunk from a zero state -> its end state and the product of its decays.
template <int N>
__global__ void __launch_bounds__(kScanThreads, N <= 16 ? 8 : 2) scan_summary_kernel(const ScanArgs p, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
  const Channel<N> ch(p);
  if (!ch.valid) return;
  const int chunk = blockIdx.y;
  const long long t0 = (long long)chunk * kChunk;
  const int len = (int)min((long long)kChunk, p.tokens - t0);
  const __nv_bfloat16* xp = p.x + t0 * p.channels + ch.d;
  const __nv_bfloat16* dtp = p.dt + t0 * p.channels + ch.d;
  const __nv_bfloat16* bp = ch.b + t0 * ch.b_stride;
  const unsigned char* sp = p.start ? p.start + t0 : nullptr;
  float h[N];
#pragma unroll
  for (int n = 0; n < N; ++n) h[n] = 0.f;
  float dt_sum = 0.f;
  bool cut = false;
  float x_next = bf2f(*xp), dt_next = bf2f(*dtp);  // one token ahead: these two come from DRAM, B rows are shared and L1-hot
  for (int i = 0; i < len; ++i) {
    const float dtv = softplus(dt_next + ch.bias);
    const float w = dtv * x_next;
    if (i + 1 < len) {
      xp += p.channels;
      dtp += p.channels;
      x_next = bf2f(*xp);
      dt_next = bf2f(*dtp);
    }
    float bv[N];
    load_state_vec<N>(bp, bv);
    bp += ch.b_stride;
    dt_sum += dtv;
    if (sp && sp[i]) {  // uniform over the grid's x dimension
      cut = true;
#pragma unroll
      for (int n = 0; n < N; ++n) h[n] = w * bv[n];
    } else {
#pragma unroll
      for (int n = 0; n < N; ++n) h[n] = fmaf(h[n], exp2f(dtv * ch.a2[n]), w * bv[n]);
    }
  }
#pragma unroll
  for (int n = 0; n < N; ++n) {
    const long long idx = scratch_index(chunk, n, N, p.channels, ch.d);
    chunk_state[idx] = h[n];
    chunk_decay[idx] = cut ? 0.f : exp2f(dt_sum * ch.a2[n]);
  }
}

// Phase 2: chain the summaries in order (REVERSE: from the last chunk back, for the adjoint).  `carried` is overwritten by
// the value ENTERING every chunk: the state at its start, or the adjoint of the state at its end.
template <bool REVERSE>
__global__ void scan_chain_kernel(float* __restrict__ carried, const float* __restrict__ chunk_decay, int chunks, long long per_chunk) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= per_chunk) return;
  constexpr int kBatch = 16;  // loads of a batch are in flight together; only the multiply-adds are serial
  float value = 0.f;
  for (int c0 = 0; c0 < chunks; c0 += kBatch) {
    float decay[kBatch], own[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const int c = REVERSE ? chunks - 1 - (c0 + k) : c0 + k;
      const bool live = c0 + k < chunks;
      decay[k] = live ? chunk_decay[c * per_chunk + i] : 0.f;
      own[k] = live ? carried[c * per_chunk + i] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      if (c0 + k < chunks) {
        const int c = REVERSE ? chunks - 1 - (c0 + k) : c0 + k;
        carried[c * per_chunk + i] = value;
        value = fmaf(decay[k], value, own[k]);
      }
    }
  }
}

// Phase 3: re-scan from the true start state.  CHECKPOINT false: emit y.  CHECKPOINT true: write the state before every
// scan_sub(N)-th token instead (the backward pass recomputes from those).
template <int N, bool CHECKPOINT>
__global__ void __launch_bounds__(kScanThreads, N <= 16 ? 8 : 2) scan_output_kernel(const ScanArgs p, const float* __restrict__ chunk_start, __nv_bfloat16* __restrict__ y,
                                                                     float* __restrict__ checkpoints) {
  constexpr int SUB = scan_sub(N);
  const Channel<N> ch(p);
  if (!ch.valid) return;
  const int chunk = blockIdx.y;
  const long long t0 = (long long)chunk * kChunk;
  const int len = (int)min((long long)kChunk, p.tokens - t0);
  const __nv_bfloat16* xp = p.x + t0 * p.channels + ch.d;
  const __nv_bfloat16* dtp = p.dt + t0 * p.channels + ch.d;
  const __nv_bfloat16* zp = p.z ? p.z + t0 * p.channels + ch.d : nullptr;
  const __nv_bfloat16* bp = ch.b + t0 * ch.b_stride;
  const __nv_bfloat16* cp = ch.c + t0 * ch.c_stride;
  const unsigned char* sp = p.start ? p.start + t0 : nullptr;
  __nv_bfloat16* yp = CHECKPOINT ? nullptr : y + t0 * p.channels + ch.d;
  float* kp = CHECKPOINT ? checkpoints + scratch_index(t0 / SUB, 0, N, p.channels, ch.d) : nullptr;
  float h[N];
#pragma unroll
  for (int n = 0; n < N; ++n) h[n] = chunk_start[scratch_index(chunk, n, N, p.channels, ch.d)];
  float x_next = bf2f(*xp), dt_next = bf2f(*dtp), z_next = (!CHECKPOINT && zp) ? bf2f(*zp) : 0.f;
  for (int i = 0; i < len; ++i) {
    if (CHECKPOINT && i % SUB == 0) {
#pragma unroll
      for (int n = 0; n < N; ++n) kp[(long long)n * p.channels] = h[n];
      kp += (long long)N * p.channels;
    }
    const float dtv = softplus(dt_next + ch.bias);
    const float xv = x_next, zv = z_next;
    const float w = dtv * xv;
    if (i + 1 < len) {
      xp += p.channels;
      dtp += p.channels;
      x_next = bf2f(*xp);
      dt_next = bf2f(*dtp);
      if (!CHECKPOINT && zp) {
        zp += p.channels;
        z_next = bf2f(*zp);
      }
    }
    float bv[N];
    load_state_vec<N>(bp, bv);
    bp += ch.b_stride;
    if (sp && sp[i]) {
#pragma unroll
      for (int n = 0; n < N; ++n) h[n] = w * bv[n];
    } else {
#pragma unroll
      for (int n = 0; n < N; ++n) h[n] = fmaf(h[n], exp2f(dtv * ch.a2[n]), w * bv[n]);
    }
    if (!CHECKPOINT) {
      float cv[N];
      load_state_vec<N>(cp, cv);
      cp += ch.c_stride;
      float out = ch.skip * xv;
#pragma unroll
      for (int n = 0; n < N; ++n) out = fmaf(h[n], cv[n], out);
      if (p.z) out *= zv * sigmoidf(zv);
      *yp = f2bf(out);
      yp += p.channels;
    }
  }
}

struct ScanGrads {
  const __nv_bfloat16* dy;  // [T, D]
  __nv_bfloat16* dx;        // [T, D]
  __nv_bfloat16* ddt;       // [T, D]
  __nv_bfloat16* dz;        // [T, D] or null
  float* db;                // [T, Gb, N] fp32, zero-initialised
  float* dc;                // [T, Gc, N] fp32, zero-initialised
  float* da_partial;        // [chunks, N, D]
  float* dskip_partial;     // [chunks, D]
  float* dbias_partial;     // [chunks, D]
};

// Backward phase 1: adjoint reaching the start of the chunk when nothing flows in from later chunks.
template <int N>
__global__ void __launch_bounds__(kScanThreads, N <= 16 ? 8 : 2) scan_bwd_summary_kernel(const ScanArgs p, const __nv_bfloat16* __restrict__ dy, float* __restrict__ chunk_adjoint) {
  const Channel<N> ch(p);
  if (!ch.valid) return;
  const int chunk = blockIdx.y;
  const long long t0 = (long long)chunk * kChunk;
  const int len = (int)min((long long)kChunk, p.tokens - t0);
  const long long last = (t0 + len - 1) * p.channels + ch.d;
  const __nv_bfloat16* dyp = dy + last;
  const __nv_bfloat16* dtp = p.dt + last;
  const __nv_bfloat16* zp = p.z ? p.z + last : nullptr;
  const __nv_bfloat16* cp = ch.c + (t0 + len - 1) * ch.c_stride;
  const unsigned char* sp = p.start ? p.start + t0 : nullptr;
  float adj[N];
#pragma unroll
  for (int n = 0; n < N; ++n) adj[n] = 0.f;
  float dy_next = bf2f(*dyp), dt_next = bf2f(*dtp), z_next = zp ? bf2f(*zp) : 0.f;
  for (int i = len - 1; i >= 0; --i) {
    float gy = dy_next;
    if (zp) gy *= z_next * sigmoidf(z_next);
    const float dtv = softplus(dt_next + ch.bias);
    if (i > 0) {
      dyp -= p.channels;
      dtp -= p.channels;
      dy_next = bf2f(*dyp);
      dt_next = bf2f(*dtp);
      if (zp) {
        zp -= p.channels;
        z_next = bf2f(*zp);
      }
    }
    if (sp && sp[i]) {  // nothing flows across a document start
#pragma unroll
      for (int n = 0; n < N; ++n) adj[n] = 0.f;
    } else {
      float cv[N];
      load_state_vec<N>(cp, cv);
#pragma unroll
      for (int n = 0; n < N; ++n) adj[n] = fmaf(gy, cv[n], adj[n]) * exp2f(dtv * ch.a2[n]);  // adjoint of the state BEFORE token t
    }
    cp -= ch.c_stride;
  }
#pragma unroll
  for (int n = 0; n < N; ++n) chunk_adjoint[scratch_index(chunk, n, N, p.channels, ch.d)] = adj[n];
}

// Sum the per-channel contributions rows[lane][i * N + n] of this warp's 32 channels into out[token, group, n].  A group
// that lies wholly inside the warp's channels is stored; one that continues in other warps is added atomically.
template <int N, int SUB>
__device__ __forceinline__ void reduce_group_grads(const float* rows, float* __restrict__ out, int groups, int group_size, int channels, int warp_c0,
                                                   long long token0, int live) {
  constexpr int ROW = SUB * N + 4;
  const int lane = threadIdx.x & 31;
  const int c_end = min(warp_c0 + 32, channels);
  const int g_hi = (c_end - 1) / group_size;
  for (int g = warp_c0 / group_size; g <= g_hi; ++g) {
    const int first = g * group_size, last = first + group_size;
    const int r0 = max(first, warp_c0) - warp_c0, r1 = min(last, c_end) - warp_c0;
    const bool whole = first >= warp_c0 && last <= c_end;
#pragma unroll
    for (int o = lane; o < SUB * N; o += 32) {
      const int i = o / N;
      if (i < live) {
        float sum = 0.f;
#pragma unroll 8
        for (int r = r0; r < r1; ++r) sum += rows[r * ROW + o];
        float* dst = out + ((token0 + i) * groups + g) * N + (o % N);
        if (whole) *dst = sum;
        else atomicAdd(dst, sum);
      }
    }
  }
}

// Backward phase 3: walk the chunk backwards, one sub-chunk of recomputed states at a time.  Warps never wait on one another.
template <int N>
__global__ void __launch_bounds__(kScanThreads, N <= 16 ? 3 : 2) scan_bwd_kernel(const ScanArgs p, const ScanGrads g, const float* __restrict__ checkpoints,
                                                                  const float* __restrict__ chunk_adjoint) {
  constexpr int SUB = scan_sub(N);
  constexpr int ROW = SUB * N + 4;  // 16-byte row writes from 8 lanes and column sums both spread over all banks
  extern __shared__ __align__(16) float scan_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_c0 = blockIdx.x * kScanThreads + warp * 32;
  if (warp_c0 >= p.channels) return;
  float* warp_c = scan_smem + (warp * 2) * 32 * ROW;
  float* warp_b = warp_c + 32 * ROW;
  float* rows_c = warp_c + lane * ROW;
  float* rows_b = warp_b + lane * ROW;
  const Channel<N> ch(p);
  const int chunk = blockIdx.y;
  const long long t0 = (long long)chunk * kChunk;
  const int len = (int)min((long long)kChunk, p.tokens - t0);
  float adj[N], grad_a[N];
#pragma unroll
  for (int n = 0; n < N; ++n) {
    adj[n] = chunk_adjoint[scratch_index(chunk, n, N, p.channels, ch.d)];
    grad_a[n] = 0.f;
  }
  float grad_skip = 0.f, grad_bias = 0.f;
  for (int s = (len + SUB - 1) / SUB - 1; s >= 0; --s) {
    const long long ts = t0 + (long long)s * SUB;
    const int live = min(SUB, len - s * SUB);
    const long long base = ts * p.channels + ch.d;
    const float* kp = checkpoints + scratch_index(ts / SUB, 0, N, p.channels, ch.d);
    // every per-channel value of the sub-chunk, loaded up front
    float raw[SUB], xv[SUB], gy[SUB], zv[SUB];
#pragma unroll
    for (int i = 0; i < SUB; ++i) {
      const bool in = i < live;
      const long long td = base + (long long)i * p.channels;
      raw[i] = in ? bf2f(p.dt[td]) + ch.bias : 0.f;
      xv[i] = in ? bf2f(p.x[td]) : 0.f;
      gy[i] = in ? bf2f(g.dy[td]) : 0.f;
      zv[i] = (in && p.z) ? bf2f(p.z[td]) : 0.f;
    }
    // recompute: after[i][n] = state after token ts + i
    float after[SUB][N], dtv[SUB];
    {
      float h[N];
#pragma unroll
      for (int n = 0; n < N; ++n) h[n] = kp[(long long)n * p.channels];
#pragma unroll
      for (int i = 0; i < SUB; ++i) {
        dtv[i] = softplus(raw[i]);
        if (i < live) {
          float bv[N];
          load_state_vec<N>(ch.b + (ts + i) * ch.b_stride, bv);
          const float w = dtv[i] * xv[i];
          if (p.start && p.start[ts + i]) {
#pragma unroll
            for (int n = 0; n < N; ++n) h[n] = w * bv[n];
          } else {
#pragma unroll
            for (int n = 0; n < N; ++n) h[n] = fmaf(h[n], exp2f(dtv[i] * ch.a2[n]), w * bv[n]);
          }
        }
#pragma unroll
        for (int n = 0; n < N; ++n) after[i][n] = h[n];
      }
    }
#pragma unroll
    for (int i = SUB - 1; i >= 0; --i) {
      if (i >= live) continue;  // uniform over the block
      const long long t = ts + i;
      float bv[N], cv[N];
      load_state_vec<N>(ch.b + t * ch.b_stride, bv);
      load_state_vec<N>(ch.c + t * ch.c_stride, cv);
      const bool is_start = p.start && p.start[t];
      const float gate = p.z ? zv[i] * sigmoidf(zv[i]) : 1.f;
      const float gyraw = gy[i] * gate;
      const float w = dtv[i] * xv[i];
      float dot = 0.f, through_a = 0.f, adj_b = 0.f;
      float4 part_c, part_b;
#pragma unroll
      for (int n = 0; n < N; ++n) {
        const float before = i > 0 ? after[i > 0 ? i - 1 : 0][n] : kp[(long long)n * p.channels];
        dot = fmaf(after[i][n], cv[n], dot);
        adj[n] = fmaf(gyraw, cv[n], adj[n]);  // adjoint of the state after token t
        reinterpret_cast<float*>(&part_c)[n & 3] = gyraw * after[i][n];
        reinterpret_cast<float*>(&part_b)[n & 3] = adj[n] * w;
        if ((n & 3) == 3) {
          *reinterpret_cast<float4*>(rows_c + i * N + n - 3) = part_c;
          *reinterpret_cast<float4*>(rows_b + i * N + n - 3) = part_b;
        }
        adj_b = fmaf(adj[n], bv[n], adj_b);
        const float decay = is_start ? 0.f : exp2f(dtv[i] * ch.a2[n]);
        adj[n] *= decay;                        // adjoint of the state before token t
        const float through = adj[n] * before;  // adjoint of the decay, times the decay
        through_a = fmaf(through, ch.a[n], through_a);
        grad_a[n] = fmaf(through, dtv[i], grad_a[n]);
      }
      const float slope = raw[i] > 20.f ? 1.f : sigmoidf(raw[i]);
      const float grad_raw = (through_a + adj_b * xv[i]) * slope;
      if (ch.valid) {
        const long long td = base + (long long)i * p.channels;
        g.dx[td] = f2bf(adj_b * dtv[i] + gyraw * ch.skip);
        g.ddt[td] = f2bf(grad_raw);
        if (g.dz) {
          const float sg = sigmoidf(zv[i]);
          g.dz[td] = f2bf(gy[i] * (dot + ch.skip * xv[i]) * sg * (1.f + zv[i] * (1.f - sg)));
        }
      }
      grad_skip = fmaf(gyraw, xv[i], grad_skip);
      grad_bias += grad_raw;
    }
    __syncwarp();
    reduce_group_grads<N, SUB>(warp_c, g.dc, p.groups_c, p.channels / p.groups_c, p.channels, warp_c0, ts, live);
    reduce_group_grads<N, SUB>(warp_b, g.db, p.groups_b, p.channels / p.groups_b, p.channels, warp_c0, ts, live);
    __syncwarp();
  }
  if (ch.valid) {
#pragma unroll
    for (int n = 0; n < N; ++n) g.da_partial[scratch_index(chunk, n, N, p.channels, ch.d)] = grad_a[n];
    g.dskip_partial[(long long)chunk * p.channels + ch.d] = grad_skip;
    g.dbias_partial[(long long)chunk * p.channels + ch.d] = grad_bias;
  }
}

template <int N>
int scan_forward(const ScanArgs& p, float* chunk_state, float* chunk_decay, __nv_bfloat16* y, cudaStream_t stream) {
  dim3 grid((unsigned)((p.channels + kScanThreads - 1) / kScanThreads), (unsigned)p.chunks);
  scan_summary_kernel<N><<<grid, kScanThreads, 0, stream>>>(p, chunk_state, chunk_decay);
  FLB_CHECK_LAUNCH();
  const long long per_chunk = (long long)p.channels * N;
  scan_chain_kernel<false><<<(unsigned)((per_chunk + 255) / 256), 256, 0, stream>>>(chunk_state, chunk_decay, p.chunks, per_chunk);
  FLB_CHECK_LAUNCH();
  scan_output_kernel<N, false><<<grid, kScanThreads, 0, stream>>>(p, chunk_state, y, nullptr);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

template <int N>
int scan_backward(const ScanArgs& p, const ScanGrads& g, const float* chunk_start, const float* chunk_decay, float* chunk_adjoint, float* checkpoints,
                  cudaStream_t stream) {
  constexpr int kSmem = 2 * kScanThreads * (scan_sub(N) * N + 4) * (int)sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(scan_bwd_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return FLB_ERR_CUDA;
    configured = true;
  }
  dim3 grid((unsigned)((p.channels + kScanThreads - 1) / kScanThreads), (unsigned)p.chunks);
  scan_output_kernel<N, true><<<grid, kScanThreads, 0, stream>>>(p, chunk_start, nullptr, checkpoints);
  FLB_CHECK_LAUNCH();
  scan_bwd_summary_kernel<N><<<grid, kScanThreads, 0, stream>>>(p, g.dy, chunk_adjoint);
  FLB_CHECK_LAUNCH();
  const long long per_chunk = (long long)p.channels * N;
  scan_chain_kernel<true><<<(unsigned)((per_chunk + 255) / 256), 256, 0, stream>>>(chunk_adjoint, chunk_decay, p.chunks, per_chunk);
  FLB_CHECK_LAUNCH();
  scan_bwd_kernel<N><<<grid, kScanThreads, kSmem, stream>>>(p, g, checkpoints, chunk_adjoint);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

int scan_check(const ScanArgs& p, int state) {
  if (state != 4 && state != 8 && state != 16 && state != 32) return FLB_ERR_SHAPE;
  if (p.channels <= 0 || p.groups_b <= 0 || p.groups_c <= 0 || p.channels % p.groups_b || p.channels % p.groups_c) return FLB_ERR_SHAPE;
  return FLB_OK;
}
}  // namespace

FLB_API int flb_selective_scan_chunks(long long tokens) { return (int)((tokens + kChunk - 1) / kChunk); }
// Number of state checkpoints the backward pass needs ([checkpoints, state, channels] fp32).
FLB_API int flb_selective_scan_checkpoints(long long tokens, int state) { return (int)((tokens + scan_sub(state) - 1) / scan_sub(state)); }

// chunk_state, chunk_decay: scratch [chunks, N, D] fp32 (chunk_state ends up holding the state at the start of every chunk and
// chunk_decay the decay product of every chunk: keep both for the backward pass).
FLB_API int flb_selective_scan_fwd(const void* x, const void* dt, const float* a, const void* b, const void* c, const float* skip, const void* z,
                                   const float* dt_bias, const unsigned char* start, long long tokens, int channels, int state, int groups_b,
                                   int groups_c, float* chunk_state, float* chunk_decay, void* y, cudaStream_t stream) {
  ScanArgs p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)dt, a, (const __nv_bfloat16*)b, (const __nv_bfloat16*)c, skip, (const __nv_bfloat16*)z,
             dt_bias, start, tokens, channels, groups_b, groups_c, flb_selective_scan_chunks(tokens)};
  if (int st = scan_check(p, state)) return st;
  if (tokens == 0) return FLB_OK;
  switch (state) {
    case 4: return scan_forward<4>(p, chunk_state, chunk_decay, (__nv_bfloat16*)y, stream);
    case 8: return scan_forward<8>(p, chunk_state, chunk_decay, (__nv_bfloat16*)y, stream);
    case 16: return scan_forward<16>(p, chunk_state, chunk_decay, (__nv_bfloat16*)y, stream);
    default: return scan_forward<32>(p, chunk_state, chunk_decay, (__nv_bfloat16*)y, stream);
  }
}

// chunk_start / chunk_decay: as left by the forward call.  chunk_adjoint: scratch [chunks, N, D]; checkpoints: scratch
// [flb_selective_scan_checkpoints, N, D].  db, dc must be zero on entry.  da_partial is [chunks, N, D].
FLB_API int flb_selective_scan_bwd(const void* x, const void* dt, const float* a, const void* b, const void* c, const float* skip, const void* z,
                                   const float* dt_bias, const unsigned char* start, long long tokens, int channels, int state, int groups_b,
                                   int groups_c, const float* chunk_start, const float* chunk_decay, float* chunk_adjoint, float* checkpoints,
                                   const void* dy, void* dx, void* ddt, void* dz, float* db, float* dc, float* da_partial, float* dskip_partial,
                                   float* dbias_partial, cudaStream_t stream) {
  ScanArgs p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)dt, a, (const __nv_bfloat16*)b, (const __nv_bfloat16*)c, skip, (const __nv_bfloat16*)z,
             dt_bias, start, tokens, channels, groups_b, groups_c, flb_selective_scan_chunks(tokens)};
  if (int st = scan_check(p, state)) return st;
  if (tokens == 0) return FLB_OK;
  ScanGrads g{(const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, (__nv_bfloat16*)ddt, (__nv_bfloat16*)dz, db, dc, da_partial, dskip_partial, dbias_partial};
  switch (state) {
    case 4: return scan_backward<4>(p, g, chunk_start, chunk_decay, chunk_adjoint, checkpoints, stream);
    case 8: return scan_backward<8>(p, g, chunk_start, chunk_decay, chunk_adjoint, checkpoints, stream);
    case 16: return scan_backward<16>(p, g, chunk_start, chunk_decay, chunk_adjoint, checkpoints, stream);
    default: return scan_backward<32>(p, g, chunk_start, chunk_decay, chunk_adjoint, checkpoints, stream);
  }
}

// ----------------------------------------------------------------------------------------------------------------------
// delta-rule state recurrence across chunks
// ----------------------------------------------------------------------------------------------------------------------
// The chunked delta rule (gated DeltaNet, Kimi delta attention) reduces, per head, to
//     S_{c+1} = decay_c o S_c - mix_c S_c + write_c          S: [dk, dv], mix_c: [dk, dk], decay_c: scalar or one per row
// with S reset to zero at chunks that start a document.  Everything else is batched over chunks; this is the only
// sequential part.  Columns of S evolve independently, so a block owns 32 columns of one head and walks the chunks with its
// [dk, 32] slice in shared memory.  REVERSE runs the adjoint:  A_c = grad_c + decay_c o A_{c+1} - mix_c^T A_{c+1}, where A_{c+1}
// is dropped if chunk c + 1 starts a document; it emits A_{c+1} (the adjoint of the state LEAVING chunk c) for every chunk.
namespace {
constexpr int kStateCols = 32;      // columns of S per block
constexpr int kStateThreads = 256;  // (dk / RPT... rows) x 8 column groups of 4; every thread owns RPT x 4 rows x 4 columns

// dk = 32 * RPT.  Shared memory: mix_c [dk][dk] (natural layout, loaded with coalesced 16-byte loads) and two copies of the
// block's [dk][32] slice of S.  Per step of the contraction a thread reads 16-byte vectors only: mix (one row, four contraction
// indices; or for the adjoint four rows, one index) and the matching rows of S, and does 16 to 64 multiply-adds on them.
template <int RPT, bool REVERSE>
__global__ void __launch_bounds__(kStateThreads) delta_state_kernel(const float* __restrict__ decay, const float* __restrict__ mix,
                                                                    const float* __restrict__ add, const unsigned char* __restrict__ first,
                                                                    float* __restrict__ out, int chunks, int heads, int dv, int decay_per_row) {
  constexpr int DK = 32 * RPT;
  extern __shared__ __align__(16) float state_smem[];
  float* mix_s = state_smem;                 // [DK][DK]
  float* current = mix_s + DK * DK;          // [DK][32]
  float* next = current + DK * kStateCols;
  const int head = blockIdx.x, col0 = blockIdx.y * kStateCols;
  const int cg = threadIdx.x % 8, rg = threadIdx.x / 8;  // column group (4 columns) and row group
  // 32 row groups x (DK / 32) rows each = DK rows; a thread owns rows rg * RPT .. rg * RPT + RPT - 1
  const int r_first = rg * RPT;
  for (int i = threadIdx.x; i < DK * kStateCols; i += kStateThreads) current[i] = 0.f;
  __syncthreads();
  for (int step = 0; step < chunks; ++step) {
    const int c = REVERSE ? chunks - 1 - step : step;
    const long long ch = (long long)c * heads + head;
    const float4* mix_c = reinterpret_cast<const float4*>(mix + ch * DK * DK);
    const float* add_c = add + ch * DK * dv;
    float* out_c = out + ch * DK * dv;
    // stage mix_c
    for (int i = threadIdx.x; i < DK * DK / 4; i += kStateThreads) reinterpret_cast<float4*>(mix_s)[i] = mix_c[i];
    // what enters this step: zero across a document start (forward: chunk c starts one; adjoint: chunk c + 1 does)
    const bool cut = REVERSE ? (c + 1 < chunks && first[c + 1]) : first[c];
    if (cut) {
      for (int i = threadIdx.x; i < DK * kStateCols; i += kStateThreads) current[i] = 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < DK * kStateCols / 4; i += kStateThreads) {
      const int row = i / (kStateCols / 4), c4 = i % (kStateCols / 4);
      *reinterpret_cast<float4*>(out_c + (long long)row * dv + col0 + c4 * 4) = reinterpret_cast<const float4*>(current)[i];
    }
    float acc[RPT][4];
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[r][q] = 0.f;
    if (!REVERSE) {
#pragma unroll 2
      for (int j = 0; j < DK; j += 4) {
        float4 s[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) s[jj] = *reinterpret_cast<const float4*>(current + (j + jj) * kStateCols + cg * 4);
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
          const float4 m = *reinterpret_cast<const float4*>(mix_s + (r_first + r) * DK + j);
          const float mv[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            acc[r][0] = fmaf(mv[jj], s[jj].x, acc[r][0]);
            acc[r][1] = fmaf(mv[jj], s[jj].y, acc[r][1]);
            acc[r][2] = fmaf(mv[jj], s[jj].z, acc[r][2]);
            acc[r][3] = fmaf(mv[jj], s[jj].w, acc[r][3]);
          }
        }
      }
    } else {
#pragma unroll 4
      for (int j = 0; j < DK; ++j) {
        const float4 sv = *reinterpret_cast<const float4*>(current + j * kStateCols + cg * 4);
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
          const float m = mix_s[j * DK + r_first + r];  // (mix^T)[row][j]
          acc[r][0] = fmaf(m, sv.x, acc[r][0]);
          acc[r][1] = fmaf(m, sv.y, acc[r][1]);
          acc[r][2] = fmaf(m, sv.z, acc[r][2]);
          acc[r][3] = fmaf(m, sv.w, acc[r][3]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int row = r_first + r;
      const float scale = decay[decay_per_row ? ch * DK + row : ch];
      const float4 old = *reinterpret_cast<const float4*>(current + row * kStateCols + cg * 4);
      const float4 plus = *reinterpret_cast<const float4*>(add_c + (long long)row * dv + col0 + cg * 4);
      float4 result;
      result.x = scale * old.x - acc[r][0] + plus.x;
      result.y = scale * old.y - acc[r][1] + plus.y;
      result.z = scale * old.z - acc[r][2] + plus.z;
      result.w = scale * old.w - acc[r][3] + plus.w;
      *reinterpret_cast<float4*>(next + row * kStateCols + cg * 4) = result;
    }
    __syncthreads();
    float* swap = current;
    current = next;
    next = swap;
  }
}

template <int RPT>
int delta_state_launch(const float* decay, const float* mix, const float* add, const unsigned char* first, float* out, int chunks, int heads, int dv,
                       int decay_per_row, int reverse, cudaStream_t stream) {
  constexpr int DK = 32 * RPT;
  constexpr int kSmem = (DK * DK + 2 * DK * kStateCols) * (int)sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(delta_state_kernel<RPT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess ||
        cudaFuncSetAttribute(delta_state_kernel<RPT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess)
      return FLB_ERR_CUDA;
    configured = true;
  }
  dim3 grid((unsigned)heads, (unsigned)(dv / kStateCols));
  if (reverse) delta_state_kernel<RPT, true><<<grid, kStateThreads, kSmem, stream>>>(decay, mix, add, first, out, chunks, heads, dv, decay_per_row);
  else delta_state_kernel<RPT, false><<<grid, kStateThreads, kSmem, stream>>>(decay, mix, add, first, out, chunks, heads, dv, decay_per_row);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
}  // namespace

// decay: [chunks, heads] or [chunks, heads, dk] (decay_per_row); mix: [chunks, heads, dk, dk]; add: [chunks, heads, dk, dv]
// (forward: the chunk's writes; reverse: the gradient of every entering state); first: [chunks] uint8; out: [chunks, heads, dk, dv]
// (forward: the state entering every chunk; reverse: the adjoint of the state leaving every chunk).  fp32; dk in {32, 64, 128},
// dv a multiple of 32.
FLB_API int flb_delta_state_scan(const float* decay, const float* mix, const float* add, const unsigned char* first, float* out, int chunks,
                                 int heads, int dk, int dv, int decay_per_row, int reverse, cudaStream_t stream) {
  if (chunks < 0 || heads <= 0 || dv <= 0 || dv % kStateCols) return FLB_ERR_SHAPE;
  if (chunks == 0) return FLB_OK;
  switch (dk) {
    case 32: return delta_state_launch<1>(decay, mix, add, first, out, chunks, heads, dv, decay_per_row, reverse, stream);
    case 64: return delta_state_launch<2>(decay, mix, add, first, out, chunks, heads, dv, decay_per_row, reverse, stream);
    case 128: return delta_state_launch<4>(decay, mix, add, first, out, chunks, heads, dv, decay_per_row, reverse, stream);
    default: return FLB_ERR_SHAPE;
  }
}
