// Cross-entropy over a (possibly vocabulary-sharded) logits matrix, in two kernels so that the per-token softmax
// statistics can be merged across tensor-parallel ranks between them:
//   flb_ce_stats : per row, local max, sum of exp(logit - max) and the target logit (0 if the label is in
//                  another shard)                                  -> stats[T, 3]
//   flb_ce_grad  : given merged (max, sumexp, target) writes the per-token loss and the logit gradients
//                  grad_j = g * ((1 + 2 z lse) softmax_j - [j == label]) * logits_scale   (may alias logits)
// Also carries the z-loss term z * lse^2.  Labels < 0 are ignored (zero loss and gradient).
// Vocabulary-parallel exchange without a collective library: `flb_ce_stats_exchange` stores this rank's three numbers per
// token straight into slot `rank` of every peer's statistics buffer (NVLink peer stores from the statistics kernel); after one
// device-side barrier `flb_ce_grad` reads `slots` local slots per token and merges them (global max, rescaled sum-exp,
// summed target logit) on the fly.
#include "common.cuh"

namespace {
using namespace flb;
constexpr int kThreads = 256;

template <typename T> struct Vec;
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) { unpack8(*reinterpret_cast<const bf16x8*>(p), f); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) { *reinterpret_cast<bf16x8*>(p) = pack8(f); }
};
template <> struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) { *reinterpret_cast<float4*>(f) = *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(f); }
};

struct StatPeers {
  float* p[8];
  int world;  // 0: write to `stats` only
  int rank;
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
ce_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ stats,
                int rows, int cols, long long ld, long long vocab_begin, float logits_scale, const StatPeers peers) {
  __shared__ float scratch[32];
  constexpr int VN = Vec<T>::N;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = logits + (long long)row * ld;
    float m = -INFINITY, s = 0.f;
    const int nvec = cols / VN;
    for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
      float f[VN];
      Vec<T>::load(p + vi * VN, f);
      float lm = f[0] * logits_scale;
#pragma unroll
      for (int j = 1; j < VN; ++j) lm = fmaxf(lm, f[j] * logits_scale);
      if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
      for (int j = 0; j < VN; ++j) s += __expf(f[j] * logits_scale - m);
    }
    for (int c = nvec * VN + threadIdx.x; c < cols; c += kThreads) {
      float f;
      if constexpr (sizeof(T) == 2) f = bf2f(p[c]) * logits_scale; else f = p[c] * logits_scale;
      if (f > m) { s *= __expf(m - f); m = f; }
      s += __expf(f - m);
    }
    const float gm = block_max(m, scratch);
    const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
    const float gs = block_sum(contrib, scratch);
    if (threadIdx.x == 0) {
      const long long lab = labels[row] - vocab_begin;
      float tgt = 0.f;
      if (lab >= 0 && lab < cols) {
        if constexpr (sizeof(T) == 2) tgt = bf2f(p[lab]) * logits_scale; else tgt = p[lab] * logits_scale;
      }
      if (peers.world == 0) {
        stats[row * 3 + 0] = gm;
        stats[row * 3 + 1] = gs;
        stats[row * 3 + 2] = tgt;
      } else {
        const long long at = ((long long)peers.rank * rows + row) * 3;
        for (int r = 0; r < peers.world; ++r) {
          float* dst = peers.p[r] + at;
          dst[0] = gm;
          dst[1] = gs;
          dst[2] = tgt;
        }
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
ce_grad_kernel(const T* __restrict__ logits, const long long* __restrict__ labels, const float* __restrict__ stats,
               T* __restrict__ grad, float* __restrict__ loss_out, float* __restrict__ z_out, int rows, int cols,
               long long ld, long long ld_grad, long long vocab_begin, float logits_scale, float grad_scale,
               const float* __restrict__ grad_scale_ptr, float z_coef, int slots) {
  constexpr int VN = Vec<T>::N;
  const float gscale = grad_scale * (grad_scale_ptr ? *grad_scale_ptr : 1.f);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = logits + (long long)row * ld;
    T* g = grad ? grad + (long long)row * ld_grad : nullptr;
    const long long label = labels[row];
    const bool valid = label >= 0;
    // merge the shards' statistics (one slot when the vocabulary is not split)
    float m = stats[row * 3 + 0], se = stats[row * 3 + 1], target = stats[row * 3 + 2];
    for (int r = 1; r < slots; ++r) {
      const float* other = stats + ((long long)r * rows + row) * 3;
      const float om = other[0];
      const float nm = fmaxf(m, om);
      se = se * __expf(m - nm) + other[1] * __expf(om - nm);
      m = nm;
      target += other[2];
    }
    const float lse = m + __logf(se);
    if (threadIdx.x == 0) {
      if (loss_out) loss_out[row] = valid ? (lse - target) : 0.f;
      if (z_out) z_out[row] = valid ? lse * lse : 0.f;
    }
    if (!g) continue;
    const float inv = 1.f / se;
    const float pc = valid ? gscale * (1.f + 2.f * z_coef * lse) * logits_scale : 0.f;
    const float lc = valid ? gscale * logits_scale : 0.f;
    const long long lab = label - vocab_begin;
    const int nvec = cols / VN;
    for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
      float f[VN];
      Vec<T>::load(p + vi * VN, f);
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        float v = pc * __expf(f[j] * logits_scale - m) * inv;
        if ((long long)(vi * VN + j) == lab) v -= lc;
        f[j] = v;
      }
      Vec<T>::store(g + vi * VN, f);
    }
    for (int c = nvec * VN + threadIdx.x; c < cols; c += kThreads) {
      float f;
      if constexpr (sizeof(T) == 2) f = bf2f(p[c]); else f = p[c];
      float v = pc * __expf(f * logits_scale - m) * inv;
      if ((long long)c == lab) v -= lc;
      if constexpr (sizeof(T) == 2) g[c] = f2bf(v); else g[c] = v;
    }
  }
}

}  // namespace

static int ce_stats_launch(const void* logits, int dtype, const long long* labels, float* stats, int rows, int cols, long long ld,
                           long long vocab_begin, float logits_scale, const StatPeers& peers, cudaStream_t stream);

FLB_API int flb_ce_stats(const void* logits, int dtype, const long long* labels, float* stats, int rows, int cols,
                         long long ld, long long vocab_begin, float logits_scale, cudaStream_t stream) {
  StatPeers none{};
  return ce_stats_launch(logits, dtype, labels, stats, rows, cols, ld, vocab_begin, logits_scale, none, stream);
}

// peer_stats[r]: rank r's statistics buffer [world, rows, 3] fp32 (peer-mapped); this rank fills slot `rank` of each.
FLB_API int flb_ce_stats_exchange(const void* logits, int dtype, const long long* labels, const void* const* peer_stats, int rank, int world,
                                  int rows, int cols, long long ld, long long vocab_begin, float logits_scale, cudaStream_t stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return FLB_ERR_SHAPE;
  StatPeers peers{};
  for (int r = 0; r < world; ++r) peers.p[r] = (float*)peer_stats[r];
  peers.world = world;
  peers.rank = rank;
  return ce_stats_launch(logits, dtype, labels, nullptr, rows, cols, ld, vocab_begin, logits_scale, peers, stream);
}

static int ce_stats_launch(const void* logits, int dtype, const long long* labels, float* stats, int rows, int cols, long long ld,
                           long long vocab_begin, float logits_scale, const StatPeers& peers, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return FLB_ERR_SHAPE;
  if (dtype == 1) {
    if (ld % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return FLB_ERR_SHAPE;
    ce_stats_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)logits, labels, stats, rows, cols, ld, vocab_begin, logits_scale, peers);
  } else {
    if (ld % 4 || (reinterpret_cast<uintptr_t>(logits) & 15)) return FLB_ERR_SHAPE;
    ce_stats_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, labels, stats, rows, cols, ld, vocab_begin, logits_scale, peers);
  }
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_ce_grad_slots(const void* logits, int dtype, const long long* labels, const float* stats, int slots, void* grad,
                              float* loss_out, float* z_out, int rows, int cols, long long ld, long long ld_grad,
                              long long vocab_begin, float logits_scale, float grad_scale, const float* grad_scale_ptr,
                              float z_coef, cudaStream_t stream);

FLB_API int flb_ce_grad(const void* logits, int dtype, const long long* labels, const float* stats, void* grad,
                        float* loss_out, float* z_out, int rows, int cols, long long ld, long long ld_grad,
                        long long vocab_begin, float logits_scale, float grad_scale, const float* grad_scale_ptr,
                        float z_coef, cudaStream_t stream) {
  return flb_ce_grad_slots(logits, dtype, labels, stats, 1, grad, loss_out, z_out, rows, cols, ld, ld_grad, vocab_begin, logits_scale, grad_scale,
                           grad_scale_ptr, z_coef, stream);
}

// stats: [slots, rows, 3]; the slots are merged per token.
FLB_API int flb_ce_grad_slots(const void* logits, int dtype, const long long* labels, const float* stats, int slots, void* grad,
                              float* loss_out, float* z_out, int rows, int cols, long long ld, long long ld_grad,
                              long long vocab_begin, float logits_scale, float grad_scale, const float* grad_scale_ptr,
                              float z_coef, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || slots < 1) return FLB_ERR_SHAPE;
  if (dtype == 1) {
    if (ld % 8 || ld_grad % 8) return FLB_ERR_SHAPE;
    ce_grad_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)logits, labels, stats, (__nv_bfloat16*)grad, loss_out, z_out, rows, cols, ld, ld_grad, vocab_begin, logits_scale, grad_scale, grad_scale_ptr, z_coef, slots);
  } else {
    if (ld % 4 || ld_grad % 4) return FLB_ERR_SHAPE;
    ce_grad_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, labels, stats, (float*)grad, loss_out, z_out, rows, cols, ld, ld_grad, vocab_begin, logits_scale, grad_scale, grad_scale_ptr, z_coef, slots);
  }
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
