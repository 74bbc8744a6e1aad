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
      if (lm > m) { s *= expf(m - lm); m = lm; }
#pragma unroll
      for (int j = 0; j < VN; ++j) s += expf(f[j] * logits_scale - m);
    }
    for (int c = nvec * VN + threadIdx.x; c < cols; c += kThreads) {
      float f;
      if constexpr (sizeof(T) == 2) f = bf2f(p[c]) * logits_scale; else f = p[c] * logits_scale;
      if (f > m) { s *= expf(m - f); m = f; }
      s += expf(f - m);
    }
    const float gm = block_max(m, scratch);
    const float contrib = (m == -INFINITY) ? 0.f : s * expf(m - gm);
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
      se = se * expf(m - nm) + other[1] * expf(om - nm);
      m = nm;
      target += other[2];
    }
    const float lse = m + logf(se);
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
        float v = pc * expf(f[j] * logits_scale - m) * inv;
        if ((long long)(vi * VN + j) == lab) v -= lc;
        f[j] = v;
      }
      Vec<T>::store(g + vi * VN, f);
    }
    for (int c = nvec * VN + threadIdx.x; c < cols; c += kThreads) {
      float f;
      if constexpr (sizeof(T) == 2) f = bf2f(p[c]); else f = p[c];
      float v = pc * expf(f * logits_scale - m) * inv;
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

// ---------------------------------------------------------------------------------------------------------------------
// Losses over one shared softmax.  Any loss that depends on the logits of a token only through lse = logsumexp(s) and
// the target logit s_label (cross-entropy, z-loss, label KL, the GRPO / GSPO / DPO log-probability ratios) has the
// logit gradient   a_t * softmax_j + b_t * [j == label_t]   with a_t = dL/dlse, b_t = dL/ds_label.  The host computes the
// two per-token coefficients of all such losses from the merged statistics (tiny [tokens] vectors), adds them up, and
// ONE pass over the logits writes the gradient of their sum (in place over the logits, or added to an existing gradient).
namespace {
using namespace flb;

template <typename T>
__global__ void __launch_bounds__(kThreads)
softmax_coeff_grad_kernel(const T* __restrict__ logits, const long long* __restrict__ labels, const float* __restrict__ stats,
                          int slots, const float* __restrict__ prob_coeff, const float* __restrict__ label_coeff,
                          T* __restrict__ grad, int rows, int cols, long long ld, long long ld_grad, long long vocab_begin,
                          float logits_scale, int accumulate) {
  constexpr int VN = Vec<T>::N;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = logits + (long long)row * ld;
    T* g = grad + (long long)row * ld_grad;
    float m = stats[row * 3 + 0], se = stats[row * 3 + 1];
    for (int r = 1; r < slots; ++r) {
      const float* other = stats + ((long long)r * rows + row) * 3;
      const float om = other[0];
      const float nm = fmaxf(m, om);
      se = se * expf(m - nm) + other[1] * expf(om - nm);
      m = nm;
    }
    const float pc = prob_coeff[row] / se;
    const float lc = label_coeff[row];
    const long long lab = labels ? labels[row] - vocab_begin : -1;
    const int nvec = cols / VN;
    for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
      float f[VN];
      Vec<T>::load(p + vi * VN, f);
      float old[VN];
      if (accumulate) Vec<T>::load(g + vi * VN, old);
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        float v = pc * expf(f[j] * logits_scale - m);
        if ((long long)(vi * VN + j) == lab) v += lc;
        f[j] = accumulate ? old[j] + v : v;
      }
      Vec<T>::store(g + vi * VN, f);
    }
    for (int c = nvec * VN + threadIdx.x; c < cols; c += kThreads) {
      float f;
      if constexpr (sizeof(T) == 2) f = bf2f(p[c]); else f = p[c];
      float v = pc * expf(f * logits_scale - m);
      if ((long long)c == lab) v += lc;
      if (accumulate) {
        if constexpr (sizeof(T) == 2) v += bf2f(g[c]); else v += g[c];
      }
      if constexpr (sizeof(T) == 2) g[c] = f2bf(v); else g[c] = v;
    }
  }
}

// Online-softmax pair: running maximum with a sum that is rescaled when the maximum moves, plus `NW` sums weighted by
// the same exponentials.
template <int NW>
struct Online {
  float m = -INFINITY, s = 0.f, w[NW];
  __device__ __forceinline__ Online() {
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] = 0.f;
  }
  __device__ __forceinline__ void add(float x, const float* weights) {
    if (x > m) {
      const float r = expf(m - x);  // exp(-inf) = 0 on the first element
      s *= r;
#pragma unroll
      for (int i = 0; i < NW; ++i) w[i] *= r;
      m = x;
    }
    const float e = expf(x - m);
    s += e;
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] += e * weights[i];
  }
  // Block-wide merge; every thread returns the merged values.
  __device__ __forceinline__ void reduce(float* scratch) {
    const float gm = block_max(m, scratch);
    const float r = (m == -INFINITY) ? 0.f : expf(m - gm);
    s = block_sum(s * r, scratch);
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] = block_sum(w[i] * r, scratch);
    m = gm;
  }
};

// Statistics of a student / teacher logits pair for cross-entropy, forward KL and reverse KL from a distribution.
// With s = student * student_scale, t = teacher * teacher_scale, per row:
//   out[0] = max s     out[1] = sum e^(s - max s)     out[2] = sum e^(s - max s) (s - t)
//   out[3] = max t     out[4] = sum e^(t - max t)     out[5] = sum e^(t - max t) s     out[6] = sum e^(t - max t) t
// Shards of a split vocabulary merge like any online softmax (rescale by the difference of the maxima, then add).
template <typename T>
__global__ void __launch_bounds__(kThreads)
dist_stats_kernel(const T* __restrict__ student, const T* __restrict__ teacher, float* __restrict__ out, int rows, int cols,
                  long long ld_s, long long ld_t, float student_scale, float teacher_scale) {
  __shared__ float scratch[32];
  constexpr int VN = Vec<T>::N;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* ps = student + (long long)row * ld_s;
    const T* pt = teacher + (long long)row * ld_t;
    Online<1> os;
    Online<2> ot;
    const int nvec = cols / VN;
    for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
      float fs[VN], ft[VN];
      Vec<T>::load(ps + vi * VN, fs);
      Vec<T>::load(pt + vi * VN, ft);
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        const float s = fs[j] * student_scale, t = ft[j] * teacher_scale;
        const float ws = s - t;
        os.add(s, &ws);
        const float wt[2] = {s, t};
        ot.add(t, wt);
      }
    }
    for (int c = nvec * VN + threadIdx.x; c < cols; c += kThreads) {
      float s, t;
      if constexpr (sizeof(T) == 2) { s = bf2f(ps[c]); t = bf2f(pt[c]); } else { s = ps[c]; t = pt[c]; }
      s *= student_scale; t *= teacher_scale;
      const float ws = s - t;
      os.add(s, &ws);
      const float wt[2] = {s, t};
      ot.add(t, wt);
    }
    os.reduce(scratch);
    ot.reduce(scratch);
    if (threadIdx.x == 0) {
      float* o = out + (long long)row * 7;
      o[0] = os.m; o[1] = os.s; o[2] = os.w[0];
      o[3] = ot.m; o[4] = ot.s; o[5] = ot.w[0]; o[6] = ot.w[1];
    }
  }
}

// grad_j (=|+=) a_t p_j + b_t q_j + c_t p_j (s_j - t_j),  p = softmax(s), q = softmax(t), given lse_s and lse_t per row.
//   cross-entropy / forward KL:  a = g, b = -g, c = 0          reverse KL:  a = g (lse_t - lse_s - L), b = 0, c = g
template <typename T>
__global__ void __launch_bounds__(kThreads)
dist_grad_kernel(const T* __restrict__ student, const T* __restrict__ teacher, const float* __restrict__ lse_s,
                 const float* __restrict__ lse_t, const float* __restrict__ ca, const float* __restrict__ cb,
                 const float* __restrict__ cc, T* __restrict__ grad, int rows, int cols, long long ld_s, long long ld_t,
                 long long ld_grad, float student_scale, float teacher_scale, int accumulate) {
  constexpr int VN = Vec<T>::N;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* ps = student + (long long)row * ld_s;
    const T* pt = teacher + (long long)row * ld_t;
    T* g = grad + (long long)row * ld_grad;
    const float ls = lse_s[row], lt = lse_t[row], a = ca[row], b = cb[row], c = cc[row];
    auto value = [&](float s, float t) {
      s *= student_scale; t *= teacher_scale;
      const float p = expf(s - ls);
      return p * (a + c * (s - t)) + b * expf(t - lt);
    };
    const int nvec = cols / VN;
    for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
      float fs[VN], ft[VN], old[VN];
      Vec<T>::load(ps + vi * VN, fs);
      Vec<T>::load(pt + vi * VN, ft);
      if (accumulate) Vec<T>::load(g + vi * VN, old);
#pragma unroll
      for (int j = 0; j < VN; ++j) fs[j] = (accumulate ? old[j] : 0.f) + value(fs[j], ft[j]);
      Vec<T>::store(g + vi * VN, fs);
    }
    for (int col = nvec * VN + threadIdx.x; col < cols; col += kThreads) {
      float s, t, o = 0.f;
      if constexpr (sizeof(T) == 2) { s = bf2f(ps[col]); t = bf2f(pt[col]); if (accumulate) o = bf2f(g[col]); }
      else { s = ps[col]; t = pt[col]; if (accumulate) o = g[col]; }
      const float v = o + value(s, t);
      if constexpr (sizeof(T) == 2) g[col] = f2bf(v); else g[col] = v;
    }
  }
}

bool aligned_rows(const void* p, long long ld, int dtype) {
  const int vec = dtype == 1 ? 8 : 4;
  return ld % vec == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}
}  // namespace

// grad[t, j] (=|+=) prob_coeff[t] * softmax(logits * scale)[t, j] + label_coeff[t] * [j == labels[t] - vocab_begin].
// stats: [slots, rows, 3] as written by flb_ce_stats / flb_ce_stats_exchange (merged per token).  labels may be null
// (no label term).  grad may alias logits when accumulate == 0.  dtype: 0 fp32, 1 bf16.
FLB_API int flb_softmax_coeff_grad(const void* logits, int dtype, const long long* labels, const float* stats, int slots,
                                   const float* prob_coeff, const float* label_coeff, void* grad, int rows, int cols, long long ld,
                                   long long ld_grad, long long vocab_begin, float logits_scale, int accumulate, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || slots < 1) return FLB_ERR_SHAPE;
  if (!aligned_rows(logits, ld, dtype) || !aligned_rows(grad, ld_grad, dtype)) return FLB_ERR_SHAPE;
  if (dtype == 1)
    softmax_coeff_grad_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)logits, labels, stats, slots, prob_coeff, label_coeff,
                                                                             (__nv_bfloat16*)grad, rows, cols, ld, ld_grad, vocab_begin, logits_scale, accumulate);
  else
    softmax_coeff_grad_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, labels, stats, slots, prob_coeff, label_coeff, (float*)grad,
                                                                     rows, cols, ld, ld_grad, vocab_begin, logits_scale, accumulate);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// out: [rows, 7] fp32 (see dist_stats_kernel).  student and teacher share dtype (0 fp32, 1 bf16) and column count.
FLB_API int flb_dist_stats(const void* student, const void* teacher, int dtype, float* out, int rows, int cols, long long ld_s,
                           long long ld_t, float student_scale, float teacher_scale, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return FLB_ERR_SHAPE;
  if (!aligned_rows(student, ld_s, dtype) || !aligned_rows(teacher, ld_t, dtype)) return FLB_ERR_SHAPE;
  if (dtype == 1)
    dist_stats_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)student, (const __nv_bfloat16*)teacher, out, rows, cols,
                                                                     ld_s, ld_t, student_scale, teacher_scale);
  else
    dist_stats_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)student, (const float*)teacher, out, rows, cols, ld_s, ld_t,
                                                             student_scale, teacher_scale);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// grad may alias student when accumulate == 0.  lse_s, lse_t, a, b, c: [rows] fp32.
FLB_API int flb_dist_grad(const void* student, const void* teacher, int dtype, const float* lse_s, const float* lse_t, const float* a,
                          const float* b, const float* c, void* grad, int rows, int cols, long long ld_s, long long ld_t,
                          long long ld_grad, float student_scale, float teacher_scale, int accumulate, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return FLB_ERR_SHAPE;
  if (!aligned_rows(student, ld_s, dtype) || !aligned_rows(teacher, ld_t, dtype) || !aligned_rows(grad, ld_grad, dtype)) return FLB_ERR_SHAPE;
  if (dtype == 1)
    dist_grad_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)student, (const __nv_bfloat16*)teacher, lse_s, lse_t, a, b, c,
                                                                    (__nv_bfloat16*)grad, rows, cols, ld_s, ld_t, ld_grad, student_scale, teacher_scale,
                                                                    accumulate);
  else
    dist_grad_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)student, (const float*)teacher, lse_s, lse_t, a, b, c, (float*)grad, rows, cols,
                                                            ld_s, ld_t, ld_grad, student_scale, teacher_scale, accumulate);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
