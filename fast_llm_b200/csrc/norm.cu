// RMSNorm / LayerNorm forward and backward for [rows, cols] bf16 activations (fp32 math).
//
// Forward optionally fuses the residual add that precedes the norm in a pre-norm decoder block:
//     r = x + delta ; y = norm(r) * w (+ b)           (r is written back as the new residual stream)
// Backward optionally fuses the add of the residual-stream gradient:
//     dx = d(norm)/dx + dres
// and produces per-CTA partial sums of dW (and dB), reduced by a second kernel that adds into (or overwrites)
// the fp32 / bf16 gradient buffer.  One CTA owns whole rows; a row lives in registers between the two passes.
#include "common.cuh"

namespace {

using namespace flb;
constexpr int kThreads = 256;

template <int VPT, bool LAYER_NORM>
__global__ void __launch_bounds__(kThreads)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ res_out, __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                float* __restrict__ mean_out, int rows, int cols, float eps, int zero_centered) {
  __shared__ float scratch[32];
  const int nvec = cols >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = (long long)row * cols;
    float v[VPT][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        bf16x8 p = *reinterpret_cast<const bf16x8*>(x + base + vec * 8);
        unpack8(p, v[i]);
        if (delta) {
          float d[8];
          bf16x8 q = *reinterpret_cast<const bf16x8*>(delta + base + vec * 8);
          unpack8(q, d);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += d[j];
          if (res_out) {
            bf16x8 o = pack8(v[i]);
            *reinterpret_cast<bf16x8*>(res_out + base + vec * 8) = o;
            unpack8(o, v[i]);  // normalise the rounded residual: backward sees exactly this tensor
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s += v[i][j];
          ss += v[i][j] * v[i][j];
        }
      }
    }
    float mean = 0.f;
    if (LAYER_NORM) {
      mean = block_sum(s, scratch) / cols;
      ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vec = threadIdx.x + i * kThreads;
        if (vec < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float c = v[i][j] - mean;
            ss += c * c;
          }
        }
      }
    }
    const float var = block_sum(ss, scratch) / cols;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (LAYER_NORM && mean_out) mean_out[row] = mean;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        float o[8];
        if (w) {
          float wf[8];
          unpack8(*reinterpret_cast<const bf16x8*>(w + vec * 8), wf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * (zero_centered ? wf[j] + 1.f : wf[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd;
        }
        if (LAYER_NORM && b) {
          float bfv[8];
          unpack8(*reinterpret_cast<const bf16x8*>(b + vec * 8), bfv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += bfv[j];
        }
        *reinterpret_cast<bf16x8*>(y + base + vec * 8) = pack8(o);
      }
    }
  }
}

template <int VPT, bool LAYER_NORM>
__global__ void __launch_bounds__(kThreads)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                const float* __restrict__ mean_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, float* __restrict__ db_partial,
                int rows, int cols, int zero_centered) {
  __shared__ float scratch[32];
  const int nvec = cols >> 3;
  float dw_acc[VPT][8], db_acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = db_acc[i][j] = 0.f;

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = (long long)row * cols;
    const float rstd = rstd_in[row];
    const float mean = LAYER_NORM ? mean_in[row] : 0.f;
    float xh[VPT][8], g[VPT][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        float xv[8], dyv[8], wf[8];
        unpack8(*reinterpret_cast<const bf16x8*>(x + base + vec * 8), xv);
        unpack8(*reinterpret_cast<const bf16x8*>(dy + base + vec * 8), dyv);
        if (w) unpack8(*reinterpret_cast<const bf16x8*>(w + vec * 8), wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          const float wj = w ? (zero_centered ? wf[j] + 1.f : wf[j]) : 1.f;
          g[i][j] = dyv[j] * wj;
          dw_acc[i][j] += dyv[j] * xh[i][j];
          db_acc[i][j] += dyv[j];
          s1 += g[i][j] * xh[i][j];
          s2 += g[i][j];
        }
      }
    }
    const float m1 = block_sum(s1, scratch) / cols;
    const float m2 = LAYER_NORM ? block_sum(s2, scratch) / cols : 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * m1 - m2);
        if (dres) {
          float d[8];
          unpack8(*reinterpret_cast<const bf16x8*>(dres + base + vec * 8), d);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += d[j];
        }
        *reinterpret_cast<bf16x8*>(dx + base + vec * 8) = pack8(o);
      }
    }
  }
  if (dw_partial) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        float* dst = dw_partial + (long long)blockIdx.x * cols + vec * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = dw_acc[i][j];
        if (LAYER_NORM && db_partial) {
          float* dstb = db_partial + (long long)blockIdx.x * cols + vec * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) dstb[j] = db_acc[i][j];
        }
      }
    }
  }
}

// out[c] (+)= sum_p partial[p][c]; out is fp32 or bf16.  A block owns 32 columns; its 32 x 32 threads split the parts 32 ways
// (coalesced 128-byte rows), then the 32 partial sums of a column are added in a fixed order through shared memory.
constexpr int kColsumCols = 32, kColsumSplit = 32;
template <typename OutT>
__global__ void __launch_bounds__(kColsumCols * kColsumSplit) colsum_kernel(const float* __restrict__ partial, OutT* __restrict__ out, int parts,
                                                                            int cols, int accumulate) {
  __shared__ float sums[kColsumSplit][kColsumCols + 1];
  const int lane = threadIdx.x % kColsumCols, group = threadIdx.x / kColsumCols;
  const int c = blockIdx.x * kColsumCols + lane;
  float s = 0.f;
  if (c < cols)
    for (int p = group; p < parts; p += kColsumSplit) s += partial[(long long)p * cols + c];
  sums[group][lane] = s;
  __syncthreads();
  if (group == 0 && c < cols) {
    float total = 0.f;
#pragma unroll
    for (int g = 0; g < kColsumSplit; ++g) total += sums[g][lane];
    if constexpr (sizeof(OutT) == 4) {
      out[c] = accumulate ? out[c] + total : total;
    } else {
      out[c] = f2bf(accumulate ? bf2f(out[c]) + total : total);
    }
  }
}

template <bool LN>
int fwd_dispatch(int vpt, dim3 grid, cudaStream_t st, const __nv_bfloat16* x, const __nv_bfloat16* delta,
                 const __nv_bfloat16* w, const __nv_bfloat16* b, __nv_bfloat16* res_out, __nv_bfloat16* y, float* rstd,
                 float* mean, int rows, int cols, float eps, int zc) {
  switch (vpt) {
    case 1: norm_fwd_kernel<1, LN><<<grid, kThreads, 0, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc); break;
    case 2: norm_fwd_kernel<2, LN><<<grid, kThreads, 0, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc); break;
    case 4: norm_fwd_kernel<4, LN><<<grid, kThreads, 0, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc); break;
    case 8: norm_fwd_kernel<8, LN><<<grid, kThreads, 0, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc); break;
    default: return FLB_ERR_SHAPE;
  }
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
template <bool LN>
int bwd_dispatch(int vpt, dim3 grid, cudaStream_t st, const __nv_bfloat16* dy, const __nv_bfloat16* x,
                 const __nv_bfloat16* w, const float* rstd, const float* mean, const __nv_bfloat16* dres,
                 __nv_bfloat16* dx, float* dwp, float* dbp, int rows, int cols, int zc) {
  switch (vpt) {
    case 1: norm_bwd_kernel<1, LN><<<grid, kThreads, 0, st>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, cols, zc); break;
    case 2: norm_bwd_kernel<2, LN><<<grid, kThreads, 0, st>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, cols, zc); break;
    case 4: norm_bwd_kernel<4, LN><<<grid, kThreads, 0, st>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, cols, zc); break;
    case 8: norm_bwd_kernel<8, LN><<<grid, kThreads, 0, st>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, cols, zc); break;
    default: return FLB_ERR_SHAPE;
  }
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

int pick_vpt(int cols) {
  if (cols % 8) return 0;
  const int nvec = cols / 8;
  for (int v = 1; v <= 8; v *= 2)
    if (nvec <= v * kThreads) return v;
  return 0;
}

}  // namespace

// y = norm(x + delta) * w (+ b).  delta, res_out, w, b, mean may be null.  layer_norm=0 -> RMSNorm.
// cols must be a multiple of 8 and at most 16384.
FLB_API int flb_norm_fwd(const void* x, const void* delta, const void* w, const void* b, void* res_out, void* y,
                         float* rstd, float* mean, int rows, int cols, float eps, int zero_centered, int layer_norm,
                         cudaStream_t stream) {
  const int vpt = pick_vpt(cols);
  if (!vpt || rows <= 0) return FLB_ERR_SHAPE;
  dim3 grid(rows);
  auto X = (const __nv_bfloat16*)x; auto D = (const __nv_bfloat16*)delta; auto W = (const __nv_bfloat16*)w;
  auto B = (const __nv_bfloat16*)b; auto R = (__nv_bfloat16*)res_out; auto Y = (__nv_bfloat16*)y;
  if (layer_norm) return fwd_dispatch<true>(vpt, grid, stream, X, D, W, B, R, Y, rstd, mean, rows, cols, eps, zero_centered);
  return fwd_dispatch<false>(vpt, grid, stream, X, D, W, B, R, Y, rstd, mean, rows, cols, eps, zero_centered);
}

// Number of per-CTA partial rows flb_norm_bwd writes into dw_partial / db_partial.
FLB_API int flb_norm_bwd_parts(int rows) { return rows < 1184 ? rows : 1184; }  // 8 resident CTAs on each of 148 SMs

// dx = dnorm(dy) (+ dres).  dw_partial/db_partial: [flb_norm_bwd_parts(rows), cols] fp32 scratch (may be null
// to skip parameter gradients).
FLB_API int flb_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const float* mean,
                         const void* dres, void* dx, float* dw_partial, float* db_partial, int rows, int cols,
                         int zero_centered, int layer_norm, cudaStream_t stream) {
  const int vpt = pick_vpt(cols);
  if (!vpt || rows <= 0) return FLB_ERR_SHAPE;
  dim3 grid(flb_norm_bwd_parts(rows));
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto DR = (const __nv_bfloat16*)dres; auto DX = (__nv_bfloat16*)dx;
  if (layer_norm) return bwd_dispatch<true>(vpt, grid, stream, DY, X, W, rstd, mean, DR, DX, dw_partial, db_partial, rows, cols, zero_centered);
  return bwd_dispatch<false>(vpt, grid, stream, DY, X, W, rstd, mean, DR, DX, dw_partial, db_partial, rows, cols, zero_centered);
}

// out[cols] (+)= column sums of partial[parts, cols].  out_is_bf16 selects the gradient-buffer dtype.
FLB_API int flb_colsum(const float* partial, void* out, int parts, int cols, int accumulate, int out_is_bf16,
                       cudaStream_t stream) {
  if (parts <= 0 || cols <= 0) return FLB_ERR_SHAPE;
  const int threads = kColsumCols * kColsumSplit;
  const int blocks = (cols + kColsumCols - 1) / kColsumCols;
  if (out_is_bf16) colsum_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(partial, (__nv_bfloat16*)out, parts, cols, accumulate);
  else colsum_kernel<float><<<blocks, threads, 0, stream>>>(partial, (float*)out, parts, cols, accumulate);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
