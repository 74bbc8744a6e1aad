// RMSNorm / LayerNorm forward and backward for [rows, cols] bf16 activations (fp32 math).
//
// Forward optionally fuses the residual add that precedes the norm in a pre-norm decoder block:
//     r = x + delta ; y = norm(r) * w (+ b)           (r is written back as the new residual stream)
// Backward optionally fuses the add of the residual-stream gradient:
//     dx = d(norm)/dx + dres
// and produces per-CTA partial sums of dW (and dB), reduced by a second kernel that adds into (or overwrites)
// the fp32 / bf16 gradient buffer.  One CTA owns whole rows; a row lives in registers between the two passes.
#include "tcgen05.cuh"
#include <mutex>
#include <vector>

namespace {

using namespace flb;
constexpr int kThreads = 256;

// Both kernels are persistent: a CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and issues the loads of its NEXT row
// (kept as packed bf16 in registers) before it reduces and stores the current one, so every resident CTA always has a row of
// reads in flight and the block-wide reduction and the stores of one row hide under the DRAM latency of the next.
template <int VPT, bool LAYER_NORM>
__global__ void __launch_bounds__(kThreads, VPT <= 2 ? 4 : (VPT == 4 ? 2 : 1))
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ res_out, __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                float* __restrict__ mean_out, int rows, int cols, float eps, int zero_centered) {
  __shared__ float scratch[32];
  const int nvec = cols >> 3;
  bf16x8 nx[VPT], nd[VPT];
  auto fetch = [&](int row) {
    const long long base = (long long)row * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        nx[i] = *reinterpret_cast<const bf16x8*>(x + base + vec * 8);
        if (delta) nd[i] = *reinterpret_cast<const bf16x8*>(delta + base + vec * 8);
      }
    }
  };
  if ((int)blockIdx.x < rows) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = (long long)row * cols;
    float v[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        unpack8(nx[i], v[i]);
        if (delta) {
          float d[8];
          unpack8(nd[i], d);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += d[j];
        }
      }
    }
    if (row + (int)gridDim.x < rows) fetch(row + gridDim.x);
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        if (delta && res_out) {
          bf16x8 o = pack8(v[i]);
          *reinterpret_cast<bf16x8*>(res_out + base + vec * 8) = o;
          unpack8(o, v[i]);  // normalise the rounded residual: backward sees exactly this tensor
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

// The row is held as packed bf16 (x, dy) and unpacked once per pass instead of living in fp32 registers between the passes:
// half the registers, so three CTAs stay resident per SM beside the prefetched next row.
template <int VPT, bool LAYER_NORM>
__global__ void __launch_bounds__(kThreads, VPT <= 2 ? 3 : 1)
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

  bf16x8 nx[VPT], ny[VPT];
  float n_rstd = 0.f, n_mean = 0.f;
  auto fetch = [&](int row) {
    const long long base = (long long)row * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        nx[i] = *reinterpret_cast<const bf16x8*>(x + base + vec * 8);
        ny[i] = *reinterpret_cast<const bf16x8*>(dy + base + vec * 8);
      }
    }
    n_rstd = rstd_in[row];
    if (LAYER_NORM) n_mean = mean_in[row];
  };
  if ((int)blockIdx.x < rows) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = (long long)row * cols;
    const float rstd = n_rstd;
    const float mean = LAYER_NORM ? n_mean : 0.f;
    bf16x8 cx[VPT], cy[VPT], cr[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      cx[i] = nx[i];
      cy[i] = ny[i];
      const int vec = threadIdx.x + i * kThreads;
      if (dres && vec < nvec) cr[i] = *reinterpret_cast<const bf16x8*>(dres + base + vec * 8);  // needed only after the reduction
    }
    if (row + (int)gridDim.x < rows) fetch(row + gridDim.x);
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        float xv[8], dyv[8], wf[8];
        unpack8(cx[i], xv);
        unpack8(cy[i], dyv);
        if (w) unpack8(*reinterpret_cast<const bf16x8*>(w + vec * 8), wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          const float wj = w ? (zero_centered ? wf[j] + 1.f : wf[j]) : 1.f;
          const float g = dyv[j] * wj;
          dw_acc[i][j] += dyv[j] * xh;
          db_acc[i][j] += dyv[j];
          s1 += g * xh;
          s2 += g;
        }
      }
    }
    const float m1 = block_sum(s1, scratch) / cols;
    const float m2 = LAYER_NORM ? block_sum(s2, scratch) / cols : 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        float xv[8], dyv[8], wf[8], o[8];
        unpack8(cx[i], xv);
        unpack8(cy[i], dyv);
        if (w) unpack8(*reinterpret_cast<const bf16x8*>(w + vec * 8), wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          const float wj = w ? (zero_centered ? wf[j] + 1.f : wf[j]) : 1.f;
          o[j] = rstd * (dyv[j] * wj - xh * m1 - m2);
        }
        if (dres) {
          float d[8];
          unpack8(cr[i], d);
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
        for (int j = 0; j < 8; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(dw_acc[i][j], dw_acc[i][j + 1], dw_acc[i][j + 2], dw_acc[i][j + 3]);
        if (LAYER_NORM && db_partial) {
          float* dstb = db_partial + (long long)blockIdx.x * cols + vec * 8;
#pragma unroll
          for (int j = 0; j < 8; j += 4) *reinterpret_cast<float4*>(dstb + j) = make_float4(db_acc[i][j], db_acc[i][j + 1], db_acc[i][j + 2], db_acc[i][j + 3]);
        }
      }
    }
  }
}

// ---- the same two kernels with the rows staged through shared memory by bulk copies -------------------------------------
// A ring of `stages` row slots per CTA; one thread issues `cp.async.bulk` copies of whole rows (x and delta, or x, dy and
// dres) that complete on the slot's mbarrier, so a CTA keeps `stages` rows of reads in flight without holding them in
// registers (the register kernels above stay for rows too wide for the ring).  A slot is re-armed for the row `stages`
// iterations ahead right after the block-wide reduction, whose __syncthreads also tells that every thread has taken its
// values out of the slot.  The wait on a slot is bounded: on expiry the kernel raises g_norm_error and every thread returns.
__device__ int g_norm_error = 0;
constexpr long long kNormWaitLimitCycles = 4000000000ll;  // about 2 s

__device__ __forceinline__ void bulk_load_row(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// All threads wait for the slot; returns false (for all of them) when the limit ran out.
__device__ __forceinline__ bool slot_wait(uint32_t bar, uint32_t parity) {
  int failed = 0;
  if (!flb_tc::mbar_try_wait(bar, parity)) {
    const long long t0 = clock64();
    while (!flb_tc::mbar_try_wait(bar, parity)) {
      if (clock64() - t0 > kNormWaitLimitCycles) {
        failed = 1;
        atomicExch(&g_norm_error, 1);
        break;
      }
    }
  }
  return !__syncthreads_or(failed);
}

__device__ __forceinline__ void ring_init(uint32_t bar_base, int stages) {
  for (int s = 0; s < stages; ++s) flb_tc::mbar_init(bar_base + 8u * s, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

template <int VPT, bool LAYER_NORM>
__global__ void __launch_bounds__(kThreads)
norm_fwd_staged_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                       const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                       __nv_bfloat16* __restrict__ res_out, __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                       float* __restrict__ mean_out, int rows, int cols, float eps, int zero_centered, int stages) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ float scratch[32];
  const int nvec = cols >> 3;
  const uint32_t row_bytes = (uint32_t)cols * 2u;
  const uint32_t slot_bytes = delta ? 2u * row_bytes : row_bytes;
  const uint32_t ring_base = flb_tc::smem_u32(ring);
  const uint32_t bar_base = ring_base + (uint32_t)stages * slot_bytes;
  auto issue = [&](long long row, int slot) {
    const uint32_t bar = bar_base + 8u * slot;
    flb_tc::mbar_expect_tx(bar, slot_bytes);
    bulk_load_row(ring_base + slot * slot_bytes, x + row * cols, row_bytes, bar);
    if (delta) bulk_load_row(ring_base + slot * slot_bytes + row_bytes, delta + row * cols, row_bytes, bar);
  };
  if (threadIdx.x == 0) {
    ring_init(bar_base, stages);
    for (int s = 0; s < stages; ++s) {
      const long long row = (long long)blockIdx.x + (long long)s * gridDim.x;
      if (row < rows) issue(row, s);
    }
  }
  __syncthreads();
  int it = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
    const int slot = it % stages;
    if (!slot_wait(bar_base + 8u * slot, (uint32_t)(it / stages) & 1u)) return;
    const long long base = (long long)row * cols;
    const uint8_t* src = ring + slot * slot_bytes;
    float v[VPT][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        unpack8(*reinterpret_cast<const bf16x8*>(src + vec * 16), v[i]);
        if (delta) {
          float d[8];
          unpack8(*reinterpret_cast<const bf16x8*>(src + row_bytes + vec * 16), d);
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
    const float var = block_sum(ss, scratch) / cols;  // its barriers: every thread has read the slot
    if (threadIdx.x == 0) {
      const long long next = (long long)row + (long long)stages * gridDim.x;
      if (next < rows) issue(next, slot);
    }
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
norm_bwd_staged_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                       const float* __restrict__ mean_in, const __nv_bfloat16* __restrict__ dres,
                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, float* __restrict__ db_partial,
                       int rows, int cols, int zero_centered, int stages) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ float scratch[32];
  const int nvec = cols >> 3;
  const uint32_t row_bytes = (uint32_t)cols * 2u;
  const uint32_t slot_bytes = (dres ? 3u : 2u) * row_bytes;
  const uint32_t ring_base = flb_tc::smem_u32(ring);
  const uint32_t bar_base = ring_base + (uint32_t)stages * slot_bytes;
  auto issue = [&](long long row, int slot) {
    const uint32_t bar = bar_base + 8u * slot;
    const uint32_t dst = ring_base + slot * slot_bytes;
    flb_tc::mbar_expect_tx(bar, slot_bytes);
    bulk_load_row(dst, x + row * cols, row_bytes, bar);
    bulk_load_row(dst + row_bytes, dy + row * cols, row_bytes, bar);
    if (dres) bulk_load_row(dst + 2u * row_bytes, dres + row * cols, row_bytes, bar);
  };
  if (threadIdx.x == 0) {
    ring_init(bar_base, stages);
    for (int s = 0; s < stages; ++s) {
      const long long row = (long long)blockIdx.x + (long long)s * gridDim.x;
      if (row < rows) issue(row, s);
    }
  }
  __syncthreads();
  float dw_acc[VPT][8], db_acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = db_acc[i][j] = 0.f;
  int it = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
    const int slot = it % stages;
    const float rstd = rstd_in[row];
    const float mean = LAYER_NORM ? mean_in[row] : 0.f;
    if (!slot_wait(bar_base + 8u * slot, (uint32_t)(it / stages) & 1u)) return;
    const long long base = (long long)row * cols;
    const uint8_t* src = ring + slot * slot_bytes;
    // the row leaves the slot as packed bf16 (x, dy, dres: 12 registers per 8 columns) and is unpacked once per pass
    bf16x8 cx[VPT], cy[VPT], cr[VPT];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        cx[i] = *reinterpret_cast<const bf16x8*>(src + vec * 16);
        cy[i] = *reinterpret_cast<const bf16x8*>(src + row_bytes + vec * 16);
        if (dres) cr[i] = *reinterpret_cast<const bf16x8*>(src + 2u * row_bytes + vec * 16);
        float xv[8], dyv[8], wf[8];
        unpack8(cx[i], xv);
        unpack8(cy[i], dyv);
        if (w) unpack8(*reinterpret_cast<const bf16x8*>(w + vec * 8), wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          const float wj = w ? (zero_centered ? wf[j] + 1.f : wf[j]) : 1.f;
          const float g = dyv[j] * wj;
          dw_acc[i][j] += dyv[j] * xh;
          db_acc[i][j] += dyv[j];
          s1 += g * xh;
          s2 += g;
        }
      }
    }
    const float m1 = block_sum(s1, scratch) / cols;  // its barriers: every thread has read the slot
    if (threadIdx.x == 0) {
      const long long next = (long long)row + (long long)stages * gridDim.x;
      if (next < rows) issue(next, slot);
    }
    const float m2 = LAYER_NORM ? block_sum(s2, scratch) / cols : 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vec = threadIdx.x + i * kThreads;
      if (vec < nvec) {
        float xv[8], dyv[8], wf[8], o[8];
        unpack8(cx[i], xv);
        unpack8(cy[i], dyv);
        if (w) unpack8(*reinterpret_cast<const bf16x8*>(w + vec * 8), wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          const float wj = w ? (zero_centered ? wf[j] + 1.f : wf[j]) : 1.f;
          o[j] = rstd * (dyv[j] * wj - xh * m1 - m2);
        }
        if (dres) {
          float d[8];
          unpack8(cr[i], d);
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
        for (int j = 0; j < 8; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(dw_acc[i][j], dw_acc[i][j + 1], dw_acc[i][j + 2], dw_acc[i][j + 3]);
        if (LAYER_NORM && db_partial) {
          float* dstb = db_partial + (long long)blockIdx.x * cols + vec * 8;
#pragma unroll
          for (int j = 0; j < 8; j += 4) *reinterpret_cast<float4*>(dstb + j) = make_float4(db_acc[i][j], db_acc[i][j + 1], db_acc[i][j + 2], db_acc[i][j + 3]);
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

int sm_count() {
  static const int sms = [] {
    int device = 0, count = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
    return count;
  }();
  return sms;
}
// CTAs that are resident at once (occupancy of this instantiation x SMs): the persistent grid is one full wave, no tail
template <typename Kernel>
int resident_ctas(Kernel kernel) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess || per_sm <= 0) per_sm = 1;
  return per_sm * sm_count();
}
template <int VPT, bool LN>
int fwd_ctas() {
  static const int n = resident_ctas(norm_fwd_kernel<VPT, LN>);
  return n;
}
template <int VPT, bool LN>
int bwd_ctas() {
  static const int n = resident_ctas(norm_bwd_kernel<VPT, LN>);
  return n;
}
template <bool LN>
int bwd_ctas_for(int vpt) {
  switch (vpt) {
    case 1: return bwd_ctas<1, LN>();
    case 2: return bwd_ctas<2, LN>();
    case 4: return bwd_ctas<4, LN>();
    default: return bwd_ctas<8, LN>();
  }
}

// ---- plan of the staged kernels: ring depth, dynamic shared memory and the persistent grid
struct StagedPlan {
  int stages = 0;  // 0: use the register kernels
  int smem = 0;
  int ctas = 0;
};
bool staged_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("FLB_NORM");
    return !(v && v[0] == 'r');  // FLB_NORM=registers keeps the register kernels (for comparisons)
  }();
  return enabled;
}
// `slot_rows`: rows of `cols` bf16 per ring slot (forward: x and delta; backward: x, dy and dres).
template <typename Kernel>
StagedPlan make_plan(Kernel kernel, int cols, int slot_rows) {
  StagedPlan plan;
  if (!staged_enabled()) return plan;
  const int slot_bytes = slot_rows * cols * 2;
  // ring budgets that leave room for 3, 2 or 1 resident CTAs per SM; the first that holds 3 slots, else the first with 2
  const int budgets[3] = {73 * 1024, 110 * 1024, 220 * 1024};
  int stages = 0;
  for (int want = 3; want >= 2 && !stages; --want)
    for (int budget : budgets)
      if (budget / slot_bytes >= want) {
        stages = budget / slot_bytes < 4 ? budget / slot_bytes : 4;
        break;
      }
  if (!stages) return plan;
  const int smem = stages * slot_bytes + 8 * stages + 16;
  // the limit is a property of the kernel, not of this plan: raise it to the largest ring any plan may ask for
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 221 * 1024) != cudaSuccess) {
    cudaGetLastError();
    return plan;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem) != cudaSuccess || per_sm <= 0) {
    cudaGetLastError();
    return plan;
  }
  plan.stages = stages;
  plan.smem = smem;
  plan.ctas = per_sm * sm_count();
  return plan;
}
// One plan per (instantiation, cols, slot_rows); the few shapes of a model are looked up in a small table.
template <typename Kernel>
StagedPlan cached_plan(Kernel kernel, int cols, int slot_rows) {
  // all instantiations of one kernel template share this function (same pointer type): the kernel is part of the key
  struct Entry { Kernel kernel; int cols, slot_rows; StagedPlan plan; };
  static std::mutex mutex;
  static std::vector<Entry> table;
  std::lock_guard<std::mutex> lock(mutex);
  for (const Entry& e : table)
    if (e.kernel == kernel && e.cols == cols && e.slot_rows == slot_rows) return e.plan;
  table.push_back({kernel, cols, slot_rows, make_plan(kernel, cols, slot_rows)});
  return table.back().plan;
}
template <bool LN>
StagedPlan fwd_plan(int vpt, int cols, int slot_rows) {
  switch (vpt) {
    case 1: return cached_plan(norm_fwd_staged_kernel<1, LN>, cols, slot_rows);
    case 2: return cached_plan(norm_fwd_staged_kernel<2, LN>, cols, slot_rows);
    case 4: return cached_plan(norm_fwd_staged_kernel<4, LN>, cols, slot_rows);
    default: return cached_plan(norm_fwd_staged_kernel<8, LN>, cols, slot_rows);
  }
}
template <bool LN>
StagedPlan bwd_plan(int vpt, int cols) {
  switch (vpt) {  // slots always sized for x, dy and dres, so that the grid does not depend on dres being given
    case 1: return cached_plan(norm_bwd_staged_kernel<1, LN>, cols, 3);
    case 2: return cached_plan(norm_bwd_staged_kernel<2, LN>, cols, 3);
    case 4: return cached_plan(norm_bwd_staged_kernel<4, LN>, cols, 3);
    default: return cached_plan(norm_bwd_staged_kernel<8, LN>, cols, 3);
  }
}

template <bool LN>
int fwd_dispatch(int vpt, cudaStream_t st, const __nv_bfloat16* x, const __nv_bfloat16* delta,
                 const __nv_bfloat16* w, const __nv_bfloat16* b, __nv_bfloat16* res_out, __nv_bfloat16* y, float* rstd,
                 float* mean, int rows, int cols, float eps, int zc) {
  // Measured at [8192, 4096] with the residual add: the register kernel (next row prefetched) 0.057 ms, the staged one 0.062 ms;
  // the forward keeps few values per thread, so the ring buys nothing.  FLB_NORM=staged selects the staged forward.
  static const bool staged_forward = [] {
    const char* v = getenv("FLB_NORM");
    return v && v[0] == 's';
  }();
  const StagedPlan plan = staged_forward ? fwd_plan<LN>(vpt, cols, delta ? 2 : 1) : StagedPlan{};
  if (plan.stages) {
    const int grid = min(rows, plan.ctas);
    switch (vpt) {
      case 1: norm_fwd_staged_kernel<1, LN><<<grid, kThreads, plan.smem, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc, plan.stages); break;
      case 2: norm_fwd_staged_kernel<2, LN><<<grid, kThreads, plan.smem, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc, plan.stages); break;
      case 4: norm_fwd_staged_kernel<4, LN><<<grid, kThreads, plan.smem, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc, plan.stages); break;
      case 8: norm_fwd_staged_kernel<8, LN><<<grid, kThreads, plan.smem, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc, plan.stages); break;
      default: return FLB_ERR_SHAPE;
    }
    FLB_CHECK_LAUNCH();
    return FLB_OK;
  }
  switch (vpt) {
    case 1: norm_fwd_kernel<1, LN><<<min(rows, fwd_ctas<1, LN>()), kThreads, 0, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc); break;
    case 2: norm_fwd_kernel<2, LN><<<min(rows, fwd_ctas<2, LN>()), kThreads, 0, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc); break;
    case 4: norm_fwd_kernel<4, LN><<<min(rows, fwd_ctas<4, LN>()), kThreads, 0, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc); break;
    case 8: norm_fwd_kernel<8, LN><<<min(rows, fwd_ctas<8, LN>()), kThreads, 0, st>>>(x, delta, w, b, res_out, y, rstd, mean, rows, cols, eps, zc); break;
    default: return FLB_ERR_SHAPE;
  }
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
template <bool LN>
int bwd_dispatch(int vpt, dim3 grid, cudaStream_t st, const __nv_bfloat16* dy, const __nv_bfloat16* x,
                 const __nv_bfloat16* w, const float* rstd, const float* mean, const __nv_bfloat16* dres,
                 __nv_bfloat16* dx, float* dwp, float* dbp, int rows, int cols, int zc) {
  const StagedPlan plan = bwd_plan<LN>(vpt, cols);
  if (plan.stages) {
    // the slot layout depends on dres; the ring was sized for three rows per slot either way
    switch (vpt) {
      case 1: norm_bwd_staged_kernel<1, LN><<<grid, kThreads, plan.smem, st>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, cols, zc, plan.stages); break;
      case 2: norm_bwd_staged_kernel<2, LN><<<grid, kThreads, plan.smem, st>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, cols, zc, plan.stages); break;
      case 4: norm_bwd_staged_kernel<4, LN><<<grid, kThreads, plan.smem, st>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, cols, zc, plan.stages); break;
      case 8: norm_bwd_staged_kernel<8, LN><<<grid, kThreads, plan.smem, st>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, cols, zc, plan.stages); break;
      default: return FLB_ERR_SHAPE;
    }
    FLB_CHECK_LAUNCH();
    return FLB_OK;
  }
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
  auto X = (const __nv_bfloat16*)x; auto D = (const __nv_bfloat16*)delta; auto W = (const __nv_bfloat16*)w;
  auto B = (const __nv_bfloat16*)b; auto R = (__nv_bfloat16*)res_out; auto Y = (__nv_bfloat16*)y;
  if (layer_norm) return fwd_dispatch<true>(vpt, stream, X, D, W, B, R, Y, rstd, mean, rows, cols, eps, zero_centered);
  return fwd_dispatch<false>(vpt, stream, X, D, W, B, R, Y, rstd, mean, rows, cols, eps, zero_centered);
}

// Number of per-CTA partial rows flb_norm_bwd writes into dw_partial / db_partial.
FLB_API int flb_norm_bwd_parts(int rows, int cols, int layer_norm) {
  const int vpt = pick_vpt(cols);
  if (!vpt) return 0;
  const StagedPlan plan = layer_norm ? bwd_plan<true>(vpt, cols) : bwd_plan<false>(vpt, cols);
  const int ctas = plan.stages ? plan.ctas : (layer_norm ? bwd_ctas_for<true>(vpt) : bwd_ctas_for<false>(vpt));
  return rows < ctas ? rows : ctas;
}

// dx = dnorm(dy) (+ dres).  dw_partial/db_partial: [flb_norm_bwd_parts(rows, cols, layer_norm), cols] fp32 scratch (may be null
// to skip parameter gradients).
FLB_API int flb_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const float* mean,
                         const void* dres, void* dx, float* dw_partial, float* db_partial, int rows, int cols,
                         int zero_centered, int layer_norm, cudaStream_t stream) {
  const int vpt = pick_vpt(cols);
  if (!vpt || rows <= 0) return FLB_ERR_SHAPE;
  dim3 grid(flb_norm_bwd_parts(rows, cols, layer_norm));
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto DR = (const __nv_bfloat16*)dres; auto DX = (__nv_bfloat16*)dx;
  if (layer_norm) return bwd_dispatch<true>(vpt, grid, stream, DY, X, W, rstd, mean, DR, DX, dw_partial, db_partial, rows, cols, zero_centered);
  return bwd_dispatch<false>(vpt, grid, stream, DY, X, W, rstd, mean, DR, DX, dw_partial, db_partial, rows, cols, zero_centered);
}

// 1 when a staged norm kernel gave up waiting for one of its own row copies since the last call (clears the flag).
FLB_API int flb_norm_error_word() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_norm_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_norm_error, &zero, sizeof(int));
  }
  return v;
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
