// bf16 GEMM family on the Blackwell 5th-generation tensor cores.
//
//   D[M,N] (+)= A[M,K] * B[N,K]^T        fp32 accumulation in tensor memory (TMEM)
//
// One persistent CTA per SM.  Warp 0 feeds shared memory with TMA (cp.async.bulk.tensor, 128-byte
// swizzle, no cluster qualifiers), warp 1 issues tcgen05.mma from a single thread, warps 2-5 drain
// the accumulator with tcgen05.ld and write the output.  The accumulator is double buffered
// (2 x BLOCK_N TMEM columns) so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Either operand may be "K-major" (the contraction index is contiguous in memory) or "MN-major"
// (the M or N index is contiguous); this covers the three training GEMMs without transposes:
//   fprop  Y = X W^T      A = X  (K-major)   B = W  (K-major)
//   dgrad  dX = dY W      A = dY (K-major)   B = W  (MN-major: stored [K][N])
//   wgrad  dW += dY^T X   A = dY (MN-major: stored [K][M])   B = X (MN-major)
// Epilogues: store bf16, store fp32, accumulate into fp32 (C += D) or accumulate into bf16.
//
// Every wait on an mbarrier is bounded: after kSpinLimitCycles the waiting thread raises a CTA-wide
// abort flag and a global error word, every role leaves its loop, TMEM is released and the kernel
// returns.  The host reads the error word with flb_gemm_error_word().
#include "common.cuh"
#include <cuda.h>
#include <mutex>

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kNumThreads = 192;
constexpr int kGroupM = 16;   // tile rasterisation: 16 row-blocks share a sweep over N (L2 reuse)
constexpr long long kSpinLimitCycles = 4000000000ll;  // about 2 s at boost clock

enum Epilogue : int { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ACC_F32 = 2, EPI_ACC_BF16 = 3 };

template <int BLOCK_N>
struct Cfg {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = TILE_BYTES + BAR_BYTES + 1024;  // + slack for 1024-byte alignment
  static constexpr int TMEM_COLS = 2 * BLOCK_N;                     // 512 or 256 (powers of two)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the CTA is aborting (deadline passed here or elsewhere).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err_word,
                                          int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kSpinLimitCycles) {
      *abort_flag = 1;
      atomicExch(err_word, where);
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int BLOCK_N, bool A_MN, bool B_MN>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  return (1u << 4)                           // D format fp32
         | (1u << 7) | (1u << 10)            // A, B format bf16
         | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16)
         | ((uint32_t)(BLOCK_N >> 3) << 17) | ((uint32_t)(BLOCK_M >> 4) << 24);
}

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int group_size = kGroupM * num_n;
  const int g = tile / group_size;
  const int first_m = g * kGroupM;
  const int gm = min(num_m - first_m, kGroupM);
  const int r = tile - g * group_size;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

template <int BLOCK_N, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, void* __restrict__ Cv,
            int M, int N, int K, long long ldc, int* __restrict__ err_word) {
  using C = Cfg<BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES);
  // layout: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then tmem slot + abort flag
  const uint32_t bar_base = smem_base + C::TILE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (M + BLOCK_M - 1) / BLOCK_M;
  const int num_n = (N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, num_m, num_n, m_blk, n_blk);
        const int m0 = m_blk * BLOCK_M, n0 = n_blk * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, err_word, 1)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_dst = a_dst + C::A_BYTES;
          const uint32_t fb = full_bar(stage);
          mbar_expect_tx(fb, C::STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, &tmap_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BLOCK_M / 64; ++c) tma_load_2d(a_dst + c * 8192, &tmap_a, fb, m0 + c * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmap_b, fb, k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BLOCK_N / 64; ++c) tma_load_2d(b_dst + c * 8192, &tmap_b, fb, n0 + c * 64, k0);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Drain: give copies already issued a bounded chance to land before the CTA exits.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<BLOCK_N, A_MN, B_MN>();
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, err_word, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, err_word, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_addr = a_addr + C::A_BYTES;
          const uint64_t adesc = A_MN ? make_smem_desc(a_addr, 8192, 1024) : make_smem_desc(a_addr, 16, 1024);
          const uint64_t bdesc = B_MN ? make_smem_desc(b_addr, 8192, 1024) : make_smem_desc(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t ak = adesc + (uint64_t)(A_MN ? (k * 2048 >> 4) : (k * 32 >> 4));
            const uint64_t bk = bdesc + (uint64_t)(B_MN ? (k * 2048 >> 4) : (k * 32 >> 4));
            umma_bf16(tmem_d, ak, bk, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else {
    // ---------------- epilogue warps (2..5) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      int m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, err_word, 4)) { ok = false; break; }
      tc_fence_after();
      const int row = m_blk * BLOCK_M + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BLOCK_N;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_wait_ld();
        const int col = n_blk * BLOCK_N + c * 32;
        if (row < M && col < N) {
          const bool full = (col + 32 <= N);
          if constexpr (EPI == EPI_STORE_BF16 || EPI == EPI_ACC_BF16) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cv) + (long long)row * ldc + col;
            if (full && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
                if constexpr (EPI == EPI_ACC_BF16) {
                  flb::bf16x8 old = *reinterpret_cast<const flb::bf16x8*>(crow + v * 8);
                  float o[8];
                  flb::unpack8(old, o);
#pragma unroll
                  for (int j = 0; j < 8; ++j) f[j] += o[j];
                }
                *reinterpret_cast<flb::bf16x8*>(crow + v * 8) = flb::pack8(f);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col + j < N) {
                  float f = __uint_as_float(r[j]);
                  if constexpr (EPI == EPI_ACC_BF16) f += flb::bf2f(crow[j]);
                  crow[j] = flb::f2bf(f);
                }
              }
            }
          } else {
            float* crow = reinterpret_cast<float*>(Cv) + (long long)row * ldc + col;
            if (full && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if constexpr (EPI == EPI_ACC_F32) {
                  const float4 p = *reinterpret_cast<const float4*>(crow + 4 * v);
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                *reinterpret_cast<float4*>(crow + 4 * v) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col + j < N) {
                  float f = __uint_as_float(r[j]);
                  if constexpr (EPI == EPI_ACC_F32) f += crow[j];
                  crow[j] = f;
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 tensor map over a matrix whose contiguous dimension has `inner` elements.
bool make_tmap(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems, uint32_t box_inner,
               uint32_t box_outer) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

struct DeviceState {
  int num_sms = 0;
  int* err_word = nullptr;
};
DeviceState* device_state() {
  static DeviceState states[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  DeviceState& s = states[dev];
  if (s.num_sms == 0) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return nullptr;
    if (cudaMalloc(&s.err_word, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(s.err_word, 0, sizeof(int));
    s.num_sms = prop.multiProcessorCount;
  }
  return &s;
}

template <int BLOCK_N, bool A_MN, bool B_MN, int EPI>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc, int max_ctas,
           DeviceState* st, cudaStream_t stream) {
  using Cf = Cfg<BLOCK_N>;
  auto kern = gemm_kernel<BLOCK_N, A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cf::SMEM_BYTES);
    if (e != cudaSuccess) return flb_record_cuda_error(e);
    configured = true;
  }
  const int tiles = ((M + BLOCK_M - 1) / BLOCK_M) * ((N + BLOCK_N - 1) / BLOCK_N);
  int grid = st->num_sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  kern<<<grid, kNumThreads, Cf::SMEM_BYTES, stream>>>(ta, tb, C, M, N, K, ldc, st->err_word);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

template <int BLOCK_N, bool A_MN, bool B_MN>
int dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc,
                 int max_ctas, DeviceState* st, cudaStream_t stream) {
  switch (epi) {
    case EPI_STORE_BF16: return launch<BLOCK_N, A_MN, B_MN, EPI_STORE_BF16>(ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
    case EPI_STORE_F32: return launch<BLOCK_N, A_MN, B_MN, EPI_STORE_F32>(ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
    case EPI_ACC_F32: return launch<BLOCK_N, A_MN, B_MN, EPI_ACC_F32>(ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
    case EPI_ACC_BF16: return launch<BLOCK_N, A_MN, B_MN, EPI_ACC_BF16>(ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
  }
  return FLB_ERR_SHAPE;
}

template <int BLOCK_N>
int dispatch_major(int a_mn, int b_mn, int epi, const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N,
                   int K, long long ldc, int max_ctas, DeviceState* st, cudaStream_t stream) {
  if (!a_mn && !b_mn) return dispatch_epi<BLOCK_N, false, false>(epi, ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
  if (!a_mn && b_mn) return dispatch_epi<BLOCK_N, false, true>(epi, ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
  if (a_mn && !b_mn) return dispatch_epi<BLOCK_N, true, false>(epi, ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
  return dispatch_epi<BLOCK_N, true, true>(epi, ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
}

}  // namespace

// D[M,N] (+)= A * B^T with bf16 operands.
//   a_mn_major = 0: A stored [M][lda] (K contiguous); 1: A stored [K][lda] (M contiguous).
//   b_mn_major = 0: B stored [N][ldb] (K contiguous); 1: B stored [K][ldb] (N contiguous).
//   epilogue: 0 store bf16, 1 store fp32, 2 C(fp32) += D, 3 C(bf16) += D.   ldc in elements of C.
//   block_n: 256 or 128 (0 = choose).  max_ctas: limit the persistent grid (0 = one CTA per SM).
// Pointers must be 16-byte aligned and lda/ldb multiples of 8 elements (TMA stride rule).
FLB_API int flb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn_major, int b_mn_major, int epilogue, int block_n, int max_ctas,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return FLB_ERR_SHAPE;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return FLB_ERR_SHAPE;
  DeviceState* st = device_state();
  if (!st) return FLB_ERR_CUDA;
  if (block_n == 0) block_n = (N >= 256 && (N % 256 == 0 || N > 2048)) ? 256 : 128;
  if (block_n != 128 && block_n != 256) return FLB_ERR_SHAPE;
  CUtensorMap ta, tb;
  bool ok;
  if (!a_mn_major) ok = make_tmap(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M);
  else ok = make_tmap(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BLOCK_K);
  if (!ok) return FLB_ERR_TMA;
  if (!b_mn_major) ok = make_tmap(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BLOCK_K, (uint32_t)block_n);
  else ok = make_tmap(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BLOCK_K);
  if (!ok) return FLB_ERR_TMA;
  if (block_n == 256)
    return dispatch_major<256>(a_mn_major, b_mn_major, epilogue, ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
  return dispatch_major<128>(a_mn_major, b_mn_major, epilogue, ta, tb, C, M, N, K, ldc, max_ctas, st, stream);
}

// Reads (and clears) the error word the GEMM kernels raise when a bounded wait expires.
// Synchronises the device.  0 = no error; 1..4 = which role gave up.
FLB_API int flb_gemm_error_word() {
  DeviceState* st = device_state();
  if (!st) return -1;
  int v = 0;
  if (cudaMemcpy(&v, st->err_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(st->err_word, 0, sizeof(int));
  return v;
}
