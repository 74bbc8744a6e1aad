// PTX wrappers shared by the tcgen05 GEMM kernels: mbarriers with bounded waits, TMA tile loads, UMMA issue and commit
// (one-CTA and CTA-pair forms), TMEM loads, shared-memory matrix descriptors, tile rasterisation and the epilogue that
// writes one 32-column chunk of an accumulator row.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace flb_tc {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kGroupM = 16;  // tile rasterisation: this many row-blocks share a sweep over N (L2 reuse)
constexpr long long kSpinLimitCycles = 4000000000ll;  // about 2 s at boost clock

// EPI_GATED_BF16: the 256 accumulator columns of a tile are 128 gate columns followed by their 128 up columns; the epilogue
// writes both halves of h (bf16) and act(gate) * up into a second matrix.
enum Epilogue : int { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ACC_F32 = 2, EPI_ACC_BF16 = 3, EPI_GATED_BF16 = 4 };

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
// Arrive on a barrier that lives in another CTA of the cluster (`bar` is a shared::cluster address).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Same with cluster-scope acquire: the barrier is completed by arrivals / transactions from the peer CTA.
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the CTA is aborting (deadline passed here or elsewhere).
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err_word, int where) {
  auto poll = [&]() { return CLUSTER ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity); };
  if (poll()) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (poll()) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kSpinLimitCycles) {
      *abort_flag = 1;
      atomicExch(err_word, where);
      return false;
    }
  }
}

// Bounded wait until the 32-bit word at `flag` (written by another GPU with st.release.sys) has reached `target`
// (wrap-around compare).  Same contract as mbar_wait: false after the limit, with the CTA's abort flag and the error word set.
__device__ __forceinline__ bool flag_wait(const unsigned* flag, unsigned target, volatile int* abort_flag, int* err_word, int where) {
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int)(v - target) >= 0) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kSpinLimitCycles) {
      *abort_flag = 1;
      atomicExch(err_word, where);
      return false;
    }
    __nanosleep(100);
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// CTA-pair form: the data lands in this CTA's shared memory, the transaction bytes are counted on `bar`, which may
// belong to either CTA of the pair (a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Pair form: `bar` is a shared::cluster address and may name a barrier of either CTA.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
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

// Instruction descriptor for bf16 x bf16 -> fp32 with the given MMA shape and operand majors.
__host__ __device__ constexpr uint32_t make_idesc(int mma_m, int mma_n, bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
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

// Writes (or accumulates into C) 32 consecutive accumulator columns r[0..31] of output row `row`, starting at `col`.
template <int EPI>
__device__ __forceinline__ void store_chunk(const uint32_t* r, void* Cv, int row, int col, int M, int N, long long ldc) {
  if (row >= M || col >= N) return;
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
        float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
                               __uint_as_float(r[4 * v + 3]));
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

// Cluster helpers.
// ---- epilogue through shared memory and TMA stores -------------------------------------------------------------------
// A warp drains its 32 accumulator rows in pieces of one 128-byte row segment (64 bf16 or 32 fp32 columns): registers ->
// swizzled shared memory (conflict-free 16-byte stores) -> one TMA tensor store (or reduce-add, for the accumulate
// epilogues) per piece.  Two 4 KiB buffers per warp alternate; `cp.async.bulk.wait_group.read 1` guards their reuse.
constexpr int kEpiWarpBytes = 2 * 4096;

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Drains `width` accumulator columns starting at TMEM address `taddr` (this warp's lane quarter) into rows row0..row0+31,
// columns col0.. of C.  `counter` alternates the two buffers across calls.  Rows / columns past M / N are clipped by TMA.
template <int EPI>
__device__ __forceinline__ void epilogue_tma(const CUtensorMap* tmap_c, uint8_t* warp_buf, uint32_t taddr, int width, int row0,
                                             int col0, int M, int N, int lane, uint32_t& counter) {
  constexpr bool kF32 = (EPI == EPI_STORE_F32 || EPI == EPI_ACC_F32);
  constexpr bool kReduce = (EPI == EPI_ACC_F32 || EPI == EPI_ACC_BF16);
  constexpr int kCols = kF32 ? 32 : 64;
#pragma unroll 1
  for (int c = 0; c < width; c += kCols) {
    if (row0 >= M || col0 + c >= N) break;  // nothing of this piece (nor of the following ones) lies inside C
    uint8_t* buf = warp_buf + (counter & 1u) * 4096;
    ++counter;
    if (lane == 0) tma_store_wait_read_1();
    __syncwarp();
    uint8_t* row_ptr = buf + lane * 128;
    if constexpr (kF32) {
      uint32_t r[32];
      tmem_ld32(taddr + c, r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(row_ptr + ((j ^ (lane & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t r[32];
        tmem_ld32(taddr + c + h * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
            pk[e] = *reinterpret_cast<uint32_t*>(&b);
          }
          *reinterpret_cast<uint4*>(row_ptr + (((h * 4 + j) ^ (lane & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      if constexpr (kReduce) tma_reduce_add_2d(tmap_c, smem_u32(buf), col0 + c, row0);
      else tma_store_2d(tmap_c, smem_u32(buf), col0 + c, row0);
      tma_store_commit();
    }
  }
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}

}  // namespace flb_tc
