// bf16 GEMM family on the Blackwell 5th-generation tensor cores.
//
//   D[M,N] (+)= A[M,K] * B[N,K]^T        fp32 accumulation in tensor memory (TMEM)
//
// Two persistent kernels share one structure: warp 0 feeds shared memory with TMA (cp.async.bulk.tensor, 128-byte
// swizzle), warp 1 issues tcgen05.mma from a single thread, warps 2-5 drain the accumulator with tcgen05.ld and write
// the output; the accumulator is double buffered in TMEM so the epilogue of tile i overlaps the main loop of tile i+1.
//
//   gemm_kernel       one CTA per SM, 128 x BLOCK_N tiles (BLOCK_N = 128 or 256).  At full tensor rate a 128x256 tile
//                     needs 94 B/clk of operand reads plus 94 B/clk of TMA writes from one SM's shared memory, more
//                     than it delivers, so this kernel tops out near two thirds of the tensor peak; it serves small
//                     and odd shapes.
//   gemm_pair_kernel  clusters of two CTAs own 256 x 256 tiles: each CTA loads its 128 rows of A and HALF of the B
//                     tile, and the leader CTA issues tcgen05.mma.cta_group::2, which reads both halves.  Shared-memory
//                     traffic per SM drops to 64 + 62.5 B/clk.  The loads carry no cluster qualifiers beyond cta_group::2.
//
// Either operand may be "K-major" (the contraction index is contiguous in memory) or "MN-major" (the M or N index is
// contiguous); this covers the three training GEMMs without transposes:
//   fprop  Y = X W^T      A = X  (K-major)   B = W  (K-major)
//   dgrad  dX = dY W      A = dY (K-major)   B = W  (MN-major: stored [K][N])
//   wgrad  dW += dY^T X   A = dY (MN-major: stored [K][M])   B = X (MN-major)
// Epilogues: store bf16, store fp32, accumulate into fp32 (C += D) or accumulate into bf16.
//
// Every wait on an mbarrier is bounded: after kSpinLimitCycles the waiting thread raises a CTA-wide abort flag and a
// global error word, every role leaves its loop, TMEM is released and the kernel returns.  The host reads the error
// word with flb_gemm_error_word().
#include "tcgen05.cuh"
#include "activations.cuh"
#include <vector>
#include <cstdlib>
#include <mutex>

namespace {
using namespace flb_tc;

constexpr int kNumThreads = 192;

template <int BLOCK_N>
struct Cfg {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int TILE_BYTES = RING_BYTES + 4 * kEpiWarpBytes;  // operand ring + epilogue staging (4 warps)
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = TILE_BYTES + BAR_BYTES + 1024;  // + slack for 1024-byte alignment
  static constexpr int TMEM_COLS = 2 * BLOCK_N;                     // 512 or 256 (powers of two)
};

template <int BLOCK_N, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_c, int use_tma_c, void* __restrict__ Cv, int M, int N, int K, long long ldc,
            int* __restrict__ err_word) {
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
      constexpr uint32_t idesc = make_idesc(BLOCK_M, BLOCK_N, A_MN, B_MN);
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
    uint32_t epi_counter = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      int m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, err_word, 4)) { ok = false; break; }
      tc_fence_after();
      const int row = m_blk * BLOCK_M + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BLOCK_N;
      if (use_tma_c) {
        epilogue_tma<EPI>(&tmap_c, smem + C::RING_BYTES + q * kEpiWarpBytes, taddr, BLOCK_N, m_blk * BLOCK_M + q * 32, n_blk * BLOCK_N, M, N,
                          lane, epi_counter);
      } else {
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_wait_ld();
          store_chunk<EPI>(r, Cv, row, n_blk * BLOCK_N + c * 32, M, N, ldc);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair kernel: clusters of two CTAs, 256 x 256 tiles, tcgen05.mma.cta_group::2 issued by the leader (cluster rank 0)
// ------------------------------------------------------------------------------------------------
constexpr int PairTileM = 256, PairTileN = 256;
struct PairCfg {
  static constexpr int TILE_M = PairTileM, TILE_N = PairTileN;
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;        // this CTA's 128 rows of A
  static constexpr int B_BYTES = (TILE_N / 2) * BLOCK_K * 2;   // this CTA's half of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;        // 32 KiB
  static constexpr int STAGES = 6;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int TILE_BYTES = RING_BYTES + 4 * kEpiWarpBytes;  // operand ring + epilogue staging (4 warps)
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = TILE_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = 2 * TILE_N;
};

// Grouped (mixture-of-experts) GEMMs on the same kernel.  Rows of A / C are sorted by expert and every expert's range is
// padded to a multiple of the tile height, so a row block belongs to one expert; `row_begin[e]` (device memory, e = 0..E)
// are the padded range starts - the launch never needs the routing result on the host.
//   kGroupRows   C[rows of e] = A[rows of e] * B_e   : B holds E matrices stacked along its row dimension
//                (fprop and dgrad of both MLP layers)
//   kGroupWgrad  C_e (+)= A[rows of e]^T * B[rows of e] : contraction over the expert's rows, C holds E matrices stacked
//                along its rows (weight gradients)
//   kGroupGathered  an ordinary GEMM whose A rows arrive chunk by chunk from tensor-parallel peers (the all-gather of a
//                sequence-parallel linear layer): chunk c of `arrive_chunk_rows` rows may be read once the word arrive[c],
//                which the peer's push kernel sets after its last store, has reached `arrive_target`.  Tiles are visited
//                starting at the local chunk (`m_rotate` row blocks in), so the math on rows that are already here covers
//                the transfer of the others; the wait is bounded like every other wait of this kernel.
//   kGroupScatter  an ordinary GEMM whose output rows leave for their owners (the reduce-scatter of a sequence-parallel linear
//                layer): rows of chunk c (`scatter_chunk_rows` rows, a multiple of the tile height) are written through
//                `scatter_maps[c]`, a tensor map in device memory over rank c's staging slot for this rank, with TMA stores from
//                the epilogue.  Row blocks are visited starting `m_rotate` blocks in (the first remote chunk), so the peer
//                stores travel under the remaining math.
enum GroupMode : int { kGroupNone = 0, kGroupRows = 1, kGroupWgrad = 2, kGroupGathered = 3, kGroupScatter = 4 };
struct GroupArgs {
  const int* row_begin;  // [experts + 1]
  int experts;
  int b_rows_per_expert;  // kGroupRows: rows of B (N if K-major, K if MN-major) per expert
  // kGroupGathered
  int m_rotate;
  const unsigned* arrive;
  unsigned arrive_target;
  int arrive_chunk_rows;
  int arrive_local_chunk;
  // kGroupScatter
  const CUtensorMap* scatter_maps;
  int scatter_chunk_rows;
};
struct TileInfo {
  int m0, n0;      // coordinates in A (row or M index) and B (N index) of the tile, before the CTA's half offset
  int c_row0;      // first row of C
  int b_row_off;   // added to B's row coordinate (kGroupRows)
  int k_begin, num_kb;
};

template <int GROUP>
__device__ __forceinline__ int grouped_num_tiles(const GroupArgs& g, int M, int N, int num_m, int num_n) {
  if constexpr (GROUP == kGroupRows) return (g.row_begin[g.experts] / PairTileM) * num_n;
  if constexpr (GROUP == kGroupWgrad) return g.experts * num_m * num_n;
  return num_m * num_n;
}

template <int GROUP>
__device__ __forceinline__ TileInfo grouped_tile(const GroupArgs& g, int tile, int num_m, int num_n, int M, int K) {
  TileInfo t;
  int m_blk, n_blk;
  if constexpr (GROUP == kGroupNone || GROUP == kGroupGathered || GROUP == kGroupScatter) {
    tile_coords(tile, num_m, num_n, m_blk, n_blk);
    if constexpr (GROUP == kGroupGathered || GROUP == kGroupScatter) m_blk = (m_blk + g.m_rotate) % num_m;
    t.m0 = m_blk * PairTileM; t.n0 = n_blk * PairTileN; t.c_row0 = t.m0; t.b_row_off = 0; t.k_begin = 0;
    t.num_kb = (K + BLOCK_K - 1) / BLOCK_K;
  } else if constexpr (GROUP == kGroupRows) {
    const int rows_m = g.row_begin[g.experts] / PairTileM;
    tile_coords(tile, rows_m, num_n, m_blk, n_blk);
    t.m0 = m_blk * PairTileM; t.n0 = n_blk * PairTileN; t.c_row0 = t.m0; t.k_begin = 0;
    t.num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    int e = 0;
    while (e + 1 < g.experts && g.row_begin[e + 1] <= t.m0) ++e;
    t.b_row_off = e * g.b_rows_per_expert;
  } else {
    const int per_expert = num_m * num_n;
    const int e = tile / per_expert;
    tile_coords(tile - e * per_expert, num_m, num_n, m_blk, n_blk);
    t.m0 = m_blk * PairTileM; t.n0 = n_blk * PairTileN; t.c_row0 = e * M + t.m0; t.b_row_off = 0;
    t.k_begin = g.row_begin[e];
    t.num_kb = (g.row_begin[e + 1] - g.row_begin[e]) / BLOCK_K;
  }
  return t;
}

// Epilogue of the first GEMM of a gated MLP: the tile holds gate columns [n0, n0 + 128) in accumulator columns 0..127 and the
// matching up columns in 128..255.  Per 64-column piece three stores leave the warp's staging buffers: the gate piece of h at
// column n0 + c, the up piece of h at column half + n0 + c, and act(gate) * up at column n0 + c of the second matrix.  The
// activation is evaluated on the bf16-rounded values, i.e. on what h holds, so a later recomputation from h reproduces it.
__device__ __forceinline__ void epilogue_gated(const CUtensorMap* tmap_h, const CUtensorMap* tmap_act, uint8_t* warp_buf, uint32_t taddr, int row0,
                                               int n0, int half, int M, int act_type, int lane, uint32_t& counter) {
  auto rounded = [](uint32_t bits) { return __bfloat162float(__float2bfloat16_rn(__uint_as_float(bits))); };
#pragma unroll 1
  for (int c = 0; c < 128; c += 64) {
    if (row0 >= M || n0 + c >= half) break;
    // three staged pieces per 64 columns (gate, up, activation); the accumulator columns are re-read from tensor memory for
    // each instead of being kept in registers (a 64-column read costs far less than the store it feeds)
#pragma unroll
    for (int which = 0; which < 3; ++which) {
      uint8_t* buf = warp_buf + (counter & 1u) * 4096;
      ++counter;
      if (lane == 0) tma_store_wait_read_1();
      __syncwarp();
      uint8_t* row_ptr = buf + lane * 128;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t g[32], u[32];
        if (which != 1) tmem_ld32(taddr + c + h * 32, g);
        if (which != 0) tmem_ld32(taddr + 128 + c + h * 32, u);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = 8 * j + 2 * e;
            float a, b;
            if (which == 0) { a = rounded(g[i]); b = rounded(g[i + 1]); }
            else if (which == 1) { a = rounded(u[i]); b = rounded(u[i + 1]); }
            else { a = act_fwd(rounded(g[i]), act_type) * rounded(u[i]); b = act_fwd(rounded(g[i + 1]), act_type) * rounded(u[i + 1]); }
            __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
            pk[e] = *reinterpret_cast<uint32_t*>(&v);
          }
          *reinterpret_cast<uint4*>(row_ptr + (((h * 4 + j) ^ (lane & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (which == 0) tma_store_2d(tmap_h, smem_u32(buf), n0 + c, row0);
        else if (which == 1) tma_store_2d(tmap_h, smem_u32(buf), half + n0 + c, row0);
        else tma_store_2d(tmap_act, smem_u32(buf), n0 + c, row0);
        tma_store_commit();
      }
    }
  }
}

template <bool A_MN, bool B_MN, int EPI, int GROUP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, int use_tma_c, void* __restrict__ Cv, int M, int N, int K, long long ldc,
                 int* __restrict__ err_word, const GroupArgs group, const __grid_constant__ CUtensorMap tmap_act, int act_type) {
  using C = PairCfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::TILE_BYTES);
  const uint32_t bar_base = smem_base + C::TILE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // leader only: its producer's arrive; bytes of both CTAs are counted on it
      mbar_init(empty_bar(s), 1);  // one tcgen05.commit from the leader per CTA
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // leader only: four epilogue warps of each CTA
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr bool kGated = (EPI == EPI_GATED_BF16);
  // gated: N counts the rows of the stacked weight (gate rows, then up rows); a tile pairs 128 gate columns with their 128 up columns
  const int gated_half = N / 2;
  const int num_m = (M + C::TILE_M - 1) / C::TILE_M;
  const int num_n = kGated ? (gated_half + 127) / 128 : (N + C::TILE_N - 1) / C::TILE_N;
  const int num_tiles = grouped_num_tiles<GROUP>(group, M, N, num_m, num_n);
  const int c_rows = (GROUP == kGroupWgrad) ? group.experts * M : ((GROUP == kGroupRows) ? group.row_begin[group.experts] : M);
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA; transaction bytes are counted on the leader's barrier) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      [[maybe_unused]] uint32_t arrived_chunks = 0;  // kGroupGathered: chunks this producer has already seen arrive (at most 16 ranks)
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const TileInfo ti = grouped_tile<GROUP>(group, tile, num_m, num_n, M, K);
        const int m0 = ti.m0 + (int)cta_rank * BLOCK_M;
        // this CTA's half of the B tile: the second 128 columns, or (gated) the up rows that belong to the leader's gate rows
        const int n0 = kGated ? ti.n0 / 2 + (int)cta_rank * gated_half : ti.n0 + (int)cta_rank * (C::TILE_N / 2);
        if constexpr (GROUP == kGroupGathered) {
          // rows [m0, m0 + BLOCK_M) must have arrived from the rank(s) that own them
          const int last_row = min(m0 + BLOCK_M, M) - 1;
          for (int c = m0 / group.arrive_chunk_rows; c <= last_row / group.arrive_chunk_rows && ok; ++c) {
            if (c == group.arrive_local_chunk || ((arrived_chunks >> c) & 1u)) continue;
            if (!flag_wait(group.arrive + c, group.arrive_target, abort_flag, err_word, 15)) { ok = false; break; }
            arrived_chunks |= 1u << c;
            // the peer wrote the rows with ordinary stores; the loads below go through the async proxy
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          if (!ok) break;
        }
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          if (!mbar_wait<true>(empty_bar(stage), phase ^ 1u, abort_flag, err_word, 11)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_dst = a_dst + C::A_BYTES;
          if (leader) mbar_expect_tx(full_bar(stage), 2 * C::STAGE_BYTES);
          const uint32_t fb = map_to_cta(full_bar(stage), 0);
          const int k0 = ti.k_begin + kb * BLOCK_K;
          if constexpr (!A_MN) {
            tma_load_2d_pair(a_dst, &tmap_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BLOCK_M / 64; ++c) tma_load_2d_pair(a_dst + c * 8192, &tmap_a, fb, m0 + c * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(b_dst, &tmap_b, fb, k0, ti.b_row_off + n0);
          } else {
#pragma unroll
            for (int c = 0; c < C::TILE_N / 2 / 64; ++c) tma_load_2d_pair(b_dst + c * 8192, &tmap_b, fb, n0 + c * 64, ti.b_row_off + k0);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(C::TILE_M, C::TILE_N, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait<true>(tempty_bar(acc), acc_phase ^ 1u, abort_flag, err_word, 12)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * C::TILE_N;
        const int num_kb = grouped_tile<GROUP>(group, tile, num_m, num_n, M, K).num_kb;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait<true>(full_bar(stage), phase, abort_flag, err_word, 13)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_addr = a_addr + C::A_BYTES;
          const uint64_t adesc = A_MN ? make_smem_desc(a_addr, 8192, 1024) : make_smem_desc(a_addr, 16, 1024);
          const uint64_t bdesc = B_MN ? make_smem_desc(b_addr, 8192, 1024) : make_smem_desc(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t ak = adesc + (uint64_t)(A_MN ? (k * 2048 >> 4) : (k * 32 >> 4));
            const uint64_t bk = bdesc + (uint64_t)(B_MN ? (k * 2048 >> 4) : (k * 32 >> 4));
            umma_bf16_pair(tmem_d, ak, bk, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(empty_bar(stage));
          umma_commit_pair(map_to_cta(empty_bar(stage), 1));
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if (num_kb > 0) {
            umma_commit_pair(tfull_bar(acc));
            umma_commit_pair(map_to_cta(tfull_bar(acc), 1));
          } else {
            // an expert without rows: nothing was issued, release the epilogue warps directly
            mbar_arrive(tfull_bar(acc));
            mbar_arrive_cluster(map_to_cta(tfull_bar(acc), 1));
          }
        }
      }
    }
  } else {
    // ---------------- epilogue warps (2..5) of both CTAs: each drains its own 128 accumulator rows ----------------
    const int q = warp & 3;
    int it = 0;
    bool ok = true;
    uint32_t epi_counter = 0;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++it) {
      const TileInfo ti = grouped_tile<GROUP>(group, tile, num_m, num_n, M, K);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait<true>(tfull_bar(acc), acc_phase, abort_flag, err_word, 14)) { ok = false; break; }
      tc_fence_after();
      const int row0 = ti.c_row0 + (int)cta_rank * BLOCK_M + q * 32;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * C::TILE_N;
      const bool empty = ti.num_kb == 0;  // grouped weight gradient of an expert without rows: the tile is zero
      if (empty) {
        if constexpr (EPI == EPI_STORE_BF16 || EPI == EPI_STORE_F32 || EPI == EPI_GATED_BF16) {
          uint32_t zeros[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) zeros[i] = 0u;
#pragma unroll 1
          for (int c = 0; c < C::TILE_N / 32; ++c) store_chunk<EPI>(zeros, Cv, row0 + lane, ti.n0 + c * 32, c_rows, N, ldc);
        }
      } else if constexpr (kGated) {
        epilogue_gated(&tmap_c, &tmap_act, smem + C::RING_BYTES + q * kEpiWarpBytes, taddr, row0, ti.n0 / 2, gated_half, M, act_type, lane, epi_counter);
      } else if (GROUP == kGroupScatter) {
        // the tile lies inside one chunk: its rows go to that rank's staging slot, addressed from the slot's first row
        const int chunk = ti.m0 / group.scatter_chunk_rows;
        const int first = chunk * group.scatter_chunk_rows;
        epilogue_tma<EPI>(group.scatter_maps + chunk, smem + C::RING_BYTES + q * kEpiWarpBytes, taddr, C::TILE_N, row0 - first, ti.n0,
                          min(group.scatter_chunk_rows, M - first), N, lane, epi_counter);
      } else if (use_tma_c) {
        epilogue_tma<EPI>(&tmap_c, smem + C::RING_BYTES + q * kEpiWarpBytes, taddr, C::TILE_N, row0, ti.n0, c_rows, N, lane, epi_counter);
      } else {
#pragma unroll 1
        for (int c = 0; c < C::TILE_N / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_wait_ld();
          store_chunk<EPI>(r, Cv, row0 + lane, ti.n0 + c * 32, c_rows, N, ldc);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();  // nobody signals into a CTA that has already left
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS)
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

// Tensor maps are pure functions of (address, extents, stride, box, kind) and a training step asks for the same few hundred
// of them again and again (weights, gradient buffers and the allocator's recycled activation blocks): each host thread keeps
// a direct-mapped table of the ones it built, so the driver's encoder runs only on a miss.
struct TmapKey {
  const void* ptr;
  uint64_t inner, outer, ld;
  uint32_t box_inner, box_outer, kind;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && ld == o.ld && box_inner == o.box_inner && box_outer == o.box_outer && kind == o.kind;
  }
};
struct TmapEntry {
  CUtensorMap map;
  TmapKey key;
  bool valid = false;
};
constexpr size_t kTmapCacheSize = 2048;  // power of two
struct TmapCounters {
  unsigned long long hits = 0, misses = 0;
};
TmapCounters& tmap_counters() {
  thread_local TmapCounters c;
  return c;
}

bool encode_tmap(CUtensorMap* map, const TmapKey& k) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  const bool f32 = k.kind == 2;
  cuuint64_t dims[2] = {k.inner, k.outer};
  cuuint64_t strides[1] = {k.ld * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {k.box_inner, k.box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(k.ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            k.kind == 0 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT) break;
    cudaFree(nullptr);  // a thread that made no runtime call yet has no current context: bind the primary one
  }
  return r == CUDA_SUCCESS;
}

bool cached_tmap(CUtensorMap* map, const TmapKey& k) {
  thread_local std::vector<TmapEntry> cache(kTmapCacheSize);
  uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= (k.inner * 0xC2B2AE3D27D4EB4Full) ^ (k.outer * 0x165667B19E3779F9ull) ^ (k.ld << 17) ^ ((uint64_t)k.box_outer << 40) ^ ((uint64_t)k.box_inner << 52) ^ k.kind;
  TmapEntry& e = cache[(h >> 20) & (kTmapCacheSize - 1)];
  if (e.valid && e.key == k) {
    ++tmap_counters().hits;
    *map = e.map;
    return true;
  }
  ++tmap_counters().misses;
  if (!encode_tmap(&e.map, k)) {
    e.valid = false;
    return false;
  }
  e.key = k;
  e.valid = true;
  *map = e.map;
  return true;
}

// 2-D bf16 operand map with the given box and a 128-byte swizzle.
bool make_tmap(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems, uint32_t box_inner,
               uint32_t box_outer) {
  return cached_tmap(map, TmapKey{ptr, inner, outer, ld_elems, box_inner, box_outer, 0u});
}

// 2-D tensor map over the output: boxes of 32 rows x 128 bytes (64 bf16 or 32 fp32 columns), 128-byte swizzle.
bool make_tmap_c(CUtensorMap* map, void* ptr, uint64_t cols, uint64_t rows, uint64_t ld_elems, bool f32) {
  return cached_tmap(map, TmapKey{ptr, cols, rows, ld_elems, f32 ? 32u : 64u, 32u, f32 ? 2u : 1u});
}

// FLB_GEMM_EPILOGUE=direct keeps the register -> global epilogue (for comparisons); default is the TMA epilogue.
bool tma_epilogue_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("FLB_GEMM_EPILOGUE");
    return !(v && v[0] == 'd');
  }();
  return enabled;
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
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, int use_tc, void* C, int M, int N, int K, long long ldc,
           int max_ctas, DeviceState* st, cudaStream_t stream) {
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
  kern<<<grid, kNumThreads, Cf::SMEM_BYTES, stream>>>(ta, tb, tc, use_tc, C, M, N, K, ldc, st->err_word);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

template <bool A_MN, bool B_MN, int EPI, int GROUP = kGroupNone>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, int use_tc, void* C, int M, int N, int K,
                long long ldc, int max_ctas, DeviceState* st, cudaStream_t stream, GroupArgs group = GroupArgs{nullptr, 0, 0},
                int tiles_upper_bound = 0, const CUtensorMap* tact = nullptr, int act_type = 0) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, EPI, GROUP>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::SMEM_BYTES);
    if (e != cudaSuccess) return flb_record_cuda_error(e);
    configured = true;
  }
  int tiles = ((M + PairCfg::TILE_M - 1) / PairCfg::TILE_M) * ((N + PairCfg::TILE_N - 1) / PairCfg::TILE_N);
  if (EPI == EPI_GATED_BF16) tiles = ((M + PairCfg::TILE_M - 1) / PairCfg::TILE_M) * ((N / 2 + 127) / 128);
  if (GROUP == kGroupRows || GROUP == kGroupWgrad) tiles = tiles_upper_bound;
  int clusters = st->num_sms / 2;
  if (max_ctas > 1 && max_ctas / 2 < clusters) clusters = max_ctas / 2;
  if (tiles < clusters) clusters = tiles;
  kern<<<2 * clusters, kNumThreads, PairCfg::SMEM_BYTES, stream>>>(ta, tb, tc, use_tc, C, M, N, K, ldc, st->err_word, group, tact ? *tact : tc, act_type);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

template <int BLOCK_N, bool A_MN, bool B_MN>
int dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, int use_tc, void* C, int M, int N, int K,
                 long long ldc, int max_ctas, DeviceState* st, cudaStream_t stream) {
  if constexpr (BLOCK_N == 0) {
    switch (epi) {
      case EPI_STORE_BF16: return launch_pair<A_MN, B_MN, EPI_STORE_BF16>(ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
      case EPI_STORE_F32: return launch_pair<A_MN, B_MN, EPI_STORE_F32>(ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
      case EPI_ACC_F32: return launch_pair<A_MN, B_MN, EPI_ACC_F32>(ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
      case EPI_ACC_BF16: return launch_pair<A_MN, B_MN, EPI_ACC_BF16>(ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
    }
  } else {
    switch (epi) {
      case EPI_STORE_BF16: return launch<BLOCK_N, A_MN, B_MN, EPI_STORE_BF16>(ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
      case EPI_STORE_F32: return launch<BLOCK_N, A_MN, B_MN, EPI_STORE_F32>(ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
      case EPI_ACC_F32: return launch<BLOCK_N, A_MN, B_MN, EPI_ACC_F32>(ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
      case EPI_ACC_BF16: return launch<BLOCK_N, A_MN, B_MN, EPI_ACC_BF16>(ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
    }
  }
  return FLB_ERR_SHAPE;
}

template <int BLOCK_N>
int dispatch_major(int a_mn, int b_mn, int epi, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, int use_tc, void* C,
                   int M, int N, int K, long long ldc, int max_ctas, DeviceState* st, cudaStream_t stream) {
  if (!a_mn && !b_mn) return dispatch_epi<BLOCK_N, false, false>(epi, ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
  if (!a_mn && b_mn) return dispatch_epi<BLOCK_N, false, true>(epi, ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
  if (a_mn && !b_mn) return dispatch_epi<BLOCK_N, true, false>(epi, ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
  return dispatch_epi<BLOCK_N, true, true>(epi, ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
}

}  // namespace

// D[M,N] (+)= A * B^T with bf16 operands.
//   a_mn_major = 0: A stored [M][lda] (K contiguous); 1: A stored [K][lda] (M contiguous).
//   b_mn_major = 0: B stored [N][ldb] (K contiguous); 1: B stored [K][ldb] (N contiguous).
//   epilogue: 0 store bf16, 1 store fp32, 2 C(fp32) += D, 3 C(bf16) += D.   ldc in elements of C.
//   block_n: 0 = choose; 128 / 256 = one-CTA kernel with that tile width; 512 = CTA-pair kernel (256 x 256 tiles).
//   max_ctas: limit the persistent grid (0 = one CTA per SM).
// Pointers must be 16-byte aligned and lda/ldb multiples of 8 elements (TMA stride rule).
// flags: bit 0 = write C with plain register stores instead of TMA (used when C is another GPU's memory).
FLB_API int flb_gemm_bf16_ex(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                             long long ldc, int a_mn_major, int b_mn_major, int epilogue, int block_n, int max_ctas, int flags,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return FLB_ERR_SHAPE;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return FLB_ERR_SHAPE;
  DeviceState* st = device_state();
  if (!st) return FLB_ERR_CUDA;
  if (block_n == 0) {
    if (M > 256 && N > 256) block_n = 512;
    else block_n = (N >= 256 && (N % 256 == 0 || N > 2048)) ? 256 : 128;
  }
  if (block_n != 128 && block_n != 256 && block_n != 512) return FLB_ERR_SHAPE;
  const uint32_t b_rows = block_n == 512 ? 128u : (uint32_t)block_n;  // B rows per TMA box (the pair kernel loads halves)
  CUtensorMap ta, tb;
  bool ok;
  if (!a_mn_major) ok = make_tmap(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M);
  else ok = make_tmap(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BLOCK_K);
  if (!ok) return FLB_ERR_TMA;
  if (!b_mn_major) ok = make_tmap(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BLOCK_K, b_rows);
  else ok = make_tmap(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BLOCK_K);
  if (!ok) return FLB_ERR_TMA;
  // C goes out through TMA stores (reduce-adds for the accumulate epilogues) when its layout allows a tensor map
  const bool c_f32 = (epilogue == EPI_STORE_F32 || epilogue == EPI_ACC_F32);
  const long long c_elem = c_f32 ? 4 : 2;
  CUtensorMap tc = ta;
  int use_tc = 0;
  if (!(flags & 1) && !(reinterpret_cast<uintptr_t>(C) & 15) && (ldc * c_elem) % 16 == 0 && tma_epilogue_enabled())
    use_tc = make_tmap_c(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, c_f32) ? 1 : 0;
  if (block_n == 512)
    return dispatch_major<0>(a_mn_major, b_mn_major, epilogue, ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
  if (block_n == 256)
    return dispatch_major<256>(a_mn_major, b_mn_major, epilogue, ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
  return dispatch_major<128>(a_mn_major, b_mn_major, epilogue, ta, tb, tc, use_tc, C, M, N, K, ldc, max_ctas, st, stream);
}

// Grouped GEMMs of a mixture-of-experts layer (CTA-pair kernel).  `row_begin`: device array [experts + 1] of the first row of
// every expert in the expert-sorted row space, each a multiple of 256; `rows_upper_bound`: host-side bound on
// row_begin[experts] (a multiple of 256; the A / C buffers have that many rows).
//   mode 1: C[rows, N] = A[rows, K] * B_e, B = experts stacked matrices, [N, K] each (b_mn 0) or [K, N] each (b_mn 1)
//   mode 2: C_e[M, N] (+)= A[rows of e, M]^T * B[rows of e, N]   (epilogue 0..3 as in flb_gemm_bf16); M % 256 == 0
FLB_API int flb_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* row_begin, int experts, int rows_upper_bound,
                                  int M, int N, int K, long long lda, long long ldb, long long ldc, int b_mn_major, int epilogue, int mode,
                                  cudaStream_t stream) {
  if (experts <= 0 || rows_upper_bound <= 0 || rows_upper_bound % PairTileM || N <= 0) return FLB_ERR_SHAPE;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return FLB_ERR_SHAPE;
  DeviceState* st = device_state();
  if (!st) return FLB_ERR_CUDA;
  const bool c_f32 = (epilogue == EPI_STORE_F32 || epilogue == EPI_ACC_F32);
  CUtensorMap ta, tb, tc;
  GroupArgs group{row_begin, experts, 0};
  const int num_n = (N + PairTileN - 1) / PairTileN;
  if (mode == kGroupRows) {
    if (K <= 0 || epilogue != EPI_STORE_BF16) return FLB_ERR_SHAPE;
    group.b_rows_per_expert = b_mn_major ? K : N;
    if (!make_tmap(&ta, A, (uint64_t)K, (uint64_t)rows_upper_bound, (uint64_t)lda, BLOCK_K, BLOCK_M)) return FLB_ERR_TMA;
    const bool ok = b_mn_major ? make_tmap(&tb, B, (uint64_t)N, (uint64_t)experts * K, (uint64_t)ldb, 64, BLOCK_K)
                               : make_tmap(&tb, B, (uint64_t)K, (uint64_t)experts * N, (uint64_t)ldb, BLOCK_K, 128u);
    if (!ok) return FLB_ERR_TMA;
    if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc * 2) % 16) return FLB_ERR_SHAPE;
    if (!make_tmap_c(&tc, C, (uint64_t)N, (uint64_t)rows_upper_bound, (uint64_t)ldc, false)) return FLB_ERR_TMA;
    const int tiles = rows_upper_bound / PairTileM * num_n;
    if (b_mn_major)
      return launch_pair<false, true, EPI_STORE_BF16, kGroupRows>(ta, tb, tc, 1, C, rows_upper_bound, N, K, ldc, 0, st, stream, group, tiles);
    return launch_pair<false, false, EPI_STORE_BF16, kGroupRows>(ta, tb, tc, 1, C, rows_upper_bound, N, K, ldc, 0, st, stream, group, tiles);
  }
  if (mode == kGroupWgrad) {
    if (M <= 0 || M % PairTileM) return FLB_ERR_SHAPE;
    if (!make_tmap(&ta, A, (uint64_t)M, (uint64_t)rows_upper_bound, (uint64_t)lda, 64, BLOCK_K)) return FLB_ERR_TMA;
    if (!make_tmap(&tb, B, (uint64_t)N, (uint64_t)rows_upper_bound, (uint64_t)ldb, 64, BLOCK_K)) return FLB_ERR_TMA;
    if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc * (c_f32 ? 4 : 2)) % 16) return FLB_ERR_SHAPE;
    if (!make_tmap_c(&tc, C, (uint64_t)N, (uint64_t)experts * M, (uint64_t)ldc, c_f32)) return FLB_ERR_TMA;
    const int tiles = experts * (M / PairTileM) * num_n;
    switch (epilogue) {
      case EPI_STORE_BF16: return launch_pair<true, true, EPI_STORE_BF16, kGroupWgrad>(ta, tb, tc, 1, C, M, N, rows_upper_bound, ldc, 0, st, stream, group, tiles);
      case EPI_STORE_F32: return launch_pair<true, true, EPI_STORE_F32, kGroupWgrad>(ta, tb, tc, 1, C, M, N, rows_upper_bound, ldc, 0, st, stream, group, tiles);
      case EPI_ACC_F32: return launch_pair<true, true, EPI_ACC_F32, kGroupWgrad>(ta, tb, tc, 1, C, M, N, rows_upper_bound, ldc, 0, st, stream, group, tiles);
      case EPI_ACC_BF16: return launch_pair<true, true, EPI_ACC_BF16, kGroupWgrad>(ta, tb, tc, 1, C, M, N, rows_upper_bound, ldc, 0, st, stream, group, tiles);
    }
  }
  return FLB_ERR_SHAPE;
}

// Grouped form of flb_gemm_gated_bf16 for the experts' first layer: rows of A / H / ACT sorted by expert (`row_begin` as in
// flb_grouped_gemm_bf16), W = experts stacked matrices [2F, K] ([gate rows; up rows] each).
FLB_API int flb_grouped_gemm_gated_bf16(const void* A, const void* W, void* H, void* ACT, const int* row_begin, int experts,
                                        int rows_upper_bound, int F, int K, long long lda, long long ldw, long long ldh, long long ldact,
                                        int act_type, cudaStream_t stream) {
  if (experts <= 0 || rows_upper_bound <= 0 || rows_upper_bound % PairTileM || F <= 0 || K <= 0) return FLB_ERR_SHAPE;
  if ((lda % 8) || (ldw % 8) || (ldh % 8) || (ldact % 8) || (F % 8)) return FLB_ERR_SHAPE;
  for (const void* ptr : {A, W, (const void*)H, (const void*)ACT})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return FLB_ERR_SHAPE;
  DeviceState* st = device_state();
  if (!st) return FLB_ERR_CUDA;
  CUtensorMap ta, tb, th, tact;
  if (!make_tmap(&ta, A, (uint64_t)K, (uint64_t)rows_upper_bound, (uint64_t)lda, BLOCK_K, BLOCK_M)) return FLB_ERR_TMA;
  if (!make_tmap(&tb, W, (uint64_t)K, (uint64_t)experts * 2 * F, (uint64_t)ldw, BLOCK_K, 128u)) return FLB_ERR_TMA;
  if (!make_tmap_c(&th, H, (uint64_t)2 * F, (uint64_t)rows_upper_bound, (uint64_t)ldh, false)) return FLB_ERR_TMA;
  if (!make_tmap_c(&tact, ACT, (uint64_t)F, (uint64_t)rows_upper_bound, (uint64_t)ldact, false)) return FLB_ERR_TMA;
  GroupArgs group{row_begin, experts, 2 * F};
  const int tiles = rows_upper_bound / PairTileM * ((F + 127) / 128);
  return launch_pair<false, false, EPI_GATED_BF16, kGroupRows>(ta, tb, th, 1, H, rows_upper_bound, 2 * F, K, ldh, 0, st, stream, group, tiles, &tact,
                                                               act_type);
}

// First GEMM of a gated MLP fused with the activation: H[M, 2F] = A[M, K] W^T with W = [gate rows; up rows] stacked ([2F, K],
// K contiguous), and ACT[M, F] = act(H[:, :F]) * H[:, F:], both bf16, from one pass over the accumulators (CTA-pair kernel).
// F must be a multiple of 8 (TMA strides); rows and columns past M / F are clipped.  act_type: see activations.cuh.
FLB_API int flb_gemm_gated_bf16(const void* A, const void* W, void* H, void* ACT, int M, int F, int K, long long lda, long long ldw,
                                long long ldh, long long ldact, int act_type, cudaStream_t stream) {
  if (M <= 0 || F <= 0 || K <= 0) return FLB_ERR_SHAPE;
  if ((lda % 8) || (ldw % 8) || (ldh % 8) || (ldact % 8) || (F % 8)) return FLB_ERR_SHAPE;
  for (const void* ptr : {A, W, (const void*)H, (const void*)ACT})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return FLB_ERR_SHAPE;
  DeviceState* st = device_state();
  if (!st) return FLB_ERR_CUDA;
  CUtensorMap ta, tb, th, tact;
  if (!make_tmap(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M)) return FLB_ERR_TMA;
  if (!make_tmap(&tb, W, (uint64_t)K, (uint64_t)2 * F, (uint64_t)ldw, BLOCK_K, 128u)) return FLB_ERR_TMA;
  if (!make_tmap_c(&th, H, (uint64_t)2 * F, (uint64_t)M, (uint64_t)ldh, false)) return FLB_ERR_TMA;
  if (!make_tmap_c(&tact, ACT, (uint64_t)F, (uint64_t)M, (uint64_t)ldact, false)) return FLB_ERR_TMA;
  return launch_pair<false, false, EPI_GATED_BF16>(ta, tb, th, 1, H, M, 2 * F, K, ldh, 0, st, stream, GroupArgs{nullptr, 0, 0}, 0, &tact, act_type);
}

// C[M, N] = A[M, K] * B (bf16 store) where A is the landing zone of a tensor-parallel all-gather: `world` chunks of
// `chunk_rows` rows, chunk `local_chunk` already in place, chunk c readable once arrive[c] >= arrive_target (set by the
// peers' flb_tp_push).  One CTA-pair launch over all rows; row blocks are visited starting at the local chunk.
// b_mn_major as in flb_gemm_bf16.  The wait gives up after the kernel's spin limit and raises the GEMM error word (15).
FLB_API int flb_gemm_gathered_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                                   int b_mn_major, const unsigned* arrive, unsigned arrive_target, int chunk_rows, int local_chunk,
                                   cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || chunk_rows <= 0 || arrive == nullptr) return FLB_ERR_SHAPE;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (M + chunk_rows - 1) / chunk_rows > 16) return FLB_ERR_SHAPE;
  for (const void* ptr : {A, B, (const void*)C})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return FLB_ERR_SHAPE;
  DeviceState* st = device_state();
  if (!st) return FLB_ERR_CUDA;
  CUtensorMap ta, tb, tc;
  if (!make_tmap(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M)) return FLB_ERR_TMA;
  const bool ok = b_mn_major ? make_tmap(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BLOCK_K)
                             : make_tmap(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BLOCK_K, 128u);
  if (!ok) return FLB_ERR_TMA;
  if (!make_tmap_c(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, false)) return FLB_ERR_TMA;
  GroupArgs group{nullptr, 0, 0, 0, arrive, arrive_target, chunk_rows, local_chunk};
  const int num_m = (M + PairCfg::TILE_M - 1) / PairCfg::TILE_M;
  group.m_rotate = (int)(((long long)local_chunk * chunk_rows / PairCfg::TILE_M) % num_m);
  if (b_mn_major) return launch_pair<false, true, EPI_STORE_BF16, kGroupGathered>(ta, tb, tc, 1, C, M, N, K, ldc, 0, st, stream, group);
  return launch_pair<false, false, EPI_STORE_BF16, kGroupGathered>(ta, tb, tc, 1, C, M, N, K, ldc, 0, st, stream, group);
}

// flb_gemm_gathered_bf16 and flb_gemm_gated_bf16 in one: the first GEMM of a tensor-parallel gated MLP, whose A rows arrive
// from the peers while the tiles of the local chunk are computed, with the activation in the epilogue.
FLB_API int flb_gemm_gathered_gated_bf16(const void* A, const void* W, void* H, void* ACT, int M, int F, int K, long long lda, long long ldw,
                                         long long ldh, long long ldact, int act_type, const unsigned* arrive, unsigned arrive_target,
                                         int chunk_rows, int local_chunk, cudaStream_t stream) {
  if (M <= 0 || F <= 0 || K <= 0 || chunk_rows <= 0 || arrive == nullptr) return FLB_ERR_SHAPE;
  if ((lda % 8) || (ldw % 8) || (ldh % 8) || (ldact % 8) || (F % 8) || (M + chunk_rows - 1) / chunk_rows > 16) return FLB_ERR_SHAPE;
  for (const void* ptr : {A, W, (const void*)H, (const void*)ACT})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return FLB_ERR_SHAPE;
  DeviceState* st = device_state();
  if (!st) return FLB_ERR_CUDA;
  CUtensorMap ta, tb, th, tact;
  if (!make_tmap(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M)) return FLB_ERR_TMA;
  if (!make_tmap(&tb, W, (uint64_t)K, (uint64_t)2 * F, (uint64_t)ldw, BLOCK_K, 128u)) return FLB_ERR_TMA;
  if (!make_tmap_c(&th, H, (uint64_t)2 * F, (uint64_t)M, (uint64_t)ldh, false)) return FLB_ERR_TMA;
  if (!make_tmap_c(&tact, ACT, (uint64_t)F, (uint64_t)M, (uint64_t)ldact, false)) return FLB_ERR_TMA;
  GroupArgs group{nullptr, 0, 0, 0, arrive, arrive_target, chunk_rows, local_chunk};
  const int num_m = (M + PairCfg::TILE_M - 1) / PairCfg::TILE_M;
  group.m_rotate = (int)(((long long)local_chunk * chunk_rows / PairCfg::TILE_M) % num_m);
  return launch_pair<false, false, EPI_GATED_BF16, kGroupGathered>(ta, tb, th, 1, H, M, 2 * F, K, ldh, 0, st, stream, group, 0, &tact, act_type);
}

// Tensor maps for flb_gemm_scatter_bf16: `world` maps of 128 bytes each written to `host_out` (64-byte aligned host memory), map
// c over the bf16 matrix [rows, n] (leading dimension ld elements) at dst_ptrs[c].  The caller copies them to device memory.
FLB_API int flb_gemm_scatter_maps(void* host_out, const void* const* dst_ptrs, int world, int rows, int n, long long ld) {
  if (world <= 0 || rows <= 0 || n <= 0 || (ld % 8) || (reinterpret_cast<uintptr_t>(host_out) & 63)) return FLB_ERR_SHAPE;
  CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(host_out);
  for (int c = 0; c < world; ++c) {
    if (reinterpret_cast<uintptr_t>(dst_ptrs[c]) & 15) return FLB_ERR_SHAPE;
    if (!encode_tmap(&maps[c], TmapKey{dst_ptrs[c], (uint64_t)n, (uint64_t)rows, (uint64_t)ld, 64u, 32u, 1u})) return FLB_ERR_TMA;
  }
  return FLB_OK;
}

// C = A[M, K] * B (bf16) where the rows of C are scattered: chunk c of `chunk_rows` rows (a multiple of 256) is stored through
// scatter_maps[c] (device memory, from flb_gemm_scatter_maps), i.e. straight into rank c's staging slot over NVLink.  One
// CTA-pair launch over all rows, starting at row block `first_chunk * chunk_rows / 256`.
FLB_API int flb_gemm_scatter_bf16(const void* A, const void* B, const void* scatter_maps, int M, int N, int K, long long lda, long long ldb,
                                  int b_mn_major, int chunk_rows, int first_chunk, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || chunk_rows <= 0 || (chunk_rows % PairCfg::TILE_M) || scatter_maps == nullptr) return FLB_ERR_SHAPE;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(scatter_maps) & 63)) return FLB_ERR_SHAPE;
  for (const void* ptr : {A, B})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return FLB_ERR_SHAPE;
  DeviceState* st = device_state();
  if (!st) return FLB_ERR_CUDA;
  CUtensorMap ta, tb;
  if (!make_tmap(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M)) return FLB_ERR_TMA;
  const bool ok = b_mn_major ? make_tmap(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BLOCK_K)
                             : make_tmap(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BLOCK_K, 128u);
  if (!ok) return FLB_ERR_TMA;
  GroupArgs group{};
  group.scatter_maps = reinterpret_cast<const CUtensorMap*>(scatter_maps);
  group.scatter_chunk_rows = chunk_rows;
  const int num_m = (M + PairCfg::TILE_M - 1) / PairCfg::TILE_M;
  group.m_rotate = (int)(((long long)first_chunk * chunk_rows / PairCfg::TILE_M) % num_m);
  // the kernel's own output map is unused in this mode: pass A's as a placeholder
  if (b_mn_major) return launch_pair<false, true, EPI_STORE_BF16, kGroupScatter>(ta, tb, ta, 1, nullptr, M, N, K, N, 0, st, stream, group);
  return launch_pair<false, false, EPI_STORE_BF16, kGroupScatter>(ta, tb, ta, 1, nullptr, M, N, K, N, 0, st, stream, group);
}

FLB_API int flb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn_major, int b_mn_major, int epilogue, int block_n, int max_ctas,
                          cudaStream_t stream) {
  return flb_gemm_bf16_ex(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, epilogue, block_n, max_ctas, 0, stream);
}

// Hits and misses of the calling thread's tensor-map table since the thread started (out[0], out[1]).
FLB_API void flb_gemm_tmap_cache_stats(unsigned long long* out) {
  out[0] = tmap_counters().hits;
  out[1] = tmap_counters().misses;
}

// Reads (and clears) the error word the GEMM kernels raise when a bounded wait expires.
// Synchronises the device.  0 = no error; 1..4 / 11..14 = which role gave up (one-CTA / pair kernel); 15 = rows of a peer did not arrive.
FLB_API int flb_gemm_error_word() {
  DeviceState* st = device_state();
  if (!st) return -1;
  int v = 0;
  if (cudaMemcpy(&v, st->err_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(st->err_word, 0, sizeof(int));
  return v;
}
