// Flash-attention forward on tcgen05 tensor cores: packed variable-length documents, causal + sliding window, GQA,
// head size 128, bf16 in / bf16 out, fp32 softmax statistics.
//
// One CTA owns TWO 128-row query tiles (256 consecutive rows) of one head of one document and walks the key/value tiles
// (128 rows) either of them may see; the two query tiles share every K / V tile and alternate on the tensor pipe, so
// the softmax of one overlaps the MMAs of the other:
//   warp 0      TMA: Q0, Q1 once, then K_j (two-deep ring) and V_j (one slot)
//   warp 1      one thread issues, per key tile:  O_0 += P_0 V_j,  S_0 = Q_0 K_{j+1}^T,  O_1 += P_1 V_j,  S_1 = Q_1 K_{j+1}^T
//               (tcgen05.mma; S_t and O_t live in TMEM, P_t in shared memory, V_j is an MN-major operand)
//   warps 2-5   softmax of query tile 0, warps 6-9 of query tile 1, one query row per thread: tcgen05.ld of the S row,
//               running max / sum in the exp2 domain, masks on the diagonal and window edges, P written as bf16 into the
//               swizzled K-major tile the second MMA reads, O rescaled in TMEM only when the running max moved by more than
//               2^8 (lazy rescaling); finally O / l is written out with the row's log-sum-exp.
// All mbarrier waits are bounded (error word).
//
// Layout contract: `qkv` rows hold [q heads | k heads | v heads] x 128 (any row stride that is a multiple of 8
// elements); out rows hold heads x 128; lse is [heads, total_tokens] fp32 (natural log), the layout the backward expects.
#include "tcgen05.cuh"
#include <cstdlib>
#include <mutex>

namespace {
using namespace flb_tc;

constexpr int D = 128;           // head size
constexpr int BM = 128;          // rows of one query tile (a CTA owns two)
constexpr int BN = 128;          // key rows per tile
constexpr int kThreadsAttn = 320;
constexpr int PANEL_BYTES = 128 * 128;  // 128 rows x 64 bf16
constexpr int TILE_BYTES_ATTN = 2 * PANEL_BYTES;
// shared memory tiles: Q0 Q1 | K ring (2) | V | P0 P1
constexpr int SMEM_Q = 0, SMEM_K = 2 * TILE_BYTES_ATTN, SMEM_V = 4 * TILE_BYTES_ATTN, SMEM_P = 5 * TILE_BYTES_ATTN;
constexpr int SMEM_BARS = 7 * TILE_BYTES_ATTN;
constexpr int SMEM_TOTAL = SMEM_BARS + 256 + 1024;
constexpr float kRescaleThreshold = 8.f;  // log2 units

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

struct AttnParams {
  const int* cu_q;       // [batch + 1] query offsets
  const int* cu_k;       // [batch + 1] key offsets (== cu_q for self attention without prefix)
  __nv_bfloat16* out;    // [total_q, heads * D]
  float* lse;            // [heads, total_q]
  long long total_q;
  int heads, kv_heads, q_col0, k_col0, v_col0;  // column (element) offsets of the q / k / v blocks inside a row
  int blocks_per_doc;    // ceil(max_seqlen_q / (2 * BM))
  int causal, window;    // window <= 0: unlimited; else a query sees the `window` most recent keys including itself
  float scale_log2;      // softmax scale * log2(e)
  int* err_word;
};

__global__ void __launch_bounds__(kThreadsAttn, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sbase = raw_addr + pad;
  const uint32_t bar0 = sbase + SMEM_BARS;
  // barriers: 0-1 q_full[t], 2-3 k_full[s], 4-5 k_empty[s], 6 v_full, 7 v_empty, 8-9 s_full[t], 10-11 s_empty[t],
  //           12-13 p_full[t], 14-15 pv_done[t]
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SMEM_BARS + 8 * 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.heads / p.kv_heads);
  const int doc = blockIdx.x / p.blocks_per_doc;
  // heavy (late) query blocks first: they see the most keys
  const int qblk = p.blocks_per_doc - 1 - (blockIdx.x % p.blocks_per_doc);
  const int q_begin = p.cu_q[doc], q_len = p.cu_q[doc + 1] - q_begin;
  const int k_begin = p.cu_k[doc], k_len = p.cu_k[doc + 1] - k_begin;
  const int q0 = qblk * 2 * BM;
  if (q0 >= q_len) return;  // uniform for the CTA: nothing allocated yet
  const int num_q = (q0 + BM < q_len) ? 2 : 1;  // query tiles of this CTA that hold rows
  const int shift = k_len - q_len;  // bottom-right aligned causal mask: query i sees keys <= i + shift
  // key range either query tile needs (a tile outside one query tile's own range is fully masked for it)
  int kv_hi = k_len;
  if (p.causal) kv_hi = min(k_len, q0 + num_q * BM + shift);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, q0 + shift - p.window + 1);
  const int tile_lo = kv_lo / BN, tile_hi = (kv_hi + BN - 1) / BN;
  const int num_tiles = max(tile_hi - tile_lo, 0);

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_kv) : "memory");
    for (int i = 0; i <= 9; ++i) mbar_init(bar(i), 1);
    for (int i = 10; i <= 13; ++i) mbar_init(bar(i), 4);
    mbar_init(bar(14), 1); mbar_init(bar(15), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S_0 | S_1 | O_0 | O_1

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer
      for (int t = 0; t < num_q; ++t) {
        mbar_expect_tx(bar(t), TILE_BYTES_ATTN);
        for (int c = 0; c < 2; ++c)
          tma_load_2d(sbase + SMEM_Q + t * TILE_BYTES_ATTN + c * PANEL_BYTES, &tmap_q, bar(t), p.q_col0 + head * D + c * 64, q_begin + q0 + t * BM);
      }
      bool ok = true;
      for (int j = 0; j < num_tiles && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int row = k_begin + (tile_lo + j) * BN;
        if (!mbar_wait(bar(4 + s), ph ^ 1u, abort_flag, p.err_word, 21)) { ok = false; break; }
        mbar_expect_tx(bar(2 + s), TILE_BYTES_ATTN);
        for (int c = 0; c < 2; ++c)
          tma_load_2d(sbase + SMEM_K + s * TILE_BYTES_ATTN + c * PANEL_BYTES, &tmap_kv, bar(2 + s), p.k_col0 + kv_head * D + c * 64, row);
        if (!mbar_wait(bar(7), (j & 1) ^ 1u, abort_flag, p.err_word, 22)) { ok = false; break; }
        mbar_expect_tx(bar(6), TILE_BYTES_ATTN);
        for (int c = 0; c < 2; ++c)
          tma_load_2d(sbase + SMEM_V + c * PANEL_BYTES, &tmap_kv, bar(6), p.v_col0 + kv_head * D + c * 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc_qk = make_idesc(BM, BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc(BM, D, false, true);
      bool ok = true;
      // S_t = Q_t K_j^T; the last query tile to read K_j releases its slot
      auto issue_qk = [&](int t, int j) -> bool {
        const int s = j & 1;
        if (t == 0 && !mbar_wait(bar(2 + s), (j >> 1) & 1, abort_flag, p.err_word, 24)) return false;       // K_j landed
        if (j > 0 && !mbar_wait(bar(10 + t), (j - 1) & 1, abort_flag, p.err_word, 25)) return false;         // S_t drained
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / UMMA_K; ++k) {
          const uint32_t off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;
          umma_bf16(tmem + t * 128, make_smem_desc(sbase + SMEM_Q + t * TILE_BYTES_ATTN + off, 16, 1024),
                    make_smem_desc(sbase + SMEM_K + s * TILE_BYTES_ATTN + off, 16, 1024), idesc_qk, k != 0);
        }
        umma_commit(bar(8 + t));                       // S_t(j) ready
        if (t == num_q - 1) umma_commit(bar(4 + s));   // K slot free
        return true;
      };
      for (int t = 0; t < num_q && ok; ++t) {
        ok = mbar_wait(bar(t), 0, abort_flag, p.err_word, 23);
        if (ok && num_tiles > 0) ok = issue_qk(t, 0);
      }
      for (int j = 0; j < num_tiles && ok; ++j) {
        for (int t = 0; t < num_q && ok; ++t) {
          // S_t of the next key tile first: it only needs S_t(j) drained, and runs while this tile's P_t is being written
          if (j + 1 < num_tiles && !issue_qk(t, j + 1)) { ok = false; break; }
          if (!mbar_wait(bar(12 + t), j & 1, abort_flag, p.err_word, 26)) { ok = false; break; }           // P_t(j) written
          if (t == 0 && !mbar_wait(bar(6), j & 1, abort_flag, p.err_word, 27)) { ok = false; break; }       // V_j landed
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BN / UMMA_K; ++k) {
            const uint32_t a_off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;  // P: K-major panels over keys
            const uint32_t b_off = k * 2048;                                // V: 16 key rows per step
            umma_bf16(tmem + 256 + t * 128, make_smem_desc(sbase + SMEM_P + t * TILE_BYTES_ATTN + a_off, 16, 1024),
                      make_smem_desc(sbase + SMEM_V + b_off, PANEL_BYTES, 1024), idesc_pv, (j | k) != 0);
          }
          umma_commit(bar(14 + t));                     // O_t updated, P_t free
          if (t == num_q - 1) umma_commit(bar(7));      // V slot free
        }
      }
    }
  } else {
    // ---- softmax / correction / epilogue: one query row per thread, warps 2-5 own query tile 0, warps 6-9 tile 1
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;          // row inside the query tile
    const int qi = q0 + t * BM + r;             // row inside the document
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_s = tmem + t * 128, tmem_o = tmem + 256 + t * 128;
    const bool active = t < num_q;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < num_tiles && ok && active; ++j) {
      if (!mbar_wait(bar(8 + t), j & 1, abort_flag, p.err_word, 28)) { ok = false; break; }
      tc_fence_after();
      const int kbase = (tile_lo + j) * BN;
      // which columns of this tile may this row see?  [col_lo, col_hi)
      int col_hi = k_len - kbase;
      if (p.causal) col_hi = min(col_hi, qi + shift + 1 - kbase);
      int col_lo = 0;
      if (p.window > 0) col_lo = max(0, qi + shift - p.window + 1 - kbase);
      const bool full_tile = (col_lo <= 0) && (col_hi >= BN);
      // pass 1: row maximum
      float tile_max = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_s + lane_addr + c * 32, v);
        tmem_wait_ld();
        if (full_tile) {
#pragma unroll
          for (int i = 0; i < 32; ++i) tile_max = fmaxf(tile_max, __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            if (col >= col_lo && col < col_hi) tile_max = fmaxf(tile_max, __uint_as_float(v[i]));
          }
        }
      }
      tile_max *= p.scale_log2;
      float m_new = m;
      float alpha = 1.f;
      if (tile_max > m + kRescaleThreshold || m == -INFINITY) {
        m_new = fmaxf(m, tile_max);
        alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
      }
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      // pass 2: probabilities, packed to bf16
      uint32_t packed[64];
      float row_sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_s + lane_addr + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float e0 = exp2f(__uint_as_float(v[i]) * p.scale_log2 - m_use);
          float e1 = exp2f(__uint_as_float(v[i + 1]) * p.scale_log2 - m_use);
          if (!full_tile) {
            const int col = c * 32 + i;
            if (col < col_lo || col >= col_hi) e0 = 0.f;
            if (col + 1 < col_lo || col + 1 >= col_hi) e1 = 0.f;
          }
          row_sum += e0 + e1;
          __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
          packed[c * 16 + (i >> 1)] = *reinterpret_cast<uint32_t*>(&b);
        }
      }
      // S_t may be overwritten by the MMA of the next key tile
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(10 + t));
      // P_t and O_t are free once the previous PV MMA of this query tile has completed
      if (j > 0) {
        if (!mbar_wait(bar(14 + t), (j - 1) & 1, abort_flag, p.err_word, 29)) { ok = false; break; }
        tc_fence_after();
      }
      l = l * alpha + row_sum;
      m = m_new;
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // rescale this warp's 32 rows of O in TMEM
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(tmem_o + lane_addr + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st32(tmem_o + lane_addr + c * 32, v);
        }
        tmem_wait_st();
      }
      // write P: two K-major panels of 64 keys, 128-byte swizzle (16-byte chunk index XOR row % 8)
      uint8_t* prow = smem + SMEM_P + t * TILE_BYTES_ATTN + r * 128;
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        const int panel = ch >> 3, chunk = ch & 7;
        uint4 val = make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
        *reinterpret_cast<uint4*>(prow + panel * PANEL_BYTES + ((chunk ^ (r & 7)) << 4)) = val;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(12 + t));
    }
    // ---- epilogue
    if (active) {
      if (ok && num_tiles > 0) ok = mbar_wait(bar(14 + t), (num_tiles - 1) & 1, abort_flag, p.err_word, 30);
      tc_fence_after();
      const bool valid_row = qi < q_len;
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + ((long long)(q_begin + qi) * p.heads + head) * D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (num_tiles > 0 && ok) {
          tmem_ld32(tmem_o + lane_addr + c * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (valid_row) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g * 8 + i]) * inv_l;
            *reinterpret_cast<flb::bf16x8*>(orow + c * 32 + g * 8) = flb::pack8(f);
          }
        }
      }
      if (valid_row) p.lse[(long long)head * p.total_q + q_begin + qi] = (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}


// ---------------------------------------------------------------------------------------------------------------------
// Second forward kernel: same tiling (two 128-row query tiles per CTA sharing K / V), with the softmax kept off shared memory.
//   * a softmax thread reads its whole S row (128 fp32 columns) with four back-to-back tcgen05.ld and ONE wait, instead
//     of eight load / wait round trips;
//   * P never touches shared memory: it is packed to bf16 and stored (tcgen05.st) over the first 64 columns of the S
//     buffer it came from, and the second MMA takes it as its A operand straight from tensor memory
//     (O_t += P_t V_j with A in TMEM).  The tensor pipe executes one thread's MMAs in issue order, so S_t(j + 1) = Q_t K^T,
//     issued right after O_t += P_t(j) V_j, overwrites the buffer only after P_t(j) has been consumed;
//   * the freed shared memory double-buffers V.
// Barriers: 0-1 q_full[t], 2-3 k_full[s], 4-5 k_empty[s], 6-7 v_full[s], 8-9 v_empty[s], 10-11 s_full[t],
//           12-13 p_full[t] (four warps), 14-15 pv_done[t].
constexpr int SMEM2_Q = 0, SMEM2_K = 2 * TILE_BYTES_ATTN, SMEM2_V = 4 * TILE_BYTES_ATTN;
constexpr int SMEM2_BARS = 6 * TILE_BYTES_ATTN;
constexpr int SMEM2_TOTAL = SMEM2_BARS + 256 + 1024;

// 2^x for x <= 8 on the FMA pipe: x = n + f with n = round(x) taken from the mantissa of x + 1.5 * 2^23, 2^f by a cubic
// (relative error below 1e-4, well under the bf16 rounding of the probabilities it feeds), 2^n by adding n to the exponent field.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float shifted = x + 12582912.f;                 // 1.5 * 2^23: the low mantissa bits now hold round(x)
  const float f = x - (shifted - 12582912.f);           // in [-0.5, 0.5]
  float pf = 0.05517167f;  // minimax cubic for 2^f on [-0.5, 0.5]: largest relative error 7.5e-5
  pf = pf * f + 0.24261112f;
  pf = pf * f + 0.69326099f;
  pf = pf * f + 0.99992807f;
  return __int_as_float(__float_as_int(pf) + (__float_as_int(shifted) << 23));
}

// D[tmem] (+)= A[tmem] * B[smem]: A is a 128-lane tile in tensor memory, two bf16 per 32-bit column.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kThreadsAttn, 1)
attn_fwd_kernel_v2(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sbase = raw_addr + pad;
  const uint32_t bar0 = sbase + SMEM2_BARS;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SMEM2_BARS + 8 * 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.heads / p.kv_heads);
  const int doc = blockIdx.x / p.blocks_per_doc;
  const int qblk = p.blocks_per_doc - 1 - (blockIdx.x % p.blocks_per_doc);  // heavy (late) query blocks first
  const int q_begin = p.cu_q[doc], q_len = p.cu_q[doc + 1] - q_begin;
  const int k_begin = p.cu_k[doc], k_len = p.cu_k[doc + 1] - k_begin;
  const int q0 = qblk * 2 * BM;
  if (q0 >= q_len) return;  // uniform for the CTA: nothing allocated yet
  const int num_q = (q0 + BM < q_len) ? 2 : 1;
  const int shift = k_len - q_len;  // bottom-right aligned causal mask: query i sees keys <= i + shift
  int kv_hi = k_len;
  if (p.causal) kv_hi = min(k_len, q0 + num_q * BM + shift);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, q0 + shift - p.window + 1);
  const int tile_lo = kv_lo / BN, tile_hi = (kv_hi + BN - 1) / BN;
  const int num_tiles = max(tile_hi - tile_lo, 0);

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_kv) : "memory");
    for (int i = 0; i <= 11; ++i) mbar_init(bar(i), 1);
    mbar_init(bar(12), 4); mbar_init(bar(13), 4);
    mbar_init(bar(14), 1); mbar_init(bar(15), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S_0 (P_0 over its first 64) | S_1 (P_1) | O_0 | O_1

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer
      for (int t = 0; t < num_q; ++t) {
        mbar_expect_tx(bar(t), TILE_BYTES_ATTN);
        for (int c = 0; c < 2; ++c)
          tma_load_2d(sbase + SMEM2_Q + t * TILE_BYTES_ATTN + c * PANEL_BYTES, &tmap_q, bar(t), p.q_col0 + head * D + c * 64, q_begin + q0 + t * BM);
      }
      bool ok = true;
      for (int j = 0; j < num_tiles && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int row = k_begin + (tile_lo + j) * BN;
        if (!mbar_wait(bar(4 + s), ph ^ 1u, abort_flag, p.err_word, 21)) { ok = false; break; }
        mbar_expect_tx(bar(2 + s), TILE_BYTES_ATTN);
        for (int c = 0; c < 2; ++c)
          tma_load_2d(sbase + SMEM2_K + s * TILE_BYTES_ATTN + c * PANEL_BYTES, &tmap_kv, bar(2 + s), p.k_col0 + kv_head * D + c * 64, row);
        if (!mbar_wait(bar(8 + s), ph ^ 1u, abort_flag, p.err_word, 22)) { ok = false; break; }
        mbar_expect_tx(bar(6 + s), TILE_BYTES_ATTN);
        for (int c = 0; c < 2; ++c)
          tma_load_2d(sbase + SMEM2_V + s * TILE_BYTES_ATTN + c * PANEL_BYTES, &tmap_kv, bar(6 + s), p.v_col0 + kv_head * D + c * 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc_qk = make_idesc(BM, BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc(BM, D, false, true);
      bool ok = true;
      auto issue_qk = [&](int t, int j) -> bool {
        const int s = j & 1;
        if (t == 0 && !mbar_wait(bar(2 + s), (j >> 1) & 1, abort_flag, p.err_word, 24)) return false;  // K_j landed
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / UMMA_K; ++k) {
          const uint32_t off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;
          umma_bf16(tmem + t * 128, make_smem_desc(sbase + SMEM2_Q + t * TILE_BYTES_ATTN + off, 16, 1024),
                    make_smem_desc(sbase + SMEM2_K + s * TILE_BYTES_ATTN + off, 16, 1024), idesc_qk, k != 0);
        }
        umma_commit(bar(10 + t));                      // S_t(j) ready (and every earlier MMA of this thread complete)
        if (t == num_q - 1) umma_commit(bar(4 + s));   // K slot free
        return true;
      };
      for (int t = 0; t < num_q && ok; ++t) {
        ok = mbar_wait(bar(t), 0, abort_flag, p.err_word, 23);
        if (ok && num_tiles > 0) ok = issue_qk(t, 0);
      }
      for (int j = 0; j < num_tiles && ok; ++j) {
        const int s = j & 1;
        for (int t = 0; t < num_q && ok; ++t) {
          if (!mbar_wait(bar(12 + t), j & 1, abort_flag, p.err_word, 26)) { ok = false; break; }                    // P_t(j) in TMEM
          if (t == 0 && !mbar_wait(bar(6 + s), (j >> 1) & 1, abort_flag, p.err_word, 27)) { ok = false; break; }     // V_j landed
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BN / UMMA_K; ++k)
            umma_bf16_ts(tmem + 256 + t * 128, tmem + t * 128 + k * 8,
                         make_smem_desc(sbase + SMEM2_V + s * TILE_BYTES_ATTN + k * 2048, PANEL_BYTES, 1024), idesc_pv, (j | k) != 0);
          umma_commit(bar(14 + t));                     // O_t updated
          if (t == num_q - 1) umma_commit(bar(8 + s));  // V slot free
          // S_t of the next key tile goes behind it: the pipe runs this thread's MMAs in order, so P_t(j) is consumed first
          if (j + 1 < num_tiles && !issue_qk(t, j + 1)) { ok = false; break; }
        }
      }
    }
  } else {
    // ---- softmax / correction / epilogue: one query row per thread, warps 2-5 own query tile 0, warps 6-9 tile 1
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qi = q0 + t * BM + r;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_s = tmem + t * 128 + lane_addr, tmem_o = tmem + 256 + t * 128 + lane_addr;
    const bool active = t < num_q;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < num_tiles && ok && active; ++j) {
      if (!mbar_wait(bar(10 + t), j & 1, abort_flag, p.err_word, 28)) { ok = false; break; }
      tc_fence_after();
      const int kbase = (tile_lo + j) * BN;
      int col_hi = k_len - kbase;
      if (p.causal) col_hi = min(col_hi, qi + shift + 1 - kbase);
      int col_lo = 0;
      if (p.window > 0) col_lo = max(0, qi + shift - p.window + 1 - kbase);
      const bool full_tile = (col_lo <= 0) && (col_hi >= BN);
      // the whole row in one go
      uint32_t v[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s + c * 32, v + c * 32);
      tmem_wait_ld();
      // eight independent running maxima: one chain of 128 dependent comparisons would cost their latency 128 times
      float mx[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) mx[a] = -INFINITY;
      if (full_tile) {
#pragma unroll
        for (int i = 0; i < 128; ++i) mx[i & 7] = fmaxf(mx[i & 7], __uint_as_float(v[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i >= col_lo && i < col_hi) mx[i & 7] = fmaxf(mx[i & 7], __uint_as_float(v[i]));
      }
      float tile_max = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
      tile_max *= p.scale_log2;
      float m_new = m;
      float alpha = 1.f;
      if (tile_max > m + kRescaleThreshold || m == -INFINITY) {
        m_new = fmaxf(m, tile_max);
        alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
      }
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      // S_t(j) being complete means O_t += P_t(j - 1) V is complete too (same issuing thread, earlier in its order)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_o + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem_o + c * 32, o);
        }
      }
      // probabilities: packed to bf16 in place and stored over the first 64 columns of S_t
      // The exponentials are the busiest resource of the loop (16 per clock and SM on the special-function unit, as long as
      // the two MMAs they sit between): every fourth one is evaluated on the FMA pipe instead (exp2_poly).
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int hblk = 0; hblk < 2; ++hblk) {
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const int col = hblk * 64 + i;
          const float x0 = __uint_as_float(v[col]) * p.scale_log2 - m_use;
          const float x1 = __uint_as_float(v[col + 1]) * p.scale_log2 - m_use;
          float e0 = ((i & 6) == 0) ? exp2_poly(x0) : exp2f(x0);
          float e1 = exp2f(x1);
          if (!full_tile) {
            if (col < col_lo || col >= col_hi) e0 = 0.f;
            if (col + 1 < col_lo || col + 1 >= col_hi) e1 = 0.f;
          }
          sums[(i >> 1) & 3] += e0 + e1;
          __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&b);
        }
        tmem_st32(tmem_s + hblk * 32, packed);
      }
      const float row_sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
      l = l * alpha + row_sum;
      m = m_new;
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(12 + t));
    }
    // ---- epilogue
    if (active) {
      if (ok && num_tiles > 0) ok = mbar_wait(bar(14 + t), (num_tiles - 1) & 1, abort_flag, p.err_word, 30);
      tc_fence_after();
      const bool valid_row = qi < q_len;
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + ((long long)(q_begin + qi) * p.heads + head) * D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        if (num_tiles > 0 && ok) {
          tmem_ld32(tmem_o + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (valid_row) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[g * 8 + i]) * inv_l;
            *reinterpret_cast<flb::bf16x8*>(orow + c * 32 + g * 8) = flb::pack8(f);
          }
        }
      }
      if (valid_row) p.lse[(long long)head * p.total_q + q_begin + qi] = (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}
bool row_tmap(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_elems) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t es[2] = {1, 1};
  CUresult res = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    res = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_ERROR_INVALID_CONTEXT) break;
    cudaFree(nullptr);  // a thread that made no runtime call yet has no current context: bind the primary one
  }
  return res == CUDA_SUCCESS;
}
// 0: P kept in tensor memory (default); 1: the first kernel, P through shared memory.  FLB_ATTENTION_FWD=smem presets 1.
int g_forward_variant = [] { const char* v = getenv("FLB_ATTENTION_FWD"); return (v && v[0] == 's') ? 1 : 0; }();

int* attn_err_word() {
  static int* words[64] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!words[dev]) {
    if (cudaMalloc(&words[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(words[dev], 0, sizeof(int));
  }
  return words[dev];
}
}  // namespace

// q rows: [total_q, q_stride] with query head h at columns q_col0 + h*128; kv rows: [total_k, kv_stride] with key head g at
// k_col0 + g*128 and value head g at v_col0 + g*128 (q and kv may be the same packed tensor).  head size must be 128.
FLB_API int flb_attention_fwd(const void* q, long long q_stride, int q_col0, const void* kv, long long kv_stride, int k_col0,
                              int v_col0, const int* cu_q, const int* cu_k, int batch, int max_seqlen_q, long long total_q,
                              long long total_k, int heads, int kv_heads, int head_dim, void* out, float* lse, int causal, int window,
                              float softmax_scale, cudaStream_t stream) {
  if (head_dim != D || heads % kv_heads || q_stride % 8 || kv_stride % 8 || batch <= 0) return FLB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(kv) & 15) || (q_col0 % 8) || (k_col0 % 8) || (v_col0 % 8))
    return FLB_ERR_SHAPE;
  CUtensorMap tq, tkv;
  if (!row_tmap(&tq, q, (uint64_t)q_stride, (uint64_t)total_q, (uint64_t)q_stride)) return FLB_ERR_TMA;
  if (!row_tmap(&tkv, kv, (uint64_t)kv_stride, (uint64_t)total_k, (uint64_t)kv_stride)) return FLB_ERR_TMA;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return flb_record_cuda_error(e);
    e = cudaFuncSetAttribute(attn_fwd_kernel_v2, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_TOTAL);
    if (e != cudaSuccess) return flb_record_cuda_error(e);
    configured = true;
  }
  const bool p_in_smem = g_forward_variant == 1;
  AttnParams p;
  p.cu_q = cu_q; p.cu_k = cu_k; p.out = (__nv_bfloat16*)out; p.lse = lse; p.total_q = total_q;
  p.heads = heads; p.kv_heads = kv_heads; p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.blocks_per_doc = (max_seqlen_q + 2 * BM - 1) / (2 * BM);
  p.causal = causal; p.window = window; p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.err_word = attn_err_word();
  if (!p.err_word) return FLB_ERR_CUDA;
  dim3 grid(p.blocks_per_doc * batch, heads);
  if (p_in_smem) attn_fwd_kernel<<<grid, kThreadsAttn, SMEM_TOTAL, stream>>>(tq, tkv, p);
  else attn_fwd_kernel_v2<<<grid, kThreadsAttn, SMEM2_TOTAL, stream>>>(tq, tkv, p);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// Selects the forward kernel of later calls (0: P in tensor memory, 1: P through shared memory); returns the previous choice.
FLB_API int flb_attention_set_forward_variant(int variant) {
  const int old = g_forward_variant;
  if (variant == 0 || variant == 1) g_forward_variant = variant;
  return old;
}

FLB_API int flb_attention_error_word() {
  int* w = attn_err_word();
  if (!w) return -1;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(w, 0, sizeof(int));
  return v;
}
