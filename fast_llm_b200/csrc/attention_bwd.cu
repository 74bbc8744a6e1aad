// Flash-attention backward on tcgen05 tensor cores (packed variable-length documents, causal + sliding window, GQA,
// head size 128).
//
// One CTA owns 128 key/value rows of one KV head and walks every (query head of the group, query block) that can see
// them.  Per (query block i, key block j) pair, five 128x128x128 MMAs:
//     S  = Q_i K_j^T          dP = dO_i V_j^T                       (accumulators T0 / T1 in TMEM, alternating)
//     dV += P^T dO_i          dK += dS^T Q_i                        (accumulators resident in TMEM for the whole CTA)
//     dQ_i = dS K_j           (into the TMEM buffer S occupied; drained with vector fp32 reductions into dq_accum)
// The MMA thread issues S of the next pair as soon as dS of this pair has left its TMEM buffer, so the compute warps work
// on P(n + 1) while dK(n) / dQ(n) run; softmax statistics are loaded one pair ahead.
// Eight compute warps (two per TMEM lane quarter, each pair splitting the 128 columns) turn S into P = exp2(S c - lse),
// dP into dS = P (dP - delta) scale, write both as bf16 into swizzled shared-memory tiles that serve as MN-major A
// operands (P^T, dS^T) and as the K-major A operand (dS) without any transposition, and drain dQ.
// Shared-memory tiles are loaded once with TMA in a layout that is simultaneously the K-major view needed by S / dP and
// the MN-major view needed by dV / dK / dQ.  All mbarrier waits are bounded (error word).
#include "tcgen05.cuh"
#include <cstdio>
#include <mutex>

namespace {
using namespace flb_tc;

constexpr int D = 128, BM = 128, BN = 128;
constexpr int kThreadsBwd = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 compute
constexpr int PANEL = 128 * 128;  // bytes: 128 rows x 64 bf16
constexpr int TILE = 2 * PANEL;
constexpr int S_K = 0, S_V = TILE, S_Q = 2 * TILE /* two stages */, S_DO = 4 * TILE, S_P = 5 * TILE, S_DS = 6 * TILE;
constexpr int S_BARS = 7 * TILE;
constexpr int SMEM_BWD = S_BARS + 256 + 1024;

struct BwdParams {
  const int* cu_q;
  const int* cu_k;
  const float* lse;     // [heads, total_q] natural log
  const float* delta;   // [heads, total_q] rowsum(dO * O)
  float* dq_accum;      // [total_q, heads * D] fp32, zero-initialised
  __nv_bfloat16* dkv;   // rows of the packed gradient: key head g at k_col0 + g*D, value head g at v_col0 + g*D
  long long dkv_stride; // elements
  long long total_q, tok_groups;
  int heads, kv_heads, q_col0, k_col0, v_col0, do_col_stride;
  int kv_blocks_per_doc;
  int causal, window;
  float scale, scale_log2;
  int* err_word;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  atomicAdd(reinterpret_cast<float4*>(addr), make_float4(a, b, c, d));  // one 16-byte reduction, result unused
}

__global__ void __launch_bounds__(kThreadsBwd, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                const __grid_constant__ CUtensorMap tmap_do, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sb = raw_addr + pad;
  const uint32_t bar0 = sb + S_BARS;
  // 0 kv_full, 1-2 q_full, 3-4 q_empty, 5 do_full, 6 do_empty, 7 s_full, 8 dp_full, 9 dq_full,
  // 10 p_ready, 11 ds_ready, 12 dq_drained
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S_BARS + 8 * 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_head = blockIdx.y;
  const int group = p.heads / p.kv_heads;
  const int doc = blockIdx.x / p.kv_blocks_per_doc;
  const int jblk = blockIdx.x % p.kv_blocks_per_doc;
  const int q_begin = p.cu_q[doc], q_len = p.cu_q[doc + 1] - q_begin;
  const int k_begin = p.cu_k[doc], k_len = p.cu_k[doc + 1] - k_begin;
  const int k0 = jblk * BN;
  if (k0 >= k_len) return;
  const int shift = k_len - q_len;
  // query rows that can see keys [k0, k0 + BN): causal -> q >= k0 - shift; window -> q <= k0 + BN - 1 - shift + window - 1
  int q_lo = 0, q_hi = q_len;
  if (p.causal) q_lo = max(0, k0 - shift);
  if (p.window > 0) q_hi = min(q_len, k0 + BN - 1 - shift + p.window);
  const int iblk_lo = q_lo / BM, iblk_hi = (q_hi + BM - 1) / BM;
  const int blocks = max(iblk_hi - iblk_lo, 0);
  const int num_pairs = blocks * group;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_kv) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_do) : "memory");
    for (int i = 0; i <= 9; ++i) mbar_init(bar(i), 1);
    for (int i = 10; i <= 12; ++i) mbar_init(bar(i), 8);
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
  auto tmem_t = [&](int i) { return tmem + 128u * (uint32_t)i; };
  const uint32_t tmem_dv = tmem + 256, tmem_dk = tmem + 384;

  auto pair_head = [&](int n) { return kv_head * group + n / blocks; };
  auto pair_q0 = [&](int n) { return (iblk_lo + n % blocks) * BM; };

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(0), 2 * TILE);
      for (int c = 0; c < 2; ++c) {
        tma_load_2d(sb + S_K + c * PANEL, &tmap_kv, bar(0), p.k_col0 + kv_head * D + c * 64, k_begin + k0);
        tma_load_2d(sb + S_V + c * PANEL, &tmap_kv, bar(0), p.v_col0 + kv_head * D + c * 64, k_begin + k0);
      }
      bool ok = true;
      for (int n = 0; n < num_pairs && ok; ++n) {
        const int s = n & 1;
        const uint32_t ph = (n >> 1) & 1;
        const int row = q_begin + pair_q0(n), head = pair_head(n);
        if (!mbar_wait(bar(3 + s), ph ^ 1u, abort_flag, p.err_word, 41)) { ok = false; break; }
        mbar_expect_tx(bar(1 + s), TILE);
        for (int c = 0; c < 2; ++c) tma_load_2d(sb + S_Q + s * TILE + c * PANEL, &tmap_q, bar(1 + s), p.q_col0 + head * D + c * 64, row);
        if (!mbar_wait(bar(6), (n & 1) ^ 1u, abort_flag, p.err_word, 42)) { ok = false; break; }
        mbar_expect_tx(bar(5), TILE);
        for (int c = 0; c < 2; ++c) tma_load_2d(sb + S_DO + c * PANEL, &tmap_do, bar(5), head * D + c * 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc(128, 128, false, false);  // A K-major, B K-major      (S, dP)
      constexpr uint32_t idesc_mm = make_idesc(128, 128, true, true);    // A MN-major, B MN-major    (dV, dK)
      constexpr uint32_t idesc_km = make_idesc(128, 128, false, true);   // A K-major, B MN-major     (dQ)
      bool ok = mbar_wait(bar(0), 0, abort_flag, p.err_word, 43);
      auto kmajor = [&](uint32_t base, int k) { return make_smem_desc(base + (k >> 2) * PANEL + (k & 3) * 32, 16, 1024); };
      auto mnmajor = [&](uint32_t base, int k) { return make_smem_desc(base + k * 2048, PANEL, 1024); };
      // S(n) = Q K^T into T[n & 1]; issued one pair ahead (right after dS(n - 1) released that buffer)
      auto issue_s = [&](int n) -> bool {
        const int s = n & 1;
        if (!mbar_wait(bar(1 + s), (n >> 1) & 1, abort_flag, p.err_word, 44)) return false;   // Q(n) landed
        tc_fence_after();
        const uint32_t qb = sb + S_Q + s * TILE;
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(tmem_t(s), kmajor(qb, k), kmajor(sb + S_K, k), idesc_kk, k != 0);
        umma_commit(bar(7));
        return true;
      };
      if (ok && num_pairs > 0) ok = issue_s(0);
      for (int n = 0; n < num_pairs && ok; ++n) {
        const int s = n & 1;
        const uint32_t par = n & 1;
        const uint32_t t_s = tmem_t(s), t_dp = tmem_t(s ^ 1);
        const uint32_t qb = sb + S_Q + s * TILE;
        // dP = dO V^T  (its buffer held dQ of the previous pair: wait until that was drained)
        if (!mbar_wait(bar(5), par, abort_flag, p.err_word, 45)) { ok = false; break; }
        if (n > 0 && !mbar_wait(bar(12), (n - 1) & 1, abort_flag, p.err_word, 46)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(t_dp, kmajor(sb + S_DO, k), kmajor(sb + S_V, k), idesc_kk, k != 0);
        umma_commit(bar(8));
        // dV += P^T dO
        if (!mbar_wait(bar(10), par, abort_flag, p.err_word, 47)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(tmem_dv, mnmajor(sb + S_P, k), mnmajor(sb + S_DO, k), idesc_mm, (n | k) != 0);
        umma_commit(bar(6));  // dO slot free
        // dS(n) is in shared memory: its source buffer T[s ^ 1] is free for S(n + 1), which goes first so that the compute
        // warps can start on P(n + 1) while dK / dQ of this pair run
        if (!mbar_wait(bar(11), par, abort_flag, p.err_word, 48)) { ok = false; break; }
        if (n + 1 < num_pairs && !issue_s(n + 1)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(tmem_dk, mnmajor(sb + S_DS, k), mnmajor(qb, k), idesc_mm, (n | k) != 0);
        umma_commit(bar(3 + s));  // Q slot free
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(t_s, kmajor(sb + S_DS, k), mnmajor(sb + S_K, k), idesc_km, k != 0);
        umma_commit(bar(9));
      }
    }
  } else {
    // ---- compute warps: thread = (row r, column half)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;            // 0: columns 0..63, 1: columns 64..127
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    uint8_t* p_row = smem + S_P + half * PANEL + r * 128;
    uint8_t* ds_row = smem + S_DS + half * PANEL + r * 128;
    bool ok = true;
    const int cbase = half * 64;
    // softmax statistics of the row this thread owns, loaded one pair ahead of their use
    auto load_stats = [&](int n, float& lse2, float& delta) {
      const bool in_range = n < num_pairs && pair_q0(min(n, num_pairs - 1)) + r < q_len;
      const int n_ = min(n, num_pairs - 1);
      const long long idx = (long long)pair_head(n_) * p.total_q + q_begin + pair_q0(n_) + r;
      lse2 = in_range ? p.lse[idx] * 1.4426950408889634f : 0.f;
      delta = in_range ? p.delta[idx] : 0.f;
    };
    uint32_t pk[32];
    // P(n) = exp2(S(n) c - lse) -> registers (kept for dS) and shared memory (operand of dV)
    auto compute_p = [&](int n, float lse2) -> bool {
      const int qi = pair_q0(n) + r;
      // visible key columns of this row inside the key block: [col_lo, col_hi)
      int col_hi = k_len - k0;
      if (p.causal) col_hi = min(col_hi, qi + shift + 1 - k0);
      int col_lo = 0;
      if (p.window > 0) col_lo = max(0, qi + shift - p.window + 1 - k0);
      if (qi >= q_len) col_hi = col_lo;  // rows past the document contribute nothing
      const bool full = (col_lo <= cbase) && (col_hi >= cbase + 64);
      if (!mbar_wait(bar(7), n & 1, abort_flag, p.err_word, 49)) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_t(n & 1) + lane_addr + cbase + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float e0 = exp2f(__uint_as_float(v[i]) * p.scale_log2 - lse2);
          float e1 = exp2f(__uint_as_float(v[i + 1]) * p.scale_log2 - lse2);
          if (!full) {
            const int col = cbase + c * 32 + i;
            if (col < col_lo || col >= col_hi) e0 = 0.f;
            if (col + 1 < col_lo || col + 1 >= col_hi) e1 = 0.f;
          }
          __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
          pk[c * 16 + (i >> 1)] = *reinterpret_cast<uint32_t*>(&b);
        }
      }
      // the completion of S(n) that was just observed also covers dV(n - 1), the last reader of the P tile
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *reinterpret_cast<uint4*>(p_row + ((ch ^ (r & 7)) << 4)) = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(10));
      return true;
    };
    float lse2_next = 0.f, delta_next = 0.f, delta = 0.f;
    if (num_pairs > 0) {
      load_stats(0, lse2_next, delta_next);
      delta = delta_next;
      ok = compute_p(0, lse2_next);
      load_stats(1, lse2_next, delta_next);
    }
    for (int n = 0; n < num_pairs && ok; ++n) {
      const int s = n & 1;
      const uint32_t par = n & 1;
      // ---- dS(n) = P (dP - delta) scale
      if (!mbar_wait(bar(8), par, abort_flag, p.err_word, 50)) { ok = false; break; }
      tc_fence_after();
      uint32_t dsk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_t(s ^ 1) + lane_addr + cbase + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 pp = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&pk[c * 16 + (i >> 1)]));
          const float d0 = pp.x * (__uint_as_float(v[i]) - delta) * p.scale;
          const float d1 = pp.y * (__uint_as_float(v[i + 1]) - delta) * p.scale;
          __nv_bfloat162 b = __floats2bfloat162_rn(d0, d1);
          dsk[c * 16 + (i >> 1)] = *reinterpret_cast<uint32_t*>(&b);
        }
      }
      // dK(n - 1) / dQ(n - 1), the last readers of the dS tile, completed before dQ(n - 1) was drained
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *reinterpret_cast<uint4*>(ds_row + ((ch ^ (r & 7)) << 4)) = make_uint4(dsk[ch * 4], dsk[ch * 4 + 1], dsk[ch * 4 + 2], dsk[ch * 4 + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(11));
      // ---- P(n + 1), while dK(n) / dQ(n) run
      if (n + 1 < num_pairs) {
        delta = delta_next;
        if (!compute_p(n + 1, lse2_next)) { ok = false; break; }
        load_stats(n + 2, lse2_next, delta_next);
      }
      // ---- drain dQ(n) (this thread: 64 of the 128 head-dimension columns of its row)
      if (!mbar_wait(bar(9), par, abort_flag, p.err_word, 51)) { ok = false; break; }
      tc_fence_after();
      const int head = pair_head(n), qi = pair_q0(n) + r;
      const bool row_ok = qi < q_len;
      // accumulator layout [head][token / 32][column / 4][token % 32][4]: the 32 rows of a warp are adjacent
      const long long tok = q_begin + qi;
      float* dq_row = p.dq_accum + ((((long long)head * p.tok_groups + (tok >> 5)) * (D / 4) + (cbase >> 2)) * 32 + (tok & 31)) * 4;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_t(s) + lane_addr + cbase + c * 32, v);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            red_add_v4(dq_row + (c * 8 + (i >> 2)) * 128, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(12));
    }
    if (ok && num_pairs > 0) tc_fence_after();
    // ---- write dK, dV of this key block (bf16); rows past the document are skipped
    if (ok && num_pairs > 0) {
      // the last commit (bar 9 of the last pair) covered every MMA; it was observed above
      tc_fence_after();
    }
    const int krow = k0 + r;
    const bool have_acc = num_pairs > 0 && ok;  // warp-uniform
    __nv_bfloat16* base = p.dkv + (long long)(k_begin + min(krow, k_len - 1)) * p.dkv_stride + kv_head * D + half * 64;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const uint32_t t = which == 0 ? tmem_dk : tmem_dv;
      __nv_bfloat16* dst = base + (which == 0 ? p.k_col0 : p.v_col0);
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        if (have_acc) {
          tmem_ld32(t + lane_addr + half * 64 + c * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (krow < k_len) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g * 8 + i]);
            *reinterpret_cast<flb::bf16x8*>(dst + c * 32 + g * 8) = flb::pack8(f);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                  long long total_q, int heads) {
  const long long idx = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 4;  // 16 lanes per (token, head)
  const int sub = threadIdx.x & 15;
  if (idx >= total_q * heads) return;
  const long long t = idx / heads;
  const int h = (int)(idx - t * heads);
  float a[8], b[8];
  flb::unpack8(*reinterpret_cast<const flb::bf16x8*>(out + idx * D + sub * 8), a);
  flb::unpack8(*reinterpret_cast<const flb::bf16x8*>(dout + idx * D + sub * 8), b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += a[i] * b[i];
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (sub == 0) delta[(long long)h * total_q + t] = s;
}

// dq (bf16, packed rows) = dq_accum (fp32, layout [head][token / 32][column / 4][token % 32][4]).
// One CTA per (head, group of 32 tokens): the group's 16 KB are read as they lie (coalesced), turned in shared memory, and
// written as 256-byte row segments (half a warp per token), instead of 16-byte pieces at the row stride.
constexpr int kConvertStride = 33;  // float4 per column group in shared memory (32 tokens + 1: spreads the turned reads over banks)
__global__ void __launch_bounds__(256) attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long dq_stride,
                                                              int q_col0, long long total_q, long long tok_groups, int heads) {
  __shared__ float4 tile[(D / 4) * kConvertStride];
  const long long blocks = tok_groups * heads;
  for (long long block = blockIdx.x; block < blocks; block += gridDim.x) {
    const long long grp = block % tok_groups;
    const int head = (int)(block / tok_groups);
    const float4* src = reinterpret_cast<const float4*>(acc) + ((long long)head * tok_groups + grp) * (D / 4) * 32;
    __syncthreads();  // the previous block's reads of the tile are done
#pragma unroll
    for (int i = threadIdx.x; i < (D / 4) * 32; i += 256) tile[(i >> 5) * kConvertStride + (i & 31)] = src[i];
    __syncthreads();
#pragma unroll
    for (int i = threadIdx.x; i < 32 * (D / 8); i += 256) {
      const int tok_in = i / (D / 8), c8 = i % (D / 8);
      const long long tok = grp * 32 + tok_in;
      if (tok >= total_q) continue;
      float f[8];
      *reinterpret_cast<float4*>(f) = tile[(2 * c8) * kConvertStride + tok_in];
      *reinterpret_cast<float4*>(f + 4) = tile[(2 * c8 + 1) * kConvertStride + tok_in];
      *reinterpret_cast<flb::bf16x8*>(dq + tok * dq_stride + q_col0 + head * D + c8 * 8) = flb::pack8(f);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn bwd_encode_fn() {
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
bool bwd_row_tmap(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t stride_elems) {
  EncodeTiledFn enc = bwd_encode_fn();
  if (!enc) {
    fprintf(stderr, "flb_attention_bwd: cuTensorMapEncodeTiled entry point not found\n");
    return false;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {stride_elems * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t es[2] = {1, 1};
  CUresult res = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    res = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_ERROR_INVALID_CONTEXT) break;
    cudaFree(nullptr);  // a thread that made no runtime call yet (an autograd worker) has no current context: bind the primary one
  }
  if (res != CUDA_SUCCESS)
    fprintf(stderr, "flb_attention_bwd: tensor map rejected (code %d): base %p cols %llu rows %llu stride %llu elements\n", (int)res, base,
            (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)stride_elems);
  return res == CUDA_SUCCESS;
}
int* bwd_err_word() {
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

// Gradients of packed attention.  q / kv as in flb_attention_fwd; out, dout: [total_q, heads*128] contiguous;
// lse: [heads, total_q]; scratch: delta [heads, total_q] fp32 and dq_accum [heads * roundup(total_q, 32) * 128] fp32 (any contents).
// Writes dq (bf16) at columns q_col0.. of `dq` rows (stride dq_stride) and dk / dv at k_col0.. / v_col0.. of `dkv` rows.
FLB_API int flb_attention_bwd(const void* q, long long q_stride, int q_col0, const void* kv, long long kv_stride, int k_col0, int v_col0,
                              const void* out, const void* dout, const float* lse, const int* cu_q, const int* cu_k, int batch,
                              int max_seqlen_k, long long total_q, long long total_k, int heads, int kv_heads, int head_dim,
                              void* dq, long long dq_stride, void* dkv, long long dkv_stride, float* delta, float* dq_accum,
                              int causal, int window, float softmax_scale, cudaStream_t stream) {
  if (head_dim != D || heads % kv_heads || q_stride % 8 || kv_stride % 8 || dq_stride % 8 || dkv_stride % 8 || q_col0 % 8 || k_col0 % 8 || v_col0 % 8 || batch <= 0) return FLB_ERR_SHAPE;
  CUtensorMap tq, tkv, tdo;
  if (!bwd_row_tmap(&tq, q, (uint64_t)q_stride, (uint64_t)total_q, (uint64_t)q_stride)) return FLB_ERR_TMA;
  if (!bwd_row_tmap(&tkv, kv, (uint64_t)kv_stride, (uint64_t)total_k, (uint64_t)kv_stride)) return FLB_ERR_TMA;
  if (!bwd_row_tmap(&tdo, dout, (uint64_t)heads * D, (uint64_t)total_q, (uint64_t)heads * D)) return FLB_ERR_TMA;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BWD);
    if (e != cudaSuccess) return flb_record_cuda_error(e);
    configured = true;
  }
  const long long pairs = total_q * heads;
  attn_delta_kernel<<<(unsigned)((pairs * 16 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, delta, total_q, heads);
  FLB_CHECK_LAUNCH();
  const long long tok_groups = (total_q + 31) / 32;
  cudaError_t e = cudaMemsetAsync(dq_accum, 0, (size_t)tok_groups * 32 * heads * D * sizeof(float), stream);
  if (e != cudaSuccess) return flb_record_cuda_error(e);
  BwdParams p;
  p.cu_q = cu_q; p.cu_k = cu_k; p.lse = lse; p.delta = delta; p.dq_accum = dq_accum;
  p.dkv = (__nv_bfloat16*)dkv; p.dkv_stride = dkv_stride; p.total_q = total_q; p.tok_groups = tok_groups;
  p.heads = heads; p.kv_heads = kv_heads; p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0; p.do_col_stride = heads * D;
  p.kv_blocks_per_doc = (max_seqlen_k + BN - 1) / BN;
  p.causal = causal; p.window = window; p.scale = softmax_scale; p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.err_word = bwd_err_word();
  if (!p.err_word) return FLB_ERR_CUDA;
  dim3 grid(p.kv_blocks_per_doc * batch, kv_heads);
  attn_bwd_kernel<<<grid, kThreadsBwd, SMEM_BWD, stream>>>(tq, tkv, tdo, p);
  FLB_CHECK_LAUNCH();
  attn_dq_convert_kernel<<<148 * 8, 256, 0, stream>>>(dq_accum, (__nv_bfloat16*)dq, dq_stride, q_col0, total_q, tok_groups, heads);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_attention_bwd_error_word() {
  int* w = bwd_err_word();
  if (!w) return -1;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(w, 0, sizeof(int));
  return v;
}
