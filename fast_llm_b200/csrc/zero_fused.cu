// ZeRO gradient reduction and optimizer step fused with their collectives, over NVLink peer memory.
//
// Every data-parallel rank holds the full fp32 (or bf16) gradient buffer of a stage and the full bf16 weight buffer in
// symmetric memory: the same allocation exists at the same offset on every rank and all of them are mapped into every
// process (peer pointers).  Two kernels replace reduce-scatter -> copy -> norm -> Adam -> cast -> all-gather:
//
//   flb_rs_reduce   rank r sums slice r of ALL ranks' gradient buffers (plain peer loads, fixed rank order, so the
//                   result is deterministic), scales by 1/dp, writes the fp32 gradient shard and per-CTA partial sums
//                   of squares for the gradient norm.
//   flb_adam_push   AdamW on the rank's fp32 shard (weights, moments) and stores the new bf16 weights straight into
//                   slice r of EVERY rank's weight buffer (peer stores) - the all-gather happens inside the update.
//
// Ranks meet through flb_symm_barrier: a one-CTA kernel that writes an epoch number into each peer's signal pad
// (st.release.sys) and waits (ld.acquire.sys) until every peer has written the same epoch into ours.  The wait is bounded
// by a clock deadline; on expiry the kernel raises an error word and returns, so a missing peer can never hang the GPU.
// No multimem / TMA is involved: loads and stores are ordinary global accesses to peer addresses.
#include "common.cuh"

namespace {
using namespace flb;
constexpr int kThreads = 256;
constexpr int kMaxRanks = 16;
// Longest wait of one barrier in SM clock cycles; about 10 s at boost clock unless flb_symm_set_barrier_limit changes it.
long long g_barrier_limit_cycles = 20000000000ll;

// True when an earlier bounded wait on this stream gave up: the kernels below then leave memory untouched, because
// the peers' buffers they would read may be stale or half written.
__device__ __forceinline__ bool wait_failed(const int* err_word) {
  return err_word != nullptr && *reinterpret_cast<const volatile int*>(err_word) != 0;
}

struct PeerPtrs {
  void* p[kMaxRanks];
};

__global__ void symm_barrier_kernel(PeerPtrs signal_pads, int rank, int world, int slot, unsigned epoch, int* err_word,
                                    long long limit_cycles) {
  const int peer = threadIdx.x;
  if (peer >= world) return;
  // tell `peer` that this rank reached the barrier: pad layout [slot][source rank]
  unsigned* remote = reinterpret_cast<unsigned*>(signal_pads.p[peer]) + slot * kMaxRanks + rank;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const unsigned* local = reinterpret_cast<const unsigned*>(signal_pads.p[rank]) + slot * kMaxRanks + peer;
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local) : "memory");
    if ((int)(v - epoch) >= 0) break;
    if (clock64() - t0 > limit_cycles) {
      atomicExch(err_word, 100 + peer);
      break;
    }
    __nanosleep(200);
  }
}

template <typename GradT>
__device__ __forceinline__ float4 load4(const GradT* p, long long i);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p, long long i) {
  return reinterpret_cast<const float4*>(p)[i];
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  const uint2 raw = reinterpret_cast<const uint2*>(p)[i];
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

// grads.p[r]: base of rank r's gradient buffer for this stage (element type GradT); this rank reduces
// elements [rank*shard, (rank+1)*shard) into grad_shard (fp32).  shard % 4 == 0.
template <typename GradT>
__global__ void __launch_bounds__(kThreads)
rs_reduce_kernel(PeerPtrs grads, int rank, int world, long long shard, float scale, float* __restrict__ grad_shard,
                 int accumulate, float* __restrict__ sumsq_partial, const int* err_word) {
  __shared__ float scratch[32];
  if (wait_failed(err_word)) return;
  const long long nvec = shard >> 2;
  const long long base = (long long)rank * nvec;
  float ss = 0.f;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec; i += (long long)gridDim.x * kThreads) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = load4<GradT>(reinterpret_cast<const GradT*>(grads.p[r]), base + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    if (accumulate) {
      const float4 o = reinterpret_cast<const float4*>(grad_shard)[i];
      acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    reinterpret_cast<float4*>(grad_shard)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  const float t = block_sum(ss, scratch);
  if (threadIdx.x == 0 && sumsq_partial) sumsq_partial[blockIdx.x] = t;
}

// The same reduction with the sum formed inside NVSwitch: `mc` is the MULTICAST address of the gradient buffer (one address that
// stands for the same offset in every rank's symmetric allocation); `multimem.ld_reduce` returns the fp32 sum over all ranks of
// the 16 bytes it names, so a rank pulls its slice once instead of once per peer.  The order of the additions is the switch's,
// not rank order: results can differ from rs_reduce_kernel in the last bit, and this path is an option, off by default.
__global__ void __launch_bounds__(kThreads)
rs_reduce_multimem_kernel(const float* __restrict__ mc, int rank, long long shard, float scale, float* __restrict__ grad_shard,
                          int accumulate, float* __restrict__ sumsq_partial, const int* err_word) {
  __shared__ float scratch[32];
  if (wait_failed(err_word)) return;
  const long long nvec = shard >> 2;
  const float4* src = reinterpret_cast<const float4*>(mc) + (long long)rank * nvec;
  float ss = 0.f;
  auto pull = [&](long long i) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(src + i)
                 : "memory");
    return v;
  };
  auto finish = [&](long long i, float4 acc) {
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    if (accumulate) {
      const float4 o = reinterpret_cast<const float4*>(grad_shard)[i];
      acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    reinterpret_cast<float4*>(grad_shard)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  };
  const long long stride = (long long)gridDim.x * kThreads;
  long long i = blockIdx.x * (long long)kThreads + threadIdx.x;
  // four reductions in flight per thread: a round trip through the switch is several microseconds
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const float4 a = pull(i), b = pull(i + stride), c = pull(i + 2 * stride), d = pull(i + 3 * stride);
    finish(i, a); finish(i + stride, b); finish(i + 2 * stride, c); finish(i + 3 * stride, d);
  }
  for (; i < nvec; i += stride) finish(i, pull(i));
  const float t = block_sum(ss, scratch);
  if (threadIdx.x == 0 && sumsq_partial) sumsq_partial[blockIdx.x] = t;
}

// AdamW on n fp32 elements; the bf16 result goes to element offset `lp_offset` of every rank's weight buffer.
__global__ void __launch_bounds__(kThreads)
adam_push_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                 PeerPtrs weight_buffers, int world, long long lp_offset, long long n, float lr, float beta1, float beta2,
                 float eps, float wd, float inv_bc1, float inv_bc2, float gscale, const float* __restrict__ gscale_ptr,
                 const int* err_word) {
  if (wait_failed(err_word)) return;
  const float sc = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)kThreads + threadIdx.x; i < nvec; i += (long long)gridDim.x * kThreads) {
    float4 wv = reinterpret_cast<float4*>(w)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* wp = &wv.x; const float* gp = &gv.x; float* mp = &mv.x; float* vp = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gp[j] * sc;
      mp[j] = beta1 * mp[j] + (1.f - beta1) * gj;
      vp[j] = beta2 * vp[j] + (1.f - beta2) * gj * gj;
      wp[j] -= lr * ((mp[j] * inv_bc1) / (sqrtf(vp[j] * inv_bc2) + eps) + wd * wp[j]);
    }
    reinterpret_cast<float4*>(w)[i] = wv;
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y), hi = __floats2bfloat162_rn(wv.z, wv.w);
    const uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    for (int r = 0; r < world; ++r)
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(weight_buffers.p[r]) + lp_offset)[i] = packed;
  }
}

int fill_ptrs(PeerPtrs& out, const void* const* ptrs, int world) {
  if (world < 1 || world > kMaxRanks) return FLB_ERR_TOO_LARGE;
  for (int i = 0; i < kMaxRanks; ++i) out.p[i] = i < world ? const_cast<void*>(ptrs[i]) : nullptr;
  return FLB_OK;
}

}  // namespace

FLB_API int flb_symm_max_ranks() { return kMaxRanks; }
// Sets the longest wait of later barriers (SM clock cycles, > 0) and returns the previous limit.
FLB_API long long flb_symm_set_barrier_limit(long long cycles) {
  const long long old = g_barrier_limit_cycles;
  if (cycles > 0) g_barrier_limit_cycles = cycles;
  return old;
}
// Bytes of signal pad each rank must provide (zero-initialised): [slots][kMaxRanks] u32.
FLB_API int flb_symm_signal_pad_bytes(int slots) { return slots * kMaxRanks * 4; }

// All ranks of the group call this with the same slot and epoch (epochs of a slot must increase).
FLB_API int flb_symm_barrier(const void* const* signal_pads, int rank, int world, int slot, unsigned epoch, int* err_word,
                             cudaStream_t stream) {
  PeerPtrs pads;
  const int st = fill_ptrs(pads, signal_pads, world);
  if (st) return st;
  symm_barrier_kernel<<<1, 32, 0, stream>>>(pads, rank, world, slot, epoch, err_word, g_barrier_limit_cycles);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// out[i] = sum over slots s (in slot order) of in[s * n + i]; bf16 in and out, fp32 accumulation.  The reduce step of the
// fused GEMM + reduce-scatter: every tensor-parallel peer stored its partial tile rows into one slot of this rank's
// staging buffer from inside its GEMM epilogue.
__global__ void slot_sum_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int slots, long long n,
                                const int* err_word) {
  if (wait_failed(err_word)) return;
  const long long nvec = n >> 3;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < slots; ++s) {
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(in + s * n + v * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    *reinterpret_cast<bf16x8*>(out + v * 8) = pack8(acc);
  }
}

// Pull `bytes` (multiple of 16) from a peer's memory into local memory with a small grid, so that it can run beside a
// GEMM on the remaining SMs: the gather half of the fused all-gather + GEMM.  Remote lines are not cached in the local
// L2, so operands that many tiles re-read must cross NVLink once and be read locally afterwards.
__global__ void peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  // four independent loads in flight per thread hide the NVLink round trip
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) dst[i] = src[i];
}

// Push half of the fused all-gather + GEMM.  Every rank stores its [rows, width] shard into slot `rank` of the landing zone
// of each peer (one read of the source, world - 1 peer stores per 16 bytes) and then raises the peer's arrival word for that
// slot to `call`; the peer's GEMM (flb_gemm_gathered_bf16) waits on that word tile by tile.  Landing zones alternate
// between two halves by call parity, and the host side promises that everything that reads the zone of call j is in the
// stream before the push of call j + 2 starts.  So the push of call k may overwrite a peer's half as soon as that peer's own
// push of call k has started: each push first tells every peer "my call k has begun" (the words at done_offset) and then
// waits, bounded, for the same word from every peer.  A peer's rows cannot arrive before its push begins anyway, so this
// meeting costs the consuming GEMM nothing.  Nothing on this GPU waits for this kernel, and this kernel waits only for
// kernels of other GPUs.
__global__ void tp_push_kernel(const uint4* __restrict__ src, long long n16, PeerPtrs bases, long long dst_offset, long long flag_offset,
                               long long done_offset, int rank, int world, unsigned call, unsigned* local_counter, int* err_word,
                               long long limit_cycles) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < world && threadIdx.x != rank) {
    const int peer = threadIdx.x;
    if (blockIdx.x == 0) {  // this rank's call has begun: its readers of the half that is about to be overwritten are done
      unsigned* remote = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(bases.p[peer]) + done_offset) + rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(call) : "memory");
    }
    {
      const unsigned* local = reinterpret_cast<const unsigned*>(reinterpret_cast<const char*>(bases.p[rank]) + done_offset) + peer;
      const long long t0 = clock64();
      for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local) : "memory");
        if ((int)(v - call) >= 0) break;
        if (clock64() - t0 > limit_cycles) {
          atomicExch(err_word, 200 + peer);
          failed = 1;
          break;
        }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
  if (failed || wait_failed(err_word)) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += 2 * stride) {
    const bool second = i + stride < n16;
    const uint4 a = src[i];
    const uint4 b = second ? src[i + stride] : a;
    for (int step = 1; step < world; ++step) {
      const int peer = (rank + step) % world;
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(bases.p[peer]) + dst_offset);
      dst[i] = a;
      if (second) dst[i + stride] = b;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned ticket = atomicAdd(local_counter, 1u);
    if (ticket == gridDim.x - 1) {  // every CTA's stores are out: raise the arrival words
      *local_counter = 0u;
      __threadfence_system();
      for (int step = 1; step < world; ++step) {
        const int peer = (rank + step) % world;
        unsigned* flag = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(bases.p[peer]) + flag_offset);
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(call) : "memory");
      }
    }
  }
}

// bases[r]: rank r's symmetric buffer.  dst_offset: byte offset of this rank's slot in the landing half of this call;
// flag_offset: byte offset of the arrival word for (half, this rank); done_offset: byte offset of the `world` done words.
// local_counter: one zero-initialised word in this rank's memory.  bytes % 16 == 0.
FLB_API int flb_tp_push(const void* src, long long bytes, const void* const* bases, long long dst_offset, long long flag_offset,
                        long long done_offset, int rank, int world, unsigned call, unsigned* local_counter, int* err_word, int ctas,
                        cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world) return FLB_ERR_SHAPE;
  if (bytes % 16 || dst_offset % 16 || flag_offset % 4 || done_offset % 4 || (reinterpret_cast<uintptr_t>(src) & 15)) return FLB_ERR_SHAPE;
  PeerPtrs ptrs;
  for (int r = 0; r < world; ++r) ptrs.p[r] = const_cast<void*>(bases[r]);
  if (ctas <= 0) ctas = 32;
  tp_push_kernel<<<ctas, 512, 0, stream>>>((const uint4*)src, bytes >> 4, ptrs, dst_offset, flag_offset, done_offset, rank, world, call,
                                           local_counter, err_word, g_barrier_limit_cycles);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// Stream-ordered wait until every peer's push of `call` has arrived (for consumers that are not flb_gemm_gathered_bf16, e.g. a
// weight-gradient GEMM over the whole gathered operand).  Waits only on words written by other GPUs; bounded.
__global__ void tp_wait_kernel(const unsigned* flags, unsigned call, int world, int rank, int* err_word, long long limit_cycles) {
  const int peer = threadIdx.x;
  if (peer >= world || peer == rank) return;
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + peer) : "memory");
    if ((int)(v - call) >= 0) break;
    if (clock64() - t0 > limit_cycles) {
      atomicExch(err_word, 300 + peer);
      break;
    }
    __nanosleep(200);
  }
}

FLB_API int flb_tp_wait(const unsigned* flags, unsigned call, int world, int rank, int* err_word, cudaStream_t stream) {
  if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world) return FLB_ERR_SHAPE;
  tp_wait_kernel<<<1, 32, 0, stream>>>(flags, call, world, rank, err_word, g_barrier_limit_cycles);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_peer_copy(const void* src, void* dst, long long bytes, int ctas, cudaStream_t stream) {
  if (bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return FLB_ERR_SHAPE;
  if (bytes == 0) return FLB_OK;
  if (ctas <= 0) ctas = 24;
  peer_copy_kernel<<<ctas, 512, 0, stream>>>((const uint4*)src, (uint4*)dst, bytes >> 4);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_slot_sum_bf16(const void* in, void* out, int slots, long long n, const int* err_word, cudaStream_t stream) {
  if (n % 8 || slots <= 0) return FLB_ERR_SHAPE;
  if (n == 0) return FLB_OK;
  long long blocks = ((n >> 3) + kThreads - 1) / kThreads;
  if (blocks > 148 * 8) blocks = 148 * 8;
  slot_sum_kernel<<<(int)blocks, kThreads, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, slots, n, err_word);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

FLB_API int flb_rs_reduce_blocks() { return 148 * 4; }

// grad_ptrs[r]: rank r's gradient buffer of the stage (grad_dtype 0 fp32 / 1 bf16).  sumsq_partial: flb_rs_reduce_blocks()
// floats (may be null).  Call between two flb_symm_barrier's: peers must have finished writing, and must not overwrite
// their buffers before every rank has read them.  err_word (may be null): the error word of those barriers; when it is
// set the kernel does nothing.
FLB_API int flb_rs_reduce(const void* const* grad_ptrs, int grad_dtype, int rank, int world, long long shard, float scale,
                          float* grad_shard, int accumulate, float* sumsq_partial, const int* err_word, cudaStream_t stream) {
  if (shard % 4) return FLB_ERR_SHAPE;
  PeerPtrs grads;
  const int st = fill_ptrs(grads, grad_ptrs, world);
  if (st) return st;
  const int blocks = flb_rs_reduce_blocks();
  if (grad_dtype == 0)
    rs_reduce_kernel<float><<<blocks, kThreads, 0, stream>>>(grads, rank, world, shard, scale, grad_shard, accumulate, sumsq_partial, err_word);
  else
    rs_reduce_kernel<__nv_bfloat16><<<blocks, kThreads, 0, stream>>>(grads, rank, world, shard, scale, grad_shard, accumulate, sumsq_partial, err_word);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// flb_rs_reduce through the multicast mapping of the fp32 gradient buffer (`multicast_grads`: the multicast address of the
// buffer's first element).  Same contract: between two barriers; shard % 4 == 0.
FLB_API int flb_rs_reduce_multimem(const void* multicast_grads, int rank, int world, long long shard, float scale, float* grad_shard,
                                   int accumulate, float* sumsq_partial, const int* err_word, cudaStream_t stream) {
  if (shard <= 0) return FLB_OK;
  if ((shard % 4) || multicast_grads == nullptr || rank < 0 || rank >= world || (reinterpret_cast<uintptr_t>(multicast_grads) & 15)) return FLB_ERR_SHAPE;
  rs_reduce_multimem_kernel<<<flb_rs_reduce_blocks(), kThreads, 0, stream>>>((const float*)multicast_grads, rank, shard, scale, grad_shard,
                                                                            accumulate, sumsq_partial, err_word);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}

// n % 4 == 0; lp_offset (elements into every rank's bf16 weight buffer) % 4 == 0.
FLB_API int flb_adam_push(float* w, const float* g, float* m, float* v, const void* const* weight_buffers, int world,
                          long long lp_offset, long long n, float lr, float beta1, float beta2, float eps, float wd, int step,
                          float gscale, const float* gscale_ptr, const int* err_word, cudaStream_t stream) {
  if (n <= 0) return FLB_OK;
  if ((n % 4) || (lp_offset % 4)) return FLB_ERR_SHAPE;
  PeerPtrs bufs;
  const int st = fill_ptrs(bufs, weight_buffers, world);
  if (st) return st;
  const float inv_bc1 = 1.f / (1.f - powf(beta1, (float)step));
  const float inv_bc2 = 1.f / (1.f - powf(beta2, (float)step));
  long long blocks = ((n >> 2) + kThreads - 1) / kThreads;
  if (blocks > 148 * 8) blocks = 148 * 8;
  adam_push_kernel<<<(int)blocks, kThreads, 0, stream>>>(w, g, m, v, bufs, world, lp_offset, n, lr, beta1, beta2, eps, wd,
                                                          inv_bc1, inv_bc2, gscale, gscale_ptr, err_word);
  FLB_CHECK_LAUNCH();
  return FLB_OK;
}
