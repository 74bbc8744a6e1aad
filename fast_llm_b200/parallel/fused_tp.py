"""Tensor-parallel GEMMs fused with their collectives over NVLink peer memory (sequence-parallel layout).

The three collectives around a sequence-parallel linear layer never run as separate operations here:

    all-gather -> GEMM      `all_gather_matmul`: every rank publishes its [T/tp, H] shard in symmetric memory; a small
                            copy kernel (`flb_peer_copy`, 24 CTAs, plain peer loads) pulls chunk j+1 into local memory on a
                            side stream while the GEMM of chunk j runs on the other SMs.  (Reading the A operand straight
                            from the peer through TMA works but is 3.7x slower: remote lines are not cached in the local
                            L2, so every N-tile re-fetches its A rows over NVLink.)
    GEMM -> reduce-scatter  `matmul_reduce_scatter`: the GEMM for token chunk j stores its partial tiles from the epilogue
                            into slot `rank` of rank j's staging buffer (peer stores leave as each tile finishes, under
                            the remaining math); one `flb_slot_sum_bf16` adds the tp slots in rank order (deterministic).
    all-gather -> wgrad     `gathered_wgrad`: dW += sum_j a_j^T b_j with one side read from peers chunk by chunk, accumulated
                            by the GEMM epilogue.

Synchronisation is one bounded device-side barrier per call (signal pads, `flb_symm_barrier`); buffers are double-buffered
so the barrier of call k also releases the buffers of call k-1.  Replaces the NCCL calls at
`fast_llm/functional/linear.py:121,154,166-168,206,225`.
"""

import logging

import torch

from fast_llm_b200.ops import _lib
from fast_llm_b200.ops.gemm import _EPI_ACC_BF16, _EPI_ACC_F32, _EPI_STORE_BF16, _EPI_STORE_F32, gemm_raw
from fast_llm_b200.parallel.symmetric import SymmetricArena

logger = logging.getLogger(__name__)

_contexts: dict[int, "FusedTensorParallel"] = {}

_GATHER_SLOT, _SCATTER_SLOT = 1, 2


def get(group) -> "FusedTensorParallel | None":
    return _contexts.get(id(group)) if group is not None else None


def enable(group, device, max_tokens: int, max_width: int) -> "FusedTensorParallel":
    """Create (once) the symmetric buffers of a tensor group.  max_tokens: tokens of a full (gathered) micro-batch;
    max_width: widest gathered / reduced activation (the hidden size)."""
    context = _contexts.get(id(group))
    if context is None:
        context = _contexts[id(group)] = FusedTensorParallel(group, device, max_tokens, max_width)
    return context


def enable_lazy(group, device) -> "FusedTensorParallel":
    """Like `enable`, but the buffers are sized (and allocated, collectively) by the first fused call."""
    context = _contexts.get(id(group))
    if context is None:
        context = _contexts[id(group)] = FusedTensorParallel(group, device, None, None)
    return context


def usable(group, sequence_parallel: bool, *tensors: torch.Tensor) -> "FusedTensorParallel | None":
    """The group's context if the fused kernels can serve these operands (bf16, contiguous, 16-byte aligned, CUDA)."""
    if not sequence_parallel or group is None:
        return None
    context = _contexts.get(id(group))
    if context is None:
        return None
    for t in tensors:
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0):
            return None
    return context


def disable(group) -> None:
    _contexts.pop(id(group), None)


class FusedTensorParallel:
    def __init__(self, group, device, max_tokens: int | None, max_width: int | None):
        self.group, self.world, self.rank = group, group.size(), group.rank()
        self._device = device
        self.max_tokens = self.max_width = None
        if max_tokens is not None:
            self._allocate(max_tokens, max_width)

    def _allocate(self, max_tokens: int, max_width: int) -> None:
        device = self._device
        assert max_tokens % self.world == 0
        self.max_tokens, self.max_width = max_tokens, max_width
        shard_bytes = max_tokens // self.world * max_width * 2
        staging_bytes = max_tokens * max_width * 2
        self._shard_bytes, self._staging_bytes = shard_bytes, staging_bytes
        self.arena = SymmetricArena(2 * shard_bytes + 2 * staging_bytes, self.group, device)
        self._gather_calls = self._scatter_calls = 0
        self.direct_peer_stores = False  # True: register stores instead of TMA tensor stores into the peers' staging slots
        # local landing zone of gathered operands, side stream and per-chunk events for the copy / GEMM pipeline
        self._gathered = torch.empty(max_tokens * max_width, dtype=torch.bfloat16, device=device)
        self._copy_stream = torch.cuda.Stream(device=device)
        self._chunk_events = [torch.cuda.Event() for _ in range(self.world)]
        self._ready_event, self._done_event = torch.cuda.Event(), torch.cuda.Event()

    # ---- helpers
    def fits(self, tokens: int, width: int) -> bool:
        if self.max_tokens is None:
            # sized by the first call (every rank makes the same call): tokens of a micro-batch and the hidden size
            if tokens % self.world or width % 8:
                return False
            self._allocate(tokens, width)
        return tokens <= self.max_tokens and width <= self.max_width and tokens % self.world == 0 and width % 8 == 0

    def _gather_offset(self, call: int) -> int:
        return (call & 1) * self._shard_bytes

    def _staging_offset(self, call: int) -> int:
        return 2 * self._shard_bytes + (call & 1) * self._staging_bytes

    def _gather(self, shard: torch.Tensor) -> tuple[torch.Tensor, list]:
        """Publish this rank's shard, meet the peers, and start pulling their shards (nearest rank first) into the local
        gathered buffer on the copy stream.  Returns the [T, width] gathered tensor and one event per chunk (None = ready)."""
        call = self._gather_calls
        self._gather_calls += 1
        offset = self._gather_offset(call)
        rows, width = shard.shape
        nbytes = rows * width * 2
        published = self.arena.buffer[offset : offset + nbytes].view(torch.bfloat16).view(rows, width)
        published.copy_(shard)
        self.arena.barrier(_GATHER_SLOT)
        gathered = self._gathered[: rows * width * self.world].view(rows * self.world, width)
        main = torch.cuda.current_stream()
        self._copy_stream.wait_event(self._done_event)  # the previous gather's consumers are done with the landing zone
        self._ready_event.record(main)
        self._copy_stream.wait_event(self._ready_event)
        events: list = [None] * self.world
        lib = _lib.get_lib()
        with torch.cuda.stream(self._copy_stream):
            for step in range(1, self.world):
                j = (self.rank + step) % self.world
                _lib.check(lib.flb_peer_copy(self.arena.peer_ptrs[j] + offset, gathered[j * rows : (j + 1) * rows].data_ptr(), nbytes, 24,
                                             _lib.stream_ptr()), "flb_peer_copy")
                _lib.count_launch()
                self._chunk_events[j].record(self._copy_stream)
                events[j] = self._chunk_events[j]
        gathered[self.rank * rows : (self.rank + 1) * rows].copy_(shard)
        return gathered, events

    def _release_gathered(self) -> None:
        self._done_event.record(torch.cuda.current_stream())

    # ---- all-gather + GEMM
    def all_gather_matmul(self, x_shard: torch.Tensor, weight: torch.Tensor, b_mn: bool) -> torch.Tensor:
        """concat_j(x_j) @ W^T (b_mn False: W is [N, K]) or @ W (b_mn True: W is [K, N]) -> [T, N]."""
        rows, k = x_shard.shape
        n = weight.shape[1] if b_mn else weight.shape[0]
        gathered, events = self._gather(x_shard)
        out = torch.empty(rows * self.world, n, dtype=x_shard.dtype, device=x_shard.device)
        main = torch.cuda.current_stream()
        for step in range(self.world):
            j = (self.rank + step) % self.world  # the local chunk first, while the peers' chunks cross the links
            if events[j] is not None:
                main.wait_event(events[j])
            gemm_raw(gathered[j * rows : (j + 1) * rows], weight, out[j * rows : (j + 1) * rows], rows, n, k, False, b_mn, _EPI_STORE_BF16)
        self._release_gathered()
        return out

    # ---- GEMM + reduce-scatter
    def matmul_reduce_scatter(self, x: torch.Tensor, weight: torch.Tensor, b_mn: bool) -> torch.Tensor:
        """reduce_scatter_rows(x @ W^T or x @ W) -> [T/tp, N]; x holds all tokens and this rank's slice of the contraction."""
        tokens, k = x.shape
        n = weight.shape[1] if b_mn else weight.shape[0]
        rows = tokens // self.world
        call = self._scatter_calls
        self._scatter_calls += 1
        offset = self._staging_offset(call)
        slot_bytes = rows * n * 2
        local = self.arena.buffer[offset : offset + self.world * slot_bytes].view(torch.bfloat16).view(self.world, rows, n)
        for step in range(self.world):
            j = (self.rank + 1 + step) % self.world  # remote chunks first: their stores travel while the local one computes
            gemm_raw(x[j * rows : (j + 1) * rows], weight, local[self.rank], rows, n, k, False, b_mn, _EPI_STORE_BF16,
                     c_ptr=self.arena.peer_ptrs[j] + offset + self.rank * slot_bytes, direct_store=self.direct_peer_stores and j != self.rank)
        self.arena.barrier(_SCATTER_SLOT)
        out = torch.empty(rows, n, dtype=x.dtype, device=x.device)
        _lib.check(_lib.get_lib().flb_slot_sum_bf16(local.data_ptr(), out.data_ptr(), self.world, rows * n, self.arena.error_word.data_ptr(),
                                                    _lib.stream_ptr()), "flb_slot_sum_bf16")
        _lib.count_launch()
        return out

    # ---- all-gather + weight gradient
    def gathered_wgrad(self, full: torch.Tensor, shard: torch.Tensor, out: torch.Tensor, accumulate: bool, shard_is_a: bool) -> torch.Tensor:
        """out (+)= sum_j a_j^T b_j over token chunks j, where one operand (`full`, [T, .]) is local and the other is the
        gather of every rank's `shard` ([T/tp, .]).  `shard_is_a`: the gathered side is `a`."""
        rows = shard.shape[0]
        gathered, events = self._gather(shard)
        m = shard.shape[1] if shard_is_a else full.shape[1]
        n = full.shape[1] if shard_is_a else shard.shape[1]
        f32 = out.dtype == torch.float32
        main = torch.cuda.current_stream()
        for step in range(self.world):
            j = (self.rank + step) % self.world
            if events[j] is not None:
                main.wait_event(events[j])
            chunk, peer_chunk = full[j * rows : (j + 1) * rows], gathered[j * rows : (j + 1) * rows]
            acc = accumulate or step > 0
            epilogue = (_EPI_ACC_F32 if acc else _EPI_STORE_F32) if f32 else (_EPI_ACC_BF16 if acc else _EPI_STORE_BF16)
            a, b = (peer_chunk, chunk) if shard_is_a else (chunk, peer_chunk)
            gemm_raw(a, b, out, m, n, rows, True, True, epilogue)
        self._release_gathered()
        return out
