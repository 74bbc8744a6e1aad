"""Tensor-parallel GEMMs fused with their collectives over NVLink peer memory (sequence-parallel layout).

The three collectives around a sequence-parallel linear layer never run as separate operations here:

    all-gather -> GEMM      `all_gather_matmul`: ONE GEMM launch over all T rows.  Every rank pushes its [T/tp, H] shard into
                            its slot of each peer's landing zone (`flb_tp_push`, 32 CTAs on a side stream, one read and
                            tp - 1 peer stores per 16 bytes) and then raises an arrival word on the peer; the GEMM's TMA
                            producer visits the row blocks of the local chunk first and, before the first load of a row
                            block that belongs to another rank, waits (bounded, error word) for that rank's arrival word
                            (`flb_gemm_gathered_bf16`).  The math on rows that are already here covers the transfer of the
                            rest, and the tile grid is that of the full GEMM instead of tp launches of a quarter of the rows.
                            Landing zones alternate by call parity; a zone may be read until the second next gather starts,
                            and a push begins by meeting the peers' pushes of the same call (a word each way), which tells
                            it that their readers of the zone it is about to overwrite are done.  `start_gather` /
                            `matmul_gathered` / `finish_gather` expose the pieces, so that one gather serves the dgrad GEMM
                            and the weight-gradient GEMM of a layer.  (Reading the A operand straight from the peer through TMA works but is 3.7x
                            slower: remote lines are not cached in the local L2, so every N-tile re-fetches its A rows over
                            NVLink.)  `single_launch = False` selects the older pipeline: a pull kernel (`flb_peer_copy`) per
                            peer chunk on a side stream and one GEMM launch per chunk, ordered by events.
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
import os

import torch

from fast_llm_b200.ops import _lib
from fast_llm_b200.ops.gemm import _EPI_ACC_BF16, _EPI_ACC_F32, _EPI_STORE_BF16, _EPI_STORE_F32, gemm_raw
from fast_llm_b200.parallel.symmetric import SymmetricArena

logger = logging.getLogger(__name__)

_contexts: dict[int, "FusedTensorParallel"] = {}

_GATHER_SLOT, _SCATTER_SLOT = 1, 2
# control words at the end of the arena: arrival words [2 halves][16 ranks], then done words [16 ranks] (4 bytes each)
_MAX_RANKS = 16
_CONTROL_BYTES = 256 * ((3 * _MAX_RANKS * 4 + 255) // 256)


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


class _PendingGather:
    """A pushed all-gather in flight: the landing zone, the address of its arrival words and the call number they will reach."""

    __slots__ = ("landing", "flags", "call", "rows", "done_event")

    def __init__(self, landing, flags, call, rows, done_event):
        self.landing, self.flags, self.call, self.rows, self.done_event = landing, flags, call, rows, done_event


class FusedTensorParallel:
    def __init__(self, group, device, max_tokens: int | None, max_width: int | None):
        self.group, self.world, self.rank = group, group.size(), group.rank()
        self._device = device
        self.max_tokens = self.max_width = None
        self._refused: set = set()
        if max_tokens is not None:
            self._allocate(max_tokens, max_width)

    def _allocate(self, max_tokens: int, max_width: int) -> None:
        device = self._device
        assert max_tokens % self.world == 0
        self.max_tokens, self.max_width = max_tokens, max_width
        shard_bytes = max_tokens // self.world * max_width * 2
        staging_bytes = max_tokens * max_width * 2
        self._shard_bytes, self._staging_bytes = shard_bytes, staging_bytes
        # [2 published shards | 2 reduce-scatter staging zones | 2 landing zones of the pushed all-gather | control words]
        self._landing_base = 2 * shard_bytes + 2 * staging_bytes
        self._control_base = self._landing_base + 2 * staging_bytes
        self.arena = SymmetricArena(self._control_base + _CONTROL_BYTES, self.group, device)
        self.arena.buffer[self._control_base :].zero_()
        torch.cuda.synchronize(device)
        torch.distributed.barrier(self.group)  # nobody pushes before every rank's control words are zero
        self._push_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self._push_calls = 0
        self._scatter_map_cache: dict = {}
        self._push_event = torch.cuda.Event()
        self._bases = self.arena.peer_pointer_array()
        self.single_launch = os.environ.get("FLB_TP_SINGLE_LAUNCH", "1") != "0"
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
        ok = tokens <= self.max_tokens and width <= self.max_width and tokens % self.world == 0 and width % 8 == 0
        if not ok and (tokens, width) not in self._refused:
            # not silent: the caller takes the NCCL path for this shape
            self._refused.add((tokens, width))
            logger.warning(f"Fused tensor-parallel kernels: a [{tokens}, {width}] activation does not fit the symmetric buffers sized for "
                           f"[{self.max_tokens}, {self.max_width}] by the first fused call (or is not divisible by the group size {self.world} / 8); "
                           f"this shape uses NCCL collectives.")
        return ok

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
    def all_gather_matmul(self, x_shard: torch.Tensor, weight: torch.Tensor, b_mn: bool, return_gathered: bool = False):
        """concat_j(x_j) @ W^T (b_mn False: W is [N, K]) or @ W (b_mn True: W is [K, N]) -> [T, N].
        `return_gathered` (single-launch path only): also return the [T, K] gathered operand, a view of the landing zone that
        stays valid until the second next call of this method."""
        rows, k = x_shard.shape
        n = weight.shape[1] if b_mn else weight.shape[0]
        if self.single_launch and self.world <= _MAX_RANKS:
            return self._pushed_all_gather_matmul(x_shard, weight, b_mn, return_gathered)
        assert not return_gathered
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

    def start_gather(self, shard: torch.Tensor) -> "_PendingGather":
        """Begin the all-gather of `shard` ([T/tp, width]) into the landing zone of this call: the push to the peers runs on the
        side stream, this rank's rows are copied in place on the current stream.  The gathered rows of the peers may be read by
        `flb_gemm_gathered_bf16` (which waits per row block) or after `finish_gather`.  The landing zone stays valid until the
        second next `start_gather`: everything that reads it must be in the stream by then (the push of call k + 2 tells the
        peers that this rank is done with the zone of call k)."""
        rows, width = shard.shape
        self._push_calls += 1
        call = self._push_calls
        half = call & 1
        nbytes = rows * width * 2
        zone = self._landing_base + half * self._staging_bytes
        landing = self.arena.buffer[zone : zone + self.world * nbytes].view(torch.bfloat16).view(self.world * rows, width)
        flags = self._control_base + half * _MAX_RANKS * 4
        done = self._control_base + 2 * _MAX_RANKS * 4
        main = torch.cuda.current_stream()
        if not shard.is_contiguous():
            shard = shard.contiguous()
        # the push starts once the shard exists; being behind this point of the main stream it also follows every earlier
        # consumer of a landing zone
        self._push_event.record(main)
        self._copy_stream.wait_event(self._push_event)
        shard.record_stream(self._copy_stream)
        with torch.cuda.stream(self._copy_stream):
            _lib.check(_lib.get_lib().flb_tp_push(shard.data_ptr(), nbytes, self._bases, zone + self.rank * nbytes, flags + self.rank * 4, done,
                                                  self.rank, self.world, call, self._push_counter.data_ptr(), self.arena.error_word.data_ptr(), 32,
                                                  _lib.stream_ptr()), "flb_tp_push")
            _lib.count_launch()
            done_event = torch.cuda.Event()
            done_event.record(self._copy_stream)
        landing[self.rank * rows : (self.rank + 1) * rows].copy_(shard)
        return _PendingGather(landing, self.arena.buffer.data_ptr() + flags, call, rows, done_event)

    def finish_gather(self, pending: "_PendingGather") -> torch.Tensor:
        """The gathered [T, width] operand, complete on the current stream from here on."""
        _lib.check(_lib.get_lib().flb_tp_wait(pending.flags, pending.call, self.world, self.rank, self.arena.error_word.data_ptr(),
                                              _lib.stream_ptr()), "flb_tp_wait")
        _lib.count_launch()
        torch.cuda.current_stream().wait_event(pending.done_event)
        return pending.landing

    def matmul_gathered(self, pending: "_PendingGather", weight: torch.Tensor, b_mn: bool) -> torch.Tensor:
        """gathered @ W^T (or @ W) in one GEMM launch that waits, row block by row block, for the peers' rows of `pending`."""
        tokens, k = pending.landing.shape
        n = weight.shape[1] if b_mn else weight.shape[0]
        out = torch.empty(tokens, n, dtype=pending.landing.dtype, device=pending.landing.device)
        _lib.check(_lib.get_lib().flb_gemm_gathered_bf16(pending.landing.data_ptr(), weight.data_ptr(), out.data_ptr(), tokens, n, k, k,
                                                         weight.stride(0), n, int(b_mn), pending.flags, pending.call, pending.rows, self.rank,
                                                         _lib.stream_ptr()), "flb_gemm_gathered_bf16")
        _lib.count_launch()
        # the shard may be rewritten in place by later work on this stream: not before the push has read it (the GEMM cannot
        # finish before the peers' pushes, which run beside this rank's, so this wait costs nothing)
        torch.cuda.current_stream().wait_event(pending.done_event)
        return out

    def matmul_gathered_gated(self, pending: "_PendingGather", w1: torch.Tensor, act_code: int) -> tuple[torch.Tensor, torch.Tensor]:
        """`matmul_gathered` for the first layer of a gated MLP (`w1` = [gate rows; up rows]) with the activation in the GEMM's
        epilogue: returns (h, act(gate) * up)."""
        tokens, k = pending.landing.shape
        f = w1.shape[0] // 2
        h = torch.empty(tokens, 2 * f, dtype=torch.bfloat16, device=w1.device)
        a = torch.empty(tokens, f, dtype=torch.bfloat16, device=w1.device)
        _lib.check(_lib.get_lib().flb_gemm_gathered_gated_bf16(pending.landing.data_ptr(), w1.data_ptr(), h.data_ptr(), a.data_ptr(), tokens, f, k, k,
                                                               w1.stride(0), 2 * f, f, act_code, pending.flags, pending.call, pending.rows,
                                                               self.rank, _lib.stream_ptr()), "flb_gemm_gathered_gated_bf16")
        _lib.count_launch()
        torch.cuda.current_stream().wait_event(pending.done_event)
        return h, a

    def _pushed_all_gather_matmul(self, x_shard: torch.Tensor, weight: torch.Tensor, b_mn: bool, return_gathered: bool = False):
        pending = self.start_gather(x_shard)
        out = self.matmul_gathered(pending, weight, b_mn)
        return (out, pending.landing) if return_gathered else out

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
        if self.single_launch and rows % 256 == 0:
            # one GEMM over all tokens; each row block leaves through the tensor map of its owner's staging slot
            maps = self._scatter_maps(offset, rows, n)
            _lib.check(_lib.get_lib().flb_gemm_scatter_bf16(x.data_ptr(), weight.data_ptr(), maps.data_ptr(), tokens, n, k, x.stride(0), weight.stride(0),
                                                            int(b_mn), rows, (self.rank + 1) % self.world, _lib.stream_ptr()), "flb_gemm_scatter_bf16")
            _lib.count_launch()
            return self._sum_slots(local, rows, n, x)
        for step in range(self.world):
            j = (self.rank + 1 + step) % self.world  # remote chunks first: their stores travel while the local one computes
            gemm_raw(x[j * rows : (j + 1) * rows], weight, local[self.rank], rows, n, k, False, b_mn, _EPI_STORE_BF16,
                     c_ptr=self.arena.peer_ptrs[j] + offset + self.rank * slot_bytes, direct_store=self.direct_peer_stores and j != self.rank)
        return self._sum_slots(local, rows, n, x)

    def _sum_slots(self, local: torch.Tensor, rows: int, n: int, like: torch.Tensor) -> torch.Tensor:
        self.arena.barrier(_SCATTER_SLOT)
        out = torch.empty(rows, n, dtype=like.dtype, device=like.device)
        _lib.check(_lib.get_lib().flb_slot_sum_bf16(local.data_ptr(), out.data_ptr(), self.world, rows * n, self.arena.error_word.data_ptr(),
                                                    _lib.stream_ptr()), "flb_slot_sum_bf16")
        _lib.count_launch()
        return out

    def _scatter_maps(self, offset: int, rows: int, n: int) -> torch.Tensor:
        """Device array of one tensor map per rank over that rank's staging slot for this rank's partial rows (built once per
        staging half and shape)."""
        key = (offset, rows, n)
        maps = self._scatter_map_cache.get(key)
        if maps is None:
            import ctypes

            host = torch.empty(self.world * 128 + 64, dtype=torch.uint8)
            shift = (-host.data_ptr()) % 64
            aligned = host[shift : shift + self.world * 128]
            slot_bytes = rows * n * 2
            destinations = (ctypes.c_void_p * self.world)(*[self.arena.peer_ptrs[j] + offset + self.rank * slot_bytes for j in range(self.world)])
            _lib.check(_lib.get_lib().flb_gemm_scatter_maps(aligned.data_ptr(), destinations, self.world, rows, n, n), "flb_gemm_scatter_maps")
            device_buffer = torch.empty(self.world * 128 + 64, dtype=torch.uint8, device=self._device)
            device_shift = (-device_buffer.data_ptr()) % 64
            maps = device_buffer[device_shift : device_shift + self.world * 128]
            maps.copy_(aligned)
            torch.cuda.current_stream().synchronize()  # once per shape: the host buffer may go away
            self._scatter_map_cache[key] = maps
        return maps

    # ---- all-gather + weight gradient
    def gathered_wgrad(self, full: torch.Tensor, shard: torch.Tensor, out: torch.Tensor, accumulate: bool, shard_is_a: bool) -> torch.Tensor:
        """out (+)= sum_j a_j^T b_j over token chunks j, where one operand (`full`, [T, .]) is local and the other is the
        gather of every rank's `shard` ([T/tp, .]).  `shard_is_a`: the gathered side is `a`."""
        rows = shard.shape[0]
        if self.single_launch and self.world <= _MAX_RANKS:
            return self.wgrad_from_gathered(full, self.finish_gather(self.start_gather(shard)), out, accumulate, shard_is_a)
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

    @staticmethod
    def wgrad_from_gathered(full: torch.Tensor, gathered: torch.Tensor, out: torch.Tensor, accumulate: bool, gathered_is_a: bool) -> torch.Tensor:
        """out (+)= a^T b over all tokens with one operand already gathered ([T, .]): one GEMM launch, one accumulate pass."""
        a, b = (gathered, full) if gathered_is_a else (full, gathered)
        f32 = out.dtype == torch.float32
        epilogue = (_EPI_ACC_F32 if accumulate else _EPI_STORE_F32) if f32 else (_EPI_ACC_BF16 if accumulate else _EPI_STORE_BF16)
        gemm_raw(a, b, out, a.shape[1], b.shape[1], a.shape[0], True, True, epilogue)
        return out
