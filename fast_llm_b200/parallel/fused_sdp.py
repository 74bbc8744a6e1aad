"""Sequence-data parallelism: key / value all-gather and gradient reduce-scatter through symmetric memory.

Every rank of a sequence-data group holds one slice of each sequence and needs the keys and values of all of them
(`fast_llm/layers/attention/attention.py:359-372` gathers with NCCL and reduce-scatters the gradient).  Here

    gather          the rank publishes its [t, w] slice in its symmetric buffer, the group meets at one bounded
                    device-side barrier, and a copy kernel (`flb_peer_copy`, plain peer loads) pulls the other slices
                    into the output;
    reduce-scatter  the rank stores chunk j of its gradient into slot `rank` of rank j's staging buffer (peer stores),
                    one barrier, and `flb_slot_sum_bf16` adds the slots in rank order (deterministic).

Both buffers are double-buffered, so the barrier of call k also proves that every peer is done with the buffer of call
k - 1.  bf16 only; anything else, or a slice larger than the buffers sized by the first call, takes the NCCL path.
"""

import logging

import torch

from fast_llm_b200.ops import _lib
from fast_llm_b200.parallel.symmetric import SymmetricArena

logger = logging.getLogger(__name__)

_contexts: dict[int, "FusedSequenceDataExchange"] = {}
_COPY_CTAS = 32


def enable(group, device) -> "FusedSequenceDataExchange":
    context = _contexts.get(id(group))
    if context is None:
        context = _contexts[id(group)] = FusedSequenceDataExchange(group, device)
    return context


def get(group) -> "FusedSequenceDataExchange | None":
    return _contexts.get(id(group)) if group is not None else None


def disable(group) -> None:
    _contexts.pop(id(group), None)


class FusedSequenceDataExchange:
    def __init__(self, group, device):
        self.group, self.world, self.rank = group, group.size(), group.rank()
        self._device = device
        self.arena: SymmetricArena | None = None
        self._slice_bytes = 0
        self._gathers = self._scatters = 0
        self._warned = False

    def usable(self, slice_: torch.Tensor) -> bool:
        """`slice_`: this rank's [t, w] part (every rank passes the same shape)."""
        if not (slice_.is_cuda and slice_.dtype == torch.bfloat16 and slice_.dim() == 2 and slice_.numel() % 8 == 0):
            return False
        nbytes = slice_.numel() * 2
        if self.arena is None:
            self._slice_bytes = (nbytes + 255) // 256 * 256
            # [publish x2 | staging (world slots) x2]
            self.arena = SymmetricArena(2 * self._slice_bytes + 2 * self.world * self._slice_bytes, self.group, self._device)
        if nbytes > self._slice_bytes and not self._warned:
            self._warned = True  # not silent: larger slices take the NCCL path
            logger.warning(f"Sequence-data exchange: a slice of {nbytes} bytes does not fit the symmetric buffers sized for "
                           f"{self._slice_bytes} bytes by the first call; slices of this size use NCCL.")
        return nbytes <= self._slice_bytes

    def gather(self, slice_: torch.Tensor) -> torch.Tensor:
        rows, width = slice_.shape
        nbytes = rows * width * 2
        offset = (self._gathers & 1) * self._slice_bytes
        self._gathers += 1
        self.arena.buffer[offset : offset + nbytes].view(torch.bfloat16).view(rows, width).copy_(slice_)
        self.arena.barrier(1)
        out = torch.empty(self.world * rows, width, dtype=slice_.dtype, device=slice_.device)
        out[self.rank * rows : (self.rank + 1) * rows].copy_(slice_)
        lib = _lib.get_lib()
        for step in range(1, self.world):
            j = (self.rank + step) % self.world
            _lib.check(lib.flb_peer_copy(self.arena.peer_ptrs[j] + offset, out[j * rows : (j + 1) * rows].data_ptr(), nbytes, _COPY_CTAS,
                                         _lib.stream_ptr()), "flb_peer_copy")
            _lib.count_launch()
        return out

    def reduce_scatter(self, full: torch.Tensor) -> torch.Tensor:
        rows, width = full.shape[0] // self.world, full.shape[1]
        nbytes = rows * width * 2
        base = 2 * self._slice_bytes + (self._scatters & 1) * self.world * self._slice_bytes
        self._scatters += 1
        lib = _lib.get_lib()
        for step in range(self.world):
            j = (self.rank + 1 + step) % self.world
            _lib.check(lib.flb_peer_copy(full[j * rows : (j + 1) * rows].data_ptr(), self.arena.peer_ptrs[j] + base + self.rank * nbytes, nbytes,
                                         _COPY_CTAS, _lib.stream_ptr()), "flb_peer_copy")
            _lib.count_launch()
        self.arena.barrier(2)
        out = torch.empty(rows, width, dtype=full.dtype, device=full.device)
        staged = self.arena.buffer[base : base + self.world * nbytes]
        _lib.check(lib.flb_slot_sum_bf16(staged.data_ptr(), out.data_ptr(), self.world, rows * width, self.arena.error_word.data_ptr(),
                                         _lib.stream_ptr()), "flb_slot_sum_bf16")
        _lib.count_launch()
        return out
