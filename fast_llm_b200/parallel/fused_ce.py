"""Vocabulary-parallel cross-entropy statistics exchanged over NVLink peer memory instead of all-reduces.

Each rank's statistics kernel stores (max, sum-exp, target logit) per token straight into slot `rank` of every peer's
buffer; one bounded device-side barrier later, the gradient kernel merges the `world` local slots per token while it
computes the loss and the logit gradients.  Replaces two all-reduces of `[tokens]` vectors per loss call
(`fast_llm/functional/triton/entropy_loss.py`, `fast_llm/functional/entropy_loss.py:44-75` in the reference use
`all_reduce` for the maximum, the sum of exponentials and the target logit).  Buffers are double-buffered: the barrier of
call k also guarantees that every peer has finished reading the buffer of call k-1.
"""

import logging

import torch

from fast_llm_b200.ops import _lib
from fast_llm_b200.parallel.symmetric import SymmetricArena

logger = logging.getLogger(__name__)
_contexts: dict[int, "FusedStatisticsExchange"] = {}


def enable(group, device) -> "FusedStatisticsExchange":
    context = _contexts.get(id(group))
    if context is None:
        context = _contexts[id(group)] = FusedStatisticsExchange(group, device)
    return context


def get(group) -> "FusedStatisticsExchange | None":
    return _contexts.get(id(group)) if group is not None else None


def disable(group) -> None:
    _contexts.pop(id(group), None)


class FusedStatisticsExchange:
    def __init__(self, group, device):
        self.group, self.world, self.rank = group, group.size(), group.rank()
        self._device = device
        self._arena: SymmetricArena | None = None
        self._rows = 0
        self._calls = 0
        self._warned = False
        self.fallbacks = 0  # calls that did not fit the buffers and went through all-reduces

    def slots(self, rows: int):
        """(local [world, rows, 3] fp32 view, peer pointer array) for this call, or None if `rows` exceeds the buffers
        (sized, collectively, by the first call: every rank of a vocabulary-parallel group sees the same tokens)."""
        if self._arena is None:
            self._rows = rows
            self._arena = SymmetricArena(2 * self.world * rows * 12, self.group, self._device)
        if rows > self._rows or self.world > 8:
            if not self._warned:
                self._warned = True
                logger.warning(f"Loss statistics of {rows} tokens exceed the peer-memory buffers sized for {self._rows} by the first call: "
                               "this and later larger calls use all-reduces instead")
            self.fallbacks += 1
            return None
        offset = (self._calls & 1) * self.world * self._rows * 12
        self._calls += 1
        local = self._arena.buffer[offset : offset + self.world * rows * 12].view(torch.float32).view(self.world, rows, 3)
        return local, self._arena.peer_pointer_array(offset)

    def barrier(self) -> None:
        self._arena.barrier(0)
