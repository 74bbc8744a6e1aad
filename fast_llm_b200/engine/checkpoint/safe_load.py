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

    def _world(self):
        distributed = getattr(self._model, "distributed", None) or getattr(self._model, "_distributed", None)
        group = getattr(distributed, "world_group", None)
        device = getattr(distributed, "device", torch.device("cpu"))
        return group, device

    def _validate(self) -> None:
        errors = []
        group, device = self._world()
        total = sum(self._model.get_shard(name).numel() for name in self._shard_names)
        # ---- no element may still hold the NaN it was pre-filled with, on any rank
        missing = torch.zeros(1, dtype=torch.int64, device=device)
        for name in self._shard_names:
            for piece in self._model.get_shard(name).flatten().split(100_000_000):  # bounded temporaries
                missing += torch.isnan(piece).sum()
        local_missing = int(missing.item())
        if group is not None:
            all_reduce(missing, group=group)
        global_missing = int(missing.item())
        if global_missing:
            errors.append(f"{global_missing:,} state entries were not loaded (on this rank: {local_missing:,})")
        # ---- every rank wrote as many elements as its shards hold
        counts = torch.tensor([self._loaded, total], dtype=torch.int64, device=device)
        if group is not None:
            all_reduce(counts, group=group)
        if int(counts[0]) != int(counts[1]):
            errors.append(f"element count mismatch: loaded {int(counts[0]):,}, expected {int(counts[1]):,} over all ranks "
                          f"(on this rank: {self._loaded:,} of {total:,}; some elements loaded more than once?)")
        # ---- per parameter and shard: the counts of all ranks add up to the ranks' shares of that parameter
        reported = torch.tensor([int(bool(self._loaded_parameters))], dtype=torch.int64, device=device)
        if group is not None:
            all_reduce(reported, op=torch.distributed.ReduceOp.MIN, group=group)
        if int(reported.item()):  # the same decision on every rank: the check below runs collectives
            self._check_parameters(errors, group, device)
        if errors:
            if local_missing:
                for _, _, fsdp, sl in self._model.iter_fsdps():
                    for shard_name in self._shard_names:
                        shard = self._model.get_shard(shard_name)[sl]
                        for pname, piece in fsdp.split_shard(shard).items():
                            n = int(torch.isnan(piece).sum().item())
                            if n:
                                errors.append(f"  {pname} [{shard_name}]: {n:,} of {piece.numel():,} local elements missing")
            raise RuntimeError("Checkpoint load incomplete:\n" + "\n".join(errors[:50]))
        logger.info(f"{self._loaded:,} state entries loaded successfully")

    def _check_parameters(self, errors: list[str], group, device) -> None:
        """Loaders that report per-parameter counts are checked parameter by parameter: for every (parameter, shard) the
        number of elements written must equal the number of elements of it that live in this rank's shard, on every rank
        (one all-reduce of the per-parameter differences, so every rank names the same offenders)."""
        expected: dict[tuple[str, str], int] = {}
        for _, _, fsdp, _sl in self._model.iter_fsdps():
            for pname in fsdp.parameter_names:
                begin, end = fsdp.parameter_range_in_shard(pname)
                for shard_name in self._shard_names:
                    expected[(pname, shard_name)] = expected.get((pname, shard_name), 0) + max(end - begin, 0)
        loaded: dict[tuple[str, str], int] = {}
        for (pname, shard_name), count in self._loaded_parameters.items():
            if shard_name == "all":  # a loader that fills every shard of a parameter at once reports their sum
                for name in self._shard_names:
                    loaded[(pname, name)] = loaded.get((pname, name), 0) + count // len(self._shard_names)
            else:
                loaded[(pname, shard_name)] = loaded.get((pname, shard_name), 0) + count
        # a parameter of another pipeline rank's stages is reported with a count of zero: nothing of it lives here
        unknown = [key for key, count in loaded.items() if key not in expected and count]
        if unknown:
            errors.append(f"counts reported for unknown (parameter, shard) pairs: {unknown[:8]}")
        keys = sorted(expected)
        difference = torch.tensor([loaded.get(k, 0) - expected[k] for k in keys], dtype=torch.int64, device=device)
        worst = difference.abs()
        if group is not None and group.size() > 1:
            # Ranks of different pipeline stages hold different parameter lists.  Every rank takes part in the same two
            # collectives whatever it holds: the first tells all of them whether the lists agree, and only then are the
            # per-parameter differences combined (otherwise each rank reports its own).
            import zlib

            digest = zlib.crc32(repr(keys).encode())
            probe = torch.tensor([digest, -digest], dtype=torch.int64, device=device)
            all_reduce(probe, op=torch.distributed.ReduceOp.MAX, group=group)
            same_keys = int(probe[0]) == digest and int(probe[1]) == -digest
            agreed = torch.tensor([int(same_keys)], dtype=torch.int64, device=device)
            all_reduce(agreed, op=torch.distributed.ReduceOp.MIN, group=group)
            if int(agreed.item()):
                all_reduce(worst, op=torch.distributed.ReduceOp.MAX, group=group)
        for key, here, anywhere in zip(keys, difference.tolist(), worst.tolist()):
            if anywhere:
                errors.append(f"  {key[0]} [{key[1]}]: loaded {loaded.get(key, 0):,} of {expected[key]:,} local elements "
                              f"(difference here {here:+,}, largest on any rank {anywhere:,})")
