"""Checkpoint formats that store one global tensor per parameter (layout independent).

`fast_llm` format: `metadata.yaml` (with a `state_index` name -> file map) + `model_{i}.safetensors`, keys
`{parameter}/{shard}`.  The same streaming machinery serves external (Hugging Face) formats through weight converters:
tensors are exported stage by stage, converted as soon as a converter has all its inputs, and flushed to a new file
whenever `parameters_per_file` is exceeded, so no rank ever holds the whole model.
Parity: `fast_llm/engine/checkpoint/state_dict.py:41-277`.
"""

import abc
import json
import logging
import pathlib
import typing

import safetensors
import safetensors.torch
import torch
import yaml

from fast_llm_b200.engine.checkpoint.config import (
    CheckpointHandler,
    CheckpointLoadConfig,
    CheckpointLoadMetadataConfig,
    CheckpointSaveConfig,
    CheckpointSaveMetadataConfig,
    FastLLMCheckpointFormat,
)
from fast_llm_b200.engine.checkpoint.safe_load import SafeLoad
from fast_llm_b200.engine.multi_stage.config import CheckpointMetadata
from fast_llm_b200.parallel.collectives import gather_object, safe_barrier
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


class StateDictSaver:
    """Accumulates tensors and writes `{base}_{i}.safetensors` files plus a name -> file index."""

    def __init__(self, config: CheckpointSaveConfig, distributed, base_file_name: str = "model", serialize_metadata=None):
        self._config = config
        self._distributed = distributed
        dc = distributed.config
        self._do_save = dc.data_rank == 0 and dc.tensor_rank == 0
        prefix = base_file_name if dc.pipeline_parallel == 1 else f"{base_file_name}_{dc.pipeline_rank}"
        self._prefix = prefix
        self._tensors: dict[str, torch.Tensor] = {}
        self._count = 0
        self._file_index = 0
        self.index: dict[str, str] = {}

    def add_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if not self._do_save:
            return
        assert name not in self._tensors and name not in self.index, f"duplicate tensor {name}"
        if self._config.data_type is not None:
            tensor = tensor.to(self._config.data_type.torch)
        self._tensors[name] = tensor.detach().cpu().contiguous()
        self._count += tensor.numel()
        if self._count >= self._config.parameters_per_file:
            self._flush()

    def _flush(self) -> None:
        if not self._tensors:
            return
        file_name = f"{self._prefix}_{self._file_index}.safetensors"
        safetensors.torch.save_file(self._tensors, str(pathlib.Path(self._config.path) / file_name), metadata={"format": "pt"})
        for name in self._tensors:
            self.index[name] = file_name
        self._tensors, self._count = {}, 0
        self._file_index += 1

    def finalize(self) -> dict[str, str]:
        """Flush, then merge the indexes of all pipeline ranks on rank 0."""
        if self._do_save:
            self._flush()
        group = self._distributed.pipeline_group
        if group is not None and self._distributed.config.data_rank == 0 and self._distributed.config.tensor_rank == 0:
            gathered = gather_object(self.index, group, 0)
            if gathered is not None:
                merged = {}
                for part in gathered:
                    merged.update(part)
                self.index = merged
        return self.index


class StateDictCheckpointHandler(CheckpointHandler):
    base_file_name = "model"

    # ---- name / tensor conversion hooks
    @abc.abstractmethod
    def _export_tensors(self, parameter_name: str, shard_name: str, tensor: torch.Tensor, pending: dict) -> dict[str, torch.Tensor]:
        """Returns the external tensors that became complete by adding this one."""

    @abc.abstractmethod
    def _import_tensors(self, name: str, tensor: torch.Tensor, pending: dict) -> list[tuple[str, str, torch.Tensor]]:
        """Returns (parameter name, shard name, global tensor) triples that became complete by adding this one."""

    def _generated_tensors(self) -> typing.Iterable[tuple[str, str, torch.Tensor]]:
        """(parameter name, shard name, global tensor) triples that come from no file (parameters the format does not hold)."""
        return ()

    def _serialize_metadata(self, config: CheckpointSaveMetadataConfig, metadata: CheckpointMetadata, index: dict) -> None:
        raise NotImplementedError

    @classmethod
    def _load_index(cls, config: CheckpointLoadMetadataConfig) -> dict[str, str]:
        raise NotImplementedError

    # ---- save / load
    def save(self, config: CheckpointSaveConfig, metadata: CheckpointMetadata) -> None:
        model = self._model
        path = pathlib.Path(config.path)
        if model.config.distributed.rank == 0:
            path.mkdir(parents=True, exist_ok=True)
        safe_barrier(model.distributed.world_group, "state dict save", device=model.distributed.device)
        saver = StateDictSaver(config, model.distributed, self.base_file_name)
        pending: dict = {}
        shard_names = self.get_shard_names(config)
        for parameter_name, shard_name, tensor in model.get_state_tensor_iterator(shard_names, None):
            for name, converted in self._export_tensors(parameter_name, shard_name, tensor, pending).items():
                saver.add_tensor(name, converted)
        Assert.empty([k for k in pending if not str(k).startswith("_")])
        index = saver.finalize()
        if model.config.distributed.rank == 0:
            self._serialize_metadata(config, metadata, index)

    def load(self, config: CheckpointLoadConfig) -> dict | None:
        model = self._model
        shard_names = self.get_shard_names(config)
        metadata = self._load_metadata(config)
        index = self._load_index(config)
        files = sorted(set(index.values()))
        pending: dict = {}
        path = pathlib.Path(config.path)
        with SafeLoad(model, shard_names=shard_names, timeout=config.timeout) as context:
            for file_name in files:
                for name, tensor in _iter_file(path / file_name):
                    for parameter_name, shard_name, converted in self._import_tensors(name, tensor, pending):
                        if shard_name not in shard_names:
                            continue
                        count = model.import_state_tensor(parameter_name, shard_name, converted)
                        context.mark_as_loaded(count, (parameter_name, shard_name))
            for parameter_name, shard_name, generated in self._generated_tensors():
                if shard_name in shard_names:
                    context.mark_as_loaded(model.import_state_tensor(parameter_name, shard_name, generated), (parameter_name, shard_name))
        return metadata.metadata if metadata is not None else None


def _iter_file(path: pathlib.Path):
    if path.suffix == ".safetensors":
        with safetensors.safe_open(str(path), framework="pt", device="cpu") as f:
            for key in f.keys():
                yield key, f.get_tensor(key)
    elif path.suffix == ".bin":
        yield from torch.load(path, map_location="cpu", weights_only=True).items()
    else:
        raise NotImplementedError(f"Unknown checkpoint file type {path}")


class FastLLMCheckpointHandler(StateDictCheckpointHandler):
    format = FastLLMCheckpointFormat

    def _export_tensors(self, parameter_name, shard_name, tensor, pending):
        return {f"{parameter_name}/{shard_name}": tensor}

    def _import_tensors(self, name, tensor, pending):
        parameter_name, shard_name = name.rsplit("/", 1)
        return [(parameter_name, shard_name, tensor)]

    @classmethod
    def save_metadata(cls, config, metadata, index: dict | None = None) -> None:
        from fast_llm_b200.engine.checkpoint.distributed import _serialize_metadata

        pathlib.Path(config.path).mkdir(parents=True, exist_ok=True)
        data = _serialize_metadata(metadata)
        if index is not None:
            data["metadata"] = {**(data.get("metadata") or {}), "state_index": index}
        (pathlib.Path(config.path) / "metadata.yaml").write_text(yaml.safe_dump(data, sort_keys=False))

    def _serialize_metadata(self, config, metadata, index):
        self.save_metadata(config, metadata, index)

    @classmethod
    def _load_metadata(cls, config: CheckpointLoadMetadataConfig) -> CheckpointMetadata:
        data = yaml.safe_load((pathlib.Path(config.path) / "metadata.yaml").read_text())
        return CheckpointMetadata.from_dict(data).validate()

    @classmethod
    def _load_index(cls, config) -> dict[str, str]:
        data = yaml.safe_load((pathlib.Path(config.path) / "metadata.yaml").read_text())
        return data["metadata"]["state_index"]
