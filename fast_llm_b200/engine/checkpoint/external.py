"""Conversion between this framework's parameters / config and external (Hugging Face style) checkpoints.

A format handler provides
  * `export_config(base_model_config) -> dict` and `import_config(dict) -> base-model config dict`,
  * `get_weight_converters(base_model_config)`: a list of `WeightConverter`s, each relating a tuple of our parameter
    names to a tuple of external names with an invertible tensor transformation (identity, split, transpose,
    key/value split, per-expert split).
Saving and loading stream through `StateDictCheckpointHandler`.  Coverage is checked: every parameter of the model must
be claimed by exactly one converter.  Parity: `fast_llm/engine/checkpoint/external.py:83-1433`,
`fast_llm/engine/checkpoint/huggingface.py:44-226`.
"""

import json
import logging
import pathlib
import shutil
import typing

import torch

from fast_llm_b200.engine.checkpoint.config import CheckpointLoadMetadataConfig, CheckpointSaveMetadataConfig
from fast_llm_b200.engine.checkpoint.state_dict import StateDictCheckpointHandler
from fast_llm_b200.engine.multi_stage.config import CheckpointMetadata
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


class WeightConverter:
    """Identity: one of our tensors <-> one external tensor."""

    def __init__(self, fast_llm_name: str | tuple[str, ...], export_name: str | tuple[str, ...], config=None):
        self.fast_llm_name = (fast_llm_name,) if isinstance(fast_llm_name, str) else tuple(fast_llm_name)
        self.export_name = (export_name,) if isinstance(export_name, str) else tuple(export_name)
        self._config = config

    def export_weight(self, weight: tuple[torch.Tensor, ...]) -> tuple[torch.Tensor, ...]:
        return weight

    def import_weight(self, weight: tuple[torch.Tensor, ...]) -> tuple[torch.Tensor, ...]:
        return weight


class IgnoreImportWeightConverter(WeightConverter):
    """External tensors with no counterpart here (e.g. rotary inverse-frequency buffers)."""

    def __init__(self, export_name):
        super().__init__((), export_name)

    def import_weight(self, weight):
        return ()


class IgnoreExportWeightConverter(WeightConverter):
    """Our tensors with no counterpart in the external format."""

    def __init__(self, fast_llm_name):
        super().__init__(fast_llm_name, ())

    def export_weight(self, weight):
        return ()

    def import_weight(self, weight):
        raise NotImplementedError("cannot import a parameter the external format does not have")


class CopyWeightConverter(WeightConverter):
    """One external tensor feeds several of ours (tied copies)."""

    def export_weight(self, weight):
        return weight[:1]

    def import_weight(self, weight):
        return tuple(weight[0].clone() for _ in self.fast_llm_name)


class SplitWeightConverter(WeightConverter):
    """Ours is the concatenation along dim 0 of the external tensors (gate|up, key|value)."""

    def export_weight(self, weight):
        (merged,) = weight
        return tuple(t.contiguous() for t in merged.chunk(len(self.export_name), dim=0))

    def import_weight(self, weight):
        return (torch.cat(list(weight), dim=0),)


KeyValueWeightConverter = SplitWeightConverter


class TransposeWeightConverter(WeightConverter):
    """Ours is stored [in, out]; the external format stores [out, in]."""

    def export_weight(self, weight):
        return (weight[0].t().contiguous(),)

    def import_weight(self, weight):
        return (weight[0].t().contiguous(),)


class ExpertSplitWeightConverter(WeightConverter):
    """Ours stacks all experts along dim 0 ([experts * rows, cols]); externally one (or `parts`) tensor per expert.
    `export_name` lists, expert by expert, the `parts` names of each expert."""

    def __init__(self, fast_llm_name, export_name, num_experts: int, parts: int = 1, transpose: bool = False):
        super().__init__(fast_llm_name, export_name)
        self._num_experts, self._parts, self._transpose = num_experts, parts, transpose
        Assert.eq(len(self.export_name), num_experts * parts)

    def export_weight(self, weight):
        (merged,) = weight
        out = []
        for expert in merged.chunk(self._num_experts, dim=0):
            for part in expert.chunk(self._parts, dim=0):
                out.append(part.t().contiguous() if self._transpose else part.contiguous())
        return tuple(out)

    def import_weight(self, weight):
        experts = []
        for e in range(self._num_experts):
            parts = weight[e * self._parts : (e + 1) * self._parts]
            parts = [p.t() if self._transpose else p for p in parts]
            experts.append(torch.cat(parts, dim=0))
        return (torch.cat(experts, dim=0).contiguous(),)


class ExternalStateDictCheckpointHandler(StateDictCheckpointHandler):
    """Base of external formats; subclasses implement the three conversion hooks."""

    architecture: typing.ClassVar[str | None] = None

    def __init__(self, model):
        super().__init__(model)
        converters = self.get_weight_converters(model.config.base_model)
        self._export_converters = {}
        for c in converters:
            for name in c.fast_llm_name:
                assert name not in self._export_converters, f"parameter {name} claimed twice"
                self._export_converters[name] = c
        self._import_converters = {name: c for c in converters for name in c.export_name}
        missing = [n for n in model.parameter_names if n not in self._export_converters]
        unknown = [n for n in self._export_converters if n not in model.parameter_names]
        if missing or unknown:
            raise ValueError(f"{type(self).__name__}: converters do not cover the model: missing {missing[:8]}, unknown {unknown[:8]}")

    # ---- to implement
    @classmethod
    def export_config(cls, base_model_config) -> dict:
        raise NotImplementedError

    @classmethod
    def import_config(cls, config: dict) -> dict:
        raise NotImplementedError

    @classmethod
    def get_weight_converters(cls, base_model_config) -> list[WeightConverter]:
        raise NotImplementedError

    # ---- streaming conversion
    def get_shard_names(self, config) -> tuple[str, ...]:
        Assert.eq(bool(config.optimizer_state), False, msg="external formats hold weights only")
        return ("weights",) if config.model_weights else ()

    def _export_tensors(self, parameter_name, shard_name, tensor, pending):
        converter = self._export_converters[parameter_name]
        slot = pending.setdefault(id(converter), {})
        slot[parameter_name] = tensor
        if len(slot) < len(converter.fast_llm_name):
            return {}
        del pending[id(converter)]
        exported = converter.export_weight(tuple(slot[n] for n in converter.fast_llm_name))
        return dict(zip(converter.export_name, exported, strict=True))

    def _import_tensors(self, name, tensor, pending):
        converter = self._import_converters.get(name)
        if converter is None:
            logger.warning(f"Ignoring unknown tensor {name} in checkpoint")
            return []
        slot = pending.setdefault(id(converter), {})
        slot[name] = tensor
        if len(slot) < len(converter.export_name):
            return []
        del pending[id(converter)]
        imported = converter.import_weight(tuple(slot[n] for n in converter.export_name))
        return [(n, "weights", t) for n, t in zip(converter.fast_llm_name, imported, strict=True)]


class HuggingfaceStateDictCheckpointHandler(ExternalStateDictCheckpointHandler):
    """Hugging Face layout: `config.json`, `model_{i}.safetensors`, `model.safetensors.index.json`."""

    @classmethod
    def save_metadata(cls, config: CheckpointSaveMetadataConfig, metadata: CheckpointMetadata, index: dict | None = None) -> None:
        path = pathlib.Path(config.path)
        path.mkdir(parents=True, exist_ok=True)
        hf_config = cls.export_config(metadata.config.base_model)
        hf_config.setdefault("architectures", [cls.architecture] if cls.architecture else [])
        # the dtype the tensors are written in: the cast requested for this save, else the fp32 master weights
        data_type = getattr(config, "data_type", None)
        hf_config["torch_dtype"] = str(data_type.torch if data_type is not None else torch.float32).removeprefix("torch.")
        (path / "config.json").write_text(json.dumps(hf_config, indent=2))
        if index is not None:
            (path / "model.safetensors.index.json").write_text(
                json.dumps({"metadata": {"fast_llm_metadata": _jsonable(metadata.metadata)}, "weight_map": index}, indent=2))
        for extra in cls.get_extra_files():
            shutil.copy(extra, path / pathlib.Path(extra).name)

    @classmethod
    def get_extra_files(cls) -> list[pathlib.Path]:
        """Modelling code to ship next to exported checkpoints (formats with custom Hugging Face code)."""
        return []

    def _serialize_metadata(self, config, metadata, index):
        self.save_metadata(config, metadata, index)

    @classmethod
    def _load_metadata(cls, config: CheckpointLoadMetadataConfig) -> CheckpointMetadata:
        path = pathlib.Path(config.path)
        hf_config = json.loads((path / "config.json").read_text())
        from fast_llm_b200.engine.multi_stage.config import FastLLMModelConfig

        model_class = cls.get_model_config_class()
        base_model = cls.import_config(hf_config)
        extra = {}
        index_path = path / "model.safetensors.index.json"
        if index_path.exists():
            extra = json.loads(index_path.read_text()).get("metadata", {}).get("fast_llm_metadata", {}) or {}
        return CheckpointMetadata(fast_llm_version="0.4.0", model=model_class, format=cls.format,
                                  config=model_class.from_dict({"base_model": base_model}), shards=["weights"], metadata=extra).validate()

    @classmethod
    def get_model_config_class(cls):
        raise NotImplementedError

    @classmethod
    def _load_index(cls, config) -> dict[str, str]:
        path = pathlib.Path(config.path)
        for index_name in ("model.safetensors.index.json", "pytorch_model.bin.index.json"):
            if (path / index_name).exists():
                return json.loads((path / index_name).read_text())["weight_map"]
        for single in ("model.safetensors", "pytorch_model.bin"):
            if (path / single).exists():
                from fast_llm_b200.engine.checkpoint.state_dict import _iter_file

                return {name: single for name, _ in _iter_file(path / single)}
        raise FileNotFoundError(f"No weights found in {path}")


def _jsonable(obj):
    if isinstance(obj, dict):
        return {str(k): _jsonable(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_jsonable(v) for v in obj]
    if isinstance(obj, (int, float, str, bool)) or obj is None:
        return obj
    return str(obj)
