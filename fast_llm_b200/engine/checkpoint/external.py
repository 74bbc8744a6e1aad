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
        self._adapt_to_lora(model)
        self._import_converters = {name: c for c in converters for name in c.export_name}
        # A tied weight whose users sit on different pipeline ranks has a copy with a name of its own there (the output
        # weights next to the embedding table).  The format holds the tensor once: the owner exports it, and an import
        # hands the owner's tensor to the copy as well (every rank reads every file, so no message is needed).
        self._tied_copies: dict[str, list[str]] = {}
        for owner, copy_, _, _ in getattr(model, "_tied_remote", ()):
            if copy_.tensor_name not in self._export_converters:
                self._tied_copies.setdefault(owner.tensor_name, []).append(copy_.tensor_name)
        copies = {name for names in self._tied_copies.values() for name in names}
        missing = [n for n in model.parameter_names if n not in self._export_converters and n not in self._adapter_owner and n not in copies]
        unknown = [n for n in self._export_converters if n not in model.parameter_names]
        if missing or unknown:
            raise ValueError(f"{type(self).__name__}: converters do not cover the model: missing {missing[:8]}, unknown {unknown[:8]}")

    def _adapt_to_lora(self, model) -> None:
        """External formats know nothing of LoRA.  A wrapped layer keeps its weight as `<layer>.base.weight` next to
        `<layer>.lora_a_weight` / `lora_b_weight`: the converter of `<layer>.weight` is pointed at the base weight; on export
        the low-rank update is merged into it (W + alpha / rank * B A, so the exported model computes what the trained one
        does); on import the adapters start from their initialisers (A random, B zero)."""
        from fast_llm_b200.layers.peft import LoRALinear

        self._adapter_owner: dict[str, WeightConverter] = {}  # adapter parameter -> converter of its base weight
        self._adapters: dict[int, list[tuple[str, str, str, float, bool]]] = {}  # converter -> (weight, A, B, scale, transposed)
        names = set(model.parameter_names)
        wrapped = {}
        for layer in model.base_model.get_layers():
            inner = layer.unwrap()
            for name, sub in inner.named_sublayers(f"{inner.module_name}."):
                if isinstance(sub, LoRALinear):
                    wrapped[name] = sub
        for prefix, lora in wrapped.items():
            for suffix in ("weight", "bias"):
                plain, based = f"{prefix}.{suffix}", f"{prefix}.base.{suffix}"
                if plain in self._export_converters and based in names:
                    converter = self._export_converters.pop(plain)
                    converter.fast_llm_name = tuple(based if n == plain else n for n in converter.fast_llm_name)
                    self._export_converters[based] = converter
            converter = self._export_converters.get(f"{prefix}.base.weight")
            if converter is None:
                continue
            a_name, b_name = f"{prefix}.lora_a_weight", f"{prefix}.lora_b_weight"
            self._adapter_owner[a_name] = self._adapter_owner[b_name] = converter
            self._adapters.setdefault(id(converter), []).append(
                (f"{prefix}.base.weight", a_name, b_name, lora._config.alpha / lora._config.rank, bool(getattr(lora.base, "transposed_weight", False))))

    def _generated_tensors(self):
        """Adapters have no counterpart in the checkpoint: they start from their initialisers."""
        model = self._model
        for name in self._adapter_owner:
            stage = model._stages[model._parameter_stages[name]]
            if model._parameter_stages[name] not in model._stages_on_device:
                continue
            meta = stage.get_parameter_meta(name)
            Assert.custom(lambda m: not m.is_tensor_parallel, meta)
            tensor = torch.empty(meta.global_shape, dtype=torch.float32, device=model.distributed.device)
            meta.init_parameter(tensor, model.distributed)
            yield name, "weights", tensor

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
        if any(parameter_name in names for names in self._tied_copies.values()):
            return {}  # the owner of the tied weight writes it
        converter = self._export_converters.get(parameter_name) or self._adapter_owner[parameter_name]
        adapters = self._adapters.get(id(converter), ())
        slot = pending.setdefault(id(converter), {})
        slot[parameter_name] = tensor
        if len(slot) < len(converter.fast_llm_name) + 2 * len(adapters):
            return {}
        del pending[id(converter)]
        for weight_name, a_name, b_name, scale, transposed in adapters:
            update = slot[b_name].float() @ slot[a_name].float() * scale  # [out, in]
            slot[weight_name] = (slot[weight_name].float() + (update.t() if transposed else update)).to(slot[weight_name].dtype)
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
        out = [(n, "weights", t) for n, t in zip(converter.fast_llm_name, imported, strict=True)]
        for name, _, value in list(out):
            out += [(copy_, "weights", value) for copy_ in self._tied_copies.get(name, ())]
        return out


class TrackedConfig(dict):
    """An external configuration dictionary that remembers which of its keys a converter looked at (nested dictionaries
    included), so that the fields a format silently dropped can be named after the import."""

    def __init__(self, data: dict, prefix: str = "", root: "TrackedConfig | None" = None):
        super().__init__(data)
        self._prefix = prefix
        self._root = self if root is None else root
        if root is None:
            self._read: set[str] = set()

    def _touch(self, key):
        self._root._read.add(self._prefix + str(key))

    def _wrap(self, key, value):
        return TrackedConfig(value, f"{self._prefix}{key}.", self._root) if isinstance(value, dict) and not isinstance(value, TrackedConfig) else value

    def __getitem__(self, key):
        self._touch(key)
        return self._wrap(key, super().__getitem__(key))

    def get(self, key, default=None):
        self._touch(key)
        return self._wrap(key, super().get(key, default))

    def __contains__(self, key):
        self._touch(key)
        return super().__contains__(key)

    def unread(self) -> list[str]:
        """Leaf keys never read, a nested dictionary counting as read when it was fetched whole and not looked into."""
        out = []

        def walk(data: dict, prefix: str):
            for key, value in dict.items(data):
                name = prefix + str(key)
                if isinstance(value, dict) and value and any(r.startswith(name + ".") for r in self._root._read):
                    walk(value, name + ".")
                elif name not in self._root._read:
                    out.append(name)

        walk(self, "")
        return out


def effective_architecture(config) -> dict:
    """The architecture of a configuration in a form where two spellings of the same model compare equal: every field hinted
    `architecture`, the dynamic type of every sub-configuration (a rotary or mixer of another type is another model), and
    for each linear layer whether it really has a bias (its own `bias.enabled`, else the owner's `add_linear_biases`).
    Parameter-efficient fine-tuning is left out: it adds trainable tensors, not architecture."""
    from fast_llm_b200.config.core import Config, FieldHint, _serialize

    out = {}
    if type(config)._dynamic_type_names:
        out["type"] = next(iter(type(config)._dynamic_type_names.values()))
    default_bias = getattr(config, "add_linear_biases", None)
    for name, field in config.fields().items():
        value = getattr(config, name)
        if name == "peft":
            continue  # adapters are merged into the weights they adapt when a model leaves in an external format
        if isinstance(value, Config):
            bias = getattr(value, "bias", None)
            if default_bias is not None and bias is not None and hasattr(bias, "enabled"):
                out[f"{name}.has_bias"] = bool(default_bias if bias.enabled is None else bias.enabled)
            sub = effective_architecture(value)
            if sub:
                out[name] = sub
        elif isinstance(value, dict) and any(isinstance(v, Config) for v in value.values()):
            out[name] = {k: effective_architecture(v) for k, v in value.items()}
        elif isinstance(value, (list, tuple)) and any(isinstance(v, Config) for v in value):
            out[name] = [effective_architecture(v) for v in value]
        elif field.hint == FieldHint.architecture and name != "add_linear_biases":
            out[name] = _serialize(value, None, True, True)
    return out


# keys of a Hugging Face `config.json` that describe the file or the runtime, not the architecture
_BOOKKEEPING_KEYS = frozenset({
    "architectures", "model_type", "torch_dtype", "dtype", "transformers_version", "_name_or_path", "auto_map", "use_cache",
    "bos_token_id", "eos_token_id", "pad_token_id", "initializer_range", "pretraining_tp", "id2label", "label2id", "return_dict",
    "output_attentions", "output_hidden_states", "is_decoder", "is_encoder_decoder", "chunk_size_feed_forward", "problem_type",
    "tokenizer_class", "torchscript", "use_bfloat16", "tf_legacy_loss", "pruned_heads", "add_cross_attention", "tie_encoder_decoder",
    "cross_attention_hidden_size", "finetuning_task", "task_specific_params", "prefix", "sep_token_id", "decoder_start_token_id",
    "layer_types", "max_window_layers",
})


class HuggingfaceStateDictCheckpointHandler(ExternalStateDictCheckpointHandler):
    """Hugging Face layout: `config.json`, `model_{i}.safetensors`, `model.safetensors.index.json`.

    Two coverage checks surround the format's hand-written `export_config` / `import_config` (the declarative converters of
    `fast_llm/engine/checkpoint/external.py:83-540` enforce the same two properties field by field):

      * export: the exported dictionary is imported again and every *architecture* field of the result must equal the
        model's - a field the format has no place for fails the export instead of being dropped (`check_export_coverage`);
      * import: every key of the external `config.json` must have been read by the converter or be listed as
        bookkeeping / explicitly ignored (`ignored_import_keys`); the rest is reported (`check_import_coverage`), and
        raises under `strict_import`.
    """

    ignored_import_keys: typing.ClassVar[frozenset[str]] = frozenset()
    strict_import: typing.ClassVar[bool] = False

    @classmethod
    def check_import_coverage(cls, hf_config: dict) -> tuple[dict, list[str]]:
        """(imported base-model dictionary, external keys nobody claimed)."""
        tracked = TrackedConfig(hf_config)
        base_model = cls.import_config(tracked)
        ignored = _BOOKKEEPING_KEYS | cls.ignored_import_keys
        # nested configurations (`text_config`, `vision_config`) carry the same bookkeeping keys as the top level
        unclaimed = [key for key in tracked.unread()
                     if key.split(".")[0] not in ignored and key not in ignored and key.split(".")[-1] not in _BOOKKEEPING_KEYS]
        return _plain(base_model), unclaimed

    @classmethod
    def check_export_coverage(cls, base_model_config, hf_config: dict) -> list[str]:
        """Architecture fields of `base_model_config` that do not survive export followed by import."""
        from fast_llm_b200.utils import compare_nested

        model_class = cls.get_model_config_class()
        again = model_class.from_dict({"base_model": cls.import_config(json.loads(json.dumps(_jsonable(hf_config))))}).base_model
        again.validate()
        return compare_nested(effective_architecture(base_model_config), effective_architecture(again))

    @classmethod
    def save_metadata(cls, config: CheckpointSaveMetadataConfig, metadata: CheckpointMetadata, index: dict | None = None) -> None:
        path = pathlib.Path(config.path)
        path.mkdir(parents=True, exist_ok=True)
        hf_config = cls.export_config(metadata.config.base_model)
        lost = cls.check_export_coverage(metadata.config.base_model, hf_config)
        if lost:
            raise ValueError(f"Format {cls.format.name!r} cannot represent this model; architecture fields that would be lost or changed:\n  "
                             + "\n  ".join(lost[:40]))
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
        base_model, unclaimed = cls.check_import_coverage(hf_config)
        if unclaimed:
            message = f"Format {cls.format.name!r}: fields of config.json that no converter claimed: {unclaimed}"
            if cls.strict_import:
                raise ValueError(message)
            logger.warning(message)
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


def _plain(obj):
    """Nested `TrackedConfig`s back to plain dictionaries."""
    if isinstance(obj, dict):
        return {k: _plain(v) for k, v in dict.items(obj)}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_plain(v) for v in obj)
    return obj


def _jsonable(obj):
    if isinstance(obj, dict):
        return {str(k): _jsonable(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_jsonable(v) for v in obj]
    if isinstance(obj, (int, float, str, bool)) or obj is None:
        return obj
    return str(obj)
