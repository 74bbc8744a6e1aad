"""Checkpoint formats and save / load configuration (parity: `fast_llm/engine/checkpoint/config.py:24-264`)."""

import abc
import enum
import logging
import pathlib
import typing

import yaml

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class, skip_valid_if_none
from fast_llm_b200.utils import Assert
from fast_llm_b200.utils.data_type import DataType

logger = logging.getLogger(__name__)

# Marker written once a checkpoint / export directory is complete.
CHECKPOINT_VERSION = "0.4.0"
KNOWN_CHECKPOINT_VERSIONS = ("0.1", "0.2", "0.3.0", "0.4.0")


class CheckpointFormat(abc.ABC):
    """A named on-disk format; subclasses bind a handler class."""

    name: typing.ClassVar[str]
    support_optimizer: typing.ClassVar[bool] = True
    support_saving: typing.ClassVar[bool] = True
    support_loading: typing.ClassVar[bool] = True
    enforce_architecture_match: typing.ClassVar[bool] = False

    @classmethod
    def get_handler_class(cls):
        raise NotImplementedError

    @classmethod
    def __fast_llm_serialize__(cls) -> str:
        return cls.name

    _registry: typing.ClassVar[dict[str, type["CheckpointFormat"]]] = {}

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        if "name" in cls.__dict__:
            CheckpointFormat._registry[cls.name] = cls

    @classmethod
    def __fast_llm_from_name__(cls, name: str):
        if name not in CheckpointFormat._registry:
            # formats of model families register on import
            import fast_llm_b200.models.auto  # noqa: F401
        if name not in CheckpointFormat._registry:
            raise KeyError(f"Unknown checkpoint format {name!r} (known: {sorted(CheckpointFormat._registry)})")
        return CheckpointFormat._registry[name]


class DistributedCheckpointFormat(CheckpointFormat):
    name: typing.ClassVar[str] = "distributed"
    enforce_architecture_match: typing.ClassVar[bool] = True

    @classmethod
    def get_handler_class(cls):
        from fast_llm_b200.engine.checkpoint.distributed import DistributedCheckpointHandler

        return DistributedCheckpointHandler


class FastLLMCheckpointFormat(CheckpointFormat):
    name: typing.ClassVar[str] = "fast_llm"

    @classmethod
    def get_handler_class(cls):
        from fast_llm_b200.engine.checkpoint.state_dict import FastLLMCheckpointHandler

        return FastLLMCheckpointHandler


class ModelConfigType(str, enum.Enum):
    none = "none"
    architecture = "architecture"
    model = "model"
    fast_llm = "fast_llm"

    @property
    def load_architecture(self) -> bool:
        return self != ModelConfigType.none

    @property
    def load_base_model(self) -> bool:
        return self in (ModelConfigType.model, ModelConfigType.fast_llm)

    @property
    def load_fast_llm(self) -> bool:
        return self == ModelConfigType.fast_llm


@config_class()
class CheckpointConfigBase(Config):
    _abstract = True
    format: type[CheckpointFormat] = Field(default=FastLLMCheckpointFormat, desc="Checkpoint format.", hint=FieldHint.core)

    def setup(self, model_config) -> None:
        """Resolve a format given by name against the formats the model class supports."""
        fmt = model_config.get_checkpoint_format(self.format)
        object.__setattr__(self, "format", fmt)


@config_class()
class CheckpointStateConfigBase(CheckpointConfigBase):
    _abstract = True
    model_weights: bool = Field(default=True, desc="Save / load the weights.", hint=FieldHint.feature)
    optimizer_state: bool = Field(default=None, desc="Save / load the optimizer state (default depends on the use).", hint=FieldHint.feature)

    def _validate(self):
        if self.optimizer_state is None:
            self.optimizer_state = False
        super()._validate()


@config_class()
class CheckpointSaveConfigBase(CheckpointConfigBase):
    _abstract = True
    parameters_per_file: int = Field(default=2**32, desc="Soft limit of parameters per safetensors file.", hint=FieldHint.feature, valid=check_field(Assert.geq, 2**20))
    data_type: DataType | None = Field(default=None, desc="Cast weights to this dtype when saving.", hint=FieldHint.feature)


@config_class()
class CheckpointStateSaveConfigBase(CheckpointSaveConfigBase, CheckpointStateConfigBase):
    _abstract = False


@config_class()
class CheckpointPathConfigBase(CheckpointConfigBase):
    _abstract = True
    path: pathlib.Path | None = Field(default=None, desc="Checkpoint directory.", hint=FieldHint.core)
    timeout: float | None = Field(default=None, desc="Timeout of the surrounding barriers (s).", hint=FieldHint.optional, valid=skip_valid_if_none(check_field(Assert.gt, 0)))


@config_class()
class CheckpointSaveMetadataConfig(CheckpointPathConfigBase):
    _abstract = False


@config_class()
class CheckpointSaveConfig(CheckpointSaveMetadataConfig, CheckpointStateSaveConfigBase):
    _abstract = False


@config_class()
class CheckpointLoadMetadataConfig(CheckpointPathConfigBase):
    _abstract = False
    load_config: ModelConfigType = Field(default=ModelConfigType.model, desc="How much of the saved config to adopt.", hint=FieldHint.core)


@config_class()
class CheckpointLoadConfig(CheckpointLoadMetadataConfig, CheckpointStateConfigBase):
    _abstract = False


class CheckpointHandler(abc.ABC):
    format: typing.ClassVar[type[CheckpointFormat]]

    def __init__(self, model):
        self._model = model

    @classmethod
    @abc.abstractmethod
    def save_metadata(cls, config: CheckpointSaveMetadataConfig, metadata) -> None:
        pass

    @classmethod
    def load_metadata(cls, config: CheckpointLoadMetadataConfig):
        updates = {}
        metadata = cls._load_metadata(config)
        if not config.load_config.load_fast_llm:
            updates[("config", "multi_stage")] = {}
            updates[("config", "distributed")] = {}
        if not config.load_config.load_architecture:
            updates[("config", "base_model")] = {}
        elif not config.load_config.load_base_model:
            from fast_llm_b200.engine.base_model import architecture_dict

            updates[("config", "base_model")] = architecture_dict(metadata.config.base_model)
        if updates:
            metadata = metadata.to_copy(updates)
        return metadata

    @classmethod
    @abc.abstractmethod
    def _load_metadata(cls, config: CheckpointLoadMetadataConfig):
        pass

    @abc.abstractmethod
    def save(self, config: CheckpointSaveConfig, metadata) -> None:
        pass

    @abc.abstractmethod
    def load(self, config: CheckpointLoadConfig) -> dict | None:
        pass

    def get_shard_names(self, config: CheckpointStateConfigBase) -> tuple[str, ...]:
        return self._model.get_shard_names(config)

    @property
    def _num_shards(self) -> int:
        return len(self._model.state_shard_names)
