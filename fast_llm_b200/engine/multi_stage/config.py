"""Configuration of staged models: stage debugging knobs, ZeRO / buffer counts, model + pretrained wrappers,
checkpoint metadata.  Parity: `fast_llm/engine/multi_stage/config.py:45-381`.
"""

import enum
import logging
import typing

from fast_llm_b200 import __version__
from fast_llm_b200.config import Config, Field, FieldHint, NoAutoValidate, UpdateType, ValidationError, check_field, config_class, skip_valid_if_none
from fast_llm_b200.engine.base_model import BaseModelConfig
from fast_llm_b200.engine.checkpoint.config import (
    CheckpointFormat,
    CheckpointLoadConfig,
    CheckpointLoadMetadataConfig,
    DistributedCheckpointFormat,
    FastLLMCheckpointFormat,
)
from fast_llm_b200.parallel.topology import DistributedConfig
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)

SHARD_PAD_TO_MULTIPLE = 32


class StageMode(str, enum.Enum):
    training = "training"  # weights, gradients, optimizer state
    inference = "inference"  # weights and buffers, forward only
    weights = "weights"  # weight shards only (conversion)
    off_device = "off_device"  # no memory at all (meta only)

    @property
    def support_forward(self) -> bool:
        return self in (StageMode.training, StageMode.inference)

    @property
    def support_backward(self) -> bool:
        return self == StageMode.training

    @property
    def support_training(self) -> bool:
        return self == StageMode.training

    @property
    def on_device(self) -> bool:
        return self != StageMode.off_device


@config_class()
class StageConfig(Config):
    full_precision_gradients: bool = Field(default=True, desc="Accumulate gradients in the optimization dtype.", hint=FieldHint.optional)
    store_frozen_weights_in_optimization_precision: bool = Field(default=True, desc="Keep fp32 shards of frozen weights.", hint=FieldHint.optional)
    debug_layer_outputs: int = Field(default=0, desc="Log layer outputs at this verbosity.", hint=FieldHint.logging, valid=check_field(Assert.geq, 0))
    debug_layer_gradients: int = Field(default=0, desc="Log layer output gradients.", hint=FieldHint.logging, valid=check_field(Assert.geq, 0))
    debug_param_init: int = Field(default=0, desc="Log parameters after initialisation.", hint=FieldHint.logging, valid=check_field(Assert.geq, 0))
    debug_param_gradients: int = Field(default=0, desc="Log parameter gradients after reduction.", hint=FieldHint.logging, valid=check_field(Assert.geq, 0))
    debug_all_param_gradients: int = Field(default=0, desc="Log every parameter gradient contribution.", hint=FieldHint.logging, valid=check_field(Assert.geq, 0))
    debug_param_update: int = Field(default=0, desc="Log parameters after the optimizer step.", hint=FieldHint.logging, valid=check_field(Assert.geq, 0))
    debug_global_tensors: bool = Field(default=True, desc="Reconstruct global tensors for the debug logs.", hint=FieldHint.logging)
    debug_activation_memory: bool = Field(default=False, desc="Log memory after each layer.", hint=FieldHint.logging)
    debug_tensor_parallel: bool = Field(default=False, desc="Check that replicated tensors match across the tensor group.", hint=FieldHint.logging)


@config_class()
class MultiStageConfig(StageConfig):
    layers_per_stage: float = Field(default=1.0, desc="Layers per stage.", hint=FieldHint.performance, valid=check_field(Assert.gt, 0))
    stages_per_pipeline_stage: int = Field(default=1, desc="Consecutive stages per pipeline rank.", hint=FieldHint.wip, valid=check_field(Assert.eq, 1))
    num_weight_buffers: int | None = Field(default=None, desc="Shared weight buffers (default from zero_stage).", hint=FieldHint.expert, valid=skip_valid_if_none(check_field(Assert.geq, 1)))
    num_grad_buffers: int | None = Field(default=None, desc="Shared gradient buffers (default from zero_stage).", hint=FieldHint.expert, valid=skip_valid_if_none(check_field(Assert.geq, 1)))
    zero_stage: int | None = Field(default=None, desc="ZeRO stage 1, 2 or 3.", hint=FieldHint.performance)
    fused_collectives: bool = Field(default=True, desc="Keep ZeRO weight/gradient buffers in NVLink symmetric memory and run the gradient reduction and the optimizer update as kernels fused with their collectives (GPU, data_parallel > 1, ZeRO-1/2 with per-stage buffers).", hint=FieldHint.performance)
    pipeline_delay: float = Field(default=0.0, desc="Estimated pipeline communication delay in units of a stage's compute time.", hint=FieldHint.expert, valid=check_field(Assert.geq, 0))

    def _validate(self):
        super()._validate()
        if self.zero_stage is not None:
            Assert.in_range_incl(self.zero_stage, 1, 3)
            if self.zero_stage >= 2:
                self.num_grad_buffers = 2 if self.num_grad_buffers is None else self.num_grad_buffers
            if self.zero_stage >= 3:
                self.num_weight_buffers = 2 if self.num_weight_buffers is None else self.num_weight_buffers


@config_class(registry=True)
class FastLLMModelConfig(Config):
    _abstract = True
    model_name: typing.ClassVar[str]
    base_model: BaseModelConfig = Field(desc="Architecture.", hint=FieldHint.core)
    multi_stage: MultiStageConfig = Field(desc="Staging / ZeRO.", hint=FieldHint.core)
    distributed: DistributedConfig = Field(desc="Parallel layout.", hint=FieldHint.core)

    @classmethod
    def __fast_llm_serialize__(cls) -> str:
        return cls.model_name

    @classmethod
    def __fast_llm_from_name__(cls, name: str):
        import fast_llm_b200.models.auto  # noqa: F401

        return FastLLMModelConfig.get_subclass(name)

    @classmethod
    def get_checkpoint_formats(cls) -> tuple[type[CheckpointFormat], ...]:
        return (DistributedCheckpointFormat, FastLLMCheckpointFormat)

    @classmethod
    def get_checkpoint_format(cls, fmt: "type[CheckpointFormat] | str") -> type[CheckpointFormat]:
        name = fmt if isinstance(fmt, str) else fmt.name
        for candidate in cls.get_checkpoint_formats():
            if candidate.name == name:
                return candidate
        raise ValueError(f"Checkpoint format {name} not supported for model {cls.model_name} "
                         f"(supported: {[f.name for f in cls.get_checkpoint_formats()]})")

    @classmethod
    def get_checkpoint_handler_class(cls, fmt):
        return cls.get_checkpoint_format(fmt).get_handler_class()

    @classmethod
    def get_model_class(cls):
        raise NotImplementedError

    @classmethod
    def get_base_model_config_class(cls):
        return cls._type_hints()["base_model"]

    @classmethod
    def from_pretrained(cls, pretrained: CheckpointLoadMetadataConfig, *updates):
        return cls.from_metadata(cls.load_metadata(pretrained), pretrained, *updates)

    @classmethod
    def from_metadata(cls, metadata: "CheckpointMetadata", pretrained: CheckpointLoadMetadataConfig, *updates, update_type=UpdateType.update):
        return cls.from_dict(metadata.config, *updates, update_type=update_type)

    @classmethod
    def load_metadata(cls, config: CheckpointLoadMetadataConfig) -> "CheckpointMetadata":
        config.setup(cls)
        fmt = config.format
        metadata = fmt.get_handler_class().load_metadata(config)
        Assert.eq(metadata.model.model_name if isinstance(metadata.model, type) else metadata.model, cls.model_name)
        return metadata

    def to_metadata(self, config, **kwargs) -> "CheckpointMetadata":
        return CheckpointMetadata(fast_llm_version=__version__, model=type(self), format=config.format, config=self, **kwargs)


@config_class()
class PretrainedFastLLMModelConfig(Config):
    _abstract = True
    model: FastLLMModelConfig = Field(desc="Model.", hint=FieldHint.core)
    pretrained: CheckpointLoadConfig = Field(desc="Checkpoint to start from.", hint=FieldHint.feature)

    def _validate(self):
        self.pretrained.validate()
        self.pretrained.setup(type(self.model))
        if self.pretrained.path is not None:
            # Start from the saved config, then apply what the user set explicitly on top of it.
            self.model = type(self.model).from_pretrained(self.pretrained, self.model)
        self._setup()
        super()._validate()

    def _setup(self):
        pass


@config_class()
class CheckpointMetadata(Config):
    fast_llm_version: str = Field(default=__version__, desc="Version that wrote the checkpoint.", hint=FieldHint.core)
    model: type[FastLLMModelConfig] = Field(default=None, desc="Model class (by name).", hint=FieldHint.core)
    format: type[CheckpointFormat] = Field(default=None, desc="Format of the checkpoint.", hint=FieldHint.core)
    config: FastLLMModelConfig = Field(desc="Model config.", hint=FieldHint.core)
    shards: list[str] = Field(default_factory=list, desc="Names of the state shards saved.", hint=FieldHint.optional)
    metadata: dict = Field(default_factory=dict, desc="Free-form metadata (training state).", hint=FieldHint.optional)

    def _validate(self):
        if isinstance(self.fast_llm_version, str) is False:
            self.fast_llm_version = str(self.fast_llm_version)
        if isinstance(self.config, dict) and self.model is not None:
            model = self.model if isinstance(self.model, type) else FastLLMModelConfig.__fast_llm_from_name__(self.model)
            self.config = model.from_dict(self.config)
        super()._validate()

    @classmethod
    def _from_dict(cls, default, strict=True, flat=False):
        default = dict(default)
        model = default.get("model")
        if isinstance(model, str):
            model = FastLLMModelConfig.__fast_llm_from_name__(model)
            default["model"] = model
        cfg = default.get("config")
        if isinstance(cfg, dict) and isinstance(model, type):
            default["config"] = model.from_dict(cfg)
        return super()._from_dict(default, strict=strict, flat=flat)
