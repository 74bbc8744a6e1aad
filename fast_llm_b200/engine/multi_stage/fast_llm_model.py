"""MultiStageModel plus checkpoint save / load and construction from pretrained checkpoints.

Parity: `fast_llm/engine/multi_stage/fast_llm_model.py:21-118`.
"""

import logging
import typing

from fast_llm_b200.config import UpdateType
from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
from fast_llm_b200.engine.multi_stage.config import FastLLMModelConfig, StageMode
from fast_llm_b200.engine.multi_stage.multi_stage import MultiStageModel
from fast_llm_b200.parallel.distributed import Distributed

logger = logging.getLogger(__name__)


class FastLLMModel(MultiStageModel):
    config_class: typing.ClassVar[type[FastLLMModelConfig]] = FastLLMModelConfig
    _is_loaded: bool = False

    def save_checkpoint(self, config: CheckpointSaveConfig, extra_metadata: dict | None = None) -> None:
        config.validate()
        config.setup(type(self._config))
        handler = config.format.get_handler_class()(self)
        metadata = self._config.to_metadata(config, shards=list(handler.get_shard_names(config)), metadata=extra_metadata or {})
        handler.save(config, metadata)

    def iter_exported_tensors(self, config):
        """Yield (shard name, exported tensor name, tensor) in the checkpoint format of `config` without touching disk
        (used to stream weights to inference workers).  Collective: every rank must iterate."""
        config.validate()
        config.setup(type(self._config))
        handler = config.format.get_handler_class()(self)
        pending: dict = {}
        data_type = config.data_type.torch if getattr(config, "data_type", None) is not None else None
        for parameter_name, shard_name, tensor in self.get_state_tensor_iterator(handler.get_shard_names(config), data_type):
            for name, converted in handler._export_tensors(parameter_name, shard_name, tensor, pending).items():
                yield shard_name, name, converted

    def load_checkpoint(self, config: CheckpointLoadConfig) -> dict | None:
        config.validate()
        config.setup(type(self._config))
        handler_class = config.format.get_handler_class()
        if hasattr(handler_class, "resolve"):  # `auto` formats pick the concrete handler from the files
            handler_class = handler_class.resolve(config.path)
        handler = handler_class(self)
        metadata = handler.load(config)
        self._finalize_load(reset_optimizer=not config.optimizer_state)
        return metadata

    @classmethod
    def from_pretrained(cls, pretrained_config: CheckpointLoadConfig, *updates, optimizer_state_names: tuple[str, ...] | None = None,
                        setup: bool = True, mode: StageMode = StageMode.training, use_cpu: bool = False,
                        stage_filter: set | None = None, distributed: Distributed | None = None) -> typing.Self:
        import fast_llm_b200.models.auto  # noqa: F401  (fills the registries: mixers, formats, datasets; the command line does the same)

        pretrained_config.validate()
        pretrained_config.setup(cls.config_class)
        metadata = cls.config_class.load_metadata(pretrained_config)
        config = cls.config_class.from_dict(metadata.config, *updates, update_type=UpdateType.update)
        if mode.support_training:
            if optimizer_state_names is None:
                optimizer_state_names = tuple(n for n in metadata.shards if n != "weights") if pretrained_config.optimizer_state else ()
        else:
            optimizer_state_names = ()
        model = cls(config, optimizer_state_names=tuple(optimizer_state_names), stage_filter=stage_filter)
        if setup:
            model.setup(distributed or Distributed(config.distributed, use_cpu=use_cpu), mode=mode)
            if mode.on_device:
                if pretrained_config.model_weights:
                    model.load_checkpoint(pretrained_config)
                else:
                    model.initialize_weights()
        return model

    def initialize_weights(self, timeout: float | None = None) -> None:
        assert self._is_setup
        super().initialize_weights()
        self._finalize_load(reset_optimizer=True)

    def _finalize_load(self, reset_optimizer: bool = True) -> None:
        if reset_optimizer:
            for name in self._state_shard_names[1:]:
                self._shards[name].zero_()
        if self._mode.support_forward:
            self.invalidate_buffers()
        self._is_loaded = True
