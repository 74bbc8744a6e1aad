"""Multimodal (vision + language) model configuration: a GPT model with a vision encoder in front.

Parity: `fast_llm/models/multimodal/config.py:21-84`, `fast_llm/layers/vision/config.py:95-112`.
"""

import typing

from fast_llm_b200.config import Field, FieldHint, config_class
from fast_llm_b200.engine.multi_stage.config import FastLLMModelConfig, PretrainedFastLLMModelConfig
from fast_llm_b200.engine.training.config import TrainerConfig
from fast_llm_b200.layers.vision import VisionEncoderConfig
from fast_llm_b200.config.runnable import RunnableConfig
from fast_llm_b200.models.gpt.config import GPTBaseModelConfig, GPTModelConfig, PretrainedGPTModelConfig
from fast_llm_b200.models.gpt.trainer import GPTTrainerConfig


@config_class()
class MultiModalBaseModelConfig(GPTBaseModelConfig):
    _abstract = False
    vision_encoder: VisionEncoderConfig = Field(desc="Vision encoder.", hint=FieldHint.architecture)
    image_token_index: int | None = Field(default=None, desc="Placeholder token of image patches (used by checkpoint conversion only).", hint=FieldHint.optional)

    def get_base_model(self, distributed_config):
        from fast_llm_b200.models.multimodal.model import MultiModalBaseModel

        return MultiModalBaseModel(self, distributed_config)


@config_class(dynamic_type={FastLLMModelConfig: "multimodal"})
class MultiModalModelConfig(GPTModelConfig):
    _abstract = False
    model_name: typing.ClassVar[str] = "multimodal"
    base_model: MultiModalBaseModelConfig = Field(desc="Architecture.", hint=FieldHint.core)

    @classmethod
    def get_checkpoint_formats(cls):
        from fast_llm_b200.models.multimodal.conversion import MULTIMODAL_CHECKPOINT_FORMATS

        return FastLLMModelConfig.get_checkpoint_formats.__func__(cls) + MULTIMODAL_CHECKPOINT_FORMATS

    @classmethod
    def get_model_class(cls):
        from fast_llm_b200.models.multimodal.model import MultiModalModel

        return MultiModalModel


@config_class()
class PretrainedMultiModalModelConfig(PretrainedGPTModelConfig):
    _abstract = False
    model: MultiModalModelConfig = Field(desc="Model.", hint=FieldHint.core)


@config_class(dynamic_type={RunnableConfig: "train_multimodal", TrainerConfig: "multimodal"})
class MultiModalTrainerConfig(PretrainedMultiModalModelConfig, GPTTrainerConfig):
    _abstract = False

    @classmethod
    def get_trainer_class(cls):
        from fast_llm_b200.models.multimodal.trainer import MultiModalTrainer

        return MultiModalTrainer
