"""GPT model, trainer and checkpoint-format registration (parity: `fast_llm/models/gpt/config.py:38-130`)."""

import typing

from fast_llm_b200.config import Field, FieldHint, FieldUpdate, config_class
from fast_llm_b200.engine.base_model import BaseModelConfig
from fast_llm_b200.engine.multi_stage.config import FastLLMModelConfig, PretrainedFastLLMModelConfig
from fast_llm_b200.layers.language_model import LanguageModelConfig
from fast_llm_b200.layers.peft import PeftConfig


@config_class()
class GPTBaseModelConfig(LanguageModelConfig, BaseModelConfig):
    _abstract = False
    peft: PeftConfig = Field(desc="Parameter-efficient fine-tuning method.", hint=FieldHint.architecture)
    use_megatron_initialization: bool = Field(default=False, desc="Reproduce Megatron-LM's initialisation order (for parity tests).", hint=FieldHint.testing)

    def get_base_model(self, distributed_config):
        from fast_llm_b200.models.gpt.model import GPTBaseModel

        return GPTBaseModel(self, distributed_config)


@config_class(dynamic_type={FastLLMModelConfig: "gpt"})
class GPTModelConfig(FastLLMModelConfig):
    _abstract = False
    model_name: typing.ClassVar[str] = "gpt"
    base_model: GPTBaseModelConfig = Field(desc="Architecture.", hint=FieldHint.core)

    @classmethod
    def get_checkpoint_formats(cls):
        from fast_llm_b200.models.gpt.conversion import GPT_CHECKPOINT_FORMATS

        return super().get_checkpoint_formats() + GPT_CHECKPOINT_FORMATS

    @classmethod
    def get_model_class(cls):
        from fast_llm_b200.models.gpt.model import GPTModel

        return GPTModel

    @classmethod
    def get_huggingface_model_for_causal_lm_class(cls):
        from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

        return HuggingfaceGPTModelForCausalLM


@config_class()
class PretrainedGPTModelConfig(PretrainedFastLLMModelConfig):
    _abstract = False
    model: GPTModelConfig = Field(desc="Model.", hint=FieldHint.core)
