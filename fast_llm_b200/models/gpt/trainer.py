"""GPT trainer registration (parity: `fast_llm/models/gpt/config.py:106-130`, `trainer.py`)."""

from fast_llm_b200.config import Field, FieldHint, config_class
from fast_llm_b200.config.runnable import RunnableConfig
from fast_llm_b200.data.config import GPTDataConfig
from fast_llm_b200.engine.training.config import TrainerConfig
from fast_llm_b200.engine.training.trainer import Trainer
from fast_llm_b200.models.gpt.config import PretrainedGPTModelConfig


@config_class(dynamic_type={RunnableConfig: "train_gpt", TrainerConfig: "gpt"})
class GPTTrainerConfig(PretrainedGPTModelConfig, TrainerConfig):
    _abstract = False
    data: GPTDataConfig = Field(desc="Data.", hint=FieldHint.core)
    reference_models: dict[str, PretrainedGPTModelConfig] = Field(default_factory=dict, hint=FieldHint.feature)

    @classmethod
    def get_trainer_class(cls):
        return GPTTrainer


class GPTTrainer(Trainer):
    config_class = GPTTrainerConfig
