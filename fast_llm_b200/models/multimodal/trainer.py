"""Multimodal trainer (parity: `fast_llm/models/multimodal/trainer.py`)."""

from fast_llm_b200.models.gpt.trainer import GPTTrainer
from fast_llm_b200.models.multimodal.config import MultiModalTrainerConfig


class MultiModalTrainer(GPTTrainer):
    config_class = MultiModalTrainerConfig
