"""Configuration of MTP-Llama: a Llama model with extra multi-token-prediction heads.

Stand-alone file: it is copied next to exported checkpoints and loaded by `transformers` with `trust_remote_code`.
"""

from transformers.models.llama.configuration_llama import LlamaConfig


class MTPLlamaConfig(LlamaConfig):
    model_type = "mtp_llama"

    def __init__(self, prediction_heads: int = 1, **kwargs):
        super().__init__(**kwargs)
        self.prediction_heads = prediction_heads
