"""Configuration of Diffusion Llama: a masked-diffusion language model on a Llama decoder.

Stand-alone file: it is copied next to exported checkpoints and loaded by `transformers` with `trust_remote_code`.
"""

from transformers.models.llama.configuration_llama import LlamaConfig


class DiffusionLlamaConfig(LlamaConfig):
    model_type = "diffusion_llama"

    def __init__(self, mask_token_id: int | None = None, bidirectional: bool = True, **kwargs):
        super().__init__(**kwargs)
        # token that stands for "not generated yet" during sampling (default: the last id of the vocabulary)
        self.mask_token_id = self.vocab_size - 1 if mask_token_id is None else mask_token_id
        # every position attends to every other one; False gives the causal decoder the weights were trained as
        self.bidirectional = bidirectional
