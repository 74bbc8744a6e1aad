"""GPT base model: embeddings -> decoder blocks -> head(s); batch preprocessing; tied embedding/output weights.

Parity: `fast_llm/models/gpt/model.py:30-110`.
"""

import logging

import torch

from fast_llm_b200.engine.base_model import BaseModel, Layer
from fast_llm_b200.engine.multi_stage.fast_llm_model import FastLLMModel
from fast_llm_b200.layers.kwargs import LanguageModelKwargs
from fast_llm_b200.parallel.topology import PhaseType
from fast_llm_b200.tensor import TensorDim

logger = logging.getLogger(__name__)


class GPTBaseModel(BaseModel):
    def __init__(self, config, distributed_config):
        super().__init__(config, distributed_config)
        hidden_dim = TensorDim("hidden", config.hidden_size)
        self._hidden_dim = hidden_dim
        peft = config.peft if type(config.peft).__name__ != "NoPeftConfig" else None
        self.embeddings = config.embeddings.get_layer(distributed_config, hidden_dim, lr_scale=config.lr_scale, peft=peft)
        heads = config.head.prediction_heads
        blocks = config.decoder.get_layers(distributed_config, hidden_dim, lr_scale=config.lr_scale, peft=peft,
                                           return_last_layer_input=heads > 1)
        self._decoder_layers = blocks
        for i, block in enumerate(blocks):
            setattr(self, f"decoder_{i}", block)
        coefficients = config.head.prediction_loss_coefficient or [1.0] * heads
        self.head = config.head.get_layer(distributed_config, config.embeddings, hidden_dim, lr_scale=config.lr_scale, peft=peft,
                                          prediction_distance=1, loss_coefficient=coefficients[0])
        self._extra_heads = []
        for d in range(2, heads + 1):
            # each extra prediction head = one more decoder block (same config as the last) + a head sharing the weights
            block_config = config.decoder.block_configs()[-1]
            block = block_config.get_layer(distributed_config, hidden_dim, lr_scale=config.lr_scale, peft=peft, return_input=d < heads)
            head = config.head.get_layer(distributed_config, config.embeddings, hidden_dim, lr_scale=config.lr_scale, peft=peft,
                                         prediction_distance=d, loss_coefficient=coefficients[d - 1])
            setattr(self, f"mtp_block_{d}", block)
            setattr(self, f"mtp_head_{d}", head)
            self._extra_heads.append((block, head))
        self.set_names()
        if config.use_megatron_initialization:
            from fast_llm_b200.models.gpt.megatron import get_init_megatron

            block_configs = config.decoder.block_configs()
            for layer, block_config in zip(self._decoder_layers, block_configs):
                for _, meta in layer.named_parameter_metas():
                    meta.init_override = get_init_megatron(meta, block_config, config.hidden_size)
            for _, meta in self.embeddings.named_parameter_metas():
                meta.init_override = get_init_megatron(meta, block_configs[0], config.hidden_size)

    def set_names(self, prefix: str = "") -> None:
        # Parameter names follow the reference layout: embeddings.*, decoder.{i}.*, head.*
        self.module_name = ""
        self.embeddings.set_names("embeddings.")
        for i, block in enumerate(self._decoder_layers):
            block.set_names(f"decoder.{i}.")
        self.head.set_names("head.")
        for d, (block, head) in enumerate(self._extra_heads, start=2):
            block.set_names(f"multi_token_prediction.blocks.{d - 2}.")
            head.set_names(f"multi_token_prediction.heads.{d - 2}.")

    def get_layers(self) -> list[Layer]:
        layers = [self.embeddings, *self._decoder_layers, self.head]
        if self._extra_heads:
            # interleave: the trunk's last block returns (input, output); head 1 reads output, block 2 reads input...
            layers = [self.embeddings, *self._decoder_layers]
            from fast_llm_b200.layers.mtp import MultiTokenPredictionStage

            layers.append(MultiTokenPredictionStage(self.head, self._extra_heads, self._distributed_config))
        return layers

    def get_tied_parameters(self):
        tied = {}
        if self._config.tied_embedding_weight:
            metas = [self.embeddings.parameter_meta("word_embeddings_weight"), self.head.parameter_meta("output_weights")]
            metas += [head.parameter_meta("output_weights") for _, head in self._extra_heads]
            tied["word_embeddings_weight"] = tuple(metas)
        elif self._extra_heads:
            tied["output_weights"] = (self.head.parameter_meta("output_weights"), *(h.parameter_meta("output_weights") for _, h in self._extra_heads))
        return tied

    def get_preprocessing_config(self, phase: PhaseType) -> dict:
        out = {"phase": phase, "predicted_tokens": self._config.head.prediction_heads, "vocab_size": self._config.embeddings.vocab_size}
        for layer in self.get_layers():
            out.update(layer.get_preprocessing_config(phase))
        return out

    def preprocess_batch(self, model_inputs, *, phase: PhaseType, iteration: int, metrics: dict | None = None, device=None):
        """model_inputs: list of `LanguageModelInput` (one per micro-sequence). Returns [(tokens, kwargs), ...]."""
        device = device or (self._distributed.device if self._distributed is not None else "cpu")
        out = []
        for model_input in model_inputs:
            kwargs = model_input.to_kwargs(device)
            kwargs[LanguageModelKwargs.phase] = phase
            kwargs[LanguageModelKwargs.iteration] = iteration
            kwargs["training"] = phase.is_training
            for name, runner in self._reference_models.items():
                ref_kwargs = dict(kwargs)
                ref_kwargs.pop(LanguageModelKwargs.labels, None)
                ref_kwargs["return_logits"] = True
                runner.forward_kwargs(kwargs[LanguageModelKwargs.token_ids], ref_kwargs, iteration=iteration)
                kwargs[f"{name}_logits"] = ref_kwargs["logits"]
                if LanguageModelKwargs.hidden_states in ref_kwargs:
                    kwargs[f"{name}_hidden_states"] = ref_kwargs[LanguageModelKwargs.hidden_states]
            for layer in self.get_layers():
                layer.preprocess(kwargs)
            out.append((kwargs[LanguageModelKwargs.token_ids], kwargs))
        return out


class GPTModel(FastLLMModel):
    from fast_llm_b200.models.gpt.config import GPTModelConfig as config_class  # noqa: E402

    base_model_class = GPTBaseModel
