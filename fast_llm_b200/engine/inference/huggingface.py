"""Hugging Face `generate()`-compatible wrapper around a staged model.

`HuggingfaceGPTModelForCausalLM(model)` behaves like a `transformers` causal LM: `forward(input_ids, attention_mask)`
returns `CausalLMOutputWithPast` with logits `[batch, sequence, vocab]`.  Every call packs the (left-padded) rows into one
variable-length token stream - padding becomes a document of its own that nothing attends to - runs the stages forward
and unpacks.  Decoders made of attention blocks generate with a key / value cache (`use_cache`, the default of `generate`):
the prompt runs once, every later step runs the new tokens against the cached keys and values of its row (the attention
layer's `past_key_values` / `presents` lists, the ones micro-sequences use in training).  Decoders with recurrent mixers
re-run the prompt for every token.

With tensor parallelism rank 0 of the tensor group acts as coordinator: it broadcasts the batch (or a stop signal) and
every other rank sits in `worker_forward()` executing the same forward passes.
Parity: `fast_llm/engine/inference/huggingface.py:31-272`, `fast_llm/models/gpt/huggingface.py:27-199`,
`fast_llm/engine/inference/config.py`.
"""

import logging
import os
import pathlib
import typing

import torch
import transformers
import transformers.modeling_outputs

from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, FastLLMCheckpointFormat
from fast_llm_b200.engine.inference.runner import InferenceRunner, KeyValueCache
from fast_llm_b200.engine.multi_stage.config import StageMode
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


class HuggingfaceModelConfig(transformers.PretrainedConfig):
    """`transformers` view of a model config; the full native config rides along as `fast_llm_config`."""

    model_type = "fast_llm"
    model_config_class: typing.ClassVar[type | None] = None

    @classmethod
    def from_fast_llm_config(cls, fast_llm_config, **kwargs) -> "HuggingfaceModelConfig":
        config = cls(**kwargs)
        base = fast_llm_config.base_model
        config.use_cache = False  # the wrapper turns it on when the decoder can keep a cache
        config.vocab_size = base.embeddings.vocab_size
        config.hidden_size = base.hidden_size
        config.num_hidden_layers = len(base.decoder.block_configs())
        config.tie_word_embeddings = base.tied_embedding_weight
        object.__setattr__(config, "fast_llm_config", fast_llm_config)
        return config

    def to_dict(self) -> dict:
        out = super().to_dict()
        native = out.pop("fast_llm_config", None) or self.__dict__.get("fast_llm_config")
        if native is not None and not isinstance(native, dict):
            native = native.to_dict()
        if native is not None:
            out["fast_llm_config"] = native
        return out

    def __deepcopy__(self, memo):
        # the wrapped config may hold process groups; share it instead of copying
        import copy

        clone = self.__class__.__new__(self.__class__)
        for key, value in self.__dict__.items():
            object.__setattr__(clone, key, value if key == "fast_llm_config" else copy.deepcopy(value, memo))
        return clone


class HuggingfacePreTrainedModel(transformers.PreTrainedModel, transformers.generation.utils.GenerationMixin):
    config_class = HuggingfaceModelConfig
    runner_class: typing.ClassVar[type[InferenceRunner]] = InferenceRunner
    model_class: typing.ClassVar[type | None] = None
    base_model_prefix = ""
    _supports_cache_class = False

    @classmethod
    def can_generate(cls) -> bool:
        return True

    @classmethod
    def _supports_default_dynamic_cache(cls) -> bool:
        return False  # `forward` makes its own `KeyValueCache`

    def __init__(self, fast_llm_model, config: HuggingfaceModelConfig | None = None, runner: InferenceRunner | None = None, **kwargs):
        if config is None:
            config = self.config_class.from_fast_llm_config(fast_llm_model.config)
        Assert.custom(lambda m: m.is_setup, fast_llm_model)
        super().__init__(config, **kwargs)
        if getattr(self, "generation_config", None) is None:
            self.generation_config = transformers.GenerationConfig.from_model_config(config)
        self._fast_llm_model = fast_llm_model
        self._inference_runner = runner or self.runner_class(fast_llm_model)
        self._inference_runner.setup()
        self._cache_supported = self._inference_runner.supports_key_value_cache()
        self._worker_cache: KeyValueCache | None = None  # tensor-parallel workers keep their own heads' cache here
        self.config.use_cache = self._cache_supported
        self.generation_config.use_cache = self._cache_supported
        distributed_config = fast_llm_model.distributed.config
        Assert.eq(distributed_config.pipeline_parallel, 1)
        Assert.eq(distributed_config.sequence_data_parallel, 1)
        self._tensor_group = fast_llm_model.distributed.tensor_group
        self._is_coordinator = distributed_config.tensor_rank == 0
        # transformers moves inputs to `self.device`, which it reads from the first parameter
        self._device_anchor = torch.nn.Parameter(torch.zeros(1, device=fast_llm_model.distributed.device), requires_grad=False)
        if fast_llm_model.config.multi_stage.zero_stage == 3:
            logger.warning("ZeRO stage 3 re-gathers the weights on every forward pass; generation will be slow.")

    # ---- construction
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: "str | os.PathLike | CheckpointLoadConfig", *updates,
                        mode: StageMode = StageMode.inference, use_cpu: bool = False, **kwargs) -> typing.Self:
        if not isinstance(pretrained_model_name_or_path, CheckpointLoadConfig):
            pretrained_model_name_or_path = CheckpointLoadConfig(path=pathlib.Path(pretrained_model_name_or_path), format=FastLLMCheckpointFormat)
        fast_llm_model = cls.model_class.from_pretrained(pretrained_model_name_or_path, *updates, setup=True, mode=mode, use_cpu=use_cpu)
        model = cls(fast_llm_model, **kwargs)
        model._apply_generation_token_ids(pretrained_model_name_or_path)
        return model

    def _apply_generation_token_ids(self, pretrained: CheckpointLoadConfig) -> None:
        """External checkpoints carry bos / eos / pad ids in their `config.json`; without them generation never stops."""
        import json

        path = pathlib.Path(pretrained.path) / "config.json"
        if not path.is_file():
            return
        source = json.loads(path.read_text())
        for key in ("bos_token_id", "eos_token_id", "pad_token_id"):
            if source.get(key) is not None:
                setattr(self.generation_config, key, source[key])

    def _init_weights(self, module) -> None:
        pass  # weights belong to the wrapped model

    @property
    def fast_llm_model(self):
        return self._fast_llm_model

    # ---- forward
    def forward(self, input_ids: torch.Tensor | None = None, attention_mask: torch.Tensor | None = None, position_ids=None,
                past_key_values=None, inputs_embeds=None, labels=None, use_cache=None, output_attentions=None,
                output_hidden_states=None, return_dict=None, coordinator_forward: bool = False, **kwargs):
        if inputs_embeds is not None or labels is not None or output_attentions:
            raise NotImplementedError("The wrapper supports token inputs and logits / hidden-state outputs only")
        if past_key_values is not None and not isinstance(past_key_values, KeyValueCache):
            raise NotImplementedError("`past_key_values` must be the cache an earlier call of this model returned")
        cache_mode = None
        if past_key_values is not None and past_key_values.length > 0:
            cache_mode = "continue"
        elif self._cache_supported and (self.config.use_cache if use_cache is None else use_cache):
            cache_mode = "new"
        if self._tensor_group is not None and self._is_coordinator:
            self._broadcast(("forward", input_ids.cpu(), None if attention_mask is None else attention_mask.cpu(), bool(output_hidden_states),
                             cache_mode))
        return self._inner_forward(input_ids, attention_mask, output_hidden_states, return_dict, cache_mode, past_key_values)

    def _inner_forward(self, input_ids, attention_mask, output_hidden_states, return_dict, cache_mode=None, cache: KeyValueCache | None = None):
        batch, length = input_ids.shape
        hidden_names = None
        if output_hidden_states:
            hidden_names = [layer.unwrap().module_name for layer in self._fast_llm_model.base_model.get_layers()
                            if layer.unwrap().module_name.startswith("decoder.")]
        if cache_mode is None:
            cache = None
            lengths = self._document_lengths(input_ids, attention_mask)
            logits, hidden = self._inference_runner.forward_tokens(input_ids.reshape(-1), lengths, output_hidden_states=hidden_names or [])
        else:
            if cache_mode == "new":  # the whole (left-padded) prompt
                cache = KeyValueCache(self._left_padding(input_ids, attention_mask))
                cache.on_reorder = self._reorder_workers
            Assert.eq(cache.rows, batch)
            logits, hidden = self._inference_runner.forward_rows(input_ids, cache, hidden_names or [])
        logits = logits.reshape(batch, length, -1)
        hidden_states = None
        if hidden_names:
            hidden_states = tuple(hidden[name].reshape(batch, length, -1) for name in hidden_names if name in hidden)
        if return_dict is False:
            return tuple(x for x in (logits, hidden_states, cache) if x is not None)
        return transformers.modeling_outputs.CausalLMOutputWithPast(logits=logits, hidden_states=hidden_states, past_key_values=cache)

    @staticmethod
    def _left_padding(input_ids: torch.Tensor, attention_mask: torch.Tensor | None) -> list[int]:
        batch, length = input_ids.shape
        if attention_mask is None:
            return [0] * batch
        first = attention_mask.argmax(dim=1)
        Assert.custom(lambda ok: bool(ok), (attention_mask.sum(1) == length - first).all())  # left-padded, contiguous
        return first.tolist()

    @staticmethod
    def _document_lengths(input_ids: torch.Tensor, attention_mask: torch.Tensor | None) -> list[int]:
        """Left padding of each row becomes a separate document in the packed stream."""
        batch, length = input_ids.shape
        if attention_mask is None:
            return [length] * batch
        first = attention_mask.argmax(dim=1)
        Assert.custom(lambda ok: bool(ok), (attention_mask.sum(1) == length - first).all())  # left-padded, contiguous
        lengths = []
        for pad in first.tolist():
            lengths += [length] if pad == 0 else [pad, length - pad]
        return lengths

    def prepare_inputs_for_generation(self, input_ids, attention_mask=None, past_key_values=None, use_cache=None, **kwargs):
        if past_key_values is not None and past_key_values.length > 0:
            input_ids = input_ids[:, past_key_values.length:]  # the cache holds the rest; the padding was settled by the first call
        return {"input_ids": input_ids, "attention_mask": attention_mask, "past_key_values": past_key_values,
                "use_cache": bool(use_cache) and self._cache_supported}

    def _reorder_workers(self, index: torch.Tensor) -> None:
        if self._tensor_group is not None and self._is_coordinator:
            self._broadcast(("reorder", index.cpu()))

    # ---- tensor-parallel coordination
    def _broadcast(self, message) -> None:
        payload = [message]
        source = torch.distributed.get_global_rank(self._tensor_group, 0) if hasattr(torch.distributed, "get_global_rank") else 0
        torch.distributed.broadcast_object_list(payload, src=source, group=self._tensor_group)
        return payload[0]

    def worker_forward(self) -> None:
        """Run on every non-coordinator tensor rank: mirror the coordinator's forward passes until it stops."""
        assert self._tensor_group is not None and not self._is_coordinator
        while True:
            message = self._broadcast(None)
            if message[0] == "stop":
                return
            if message[0] == "reorder":
                self._worker_cache.reorder(message[1])
                continue
            _, input_ids, attention_mask, output_hidden_states, cache_mode = message
            device = self._fast_llm_model.distributed.device
            out = self._inner_forward(input_ids.to(device), None if attention_mask is None else attention_mask.to(device), output_hidden_states,
                                      True, cache_mode, self._worker_cache if cache_mode == "continue" else None)
            self._worker_cache = out.past_key_values

    def stop_workers(self) -> None:
        if self._tensor_group is not None and self._is_coordinator:
            self._broadcast(("stop",))


class HuggingfaceGPTModelConfig(HuggingfaceModelConfig):
    model_type = "fast_llm_gpt"


class HuggingfaceGPTModelForCausalLM(HuggingfacePreTrainedModel):
    config_class = HuggingfaceGPTModelConfig

    @classmethod
    def _model_class(cls):
        from fast_llm_b200.models.gpt.model import GPTModel

        return GPTModel


def _bind_model_class():
    from fast_llm_b200.models.gpt.config import GPTModelConfig
    from fast_llm_b200.models.gpt.model import GPTModel

    HuggingfaceGPTModelForCausalLM.model_class = GPTModel
    HuggingfaceGPTModelConfig.model_config_class = GPTModelConfig


_bind_model_class()
