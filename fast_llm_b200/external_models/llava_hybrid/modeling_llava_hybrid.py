"""Llava (vision tower -> two-layer projector -> language model) around the Apriel hybrid SSM language model.

Weight names follow the checkpoint layout the `llava_hybrid_ssm` format writes: `vision_tower.*` (a Pixtral vision model),
`multi_modal_projector.linear_{1,2}.*`, `language_model.model.*` and `language_model.lm_head.*`.  Image features replace the
embeddings of the `image_token_index` placeholders, one feature per placeholder in order.  During generation the language
model's cache holds the prompt, images included, so `pixel_values` go in with the first step only.
Same role as `fast_llm_external_models/llava_hybrid/modeling_llava_hybrid.py`.
"""

import torch
import torch.nn.functional as F
from torch import nn
from transformers import AutoModel, GenerationMixin, PreTrainedModel
from transformers.activations import ACT2FN
from transformers.modeling_outputs import CausalLMOutputWithPast

try:
    from fast_llm_b200.external_models.apriel_hybrid_ssm.modeling_apriel_hybrid_ssm import AprielHybridSSMForCausalLM
    from fast_llm_b200.external_models.llava_hybrid.configuration_llava_hybrid import LlavaHybridConfig
except ImportError:  # pragma: no cover - the flat directory of an exported checkpoint
    from .configuration_llava_hybrid import LlavaHybridConfig
    from .modeling_apriel_hybrid_ssm import AprielHybridSSMForCausalLM


class LlavaHybridProjector(nn.Module):
    def __init__(self, config: LlavaHybridConfig):
        super().__init__()
        layers = 1 if isinstance(config.vision_feature_layer, int) else len(config.vision_feature_layer)
        hidden = config.text_config.hidden_size
        self.linear_1 = nn.Linear(config.vision_config.hidden_size * layers, hidden, bias=config.multimodal_projector_bias)
        self.act = ACT2FN[config.projector_hidden_act]
        self.linear_2 = nn.Linear(hidden, hidden, bias=config.multimodal_projector_bias)

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        return self.linear_2(self.act(self.linear_1(features)))


class LlavaHybridPreTrainedModel(PreTrainedModel):
    config_class = LlavaHybridConfig
    base_model_prefix = ""
    _no_split_modules = ["Layer"]
    _is_stateful = True

    @classmethod
    def _supports_default_dynamic_cache(cls) -> bool:
        return False  # the language model makes its own cache


class LlavaHybridModel(LlavaHybridPreTrainedModel):
    """Vision tower, projector and language model; returns the language model's outputs for merged embeddings."""

    def __init__(self, config: LlavaHybridConfig):
        super().__init__(config)
        assert config.text_config.model_type == "apriel_ssm_thinker_hybrid", "the language model must be the Apriel hybrid SSM model"
        self.vision_tower = AutoModel.from_config(config.vision_config)
        self.multi_modal_projector = LlavaHybridProjector(config)
        self.language_model = AprielHybridSSMForCausalLM(config.text_config)
        self.post_init()

    def get_input_embeddings(self):
        return self.language_model.model.embed_tokens

    def set_input_embeddings(self, value):
        self.language_model.model.embed_tokens = value

    def get_image_features(self, pixel_values: torch.Tensor, image_sizes=None) -> torch.Tensor:
        """[number of patches of all images, text hidden size]."""
        kwargs = {} if image_sizes is None else {"image_sizes": image_sizes}
        outputs = self.vision_tower(pixel_values, output_hidden_states=True, **kwargs)
        layer = self.config.vision_feature_layer
        if isinstance(layer, int):
            features = outputs.hidden_states[layer]
        else:
            features = torch.cat([outputs.hidden_states[index] for index in layer], dim=-1)
        if self.config.vision_feature_select_strategy == "default":
            features = features[:, 1:]  # drop a class token
        return self.multi_modal_projector(features.reshape(-1, features.shape[-1]))

    def merge(self, input_ids: torch.Tensor, pixel_values: torch.Tensor | None, image_sizes=None) -> torch.Tensor:
        embeddings = self.get_input_embeddings()(input_ids)
        if pixel_values is None:
            return embeddings
        features = self.get_image_features(pixel_values, image_sizes).to(embeddings.dtype)
        mask = input_ids == self.config.image_token_index
        if int(mask.sum()) != features.shape[0]:
            raise ValueError(f"{int(mask.sum())} image placeholder tokens but {features.shape[0]} image features")
        return embeddings.masked_scatter(mask.unsqueeze(-1), features)

    def forward(self, input_ids=None, pixel_values=None, image_sizes=None, inputs_embeds=None, past_key_values=None, use_cache: bool = False,
                output_hidden_states: bool = False, **kwargs):
        if inputs_embeds is None:
            inputs_embeds = self.merge(input_ids, pixel_values, image_sizes)
        return self.language_model.model(inputs_embeds=inputs_embeds, past_key_values=past_key_values, use_cache=use_cache,
                                         output_hidden_states=output_hidden_states)


class LlavaHybridForConditionalGeneration(LlavaHybridModel, GenerationMixin):
    def get_output_embeddings(self):
        return self.language_model.lm_head

    def set_output_embeddings(self, value):
        self.language_model.lm_head = value

    def prepare_inputs_for_generation(self, input_ids, pixel_values=None, image_sizes=None, past_key_values=None, use_cache: bool = True, **kwargs):
        if past_key_values is not None and past_key_values.get_seq_length() > 0:  # the images went in with the prompt
            return {"input_ids": input_ids[:, past_key_values.get_seq_length():], "past_key_values": past_key_values, "use_cache": use_cache}
        return {"input_ids": input_ids, "pixel_values": pixel_values, "image_sizes": image_sizes, "past_key_values": past_key_values,
                "use_cache": use_cache}

    def forward(self, input_ids=None, pixel_values=None, image_sizes=None, inputs_embeds=None, labels=None, past_key_values=None,
                use_cache: bool = False, output_hidden_states: bool = False, **kwargs):
        outputs = LlavaHybridModel.forward(self, input_ids=input_ids, pixel_values=pixel_values, image_sizes=image_sizes,
                                           inputs_embeds=inputs_embeds, past_key_values=past_key_values, use_cache=use_cache,
                                           output_hidden_states=output_hidden_states)
        logits = self.language_model.lm_head(outputs.last_hidden_state)
        loss = None
        if labels is not None:
            loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1), ignore_index=-100)
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=outputs.past_key_values, hidden_states=outputs.hidden_states)


__all__ = ["LlavaHybridForConditionalGeneration", "LlavaHybridModel", "LlavaHybridPreTrainedModel"]
