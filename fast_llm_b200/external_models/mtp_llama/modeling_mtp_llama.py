"""MTP-Llama for `transformers`: Llama whose last transformer layer is the first of `prediction_heads` parallel heads.

Every head applies its own transformer layer (`model.layers[-1]` for the first, `model.mtp_heads[i-1]` for the others) to
the output of the second-to-last layer, followed by its own RMS norm (`model.mtp_norms[i]`); all heads share `lm_head`.
Head i predicts the token i + 1 positions ahead.  Generation uses the first head only.
Stand-alone file (depends on `transformers` only): copied next to exported checkpoints.
"""

import torch
from torch import nn
from transformers.generation import GenerationMixin
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast
from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaModel, LlamaPreTrainedModel, LlamaRMSNorm

try:  # relative import when loaded as remote code next to a checkpoint
    from .configuration_mtp_llama import MTPLlamaConfig
except ImportError:  # pragma: no cover
    from configuration_mtp_llama import MTPLlamaConfig


class MTPLlamaModel(LlamaModel):
    config_class = MTPLlamaConfig

    def __init__(self, config: MTPLlamaConfig):
        super().__init__(config)
        heads = config.prediction_heads
        self.mtp_heads = nn.ModuleList([LlamaDecoderLayer(config, config.num_hidden_layers + i) for i in range(heads - 1)])
        self.mtp_norms = nn.ModuleList([LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps) for _ in range(heads)])
        del self.norm  # replaced by one norm per head
        self.post_init()

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, inputs_embeds=None, return_all_prediction_heads: bool = False,
                **kwargs):
        """Returns hidden states `[batch, sequence, hidden]`, or `[batch, sequence, heads, hidden]` for all heads.  No KV cache."""
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        batch, length = inputs_embeds.shape[:2]
        if position_ids is None:
            position_ids = torch.arange(length, device=inputs_embeds.device).unsqueeze(0).expand(batch, -1)
        mask = torch.full((length, length), torch.finfo(inputs_embeds.dtype).min, device=inputs_embeds.device, dtype=inputs_embeds.dtype).triu(1)
        mask = mask[None, None].expand(batch, 1, length, length)
        if attention_mask is not None:
            padding = (1.0 - attention_mask[:, None, None, :].to(inputs_embeds.dtype)) * torch.finfo(inputs_embeds.dtype).min
            mask = mask + padding
        position_embeddings = self.rotary_emb(inputs_embeds, position_ids)
        hidden = inputs_embeds

        def run(layer, states):
            out = layer(states, attention_mask=mask, position_ids=position_ids, position_embeddings=position_embeddings)
            return out[0] if isinstance(out, tuple) else out

        for layer in self.layers[:-1]:
            hidden = run(layer, hidden)
        head_layers = [self.layers[-1], *self.mtp_heads] if return_all_prediction_heads else [self.layers[-1]]
        outputs = [self.mtp_norms[i](run(layer, hidden)) for i, layer in enumerate(head_layers)]
        states = torch.stack(outputs, dim=2) if return_all_prediction_heads else outputs[0]
        return BaseModelOutputWithPast(last_hidden_state=states)


class MTPLlamaForCausalLM(LlamaPreTrainedModel, GenerationMixin):
    config_class = MTPLlamaConfig
    _tied_weights_keys = {"lm_head.weight": "model.embed_tokens.weight"}

    def __init__(self, config: MTPLlamaConfig):
        super().__init__(config)
        self.model = MTPLlamaModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, inputs_embeds=None, labels=None,
                return_all_prediction_heads: bool = False, **kwargs):
        states = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids, inputs_embeds=inputs_embeds,
                            return_all_prediction_heads=return_all_prediction_heads).last_hidden_state
        logits = self.lm_head(states)
        loss = None
        if labels is not None:
            first = logits[:, :, 0] if return_all_prediction_heads else logits
            loss = nn.functional.cross_entropy(first[:, :-1].reshape(-1, first.shape[-1]).float(), labels[:, 1:].reshape(-1), ignore_index=-100)
        return CausalLMOutputWithPast(loss=loss, logits=logits)

    def prepare_inputs_for_generation(self, input_ids, attention_mask=None, **kwargs):
        return {"input_ids": input_ids, "attention_mask": attention_mask}
