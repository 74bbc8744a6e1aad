"""Hugging Face `llava` format of the multimodal model: a Pixtral vision tower, a two-layer projector and a Mistral
language model.

Weight map (parity: `fast_llm/models/multimodal/conversion/llava.py:43-417`):
  vision_encoder.embeddings.patch_embeddings.weight [hidden, 3*p*p]  <-> vision_tower.patch_conv.weight [hidden, 3, p, p]
  vision_encoder.embeddings.normalization.weight                     <-> vision_tower.ln_pre.weight
  vision_encoder.encoder.{i}.norm_1 / norm_2                         <-> vision_tower.transformer.layers.{i}.attention_norm / ffn_norm
  vision_encoder.encoder.{i}.mixer.{query,key_value,dense}           <-> ...attention.{q_proj | k_proj + v_proj | o_proj}
  vision_encoder.encoder.{i}.mlp.{layer_1,layer_2}                   <-> ...feed_forward.{gate_proj + up_proj | down_proj}
  vision_encoder.adapter.{layer_1,layer_2}                           <-> multi_modal_projector.{linear_1,linear_2}
  embeddings / decoder / head                                        <-> language_model.* with the Mistral names
"""

import typing

import torch

from fast_llm_b200.engine.checkpoint.config import CheckpointFormat
from fast_llm_b200.engine.checkpoint.external import (
    HuggingfaceStateDictCheckpointHandler,
    SplitWeightConverter,
    TransposeWeightConverter,
    WeightConverter,
)
from fast_llm_b200.models.gpt.conversion.formats import MistralHuggingfaceCheckpointHandler
from fast_llm_b200.ops.activation import ActivationType
from fast_llm_b200.utils import Assert, div


class LlavaCheckpointFormat(CheckpointFormat):
    support_optimizer: typing.ClassVar[bool] = False
    name: typing.ClassVar[str] = "llava"

    @classmethod
    def get_handler_class(cls):
        return LlavaHuggingfaceCheckpointHandler


class PatchEmbeddingWeightConverter(WeightConverter):
    """Our linear over flattened patches <-> the convolution kernel of the vision tower."""

    def export_weight(self, weight):
        shape = self._config
        return (weight[0].reshape(weight[0].shape[0], *shape),)

    def import_weight(self, weight):
        return (weight[0].flatten(1),)


class LlavaHuggingfaceCheckpointHandler(HuggingfaceStateDictCheckpointHandler):
    format = LlavaCheckpointFormat
    architecture = "LlavaForConditionalGeneration"
    text_handler = MistralHuggingfaceCheckpointHandler

    @classmethod
    def get_model_config_class(cls):
        from fast_llm_b200.models.multimodal.config import MultiModalModelConfig

        return MultiModalModelConfig

    # ---- config
    @classmethod
    def export_config(cls, c) -> dict:
        vision = c.vision_encoder
        Assert.not_none(c.image_token_index)
        blocks = vision.encoder.block_configs()
        block = blocks[0]
        mixer, mlp = block.mixer, block.mlp
        Assert.eq(vision.embeddings.patch_height, vision.embeddings.patch_width)
        assert not mixer.causal and mixer.heads == mixer.head_groups and mlp.gated
        adapter = vision.adapter
        Assert.eq(adapter.intermediate_size, c.hidden_size)
        text = cls.text_handler.export_config(c)
        text.pop("architectures", None)
        return {
            "model_type": "llava", "architectures": [cls.architecture], "text_config": text,
            "vision_config": {
                "model_type": "pixtral", "hidden_size": vision.hidden_size, "num_hidden_layers": len(blocks),
                "num_attention_heads": mixer.heads, "head_dim": mixer.head_size, "intermediate_size": mlp.intermediate_size,
                "hidden_act": mlp.activation.hf_name, "patch_size": vision.embeddings.patch_height, "num_channels": 3,
                "rope_theta": mixer.rotary.theta, "image_size": 1024,
            },
            "projector_hidden_act": adapter.activation.hf_name, "multimodal_projector_bias": adapter.add_linear_biases,
            "image_token_index": c.image_token_index, "vision_feature_layer": -1, "vision_feature_select_strategy": "full",
            "tie_word_embeddings": False, "torch_dtype": "bfloat16",
        }

    @classmethod
    def import_config(cls, h: dict) -> dict:
        out = cls.text_handler.import_config(h["text_config"])
        v = h["vision_config"]
        heads = v["num_attention_heads"]
        head_size = v.get("head_dim") or div(v["hidden_size"], heads)
        norm = {"type": "rms_norm", "epsilon": 1e-5}
        theta = v.get("rope_theta") or (v.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        out["vision_encoder"] = {
            "hidden_size": v["hidden_size"],
            "embeddings": {"patch_height": v["patch_size"], "patch_width": v["patch_size"], "normalization": norm},
            "encoder": {"type": "fixed", "num_blocks": v["num_hidden_layers"], "block": {
                "mixer": {"type": "attention", "heads": heads, "head_groups": heads, "head_size": head_size, "causal": False,
                          "add_linear_biases": False, "rotary": {"type": "default_2d", "theta": theta}},
                "mlp": {"type": "mlp", "intermediate_size": v["intermediate_size"], "gated": True, "add_linear_biases": False,
                        "activation": ActivationType.from_hf_name(v.get("hidden_act", "silu")).value},
                "normalization": norm}},
            "adapter": {"type": "mlp", "intermediate_size": h["text_config"]["hidden_size"], "gated": False,
                        "add_linear_biases": bool(h.get("multimodal_projector_bias", True)),
                        "activation": ActivationType.from_hf_name(h.get("projector_hidden_act", "gelu")).value},
        }
        out["image_token_index"] = h.get("image_token_index")
        return out

    # ---- weights
    @classmethod
    def get_weight_converters(cls, c) -> list[WeightConverter]:
        vision = c.vision_encoder
        e = vision.embeddings
        out = [PatchEmbeddingWeightConverter("vision_encoder.embeddings.patch_embeddings.weight", "vision_tower.patch_conv.weight",
                                             (e.input_channels, e.patch_height, e.patch_width)),
               WeightConverter("vision_encoder.embeddings.normalization.weight", "vision_tower.ln_pre.weight")]
        for i, block in enumerate(vision.encoder.block_configs()):
            ours, theirs = f"vision_encoder.encoder.{i}", f"vision_tower.transformer.layers.{i}"
            out.append(WeightConverter(f"{ours}.norm_1.weight", f"{theirs}.attention_norm.weight"))
            out.append(WeightConverter(f"{ours}.norm_2.weight", f"{theirs}.ffn_norm.weight"))
            out.append(WeightConverter(f"{ours}.mixer.query.weight", f"{theirs}.attention.q_proj.weight"))
            out.append(SplitWeightConverter(f"{ours}.mixer.key_value.weight", (f"{theirs}.attention.k_proj.weight", f"{theirs}.attention.v_proj.weight")))
            out.append(WeightConverter(f"{ours}.mixer.dense.weight", f"{theirs}.attention.o_proj.weight"))
            out.append(SplitWeightConverter(f"{ours}.mlp.layer_1.weight", (f"{theirs}.feed_forward.gate_proj.weight", f"{theirs}.feed_forward.up_proj.weight")))
            out.append(TransposeWeightConverter(f"{ours}.mlp.layer_2.weight", f"{theirs}.feed_forward.down_proj.weight"))
        adapter = vision.adapter
        out.append(WeightConverter("vision_encoder.adapter.layer_1.weight", "multi_modal_projector.linear_1.weight"))
        out.append(TransposeWeightConverter("vision_encoder.adapter.layer_2.weight", "multi_modal_projector.linear_2.weight"))
        if adapter.add_linear_biases:
            out.append(WeightConverter("vision_encoder.adapter.layer_1.bias", "multi_modal_projector.linear_1.bias"))
            out.append(WeightConverter("vision_encoder.adapter.layer_2.bias", "multi_modal_projector.linear_2.bias"))
        for converter in cls.text_handler.get_weight_converters(c):
            converter.export_name = tuple(f"language_model.{name}" for name in converter.export_name)
            out.append(converter)
        return out


MULTIMODAL_CHECKPOINT_FORMATS: tuple = (LlavaCheckpointFormat,)
