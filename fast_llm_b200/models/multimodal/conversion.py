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

import pathlib
import typing

import torch

from fast_llm_b200.engine.checkpoint.config import CheckpointFormat
from fast_llm_b200.engine.checkpoint.external import (
    HuggingfaceStateDictCheckpointHandler,
    SplitWeightConverter,
    TransposeWeightConverter,
    WeightConverter,
)
from fast_llm_b200.models.gpt.conversion.formats import AprielHybridSSMHuggingfaceCheckpointHandler, MistralHuggingfaceCheckpointHandler
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
    # the number of placeholder tokens per image and the largest image are properties of the processor / the data
    ignored_import_keys = frozenset({"image_seq_length", "vision_config.image_size"})
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
        Assert.eq(adapter.intermediate_size, c.hidden_size, msg="the Llava projector is hidden -> hidden: vision_encoder.adapter.intermediate_size must equal hidden_size")
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
            "tie_word_embeddings": False,
        }

    @classmethod
    def import_config(cls, h: dict) -> dict:
        out = cls.text_handler.import_config(h["text_config"])
        v = h["vision_config"]
        # what this model implements of Llava: features of the last vision layer, every patch, untied output weights, RGB
        layer, strategy = h.get("vision_feature_layer", -1), h.get("vision_feature_select_strategy", "full")
        if layer not in (-1, v["num_hidden_layers"] - 1) or strategy != "full":
            raise NotImplementedError(f"Llava with vision_feature_layer={layer}, vision_feature_select_strategy={strategy!r}")
        Assert.eq(v.get("num_channels", 3), 3)
        Assert.eq(v.get("attention_dropout", 0.0), 0.0)
        if h.get("tie_word_embeddings"):
            out["tied_embedding_weight"] = True
        rope_kind = (v.get("rope_parameters") or {}).get("rope_type", "default")
        Assert.eq(rope_kind, "default")
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
    @staticmethod
    def _legacy_name(name: str) -> str:
        """Llava files come in three spellings: the original one that this exporter writes and `transformers` still loads
        (`vision_tower.*`, `multi_modal_projector.*`, `language_model.model.*`, `language_model.lm_head.*`); the in-memory
        names of `transformers` >= 4.52 (`model.vision_tower.*`, `model.language_model.*`, `lm_head.*`); and what its
        `save_pretrained` writes today (`model.language_model.model.*`, `language_model.lm_head.*`).  All map to the first."""
        if name.startswith("lm_head."):
            return f"language_model.{name}"
        if name.startswith(("model.vision_tower.", "model.multi_modal_projector.", "model.language_model.")):
            name = name[len("model."):]
        if name.startswith("language_model.") and not name.startswith(("language_model.model.", "language_model.lm_head.")):
            name = "language_model.model." + name[len("language_model."):]
        return name

    def _import_tensors(self, name, tensor, pending):
        return super()._import_tensors(self._legacy_name(name), tensor, pending)

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


class LlavaHybridSSMCheckpointFormat(CheckpointFormat):
    support_optimizer: typing.ClassVar[bool] = False
    name: typing.ClassVar[str] = "llava_hybrid_ssm"

    @classmethod
    def get_handler_class(cls):
        return LlavaHybridSSMHuggingfaceCheckpointHandler


class LlavaHybridSSMHuggingfaceCheckpointHandler(LlavaHuggingfaceCheckpointHandler):
    """Llava with an Apriel hybrid (attention / Mamba / gated DeltaNet) language model
    (`fast_llm/models/multimodal/conversion/llava_hybrid.py:13-47`)."""

    format = LlavaHybridSSMCheckpointFormat
    architecture = "LlavaHybridForConditionalGeneration"
    text_handler = AprielHybridSSMHuggingfaceCheckpointHandler

    @classmethod
    def export_config(cls, c) -> dict:
        out = super().export_config(c)
        out["model_type"] = "llava_hybrid"  # the type of `LlavaHybridConfig`, which `auto_map` resolves
        out["text_config"].pop("auto_map", None)
        out["auto_map"] = {"AutoConfig": "configuration_llava_hybrid.LlavaHybridConfig", "AutoModel": "modeling_llava_hybrid.LlavaHybridModel",
                           "AutoModelForCausalLM": "modeling_llava_hybrid.LlavaHybridForConditionalGeneration",
                           "AutoModelForImageTextToText": "modeling_llava_hybrid.LlavaHybridForConditionalGeneration"}
        return out

    @classmethod
    def get_extra_files(cls):
        from fast_llm_b200.external_models.llava_hybrid import configuration_llava_hybrid, modeling_llava_hybrid

        return [*cls.text_handler.get_extra_files(), pathlib.Path(configuration_llava_hybrid.__file__), pathlib.Path(modeling_llava_hybrid.__file__)]


class Apriel2CheckpointFormat(CheckpointFormat):
    support_optimizer: typing.ClassVar[bool] = False
    name: typing.ClassVar[str] = "apriel2"

    @classmethod
    def get_handler_class(cls):
        return Apriel2MultimodalHuggingfaceCheckpointHandler


class Apriel2MultimodalHuggingfaceCheckpointHandler(HuggingfaceStateDictCheckpointHandler):
    """Apriel2 with a vision encoder: the text format's keys at the top level plus a `vision_encoder` section
    {hidden_size, embeddings {patch_height, patch_width, normalization}, encoder {type: fixed, num_blocks, block},
    adapter {type: mlp, ...}} and `image_token_index`.  Vision weights live under `model.vision_encoder.{embeddings,
    encoder.blocks.{i}, adapter}`; the adapter keeps the llava names `linear_1` / `linear_2`
    (`fast_llm/models/multimodal/conversion/apriel2.py:48-528`)."""

    format = Apriel2CheckpointFormat
    architecture = "Apriel2ForConditionalGeneration"
    model_type = "apriel2"

    @classmethod
    def get_model_config_class(cls):
        from fast_llm_b200.models.multimodal.config import MultiModalModelConfig

        return MultiModalModelConfig

    @classmethod
    def get_extra_files(cls):
        """The stand-alone Apriel2 modelling files hold the multimodal classes the `auto_map` below names."""
        from fast_llm_b200.models.gpt.conversion import apriel2 as text

        return text.Apriel2HuggingfaceCheckpointHandler.get_extra_files()

    @classmethod
    def export_config(cls, c) -> dict:
        from fast_llm_b200.models.gpt.conversion import apriel2 as text

        out = text.Apriel2HuggingfaceCheckpointHandler.export_config(c)
        vision = c.vision_encoder
        e = vision.embeddings
        Assert.eq(e.patch_height, e.patch_width)
        block = vision.encoder.block
        mixer = block.mixer
        Assert.eq(type(mixer).__name__, "AttentionConfig")
        rotary_kind = type(mixer.rotary).__name__
        rotary = ({"type": "pixtral_2d", "theta": mixer.rotary.theta, "patch_size": e.patch_height, "max_image_size": 1024}
                  if rotary_kind == "Rotary2DConfig" else {"type": "mistral_1d", "theta": mixer.rotary.theta})
        mlp, adapter = block.mlp, vision.adapter

        def mlp_section(m):
            return {"type": "mlp", "intermediate_size": m.intermediate_size, "activation": m.activation.hf_name, "gated": m.gated,
                    "add_linear_biases": m.add_linear_biases}

        out.update({
            "model_type": cls.model_type, "architectures": [cls.architecture], "image_token_index": c.image_token_index,
            "vision_encoder": {
                "hidden_size": vision.hidden_size, "num_hidden_layers": vision.encoder.num_blocks, "patch_size": e.patch_height, "num_channels": 3,
                "embeddings": {"patch_height": e.patch_height, "patch_width": e.patch_width, "input_channels": 3,
                               "normalization": text._normalization_export(e.normalization)},
                "encoder": {"type": "fixed", "num_blocks": vision.encoder.num_blocks, "block": {
                    "mixer": {"type": "attention", "heads": mixer.heads, "head_groups": mixer.head_groups, "head_size": mixer.head_size,
                              "add_linear_biases": mixer.add_linear_biases, "causal": mixer.causal, "cross_document_attention": False, "rotary": rotary},
                    "mlp": mlp_section(mlp), "normalization": text._normalization_export(block.normalization)}},
                "adapter": mlp_section(adapter),
            },
            "auto_map": {"AutoConfig": "configuration_apriel2.Apriel2Config", "AutoModel": "modeling_apriel2.Apriel2Model",
                         "AutoModelForCausalLM": "modeling_apriel2.Apriel2ForConditionalGeneration",
                         "AutoModelForImageTextToText": "modeling_apriel2.Apriel2ForConditionalGeneration"},
        })
        return out

    @classmethod
    def import_config(cls, h: dict) -> dict:
        from fast_llm_b200.models.gpt.conversion import apriel2 as text

        out = text.Apriel2HuggingfaceCheckpointHandler.import_config(h)
        v = h["vision_encoder"]
        block = v["encoder"]["block"]
        mixer = dict(block["mixer"])
        rotary = dict(mixer.get("rotary", {"type": "pixtral_2d"}))
        rotary["type"] = {"pixtral_2d": "default_2d", "mistral_1d": "default"}.get(rotary.get("type"), rotary.get("type"))
        rotary.pop("patch_size", None)
        rotary.pop("max_image_size", None)
        mixer["rotary"] = rotary
        mixer.pop("cross_document_attention", None)

        def mlp_section(m):
            section = {"type": "mlp", **{k: m[k] for k in ("intermediate_size", "gated", "add_linear_biases") if k in m}}
            if "activation" in m:
                section["activation"] = ActivationType.from_hf_name(m["activation"]).value
            return section

        out["vision_encoder"] = {
            "hidden_size": v["hidden_size"],
            "embeddings": {"patch_height": v["embeddings"]["patch_height"], "patch_width": v["embeddings"]["patch_width"],
                           "normalization": dict(v["embeddings"]["normalization"])},
            "encoder": {"type": "fixed", "num_blocks": v["encoder"]["num_blocks"],
                        "block": {"mixer": mixer, "mlp": mlp_section(block["mlp"]), "normalization": dict(block["normalization"])}},
            "adapter": mlp_section(v["adapter"]),
        }
        out["image_token_index"] = h.get("image_token_index")
        return out

    @classmethod
    def get_weight_converters(cls, c) -> list[WeightConverter]:
        from fast_llm_b200.models.gpt.conversion import apriel2 as text

        vision = c.vision_encoder
        e = vision.embeddings
        prefix = "model.vision_encoder"
        out = [PatchEmbeddingWeightConverter("vision_encoder.embeddings.patch_embeddings.weight", f"{prefix}.embeddings.patch_embeddings.weight",
                                             (e.input_channels, e.patch_height, e.patch_width)),
               WeightConverter("vision_encoder.embeddings.normalization.weight", f"{prefix}.embeddings.normalization.weight")]
        for i, block in enumerate(vision.encoder.block_configs()):
            out += text._block_weights(block, f"vision_encoder.encoder.{i}", f"{prefix}.encoder.blocks.{i}")
        adapter = vision.adapter
        out.append(WeightConverter("vision_encoder.adapter.layer_1.weight", f"{prefix}.adapter.linear_1.weight"))
        out.append(TransposeWeightConverter("vision_encoder.adapter.layer_2.weight", f"{prefix}.adapter.linear_2.weight"))
        if adapter.add_linear_biases:
            out.append(WeightConverter("vision_encoder.adapter.layer_1.bias", f"{prefix}.adapter.linear_1.bias"))
            out.append(WeightConverter("vision_encoder.adapter.layer_2.bias", f"{prefix}.adapter.linear_2.bias"))
        return out + text.Apriel2HuggingfaceCheckpointHandler.get_weight_converters(c)


class AutoMultimodalCheckpointFormat(CheckpointFormat):
    support_optimizer: typing.ClassVar[bool] = False
    name: typing.ClassVar[str] = "auto"

    @classmethod
    def get_handler_class(cls):
        return AutoMultimodalHuggingfaceCheckpointHandler


class AutoMultimodalHuggingfaceCheckpointHandler(HuggingfaceStateDictCheckpointHandler):
    """Picks the handler from config.json (`fast_llm/models/multimodal/conversion/auto.py:1-23`); loading only."""

    format = AutoMultimodalCheckpointFormat

    def __new__(cls, model):
        raise TypeError("resolve the concrete handler with resolve(path) first")

    @classmethod
    def resolve(cls, path):
        import json
        import pathlib

        config = json.loads((pathlib.Path(path) / "config.json").read_text())
        architecture = (config.get("architectures") or [None])[0]
        by_architecture = {handler.architecture: handler for handler in (LlavaHuggingfaceCheckpointHandler, LlavaHybridSSMHuggingfaceCheckpointHandler,
                                                                        Apriel2MultimodalHuggingfaceCheckpointHandler)}
        return by_architecture[architecture]

    @classmethod
    def load_metadata(cls, config):
        return cls.resolve(config.path).load_metadata(config)

    @classmethod
    def get_model_config_class(cls):
        from fast_llm_b200.models.multimodal.config import MultiModalModelConfig

        return MultiModalModelConfig


MULTIMODAL_CHECKPOINT_FORMATS: tuple = (AutoMultimodalCheckpointFormat, LlavaCheckpointFormat, LlavaHybridSSMCheckpointFormat, Apriel2CheckpointFormat)
