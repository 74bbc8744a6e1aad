"""Apriel2 text format: a hierarchical Hugging Face config that names every block's mixer by type.

    config.json   hidden_size, vocab_size, tie_word_embeddings,
                  decoder {type: fixed, num_blocks, block} | {type: pattern, num_blocks, pattern, blocks{name: block}},
                  block   {mixer {type: attention | mamba | gdn | kda | stochastic, ...}, mlp {type: mlp, ...},
                           normalization {type: rms_norm, epsilon}},
                  head    {normalization {...}}
    weights       model.embed_tokens.weight, model.decoder.blocks.{i}.{mixer, mlp, input_layernorm,
                  post_attention_layernorm}, model.norm.weight, lm_head.weight; the mixers of a stochastic mixer live
                  under mixer.mixers.{name}.

Mixer sub-configs carry our own field names (heads, head_groups, head_size, rotary {type: mistral_1d | llama3 | yarn},
state_size, d_inner, d_xb, dt_rank, value_heads, key_heads, ...), so the translation is mostly structural.
Parity: `fast_llm/models/gpt/conversion/apriel2.py:151-764`.
"""

import typing

from fast_llm_b200.engine.checkpoint.external import (
    HuggingfaceStateDictCheckpointHandler,
    IgnoreImportWeightConverter,
    SplitWeightConverter,
    TransposeWeightConverter,
    WeightConverter,
)
from fast_llm_b200.models.gpt.conversion.formats import GPTHuggingfaceCheckpointFormat
from fast_llm_b200.ops.activation import ActivationType
from fast_llm_b200.utils import Assert


class Apriel2TextCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "apriel2_text"

    @classmethod
    def get_handler_class(cls):
        return Apriel2HuggingfaceCheckpointHandler


def _enabled(layer_config, default: bool) -> bool:
    enabled = layer_config.bias.enabled
    return default if enabled is None else enabled


def _explicit_biases(config, layer_names: tuple[str, ...]) -> dict:
    """{layer: {"bias": {"enabled": ...}}} for the sub-layers whose bias flag is set explicitly."""
    return {name: {"bias": {"enabled": getattr(config, name).bias.enabled}} for name in layer_names
            if getattr(config, name).bias.enabled is not None}


def _copy_keys(source: dict, names: tuple[str, ...]) -> dict:
    return {name: source[name] for name in names if name in source}


# ---------------------------------------------------------------------------------------------------------------- rotary
def _rotary_export(rotary) -> dict:
    kind = type(rotary).__name__
    if kind == "DefaultRotaryConfig":
        return {"type": "mistral_1d", "theta": rotary.theta}
    if kind == "Llama3RotaryConfig":
        return {"type": "llama3", "theta": rotary.theta, "scale_factor": rotary.scale_factor, "low_frequency_factor": rotary.low_frequency_factor,
                "high_frequency_factor": rotary.high_frequency_factor, "original_context_length": rotary.original_context_length}
    if kind == "YarnRotaryConfig":
        return {"type": "yarn", "theta": rotary.theta, "scale_factor": rotary.scale_factor, "attention_factor": rotary.attention_factor,
                "beta_fast": rotary.beta_fast, "beta_slow": rotary.beta_slow, "original_context_length": rotary.original_context_length}
    raise NotImplementedError(f"The Apriel2 format has no rotary type for {kind}")


def _rotary_import(rotary: dict) -> dict:
    out = dict(rotary)
    if out.get("type") == "mistral_1d":
        out["type"] = "default"
    return out


# ---------------------------------------------------------------------------------------------------------------- mixers
_ATTENTION_LAYERS = ("query_layer", "key_layer", "value_layer", "dense_layer")
_MLP_LAYERS = ("layer_1", "layer_2")


def _mixer_export(mixer) -> dict:
    kind = type(mixer).__name__
    if kind == "AttentionConfig":
        out = {"type": "attention", "heads": mixer.heads, "head_groups": mixer.head_groups, "head_size": mixer.head_size,
               "rotary": _rotary_export(mixer.rotary), "add_linear_biases": mixer.add_linear_biases}
        if mixer.window_size is not None:
            out["window_size"] = mixer.window_size
        out.update(_explicit_biases(mixer, _ATTENTION_LAYERS))
        return out
    if kind == "MambaConfig":
        return {"type": "mamba", "state_size": mixer.state_size, "d_inner": mixer.d_inner, "d_xb": mixer.d_xb, "dt_rank": mixer.dt_rank,
                "add_linear_biases": mixer.add_linear_biases, "repeat_kv_before_conv": mixer.repeat_kv_before_conv,
                "d_conv": mixer.convolution_layer.kernel_size,
                "conv_bias": _enabled(mixer.convolution_layer, mixer.add_linear_biases), "dt_proj_bias": _enabled(mixer.dt_layer, mixer.add_linear_biases)}
    if kind == "GatedDeltaNetConfig":
        return {"type": "gdn", "value_heads": mixer.value_heads, "key_heads": mixer.key_heads, "key_head_dim": mixer.key_head_dim,
                "value_head_dim": mixer.value_head_dim, "convolution_layer": {"kernel_size": mixer.convolution_layer.kernel_size}}
    if kind == "KimiDeltaAttentionConfig":
        return {"type": "kda", "heads": mixer.heads, "head_dim": mixer.head_dim, "convolution_layer": {"kernel_size": mixer.convolution_layer.kernel_size},
                "normalization": {"epsilon": mixer.normalization.epsilon}}
    if kind == "StochasticMixerConfig":
        out = {"type": "stochastic", "mixers": {}, "main_mixer_name": mixer.main_mixer_name, "sampling_strategy": mixer.sampling_strategy.value}
        for name, sub in mixer.mixers.items():
            Assert.custom(lambda k: k != "StochasticMixerConfig", type(sub).__name__)  # no nesting in the format
            out["mixers"][name] = _mixer_export(sub)
        return out
    raise NotImplementedError(f"The Apriel2 format has no mixer type for {kind}")


def _mixer_import(h: dict) -> dict:
    kind = h.get("type", "attention")
    if kind == "attention":
        out = {"type": "attention", **_copy_keys(h, ("heads", "head_groups", "head_size", "window_size") + _ATTENTION_LAYERS),
               "rotary": _rotary_import(h.get("rotary", {"type": "mistral_1d"})), "add_linear_biases": h.get("add_linear_biases", True)}
        return out
    if kind == "mamba":
        out = {"type": "mamba", **_copy_keys(h, ("state_size", "d_inner", "d_xb", "dt_rank", "add_linear_biases", "repeat_kv_before_conv"))}
        convolution, dt_layer = {}, {}
        if "d_conv" in h:
            convolution["kernel_size"] = h["d_conv"]
        if "conv_bias" in h:
            convolution["bias"] = {"enabled": h["conv_bias"]}
        if "dt_proj_bias" in h:
            dt_layer["bias"] = {"enabled": h["dt_proj_bias"]}
        if convolution:
            out["convolution_layer"] = convolution
        if dt_layer:
            out["dt_layer"] = dt_layer
        return out
    if kind == "gdn":
        return {"type": "gdn", **_copy_keys(h, ("value_heads", "key_heads", "key_head_dim", "value_head_dim", "convolution_layer"))}
    if kind == "kda":
        return {"type": "kda", **_copy_keys(h, ("heads", "head_dim", "convolution_layer", "normalization"))}
    if kind == "stochastic":
        out = {"type": "stochastic", "mixers": {name: _mixer_import(sub) for name, sub in h["mixers"].items()},
               **_copy_keys(h, ("main_mixer_name", "sampling_strategy"))}
        return out
    raise NotImplementedError(f"Unknown Apriel2 mixer type {kind}")


def _linear(ours: str, theirs: str, has_bias: bool) -> list[WeightConverter]:
    out = [WeightConverter(f"{ours}.weight", f"{theirs}.weight")]
    if has_bias:
        out.append(WeightConverter(f"{ours}.bias", f"{theirs}.bias"))
    return out


def _mixer_weights(mixer, ours: str, theirs: str) -> list[WeightConverter]:
    kind = type(mixer).__name__
    if kind == "AttentionConfig":
        default = mixer.add_linear_biases
        out = _linear(f"{ours}.query", f"{theirs}.q_proj", _enabled(mixer.query_layer, default))
        out.append(SplitWeightConverter(f"{ours}.key_value.weight", (f"{theirs}.k_proj.weight", f"{theirs}.v_proj.weight")))
        if _enabled(mixer.key_layer, default):
            out.append(SplitWeightConverter(f"{ours}.key_value.bias", (f"{theirs}.k_proj.bias", f"{theirs}.v_proj.bias")))
        return out + _linear(f"{ours}.dense", f"{theirs}.o_proj", _enabled(mixer.dense_layer, default))
    if kind == "MambaConfig":
        bias = mixer.add_linear_biases
        out = []
        for name in ("in_proj", "dt_in_proj", "out_proj"):
            out += _linear(f"{ours}.{name}", f"{theirs}.{name}", bias)
        out += _linear(f"{ours}.dt_proj", f"{theirs}.dt_proj", _enabled(mixer.dt_layer, bias))
        out += _linear(f"{ours}.convolution", f"{theirs}.conv1d", _enabled(mixer.convolution_layer, bias))
        return out + [WeightConverter(f"{ours}.A_log", f"{theirs}.A_log"), WeightConverter(f"{ours}.D", f"{theirs}.D")]
    if kind == "GatedDeltaNetConfig":
        out = []
        for name in ("in_proj_qkvz", "in_proj_ba", "out_proj"):
            out += _linear(f"{ours}.{name}", f"{theirs}.{name}", False)
        out += _linear(f"{ours}.convolution", f"{theirs}.convolution", _enabled(mixer.convolution_layer, False))
        return out + [WeightConverter(f"{ours}.{name}", f"{theirs}.{name}") for name in ("dt_bias", "A_log", "norm.weight")]
    if kind == "KimiDeltaAttentionConfig":
        out = []
        for name in ("q_proj", "k_proj", "v_proj", "q_conv", "k_conv", "v_conv", "f_a_proj", "f_b_proj", "g_a_proj", "g_b_proj", "beta_proj", "o_proj"):
            out += _linear(f"{ours}.{name}", f"{theirs}.{name}", False)
        return out + [WeightConverter(f"{ours}.{name}", f"{theirs}.{name}") for name in ("A_log", "dt_bias", "norm.weight")]
    if kind == "StochasticMixerConfig":
        out = []
        for name, sub in mixer.mixers.items():
            out += _mixer_weights(sub, f"{ours}.mixers.{name}", f"{theirs}.mixers.{name}")
        return out
    raise NotImplementedError(f"The Apriel2 format has no mixer type for {kind}")


# ---------------------------------------------------------------------------------------------------------------- blocks
def _normalization_export(norm) -> dict:
    kind = type(norm).__name__
    if kind == "RMSNormalizationConfig":
        return {"type": "rms_norm", "epsilon": norm.epsilon}
    if kind == "LayerNormalizationConfig":
        return {"type": "layer_norm", "epsilon": norm.epsilon}
    if kind == "NoNormalizationConfig":
        return {"type": "none"}
    raise NotImplementedError(f"The Apriel2 format has no normalization type for {kind}")


def _block_export(block) -> dict:
    mlp = block.mlp
    Assert.eq(type(mlp).__name__, "MLPConfig")  # the format has no mixture-of-experts MLP
    Assert.eq(type(block.normalization).__name__, "RMSNormalizationConfig")  # weights are mapped for RMS norm only
    mlp_out = {"type": "mlp", "intermediate_size": mlp.intermediate_size, "gated": mlp.gated, "add_linear_biases": mlp.add_linear_biases,
               "activation": mlp.activation.hf_name, **_explicit_biases(mlp, _MLP_LAYERS)}
    return {"mixer": _mixer_export(block.mixer), "mlp": mlp_out, "normalization": _normalization_export(block.normalization)}


def _block_import(h: dict) -> dict:
    mlp = h["mlp"]
    mlp_out = {"type": "mlp", **_copy_keys(mlp, ("intermediate_size", "gated", "add_linear_biases") + _MLP_LAYERS)}
    if "activation" in mlp:
        mlp_out["activation"] = ActivationType.from_hf_name(mlp["activation"]).value
    return {"type": "decoder", "mixer": _mixer_import(h["mixer"]), "mlp": mlp_out, "normalization": dict(h["normalization"])}


def _block_weights(block, ours: str, theirs: str) -> list[WeightConverter]:
    out = [WeightConverter(f"{ours}.norm_1.weight", f"{theirs}.input_layernorm.weight"),
           WeightConverter(f"{ours}.norm_2.weight", f"{theirs}.post_attention_layernorm.weight")]
    out += _mixer_weights(block.mixer, f"{ours}.mixer", f"{theirs}.mixer")
    mlp = block.mlp
    bias_1, bias_2 = _enabled(mlp.layer_1, mlp.add_linear_biases), _enabled(mlp.layer_2, mlp.add_linear_biases)
    first = (f"{theirs}.mlp.gate_proj", f"{theirs}.mlp.up_proj") if mlp.gated else (f"{theirs}.mlp.up_proj",)
    converter = SplitWeightConverter if mlp.gated else WeightConverter
    out.append(converter(f"{ours}.mlp.layer_1.weight", tuple(f"{n}.weight" for n in first)))
    if bias_1:
        out.append(converter(f"{ours}.mlp.layer_1.bias", tuple(f"{n}.bias" for n in first)))
    out.append(TransposeWeightConverter(f"{ours}.mlp.layer_2.weight", f"{theirs}.mlp.down_proj.weight"))
    if bias_2:
        out.append(WeightConverter(f"{ours}.mlp.layer_2.bias", f"{theirs}.mlp.down_proj.bias"))
    return out


class Apriel2HuggingfaceCheckpointHandler(HuggingfaceStateDictCheckpointHandler):
    format = Apriel2TextCheckpointFormat
    architecture = "Apriel2ForCausalLM"
    model_type = "apriel2_text"

    @classmethod
    def get_model_config_class(cls):
        from fast_llm_b200.models.gpt.config import GPTModelConfig

        return GPTModelConfig

    @classmethod
    def get_extra_files(cls):
        """Stand-alone modelling code that `transformers` loads from the exported directory (`auto_map`)."""
        import pathlib

        from fast_llm_b200.external_models.apriel2 import configuration_apriel2, modeling_apriel2

        return [pathlib.Path(configuration_apriel2.__file__), pathlib.Path(modeling_apriel2.__file__)]

    @classmethod
    def export_config(cls, c) -> dict:
        decoder = c.decoder
        Assert.eq(c.head.prediction_heads, 1)  # the format has no multi-token prediction
        Assert.eq(type(c.head.normalization).__name__, "RMSNormalizationConfig")
        if type(decoder).__name__ == "FixedBlockSequenceConfig":
            decoder_out = {"type": "fixed", "num_blocks": decoder.num_blocks, "block": _block_export(decoder.block)}
        else:
            decoder_out = {"type": "pattern", "num_blocks": decoder.num_blocks, "pattern": list(decoder.pattern),
                           "blocks": {name: _block_export(block) for name, block in decoder.blocks.items()}}
        return {
            "model_type": cls.model_type, "architectures": [cls.architecture],
            "hidden_size": c.hidden_size, "vocab_size": c.embeddings.vocab_size, "tie_word_embeddings": c.tied_embedding_weight,
            "decoder": decoder_out, "head": {"normalization": _normalization_export(c.head.normalization)},
            "auto_map": {"AutoConfig": "configuration_apriel2.Apriel2TextConfig", "AutoModel": "modeling_apriel2.Apriel2TextModel",
                         "AutoModelForCausalLM": "modeling_apriel2.Apriel2ForCausalLM"},
        }

    @classmethod
    def import_config(cls, h: dict) -> dict:
        decoder = h["decoder"]
        if decoder.get("type", "fixed") == "fixed":
            decoder_out = {"type": "fixed", "num_blocks": decoder["num_blocks"], "block": _block_import(decoder["block"])}
        else:
            decoder_out = {"type": "pattern", "num_blocks": decoder["num_blocks"], "pattern": list(decoder["pattern"]),
                           "blocks": {name: _block_import(block) for name, block in decoder["blocks"].items()}}
        head = {"normalization": dict(h["head"]["normalization"])} if "head" in h and "normalization" in h["head"] else {}
        return {"embeddings": {"vocab_size": h["vocab_size"]}, "decoder": decoder_out, "head": head, "hidden_size": h["hidden_size"],
                "tied_embedding_weight": bool(h.get("tie_word_embeddings", False))}

    @classmethod
    def get_weight_converters(cls, c) -> list[WeightConverter]:
        out = [WeightConverter("embeddings.word_embeddings_weight", "model.embed_tokens.weight")]
        for i, block in enumerate(c.decoder.block_configs()):
            out += _block_weights(block, f"decoder.{i}", f"model.decoder.blocks.{i}")
        out.append(WeightConverter("head.final_norm.weight", "model.norm.weight"))
        out.append(IgnoreImportWeightConverter("lm_head.weight") if c.tied_embedding_weight else WeightConverter("head.output_weights", "lm_head.weight"))
        return out
