"""Hugging Face formats of the GPT family: llama, mistral, qwen2, mixtral, plus `auto` (picked from config.json).

Weight map (parity: `fast_llm/models/gpt/conversion/llama.py:201-427`, `mistral.py`, `qwen2.py`, `mixtral.py:64-81`):
  embeddings.word_embeddings_weight          <-> model.embed_tokens.weight
  decoder.{i}.norm_1/2.weight                <-> model.layers.{i}.input_layernorm / post_attention_layernorm.weight
  decoder.{i}.mixer.query.weight             <-> self_attn.q_proj.weight
  decoder.{i}.mixer.key_value.weight         <-> self_attn.k_proj.weight + v_proj.weight          (rows concatenated)
  decoder.{i}.mixer.dense.weight             <-> self_attn.o_proj.weight
  decoder.{i}.mlp.layer_1.weight             <-> mlp.gate_proj.weight + up_proj.weight            (rows concatenated)
  decoder.{i}.mlp.layer_2.weight             <-> mlp.down_proj.weight                             (transposed)
  head.final_norm.weight, head.output_weights <-> model.norm.weight, lm_head.weight
Rotary uses the half-split pairing on both sides, so projections need no permutation.
"""

import json
import pathlib
import typing

from fast_llm_b200.engine.checkpoint.config import CheckpointFormat
from fast_llm_b200.engine.checkpoint.external import (
    ExpertSplitWeightConverter,
    HuggingfaceStateDictCheckpointHandler,
    IgnoreImportWeightConverter,
    SplitWeightConverter,
    TransposeWeightConverter,
    WeightConverter,
)
from fast_llm_b200.ops.activation import ActivationType
from fast_llm_b200.utils import Assert


class GPTHuggingfaceCheckpointFormat(CheckpointFormat):
    support_optimizer: typing.ClassVar[bool] = False


class LlamaCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "llama"

    @classmethod
    def get_handler_class(cls):
        return LlamaHuggingfaceCheckpointHandler


class MistralCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "mistral"

    @classmethod
    def get_handler_class(cls):
        return MistralHuggingfaceCheckpointHandler


class Qwen2CheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "qwen2"

    @classmethod
    def get_handler_class(cls):
        return Qwen2HuggingfaceCheckpointHandler


class MixtralCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "mixtral"

    @classmethod
    def get_handler_class(cls):
        return MixtralHuggingfaceCheckpointHandler


class MTPLlamaCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "mtp_llama"

    @classmethod
    def get_handler_class(cls):
        return MTPLlamaHuggingfaceCheckpointHandler


class DiffusionDreamCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "dream"

    @classmethod
    def get_handler_class(cls):
        return DiffusionDreamHuggingfaceCheckpointHandler


class DiffusionLlamaCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "diffusion_llama"

    @classmethod
    def get_handler_class(cls):
        return DiffusionLlamaHuggingfaceCheckpointHandler


class AprielHybridSSMCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "apriel_hybrid_ssm"

    @classmethod
    def get_handler_class(cls):
        return AprielHybridSSMHuggingfaceCheckpointHandler


class AutoGPTHuggingfaceCheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "auto"

    @classmethod
    def get_handler_class(cls):
        return AutoGPTHuggingfaceCheckpointHandler


def _rotary_to_hf(rotary) -> tuple[float, dict | None]:
    kind = type(rotary).__name__
    if kind == "NoRotaryConfig":
        raise NotImplementedError("Llama-style formats need rotary embeddings")
    theta = rotary.theta
    if kind == "Llama3RotaryConfig":
        return theta, {"rope_type": "llama3", "factor": rotary.scale_factor, "low_freq_factor": rotary.low_frequency_factor,
                       "high_freq_factor": rotary.high_frequency_factor, "original_max_position_embeddings": rotary.original_context_length}
    if kind == "YarnRotaryConfig":
        return theta, {"rope_type": "yarn", "factor": rotary.scale_factor, "attention_factor": rotary.attention_factor,
                       "beta_fast": rotary.beta_fast, "beta_slow": rotary.beta_slow,
                       "original_max_position_embeddings": rotary.original_context_length}
    return theta, None


def _rotary_from_hf(config: dict) -> dict:
    theta = config.get("rope_theta", 10000.0)
    scaling = config.get("rope_scaling") or config.get("rope_parameters")
    if isinstance(scaling, dict) and "rope_theta" in scaling:
        theta = scaling.get("rope_theta", theta)
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type", "default")) if scaling else "default"
    if kind in ("default", None, "linear") or not scaling:
        return {"type": "default", "theta": theta}
    if kind == "llama3":
        return {"type": "llama3", "theta": theta, "scale_factor": scaling["factor"], "low_frequency_factor": scaling["low_freq_factor"],
                "high_frequency_factor": scaling["high_freq_factor"], "original_context_length": scaling["original_max_position_embeddings"]}
    if kind == "yarn":
        out = {"type": "yarn", "theta": theta, "scale_factor": scaling["factor"], "beta_fast": scaling.get("beta_fast", 32.0),
               "beta_slow": scaling.get("beta_slow", 1.0), "original_context_length": scaling["original_max_position_embeddings"]}
        if scaling.get("attention_factor") is not None:
            out["attention_factor"] = scaling["attention_factor"]
        return out
    raise NotImplementedError(f"Unsupported rope scaling {kind}")


class LlamaHuggingfaceCheckpointHandler(HuggingfaceStateDictCheckpointHandler):
    format = LlamaCheckpointFormat
    architecture = "LlamaForCausalLM"
    model_type = "llama"
    attention_bias_key = "attention_bias"

    @classmethod
    def get_model_config_class(cls):
        from fast_llm_b200.models.gpt.config import GPTModelConfig

        return GPTModelConfig

    # ------------------------------------------------------------------ config
    @classmethod
    def _block(cls, base_model_config):
        decoder = base_model_config.decoder
        Assert.eq(type(decoder).__name__, "FixedBlockSequenceConfig")
        return decoder.block

    @classmethod
    def export_config(cls, c) -> dict:
        block = cls._block(c)
        mixer, mlp, norm = block.mixer, block.mlp, block.normalization
        Assert.eq(type(mixer).__name__, "AttentionConfig")
        Assert.eq(type(norm).__name__, "RMSNormalizationConfig")
        assert mlp.gated, "Llama-style formats need a gated MLP"
        theta, scaling = _rotary_to_hf(mixer.rotary)
        out = {
            "model_type": cls.model_type, "architectures": [cls.architecture],
            "vocab_size": c.embeddings.vocab_size, "hidden_size": c.hidden_size, "num_hidden_layers": c.decoder.num_blocks,
            "num_attention_heads": mixer.heads, "num_key_value_heads": mixer.head_groups, "head_dim": mixer.head_size,
            "intermediate_size": mlp.intermediate_size, "hidden_act": mlp.activation.hf_name, "rms_norm_eps": norm.epsilon,
            "rope_theta": theta, "rope_scaling": scaling, "tie_word_embeddings": c.tied_embedding_weight,
            "mlp_bias": mlp.add_linear_biases, "attention_dropout": mixer.dropout,
            "max_position_embeddings": c.embeddings.num_position_embeddings,
        }
        out.update(cls._export_attention_bias(mixer))
        cls._export_extra(c, out)
        return out

    @classmethod
    def _export_attention_bias(cls, mixer) -> dict:
        return {cls.attention_bias_key: mixer.add_linear_biases}

    @classmethod
    def _export_extra(cls, c, out: dict) -> None:
        pass

    @classmethod
    def import_config(cls, h: dict) -> dict:
        heads = h["num_attention_heads"]
        head_size = h.get("head_dim") or h["hidden_size"] // heads
        mixer = {
            "type": "attention", "rotary": _rotary_from_hf(h), "heads": heads, "head_groups": h.get("num_key_value_heads", heads),
            "head_size": head_size, "add_linear_biases": bool(h.get(cls.attention_bias_key, False)),
            "dropout": h.get("attention_dropout", 0.0),
        }
        cls._import_attention_extra(h, mixer)
        mlp = {"type": "mlp", "intermediate_size": h["intermediate_size"], "add_linear_biases": bool(h.get("mlp_bias", False)),
               "gated": True, "activation": ActivationType.from_hf_name(h.get("hidden_act", "silu")).value}
        cls._import_mlp_extra(h, mlp)
        norm = {"type": "rms_norm", "epsilon": h.get("rms_norm_eps", 1e-6)}
        return {
            "embeddings": {"vocab_size": h["vocab_size"], "num_position_embeddings": h.get("max_position_embeddings", 2048)},
            "decoder": {"type": "fixed", "num_blocks": h["num_hidden_layers"], "block": {"type": "decoder", "mixer": mixer, "mlp": mlp, "normalization": norm}},
            "head": {"normalization": norm},
            "hidden_size": h["hidden_size"],
            "tied_embedding_weight": bool(h.get("tie_word_embeddings", False)),
        }

    @classmethod
    def _import_attention_extra(cls, h: dict, mixer: dict) -> None:
        pass

    @classmethod
    def _import_mlp_extra(cls, h: dict, mlp: dict) -> None:
        pass

    # ------------------------------------------------------------------ weights
    @classmethod
    def _linear(cls, ours: str, theirs: str, has_bias: bool, converter=WeightConverter, theirs_many: tuple[str, ...] | None = None):
        names = theirs_many or (theirs,)
        out = [converter(f"{ours}.weight", tuple(f"{n}.weight" for n in names))]
        if has_bias:
            bias_converter = SplitWeightConverter if len(names) > 1 else WeightConverter
            out.append(bias_converter(f"{ours}.bias", tuple(f"{n}.bias" for n in names)))
        return out

    @classmethod
    def _attention_converters(cls, mixer, ours: str, theirs: str) -> list[WeightConverter]:
        qb = cls._projection_bias(mixer, "query")
        kb = cls._projection_bias(mixer, "key")
        ob = cls._projection_bias(mixer, "dense")
        out = cls._linear(f"{ours}.query", f"{theirs}.q_proj", qb)
        out += cls._linear(f"{ours}.key_value", "", kb, SplitWeightConverter, (f"{theirs}.k_proj", f"{theirs}.v_proj"))
        out += cls._linear(f"{ours}.dense", f"{theirs}.o_proj", ob)
        return out

    @classmethod
    def _projection_bias(cls, mixer, which: str) -> bool:
        layer = {"query": mixer.query_layer, "key": mixer.key_layer, "dense": mixer.dense_layer}[which]
        enabled = layer.bias.enabled
        return mixer.add_linear_biases if enabled is None else enabled

    @classmethod
    def _mlp_converters(cls, mlp, ours: str, theirs: str) -> list[WeightConverter]:
        bias = mlp.add_linear_biases
        out = cls._linear(f"{ours}.layer_1", "", bias, SplitWeightConverter, (f"{theirs}.gate_proj", f"{theirs}.up_proj"))
        out.append(TransposeWeightConverter(f"{ours}.layer_2.weight", f"{theirs}.down_proj.weight"))
        if bias:
            out.append(WeightConverter(f"{ours}.layer_2.bias", f"{theirs}.down_proj.bias"))
        return out

    mlp_name = "mlp"

    @classmethod
    def get_weight_converters(cls, c) -> list[WeightConverter]:
        block = cls._block(c)
        out = [WeightConverter("embeddings.word_embeddings_weight", "model.embed_tokens.weight")]
        for i in range(c.decoder.num_blocks):
            ours, theirs = f"decoder.{i}", f"model.layers.{i}"
            out.append(WeightConverter(f"{ours}.norm_1.weight", f"{theirs}.input_layernorm.weight"))
            out.append(WeightConverter(f"{ours}.norm_2.weight", f"{theirs}.post_attention_layernorm.weight"))
            out += cls._attention_converters(block.mixer, f"{ours}.mixer", f"{theirs}.self_attn")
            out += cls._mlp_converters(block.mlp, f"{ours}.mlp", f"{theirs}.{cls.mlp_name}")
        out.append(WeightConverter("head.final_norm.weight", "model.norm.weight"))
        if c.tied_embedding_weight:
            out.append(IgnoreImportWeightConverter("lm_head.weight"))
        else:
            out.append(WeightConverter("head.output_weights", "lm_head.weight"))
        return out


class MistralHuggingfaceCheckpointHandler(LlamaHuggingfaceCheckpointHandler):
    format = MistralCheckpointFormat
    architecture = "MistralForCausalLM"
    model_type = "mistral"

    @classmethod
    def _export_attention_bias(cls, mixer) -> dict:
        assert not mixer.add_linear_biases, "Mistral has no attention biases"
        return {}

    @classmethod
    def _export_extra(cls, c, out):
        out["sliding_window"] = cls._block(c).mixer.window_size
        out.pop("mlp_bias", None)

    @classmethod
    def _import_attention_extra(cls, h, mixer):
        mixer["add_linear_biases"] = False
        if h.get("sliding_window") is not None:
            mixer["window_size"] = h["sliding_window"]


class Qwen2HuggingfaceCheckpointHandler(LlamaHuggingfaceCheckpointHandler):
    """Qwen2: biases on q/k/v projections only."""

    format = Qwen2CheckpointFormat
    architecture = "Qwen2ForCausalLM"
    model_type = "qwen2"

    @classmethod
    def _export_attention_bias(cls, mixer) -> dict:
        return {}

    @classmethod
    def _export_extra(cls, c, out):
        mixer = cls._block(c).mixer
        assert cls._projection_bias(mixer, "query") and cls._projection_bias(mixer, "key") and not cls._projection_bias(mixer, "dense"), \
            "Qwen2 needs biases on query/key/value and none on the output projection"
        out["use_sliding_window"] = mixer.window_size is not None
        if mixer.window_size is not None:
            out["sliding_window"] = mixer.window_size
            out["max_window_layers"] = 0  # every layer uses the window (Hugging Face keeps full attention below this layer index)
        out.pop("mlp_bias", None)

    @classmethod
    def _import_attention_extra(cls, h, mixer):
        mixer["add_linear_biases"] = True
        mixer["dense_layer"] = {"bias": {"enabled": False}}
        window = h.get("sliding_window")  # always read: the key is present (and inert) when `use_sliding_window` is off
        if h.get("use_sliding_window") and window is not None:
            # layers below `max_window_layers` attend to everything, the others through the window
            full_layers = min(h.get("max_window_layers") or 0, h["num_hidden_layers"])
            if full_layers == 0:
                mixer["window_size"] = window
            elif full_layers < h["num_hidden_layers"]:
                raise NotImplementedError(f"Qwen2 with a sliding window on layers {full_layers}.. only: import it as a pattern decoder")


class MixtralHuggingfaceCheckpointHandler(MistralHuggingfaceCheckpointHandler):
    format = MixtralCheckpointFormat
    architecture = "MixtralForCausalLM"
    model_type = "mixtral"
    mlp_name = "block_sparse_moe"

    @classmethod
    def _export_extra(cls, c, out):
        super()._export_extra(c, out)
        mlp = cls._block(c).mlp
        Assert.eq(type(mlp).__name__, "MoEMLPConfig")
        out["num_local_experts"] = mlp.experts
        out["num_experts_per_tok"] = mlp.experts_per_token
        out["router_aux_loss_coef"] = mlp.auxiliary_loss_coefficient
        out["router_jitter_noise"] = mlp.jitter_eps

    # `output_router_logits` asks the Hugging Face model to return router logits: a run-time switch, not architecture
    ignored_import_keys = MistralHuggingfaceCheckpointHandler.ignored_import_keys | {"output_router_logits"}

    @classmethod
    def _import_mlp_extra(cls, h, mlp):
        mlp.update(type="moe", experts=h["num_local_experts"], experts_per_token=h["num_experts_per_tok"],
                   auxiliary_loss_coefficient=h.get("router_aux_loss_coef", 0.01), jitter_eps=h.get("router_jitter_noise", 0.0))

    @classmethod
    def _mlp_converters(cls, mlp, ours, theirs):
        n = mlp.experts
        assert not mlp.add_linear_biases
        return [
            WeightConverter(f"{ours}.router.weight", f"{theirs}.gate.weight"),
            ExpertSplitWeightConverter(f"{ours}.layer_1.weight", tuple(f"{theirs}.experts.{e}.{w}.weight" for e in range(n) for w in ("w1", "w3")), n, parts=2),
            ExpertSplitWeightConverter(f"{ours}.layer_2.weight", tuple(f"{theirs}.experts.{e}.w2.weight" for e in range(n)), n, parts=1, transpose=True),
        ]


class MTPLlamaHuggingfaceCheckpointHandler(LlamaHuggingfaceCheckpointHandler):
    """Llama with multi-token-prediction heads: head d > 1 = one more transformer layer `model.mtp_heads.{d-2}` plus its own
    final norm `model.mtp_norms.{d-1}`; the first head's norm is `model.mtp_norms.0` (`mtp_llama.py:32-107`)."""

    format = MTPLlamaCheckpointFormat
    architecture = "MTPLlamaForCausalLM"
    model_type = "mtp_llama"

    @classmethod
    def _export_extra(cls, c, out):
        out["prediction_heads"] = c.head.prediction_heads
        out["auto_map"] = {"AutoConfig": "configuration_mtp_llama.MTPLlamaConfig", "AutoModel": "modeling_mtp_llama.MTPLlamaModel",
                           "AutoModelForCausalLM": "modeling_mtp_llama.MTPLlamaForCausalLM"}

    @classmethod
    def import_config(cls, h):
        out = super().import_config(h)
        out["head"]["prediction_heads"] = h.get("prediction_heads", 1)
        return out

    @classmethod
    def get_extra_files(cls):
        from fast_llm_b200.external_models.mtp_llama import configuration_mtp_llama, modeling_mtp_llama

        return [pathlib.Path(configuration_mtp_llama.__file__), pathlib.Path(modeling_mtp_llama.__file__)]

    @classmethod
    def get_weight_converters(cls, c):
        block = cls._block(c)
        out = [conv for conv in super().get_weight_converters(c) if conv.fast_llm_name != ("head.final_norm.weight",)]
        out.append(WeightConverter("head.final_norm.weight", "model.mtp_norms.0.weight"))
        for index in range(c.head.prediction_heads - 1):
            ours, theirs = f"multi_token_prediction.blocks.{index}", f"model.mtp_heads.{index}"
            out.append(WeightConverter(f"{ours}.norm_1.weight", f"{theirs}.input_layernorm.weight"))
            out.append(WeightConverter(f"{ours}.norm_2.weight", f"{theirs}.post_attention_layernorm.weight"))
            out += cls._attention_converters(block.mixer, f"{ours}.mixer", f"{theirs}.self_attn")
            out += cls._mlp_converters(block.mlp, f"{ours}.mlp", f"{theirs}.mlp")
            out.append(WeightConverter(f"multi_token_prediction.heads.{index}.final_norm.weight", f"model.mtp_norms.{index + 1}.weight"))
        return out


class DiffusionDreamHuggingfaceCheckpointHandler(Qwen2HuggingfaceCheckpointHandler):
    """Dream (masked-diffusion language model on the Qwen2 architecture): same tensors, its own modeling files."""

    format = DiffusionDreamCheckpointFormat
    architecture = "DreamModel"
    model_type = "Dream"

    @classmethod
    def _export_extra(cls, c, out):
        super()._export_extra(c, out)
        out["auto_map"] = {"AutoConfig": "configuration_dream.DreamConfig", "AutoModel": "modeling_dream.DreamModel"}

    @classmethod
    def get_extra_files(cls):
        from fast_llm_b200.external_models.diffusion_dream import configuration_dream, modeling_dream

        return [pathlib.Path(configuration_dream.__file__), pathlib.Path(modeling_dream.__file__)]


class DiffusionLlamaHuggingfaceCheckpointHandler(LlamaHuggingfaceCheckpointHandler):
    format = DiffusionLlamaCheckpointFormat
    architecture = "DiffusionLlamaModel"
    model_type = "diffusion_llama"

    @classmethod
    def _export_extra(cls, c, out):
        out["auto_map"] = {"AutoConfig": "configuration_diffusion_llama.DiffusionLlamaConfig", "AutoModel": "modeling_diffusion_llama.DiffusionLlamaModel"}

    @classmethod
    def get_extra_files(cls):
        from fast_llm_b200.external_models.diffusion_llama import configuration_diffusion_llama, modeling_diffusion_llama

        return [pathlib.Path(configuration_diffusion_llama.__file__), pathlib.Path(modeling_diffusion_llama.__file__)]


class AprielHybridSSMHuggingfaceCheckpointHandler(MistralHuggingfaceCheckpointHandler):
    """Apriel hybrid: a per-layer `hybrid_block_layout` of "t" (attention), "m2" (Mamba) and "gdn" (gated DeltaNet) blocks
    sharing one MLP / normalization config; Mamba sizes sit in `ssm_cfg` (`apriel.py:36-469`)."""

    format = AprielHybridSSMCheckpointFormat
    architecture = "AprielHybridSSMForCausalLM"
    model_type = "apriel_ssm_thinker_hybrid"
    layout_names = {"AttentionConfig": "t", "MambaConfig": "m2", "GatedDeltaNetConfig": "gdn"}

    @classmethod
    def _blocks(cls, c) -> list:
        return c.decoder.block_configs()

    @classmethod
    def _block(cls, base_model_config):
        blocks = cls._blocks(base_model_config)
        attention = [b for b in blocks if type(b.mixer).__name__ == "AttentionConfig"]
        return (attention or blocks)[0]

    @classmethod
    def export_config(cls, c) -> dict:
        blocks = cls._blocks(c)
        layout = [cls.layout_names[type(b.mixer).__name__] for b in blocks]
        if "t" in layout:
            out = super().export_config(c)
        else:  # no attention block to describe: borrow the shared parts from the first block
            first = blocks[0]
            out = {"model_type": cls.model_type, "architectures": [cls.architecture], "vocab_size": c.embeddings.vocab_size,
                   "hidden_size": c.hidden_size, "num_hidden_layers": len(blocks), "intermediate_size": first.mlp.intermediate_size,
                   "hidden_act": first.mlp.activation.hf_name, "rms_norm_eps": first.normalization.epsilon,
                   "tie_word_embeddings": c.tied_embedding_weight}
        out["num_hidden_layers"] = len(blocks)
        out["hybrid_block_layout"] = layout
        mamba = next((b.mixer for b in blocks if type(b.mixer).__name__ == "MambaConfig"), None)
        if mamba is not None:
            out["ssm_cfg"] = {"d_state": mamba.state_size, "d_inner": mamba.d_inner, "d_xb": mamba.d_xb, "dt_rank": mamba.dt_rank,
                              "bias": mamba.add_linear_biases, "repeat_kv_before_conv": mamba.repeat_kv_before_conv,
                              "conv_bias": cls._enabled(mamba.convolution_layer.bias, mamba.add_linear_biases),
                              "dt_proj_bias": cls._enabled(mamba.dt_layer.bias, mamba.add_linear_biases), "d_conv": mamba.convolution_layer.kernel_size}
        gdn = next((b.mixer for b in blocks if type(b.mixer).__name__ == "GatedDeltaNetConfig"), None)
        if gdn is not None:
            out["linear_attn_config"] = {"gdn_value_head_dim": gdn.value_head_dim, "gdn_key_head_dim": gdn.key_head_dim,
                                         "gdn_num_value_heads": gdn.value_heads, "gdn_num_key_heads": gdn.key_heads,
                                         "gdn_linear_conv_kernel_size": gdn.convolution_layer.kernel_size}
        out["auto_map"] = {"AutoConfig": "configuration_apriel_hybrid_ssm.AprielHybridSSMConfig",
                           "AutoModel": "modeling_apriel_hybrid_ssm.AprielHybridSSMModel",
                           "AutoModelForCausalLM": "modeling_apriel_hybrid_ssm.AprielHybridSSMForCausalLM"}
        return out

    @staticmethod
    def _enabled(bias_config, default: bool) -> bool:
        return default if bias_config.enabled is None else bias_config.enabled

    @classmethod
    def get_extra_files(cls):
        from fast_llm_b200.external_models.apriel_hybrid_ssm import configuration_apriel_hybrid_ssm, modeling_apriel_hybrid_ssm

        return [pathlib.Path(configuration_apriel_hybrid_ssm.__file__), pathlib.Path(modeling_apriel_hybrid_ssm.__file__)]

    @classmethod
    def import_config(cls, h: dict) -> dict:
        out = super().import_config(h)
        shared = out["decoder"]["block"]
        layout = h.get("hybrid_block_layout") or ["t"] * h["num_hidden_layers"]
        ssm = h.get("ssm_cfg", {})
        hidden = h["hidden_size"]
        d_inner = ssm.get("d_inner") or hidden * ssm.get("expand", 1)
        dt_rank = ssm.get("dt_rank", "auto")
        mixers = {
            "t": shared["mixer"],
            "m2": {"type": "mamba", "state_size": ssm.get("d_state", 16), "d_inner": d_inner, "d_xb": ssm.get("d_xb") or hidden,
                   "dt_rank": -(-hidden // 16) if dt_rank == "auto" else dt_rank, "add_linear_biases": ssm.get("bias", False),
                   "repeat_kv_before_conv": ssm.get("repeat_kv_before_conv", True),
                   "convolution_layer": {"kernel_size": ssm.get("d_conv", 4), "bias": {"enabled": ssm.get("conv_bias", True)}},
                   "dt_layer": {"bias": {"enabled": ssm.get("dt_proj_bias", True)}}},
        }
        linear = h.get("linear_attn_config", {})
        if linear:
            mixers["gdn"] = {"type": "gdn", "value_head_dim": linear["gdn_value_head_dim"], "key_head_dim": linear["gdn_key_head_dim"],
                             "value_heads": linear["gdn_num_value_heads"], "key_heads": linear["gdn_num_key_heads"],
                             "convolution_layer": {"kernel_size": linear.get("gdn_linear_conv_kernel_size", 4)}}
        names = list(dict.fromkeys(layout))
        out["decoder"] = {"type": "pattern", "num_blocks": len(layout), "pattern": layout,
                          "blocks": {name: {**shared, "mixer": mixers[name]} for name in names}}
        return out

    @classmethod
    def _mixer_converters(cls, mixer, ours: str, theirs: str) -> list[WeightConverter]:
        kind = type(mixer).__name__
        if kind == "AttentionConfig":
            return cls._attention_converters(mixer, ours, f"{theirs}.self_attn")
        theirs = f"{theirs}.mixer"
        if kind == "MambaConfig":
            bias = mixer.add_linear_biases
            out = []
            for name in ("in_proj", "dt_in_proj", "out_proj"):
                out += cls._linear(f"{ours}.{name}", f"{theirs}.{name}", bias)
            out += cls._linear(f"{ours}.dt_proj", f"{theirs}.dt_proj", cls._enabled(mixer.dt_layer.bias, bias))
            out += cls._linear(f"{ours}.convolution", f"{theirs}.conv1d", cls._enabled(mixer.convolution_layer.bias, bias))
            out += [WeightConverter(f"{ours}.A_log", f"{theirs}.A_log"), WeightConverter(f"{ours}.D", f"{theirs}.D")]
            return out
        if kind == "GatedDeltaNetConfig":
            out = []
            for name in ("in_proj_qkvz", "in_proj_ba", "out_proj"):
                out += cls._linear(f"{ours}.{name}", f"{theirs}.{name}", False)
            out += cls._linear(f"{ours}.convolution", f"{theirs}.conv1d", False)
            out += [WeightConverter(f"{ours}.A_log", f"{theirs}.A_log"), WeightConverter(f"{ours}.dt_bias", f"{theirs}.dt_bias"),
                    WeightConverter(f"{ours}.norm.weight", f"{theirs}.norm.weight")]
            return out
        raise NotImplementedError(f"No Apriel mapping for {kind}")

    @classmethod
    def get_weight_converters(cls, c) -> list[WeightConverter]:
        out = [WeightConverter("embeddings.word_embeddings_weight", "model.embed_tokens.weight")]
        for i, block in enumerate(cls._blocks(c)):
            ours, theirs = f"decoder.{i}", f"model.layers.{i}"
            out.append(WeightConverter(f"{ours}.norm_1.weight", f"{theirs}.input_layernorm.weight"))
            out.append(WeightConverter(f"{ours}.norm_2.weight", f"{theirs}.post_attention_layernorm.weight"))
            out += cls._mixer_converters(block.mixer, f"{ours}.mixer", theirs)
            out += cls._mlp_converters(block.mlp, f"{ours}.mlp", f"{theirs}.mlp")
        out.append(WeightConverter("head.final_norm.weight", "model.norm.weight"))
        out.append(IgnoreImportWeightConverter("lm_head.weight") if c.tied_embedding_weight else WeightConverter("head.output_weights", "lm_head.weight"))
        return out


class AutoGPTHuggingfaceCheckpointHandler(HuggingfaceStateDictCheckpointHandler):
    """Dispatches on `model_type` of config.json when loading; cannot be used for saving."""

    format = AutoGPTHuggingfaceCheckpointFormat
    handler_map = {"llama": LlamaHuggingfaceCheckpointHandler, "mistral": MistralHuggingfaceCheckpointHandler,
                   "qwen2": Qwen2HuggingfaceCheckpointHandler, "mixtral": MixtralHuggingfaceCheckpointHandler,
                   "mtp_llama": MTPLlamaHuggingfaceCheckpointHandler, "Dream": DiffusionDreamHuggingfaceCheckpointHandler,
                   "diffusion_llama": DiffusionLlamaHuggingfaceCheckpointHandler,
                   "apriel_ssm_thinker_hybrid": AprielHybridSSMHuggingfaceCheckpointHandler}

    def __new__(cls, model):
        raise TypeError("resolve the concrete handler with get_handler_class(path) first")

    @classmethod
    def resolve(cls, path) -> type[HuggingfaceStateDictCheckpointHandler]:
        model_type = json.loads((pathlib.Path(path) / "config.json").read_text())["model_type"]
        if model_type == "apriel2_text":
            from fast_llm_b200.models.gpt.conversion.apriel2 import Apriel2HuggingfaceCheckpointHandler

            return Apriel2HuggingfaceCheckpointHandler
        if model_type == "gemma4_text":
            from fast_llm_b200.models.gpt.conversion.gemma4 import Gemma4HuggingfaceCheckpointHandler

            return Gemma4HuggingfaceCheckpointHandler
        return cls.handler_map[model_type]

    @classmethod
    def load_metadata(cls, config):
        handler = cls.resolve(config.path)
        metadata = handler.load_metadata(config)
        return metadata

    @classmethod
    def get_model_config_class(cls):
        from fast_llm_b200.models.gpt.config import GPTModelConfig

        return GPTModelConfig


GPT_CHECKPOINT_FORMATS = (AutoGPTHuggingfaceCheckpointFormat, LlamaCheckpointFormat, Qwen2CheckpointFormat, MistralCheckpointFormat,
                          MixtralCheckpointFormat, MTPLlamaCheckpointFormat, DiffusionDreamCheckpointFormat, DiffusionLlamaCheckpointFormat,
                          AprielHybridSSMCheckpointFormat)
