"""Gemma 4 text format (`model_type: gemma4_text`).

The decoder is a pattern of two block kinds, `sliding_attention` (windowed, default rotary, `head_dim`) and
`full_attention` (proportional rotary over part of `global_head_dim`, optionally keys reused as values), described by ONE
flat Hugging Face config.  Every block has query / key RMS norms and a weight-free value norm, scores are not scaled
(`softmax_scale_power = 0`), mixer and MLP outputs are normalized again before the residual add, and the block output is
multiplied by a frozen scalar (`layer_scalar`).  With `enable_moe_block` the MLP is a dense branch plus a routed
mixture of experts, each with its own pre / post norm; expert weights are stored batched
(`experts.gate_up_proj [E, 2 I, H]`, `experts.down_proj [E, H, I]`).  Embeddings are scaled by sqrt(hidden_size), logits
optionally soft-capped.  Parity: `fast_llm/models/gpt/conversion/gemma4.py:52-738`.
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

_SLIDING, _FULL = "sliding_attention", "full_attention"


class Gemma4CheckpointFormat(GPTHuggingfaceCheckpointFormat):
    name: typing.ClassVar[str] = "gemma4"

    @classmethod
    def get_handler_class(cls):
        return Gemma4HuggingfaceCheckpointHandler


class BatchedExpertLayer1Converter(WeightConverter):
    """layer_1 [experts * 2 * intermediate, hidden] <-> experts.gate_up_proj [experts, 2 * intermediate, hidden]."""

    def export_weight(self, weight):
        return (weight[0].reshape(self._config, -1, weight[0].shape[-1]),)

    def import_weight(self, weight):
        w = weight[0][:]
        return (w.reshape(-1, w.shape[-1]),)


class BatchedExpertLayer2Converter(WeightConverter):
    """layer_2 [experts * intermediate, hidden] <-> experts.down_proj [experts, hidden, intermediate]."""

    def export_weight(self, weight):
        w = weight[0]
        return (w.reshape(self._config, -1, w.shape[-1]).permute(0, 2, 1).contiguous(),)

    def import_weight(self, weight):
        w = weight[0][:]
        return (w.permute(0, 2, 1).reshape(-1, w.shape[1]).contiguous(),)


def _is_hybrid(mlp) -> bool:
    return type(mlp).__name__ == "HybridMoEMLPConfig"


class Gemma4HuggingfaceCheckpointHandler(HuggingfaceStateDictCheckpointHandler):
    format = Gemma4CheckpointFormat
    architecture = "Gemma4ForCausalLM"
    model_type = "gemma4_text"

    @classmethod
    def get_model_config_class(cls):
        from fast_llm_b200.models.gpt.config import GPTModelConfig

        return GPTModelConfig

    # ------------------------------------------------------------------ export
    @classmethod
    def _check_dense(cls, mlp) -> None:
        Assert.eq(type(mlp).__name__, "MLPConfig")
        assert mlp.gated and not mlp.add_linear_biases, "Gemma 4 MLPs are gated and have no biases"

    @classmethod
    def export_config(cls, c) -> dict:
        decoder = c.decoder
        Assert.eq(type(decoder).__name__, "PatternBlockSequenceConfig")
        sliding, full = decoder.blocks[_SLIDING], decoder.blocks[_FULL]
        s, f = sliding.mixer, full.mixer
        for mixer in (s, f):
            Assert.eq(type(mixer).__name__, "AttentionConfig")
            assert not mixer.add_linear_biases and mixer.softmax_scale_power == 0
            Assert.eq(type(mixer.query_norm).__name__, "RMSNormalizationConfig")
            Assert.eq(type(mixer.key_norm).__name__, "RMSNormalizationConfig")
            Assert.eq(type(mixer.value_norm).__name__, "FixedRMSNormConfig")
        Assert.eq(type(s.rotary).__name__, "DefaultRotaryConfig")
        Assert.eq(type(f.rotary).__name__, "ProportionalRotaryConfig")
        Assert.eq(type(sliding.normalization).__name__, "RMSNormalizationConfig")
        Assert.eq(c.embeddings.embedding_scale, c.hidden_size**0.5)
        hybrid = _is_hybrid(sliding.mlp)
        Assert.eq(_is_hybrid(full.mlp), hybrid)
        out = {
            "model_type": cls.model_type, "architectures": [cls.architecture],
            "vocab_size": c.embeddings.vocab_size, "hidden_size": c.hidden_size, "tie_word_embeddings": c.tied_embedding_weight,
            "num_hidden_layers": decoder.num_blocks, "layer_types": list(decoder.expanded_pattern),
            "num_attention_heads": s.heads, "num_key_value_heads": s.head_groups, "head_dim": s.head_size, "global_head_dim": f.head_size,
            "num_global_key_value_heads": None if f.head_groups == s.head_groups else f.head_groups,
            "attention_bias": False, "attention_dropout": s.dropout, "sliding_window": s.window_size, "rms_norm_eps": sliding.normalization.epsilon,
            "attention_k_eq_v": f.shared_key_value,
            "rope_parameters": {_SLIDING: {"rope_type": "default", "rope_theta": s.rotary.theta},
                                _FULL: {"rope_type": "proportional", "rope_theta": f.rotary.theta, "partial_rotary_factor": f.rotary.partial_rotary_factor}},
            "enable_moe_block": hybrid,
            # features of the Hugging Face model that this framework does not have: switched off in what we export
            "hidden_size_per_layer_input": 0, "num_kv_shared_layers": 0, "use_double_wide_mlp": False, "use_bidirectional_attention": None,
        }
        dense = sliding.mlp.dense if hybrid else sliding.mlp
        cls._check_dense(dense)
        out.update({"intermediate_size": dense.intermediate_size, "hidden_activation": dense.activation.hf_name})
        if hybrid:
            routed = sliding.mlp.routed
            assert routed.gated and not routed.add_linear_biases
            Assert.eq(type(routed.router_normalization).__name__, "FixedRMSNormConfig")
            assert routed.router_scale.enabled and routed.router_per_expert_scale.enabled
            Assert.eq(routed.router_input_scale, c.hidden_size**-0.5)
            out.update({"num_experts": routed.experts, "top_k_experts": routed.experts_per_token, "moe_intermediate_size": routed.intermediate_size})
        if c.head.final_logit_softcap is not None:
            out["final_logit_softcapping"] = c.head.final_logit_softcap
        return out

    # ------------------------------------------------------------------ import
    @classmethod
    def _import_attention(cls, h: dict, sliding: bool) -> dict:
        eps = h["rms_norm_eps"]
        if sliding:
            rope = h["rope_parameters"][_SLIDING]
            Assert.eq(rope.get("rope_type", "default"), "default")
            out = {"rotary": {"type": "default", "theta": rope["rope_theta"]}, "head_size": h["head_dim"], "head_groups": h["num_key_value_heads"],
                   "window_size": h["sliding_window"]}
        else:
            rope = h["rope_parameters"][_FULL]
            Assert.eq(rope.get("rope_type", "proportional"), "proportional")
            groups = h.get("num_global_key_value_heads")
            out = {"rotary": {"type": "proportional", "theta": rope["rope_theta"], "partial_rotary_factor": rope["partial_rotary_factor"]},
                   "head_size": h["global_head_dim"], "head_groups": h["num_key_value_heads"] if groups is None else groups}
            if h.get("attention_k_eq_v", False):
                out["shared_key_value"] = True
        out.update({"type": "attention", "heads": h["num_attention_heads"], "add_linear_biases": False, "dropout": h.get("attention_dropout", 0.0),
                    "softmax_scale_power": 0, "query_norm": {"type": "rms_norm", "epsilon": eps}, "key_norm": {"type": "rms_norm", "epsilon": eps},
                    "value_norm": {"type": "fixed_rms_norm", "epsilon": eps}})
        return out

    @classmethod
    def _import_block(cls, h: dict, sliding: bool) -> dict:
        eps = h["rms_norm_eps"]
        norm = lambda: {"type": "rms_norm", "epsilon": eps}  # noqa: E731
        activation = ActivationType.from_hf_name(h["hidden_activation"]).value
        dense = {"type": "mlp", "intermediate_size": h["intermediate_size"], "add_linear_biases": False, "activation": activation, "gated": True}
        out = {"type": "decoder", "mixer": cls._import_attention(h, sliding), "normalization": norm(), "post_mixer_normalization": norm(),
               "post_mlp_normalization": norm(), "output_scale": {"enabled": True, "lr_scale": 0}}  # `layer_scalar` is a buffer there: frozen here
        if h.get("enable_moe_block"):
            routed = {"type": "moe", "intermediate_size": h["moe_intermediate_size"], "add_linear_biases": False, "activation": activation, "gated": True,
                      "experts": h["num_experts"], "experts_per_token": h["top_k_experts"], "router_normalization": {"type": "fixed_rms_norm", "epsilon": eps},
                      "router_scale": {"enabled": True}, "router_input_scale": h["hidden_size"] ** -0.5, "router_per_expert_scale": {"enabled": True},
                      "pre_norm": norm(), "post_norm": norm()}
            out["mlp"] = {"type": "hybrid_moe", "dense": {**dense, "pre_norm": norm(), "post_norm": norm()}, "routed": routed}
            out["pre_mlp_normalization"] = {"type": "none"}
        else:
            out["mlp"] = dense
            out["pre_mlp_normalization"] = norm()
        return out

    @classmethod
    def import_config(cls, h: dict) -> dict:
        if h.get("use_bidirectional_attention") == "all":
            raise NotImplementedError("Gemma 4 with bidirectional text attention is not supported")
        # features of the Hugging Face model that have no counterpart here: a checkpoint that uses one is refused, not
        # loaded as a different model
        for key, off in (("attention_bias", (False, None)), ("hidden_size_per_layer_input", (0, None)), ("num_kv_shared_layers", (0, None)),
                         ("use_double_wide_mlp", (False, None))):
            if h.get(key) not in off:
                raise NotImplementedError(f"Gemma 4 checkpoints with {key}={h.get(key)!r} are not supported")
        layer_types = list(h["layer_types"])
        head = {"normalization": {"type": "rms_norm", "epsilon": h["rms_norm_eps"]}}
        if h.get("final_logit_softcapping") is not None:
            head["final_logit_softcap"] = h["final_logit_softcapping"]
        return {
            "embeddings": {"vocab_size": h["vocab_size"], "embedding_scale": h["hidden_size"] ** 0.5},
            "decoder": {"type": "pattern", "num_blocks": h["num_hidden_layers"], "pattern": layer_types,
                        "blocks": {kind: cls._import_block(h, kind == _SLIDING) for kind in dict.fromkeys(layer_types)}},
            "head": head, "hidden_size": h["hidden_size"], "tied_embedding_weight": bool(h.get("tie_word_embeddings", True)),
        }

    # ------------------------------------------------------------------ weights
    @classmethod
    def _dense_weights(cls, ours: str, theirs: str) -> list[WeightConverter]:
        return [SplitWeightConverter(f"{ours}.layer_1.weight", (f"{theirs}.gate_proj.weight", f"{theirs}.up_proj.weight")),
                TransposeWeightConverter(f"{ours}.layer_2.weight", f"{theirs}.down_proj.weight")]

    @classmethod
    def _block_weights(cls, block, ours: str, theirs: str) -> list[WeightConverter]:
        mixer = block.mixer
        rename = lambda a, b: WeightConverter(f"{ours}.{a}", f"{theirs}.{b}")  # noqa: E731
        out = [rename("norm_1.weight", "input_layernorm.weight"), rename("mixer.query.weight", "self_attn.q_proj.weight"),
               rename("mixer.dense.weight", "self_attn.o_proj.weight")]
        if mixer.shared_key_value:  # one projection serves keys and values
            out.append(rename("mixer.key_value.weight", "self_attn.k_proj.weight"))
        else:
            out.append(SplitWeightConverter(f"{ours}.mixer.key_value.weight", (f"{theirs}.self_attn.k_proj.weight", f"{theirs}.self_attn.v_proj.weight")))
        if mixer.query_norm is not None:
            out.append(rename("mixer.query_norm.weight", "self_attn.q_norm.weight"))
        if mixer.key_norm is not None:
            out.append(rename("mixer.key_norm.weight", "self_attn.k_norm.weight"))
        out += [rename("post_mixer_norm.weight", "post_attention_layernorm.weight"), rename("post_mlp_norm.weight", "post_feedforward_layernorm.weight"),
                rename("output_scale", "layer_scalar")]
        if _is_hybrid(block.mlp):
            experts = block.mlp.routed.experts
            out += cls._dense_weights(f"{ours}.mlp.dense", f"{theirs}.mlp")
            out += [rename("mlp.dense.pre_norm.weight", "pre_feedforward_layernorm.weight"),
                    rename("mlp.dense.post_norm.weight", "post_feedforward_layernorm_1.weight"),
                    rename("mlp.routed.pre_norm.weight", "pre_feedforward_layernorm_2.weight"),
                    rename("mlp.routed.post_norm.weight", "post_feedforward_layernorm_2.weight"),
                    rename("mlp.routed.router.weight", "router.proj.weight"), rename("mlp.routed.router_scale", "router.scale"),
                    rename("mlp.routed.router_per_expert_scale", "router.per_expert_scale"),
                    BatchedExpertLayer1Converter(f"{ours}.mlp.routed.layer_1.weight", f"{theirs}.experts.gate_up_proj", experts),
                    BatchedExpertLayer2Converter(f"{ours}.mlp.routed.layer_2.weight", f"{theirs}.experts.down_proj", experts)]
        else:
            out.append(rename("norm_2.weight", "pre_feedforward_layernorm.weight"))
            out += cls._dense_weights(f"{ours}.mlp", f"{theirs}.mlp")
        return out

    @classmethod
    def get_weight_converters(cls, c) -> list[WeightConverter]:
        out = [WeightConverter("embeddings.word_embeddings_weight", "model.embed_tokens.weight")]
        for i, block in enumerate(c.decoder.block_configs()):
            out += cls._block_weights(block, f"decoder.{i}", f"model.layers.{i}")
        out.append(WeightConverter("head.final_norm.weight", "model.norm.weight"))
        out.append(IgnoreImportWeightConverter("lm_head.weight") if c.tied_embedding_weight else WeightConverter("head.output_weights", "lm_head.weight"))
        return out
