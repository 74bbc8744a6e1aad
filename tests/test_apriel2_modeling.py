"""The stand-alone Apriel2 modelling code (`external_models/apriel2/modeling_apriel2.py`): its generation cache.

Every mixer kind keeps what it needs of the prefix (keys and values, convolution inputs, recurrent state); a pass over new tokens
with the cache must give the logits of one pass over the whole sequence.
"""

import pytest
import torch

from fast_llm_b200.external_models.apriel2.configuration_apriel2 import Apriel2TextConfig
from fast_llm_b200.external_models.apriel2.modeling_apriel2 import Apriel2Cache, Apriel2ForCausalLM

_MLP = {"type": "mlp", "intermediate_size": 48, "gated": True, "activation": "silu", "add_linear_biases": False}
_NORM = {"type": "rms_norm", "epsilon": 1e-5}
_MIXERS = {
    "attention": {"type": "attention", "heads": 4, "head_groups": 2, "head_size": 8, "add_linear_biases": False,
                  "rotary": {"type": "mistral_1d", "theta": 10000.0}},
    "window": {"type": "attention", "heads": 4, "head_groups": 2, "head_size": 8, "add_linear_biases": True, "window_size": 5,
               "rotary": {"type": "llama3", "theta": 10000.0, "scale_factor": 8.0, "low_frequency_factor": 1.0, "high_frequency_factor": 4.0,
                          "original_context_length": 64}},
    "mamba": {"type": "mamba", "d_inner": 32, "d_xb": 16, "state_size": 8, "dt_rank": 4, "d_conv": 4, "conv_bias": True, "dt_proj_bias": True},
    "mamba_late_repeat": {"type": "mamba", "d_inner": 32, "d_xb": 16, "state_size": 8, "dt_rank": 4, "d_conv": 3, "repeat_kv_before_conv": False},
    "gdn": {"type": "gdn", "value_heads": 4, "key_heads": 2, "key_head_dim": 8, "value_head_dim": 8, "convolution_layer": {"kernel_size": 3}},
    "kda": {"type": "kda", "heads": 2, "head_dim": 8, "convolution_layer": {"kernel_size": 4}},
}
_MIXERS["stochastic"] = {"type": "stochastic", "mixers": {"a": _MIXERS["attention"], "g": _MIXERS["gdn"]}, "main_mixer_name": "g"}


def _model(names):
    torch.manual_seed(0)
    blocks = {name: {"mixer": _MIXERS[name], "mlp": _MLP, "normalization": _NORM} for name in names}
    config = Apriel2TextConfig(hidden_size=32, vocab_size=96, head={"normalization": _NORM},
                               decoder={"type": "pattern", "num_blocks": len(names), "pattern": list(names), "blocks": blocks})
    model = Apriel2ForCausalLM(config).eval()
    with torch.no_grad():
        for name, parameter in model.named_parameters():  # leave no parameter at a value that hides a missing state
            if name.endswith(("A_log", "dt_bias", "D")) or "conv" in name:
                parameter.copy_(torch.randn_like(parameter) * 0.5)
    return model


@pytest.mark.parametrize("mixer", list(_MIXERS))
def test_cached_passes_match_one_pass(mixer):
    model = _model([mixer, mixer])
    tokens = torch.randint(0, 96, (2, 19))
    with torch.no_grad():
        full = model(input_ids=tokens).logits
        out = model(input_ids=tokens[:, :7], use_cache=True)
        cache, pieces = out.past_key_values, [out.logits]
        assert isinstance(cache, Apriel2Cache) and cache.get_seq_length() == 7
        for begin, end in ((7, 8), (8, 9), (9, 14), (14, 19)):  # single tokens and longer pieces
            out = model(input_ids=tokens[:, begin:end], past_key_values=cache, use_cache=True)
            pieces.append(out.logits)
            assert cache.get_seq_length() == end
    torch.testing.assert_close(torch.cat(pieces, dim=1), full, rtol=1e-4, atol=1e-5)
    if mixer == "window":  # a sliding window keeps window - 1 keys, however long the prefix
        assert all(layer["k"].shape[1] == 4 for layer in cache.layers)


def test_generate_uses_the_cache_and_matches_generation_without():
    model = _model(["attention", "mamba", "gdn", "kda", "window", "stochastic"])
    prompt = torch.randint(0, 96, (2, 6))
    calls = []
    hook = model.model.register_forward_pre_hook(lambda module, args, kwargs: calls.append(kwargs["input_ids"].shape[1]), with_kwargs=True)
    with torch.no_grad():
        cached = model.generate(prompt, max_new_tokens=8, do_sample=False)
    hook.remove()
    assert calls == [6] + [1] * 7, calls  # the prompt once, then one token per step
    with torch.no_grad():
        plain = model.generate(prompt, max_new_tokens=8, do_sample=False, use_cache=False)
        beams = model.generate(prompt, max_new_tokens=6, do_sample=False, num_beams=3)
        beams_plain = model.generate(prompt, max_new_tokens=6, do_sample=False, num_beams=3, use_cache=False)
    assert torch.equal(cached, plain)
    assert torch.equal(beams, beams_plain)  # beam search reorders the rows of every cached tensor


def test_hybrid_ssm_model_cache():
    """The Apriel hybrid SSM modelling code keeps the same kind of cache (attention with a sliding window, Mamba, gated DeltaNet)."""
    from fast_llm_b200.external_models.apriel_hybrid_ssm.configuration_apriel_hybrid_ssm import AprielHybridSSMConfig
    from fast_llm_b200.external_models.apriel_hybrid_ssm.modeling_apriel_hybrid_ssm import AprielHybridSSMForCausalLM, HybridCache

    torch.manual_seed(0)
    config = AprielHybridSSMConfig(
        hidden_size=32, intermediate_size=48, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=8, vocab_size=96,
        sliding_window=6, hybrid_block_layout=["t", "m2", "gdn"], ssm_cfg={"d_state": 8, "d_inner": 32, "d_xb": 16, "dt_rank": 4, "d_conv": 4},
        linear_attn_config={"gdn_num_value_heads": 4, "gdn_num_key_heads": 2, "gdn_key_head_dim": 8, "gdn_value_head_dim": 8,
                            "gdn_linear_conv_kernel_size": 3})
    model = AprielHybridSSMForCausalLM(config).eval()
    with torch.no_grad():
        for name, parameter in model.named_parameters():
            if name.endswith(("A_log", "dt_bias", "D")) or "conv" in name:
                parameter.copy_(torch.randn_like(parameter) * 0.5)
    tokens = torch.randint(0, 96, (2, 17))
    with torch.no_grad():
        full = model(input_ids=tokens).logits
        out = model(input_ids=tokens[:, :9], use_cache=True)
        cache, pieces = out.past_key_values, [out.logits]
        assert isinstance(cache, HybridCache)
        for begin, end in ((9, 10), (10, 11), (11, 17)):
            pieces.append(model(input_ids=tokens[:, begin:end], past_key_values=cache, use_cache=True).logits)
        assert cache.get_seq_length() == 17 and cache.layers[0]["k"].shape[1] == 5
        torch.testing.assert_close(torch.cat(pieces, dim=1), full, rtol=1e-4, atol=1e-5)
        cached = model.generate(tokens[:, :5], max_new_tokens=6, do_sample=False)
        plain = model.generate(tokens[:, :5], max_new_tokens=6, do_sample=False, use_cache=False)
    assert torch.equal(cached, plain)
