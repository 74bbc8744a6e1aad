"""Apriel2 checkpoint surgery: configuration algebra, plans as data, and converted checkpoints that both the stand-alone
modelling code and this framework load (the subject of `fast_llm_external_models/tests/test_apriel2/test_compose_configs.py`,
`test_expr_plan.py`, `test_plan_execution.py` and `test_conversion_e2e.py` in the reference)."""

import copy
import json

import pytest
import torch

from fast_llm_b200.external_models.apriel2.conversion import (
    Concat, Init, Plan, Ref, Slice, apply_surgeries, compose_configs, compose_plans, convert_checkpoint, plan_surgery, strip_init_fields,
)
from tests.common import TINY_BASE_MODEL, build_trainer, tiny_trainer_config


def _state(heads=4, groups=2, size=16, blocks=2):
    return {
        "model_type": "apriel2_text", "hidden_size": 64, "vocab_size": 512, "tie_word_embeddings": False,
        "decoder": {"type": "fixed", "num_blocks": blocks, "block": {
            "mixer": {"type": "attention", "heads": heads, "head_groups": groups, "head_size": size, "add_linear_biases": False,
                      "rotary": {"type": "mistral_1d", "theta": 10000.0}},
            "mlp": {"type": "mlp", "intermediate_size": 128, "gated": True, "activation": "silu", "add_linear_biases": False},
            "normalization": {"type": "rms_norm", "epsilon": 1e-5}}},
        "head": {"normalization": {"type": "rms_norm", "epsilon": 1e-5}},
    }


def _mixer_surgery(mixer):
    return {"decoder": {"block": {"mixer": mixer}}}


def test_configuration_algebra():
    state = _state()
    # replacing the mixer type derives the new mixer's geometry from the attention it replaces and keeps the init mark
    transition = compose_configs(state, _mixer_surgery({"type": "gdn", "init": "random", "convolution_layer": {"kernel_size": 3}}))
    mixer = transition["decoder"]["block"]["mixer"]
    assert (mixer["value_heads"], mixer["key_heads"], mixer["key_head_dim"], mixer["value_head_dim"]) == (4, 2, 16, 16)
    assert mixer["init"] == "random" and "heads" not in mixer and transition["decoder"]["block"]["mlp"] == state["decoder"]["block"]["mlp"]
    target = strip_init_fields(transition)
    assert "init" not in json.dumps(target) and target["decoder"]["block"]["mixer"]["type"] == "gdn"
    assert state["decoder"]["block"]["mixer"]["type"] == "attention"  # inputs are not modified
    # Mamba: inner width = all heads, B / x width = the key-value heads
    mamba = compose_configs(state, _mixer_surgery({"type": "mamba"}))["decoder"]["block"]["mixer"]
    assert (mamba["d_inner"], mamba["d_xb"], mamba["dt_rank"], mamba["init"]) == (64, 32, 4, "transfer")
    # wrapping into a stochastic mixer: the sub-mixer that names no type is the old attention, unchanged
    wrap = _mixer_surgery({"type": "stochastic", "main_mixer_name": "attention",
                           "mixers": {"attention": {}, "kda": {"type": "kda", "init": "transfer"}}})
    wrapped = compose_configs(state, wrap)["decoder"]["block"]["mixer"]
    assert strip_init_fields(wrapped["mixers"]["attention"]) == state["decoder"]["block"]["mixer"]
    assert (wrapped["mixers"]["kda"]["heads"], wrapped["mixers"]["kda"]["head_dim"]) == (4, 16)
    # additive surgeries: applying them in turn equals applying their merge; surgeries merge among themselves
    first, second = {"decoder": {"block": {"mlp": {"activation": "gelu"}}}}, {"decoder": {"block": {"mixer": {"window_size": 64}}}, "head": {"x": 1}}
    in_turn = compose_configs(compose_configs(state, first), second)
    assert in_turn == compose_configs(state, compose_configs(first, second))
    assert in_turn["decoder"]["block"]["mixer"]["window_size"] == 64 and in_turn["decoder"]["block"]["mlp"]["activation"] == "gelu"
    # a fixed decoder becomes a pattern whose named blocks are described relative to the one old block
    pattern = compose_configs(state, {"decoder": {"type": "pattern", "pattern": ["a", "m"], "blocks": {"a": {}, "m": {"mixer": {"type": "mamba"}}}}})
    assert pattern["decoder"]["blocks"]["a"] == state["decoder"]["block"] and pattern["decoder"]["blocks"]["m"]["mixer"]["type"] == "mamba"
    assert pattern["decoder"]["num_blocks"] == 2
    # a later surgery on the stochastic mixer adds a sub-mixer relative to the main one and leaves the others alone
    more = compose_configs(strip_init_fields(compose_configs(state, wrap)), _mixer_surgery({"mixers": {"gdn": {"type": "gdn", "init": "random"}}}))
    assert set(more["decoder"]["block"]["mixer"]["mixers"]) == {"attention", "kda", "gdn"}
    assert "init" not in more["decoder"]["block"]["mixer"]["mixers"]["kda"]


def test_expressions_are_data():
    source = {"a": torch.arange(12.0).reshape(4, 3), "b": torch.ones(2, 3)}
    expr = Concat([Slice(Ref("a"), 0, 1, 3), Ref("b"), Init((1, 3), "normal", "fresh", 0.5)], 0)
    value = expr.evaluate(source, seed=7)
    assert value.shape == (5, 3) and torch.equal(value[:2], source["a"][1:3]) and torch.equal(value[2:4], source["b"])
    assert torch.equal(value[4], expr.evaluate(source, seed=7)[4]) and not torch.equal(value[4], expr.evaluate(source, seed=8)[4])
    assert expr.references() == {"a", "b"}
    again = Plan.from_dict(json.loads(json.dumps(Plan({"t": expr}).to_dict())))
    assert torch.equal(again["t"].evaluate(source, seed=7), value)
    # composition by substitution: `then` over the outputs of `first`, as one plan over the first plan's sources
    first = Plan({"x": Slice(Ref("a"), 0, 0, 2), "y": Concat([Ref("b"), Ref("b")], 0)})
    then = Plan({"z": Concat([Ref("y"), Ref("x")], 0), "w": Init((2,), "ones", "w")})
    fused = compose_plans(first, then)
    assert fused.source_keys() == {"a", "b"}
    staged = then.execute(first.execute(source, 3), 3)
    direct = fused.execute(source, 3)
    assert all(torch.equal(staged[name], direct[name]) for name in staged)


def _export(tmp_path, base_model=None):
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig

    trainer, _ = build_trainer(tiny_trainer_config({("model", "base_model"): base_model or copy.deepcopy(TINY_BASE_MODEL)}))
    path = tmp_path / "source"
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="apriel2_text"))
    return path


def _load(path):
    from fast_llm_b200.external_models.apriel2.modeling_apriel2 import Apriel2ForCausalLM

    model, info = Apriel2ForCausalLM.from_pretrained(str(path), torch_dtype=torch.float32, output_loading_info=True)
    assert not info["missing_keys"] and not info["unexpected_keys"], info
    return model.eval()


def test_surgery_keeps_what_it_does_not_touch_and_initialises_from_attention(tmp_path):
    source_path = _export(tmp_path)
    source_state = json.loads((source_path / "config.json").read_text())
    # identity: every tensor is a reference
    state, plan = apply_surgeries(source_state, [])
    assert all(isinstance(e, Ref) and e.key == name for name, e in plan.items()) and state == strip_init_fields(source_state)

    # 1. wrap the attention into a stochastic mixer beside a delta-net that starts from it; the main mixer stays attention
    wrap = _mixer_surgery({"type": "stochastic", "main_mixer_name": "attention",
                           "mixers": {"attention": {}, "gdn": {"type": "gdn", "init": "transfer", "convolution_layer": {"kernel_size": 3}}}})
    # 2. then turn the second block (only) into Mamba, initialised from the attention inside the stochastic mixer
    to_pattern = {"decoder": {"type": "pattern", "pattern": ["keep", "mamba"], "blocks": {"keep": {}, "mamba": {"mixer": {"type": "mamba", "init": "transfer"}}}}}
    convert_checkpoint(source_path, tmp_path / "wrapped", [wrap], seed=1)
    convert_checkpoint(source_path, tmp_path / "both", [wrap, to_pattern], seed=1)
    original, wrapped, both = _load(source_path), _load(tmp_path / "wrapped"), _load(tmp_path / "both")
    tokens = torch.randint(0, 512, (1, 20))
    with torch.no_grad():
        reference = original(input_ids=tokens).logits
        # the main mixer is the untouched attention: same function
        torch.testing.assert_close(wrapped(input_ids=tokens).logits, reference, rtol=1e-5, atol=1e-5)
        assert torch.isfinite(both(input_ids=tokens).logits).all()
    old, new = original.state_dict(), wrapped.state_dict()
    prefix = "model.decoder.blocks.0.mixer"
    heads, groups, size = 4, 2, 16
    qkvz = new[f"{prefix}.mixers.gdn.in_proj_qkvz.weight"]
    # [q: first head of every group | k | v: every head gets its group's rows | z: new]
    assert torch.equal(qkvz[:size], old[f"{prefix}.q_proj.weight"][:size])
    assert torch.equal(qkvz[size : 2 * size], old[f"{prefix}.q_proj.weight"][2 * size : 3 * size])
    assert torch.equal(qkvz[groups * size : 2 * groups * size], old[f"{prefix}.k_proj.weight"])
    v = qkvz[2 * groups * size : 2 * groups * size + heads * size]
    assert torch.equal(v[:size], old[f"{prefix}.v_proj.weight"][:size]) and torch.equal(v[size : 2 * size], old[f"{prefix}.v_proj.weight"][:size])
    assert torch.equal(v[3 * size :], old[f"{prefix}.v_proj.weight"][size:])
    assert torch.equal(new[f"{prefix}.mixers.gdn.out_proj.weight"], old[f"{prefix}.o_proj.weight"])
    assert torch.equal(new[f"{prefix}.mixers.gdn.norm.weight"], torch.ones(size))
    # the Mamba of block 1: [z: new | x <- value | B <- key | C <- query], output projection kept
    mamba = both.state_dict()
    prefix1 = "model.decoder.blocks.1.mixer"
    in_proj = mamba[f"{prefix1}.in_proj.weight"]
    assert torch.equal(in_proj[64:96], old[f"{prefix1}.v_proj.weight"]) and torch.equal(in_proj[96:128], old[f"{prefix1}.k_proj.weight"])
    assert torch.equal(in_proj[128:], old[f"{prefix1}.q_proj.weight"]) and torch.equal(mamba[f"{prefix1}.out_proj.weight"], old[f"{prefix1}.o_proj.weight"])
    assert (mamba[f"{prefix1}.A_log"] >= 0).all() and (mamba[f"{prefix1}.A_log"] <= 2.78).all()
    # block 0 of the chained conversion is block 0 of the first one: the second surgery did not draw new values for it
    assert torch.equal(mamba[f"{prefix}.mixers.gdn.in_proj_qkvz.weight"], qkvz)
    # the chain ran as one plan over the source tensors, and the plan is written next to the checkpoint
    written = Plan.from_dict(json.loads((tmp_path / "both" / "surgery_plan.json").read_text()))
    assert written.source_keys() <= set(old) and "Init" in repr(written[f"{prefix1}.in_proj.weight"])

    # this framework imports the converted checkpoint and computes the same logits as the stand-alone code
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.engine.inference.runner import InferenceRunner
    from fast_llm_b200.models.gpt.model import GPTModel

    runner = InferenceRunner(GPTModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / "both", format="apriel2_text"), use_cpu=True))
    runner.setup()
    with torch.no_grad():
        torch.testing.assert_close(runner.forward_tokens(tokens[0]), both(input_ids=tokens).logits[0], rtol=2e-4, atol=2e-4)


def test_random_init_and_mismatched_geometry_fall_back_to_new_values():
    state = _state()
    transition = compose_configs(state, _mixer_surgery({"type": "kda", "init": "random"}))
    plan = plan_surgery(state, transition)
    mixer = {n: e for n, e in plan.items() if ".blocks.0.mixer." in n}
    assert mixer and all(isinstance(e, Init) for e in mixer.values())
    assert isinstance(plan["model.embed_tokens.weight"], Ref) and isinstance(plan["model.decoder.blocks.1.mlp.up_proj.weight"], Ref)
    # a Mamba whose width does not match the attention cannot take its rows
    narrow = plan_surgery(state, compose_configs(state, _mixer_surgery({"type": "mamba", "d_inner": 32, "init": "transfer"})))
    assert isinstance(narrow["model.decoder.blocks.0.mixer.in_proj.weight"], Init)
    with pytest.raises(KeyError):
        Plan({"t": Ref("absent")}).execute({}, 0)
