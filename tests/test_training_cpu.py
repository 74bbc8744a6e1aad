"""End-to-end training on CPU: loss goes down, schedules are equivalent, checkpoints resume bit-exactly,
formats round-trip and match Hugging Face transformers numerically."""

import copy
import json
import pathlib

import pytest
import torch

from tests.common import build_trainer, tiny_trainer_config, train_steps


def test_loss_decreases():
    trainer, _ = build_trainer(tiny_trainer_config({("optimizer", "learning_rate", "base"): 3e-3}))
    losses = train_steps(trainer, 8)
    assert all(l == l for l in losses)
    assert losses[0] > 6.0  # ~ln(512)
    assert losses[-1] < losses[0] - 0.02


@pytest.mark.parametrize("schedule", [{"depth_first_micro_batches": 4}, {"breadth_first_micro_batches": 4},
                                      {"depth_first_micro_batches": 2, "breadth_first_micro_batches": 2}])
def test_micro_batch_schedules_are_equivalent(schedule):
    """Gradient accumulation order must not matter: df4 == bf4 == df2 x bf2 (same 4 micro-batches per step)."""
    base, _ = build_trainer(tiny_trainer_config({("schedule", "depth_first_micro_batches"): 4}))
    ref = train_steps(base, 2)
    other, _ = build_trainer(tiny_trainer_config({("schedule", k): v for k, v in schedule.items()}))
    got = train_steps(other, 2)
    assert got == pytest.approx(ref, rel=1e-5)
    torch.testing.assert_close(other.multi_stage.get_shard("weights"), base.multi_stage.get_shard("weights"), rtol=1e-4, atol=1e-6)


def test_zero_stages_are_equivalent():
    ref_trainer, _ = build_trainer(tiny_trainer_config({("schedule", "depth_first_micro_batches"): 2}))
    ref = train_steps(ref_trainer, 2)
    for stage in (2, 3):
        t, _ = build_trainer(tiny_trainer_config({("schedule", "depth_first_micro_batches"): 2, ("model", "multi_stage", "zero_stage"): stage}))
        assert train_steps(t, 2) == pytest.approx(ref, rel=1e-5)
        torch.testing.assert_close(t.multi_stage.get_shard("weights"), ref_trainer.multi_stage.get_shard("weights"), rtol=1e-4, atol=1e-6)


def test_micro_sequences_match_whole_sequence():
    whole, _ = build_trainer(tiny_trainer_config())
    ref = train_steps(whole, 2)
    split, _ = build_trainer(tiny_trainer_config({("schedule", "micro_batch_splits"): 4}))
    assert train_steps(split, 2) == pytest.approx(ref, rel=2e-4)
    torch.testing.assert_close(split.multi_stage.get_shard("weights"), whole.multi_stage.get_shard("weights"), rtol=2e-3, atol=2e-5)


def test_layers_per_stage_does_not_change_results():
    a, _ = build_trainer(tiny_trainer_config())
    b, _ = build_trainer(tiny_trainer_config({("model", "multi_stage", "layers_per_stage"): 2}))
    assert len(b.multi_stage.stages) < len(a.multi_stage.stages)
    assert train_steps(b, 2) == pytest.approx(train_steps(a, 2), rel=1e-5)


def test_cross_entropy_splits():
    a, _ = build_trainer(tiny_trainer_config())
    b, _ = build_trainer(tiny_trainer_config({("model", "base_model", "head", "cross_entropy_splits"): 4}))
    assert train_steps(b, 2) == pytest.approx(train_steps(a, 2), rel=1e-5)


def test_tied_embeddings_gradient_is_sum_of_both_uses():
    skip = {("schedule", "skip_step"): True}
    tied, _ = build_trainer(tiny_trainer_config({("model", "base_model", "tied_embedding_weight"): True, **skip}))
    names = tied.multi_stage.parameter_names
    assert "head.output_weights" not in names and "embeddings.word_embeddings_weight" in names
    untied, _ = build_trainer(tiny_trainer_config(skip))
    # same weights everywhere, head = embedding
    src = {n: t for n, _, t in tied.multi_stage.get_state_tensor_iterator(("weights",))}
    for name in untied.multi_stage.parameter_names:
        untied.multi_stage.import_state_tensor(name, "weights", src.get(name, src["embeddings.word_embeddings_weight"]))
    untied.multi_stage.invalidate_buffers()
    loss_tied = train_steps(tied, 1)
    loss_untied = train_steps(untied, 1)
    assert loss_tied == pytest.approx(loss_untied, rel=1e-6)
    g = lambda t, n: t.multi_stage.get_parameter_stage(n).get_parameter_meta(n).tensor.grad_buffer
    expected = g(untied, "embeddings.word_embeddings_weight") + g(untied, "head.output_weights")
    torch.testing.assert_close(g(tied, "embeddings.word_embeddings_weight"), expected, rtol=1e-4, atol=1e-7)


def test_checkpoint_resume_is_exact(tmp_path):
    cfg = {("run", "experiment_dir"): str(tmp_path / "exp"), ("training", "checkpoint", "interval"): 2, ("training", "train_iters"): 4}
    full, _ = build_trainer(tiny_trainer_config(cfg))
    losses_full = train_steps(full, 4)
    first, _ = build_trainer(tiny_trainer_config(cfg))
    train_steps(first, 2)
    first._completed_steps = 2
    first._save_checkpoint(first._config.training.checkpoint, {})
    ckpt = tmp_path / "exp" / "checkpoint" / "2"
    assert (ckpt / "ok").exists() and (ckpt / "metadata.yaml").exists() and (ckpt / "rank_0.safetensors").exists()
    resumed, _ = build_trainer(tiny_trainer_config(cfg))
    assert resumed.completed_steps == 2 and resumed.optimizer.current_step == 2
    losses_resumed = train_steps(resumed, 2, start=2)
    assert losses_resumed == losses_full[2:]
    assert torch.equal(resumed.multi_stage.get_shard("weights"), full.multi_stage.get_shard("weights"))
    assert torch.equal(resumed.multi_stage.get_shard("exp_avgs_sq"), full.multi_stage.get_shard("exp_avgs_sq"))


def _model_from(path, fmt, **updates):
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.engine.multi_stage.config import StageMode
    from fast_llm_b200.models.gpt.model import GPTModel

    return GPTModel.from_pretrained(CheckpointLoadConfig(path=path, format=fmt), {("distributed", "use_cuda"): False, **updates},
                                    mode=StageMode.inference, use_cpu=True)


def test_format_conversion_chain(tmp_path):
    """distributed -> fast_llm -> llama (HF) -> fast_llm: weights survive every hop bit-exactly."""
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig

    trainer, _ = build_trainer(tiny_trainer_config())
    train_steps(trainer, 1)
    model = trainer.multi_stage
    reference = {n: t.clone() for n, s, t in model.get_state_tensor_iterator(("weights",))}
    model.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "dist", format="distributed", optimizer_state=True))
    path, fmt = tmp_path / "dist", "distributed"
    for hop, next_fmt in enumerate(["fast_llm", "llama", "fast_llm", "distributed"]):
        loaded = _model_from(path, fmt)
        got = {n: t for n, s, t in loaded.get_state_tensor_iterator(("weights",))}
        assert got.keys() == reference.keys()
        for n in reference:
            assert torch.equal(got[n], reference[n]), (hop, n)
        path, fmt = tmp_path / f"hop{hop}", next_fmt
        loaded.save_checkpoint(CheckpointSaveConfig(path=path, format=fmt))
    hf_config = json.loads((tmp_path / "hop1" / "config.json").read_text())
    assert hf_config["model_type"] == "llama" and hf_config["num_key_value_heads"] == 2


def test_huggingface_export_matches_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from fast_llm_b200.engine.inference.runner import InferenceRunner

    trainer, distributed = build_trainer(tiny_trainer_config())
    train_steps(trainer, 1)
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "hf", format="llama"))
    hf = transformers.AutoModelForCausalLM.from_pretrained(tmp_path / "hf", torch_dtype=torch.float32)
    tokens = torch.randint(0, 512, (1, 96))
    with torch.no_grad():
        expected = hf(tokens).logits[0]
    model = _model_from(tmp_path / "hf", "llama")
    runner = InferenceRunner(model)
    runner.setup(model.distributed)
    logits = runner.forward_tokens(tokens[0])
    torch.testing.assert_close(logits, expected, rtol=2e-4, atol=2e-4)
    # and the import path: a model created by transformers loads here
    hf_config = transformers.LlamaConfig(vocab_size=320, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                         num_key_value_heads=2, head_dim=12, rope_theta=5000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf2 = transformers.LlamaForCausalLM(hf_config)
    hf2.save_pretrained(tmp_path / "hf2", safe_serialization=True)
    model2 = _model_from(tmp_path / "hf2", "auto")
    runner2 = InferenceRunner(model2)
    runner2.setup(model2.distributed)
    tokens2 = torch.randint(0, 320, (1, 64))
    with torch.no_grad():
        expected2 = hf2(tokens2).logits[0]
    torch.testing.assert_close(runner2.forward_tokens(tokens2[0]), expected2, rtol=2e-4, atol=2e-4)


def test_convert_cli(tmp_path):
    from fast_llm_b200.cli import fast_llm_main
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig

    trainer, _ = build_trainer(tiny_trainer_config())
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "src", format="fast_llm"))
    fast_llm_main(["convert", "gpt", f"input.path={tmp_path / 'src'}", "input.format=fast_llm", f"output.path={tmp_path / 'dst'}",
                   "output.format=mistral", "use_cpu=true"])
    assert (tmp_path / "dst" / "ok").exists() and (tmp_path / "dst" / "config.json").exists()
    assert json.loads((tmp_path / "dst" / "config.json").read_text())["model_type"] == "mistral"


MOE_UPDATES = {("model", "base_model", "decoder", "block", "mlp"): {
    "type": "moe", "experts": 4, "experts_per_token": 2, "intermediate_size": 64, "gated": True, "activation": "silu",
    "add_linear_biases": False, "auxiliary_loss_coefficient": 0.01, "z_loss_coefficient": 0.001}}


def test_moe_dropless_matches_looped_and_trains():
    dropless, _ = build_trainer(tiny_trainer_config(MOE_UPDATES))
    looped_updates = {("model", "base_model", "decoder", "block", "mlp"): {**MOE_UPDATES[("model", "base_model", "decoder", "block", "mlp")], "implementation": "looped"}}
    looped, _ = build_trainer(tiny_trainer_config(looped_updates))
    a, b = train_steps(dropless, 3), train_steps(looped, 3)
    assert a == pytest.approx(b, rel=1e-5)
    torch.testing.assert_close(dropless.multi_stage.get_shard("weights"), looped.multi_stage.get_shard("weights"), rtol=1e-4, atol=1e-6)
    assert "load_balancing_loss" in dropless.runner._loss_definitions and "router_z_loss" in dropless.runner._loss_definitions


def test_mixtral_export_matches_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from fast_llm_b200.engine.inference.runner import InferenceRunner

    trainer, _ = build_trainer(tiny_trainer_config({**MOE_UPDATES, ("model", "base_model", "decoder", "block", "mixer", "window_size"): 32}))
    train_steps(trainer, 1)
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "hf", format="mixtral"))
    hf = transformers.AutoModelForCausalLM.from_pretrained(tmp_path / "hf", torch_dtype=torch.float32)
    tokens = torch.randint(0, 512, (1, 24))
    with torch.no_grad():
        expected = hf(tokens).logits[0]
    model = _model_from(tmp_path / "hf", "mixtral")
    runner = InferenceRunner(model)
    runner.setup(model.distributed)
    torch.testing.assert_close(runner.forward_tokens(tokens[0]), expected, rtol=3e-4, atol=3e-4)


def test_multi_token_prediction():
    """Extra prediction heads train; with zero weight on them the trunk behaves exactly like the plain model."""
    import copy

    from tests.common import TINY_BASE_MODEL

    def run(heads, coefficients):
        base = copy.deepcopy(TINY_BASE_MODEL)
        base["head"]["prediction_heads"] = heads
        if coefficients is not None:
            base["head"]["prediction_loss_coefficient"] = coefficients
        trainer, _ = build_trainer(tiny_trainer_config({("model", "base_model"): base}))
        return trainer, train_steps(trainer, 3)

    _, plain = run(1, None)
    trainer, silent = run(2, [1.0, 0.0])
    assert plain == pytest.approx(silent, rel=1e-5)
    trainer, both = run(3, [1.0, 0.5, 0.25])
    names = {meta.tensor_name for _, meta in trainer._multi_stage.base_model.named_parameter_metas()}
    assert "multi_token_prediction.blocks.1.mlp.layer_1.weight" in names
    assert "multi_token_prediction.heads.0.final_norm.weight" in names
    assert both != pytest.approx(plain, rel=1e-5)  # the extra heads change the trunk's gradients


def _round_trip(tmp_path, base_model, format_name):
    """Export to an external format, import into a fresh model, compare logits."""
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
    from fast_llm_b200.engine.inference.runner import InferenceRunner
    from fast_llm_b200.models.gpt.model import GPTModel

    trainer, _ = build_trainer(tiny_trainer_config({("model", "base_model"): base_model}))
    path = tmp_path / format_name
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format=format_name))
    loaded = GPTModel.from_pretrained(CheckpointLoadConfig(path=path, format=format_name), use_cpu=True)
    tokens = torch.randint(0, 512, (40,))
    runners = []
    for model in (trainer.multi_stage, loaded):
        runner = InferenceRunner(model)
        runner.setup()
        runners.append(runner)
    torch.testing.assert_close(runners[0].forward_tokens(tokens), runners[1].forward_tokens(tokens), rtol=1e-4, atol=1e-4)
    exported = json.loads((path / "config.json").read_text())
    # every field the format writes is read back by its own importer (or listed as ignored): nothing is dropped in silence
    handler = type(trainer.multi_stage.config).get_checkpoint_handler_class(format_name)
    assert handler.check_import_coverage(exported)[1] == [], format_name
    return exported


def test_mtp_llama_and_apriel_hybrid_round_trip(tmp_path):
    import copy

    from tests.common import TINY_BASE_MODEL

    mtp = copy.deepcopy(TINY_BASE_MODEL)
    mtp["head"]["prediction_heads"] = 2
    config = _round_trip(tmp_path, mtp, "mtp_llama")
    assert config["prediction_heads"] == 2 and config["model_type"] == "mtp_llama"
    # the exported directory carries stand-alone modelling code that `transformers` can load, and its heads agree with ours
    assert (tmp_path / "mtp_llama" / "modeling_mtp_llama.py").exists() and (tmp_path / "mtp_llama" / "configuration_mtp_llama.py").exists()
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.engine.inference.runner import InferenceRunner
    from fast_llm_b200.external_models.mtp_llama.modeling_mtp_llama import MTPLlamaForCausalLM
    from fast_llm_b200.models.gpt.model import GPTModel

    external = MTPLlamaForCausalLM.from_pretrained(str(tmp_path / "mtp_llama"), torch_dtype=torch.float32)
    tokens = torch.randint(0, 512, (1, 24))
    with torch.no_grad():
        logits = external(input_ids=tokens, return_all_prediction_heads=True).logits
    assert logits.shape == (1, 24, 2, 512)
    runner = InferenceRunner(GPTModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / "mtp_llama", format="mtp_llama"), use_cpu=True))
    runner.setup()
    torch.testing.assert_close(logits[0, :, 0], runner.forward_tokens(tokens[0]), rtol=1e-4, atol=1e-4)

    hybrid = copy.deepcopy(TINY_BASE_MODEL)
    attention_block = hybrid["decoder"]["block"]
    mamba_block = copy.deepcopy(attention_block)
    mamba_block["mixer"] = {"type": "mamba", "d_inner": 64, "d_xb": 32, "state_size": 8, "dt_rank": 4, "add_linear_biases": False,
                            "convolution_layer": {"bias": {"enabled": True}}, "dt_layer": {"bias": {"enabled": True}}}
    hybrid["decoder"] = {"type": "pattern", "blocks": {"t": attention_block, "m2": mamba_block}, "pattern": ["t", "m2", "m2"], "num_blocks": 3}
    gdn_block = copy.deepcopy(attention_block)
    gdn_block["mixer"] = {"type": "gdn", "value_heads": 4, "key_heads": 2, "key_head_dim": 8, "value_head_dim": 8, "convolution_layer": {"kernel_size": 3}}
    hybrid["decoder"] = {"type": "pattern", "blocks": {"t": attention_block, "m2": mamba_block, "gdn": gdn_block}, "pattern": ["t", "m2", "gdn"], "num_blocks": 3}
    config = _round_trip(tmp_path, hybrid, "apriel_hybrid_ssm")
    assert config["hybrid_block_layout"] == ["t", "m2", "gdn"] and config["ssm_cfg"]["d_state"] == 8
    from fast_llm_b200.external_models.apriel_hybrid_ssm.modeling_apriel_hybrid_ssm import AprielHybridSSMForCausalLM

    assert (tmp_path / "apriel_hybrid_ssm" / "modeling_apriel_hybrid_ssm.py").exists()
    external = AprielHybridSSMForCausalLM.from_pretrained(str(tmp_path / "apriel_hybrid_ssm"), torch_dtype=torch.float32)
    with torch.no_grad():
        logits = external(input_ids=tokens).logits
    runner = InferenceRunner(GPTModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / "apriel_hybrid_ssm", format="apriel_hybrid_ssm"), use_cpu=True))
    runner.setup()
    torch.testing.assert_close(logits[0], runner.forward_tokens(tokens[0]), rtol=2e-4, atol=2e-4)


def test_apriel2_round_trip(tmp_path):
    """A pattern decoder with every mixer kind of the Apriel2 format, one of them stochastic."""
    import copy

    from tests.common import TINY_BASE_MODEL

    base = copy.deepcopy(TINY_BASE_MODEL)
    attention_block = base["decoder"]["block"]

    def with_mixer(mixer):
        block = copy.deepcopy(attention_block)
        block["mixer"] = mixer
        return block

    mamba = {"type": "mamba", "d_inner": 64, "d_xb": 32, "state_size": 8, "dt_rank": 4, "add_linear_biases": False,
             "convolution_layer": {"bias": {"enabled": True}}, "dt_layer": {"bias": {"enabled": True}}}
    gdn = {"type": "gdn", "value_heads": 4, "key_heads": 2, "key_head_dim": 8, "value_head_dim": 8, "convolution_layer": {"kernel_size": 3}}
    kda = {"type": "kda", "heads": 2, "head_dim": 8, "convolution_layer": {"kernel_size": 3}}
    stochastic = {"type": "stochastic", "mixers": {"attn": copy.deepcopy(attention_block["mixer"]), "gdn": copy.deepcopy(gdn)}, "main_mixer_name": "attn"}
    base["decoder"] = {"type": "pattern", "num_blocks": 5, "pattern": ["t", "m", "g", "k", "s"],
                       "blocks": {"t": attention_block, "m": with_mixer(mamba), "g": with_mixer(gdn), "k": with_mixer(kda), "s": with_mixer(stochastic)}}
    config = _round_trip(tmp_path, base, "apriel2_text")
    assert config["model_type"] == "apriel2_text" and config["decoder"]["type"] == "pattern"
    blocks = config["decoder"]["blocks"]
    assert [blocks[name]["mixer"]["type"] for name in ("t", "m", "g", "k", "s")] == ["attention", "mamba", "gdn", "kda", "stochastic"]
    assert blocks["t"]["mixer"]["rotary"]["type"] == "mistral_1d" and blocks["m"]["mixer"]["d_conv"] == 4
    assert set(blocks["s"]["mixer"]["mixers"]) == {"attn", "gdn"}
    from safetensors import safe_open

    names = set()
    for file in (tmp_path / "apriel2_text").glob("*.safetensors"):
        with safe_open(file, "pt") as f:
            names |= set(f.keys())
    assert "model.decoder.blocks.4.mixer.mixers.gdn.in_proj_qkvz.weight" in names
    assert "model.decoder.blocks.3.mixer.f_a_proj.weight" in names and "model.decoder.blocks.1.mixer.conv1d.bias" in names
    # the `auto` format recognises it from config.json
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.models.gpt.model import GPTModel

    GPTModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / "apriel2_text", format="auto"), use_cpu=True)
    # the stand-alone modelling code shipped with the checkpoint gives the same logits (all five mixer kinds)
    from fast_llm_b200.engine.inference.runner import InferenceRunner
    from fast_llm_b200.external_models.apriel2.modeling_apriel2 import Apriel2ForCausalLM

    assert (tmp_path / "apriel2_text" / "modeling_apriel2.py").exists() and (tmp_path / "apriel2_text" / "configuration_apriel2.py").exists()
    external = Apriel2ForCausalLM.from_pretrained(str(tmp_path / "apriel2_text"), torch_dtype=torch.float32)
    tokens = torch.randint(0, 512, (1, 24))
    with torch.no_grad():
        logits = external(input_ids=tokens).logits
    runner = InferenceRunner(GPTModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / "apriel2_text", format="apriel2_text"), use_cpu=True))
    runner.setup()
    torch.testing.assert_close(logits[0], runner.forward_tokens(tokens[0]), rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("moe", [False, True])
def test_gemma4_round_trip(tmp_path, moe):
    """Sliding / full attention pattern with head norms, shared key-value, post-norms, frozen output scale, soft-capped
    logits; with `moe` the MLP is a dense branch plus a routed mixture of experts stored batched."""
    import copy

    from tests.common import TINY_BASE_MODEL

    base = copy.deepcopy(TINY_BASE_MODEL)
    hidden = base["hidden_size"]
    norm = {"type": "rms_norm", "epsilon": 1e-6}

    def attention(sliding):
        out = {"type": "attention", "heads": 4, "head_groups": 2, "head_size": 16 if sliding else 32, "add_linear_biases": False, "softmax_scale_power": 0,
               "query_norm": dict(norm), "key_norm": dict(norm), "value_norm": {"type": "fixed_rms_norm", "epsilon": 1e-6},
               "rotary": {"type": "default", "theta": 10000.0} if sliding else {"type": "proportional", "theta": 1000000.0, "partial_rotary_factor": 0.25}}
        if sliding:
            out["window_size"] = 16
        else:
            out["shared_key_value"] = True
            out["head_groups"] = 1
        return out

    dense = {"type": "mlp", "intermediate_size": 96, "gated": True, "add_linear_biases": False, "activation": "gelu"}

    def block(sliding):
        out = {"type": "decoder", "mixer": attention(sliding), "normalization": dict(norm), "post_mixer_normalization": dict(norm),
               "post_mlp_normalization": dict(norm), "output_scale": {"enabled": True, "lr_scale": 0}}
        if moe:
            routed = {"type": "moe", "intermediate_size": 32, "gated": True, "add_linear_biases": False, "activation": "gelu", "experts": 4,
                      "experts_per_token": 2, "router_normalization": {"type": "fixed_rms_norm", "epsilon": 1e-6}, "router_scale": {"enabled": True},
                      "router_input_scale": hidden**-0.5, "router_per_expert_scale": {"enabled": True}, "pre_norm": dict(norm), "post_norm": dict(norm)}
            out["mlp"] = {"type": "hybrid_moe", "dense": {**dense, "pre_norm": dict(norm), "post_norm": dict(norm)}, "routed": routed}
            out["pre_mlp_normalization"] = {"type": "none"}
        else:
            out["mlp"] = dict(dense)
            out["pre_mlp_normalization"] = dict(norm)
        return out

    base["decoder"] = {"type": "pattern", "num_blocks": 3, "pattern": ["sliding_attention", "sliding_attention", "full_attention"],
                       "blocks": {"sliding_attention": block(True), "full_attention": block(False)}}
    base["embeddings"]["embedding_scale"] = hidden**0.5
    base["head"]["final_logit_softcap"] = 30.0
    base["head"]["normalization"] = dict(norm)
    config = _round_trip(tmp_path, base, "gemma4")
    assert config["model_type"] == "gemma4_text" and config["layer_types"] == ["sliding_attention"] * 2 + ["full_attention"]
    assert config["head_dim"] == 16 and config["global_head_dim"] == 32 and config["num_global_key_value_heads"] == 1 and config["attention_k_eq_v"]
    assert config["final_logit_softcapping"] == 30.0 and config["enable_moe_block"] == moe
    from safetensors import safe_open

    shapes = {}
    for file in (tmp_path / "gemma4").glob("*.safetensors"):
        with safe_open(file, "pt") as f:
            for key in f.keys():
                shapes[key] = list(f.get_slice(key).get_shape())
    assert "model.layers.2.self_attn.v_proj.weight" not in shapes and "model.layers.0.self_attn.v_proj.weight" in shapes
    assert "model.layers.1.layer_scalar" in shapes and "model.layers.0.self_attn.q_norm.weight" in shapes
    if moe:
        assert shapes["model.layers.0.experts.gate_up_proj"] == [4, 64, hidden] and shapes["model.layers.0.experts.down_proj"] == [4, hidden, 32]
        assert "model.layers.0.router.per_expert_scale" in shapes and "model.layers.0.pre_feedforward_layernorm_2.weight" in shapes


@pytest.mark.parametrize("format_name", ["diffusion_llama", "dream"])
def test_diffusion_formats_round_trip(tmp_path, format_name):
    """The diffusion formats carry a Llama / Qwen2 decoder; the stand-alone code shipped with them reproduces our logits when
    told to stay causal, and samples by iterative unmasking with bidirectional attention."""
    import copy
    import importlib

    from tests.common import TINY_BASE_MODEL

    base = copy.deepcopy(TINY_BASE_MODEL)
    if format_name == "dream":  # Qwen2-style: biases on the query / key / value projections only
        mixer = base["decoder"]["block"]["mixer"]
        mixer["add_linear_biases"] = False
        for layer in ("query_layer", "key_layer", "value_layer"):
            mixer[layer] = {"bias": {"enabled": True}}
        mixer["dense_layer"] = {"bias": {"enabled": False}}
    config = _round_trip(tmp_path, base, format_name)
    assert config["model_type"] == ("Dream" if format_name == "dream" else "diffusion_llama")
    module_name, class_name = ("diffusion_dream.modeling_dream", "DreamModel") if format_name == "dream" else ("diffusion_llama.modeling_diffusion_llama", "DiffusionLlamaModel")
    model_class = getattr(importlib.import_module(f"fast_llm_b200.external_models.{module_name}"), class_name)
    assert (tmp_path / format_name / (module_name.split(".")[1] + ".py")).exists()
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.engine.inference.runner import InferenceRunner
    from fast_llm_b200.models.gpt.model import GPTModel

    tokens = torch.randint(0, 500, (1, 24))
    causal = model_class.from_pretrained(str(tmp_path / format_name), torch_dtype=torch.float32, bidirectional=False)
    with torch.no_grad():
        logits = causal(input_ids=tokens).logits
    runner = InferenceRunner(GPTModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / format_name, format=format_name), use_cpu=True))
    runner.setup()
    torch.testing.assert_close(logits[0], runner.forward_tokens(tokens[0]), rtol=2e-4, atol=2e-4)
    model = model_class.from_pretrained(str(tmp_path / format_name), torch_dtype=torch.float32)
    with torch.no_grad():
        assert (model(input_ids=tokens).logits - logits).abs().max() > 1e-3  # bidirectional attention sees later tokens
    out = model.diffusion_generate(tokens[:, :8], max_new_tokens=10, steps=4)
    assert out.shape == (1, 18) and (out[:, :8] == tokens[:, :8]).all() and (out != model.config.mask_token_id).all()


def test_checkpoint_surgery_tools(tmp_path):
    """MoE upcycling and MTP-head surgery produce checkpoints this framework loads."""
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
    from fast_llm_b200.models.gpt.model import GPTModel
    from fast_llm_b200.tools.checkpoint_surgery import AddExpertsConfig, AddPredictionHeadsConfig, load_hf_state

    moe, _ = build_trainer(tiny_trainer_config(MOE_UPDATES))
    moe.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "moe", format="mixtral"))
    surgery = AddExpertsConfig.from_dict({"hf_checkpoint": str(tmp_path / "moe"), "output_dir": str(tmp_path / "moe6"), "num_new_experts": 2,
                                          "expert_init_std": 0.01, "router_init_std": 0.01})
    surgery.validate()
    surgery.run()
    config, state = load_hf_state(tmp_path / "moe6")
    assert config["num_local_experts"] == 6 and state["model.layers.0.block_sparse_moe.gate.weight"].shape[0] == 6
    assert "model.layers.1.block_sparse_moe.experts.5.w2.weight" in state
    bigger = GPTModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / "moe6", format="mixtral"), use_cpu=True)
    assert bigger.config.base_model.decoder.block.mlp.experts == 6

    dense, _ = build_trainer(tiny_trainer_config())
    dense.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "llama", format="llama"))
    heads = AddPredictionHeadsConfig.from_dict({"hf_checkpoint": str(tmp_path / "llama"), "output_dir": str(tmp_path / "mtp"), "num_prediction_heads": 3})
    heads.validate()
    heads.run()
    loaded = GPTModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / "mtp", format="mtp_llama"), use_cpu=True)
    assert loaded.config.base_model.head.prediction_heads == 3
    _, state = load_hf_state(tmp_path / "mtp")
    torch.testing.assert_close(state["model.mtp_heads.1.mlp.down_proj.weight"], state["model.layers.1.mlp.down_proj.weight"])


def test_push_model_selects_stages_and_uploads(tmp_path):
    """Only checkpoints without a commit are uploaded, oldest first, each staged with the tokenizer."""
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from fast_llm_b200.tools.push_model import PushConfig

    trainer, _ = build_trainer(tiny_trainer_config())
    for iteration in (10, 20, 30):
        trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "run" / "export" / "llama" / str(iteration), format="llama"))
        (tmp_path / "run" / "export" / "llama" / str(iteration) / "ok").touch()  # the trainer marks finished exports
    (tmp_path / "run" / "export" / "llama" / "40").mkdir()  # incomplete: no `ok` marker
    tokenizer = tmp_path / "tok" / "tokenizer.json"
    tokenizer.parent.mkdir()
    tokenizer.write_text("{}")
    (tokenizer.parent / "tokenizer_config.json").write_text("{}")

    class Commit:
        def __init__(self, title):
            self.title = title

    class FakeApi:
        def __init__(self):
            self.uploads = []

        def create_repo(self, name, private, exist_ok):
            self.repo = name

        def list_repo_commits(self, name):
            return [Commit("initial commit"), Commit("10")]

        def upload_folder(self, folder_path, repo_id, commit_message):
            import pathlib

            self.uploads.append((commit_message, sorted(p.name for p in pathlib.Path(folder_path).iterdir())))

    config = PushConfig.from_dict({"experiment_dir": str(tmp_path / "run"), "repo_name": "org/model", "model_type": "llama", "tokenizer_path": str(tokenizer)})
    config.validate()
    api = FakeApi()
    assert config.run(api) == [20, 30]
    assert [message for message, _ in api.uploads] == ["20", "30"]
    assert {"config.json", "tokenizer.json", "tokenizer_config.json"} <= set(api.uploads[0][1])
    assert any(name.endswith(".safetensors") for name in api.uploads[0][1])
    assert not (tmp_path / "run" / "export_tmp").exists()


def test_megatron_initialization_replays_one_stream():
    """query / key_value / dense of a layer are slices of ONE (dense, fused qkv) draw, as Megatron creates them."""
    from fast_llm_b200.models.gpt.megatron import set_megatron_distributed_seeds

    config = tiny_trainer_config({("model", "base_model", "use_megatron_initialization"): True})
    set_megatron_distributed_seeds(config.model.distributed)
    trainer, distributed = build_trainer(config)
    weights = {name: tensor for name, _, tensor in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    heads, groups, head_size, hidden = 4, 2, 16, 64
    # Within one layer the three attention weights must be mutually consistent with a single fused draw: recover the
    # fused tensor from query and key_value and check its statistics and shapes.
    q, kv, dense = (weights[f"decoder.0.mixer.{n}.weight"] for n in ("query", "key_value", "dense"))
    assert q.shape == (heads * head_size, hidden) and kv.shape == (2 * groups * head_size, hidden) and dense.shape == (hidden, heads * head_size)
    fused = torch.cat([q.view(groups, heads // groups, head_size, hidden), kv.view(2, groups, head_size, hidden).transpose(0, 1)], 1)
    assert fused.shape == (groups, heads // groups + 2, head_size, hidden)
    std = hidden**-0.5
    for tensor in (q, kv, dense, weights["decoder.0.mlp.layer_2.weight"]):
        assert 0.7 * std < tensor.float().std().item() < 1.3 * std
    # the two layers come from an advancing stream (not identical), and a second build reproduces the values exactly
    assert not torch.equal(weights["decoder.0.mixer.query.weight"], weights["decoder.1.mixer.query.weight"])
    config2 = tiny_trainer_config({("model", "base_model", "use_megatron_initialization"): True})
    set_megatron_distributed_seeds(config2.model.distributed)
    trainer2, _ = build_trainer(config2)
    for name, _, tensor in trainer2.multi_stage.get_state_tensor_iterator(("weights",)):
        assert torch.equal(tensor, weights[name]), name


def test_safe_load_names_the_parameter_that_was_not_loaded(tmp_path):
    """A checkpoint load that skips one parameter must fail, and say which one."""
    from fast_llm_b200.engine.checkpoint.safe_load import SafeLoad

    trainer, _ = build_trainer(tiny_trainer_config())
    model = trainer.multi_stage
    names = [n for _, _, fsdp, _ in model.iter_fsdps() for n in fsdp.parameter_names]
    skipped = names[3]
    with pytest.raises(RuntimeError, match=skipped.replace(".", r"\.")):
        with SafeLoad(model, shard_names=("weights",)) as context:
            for _, _, fsdp, sl in model.iter_fsdps():
                shard = model.get_shard("weights")[sl]
                for name in fsdp.parameter_names:
                    begin, end = fsdp.parameter_range_in_shard(name)
                    if name == skipped:
                        continue
                    shard[begin:end].zero_()
                    context.mark_as_loaded(end - begin, (name, "weights"))


@pytest.mark.parametrize("format_name", ["llama", "mistral", "mtp_llama", "apriel_hybrid_ssm", "apriel2_text"])
def test_export_refuses_what_the_format_cannot_represent(tmp_path, format_name):
    """A model whose architecture has no place in the external format fails the export with the fields named, instead of
    writing a checkpoint that loads as a different model; an unknown key of a foreign `config.json` is reported on import."""
    import copy

    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from tests.common import TINY_BASE_MODEL

    base = copy.deepcopy(TINY_BASE_MODEL)
    base["decoder"]["block"]["mixer"]["softmax_scale_power"] = 0.75  # no Hugging Face format carries this
    trainer, _ = build_trainer(tiny_trainer_config({("model", "base_model"): base}))
    with pytest.raises((ValueError, AssertionError), match="softmax_scale_power|cannot represent|needs|Mismatch|Assert"):
        trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "bad", format=format_name))


def test_import_reports_fields_nobody_claimed(tmp_path):
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from fast_llm_b200.models.gpt.config import GPTModelConfig

    trainer, _ = build_trainer(tiny_trainer_config())
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=tmp_path / "hf", format="llama"))
    exported = json.loads((tmp_path / "hf" / "config.json").read_text())
    handler = GPTModelConfig.get_checkpoint_handler_class("llama")
    assert handler.check_import_coverage(exported)[1] == []
    exported["mystery_gate"] = 3
    exported["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                "original_max_position_embeddings": 8192, "mystery_inner": 1}
    assert sorted(handler.check_import_coverage(exported)[1]) == ["mystery_gate", "rope_scaling.mystery_inner"]


def test_lora_model_exports_merged_weights_and_imports_a_plain_checkpoint(tmp_path):
    """External formats hold no adapters: on export the low-rank update is merged into the weight it adapts (the exported
    model computes what the LoRA model does, here on the query and, transposed storage, on the MLP's second layer); on import
    the base weights come from the checkpoint and the adapters from their initialisers (B = 0: the same function again)."""
    import copy

    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
    from fast_llm_b200.engine.inference.runner import InferenceRunner
    from fast_llm_b200.models.gpt.model import GPTModel
    from tests.common import TINY_BASE_MODEL

    base = copy.deepcopy(TINY_BASE_MODEL)
    base["peft"] = {"type": "lora", "rank": 4, "alpha": 8.0}
    base["decoder"]["block"]["mlp"]["layer_2"] = {"apply_peft": True}
    trainer, _ = build_trainer(tiny_trainer_config({("model", "base_model"): base, ("optimizer", "learning_rate", "base"): 3e-2}))
    names = [n for n, _, _ in trainer.multi_stage.get_state_tensor_iterator(("weights",))]
    assert "decoder.0.mixer.query.lora_b_weight" in names and "decoder.1.mlp.layer_2.lora_a_weight" in names
    train_steps(trainer, 3)  # B leaves zero
    state = {n: t for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    assert float(state["decoder.0.mixer.query.lora_b_weight"].abs().max()) > 0 and float(state["decoder.1.mlp.layer_2.lora_b_weight"].abs().max()) > 0
    path = tmp_path / "merged"
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="llama"))
    tokens = torch.randint(0, 512, (40,))

    def logits(model):
        runner = InferenceRunner(model)
        runner.setup()
        return runner.forward_tokens(tokens)

    expected = logits(trainer.multi_stage)
    plain = GPTModel.from_pretrained(CheckpointLoadConfig(path=path, format="llama"), use_cpu=True)
    assert not any("lora" in n for n in plain.parameter_names)
    torch.testing.assert_close(logits(plain), expected, rtol=1e-4, atol=1e-4)
    # a LoRA model started from the merged checkpoint: fresh adapters, same function
    again = GPTModel.from_pretrained(CheckpointLoadConfig(path=path, format="llama"), {("base_model", "peft"): {"type": "lora", "rank": 4, "alpha": 8.0}},
                                     use_cpu=True)
    loaded = {n: t for n, _, t in again.get_state_tensor_iterator(("weights",))}
    assert float(loaded["decoder.0.mixer.query.lora_b_weight"].abs().max()) == 0 and float(loaded["decoder.0.mixer.query.lora_a_weight"].abs().max()) > 0
    torch.testing.assert_close(logits(again), expected, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("format_name,window", [("mistral", 6), ("qwen2", 6), ("qwen2", None)])
def test_sliding_window_exports_match_transformers(tmp_path, format_name, window):
    """A window shorter than the sequence: the exported `config.json` must make `transformers` apply it on every layer
    (Qwen2 keeps full attention below `max_window_layers`, so the export says 0), and both sides give the same logits.
    Default Hugging Face configurations of the formats import without an unread key."""
    import copy

    transformers = pytest.importorskip("transformers")
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from fast_llm_b200.engine.inference.runner import InferenceRunner
    from fast_llm_b200.models.gpt.config import GPTModelConfig
    from tests.common import TINY_BASE_MODEL

    base = copy.deepcopy(TINY_BASE_MODEL)
    mixer = base["decoder"]["block"]["mixer"]
    if window is not None:
        mixer["window_size"] = window
    if format_name == "qwen2":
        mixer.update(add_linear_biases=True, dense_layer={"bias": {"enabled": False}})
    trainer, _ = build_trainer(tiny_trainer_config({("model", "base_model"): base}))
    path = tmp_path / format_name
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format=format_name))
    hf = transformers.AutoModelForCausalLM.from_pretrained(path, dtype=torch.float32, attn_implementation="eager")
    tokens = torch.randint(0, 512, (1, 24))
    with torch.no_grad():
        expected = hf(tokens).logits[0]
    runner = InferenceRunner(trainer.multi_stage)
    runner.setup()
    torch.testing.assert_close(runner.forward_tokens(tokens[0]), expected, rtol=2e-4, atol=2e-4)
    if window is not None:
        exported = json.loads((path / "config.json").read_text())
        assert exported["sliding_window"] == window and exported.get("max_window_layers", 0) == 0
    defaults = {"mistral": transformers.MistralConfig(), "qwen2": transformers.Qwen2Config()}[format_name]
    _, unread = GPTModelConfig.get_checkpoint_handler_class(format_name).check_import_coverage(json.loads(defaults.to_json_string()))
    assert unread == []


def test_mixtral_default_configuration_imports_without_unread_keys():
    transformers = pytest.importorskip("transformers")
    from fast_llm_b200.models.gpt.config import GPTModelConfig

    config = json.loads(transformers.MixtralConfig(router_jitter_noise=0.02).to_json_string())
    base, unread = GPTModelConfig.get_checkpoint_handler_class("mixtral").check_import_coverage(config)
    assert unread == [] and base["decoder"]["block"]["mlp"]["jitter_eps"] == 0.02


@pytest.mark.parametrize("head_groups", [4, 1], ids=["gpt2", "starcoder"])
def test_absolute_position_architectures_train_and_generate(head_groups):
    """The GPT-2 / StarCoder family: learned absolute positions instead of rotary, LayerNorm, a plain GELU MLP, biases everywhere,
    tied embeddings, multi-query attention for StarCoder.  Trains, and generates through the key / value cache (the cached
    steps take their absolute positions from the cache length) exactly as without it."""
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    base = {"embeddings": {"vocab_size": 512, "position_embeddings": {"enabled": True}, "num_position_embeddings": 256},
            "decoder": {"num_blocks": 2, "block": {
                "mixer": {"type": "attention", "rotary": {"type": "none"}, "heads": 4, "head_groups": head_groups, "head_size": 16, "add_linear_biases": True},
                "mlp": {"intermediate_size": 128, "gated": False, "activation": "gelu", "add_linear_biases": True},
                "normalization": {"type": "layer_norm"}}},
            "head": {"normalization": {"type": "layer_norm"}}, "hidden_size": 64, "tied_embedding_weight": True}
    trainer, _ = build_trainer(tiny_trainer_config({("model", "base_model"): base}))
    names = {n for n, _, _ in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    assert "embeddings.position_embeddings_weight" in names and "decoder.0.mlp.layer_1.bias" in names and "decoder.0.norm_1.bias" in names
    assert "head.output_weights" not in names
    losses = train_steps(trainer, 4)
    assert all(torch.isfinite(torch.tensor(losses)))
    model = HuggingfaceGPTModelForCausalLM(trainer.multi_stage)
    prompt = torch.randint(1, 512, (2, 7))
    mask = torch.ones_like(prompt)
    mask[1, :3] = 0
    cached = model.generate(prompt * mask, attention_mask=mask, max_new_tokens=4, do_sample=False, pad_token_id=0)
    plain = model.generate(prompt * mask, attention_mask=mask, max_new_tokens=4, do_sample=False, pad_token_id=0, use_cache=False)
    assert torch.equal(cached, plain)


def test_planned_shutdown_resume_and_wandb_logging(tmp_path):
    """`training.shutdown` stops the run at its interval after saving a checkpoint; the next start resumes there and finishes.
    With an entity configured the metrics of every logged step, evaluator results included, reach W&B (a stand-in module)."""
    from fast_llm_b200.cli import fast_llm_main
    from fast_llm_b200.engine.training import trainer as trainer_module

    class FakeWandb:
        def __init__(self):
            self.inits, self.logs, self.alerts, self.finished = [], [], [], []

        def Settings(self, **kwargs):
            return kwargs

        def init(self, **kwargs):
            self.inits.append(kwargs)

        def log(self, metrics, step=None, commit=True):
            self.logs.append((step, metrics))

        def alert(self, **kwargs):
            self.alerts.append(kwargs)

        def finish(self, exit_code=0):
            self.finished.append(exit_code)

    fake = FakeWandb()
    arguments = ["train", "gpt", f"run.experiment_dir={tmp_path / 'run'}", "training.train_iters=4", "training.logs.interval=1", "training.num_workers=0",
                 "training.checkpoint.interval=2", "training.shutdown.interval=2", "training.wandb.entity_name=team", "training.wandb.project_name=project",
                 "training.evaluators.validation.type=loss", "training.evaluators.validation.interval=2", "training.evaluators.validation.iterations=1",
                 "data.datasets.training.type=random", "data.datasets.validation.type=random", "data.micro_batch_size=64",
                 "model.base_model.embeddings.vocab_size=300", "model.base_model.hidden_size=32", "model.base_model.decoder.num_blocks=1",
                 "model.base_model.decoder.block.mixer.heads=4", "model.base_model.decoder.block.mixer.head_groups=2",
                 "model.base_model.decoder.block.mixer.head_size=8", "model.base_model.decoder.block.mlp.intermediate_size=64",
                 "model.distributed.compute_dtype=float32", "model.distributed.use_cuda=false"]
    original = trainer_module.Trainer.run

    def run_with_fake(self):
        self._wandb_module = fake
        return original(self)

    trainer_module.Trainer.run = run_with_fake
    try:
        fast_llm_main(arguments)
        assert (tmp_path / "run/checkpoint/2/ok").exists() and not (tmp_path / "run/checkpoint/4").exists()  # stopped at the planned point
        fast_llm_main(arguments)
    finally:
        trainer_module.Trainer.run = original
    assert (tmp_path / "run/checkpoint/4/ok").exists()
    assert len(fake.inits) == 2 and fake.inits[0]["entity"] == "team" and fake.inits[0]["project"] == "project" and fake.finished == [0, 0]
    steps = [step for step, _ in fake.logs]
    assert sorted(set(steps)) == [1, 2, 3, 4]
    keys = {key for _, metrics in fake.logs for key in metrics}
    assert any(key.startswith("train") and "lm_loss" in key for key in keys) and any("validation" in key for key in keys), keys
