"""Vision encoder + language model: the multimodal model trains end to end and image patches reach the right tokens."""

import copy

import torch

from tests.common import TINY_BASE_MODEL, build_trainer, train_steps


def _config(updates=None):
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.models.multimodal.config import MultiModalTrainerConfig

    base = copy.deepcopy(TINY_BASE_MODEL)
    base["vision_encoder"] = {
        "hidden_size": 32,
        "embeddings": {"patch_height": 4, "patch_width": 4, "normalization": {"type": "rms_norm"}},
        "encoder": {"num_blocks": 2, "block": {
            "mixer": {"heads": 2, "head_groups": 2, "head_size": 16, "causal": False, "rotary": {"type": "default_2d"}, "add_linear_biases": False},
            "mlp": {"intermediate_size": 64, "gated": True, "add_linear_biases": False}, "normalization": {"type": "rms_norm"}}},
        "adapter": {"intermediate_size": 48, "add_linear_biases": True},
    }
    config = {
        "training": {"train_iters": 4, "num_workers": 0, "logs": {"interval": 1}},
        "data": {"datasets": {"training": {"type": "random", "images_per_sample": 3, "image_patch_grid": [2, 3], "image_patch_shape": [3, 4, 4]}},
                 "micro_batch_size": 128, "seed": 0},
        "optimizer": {"learning_rate": {"base": 1e-3}},
        "model": {"base_model": base,
                  "distributed": {"compute_dtype": "float32", "use_cuda": False, "seed": 0, "world_size": 1, "rank": 0, "local_world_size": 1}},
    }
    return MultiModalTrainerConfig.from_dict(config, updates or {})


def test_multimodal_model_trains():
    trainer, _ = build_trainer(_config())
    losses = train_steps(trainer, 5)
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < losses[0]
    names = {meta.tensor_name for _, meta in trainer._multi_stage.base_model.named_parameter_metas()}
    assert "vision_encoder.embeddings.patch_embeddings.weight" in names
    assert "vision_encoder.encoder.1.mixer.query.weight" in names
    assert "vision_encoder.adapter.layer_2.weight" in names
    # every vision parameter received gradient signal: it moved away from its initial value
    assert "decoder.0.mlp.layer_1.weight" in names


def test_image_patches_are_added_at_their_tokens():
    """Zeroing the pixels of one image changes the embedding output only at that image's token positions."""
    from fast_llm_b200.data.document import LanguageModelBatch, LanguageModelDocument
    from fast_llm_b200.parallel.topology import PhaseType

    trainer, _ = build_trainer(_config())
    model = trainer._multi_stage.base_model
    for stage in trainer._multi_stage.stages:
        stage.restore_parameters()
    torch.manual_seed(0)
    tokens = torch.randint(0, 512, (129,))
    coordinates = torch.tensor([[0, 0], [0, 1], [1, 0], [1, 1]] * 2)
    positions = torch.tensor([5, 6, 7, 8, 40, 41, 42, 43])

    def embed(pixels):
        document = LanguageModelDocument(tokens=tokens, image_patches=pixels, image_patch_positions=positions, image_patch_coordinates=coordinates)
        batch = LanguageModelBatch.from_documents([document], 129)
        inputs = batch.get_model_inputs(micro_batch_size=128)
        (ids, kwargs), = model.preprocess_batch(inputs, phase=PhaseType.inference, iteration=0)
        hidden = None
        for layer in model.get_layers()[:5]:  # patch embeddings, 2 encoder blocks, adapter, token embeddings
            hidden = layer.forward(ids if hidden is None else hidden, kwargs)
        return hidden

    pixels = torch.randint(0, 256, (8, 3, 4, 4), dtype=torch.uint8)
    changed = pixels.clone()
    changed[4:] = 0
    with torch.no_grad():
        a, b = embed(pixels), embed(changed)
    moved = ((a - b).abs().sum(-1) > 1e-6).nonzero().flatten().tolist()
    assert moved == [40, 41, 42, 43]


def test_llava_round_trip(tmp_path):
    """Export to the llava layout (conv-shaped patch kernel, language_model.* prefix) and load it back."""
    import json

    import safetensors

    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
    from fast_llm_b200.models.multimodal.model import MultiModalModel

    trainer, _ = build_trainer(_config({("model", "base_model", "image_token_index"): 7,
                                        ("model", "base_model", "vision_encoder", "adapter", "intermediate_size"): 64}))  # llava: adapter width = text hidden size
    path = tmp_path / "llava"
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="llava"))
    config = json.loads((path / "config.json").read_text())
    assert config["model_type"] == "llava" and config["vision_config"]["patch_size"] == 4 and config["text_config"]["model_type"] == "mistral"
    names = {}
    for file in path.glob("*.safetensors"):
        with safetensors.safe_open(str(file), framework="pt") as f:
            for key in f.keys():
                names[key] = f.get_slice(key).get_shape()
    assert names["vision_tower.patch_conv.weight"] == [32, 3, 4, 4]
    assert "language_model.model.layers.0.self_attn.q_proj.weight" in names and "multi_modal_projector.linear_2.bias" in names
    loaded = MultiModalModel.from_pretrained(CheckpointLoadConfig(path=path, format="llava"), use_cpu=True)
    original = {n: t for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    for name, _, tensor in loaded.get_state_tensor_iterator(("weights",)):
        torch.testing.assert_close(tensor.float(), original[name].float(), rtol=1e-2, atol=1e-2, msg=lambda m: f"{name}: {m}")


def test_apriel2_multimodal_round_trip(tmp_path):
    """The Apriel2 layout nests the vision encoder under `vision_encoder` and keeps the text keys at the top level."""
    import json

    import safetensors

    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
    from fast_llm_b200.models.multimodal.model import MultiModalModel

    trainer, _ = build_trainer(_config({("model", "base_model", "image_token_index"): 7}))
    path = tmp_path / "apriel2"
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="apriel2"))
    config = json.loads((path / "config.json").read_text())
    assert config["model_type"] == "apriel2" and config["architectures"] == ["Apriel2ForConditionalGeneration"]
    assert config["decoder"]["type"] == "fixed" and config["vision_encoder"]["encoder"]["block"]["mixer"]["rotary"]["type"] == "pixtral_2d"
    assert config["vision_encoder"]["adapter"]["intermediate_size"] == 48 and config["image_token_index"] == 7
    names = {}
    for file in path.glob("*.safetensors"):
        with safetensors.safe_open(str(file), framework="pt") as f:
            for key in f.keys():
                names[key] = f.get_slice(key).get_shape()
    assert names["model.vision_encoder.embeddings.patch_embeddings.weight"] == [32, 3, 4, 4]
    assert "model.vision_encoder.encoder.blocks.1.mixer.k_proj.weight" in names and "model.vision_encoder.adapter.linear_2.bias" in names
    assert "model.decoder.blocks.0.mixer.q_proj.weight" in names
    for format_name in ("apriel2", "auto"):
        loaded = MultiModalModel.from_pretrained(CheckpointLoadConfig(path=path, format=format_name), use_cpu=True)
        original = {n: t for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
        for name, _, tensor in loaded.get_state_tensor_iterator(("weights",)):
            torch.testing.assert_close(tensor.float(), original[name].float(), rtol=1e-2, atol=1e-2, msg=lambda m: f"{name}: {m}")


def test_llava_hybrid_round_trip(tmp_path):
    """Llava around an Apriel hybrid language model (attention + Mamba blocks)."""
    import json

    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig, CheckpointSaveConfig
    from fast_llm_b200.models.multimodal.model import MultiModalModel

    attention_block = copy.deepcopy(TINY_BASE_MODEL["decoder"]["block"])
    mamba_block = copy.deepcopy(attention_block)
    mamba_block["mixer"] = {"type": "mamba", "d_inner": 64, "d_xb": 32, "state_size": 8, "dt_rank": 4, "add_linear_biases": False,
                            "convolution_layer": {"bias": {"enabled": True}}, "dt_layer": {"bias": {"enabled": True}}}
    decoder = {"type": "pattern", "blocks": {"t": attention_block, "m2": mamba_block}, "pattern": ["t", "m2"], "num_blocks": 2}
    trainer, _ = build_trainer(_config({("model", "base_model", "image_token_index"): 7, ("model", "base_model", "decoder"): decoder,
                                        ("model", "base_model", "vision_encoder", "adapter", "intermediate_size"): 64}))
    path = tmp_path / "llava_hybrid"
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="llava_hybrid_ssm"))
    config = json.loads((path / "config.json").read_text())
    assert config["architectures"] == ["LlavaHybridForConditionalGeneration"] and config["text_config"]["hybrid_block_layout"] == ["t", "m2"]
    loaded = MultiModalModel.from_pretrained(CheckpointLoadConfig(path=path, format="llava_hybrid_ssm"), use_cpu=True)
    original = {n: t for n, _, t in trainer.multi_stage.get_state_tensor_iterator(("weights",))}
    count = 0
    for name, _, tensor in loaded.get_state_tensor_iterator(("weights",)):
        torch.testing.assert_close(tensor.float(), original[name].float(), rtol=1e-2, atol=1e-2, msg=lambda m: f"{name}: {m}")
        count += 1
    assert count == len(original)


def test_llava_hybrid_modeling_code_loads_the_export_and_reproduces_the_logits(tmp_path):
    """The stand-alone Llava-hybrid modelling files shipped with a `llava_hybrid_ssm` export load every tensor of it, and the
    `transformers` model they build (Pixtral vision tower, projector, Apriel hybrid decoder) gives this framework's logits for
    text alone and for text with an image."""
    import json

    from fast_llm_b200.data.document import LanguageModelBatch, LanguageModelDocument
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from fast_llm_b200.external_models.llava_hybrid.modeling_llava_hybrid import LlavaHybridForConditionalGeneration
    from fast_llm_b200.parallel.topology import PhaseType

    attention_block = copy.deepcopy(TINY_BASE_MODEL["decoder"]["block"])
    mamba_block = copy.deepcopy(attention_block)
    mamba_block["mixer"] = {"type": "mamba", "d_inner": 64, "d_xb": 32, "state_size": 8, "dt_rank": 4, "add_linear_biases": False,
                            "convolution_layer": {"bias": {"enabled": True}}, "dt_layer": {"bias": {"enabled": True}}}
    decoder = {"type": "pattern", "blocks": {"t": attention_block, "m2": mamba_block}, "pattern": ["t", "m2"], "num_blocks": 2}
    trainer, _ = build_trainer(_config({("model", "base_model", "image_token_index"): 7, ("model", "base_model", "decoder"): decoder,
                                        ("model", "base_model", "vision_encoder", "adapter", "intermediate_size"): 64}))
    path = tmp_path / "llava_hybrid"
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="llava_hybrid_ssm"))
    for name in ("configuration_llava_hybrid.py", "modeling_llava_hybrid.py", "configuration_apriel_hybrid_ssm.py", "modeling_apriel_hybrid_ssm.py"):
        assert (path / name).exists(), name
    assert json.loads((path / "config.json").read_text())["auto_map"]["AutoModelForCausalLM"].endswith("LlavaHybridForConditionalGeneration")
    external, info = LlavaHybridForConditionalGeneration.from_pretrained(str(path), torch_dtype=torch.float32, output_loading_info=True)
    assert not info["missing_keys"] and not info["unexpected_keys"], info
    external.eval()

    model = trainer._multi_stage.base_model
    for stage in trainer._multi_stage.stages:
        stage.restore_parameters()

    def ours(tokens, **image):
        document = LanguageModelDocument(tokens=tokens, **image)
        batch = LanguageModelBatch.from_documents([document], tokens.numel())
        inputs = batch.get_model_inputs(micro_batch_size=tokens.numel() - 1)
        (ids, kwargs), = model.preprocess_batch(inputs, phase=PhaseType.inference, iteration=0)
        kwargs["return_logits"] = True
        hidden = None
        with torch.no_grad():
            for layer in model.get_layers():
                hidden = layer.forward(ids if hidden is None else hidden, kwargs)
        return kwargs["logits"]

    torch.manual_seed(0)
    tokens = torch.randint(8, 512, (41,))
    with torch.no_grad():
        theirs = external(input_ids=tokens[None, :-1]).logits[0]
    torch.testing.assert_close(ours(tokens), theirs, rtol=2e-4, atol=2e-4)

    # one 2 x 3 grid of 4 x 4 patches at tokens 5..10; the Hugging Face side takes the normalised image
    pixels = torch.randint(0, 256, (3, 8, 12), dtype=torch.uint8)
    patches = pixels.view(3, 2, 4, 3, 4).permute(1, 3, 0, 2, 4).reshape(6, 3, 4, 4)
    coordinates = torch.tensor([[r, c] for r in range(2) for c in range(3)])
    positions = torch.arange(5, 11)
    with_image = tokens.clone()
    with_image[positions] = 7
    masked = with_image.clone()
    masked[positions] = -100  # this framework marks the patch positions with a negative id, Llava with `image_token_index`
    mine = ours(masked, image_patches=patches, image_patch_positions=positions, image_patch_coordinates=coordinates)
    image = trainer._config.model.base_model.vision_encoder.normalization.normalize(pixels[None])  # what an image processor hands over
    with torch.no_grad():
        theirs = external(input_ids=with_image[None, :-1], pixel_values=image, image_sizes=[(8, 12)]).logits[0]
    torch.testing.assert_close(mine, theirs, rtol=5e-4, atol=5e-4)
    # generation keeps the prompt (image included) in the language model's cache: the image goes in once
    with torch.no_grad():
        cached = external.generate(with_image[None, :30], pixel_values=image, image_sizes=[(8, 12)], max_new_tokens=4, do_sample=False)
        plain = external.generate(with_image[None, :30], pixel_values=image, image_sizes=[(8, 12)], max_new_tokens=4, do_sample=False, use_cache=False)
    assert torch.equal(cached, plain)


def test_apriel2_multimodal_modeling_code_loads_the_export_and_reproduces_the_logits(tmp_path):
    """The stand-alone Apriel2 modelling files shipped with an `apriel2` export hold the classes its `auto_map` names, load every
    tensor of it, and give this framework's logits for text alone and for text with two images of different sizes."""
    import json

    from fast_llm_b200.data.document import LanguageModelBatch, LanguageModelDocument
    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from fast_llm_b200.external_models.apriel2 import modeling_apriel2
    from fast_llm_b200.parallel.topology import PhaseType

    trainer, _ = build_trainer(_config({("model", "base_model", "image_token_index"): 7}))
    path = tmp_path / "apriel2"
    trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format="apriel2"))
    auto_map = json.loads((path / "config.json").read_text())["auto_map"]
    for target in auto_map.values():
        file, name = target.split(".")
        assert (path / f"{file}.py").exists(), target
        assert f"class {name}(" in (path / f"{file}.py").read_text(), target
    external, info = modeling_apriel2.Apriel2ForConditionalGeneration.from_pretrained(str(path), torch_dtype=torch.float32, output_loading_info=True)
    assert not info["missing_keys"] and not info["unexpected_keys"], info
    external.eval()

    model = trainer._multi_stage.base_model
    for stage in trainer._multi_stage.stages:
        stage.restore_parameters()

    def ours(tokens, **image):
        document = LanguageModelDocument(tokens=tokens, **image)
        batch = LanguageModelBatch.from_documents([document], tokens.numel())
        inputs = batch.get_model_inputs(micro_batch_size=tokens.numel() - 1)
        (ids, kwargs), = model.preprocess_batch(inputs, phase=PhaseType.inference, iteration=0)
        kwargs["return_logits"] = True
        hidden = None
        with torch.no_grad():
            for layer in model.get_layers():
                hidden = layer.forward(ids if hidden is None else hidden, kwargs)
        return kwargs["logits"]

    torch.manual_seed(0)
    tokens = torch.randint(8, 512, (41,))
    with torch.no_grad():
        theirs = external(input_ids=tokens[None, :-1]).logits[0]
    torch.testing.assert_close(ours(tokens), theirs, rtol=2e-4, atol=2e-4)

    # a 2 x 3 grid of 4 x 4 patches at tokens 5..10 and a 1 x 2 grid at tokens 20..21
    first, second = torch.randint(0, 256, (3, 8, 12), dtype=torch.uint8), torch.randint(0, 256, (3, 4, 8), dtype=torch.uint8)
    patches = torch.cat([first.view(3, 2, 4, 3, 4).permute(1, 3, 0, 2, 4).reshape(6, 3, 4, 4),
                         second.view(3, 1, 4, 2, 4).permute(1, 3, 0, 2, 4).reshape(2, 3, 4, 4)])
    coordinates = torch.tensor([[r, c] for r in range(2) for c in range(3)] + [[0, 0], [0, 1]])
    positions = torch.cat([torch.arange(5, 11), torch.arange(20, 22)])
    with_image = tokens.clone()
    with_image[positions] = 7
    masked = with_image.clone()
    masked[positions] = -100  # this framework marks the patch positions with a negative id, the export with `image_token_index`
    mine = ours(masked, image_patches=patches, image_patch_positions=positions, image_patch_coordinates=coordinates)
    normalize = trainer._config.model.base_model.vision_encoder.normalization.normalize
    with torch.no_grad():
        theirs = external(input_ids=with_image[None, :-1], pixel_values=[normalize(first[None])[0], normalize(second[None])[0]]).logits[0]
    torch.testing.assert_close(mine, theirs, rtol=5e-4, atol=5e-4)
    # the same through a padded batch with the true sizes
    padded = torch.zeros(2, 3, 8, 12)
    padded[0], padded[1, :, :4, :8] = normalize(first[None])[0], normalize(second[None])[0]
    with torch.no_grad():
        again = external(input_ids=with_image[None, :-1], pixel_values=padded, image_sizes=[(8, 12), (4, 8)]).logits[0]
    torch.testing.assert_close(again, theirs, rtol=1e-5, atol=1e-5)
    # generation with the cache: the images go in with the prompt only
    with torch.no_grad():
        cached = external.generate(with_image[None, :30], pixel_values=padded, image_sizes=[(8, 12), (4, 8)], max_new_tokens=5, do_sample=False)
        uncached = external.generate(with_image[None, :30], pixel_values=padded, image_sizes=[(8, 12), (4, 8)], max_new_tokens=5, do_sample=False,
                                     use_cache=False)
    assert torch.equal(cached, uncached)


def test_auto_classes_load_custom_exports_with_remote_code(tmp_path, monkeypatch):
    """What a user of an exported checkpoint does: `transformers.AutoModelForCausalLM.from_pretrained(path, trust_remote_code=True)`
    resolves `auto_map` to the modelling files shipped in the directory (copied into the dynamic-module cache and imported from
    there, with their relative imports), for the text-only and the multimodal custom architectures; `model_type` in the exported
    `config.json` is the type of the configuration class that loads it."""
    import json

    import transformers
    import transformers.dynamic_module_utils

    from fast_llm_b200.engine.checkpoint.config import CheckpointSaveConfig
    from tests.common import tiny_trainer_config

    monkeypatch.setattr(transformers.dynamic_module_utils, "HF_MODULES_CACHE", str(tmp_path / "modules"))
    block = copy.deepcopy(TINY_BASE_MODEL["decoder"]["block"])
    mamba = copy.deepcopy(block)
    mamba["mixer"] = {"type": "mamba", "d_inner": 64, "d_xb": 32, "state_size": 8, "dt_rank": 4, "add_linear_biases": False,
                      "convolution_layer": {"bias": {"enabled": True}}, "dt_layer": {"bias": {"enabled": True}}}
    hybrid_decoder = {"type": "pattern", "blocks": {"t": block, "m2": mamba}, "pattern": ["t", "m2"], "num_blocks": 2}
    hybrid = copy.deepcopy(TINY_BASE_MODEL)
    hybrid["decoder"] = hybrid_decoder
    cases = [
        ("apriel2_text", tiny_trainer_config({("model", "base_model"): hybrid}), "Apriel2ForCausalLM", "apriel2_text"),
        ("apriel_hybrid_ssm", tiny_trainer_config({("model", "base_model"): hybrid}), "AprielHybridSSMForCausalLM", "apriel_ssm_thinker_hybrid"),
        ("apriel2", _config({("model", "base_model", "image_token_index"): 7}), "Apriel2ForConditionalGeneration", "apriel2"),
        ("llava_hybrid_ssm", _config({("model", "base_model", "image_token_index"): 7, ("model", "base_model", "decoder"): hybrid_decoder,
                                      ("model", "base_model", "vision_encoder", "adapter", "intermediate_size"): 64}),
         "LlavaHybridForConditionalGeneration", "llava_hybrid"),
    ]
    for format_name, config, class_name, model_type in cases:
        trainer, _ = build_trainer(config)
        path = tmp_path / format_name
        trainer.multi_stage.save_checkpoint(CheckpointSaveConfig(path=path, format=format_name))
        assert json.loads((path / "config.json").read_text())["model_type"] == model_type
        model = transformers.AutoModelForCausalLM.from_pretrained(str(path), trust_remote_code=True, dtype=torch.float32)
        assert type(model).__name__ == class_name and type(model).__module__.startswith("transformers_modules"), format_name
        assert type(model.config).model_type == model_type
        tokens = torch.randint(8, 512, (1, 9))
        assert model.generate(tokens, max_new_tokens=2, do_sample=False).shape == (1, 11), format_name


def test_llava_created_by_transformers_imports_and_gives_its_logits(tmp_path):
    """The import direction: a Llava model (Pixtral vision tower, Mistral decoder) built and saved by `transformers` loads through
    `format: auto`, whichever of the three key spellings the file uses, and gives `transformers`' logits for text and for text
    with an image."""
    import safetensors.torch
    import transformers

    from fast_llm_b200.data.document import LanguageModelBatch, LanguageModelDocument
    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.models.multimodal.conversion import LlavaHuggingfaceCheckpointHandler
    from fast_llm_b200.models.multimodal.model import MultiModalModel
    from fast_llm_b200.parallel.topology import PhaseType

    text = transformers.MistralConfig(vocab_size=320, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=2, head_dim=12, sliding_window=None)
    vision = transformers.PixtralVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, head_dim=16,
                                              patch_size=4, image_size=16, num_channels=3)
    config = transformers.LlavaConfig(vision_config=vision, text_config=text, image_token_index=7, projector_hidden_act="gelu",
                                      vision_feature_layer=-1, vision_feature_select_strategy="full", multimodal_projector_bias=True)
    torch.manual_seed(0)
    hf = transformers.LlavaForConditionalGeneration(config).eval()
    hf.save_pretrained(tmp_path / "saved", safe_serialization=True)
    # the same weights under the in-memory names of recent `transformers` (`model.language_model.*`, `lm_head.*`)
    (tmp_path / "in_memory_names").mkdir()
    safetensors.torch.save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(tmp_path / "in_memory_names/model.safetensors"),
                                metadata={"format": "pt"})
    (tmp_path / "in_memory_names/config.json").write_text((tmp_path / "saved/config.json").read_text())
    assert {LlavaHuggingfaceCheckpointHandler._legacy_name(k) for k in hf.state_dict()} == \
        {LlavaHuggingfaceCheckpointHandler._legacy_name(k) for k in safetensors.torch.load_file(str(tmp_path / "saved/model.safetensors"))}

    tokens = torch.randint(8, 320, (41,))
    pixels = torch.randint(0, 256, (3, 8, 12), dtype=torch.uint8)
    patches = pixels.view(3, 2, 4, 3, 4).permute(1, 3, 0, 2, 4).reshape(6, 3, 4, 4)
    coordinates = torch.tensor([[r, c] for r in range(2) for c in range(3)])
    positions = torch.arange(5, 11)
    with_image = tokens.clone()
    with_image[positions] = 7
    masked = with_image.clone()
    masked[positions] = -100
    for directory in ("saved", "in_memory_names"):
        model = MultiModalModel.from_pretrained(CheckpointLoadConfig(path=tmp_path / directory, format="auto"), use_cpu=True)
        base = model.base_model
        for stage in model.stages:
            stage.restore_parameters()

        def ours(ids, **image):
            batch = LanguageModelBatch.from_documents([LanguageModelDocument(tokens=ids, **image)], ids.numel())
            (inputs, kwargs), = base.preprocess_batch(batch.get_model_inputs(micro_batch_size=ids.numel() - 1), phase=PhaseType.inference, iteration=0)
            kwargs["return_logits"] = True
            hidden = None
            with torch.no_grad():
                for layer in base.get_layers():
                    hidden = layer.forward(inputs if hidden is None else hidden, kwargs)
            return kwargs["logits"]

        with torch.no_grad():
            expected = hf(input_ids=tokens[None, :-1]).logits[0]
        torch.testing.assert_close(ours(tokens), expected, rtol=2e-4, atol=2e-4)
        image = model.config.base_model.vision_encoder.normalization.normalize(pixels[None])
        with torch.no_grad():
            expected = hf(input_ids=with_image[None, :-1], pixel_values=image, image_sizes=[(8, 12)]).logits[0]
        mine = ours(masked, image_patches=patches, image_patch_positions=positions, image_patch_coordinates=coordinates)
        torch.testing.assert_close(mine, expected, rtol=5e-4, atol=5e-4)
