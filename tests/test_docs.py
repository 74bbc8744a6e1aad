"""The user documentation stays true: every tagged YAML block under `docs/` is a valid configuration of the command its
first line names, relative links resolve, and the quick-start flow (prepare -> train -> export -> convert -> generate) runs
on CPU with the documented files scaled down."""

import json
import pathlib
import re

import pytest
import torch
import yaml

DOCS = pathlib.Path(__file__).resolve().parents[1] / "docs"
PAGES = sorted(p for p in DOCS.rglob("*.md") if "reference" not in p.relative_to(DOCS).parts)


def _blocks():
    for page in PAGES:
        for index, block in enumerate(re.findall(r"```yaml\n(.*?)```", page.read_text(), re.S)):
            first = block.splitlines()[0]
            if first.startswith("# fast-llm "):
                yield pytest.param(page, first[len("# fast-llm "):].split("(")[0].split(), block, id=f"{page.relative_to(DOCS)}#{index}")


def _config_class(command):
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.config.runnable import RunnableConfig

    cls = RunnableConfig
    for word in command:
        cls = cls.get_subclass(word)
    return cls


@pytest.mark.parametrize("page,command,block", list(_blocks()))
def test_yaml_blocks_are_valid_configurations(page, command, block):
    from fast_llm_b200.config.core import NoAutoValidate

    cls = _config_class(command)
    with NoAutoValidate():
        config = cls.from_dict(yaml.safe_load(block))  # unknown keys and unknown `type:` names fail here
    try:
        config.validate()
    except (FileNotFoundError, OSError):
        pass  # the block names checkpoints, datasets or tokenizers of the reader's machine


def test_there_are_blocks_to_check():
    assert len(list(_blocks())) >= 12


@pytest.mark.parametrize("page", PAGES, ids=lambda p: str(p.relative_to(DOCS)))
def test_relative_links_resolve(page):
    for target in re.findall(r"\]\(([^)#]+)(?:#[^)]*)?\)", page.read_text()):
        if "://" in target:
            continue
        assert (page.parent / target).exists(), f"{page.relative_to(DOCS)} links to {target}"


def test_quick_start_flow(tmp_path, monkeypatch):
    """The commands of docs/quick-start.md, on a corpus of a few lines and a model of two tiny blocks."""
    import tokenizers
    import transformers

    from fast_llm_b200.cli import fast_llm_main

    monkeypatch.chdir(tmp_path)
    corpus = ["the quick brown fox jumps over the lazy dog", "pack my box with five dozen liquor jugs", "hello world, this is a test"] * 30
    (tmp_path / "corpus.jsonl").write_text("\n".join(json.dumps({"text": f"{line} {i}"}) for i, line in enumerate(corpus)))
    tok = tokenizers.Tokenizer(tokenizers.models.BPE())
    tok.pre_tokenizer = tokenizers.pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    tok.train_from_iterator(corpus, tokenizers.trainers.BpeTrainer(vocab_size=300, initial_alphabet=tokenizers.pre_tokenizers.ByteLevel.alphabet(),
                                                                   special_tokens=["<s>", "</s>"]))
    transformers.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>").save_pretrained(str(tmp_path / "tokenizer_dir"))

    quick_start = (DOCS / "quick-start.md").read_text()
    prepare, train = (yaml.safe_load(block) for block in re.findall(r"```yaml\n(.*?)```", quick_start, re.S)[:2])
    prepare.update(documents_per_shard=50, num_workers=1, splits={"training": 0.8, "validation": 0.2})
    (tmp_path / "prepare.yaml").write_text(yaml.safe_dump(prepare))
    fast_llm_main(["prepare", "gpt_memmap", "-c", "prepare.yaml"])
    assert (tmp_path / "data/my_corpus/fast_llm_config_training.yaml").exists()

    # the documented training file, scaled down by command-line overrides (the mechanism the page describes)
    (tmp_path / "train.yaml").write_text(yaml.safe_dump(train))
    block = "model.base_model.decoder.block"
    overrides = [
        "training.train_iters=4", "training.logs.interval=1", "training.checkpoint.interval=2", "training.export.interval=4", "training.num_workers=0",
        "training.evaluators.validation.interval=2", "training.evaluators.validation.iterations=1",
        "data.micro_batch_size=64", "data.maximum_document_length=64", "schedule.depth_first_micro_batches=1",
        "optimizer.learning_rate.decay_iterations=4", "optimizer.learning_rate.warmup_iterations=1",
        "model.base_model.embeddings.vocab_size=300", "model.base_model.hidden_size=32", "model.base_model.decoder.num_blocks=2",
        f"{block}.mixer.heads=4", f"{block}.mixer.head_groups=2", f"{block}.mixer.head_size=8", f"{block}.mlp.intermediate_size=64",
        "model.distributed.compute_dtype=float32", "model.distributed.use_cuda=false",
    ]
    fast_llm_main(["train", "gpt", "-c", "train.yaml", *overrides])
    run = tmp_path / "runs/quick_start"
    assert (run / "config.yaml").exists() and (run / "checkpoint/4/ok").exists() and (run / "export/llama/4/config.json").exists()
    assert list((run / "runs/0/logs").glob("logs_rank_*.txt"))

    fast_llm_main(["convert", "gpt", "input.path=runs/quick_start/checkpoint/4", "input.format=distributed", "output.path=exported",
                   "output.format=llama", "use_cpu=true"])
    reference = transformers.AutoModelForCausalLM.from_pretrained(str(run / "export/llama/4"), torch_dtype=torch.float32)
    converted = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "exported"), torch_dtype=torch.float32)
    for (name, a), (_, b) in zip(reference.state_dict().items(), converted.state_dict().items()):
        torch.testing.assert_close(a, b, msg=lambda m: f"{name}: {m}")

    from fast_llm_b200.engine.checkpoint.config import CheckpointLoadConfig
    from fast_llm_b200.engine.inference.huggingface import HuggingfaceGPTModelForCausalLM

    model = HuggingfaceGPTModelForCausalLM.from_pretrained(CheckpointLoadConfig(path="exported", format="llama"), use_cpu=True)
    prompt = torch.randint(2, 300, (2, 5))
    tokens = model.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=3, do_sample=False, pad_token_id=0)
    with torch.no_grad():
        expected = reference.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=3, do_sample=False, pad_token_id=0)
    assert torch.equal(tokens, expected)


def _tiny_tokenizer(path, corpus, chat_template=None):
    import tokenizers
    import transformers

    tok = tokenizers.Tokenizer(tokenizers.models.BPE())
    tok.pre_tokenizer = tokenizers.pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    tok.train_from_iterator(corpus, tokenizers.trainers.BpeTrainer(vocab_size=300, initial_alphabet=tokenizers.pre_tokenizers.ByteLevel.alphabet(),
                                                                   special_tokens=["<s>", "</s>", "<u>", "<a>"]))
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>")
    if chat_template:
        fast.chat_template = chat_template
    fast.save_pretrained(str(path))


_TINY = ["model.base_model.embeddings.vocab_size=300", "model.base_model.hidden_size=32", "model.base_model.decoder.num_blocks=2",
         "model.base_model.decoder.block.mixer.heads=4", "model.base_model.decoder.block.mixer.head_groups=2",
         "model.base_model.decoder.block.mixer.head_size=8", "model.base_model.decoder.block.mixer.add_linear_biases=false",
         "model.base_model.decoder.block.mixer.rotary.type=default", "model.base_model.decoder.block.mlp.intermediate_size=64",
         "model.base_model.decoder.block.mlp.gated=true", "model.base_model.decoder.block.mlp.add_linear_biases=false",
         "model.base_model.decoder.block.normalization.type=rms_norm", "model.base_model.head.normalization.type=rms_norm"]
_CPU = ["model.distributed.compute_dtype=float32", "model.distributed.use_cuda=false", "training.num_workers=0", "training.logs.interval=1"]


def _doc_block(page: str, index: int) -> dict:
    return yaml.safe_load(re.findall(r"```yaml\n(.*?)```", (DOCS / page).read_text(), re.S)[index])


def test_fine_tuning_and_continued_training_recipes(tmp_path, monkeypatch):
    """docs/recipes/instruction-finetuning.md and continue-training.md: chat data through the conversation schema, a pretrained
    Llama checkpoint continued with whole documents, LoRA on top, then `fast-llm evaluate` on the result."""
    from fast_llm_b200.cli import fast_llm_main

    monkeypatch.chdir(tmp_path)
    template = ("{% for m in messages %}{% if m['role'] == 'assistant' %}<a>{% generation %}{{ m['content'] }}</s>{% endgeneration %}"
                "{% else %}<u>{{ m['content'] }}{% endif %}{% endfor %}")
    lines = ["the quick brown fox", "jumps over the lazy dog", "hello world", "this is a test"]
    _tiny_tokenizer(tmp_path / "tokenizer", lines * 10, template)
    rows = [{"messages": [{"role": "user", "content": lines[i % 4]}, {"role": "assistant", "content": lines[(i + 1) % 4] + f" {i}"}]} for i in range(60)]
    (tmp_path / "chat.jsonl").write_text("\n".join(json.dumps(r) for r in rows))

    # a "pretrained" Llama checkpoint: two iterations of the tiny model, exported
    fast_llm_main(["train", "gpt", "run.experiment_dir=base", "training.train_iters=1", "training.export.interval=1", "training.export.format=llama",
                   "data.datasets.training.type=random", "data.micro_batch_size=64", *_TINY, *_CPU])
    pretrained = tmp_path / "base/export/llama/1"
    assert (pretrained / "config.json").exists()

    prepare = _doc_block("recipes/instruction-finetuning.md", 0)
    prepare["dataset"].update(path="json", data_files="chat.jsonl", split="train")
    prepare.update(output_path="sft_data", tokenizer={"path": "tokenizer"}, num_workers=1)
    (tmp_path / "prepare.yaml").write_text(yaml.safe_dump(prepare))
    fast_llm_main(["prepare", "gpt_memmap", "-c", "prepare.yaml"])

    train = _doc_block("recipes/instruction-finetuning.md", 1)
    train["pretrained"]["path"] = str(pretrained)
    train["data"]["datasets"]["training"]["path"] = "sft_data/fast_llm_config.yaml"
    train["model"]["base_model"] = _doc_block("recipes/instruction-finetuning.md", 2)["model"]["base_model"]  # the LoRA section
    train["run"]["experiment_dir"] = "sft"
    (tmp_path / "sft.yaml").write_text(yaml.safe_dump(train))
    fast_llm_main(["train", "gpt", "-c", "sft.yaml", "training.train_iters=2", "training.export.interval=2", "data.micro_batch_size=64",
                   "data.maximum_document_length=64", "optimizer.learning_rate.decay_iterations=2", "optimizer.learning_rate.warmup_iterations=1", *_CPU])
    assert (tmp_path / "sft/export/llama/2/config.json").exists()
    sft_config = yaml.safe_load((tmp_path / "sft/config.yaml").read_text())
    assert sft_config["model"]["base_model"]["peft"]["type"] == "lora"

    # continued training + evaluation from the documented files
    evaluate = _doc_block("recipes/generate.md", 0)
    evaluate["pretrained"] = {"path": str(pretrained), "format": "llama"}
    evaluate["training"]["evaluators"].pop("harness")  # needs the lm-eval package and its task data
    evaluate["data"]["datasets"]["validation"] = {"type": "file", "path": "sft_data/fast_llm_config.yaml"}
    evaluate["run"] = {"experiment_dir": "evaluation"}
    (tmp_path / "evaluate.yaml").write_text(yaml.safe_dump(evaluate))
    fast_llm_main(["evaluate", "gpt", "-c", "evaluate.yaml", "training.evaluators.validation.iterations=2", "data.micro_batch_size=64",
                   "model.distributed.compute_dtype=float32", "model.distributed.use_cuda=false", "training.num_workers=0"])
    logs = "".join(p.read_text() for p in (tmp_path / "evaluation/runs/0/logs").glob("*.txt"))
    assert "validation @ validation" in logs and "lm loss" in logs


def test_upcycling_recipe(tmp_path, monkeypatch):
    """docs/recipes/upcycle-to-moe.md: a Mixtral-style export, `add_experts`, then training from the result."""
    from fast_llm_b200.cli import fast_llm_main
    from fast_llm_b200.tools import checkpoint_surgery  # noqa: F401  (registers the commands)

    monkeypatch.chdir(tmp_path)
    moe = ["model.base_model.decoder.block.mlp.type=moe", "model.base_model.decoder.block.mlp.experts=2", "model.base_model.decoder.block.mlp.experts_per_token=1"]
    fast_llm_main(["train", "gpt", "run.experiment_dir=base", "training.train_iters=1", "training.export.interval=1", "training.export.format=mixtral",
                   "data.datasets.training.type=random", "data.micro_batch_size=64", *_TINY, *moe, *_CPU])
    source = tmp_path / "base/export/mixtral/1"
    fast_llm_main(["add_experts", f"hf_checkpoint={source}", "output_dir=upcycled", "num_new_experts=2", "expert_init_method=from_existing",
                   "expert_init_std=0.01", "router_init_method=from_scratch", "router_init_std=0.02", "seed=0"])
    assert json.loads((tmp_path / "upcycled/config.json").read_text())["num_local_experts"] == 4

    train = _doc_block("recipes/upcycle-to-moe.md", 0)
    train["pretrained"]["path"] = "upcycled"
    train["data"]["datasets"]["training"] = {"type": "random"}
    train["run"]["experiment_dir"] = "upcycled_run"
    (tmp_path / "train.yaml").write_text(yaml.safe_dump(train))
    fast_llm_main(["train", "gpt", "-c", "train.yaml", "training.train_iters=2", "training.checkpoint.interval=2", "data.micro_batch_size=64",
                   "optimizer.learning_rate.decay_iterations=2", "optimizer.learning_rate.warmup_iterations=1", *_CPU])
    saved = yaml.safe_load((tmp_path / "upcycled_run/checkpoint/2/metadata.yaml").read_text())
    assert "experts: 4" in yaml.safe_dump(saved)


def test_multimodal_recipe(tmp_path, monkeypatch):
    """docs/recipes/multimodal.md: a dataset with an Image feature (rows with zero, one and two pictures of two sizes) is
    prepared into patches, a tiny vision-language model trains on it, and the Llava export loads in `transformers`."""
    import datasets
    import numpy as np
    import PIL.Image
    import transformers

    from fast_llm_b200.cli import fast_llm_main

    monkeypatch.chdir(tmp_path)
    lines = ["the quick brown fox", "jumps over the lazy dog", "hello world", "this is a test"]
    _tiny_tokenizer(tmp_path / "tokenizer", lines * 10)
    rng = np.random.RandomState(0)
    rows = {"text": [], "images": [], "positions": []}
    for i in range(40):
        count = i % 3
        rows["text"].append(f"{lines[i % 4]} and {lines[(i + 1) % 4]} {i}")
        rows["images"].append([PIL.Image.fromarray(rng.randint(0, 256, size=(8 + 4 * (i % 2), 12, 3)).astype(np.uint8)) for _ in range(count)])
        rows["positions"].append([3 + 5 * k for k in range(count)])
    features = datasets.Features({"text": datasets.Value("string"), "images": datasets.Sequence(datasets.Image()),
                                  "positions": datasets.Sequence(datasets.Value("int32"))})
    datasets.Dataset.from_dict(rows, features=features).save_to_disk(str(tmp_path / "raw"))

    prepare = _doc_block("recipes/multimodal.md", 0)
    prepare["dataset"]["path"] = "raw"
    prepare.update(output_path="captions", tokenizer={"path": "tokenizer"}, num_workers=1, documents_per_shard=16)
    prepare["image_patches"].update(height=4, width=4, max_image_height=16, max_image_width=16, image_break_token=None, image_end_token=None)
    (tmp_path / "prepare.yaml").write_text(yaml.safe_dump(prepare))
    fast_llm_main(["prepare", "gpt_memmap", "-c", "prepare.yaml"])

    train = _doc_block("recipes/multimodal.md", 1)
    train["data"]["datasets"]["training"]["path"] = "captions/fast_llm_config.yaml"
    (tmp_path / "train.yaml").write_text(yaml.safe_dump(train))
    vision = "model.base_model.vision_encoder"
    fast_llm_main(["train", "multimodal", "-c", "train.yaml", "training.train_iters=3", "training.checkpoint.interval=null", "training.export.interval=3",
                   "data.micro_batch_size=96", "data.maximum_document_length=96", "optimizer.learning_rate.decay_iterations=3",
                   "optimizer.learning_rate.warmup_iterations=1", "model.base_model.image_token_index=7", *_TINY,
                   f"{vision}.hidden_size=32", f"{vision}.embeddings.patch_height=4", f"{vision}.embeddings.patch_width=4", f"{vision}.encoder.num_blocks=2",
                   f"{vision}.encoder.block.mixer.heads=2", f"{vision}.encoder.block.mixer.head_groups=2", f"{vision}.encoder.block.mixer.head_size=16",
                   f"{vision}.encoder.block.mlp.intermediate_size=64", f"{vision}.adapter.intermediate_size=32", *_CPU])
    export = tmp_path / "runs/vlm/export/llava/3"
    model, info = transformers.LlavaForConditionalGeneration.from_pretrained(str(export), torch_dtype=torch.float32, output_loading_info=True)
    assert not info["missing_keys"] and not info["unexpected_keys"], info


def test_reference_model_flows(tmp_path, monkeypatch):
    """Losses that need a frozen reference model, driven from the command line as docs/recipes/train.md and
    instruction-finetuning.md describe them: distillation from a teacher checkpoint, and DPO on prepared preference pairs
    (policy and reference start equal, so the first loss is ln 2)."""
    import math

    from fast_llm_b200.cli import fast_llm_main

    monkeypatch.chdir(tmp_path)
    fast_llm_main(["train", "gpt", "run.experiment_dir=base", "training.train_iters=1", "training.export.interval=1", "training.export.format=llama",
                   "data.datasets.training.type=random", "data.micro_batch_size=64", *_TINY, *_CPU])
    teacher = str(tmp_path / "base/export/llama/1")

    def losses(run: str, name: str) -> list[float]:
        logs = "".join(p.read_text() for p in (tmp_path / run / "runs/0/logs").glob("*.txt"))
        return [float(v) for v in re.findall(rf"training iteration .*\| {name}: ([0-9.]+)", logs)]

    distill = {"run": {"experiment_dir": "distill"}, "training": {"train_iters": 3},
               "reference_models": {"teacher": {"pretrained": {"path": teacher, "format": "llama"}}},
               "data": {"datasets": {"training": {"type": "random"}}, "micro_batch_size": 64},
               "model": {"base_model": {"head": {"losses": {"lm": {"type": "label", "weight": 0.5},
                                                            "distill": {"type": "distillation", "reference_model": "teacher", "weight": 0.5}}}}}}
    (tmp_path / "distill.yaml").write_text(yaml.safe_dump(distill))
    fast_llm_main(["train", "gpt", "-c", "distill.yaml", *_TINY, *_CPU])
    assert len(losses("distill", "distill")) == 3 and len(losses("distill", "lm")) == 3

    lines = ["the quick brown fox", "jumps over the lazy dog", "hello world", "this is a test"]
    _tiny_tokenizer(tmp_path / "tokenizer", lines * 10)
    rows = []
    for i in range(60):
        prompt, chosen, rejected = f"{lines[i % 4]} {i} : ", lines[(i + 1) % 4], lines[(i + 2) % 4]
        rows.append({"text": prompt + chosen + rejected, "chosen": [len(prompt), len(prompt) + len(chosen)],
                     "rejected": [len(prompt) + len(chosen), len(prompt) + len(chosen) + len(rejected)]})
    (tmp_path / "prefs.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    prepare = {"output_path": "prefs", "tokenizer": {"path": "tokenizer"},
               "dataset": {"path": "json", "data_files": "prefs.jsonl",
                           "source_schema": {"type": "document", "text": "text", "chosen_span": "chosen", "rejected_span": "rejected"}}}
    (tmp_path / "prepare.yaml").write_text(yaml.safe_dump(prepare))
    fast_llm_main(["prepare", "gpt_memmap", "-c", "prepare.yaml"])
    dpo = {"run": {"experiment_dir": "dpo"}, "training": {"train_iters": 3}, "pretrained": {"path": teacher, "format": "llama"},
           "reference_models": {"reference": {"pretrained": {"path": teacher, "format": "llama"}}},
           "data": {"datasets": {"training": {"type": "file", "path": "prefs/fast_llm_config.yaml"}}, "micro_batch_size": 64,
                    "maximum_document_length": 64, "truncate_documents": False},
           "model": {"base_model": {"head": {"losses": {"dpo": {"type": "dpo", "beta": 0.1, "reference_model": "reference"}}}}}}
    (tmp_path / "dpo.yaml").write_text(yaml.safe_dump(dpo))
    fast_llm_main(["train", "gpt", "-c", "dpo.yaml", *_CPU])
    values = losses("dpo", "dpo")
    assert len(values) == 3 and values[0] == pytest.approx(math.log(2), abs=1e-4) and values[-1] < values[0]


def test_configuration_reference_is_current(tmp_path):
    """`docs/reference/configuration` is what `tools/generate_config_docs` writes from the classes as they are now."""
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.tools import checkpoint_surgery, push_model  # noqa: F401  (their configs are part of the reference)
    from fast_llm_b200.tools.generate_config_docs import generate

    generate(tmp_path)
    committed = DOCS / "reference" / "configuration"
    fresh = {p.relative_to(tmp_path): p.read_text() for p in tmp_path.rglob("*.md")}
    current = {p.relative_to(committed): p.read_text() for p in committed.rglob("*.md")}
    assert sorted(fresh) == sorted(current), "pages added or removed: run python -m fast_llm_b200.tools.generate_config_docs"
    stale = [str(name) for name in fresh if fresh[name] != current[name]]
    assert not stale, f"stale pages (run python -m fast_llm_b200.tools.generate_config_docs): {stale[:10]}"


@pytest.mark.parametrize("name", ["tiny_llama.yaml", "mistral.yaml"])
def test_example_configurations_validate(name):
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.models.gpt.trainer import GPTTrainerConfig

    config = GPTTrainerConfig.from_dict(yaml.safe_load((DOCS.parent / "examples" / name).read_text()))
    config.validate()
    assert config.model.base_model.decoder.num_blocks >= 2


def test_launch_examples_parse():
    """The Slurm script is valid shell and the Kubeflow manifest valid YAML that starts the documented module."""
    import subprocess

    examples = DOCS.parent / "examples"
    subprocess.run(["bash", "-n", str(examples / "slurm_train.sbatch")], check=True)
    assert "fast_llm_b200.cli train gpt" in (examples / "slurm_train.sbatch").read_text()
    job = yaml.safe_load((examples / "pytorchjob.yaml").read_text())
    container = job["spec"]["pytorchReplicaSpecs"]["Worker"]["template"]["spec"]["containers"][0]
    assert container["command"] == ["torchrun"] and "fast_llm_b200.cli" in container["args"]
