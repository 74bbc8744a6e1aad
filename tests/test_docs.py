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
