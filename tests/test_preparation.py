"""Tokenizer, fill-in-the-middle and dataset preparation, on a tokenizer trained on the spot (no downloads)."""

import json

import numpy as np
import pytest
import torch
import yaml

CORPUS = ["the quick brown fox jumps over the lazy dog", "def add(a, b):\n    return a + b\n", "hello world, this is a test of the tokenizer",
          "pack my box with five dozen liquor jugs", "import numpy as np\nx = np.zeros(3)\n"] * 4

CHAT_TEMPLATE = ("{% for m in messages %}{% if m['role'] == 'assistant' %}<a>{% generation %}{{ m['content'] }}</s>{% endgeneration %}"
                 "{% else %}<u>{{ m['content'] }}{% endif %}{% endfor %}")


@pytest.fixture(scope="module")
def tokenizer_path(tmp_path_factory):
    import tokenizers
    import transformers

    tok = tokenizers.Tokenizer(tokenizers.models.BPE())
    tok.pre_tokenizer = tokenizers.pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    trainer = tokenizers.trainers.BpeTrainer(vocab_size=400, initial_alphabet=tokenizers.pre_tokenizers.ByteLevel.alphabet(),
                                             special_tokens=["<s>", "</s>", "<fim_prefix>", "<fim_middle>", "<fim_suffix>", "<fim_pad>", "<u>", "<a>"])
    tok.train_from_iterator(CORPUS, trainer)
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>")
    fast.chat_template = CHAT_TEMPLATE
    path = tmp_path_factory.mktemp("tokenizer")
    fast.save_pretrained(str(path))
    return path


def _tokenizer(path):
    from fast_llm_b200.data.config import TokenizerConfig

    return TokenizerConfig.from_dict({"path": str(path)}).get_tokenizer()


def test_tokenizer_round_trip_and_spans(tokenizer_path):
    tokenizer = _tokenizer(tokenizer_path)
    text = "the quick brown fox jumps"
    tokens = tokenizer.tokenize(text)
    assert tokens[0] == tokenizer.bod_id and tokens[-1] == tokenizer.eod_id
    assert tokenizer.detokenize(tokens, begin=True, end=True) == text
    assert len(tokenizer.tokenize(text, begin=False, end=False)) == len(tokens) - 2
    spans = [(4, 9), (16, 19)]
    tokens, token_spans = tokenizer.tokenize_with_spans(text, text_spans=spans)
    for (tb, te), (cb, ce) in zip(token_spans, spans):
        assert tokenizer.detokenize(tokens[tb:te]) == text[cb:ce]
    recovered, text_spans = tokenizer.detokenize_with_spans(tokens, begin=True, end=True, token_spans=token_spans)
    assert recovered == text and text_spans == spans


def test_tokenize_chat_masks_everything_but_assistant_turns(tokenizer_path):
    tokenizer = _tokenizer(tokenizer_path)
    tokenizer.validate_chat_template()
    messages = [{"role": "user", "content": "hello world"}, {"role": "assistant", "content": "the lazy dog"},
                {"role": "user", "content": "a test"}, {"role": "assistant", "content": "quick fox"}]
    tokens, spans = tokenizer.tokenize_chat(messages)
    trained = torch.ones(len(tokens), dtype=torch.bool)
    for begin, end in spans:
        trained[begin:end] = False
    text = tokenizer.detokenize(tokens[trained])
    assert text == "the lazy dog</s>quick fox</s>"


def test_fim_keeps_length_and_content(tokenizer_path):
    from fast_llm_b200.data.config import GPTFimSampledDatasetConfig, SamplingConfig

    tokenizer = _tokenizer(tokenizer_path)

    class Source:
        name = "source"

        def __len__(self):
            return 8

        def __getitem__(self, index):
            from fast_llm_b200.data.document import LanguageModelDocument

            parts = [tokenizer.tokenize(CORPUS[(index + i) % 5], begin=False, end=True) for i in range(3)]
            return [LanguageModelDocument(tokens=torch.cat(parts))]

    config = GPTFimSampledDatasetConfig.from_dict({"type": "fim", "rate": 1.0, "spm_rate": 0.5, "tokenizer": {"path": str(tokenizer_path)},
                                                   "dataset": {"type": "random"}})
    from fast_llm_b200.data.fim import GPTFimDataset

    dataset = GPTFimDataset(config, Source(), SamplingConfig.from_dict({}), seed=3)
    vocab = tokenizer.vocab
    sentinels = {vocab[t] for t in ("<fim_prefix>", "<fim_middle>", "<fim_suffix>", "<fim_pad>")}
    seen_orders = set()
    for index in range(8):
        (original,), (transformed,) = Source()[index], dataset[index]
        assert len(transformed.tokens) == len(original.tokens)
        assert torch.equal(dataset[index][0].tokens, transformed.tokens)  # deterministic per index
        ids = transformed.tokens.tolist()
        assert vocab["<fim_middle>"] in ids
        first = ids.index(vocab["<fim_prefix>"])
        seen_orders.add("spm" if ids[first + 1] == vocab["<fim_suffix>"] else "psm")
        # undo the first document's permutation (prefix-suffix-middle order) and compare with the source text
        p, s_, m = first, ids.index(vocab["<fim_suffix>"]), ids.index(vocab["<fim_middle>"])
        if s_ > p + 1:
            strip = lambda piece: [t for t in piece if t not in (tokenizer.bod_id, tokenizer.eod_id)]
            rest = ids[m + 1 :]
            stop = min([rest.index(t) for t in (tokenizer.eod_id, *sentinels) if t in rest], default=len(rest))
            prefix, suffix, middle = strip(ids[p + 1 : s_]), strip(ids[s_ + 1 : m]), rest[:stop]
            assert tokenizer.detokenize(prefix) + tokenizer.detokenize(middle) + tokenizer.detokenize(suffix) == CORPUS[index % 5]
    assert seen_orders == {"spm", "psm"}


def test_prepare_gpt_memmap_with_spans_and_splits(tokenizer_path, tmp_path):
    import fast_llm_b200.models.auto  # noqa: F401
    from fast_llm_b200.data.config import SampledDatasetConfig
    from fast_llm_b200.data.preparation.config import GPTMemmapDatasetPreparatorConfig

    rows = [{"text": CORPUS[i % 5] + f" number {i}", "spans": [[0, 3], [10, 15]]} for i in range(40)]
    source = tmp_path / "source.jsonl"
    source.write_text("\n".join(json.dumps(r) for r in rows))
    config = GPTMemmapDatasetPreparatorConfig.from_dict({
        "output_path": str(tmp_path / "out"), "documents_per_shard": 16, "tokenizer": {"path": str(tokenizer_path)},
        "dataset": {"path": "json", "data_files": str(source), "source_schema": {"text": "text", "loss_masking_spans": "spans"}},
        "splits": {"training": 0.8, "validation": 0.2}, "distributed": {"world_size": 1, "rank": 0}})
    config.validate()
    config.get_dataset_preparator_class()(config).run()
    out = tmp_path / "out"
    assert len(list(out.glob("shard_0_*.fast_llm_dataset"))) == 3
    tokenizer = _tokenizer(tokenizer_path)
    totals = {}
    for split in ("training", "validation"):
        saved = yaml.safe_load((out / f"fast_llm_config_{split}.yaml").read_text())
        totals[split] = saved["metadata"]["num_tokens"]
        from fast_llm_b200.data.config import _resolve_paths

        dataset_config = SampledDatasetConfig.from_dict(_resolve_paths(saved["config"], out))
        assert dataset_config is not None
    assert 0.7 < totals["training"] / (totals["training"] + totals["validation"]) < 0.9
    # a document read back: tokens decode to the text, spans point at the masked characters
    from fast_llm_b200.data.memmap import MemmapDataset

    shard = MemmapDataset("shard", out / "shard_0_0.fast_llm_dataset")
    document = shard.get_document(0)
    text = tokenizer.detokenize(document.tokens.to(torch.int64), begin=True, end=True)
    assert text in {r["text"] for r in rows}
    (b0, e0), (b1, e1) = document.loss_masking_spans
    assert tokenizer.detokenize(document.tokens[b0:e0].to(torch.int64)) == text[0:3]
    assert tokenizer.detokenize(document.tokens[b1:e1].to(torch.int64)) == text[10:15]


def test_prepare_conversations_images_and_discovery(tokenizer_path, tmp_path):
    from fast_llm_b200.data.preparation.config import DatasetDiscoveryConfig, GPTMemmapDatasetPreparatorConfig

    chat = GPTMemmapDatasetPreparatorConfig.from_dict({
        "output_path": str(tmp_path / "chat"), "tokenizer": {"path": str(tokenizer_path)},
        "dataset": {"path": "json", "source_schema": {"type": "conversation"}}, "distributed": {"world_size": 1, "rank": 0}})
    chat.validate()
    preparator = chat.get_dataset_preparator_class()(chat)
    document = preparator.prepare_document({"messages": [{"role": "user", "content": "hello"}, {"role": "assistant", "content": "world"}]})
    tokenizer = _tokenizer(tokenizer_path)
    kept = torch.ones(len(document.tokens), dtype=torch.bool)
    for b, e in document.loss_masking_spans:
        kept[b:e] = False
    assert tokenizer.detokenize(document.tokens[kept].to(torch.int64)) == "world</s>"

    images = GPTMemmapDatasetPreparatorConfig.from_dict({
        "output_path": str(tmp_path / "images"), "tokenizer": {"path": str(tokenizer_path)},
        "image_patches": {"height": 4, "width": 4, "max_image_height": 16, "max_image_width": 16, "image_break_token": 7, "image_end_token": 8, "placeholder_token": 6},
        "dataset": {"path": "json", "source_schema": {"text": "text", "images": "images", "image_positions": "positions"}},
        "distributed": {"world_size": 1, "rank": 0}})
    images.validate()
    preparator = images.get_dataset_preparator_class()(images)
    picture = np.random.RandomState(0).randint(0, 256, size=(8, 12, 3)).astype(np.uint8)
    document = preparator.prepare_document({"text": "hello world", "images": [picture], "positions": [5]})
    assert document.image_patches.shape == (6, 3, 4, 4)  # 2 rows x 3 columns
    ids = document.tokens.tolist()
    assert [ids[p] for p in document.image_patch_positions.tolist()] == [6] * 6
    assert ids.count(7) == 1 and ids.count(8) == 1
    assert document.image_patch_coordinates.tolist() == [[0, 0], [0, 1], [0, 2], [1, 0], [1, 1], [1, 2]]
    # top-left patch holds the top-left pixels
    assert torch.equal(document.image_patches[0], torch.from_numpy(picture[:4, :4]).permute(2, 0, 1))
    text_tokens = [t for t in ids if t not in (6, 7, 8)]
    assert tokenizer.detokenize(text_tokens, begin=True, end=True) == "hello world"

    # discovery over a tree of prepared files
    from fast_llm_b200.data.document import LanguageModelDocument
    from fast_llm_b200.data.memmap import MemmapDataset

    for name, count in (("a/x", 3), ("a/y", 5), ("b/z", 2)):
        MemmapDataset.write_dataset(tmp_path / "tree" / f"{name}.fast_llm_dataset",
                                    [LanguageModelDocument(tokens=torch.arange(10, dtype=torch.int32)) for _ in range(count)])
    discovery = DatasetDiscoveryConfig.from_dict({"directory": str(tmp_path / "tree"), "output": str(tmp_path / "tree.yaml")})
    discovery.validate()
    discovery.get_dataset_preparator_class()(discovery).run()
    found = yaml.safe_load((tmp_path / "tree.yaml").read_text())
    assert found["metadata"]["num_tokens"] == 100
    assert found["config"]["type"] == "blended" and found["config"]["weights"] == [80, 20]
