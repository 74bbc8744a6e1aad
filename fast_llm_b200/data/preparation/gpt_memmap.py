"""Tokenize a Hugging Face dataset into sharded memmap files and write the dataset configs that read them back.

Work is split three ways: ranks (`distributed`) take interleaved slices of the dataset, every rank cuts its slice into
shards of `documents_per_shard`, and a pool of `num_workers` processes tokenizes shards in parallel, each writing one
`shard_<rank>_<index>.fast_llm_dataset`.  Rank 0 then writes `fast_llm_config.yaml` (one memmap dataset, or a blend
weighted by token counts) - or, with `splits`, one config per split whose boundaries fall inside shards as `slice`s.
Parity: `fast_llm/data/preparation/gpt_memmap/prepare.py:57-522`.
"""

import datetime
import logging
import math
import multiprocessing
import pathlib

import numpy as np
import torch
import yaml

from fast_llm_b200.data.document import LanguageModelDocument
from fast_llm_b200.data.memmap import MemmapDataset
from fast_llm_b200.data.preparation.config import ConversationSourceConfig, GPTMemmapDatasetPreparatorConfig
from fast_llm_b200.data.preparation.image_patch import image_to_patches, image_token_layout
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


def unsigned_dtype_for(vocab_size: int) -> torch.dtype:
    """Smallest torch integer type holding every token id (torch has no uint32: int32 covers up to 2^31)."""
    if vocab_size <= 2**16:
        return torch.uint16
    return torch.int32 if vocab_size <= 2**31 else torch.int64


class GPTMemmapDatasetPreparator:
    def __init__(self, config: GPTMemmapDatasetPreparatorConfig):
        self._config = config
        self._schema = config.dataset.source_schema
        self._tokenizer = None

    # ---- loading
    def _load_dataset(self):
        import datasets

        c = self._config.dataset
        if c.load_from_disk:
            loaded = datasets.load_from_disk(str(c.path))
            return loaded[c.split] if isinstance(loaded, datasets.DatasetDict) else loaded
        return datasets.load_dataset(path=str(c.path), name=c.config_name, data_dir=c.data_directory, data_files=c.data_files, split=c.split,
                                     num_proc=self._config.num_workers if self._config.num_workers > 1 else None)

    def run(self) -> None:
        c = self._config
        self._setup_tokenizer()
        distributed = c.distributed
        if distributed.world_size > 1:
            torch.distributed.init_process_group(backend=distributed.backend, rank=distributed.rank, world_size=distributed.world_size,
                                                 timeout=datetime.timedelta(seconds=distributed.timeout))
        c.output_path.mkdir(parents=True, exist_ok=True)
        if distributed.world_size > 1 and distributed.rank != 0:
            torch.distributed.barrier()  # rank 0 populates the datasets cache first
        dataset = self._load_dataset()
        if distributed.world_size > 1 and distributed.rank == 0:
            torch.distributed.barrier()
        dataset = dataset.shard(num_shards=distributed.world_size, index=distributed.rank)
        for column in self._schema.columns:
            if column not in dataset.column_names:
                raise ValueError(f"The dataset has no column '{column}' (columns: {dataset.column_names})")
        num_shards = max(math.ceil(len(dataset) / c.documents_per_shard), 1)
        shards = [(i, dataset.shard(num_shards=num_shards, index=i)) for i in range(num_shards)]
        if c.num_workers > 1 and len(shards) > 1:
            with multiprocessing.get_context("fork").Pool(processes=c.num_workers) as pool:
                results = pool.map(self._prepare_shard, shards)
        else:
            results = [self._prepare_shard(shard) for shard in shards]
        self._write_configs(results)

    def _setup_tokenizer(self) -> None:
        c = self._config
        self._tokenizer = c.tokenizer.get_tokenizer()
        if c.add_bos and self._tokenizer.bod_id is None:
            raise ValueError("`add_bos` needs a tokenizer with a beginning-of-document token (or set tokenizer.bos_token)")
        if c.add_eos and self._tokenizer.eod_id is None:
            raise ValueError("`add_eos` needs a tokenizer with an end-of-document token")
        if isinstance(self._schema, ConversationSourceConfig):
            self._tokenizer.validate_chat_template()
        self._dtype = unsigned_dtype_for(self._tokenizer.vocab_size) if c.dataset.data_type is None else c.dataset.data_type.torch

    def _prepare_shard(self, args) -> tuple[str, dict]:
        index, shard = args
        file_name = f"shard_{self._config.distributed.rank}_{index}.fast_llm_dataset"
        reader_config = MemmapDataset.write_dataset(self._config.output_path / file_name, (self.prepare_document(row) for row in shard))
        return file_name, reader_config

    # ---- one document
    def prepare_document(self, row: dict) -> LanguageModelDocument:
        if self._tokenizer is None:
            self._setup_tokenizer()
        c, schema = self._config, self._schema
        if isinstance(schema, ConversationSourceConfig):
            tokens, spans = self._tokenizer.tokenize_chat(row[schema.messages], c.add_bos, c.add_eos, data_type=torch.int64)
            if not schema.train_on_eos and c.add_eos:
                spans = _merge_spans([*spans, (len(tokens) - 1, len(tokens))])
            return LanguageModelDocument(tokens=tokens.to(self._dtype), loss_masking_spans=spans)
        text = row[schema.text]
        # every boundary that must fall between two tokens: (character position, order, kind, payload)
        events = []
        if schema.has_loss_masking_spans:
            for begin, end in row[schema.loss_masking_spans] or ():
                events += [(int(begin), 1, "mask_begin", None), (int(end), 0, "mask_end", None)]
        if schema.has_preference_spans:
            for kind, column in (("chosen", schema.chosen_span), ("rejected", schema.rejected_span)):
                begin, end = row[column]
                events += [(int(begin), 1, f"{kind}_begin", None), (int(end), 0, f"{kind}_end", None)]
        if schema.has_images:
            for image, position in zip(row[schema.images] or (), row[schema.image_positions] or ()):
                events.append((int(position), 2, "image", image))
        events.sort(key=lambda e: (e[0], e[1]))
        pieces, total = [], 0
        marks: dict[str, list[int]] = {}
        patches, patch_positions, patch_coordinates = [], [], []
        cursor = 0

        def emit_text(upto: int, first: bool, last: bool):
            nonlocal cursor, total
            piece = self._tokenizer.tokenize(text[cursor:upto], c.add_bos and first, c.add_eos and last, data_type=torch.int64)
            pieces.append(piece)
            total += len(piece)
            cursor = upto

        first = True
        for position, _, kind, payload in events:
            Assert.in_range_incl(position, cursor, len(text))
            if position > cursor or first:
                emit_text(position, first, False)
                first = False
            if kind == "image":
                image_patches, coordinates, (rows, columns) = image_to_patches(payload, c.image_patches)
                image_tokens, patch_indices = image_token_layout(rows, columns, c.image_patches)
                patches.append(image_patches)
                patch_coordinates.append(coordinates)
                patch_positions.append(torch.tensor(patch_indices, dtype=torch.int64) + total)
                pieces.append(torch.tensor(image_tokens, dtype=torch.int64))
                total += len(image_tokens)
            else:
                marks.setdefault(kind, []).append(total)
        emit_text(len(text), first, True)
        tokens = torch.cat(pieces)
        if self._config.tokenizer.max_vocab_size is None and len(tokens) and int(tokens.max()) >= 2**16 and self._dtype == torch.uint16:
            raise ValueError("token id does not fit the chosen data type")
        document = LanguageModelDocument(tokens=tokens.to(self._dtype))
        if schema.has_loss_masking_spans:
            document.loss_masking_spans = [(b, e) for b, e in zip(marks.get("mask_begin", []), marks.get("mask_end", [])) if e > b]
        if schema.has_preference_spans:
            document.chosen_span = (marks["chosen_begin"][0], marks["chosen_end"][0])
            document.rejected_span = (marks["rejected_begin"][0], marks["rejected_end"][0])
        if schema.has_images:
            shape = (3, c.image_patches.height, c.image_patches.width)
            document.image_patches = torch.cat(patches) if patches else torch.zeros((0, *shape), dtype=torch.uint8)
            document.image_patch_positions = torch.cat(patch_positions) if patches else torch.zeros(0, dtype=torch.int64)
            document.image_patch_coordinates = torch.cat(patch_coordinates) if patches else torch.zeros((0, 2), dtype=torch.int64)
        if schema.has_grpo_data:
            document.advantages = torch.full((len(tokens),), float(row[schema.advantages]), dtype=torch.float32)
            if schema.old_log_probabilities is not None:
                old = torch.tensor(row[schema.old_log_probabilities], dtype=torch.float32)
                Assert.eq(len(old), len(tokens))
                document.old_log_probabilities = old
        return document

    # ---- dataset configs
    def _write_configs(self, results: list[tuple[str, dict]]) -> None:
        distributed = self._config.distributed
        if distributed.world_size > 1:
            gathered = [None] * distributed.world_size if distributed.rank == 0 else None
            torch.distributed.gather_object(results, gathered, dst=0)
            if distributed.rank == 0:
                results = [item for part in gathered for item in part]
        if distributed.rank == 0:
            results = [(name, config) for name, config in results if _metadata(config)["num_documents"] > 0]
            if self._config.splits:
                for split, (config, metadata) in split_and_blend(results, self._config.splits, self._config.output_path).items():
                    _save(self._config.output_path / f"fast_llm_config_{split}.yaml", config, metadata)
            else:
                _save(self._config.output_path / "fast_llm_config.yaml", *blend(results))
        if distributed.world_size > 1:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()


def _merge_spans(spans: list[tuple[int, int]]) -> list[tuple[int, int]]:
    out: list[tuple[int, int]] = []
    for begin, end in sorted(spans):
        if out and begin <= out[-1][1]:
            out[-1] = (out[-1][0], max(out[-1][1], end))
        else:
            out.append((begin, end))
    return out


def _metadata(reader_config: dict) -> dict:
    tokens = reader_config.get("tokens", reader_config)  # the language-model reader nests the token reader's counts
    return {"num_documents": int(tokens.get("num_documents", 0)), "num_tokens": int(tokens.get("num_tokens", 0))}


def _sum_metadata(items: list[dict]) -> dict:
    return {key: sum(item[key] for item in items) for key in ("num_documents", "num_tokens")}


def _save(path: pathlib.Path, config: dict, metadata: dict) -> None:
    logger.info(f"Saving dataset config to {path}")
    path.write_text(yaml.safe_dump({"config": config, "metadata": metadata}))


def blend(results: list[tuple[str, dict]]) -> tuple[dict, dict]:
    """One dataset, or a blend of the shards weighted by their token counts."""
    configs = [{"type": "memmap", "path": name} for name, _ in results]
    metadata = [_metadata(reader) for _, reader in results]
    if len(configs) == 1:
        return configs[0], metadata[0]
    return {"type": "blended", "datasets": configs, "weights": [m["num_tokens"] for m in metadata]}, _sum_metadata(metadata)


def split_and_blend(results: list[tuple[str, dict]], splits: dict[str, float], output_path: pathlib.Path) -> dict[str, tuple[dict, dict]]:
    """Cut the concatenation of all shards (measured in tokens) at the split fractions; a shard crossed by a boundary is
    divided at the document whose cumulative token count is nearest to it."""
    shares = np.array(list(splits.values()), dtype=np.float64)
    Assert.custom(lambda s: (s >= 0).all() and s.sum() > 0, shares)
    split_edges = np.concatenate([[0.0], np.cumsum(shares / shares.sum())])
    sizes = np.array([_metadata(reader)["num_tokens"] for _, reader in results], dtype=np.float64)
    shard_share = sizes / sizes.sum()
    shard_edges = np.concatenate([[0.0], np.cumsum(shard_share)])
    out = {}
    for s, name in enumerate(splits):
        parts, metadata = [], []
        for d, (file_name, reader) in enumerate(results):
            begin = max((split_edges[s] - shard_edges[d]) / shard_share[d], 0.0)
            end = min((split_edges[s + 1] - shard_edges[d]) / shard_share[d], 1.0)
            if begin <= 1e-12 and end >= 1 - 1e-12:
                parts.append({"type": "memmap", "path": file_name})
                metadata.append(_metadata(reader))
            elif end > begin:
                document_sizes = MemmapDataset(file_name, output_path / file_name).get_document_sizes()
                cumsum = np.concatenate([[0], np.cumsum(document_sizes)])
                first, last = _nearest(cumsum, begin * cumsum[-1]), _nearest(cumsum, end * cumsum[-1])
                if last > first:
                    count = len(document_sizes)
                    parts.append({"type": "slice", "dataset": {"type": "memmap", "path": file_name}, "begin": first / count, "end": last / count})
                    metadata.append({"num_documents": int(last - first), "num_tokens": int(cumsum[last] - cumsum[first])})
        if not parts:
            logger.error(f"Dataset split {name} is empty")
        elif len(parts) == 1:
            out[name] = (parts[0], metadata[0])
        else:
            out[name] = ({"type": "blended", "datasets": parts, "weights": [m["num_tokens"] for m in metadata]}, _sum_metadata(metadata))
    return out


def _nearest(cumsum: np.ndarray, value: float) -> int:
    right = int(np.searchsorted(cumsum, value, side="right"))
    left = max(right - 1, 0)
    right = min(right, len(cumsum) - 1)
    return left if value - cumsum[left] <= cumsum[right] - value else right
