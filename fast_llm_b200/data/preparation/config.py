"""`fast-llm prepare <kind> ...`: dataset preparation commands.

`gpt_memmap` tokenizes a Hugging Face dataset (plain text with optional loss-masking / preference spans, images and GRPO
fields, or chat conversations) into sharded memmap files plus ready-to-use dataset configs; `dataset_discovery` builds a
blended config for a directory tree of prepared files.
Parity: `fast_llm/data/preparation/config.py`, `fast_llm/data/preparation/gpt_memmap/config.py:19-344`,
`fast_llm/data/preparation/dataset_discovery/config.py`.
"""

import pathlib
import typing

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class
from fast_llm_b200.config.runnable import RunnableConfig
from fast_llm_b200.data.config import TokenizerConfig
from fast_llm_b200.utils import Assert
from fast_llm_b200.utils.data_type import DataType


@config_class(registry=True, dynamic_type={RunnableConfig: "prepare"})
class DatasetPreparatorConfig(RunnableConfig):
    _abstract: typing.ClassVar[bool] = True

    @classmethod
    def get_dataset_preparator_class(cls):
        raise NotImplementedError

    def _get_runnable(self):
        preparator = self.get_dataset_preparator_class()(self)
        return preparator.run


@config_class(registry=True)
class LanguageModelSourceConfig(Config):
    """Which columns of the source dataset hold what."""

    _abstract: typing.ClassVar[bool] = True

    @classmethod
    def _get_default_subclass(cls):
        return DocumentSourceConfig if cls is LanguageModelSourceConfig else cls

    @property
    def columns(self) -> list[str]:
        raise NotImplementedError

    has_loss_masking_spans = False
    has_preference_spans = False
    has_images = False
    has_grpo_data = False


@config_class(dynamic_type={LanguageModelSourceConfig: "document"})
class DocumentSourceConfig(LanguageModelSourceConfig):
    _abstract: typing.ClassVar[bool] = False
    text: str = Field(default="text", desc="Column holding the text.", hint=FieldHint.optional)
    loss_masking_spans: str | None = Field(default=None, desc="Column of character spans [(begin, end), ...] excluded from the loss.", hint=FieldHint.optional)
    chosen_span: str | None = Field(default=None, desc="Column of the chosen-completion character span (preference data).", hint=FieldHint.optional)
    rejected_span: str | None = Field(default=None, desc="Column of the rejected-completion character span.", hint=FieldHint.optional)
    images: str | None = Field(default=None, desc="Column of images (bytes, paths or arrays).", hint=FieldHint.optional)
    image_positions: str | None = Field(default=None, desc="Column of the character position of each image.", hint=FieldHint.optional)
    advantages: str | None = Field(default=None, desc="Column of the per-document advantage (GRPO).", hint=FieldHint.optional)
    old_log_probabilities: str | None = Field(default=None, desc="Column of per-token behaviour-policy log-probabilities (GRPO).", hint=FieldHint.optional)

    @property
    def columns(self) -> list[str]:
        names = [self.text, self.loss_masking_spans, self.chosen_span, self.rejected_span, self.images, self.image_positions,
                 self.advantages, self.old_log_probabilities]
        return [n for n in names if n is not None]

    @property
    def has_loss_masking_spans(self) -> bool:
        return self.loss_masking_spans is not None

    @property
    def has_preference_spans(self) -> bool:
        Assert.eq(self.chosen_span is None, self.rejected_span is None)
        return self.chosen_span is not None

    @property
    def has_images(self) -> bool:
        Assert.eq(self.images is None, self.image_positions is None)
        return self.images is not None

    @property
    def has_grpo_data(self) -> bool:
        return self.advantages is not None

    def _validate(self):
        super()._validate()
        if self.has_preference_spans and self.has_loss_masking_spans:
            raise ValueError("Preference spans and loss-masking spans cannot be combined")


@config_class(dynamic_type={LanguageModelSourceConfig: "conversation"})
class ConversationSourceConfig(LanguageModelSourceConfig):
    """Chat data: a column of `[{"role": ..., "content": ...}, ...]`; only assistant turns are trained on."""

    _abstract: typing.ClassVar[bool] = False
    messages: str = Field(default="messages", desc="Column holding the list of messages.", hint=FieldHint.optional)
    train_on_eos: bool = Field(default=True, desc="Keep the end-of-document token in the loss.", hint=FieldHint.feature)

    @property
    def columns(self) -> list[str]:
        return [self.messages]

    has_loss_masking_spans = True


@config_class()
class GPTHuggingfaceDatasetConfig(Config):
    path: str | pathlib.Path = Field(default=None, desc="Dataset name, directory or loading script.", hint=FieldHint.core)
    config_name: str | None = Field(default=None, desc="Dataset configuration name.", hint=FieldHint.optional)
    data_directory: str | None = Field(default=None, hint=FieldHint.optional)
    data_files: str | list[str] | None = Field(default=None, desc="Explicit data files (json, parquet, ...).", hint=FieldHint.optional)
    split: str = Field(default="train", hint=FieldHint.optional)
    source_schema: LanguageModelSourceConfig = Field(desc="Column mapping.", hint=FieldHint.optional)
    data_type: DataType | None = Field(default=None, desc="Token dtype (default: the smallest unsigned type holding the vocabulary).", hint=FieldHint.optional)
    trust_remote_code: bool = Field(default=False, hint=FieldHint.optional)
    disable_disk_space_check: bool = Field(default=False, hint=FieldHint.optional)
    load_from_disk: bool = Field(default=False, desc="The path was written by `datasets.save_to_disk`.", hint=FieldHint.feature)


@config_class()
class DatasetPreparatorDistributedConfig(Config):
    world_size: int = Field(default=None, desc="Processes sharing the work (default: WORLD_SIZE).", hint=FieldHint.expert)
    rank: int = Field(default=None, desc="Rank of this process (default: RANK).", hint=FieldHint.expert)
    backend: str = Field(default="gloo", hint=FieldHint.optional)
    timeout: int = Field(default=3600, desc="Process-group timeout in seconds.", hint=FieldHint.optional)

    def _validate(self):
        import os

        if self.world_size is None:
            self.world_size = int(os.environ.get("WORLD_SIZE", 1))
        if self.rank is None:
            self.rank = int(os.environ.get("RANK", 0))
        super()._validate()
        Assert.in_range(self.rank, 0, self.world_size)


@config_class()
class ImagePreparationConfig(Config):
    """How images become patches: resize so both sides are multiples of the patch size (bounded), cut row-major."""

    height: int = Field(default=16, desc="Patch height.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    width: int = Field(default=16, desc="Patch width.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    max_image_height: int = Field(default=1024, hint=FieldHint.optional, valid=check_field(Assert.gt, 0))
    max_image_width: int = Field(default=1024, hint=FieldHint.optional, valid=check_field(Assert.gt, 0))
    image_break_token: int | None = Field(default=None, desc="Token inserted after every row of patches.", hint=FieldHint.optional)
    image_end_token: int | None = Field(default=None, desc="Token inserted after the image.", hint=FieldHint.optional)
    placeholder_token: int = Field(default=-100, desc="Token occupying the position of each patch; negative ids embed to zero, so the patch embedding stands alone there, and are ignored as labels.", hint=FieldHint.optional)


@config_class(dynamic_type={RunnableConfig: "prepare_gpt_memmap", DatasetPreparatorConfig: "gpt_memmap"})
class GPTMemmapDatasetPreparatorConfig(DatasetPreparatorConfig):
    _abstract: typing.ClassVar[bool] = False
    output_path: pathlib.Path = Field(default=None, desc="Output directory.", hint=FieldHint.core)
    distributed: DatasetPreparatorDistributedConfig = Field(desc="Multi-process layout.", hint=FieldHint.feature)
    documents_per_shard: int = Field(default=1_000_000, desc="Documents per output file.", hint=FieldHint.optional, valid=check_field(Assert.gt, 0))
    num_workers: int = Field(default=1, desc="Worker processes tokenizing shards.", hint=FieldHint.optional, valid=check_field(Assert.geq, 1))
    dataset: GPTHuggingfaceDatasetConfig = Field(desc="Source dataset.", hint=FieldHint.feature)
    tokenizer: TokenizerConfig = Field(desc="Tokenizer.", hint=FieldHint.feature)
    add_bos: bool = Field(default=True, desc="Prepend the beginning-of-document token.", hint=FieldHint.feature)
    add_eos: bool = Field(default=True, desc="Append the end-of-document token.", hint=FieldHint.feature)
    image_patches: ImagePreparationConfig = Field(desc="Image patching.", hint=FieldHint.optional)
    splits: dict[str, float] | None = Field(default=None, desc="Name -> share of the tokens; writes one dataset config per split.", hint=FieldHint.optional)

    def _validate(self):
        Assert.not_none(self.output_path)
        super()._validate()

    @classmethod
    def get_dataset_preparator_class(cls):
        from fast_llm_b200.data.preparation.gpt_memmap import GPTMemmapDatasetPreparator

        return GPTMemmapDatasetPreparator


@config_class(dynamic_type={RunnableConfig: "prepare_dataset_discovery", DatasetPreparatorConfig: "dataset_discovery"})
class DatasetDiscoveryConfig(DatasetPreparatorConfig):
    """Scan a directory tree for prepared `.fast_llm_dataset` files and write one blended config weighted by tokens."""

    _abstract: typing.ClassVar[bool] = False
    directory: pathlib.Path = Field(default=None, desc="Root of the tree to scan.", hint=FieldHint.core)
    output: pathlib.Path = Field(default=None, desc="YAML file to write.", hint=FieldHint.core)
    ignore_paths: list[pathlib.Path] = Field(default_factory=list, desc="Sub-trees to skip.", hint=FieldHint.optional)

    def _validate(self):
        Assert.not_none(self.directory)
        Assert.not_none(self.output)
        super()._validate()

    @classmethod
    def get_dataset_preparator_class(cls):
        from fast_llm_b200.data.preparation.dataset_discovery import DatasetDiscoveryPreparator

        return DatasetDiscoveryPreparator
