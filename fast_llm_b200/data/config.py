"""Dataset and sampling configuration: the `data:` section of a training config.

`datasets:` maps a phase / evaluator name to a dataset config chosen by `type:` (memmap, concatenated, slice, blended,
random, file, fim, streaming, test_slow).  Sampling works in *tokens*: every sample is a packed stream of
`micro_batch_size` tokens.  Parity: `fast_llm/data/dataset/config.py:21-320`, `fast_llm/data/dataset/gpt/config.py:21-209`,
`fast_llm/data/data/gpt/config.py:16-43`.
"""

import enum
import pathlib
import typing

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class, skip_valid_if_none
from fast_llm_b200.utils import Assert


class ShufflingType(str, enum.Enum):
    full = "full"  # shuffle all epochs together
    epoch = "epoch"  # shuffle each epoch separately
    skip_first_epoch = "skip_first_epoch"
    disabled = "disabled"


class MultiprocessingContext(str, enum.Enum):
    fork = "fork"
    forkserver = "forkserver"
    spawn = "spawn"


@config_class()
class SamplingConfigBase(Config):
    gpu: bool = Field(default=True, desc="Build shuffling indices on the GPU when one is available.", hint=FieldHint.feature)
    shuffle: ShufflingType = Field(default=ShufflingType.epoch, desc="Shuffling strategy.", hint=FieldHint.feature)
    micro_batch_size: int = Field(default=2048, desc="Tokens per micro-batch.", hint=FieldHint.core, valid=check_field(Assert.gt, 0))
    maximum_document_length: int | None = Field(default=None, desc="Longer documents are split (truncate_documents) or dropped.", hint=FieldHint.core)
    truncate_documents: bool | None = Field(default=True, desc="Cut documents at sample boundaries (True) or pad samples so documents stay whole.", hint=FieldHint.feature)


@config_class()
class SamplingConfig(SamplingConfigBase):
    """Everything a dataset needs to produce samples for one (dataset name, phase)."""

    predicted_tokens: int = Field(default=1, desc="Extra tokens per sample used as labels.")
    token_cumsum_rate: int = Field(default=10, desc="Keep one token-count checkpoint every this many documents.", hint=FieldHint.performance, valid=check_field(Assert.gt, 0))
    cache_directory: pathlib.Path | None = Field(default=None, desc="Where sampling indices are cached.")
    dataset_name: str = Field(default="dataset")
    world_size: int = Field(default=1)
    rank: int = Field(default=0)
    seed: int = Field(default=784569)
    num_samples: int = Field(default=0, desc="Samples needed from the dataset.")
    vocab_size: int | None = Field(default=None, desc="Vocabulary size (random data, token range checks).")
    use_loss_masking_spans: bool = Field(default=True)
    use_preference_spans: bool = Field(default=False)
    use_grpo_data: bool = Field(default=False)
    use_images: bool = Field(default=False)

    @property
    def sample_size(self) -> int:
        return self.micro_batch_size + self.predicted_tokens

    @property
    def sampling_maximum_document_length(self) -> int:
        if self.maximum_document_length is None:
            return self.sample_size
        return min(self.maximum_document_length, self.sample_size)


@config_class()
class DatasetConfig(Config):
    _abstract: typing.ClassVar[bool] = True


@config_class(registry=True)
class SampledDatasetConfig(DatasetConfig):
    """A dataset that can be turned into an indexable sequence of fixed-size samples."""

    @classmethod
    def _get_default_subclass(cls):
        if cls is SampledDatasetConfig:
            from fast_llm_b200.data.memmap import MemmapDatasetConfig

            return MemmapDatasetConfig
        return cls

    def build_and_sample(self, sampling: SamplingConfig, num_samples: int, seed: int):
        raise NotImplementedError


@config_class()
class SamplableDatasetConfig(SampledDatasetConfig):
    def build(self):
        raise NotImplementedError

    def build_and_sample(self, sampling: SamplingConfig, num_samples: int, seed: int):
        from fast_llm_b200.data.sampled import SampledIndexedDataset

        return SampledIndexedDataset(self.build(), sampling, num_samples, seed)


@config_class()
class IndexedDatasetConfig(SamplableDatasetConfig):
    pass


@config_class(dynamic_type={SampledDatasetConfig: "concatenated"})
class ConcatenatedDatasetConfig(SamplableDatasetConfig):
    _abstract = False
    name: str = Field(default="concatenated", hint=FieldHint.core)
    datasets: list[IndexedDatasetConfig] = Field(default_factory=list, desc="Datasets to concatenate.", hint=FieldHint.core)

    def build(self):
        from fast_llm_b200.data.indexed import ConcatenatedDataset

        Assert.gt(len(self.datasets), 0)
        return ConcatenatedDataset(self.name, [d.build() for d in self.datasets])


@config_class(dynamic_type={SampledDatasetConfig: "slice"})
class DatasetSliceConfig(SamplableDatasetConfig):
    _abstract = False
    dataset: IndexedDatasetConfig = Field(default=None, desc="Dataset to slice.", hint=FieldHint.core)
    begin: float = Field(default=0, desc="Start, as a fraction of the documents.", hint=FieldHint.core)
    end: float = Field(default=1, desc="End, as a fraction of the documents.", hint=FieldHint.core)

    def build(self):
        from fast_llm_b200.data.indexed import DatasetSlice

        dataset = self.dataset.build()
        n = len(dataset)
        return DatasetSlice(f"{dataset.name}_{self.begin}_{self.end}", dataset, round(self.begin * n), round(self.end * n))


@config_class(dynamic_type={SampledDatasetConfig: "blended"})
class BlendedDatasetConfig(SampledDatasetConfig):
    _abstract = False
    name: str = Field(default="blended", hint=FieldHint.core)
    datasets: list[SampledDatasetConfig] = Field(default_factory=list, hint=FieldHint.core)
    weights: list[float] = Field(default_factory=list, desc="Sampling probability of each dataset.", hint=FieldHint.core)

    def _validate(self):
        super()._validate()
        Assert.geq(len(self.datasets), 1)
        Assert.eq(len(self.datasets), len(self.weights))

    def build_and_sample(self, sampling: SamplingConfig, num_samples: int, seed: int):
        from fast_llm_b200.data.blended import BlendedDataset

        total = sum(self.weights)
        sampled = []
        for i, (dataset, weight) in enumerate(zip(self.datasets, self.weights)):
            # a 5% + 1 margin covers the rounding of the deterministic blending sequence
            n = int(num_samples * weight / total * 1.05) + 1
            sampled.append(dataset.build_and_sample(sampling.to_copy({"dataset_name": f"{sampling.dataset_name}_{i}"}), n, seed + i * 7919))
        return BlendedDataset(self.name, sampled, self.weights, num_samples)


@config_class(dynamic_type={SampledDatasetConfig: "random"})
class GPTRandomDatasetConfig(SampledDatasetConfig):
    _abstract: typing.ClassVar[bool] = False
    name: str = Field(default="dummy", hint=FieldHint.core)
    images_per_sample: int = Field(default=0, desc="Synthetic images placed in every sample (multimodal models).", hint=FieldHint.testing)
    image_patch_grid: tuple[int, int] = Field(default=(2, 2), desc="Patches per synthetic image (rows, columns).", hint=FieldHint.testing)
    image_patch_shape: tuple[int, int, int] = Field(default=(3, 16, 16), desc="Shape of one patch (channels, height, width).", hint=FieldHint.testing)

    def build_and_sample(self, sampling: SamplingConfig, num_samples: int, seed: int):
        from fast_llm_b200.data.random import GPTRandomSampledDataset

        return GPTRandomSampledDataset(sampling, self.name, num_samples, seed, images_per_sample=self.images_per_sample,
                                       image_patch_grid=tuple(self.image_patch_grid), image_patch_shape=tuple(self.image_patch_shape))


@config_class(dynamic_type={SampledDatasetConfig: "file"})
class GPTDatasetFromFileConfig(SamplableDatasetConfig):
    """Reads another dataset config from a YAML file (relative paths resolve against that file)."""

    _abstract: typing.ClassVar[bool] = False
    path: pathlib.Path = Field(default=None, desc="YAML file holding a dataset config.", hint=FieldHint.core)

    def _load(self) -> SampledDatasetConfig:
        import yaml

        Assert.custom(lambda p: p is not None and pathlib.Path(p).is_file(), self.path)
        data = yaml.safe_load(self.path.read_text())
        if isinstance(data, dict) and set(data) == {"config", "metadata"}:
            data = data["config"]  # what `prepare` writes: the dataset config next to token / document counts
        data = _resolve_paths(data, self.path.parent)
        return SampledDatasetConfig.from_dict(data).validate()

    def build(self):
        return self._load().build()

    def build_and_sample(self, sampling: SamplingConfig, num_samples: int, seed: int):
        return self._load().build_and_sample(sampling, num_samples, seed)


def _resolve_paths(data, base: pathlib.Path):
    if isinstance(data, dict):
        return {k: (str(base / v) if k == "path" and isinstance(v, str) and not pathlib.Path(v).is_absolute() else _resolve_paths(v, base))
                for k, v in data.items()}
    if isinstance(data, list):
        return [_resolve_paths(v, base) for v in data]
    return data


@config_class()
class TokenizerConfig(Config):
    _abstract = False
    path: pathlib.Path = Field(default=None, desc="Hugging Face tokenizer directory or file.", hint=FieldHint.core)
    bos_token: str | None = Field(default=None, desc="Override the beginning-of-sequence token.", hint=FieldHint.core)
    max_vocab_size: int | None = Field(default=None, desc="Map token ids above this to the range (testing).", hint=FieldHint.testing)
    trust_remote_code: bool = Field(default=False, hint=FieldHint.feature)

    def get_tokenizer(self):
        from fast_llm_b200.data.tokenizer import Tokenizer

        return Tokenizer(self)


@config_class()
class FimConfig(Config):
    tokenizer: TokenizerConfig = Field(desc="Tokenizer providing the FIM sentinel tokens.", hint=FieldHint.feature)
    rate: float = Field(default=0.0, desc="Probability of applying FIM to a document.", hint=FieldHint.core, valid=check_field(Assert.in_range_incl, 0, 1))
    max_middle_len: int | None = Field(default=None, hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.gt, 0)))
    split_sample: str | None = Field(default=None, desc="Apply FIM separately to the pieces between this token.", hint=FieldHint.feature)
    fragment_rate: float = Field(default=0.0, hint=FieldHint.feature, valid=check_field(Assert.in_range_incl, 0, 1))
    ignore_prefix: str | None = Field(default=None, hint=FieldHint.feature)
    spm_rate: float = Field(default=0.5, desc="Probability of suffix-prefix-middle order (else prefix-suffix-middle).", hint=FieldHint.feature, valid=check_field(Assert.in_range_incl, 0, 1))
    truncate_or_pad: bool = Field(default=False, hint=FieldHint.feature)
    prefix_token: str = Field(default="<fim_prefix>", hint=FieldHint.feature)
    middle_token: str = Field(default="<fim_middle>", hint=FieldHint.feature)
    pad_token: str = Field(default="<fim_pad>", hint=FieldHint.feature)
    suffix_token: str = Field(default="<fim_suffix>", hint=FieldHint.feature)


@config_class(dynamic_type={SampledDatasetConfig: "fim"})
class GPTFimSampledDatasetConfig(SampledDatasetConfig, FimConfig):
    _abstract: typing.ClassVar[bool] = False
    dataset: SampledDatasetConfig = Field(default=None, desc="Dataset to wrap.", hint=FieldHint.core)

    def build_and_sample(self, sampling: SamplingConfig, num_samples: int, seed: int):
        from fast_llm_b200.data.fim import GPTFimDataset

        return GPTFimDataset(self, self.dataset.build_and_sample(sampling, num_samples, seed), sampling, seed)


@config_class(dynamic_type={SampledDatasetConfig: "test_slow"})
class GPTTestSlowDatasetConfig(SampledDatasetConfig):
    _abstract: typing.ClassVar[bool] = False
    sleep: float = Field(default=1, desc="Seconds to sleep per sample.", hint=FieldHint.core)

    def build_and_sample(self, sampling: SamplingConfig, num_samples: int, seed: int):
        from fast_llm_b200.data.random import GPTRandomSampledDataset, SlowDataset

        return SlowDataset(GPTRandomSampledDataset(sampling, "slow", num_samples, seed), self.sleep)


@config_class()
class RedisConfig(Config):
    REDIS_FIELD: typing.ClassVar[str] = "data"
    REDIS_GROUP_NAME: typing.ClassVar[str] = "fast_llm_group"
    host: str = Field(default="localhost", hint=FieldHint.core)
    port: int = Field(default=6379, hint=FieldHint.core)
    timeout: float = Field(default=600.0)

    def get_client(self):
        import redis

        return redis.Redis(host=self.host, port=self.port)


@config_class(dynamic_type={SampledDatasetConfig: "streaming"})
class StreamingDatasetConfig(RedisConfig, SamplableDatasetConfig):
    _abstract = False

    def build_and_sample(self, sampling: SamplingConfig, num_samples: int, seed: int):
        from fast_llm_b200.data.streaming import RedisStreamingDataset

        return RedisStreamingDataset(self, sampling)


@config_class()
class DataConfig(Config):
    _abstract = True


@config_class()
class GPTDataConfig(DataConfig, SamplingConfigBase):
    _abstract = False
    datasets: dict[str, SampledDatasetConfig] = Field(default_factory=dict, desc="Dataset of each phase / evaluator.", hint=FieldHint.core)
    data_sample_warn_time_ms: float = Field(default=1000, desc="Warn when loading one sample takes longer.", hint=FieldHint.feature, valid=check_field(Assert.gt, 0))
    multiprocessing_context: MultiprocessingContext = Field(default=MultiprocessingContext.spawn, hint=FieldHint.expert)
    seed: int = Field(default=784569, desc="Sampling seed.", hint=FieldHint.feature)
