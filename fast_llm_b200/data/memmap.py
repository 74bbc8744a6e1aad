"""The single-file memory-mapped dataset format (`fast_llm_prepared_dataset`) and its readers / writers.

File layout (byte compatible with `fast_llm/data/dataset/memmap/*.py`):

    b"fast_llm_prepared_dataset" | u64 BE offset of the config | sections ... | u32 BE config size | JSON reader config

Every section is `header bytes | payload | footer bytes`; the JSON config records `begin` / `end` of each section and
its shape.  Sections:
    token       tokens of all documents back to back (dtype from the config), then int64 cumulative sizes
    range       int32 (begin, end) pairs, then int32 cumulative counts per document  (loss-masking / preference spans)
    patch       image patches [n, *patch_shape], then per-patch int32 token positions, (row, col) coordinates and per-
                document cumulative counts
    token_data  per-token values (advantages, old log-probabilities): data then int64 cumulative sizes
    language_model   "lm begin" | token | range? | range? range? | patch? | token_data? token_data? | "lm end"
"""

import io
import json
import logging
import pathlib
import typing

import numpy as np
import torch

from fast_llm_b200.config import Config, Field, FieldHint, config_class
from fast_llm_b200.data.config import IndexedDatasetConfig, SampledDatasetConfig
from fast_llm_b200.data.document import LanguageModelDocument
from fast_llm_b200.utils import Assert
from fast_llm_b200.utils.data_type import DataType

FILE_HEADER = b"fast_llm_prepared_dataset"


logger = logging.getLogger(__name__)

@config_class(dynamic_type={SampledDatasetConfig: "memmap"})
class MemmapDatasetConfig(IndexedDatasetConfig):
    _abstract: typing.ClassVar[bool] = False
    path: pathlib.Path = Field(default=None, desc="Path of the dataset file (or the prefix of a Megatron-style `.bin` / `.idx` pair).", hint=FieldHint.core)

    def build(self):
        name = str(self.path).replace("/", "__")
        path = pathlib.Path(self.path)
        if path.is_file():
            return MemmapDataset(name, path)
        if path.with_suffix(".bin").is_file() and path.with_suffix(".idx").is_file():
            from fast_llm_b200.data.legacy_memmap import LegacyMemmapDataset

            logger.warning(f"{path}: Megatron-style pair of files; new datasets should use the single-file format")
            return LegacyMemmapDataset(name, path)
        raise FileNotFoundError(path)


# ---------------------------------------------------------------------------------------------------------------------
# Reader configs (what the JSON at the end of the file deserialises to)
# ---------------------------------------------------------------------------------------------------------------------
@config_class(registry=True)
class MemmapReaderBaseConfig(Config):
    _abstract = True

    @classmethod
    def _get_default_subclass(cls):
        return NullReaderConfig if cls is MemmapReaderBaseConfig else cls

    def get_reader(self, buffer: memoryview):
        raise NotImplementedError

    @property
    def expected_buffer_size(self) -> int:
        raise NotImplementedError


@config_class(dynamic_type={MemmapReaderBaseConfig: "none"})
class NullReaderConfig(MemmapReaderBaseConfig):
    _abstract = False

    def get_reader(self, buffer):
        return None

    @property
    def expected_buffer_size(self) -> int:
        return 0


@config_class(registry=True)
class MemmapReaderConfig(MemmapReaderBaseConfig):
    begin: int = Field(default=None, desc="Offset of the section's header in the file.")
    end: int = Field(default=None, desc="Offset just past the section's footer.")
    header: typing.ClassVar[bytes]
    footer: typing.ClassVar[bytes]

    def payload(self, buffer: memoryview) -> memoryview:
        b, e = self.begin + len(self.header), self.end - len(self.footer)
        Assert.eq(bytes(buffer[self.begin : b]), self.header)
        Assert.eq(bytes(buffer[e : self.end]), self.footer)
        return buffer[b:e]

    def _validate(self):
        super()._validate()
        Assert.eq(self.end - self.begin, self.expected_buffer_size)

    @property
    def expected_buffer_size(self) -> int:
        return self._payload_size + len(self.header) + len(self.footer)


@config_class(dynamic_type={MemmapReaderBaseConfig: "token"})
class TokenReaderConfig(MemmapReaderConfig):
    _abstract = False
    header: typing.ClassVar[bytes] = b"token begin"
    footer: typing.ClassVar[bytes] = b"token end"
    num_documents: int = Field(default=None)
    num_tokens: int = Field(default=None)
    data_type: DataType = Field(default=None)

    @property
    def _payload_size(self) -> int:
        return self.num_tokens * self.data_type.itemsize + (self.num_documents + 1) * 8

    def get_reader(self, buffer):
        return TokenReader(self, buffer)


@config_class(dynamic_type={MemmapReaderBaseConfig: "range"})
class RangeReaderConfig(MemmapReaderConfig):
    _abstract = False
    header: typing.ClassVar[bytes] = b"range begin"
    footer: typing.ClassVar[bytes] = b"range end"
    num_documents: int = Field(default=None)
    num_ranges: int = Field(default=None)

    @property
    def _payload_size(self) -> int:
        return self.num_ranges * 8 + (self.num_documents + 1) * 4

    def get_reader(self, buffer):
        return RangeReader(self, buffer)


@config_class(dynamic_type={MemmapReaderBaseConfig: "patch"})
class PatchReaderConfig(MemmapReaderConfig):
    _abstract = False
    header: typing.ClassVar[bytes] = b"patch begin"
    footer: typing.ClassVar[bytes] = b"patch end"
    num_documents: int = Field(default=None)
    num_patches: int = Field(default=None)
    num_patch_groups: int = Field(default=0)
    patch_shape: tuple[int, ...] = Field(default=(3, 16, 16))
    data_type: DataType = Field(default=DataType.uint8)

    @property
    def patch_size(self) -> int:
        return int(np.prod(self.patch_shape))

    @property
    def grid_dims(self) -> int:
        return len(self.patch_shape) - 1

    @property
    def _payload_size(self) -> int:
        return (self.num_patches * self.patch_size * self.data_type.itemsize + self.num_patches * 4 * (1 + self.grid_dims)
                + (self.num_documents + 1) * 4 + (self.num_patch_groups + self.num_documents + 1) * 4 * (self.num_patch_groups > 0))

    def get_reader(self, buffer):
        return PatchReader(self, buffer)


@config_class(dynamic_type={MemmapReaderBaseConfig: "token_data"})
class TokenDataReaderConfig(MemmapReaderConfig):
    _abstract = False
    header: typing.ClassVar[bytes] = b"token data begin"
    footer: typing.ClassVar[bytes] = b"token data end"
    num_documents: int = Field(default=None)
    num_tokens: int = Field(default=None)
    shape: tuple[int, ...] = Field(default=())
    data_type: DataType = Field(default=DataType.float32)

    @property
    def _payload_size(self) -> int:
        return self.num_tokens * int(np.prod(self.shape or (1,))) * self.data_type.itemsize + (self.num_documents + 1) * 8

    def get_reader(self, buffer):
        return TokenDataReader(self, buffer)


@config_class(dynamic_type={MemmapReaderBaseConfig: "language_model"})
class LanguageModelReaderConfig(MemmapReaderConfig):
    _abstract = False
    header: typing.ClassVar[bytes] = b"lm begin"
    footer: typing.ClassVar[bytes] = b"lm end"
    tokens: TokenReaderConfig = Field(desc="Token section.")
    loss_masking_spans: MemmapReaderBaseConfig = Field(desc="Spans excluded from the loss.")
    chosen_spans: MemmapReaderBaseConfig = Field(desc="Preferred completions (preference data).")
    rejected_spans: MemmapReaderBaseConfig = Field(desc="Rejected completions (preference data).")
    image_patches: MemmapReaderBaseConfig = Field(desc="Image patches.")
    advantages: MemmapReaderBaseConfig = Field(desc="Per-token advantages (policy-gradient data).")
    old_log_probabilities: MemmapReaderBaseConfig = Field(desc="Per-token log-probabilities of the sampling policy.")

    @property
    def _parts(self):
        return (self.tokens, self.loss_masking_spans, self.chosen_spans, self.rejected_spans, self.image_patches,
                self.advantages, self.old_log_probabilities)

    @property
    def _payload_size(self) -> int:
        return sum(p.expected_buffer_size for p in self._parts)

    @property
    def num_documents(self) -> int:
        return self.tokens.num_documents

    @property
    def num_tokens(self) -> int:
        return self.tokens.num_tokens

    def get_reader(self, buffer):
        return LanguageModelReader(self, buffer)


MemmapIndexDatasetReaderConfig = MemmapReaderBaseConfig


# ---------------------------------------------------------------------------------------------------------------------
# Readers
# ---------------------------------------------------------------------------------------------------------------------
class TokenReader:
    def __init__(self, config: TokenReaderConfig, buffer: memoryview):
        self._config = config
        payload = config.payload(buffer)
        nbytes = config.num_tokens * config.data_type.itemsize
        self._tokens = np.frombuffer(payload, dtype=config.data_type.numpy, count=config.num_tokens)
        self._cumsum = np.frombuffer(payload, dtype=np.int64, count=config.num_documents + 1, offset=nbytes)

    def get(self, index: int, begin: int, end: int) -> torch.Tensor:
        base = int(self._cumsum[index])
        return torch.from_numpy(self._tokens[base + begin : base + end].astype(np.int64))

    @property
    def sizes(self) -> np.ndarray:
        return np.diff(self._cumsum)

    def size(self, index: int) -> int:
        return int(self._cumsum[index + 1] - self._cumsum[index])


class RangeReader:
    def __init__(self, config: RangeReaderConfig, buffer: memoryview):
        payload = config.payload(buffer)
        self._ranges = np.frombuffer(payload, dtype=np.int32, count=config.num_ranges * 2).reshape(-1, 2)
        self._cumsum = np.frombuffer(payload, dtype=np.int32, count=config.num_documents + 1, offset=config.num_ranges * 8)

    def get(self, index: int, begin: int, end: int) -> list[tuple[int, int]]:
        out = []
        for b, e in self._ranges[self._cumsum[index] : self._cumsum[index + 1]].tolist():
            b, e = max(b - begin, 0), min(e - begin, end - begin)
            if e > b:
                out.append((b, e))
        return out


class TokenDataReader:
    def __init__(self, config: TokenDataReaderConfig, buffer: memoryview):
        payload = config.payload(buffer)
        per = int(np.prod(config.shape or (1,)))
        count = config.num_tokens * per
        self._data = np.frombuffer(payload, dtype=config.data_type.numpy, count=count).reshape(config.num_tokens, *config.shape)
        self._cumsum = np.frombuffer(payload, dtype=np.int64, count=config.num_documents + 1, offset=count * config.data_type.itemsize)

    def get(self, index: int, begin: int, end: int) -> torch.Tensor:
        base = int(self._cumsum[index])
        return torch.from_numpy(np.array(self._data[base + begin : base + end]))


class PatchReader:
    def __init__(self, config: PatchReaderConfig, buffer: memoryview):
        self._config = config
        payload = config.payload(buffer)
        n, psize, item = config.num_patches, config.patch_size, config.data_type.itemsize
        off = 0
        self._patches = np.frombuffer(payload, dtype=config.data_type.numpy, count=n * psize, offset=off).reshape(n, *config.patch_shape)
        off += n * psize * item
        self._positions = np.frombuffer(payload, dtype=np.int32, count=n, offset=off)
        off += n * 4
        self._coordinates = np.frombuffer(payload, dtype=np.int32, count=n * config.grid_dims, offset=off).reshape(n, config.grid_dims)
        off += n * 4 * config.grid_dims
        self._cumsum = np.frombuffer(payload, dtype=np.int32, count=config.num_documents + 1, offset=off)

    def get(self, index: int, begin: int, end: int):
        lo, hi = int(self._cumsum[index]), int(self._cumsum[index + 1])
        pos = self._positions[lo:hi]
        keep = (pos >= begin) & (pos < end)
        return (torch.from_numpy(np.array(self._patches[lo:hi][keep])), torch.from_numpy(pos[keep] - begin),
                torch.from_numpy(np.array(self._coordinates[lo:hi][keep])))


class LanguageModelReader:
    def __init__(self, config: LanguageModelReaderConfig, buffer: memoryview):
        self._config = config
        config.payload(buffer)  # checks header and footer
        self._tokens = config.tokens.get_reader(buffer)
        self._loss_masking = config.loss_masking_spans.get_reader(buffer)
        self._chosen = config.chosen_spans.get_reader(buffer)
        self._rejected = config.rejected_spans.get_reader(buffer)
        self._patches = config.image_patches.get_reader(buffer)
        self._advantages = config.advantages.get_reader(buffer)
        self._old_log_probs = config.old_log_probabilities.get_reader(buffer)

    def __len__(self) -> int:
        return self._config.num_documents

    @property
    def num_tokens(self) -> int:
        return self._config.num_tokens

    def get_document_sizes(self) -> np.ndarray:
        return self._tokens.sizes

    def get_document_size(self, index: int) -> int:
        return self._tokens.size(index)

    def get_document(self, index: int, begin: int, end: int) -> LanguageModelDocument:
        doc = LanguageModelDocument(tokens=self._tokens.get(index, begin, end))
        if self._loss_masking is not None:
            doc.loss_masking_spans = self._loss_masking.get(index, begin, end)
        if self._chosen is not None:
            spans = self._chosen.get(index, begin, end)
            doc.chosen_span = spans[0] if spans else None
            spans = self._rejected.get(index, begin, end)
            doc.rejected_span = spans[0] if spans else None
        if self._patches is not None:
            doc.image_patches, doc.image_patch_positions, doc.image_patch_coordinates = self._patches.get(index, begin, end)
        if self._advantages is not None:
            doc.advantages = self._advantages.get(index, begin, end).float()
            doc.old_log_probabilities = self._old_log_probs.get(index, begin, end).float()
        return doc


# ---------------------------------------------------------------------------------------------------------------------
# Dataset and writer
# ---------------------------------------------------------------------------------------------------------------------
class MemmapDataset:
    """Lazily memory-mapped indexed dataset of documents."""

    def __init__(self, name: str, path: pathlib.Path | str):
        self._name = name
        self._path = pathlib.Path(path)
        self._open()

    def _open(self) -> None:
        size = self._path.stat().st_size
        with self._path.open("rb") as stream:
            assert stream.read(len(FILE_HEADER)) == FILE_HEADER, f"Invalid file header in {self._path}"
            config_offset = int.from_bytes(stream.read(8), "big", signed=False)
            assert config_offset + 4 <= size, f"Config offset out of range in {self._path}"
            stream.seek(config_offset)
            config_size = int.from_bytes(stream.read(4), "big", signed=False)
            assert config_offset + 4 + config_size <= size
            config = json.loads(stream.read(config_size).decode("utf-8"))
        self._reader_config = MemmapReaderBaseConfig.from_dict(config).validate()
        self._memmap = np.memmap(self._path, mode="r")
        self._reader = self._reader_config.get_reader(memoryview(self._memmap))

    def __getstate__(self):
        return self._name, self._path

    def __setstate__(self, state):
        self._name, self._path = state
        self._open()

    @property
    def name(self) -> str:
        return self._name

    @property
    def reader_config(self):
        return self._reader_config

    def __len__(self) -> int:
        return len(self._reader)

    @property
    def num_tokens(self) -> int:
        return self._reader.num_tokens

    def get_document_sizes(self) -> np.ndarray:
        return self._reader.get_document_sizes()

    def get_document_size(self, index: int) -> int:
        return self._reader.get_document_size(index)

    def get_document(self, index: int, begin: int = 0, end: int | None = None) -> LanguageModelDocument:
        end = self._reader.get_document_size(index) if end is None else end
        return self._reader.get_document(index, begin, end)

    @classmethod
    def write_dataset(cls, path: pathlib.Path | str, documents: typing.Iterable[LanguageModelDocument]) -> dict:
        """Write documents into one file; returns the reader config (as a dict) stored at its end."""
        path = pathlib.Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        with path.open("wb") as stream:
            stream.write(FILE_HEADER)
            start = stream.tell()
            stream.write(b"\0" * 8)
            config = _write_language_model(stream, documents)
            config_offset = stream.tell()
            payload = json.dumps(config).encode("utf-8")
            stream.write(len(payload).to_bytes(4, "big", signed=False))
            stream.write(payload)
            stream.seek(start)
            stream.write(config_offset.to_bytes(8, "big", signed=False))
        return config


def _write_language_model(stream: io.BufferedWriter, documents: typing.Iterable[LanguageModelDocument]) -> dict:
    """Streams tokens straight to the file and buffers the (much smaller) side data in memory."""
    begin = stream.tell()
    stream.write(LanguageModelReaderConfig.header)
    token_begin = stream.tell()
    stream.write(TokenReaderConfig.header)
    sizes, dtype = [0], None
    spans, span_counts = [], [0]
    chosen, chosen_counts, rejected, rejected_counts = [], [0], [], [0]
    patches, patch_pos, patch_coord, patch_counts, patch_shape = [], [], [], [0], None
    advantages, old_log_probs = [], []
    flags = None
    for doc in documents:
        tokens = doc.tokens.numpy() if torch.is_tensor(doc.tokens) else np.asarray(doc.tokens)
        if dtype is None:
            dtype = tokens.dtype
            flags = (doc.loss_masking_spans is not None, doc.chosen_span is not None, doc.image_patches is not None, doc.advantages is not None)
        Assert.eq(tokens.dtype, dtype)
        Assert.eq(flags, (doc.loss_masking_spans is not None, doc.chosen_span is not None, doc.image_patches is not None, doc.advantages is not None),
                  msg="all documents of a dataset must carry the same optional fields")
        stream.write(tokens.tobytes())
        sizes.append(sizes[-1] + len(tokens))
        if flags[0]:
            spans += [list(s) for s in doc.loss_masking_spans]
            span_counts.append(len(spans))
        if flags[1]:
            chosen.append(list(doc.chosen_span))
            chosen_counts.append(len(chosen))
            rejected.append(list(doc.rejected_span))
            rejected_counts.append(len(rejected))
        if flags[2]:
            p = doc.image_patches.numpy() if torch.is_tensor(doc.image_patches) else np.asarray(doc.image_patches)
            patch_shape = tuple(p.shape[1:]) if patch_shape is None else patch_shape
            patches.append(p)
            patch_pos.append(np.asarray(doc.image_patch_positions, dtype=np.int32))
            coords = doc.image_patch_coordinates if doc.image_patch_coordinates is not None else np.zeros((len(p), len(patch_shape) - 1))
            patch_coord.append(np.asarray(coords, dtype=np.int32).reshape(len(p), 2))  # (row, column); a document may have no image
            patch_counts.append(patch_counts[-1] + len(p))
        if flags[3]:
            advantages.append(np.asarray(doc.advantages, dtype=np.float32))
            old_log_probs.append(np.asarray(doc.old_log_probabilities, dtype=np.float32))
    assert dtype is not None, "cannot write an empty dataset"
    num_documents = len(sizes) - 1
    stream.write(np.array(sizes, dtype=np.int64).tobytes())
    stream.write(TokenReaderConfig.footer)
    config = {"type": "language_model", "begin": begin,
              "tokens": {"type": "token", "begin": token_begin, "end": stream.tell(), "num_documents": num_documents,
                         "num_tokens": sizes[-1], "data_type": DataType.from_numpy(dtype).value}}

    def write_ranges(name, ranges, counts):
        b = stream.tell()
        stream.write(RangeReaderConfig.header)
        stream.write(np.array(ranges, dtype=np.int32).reshape(-1, 2).tobytes())
        stream.write(np.array(counts, dtype=np.int32).tobytes())
        stream.write(RangeReaderConfig.footer)
        config[name] = {"type": "range", "begin": b, "end": stream.tell(), "num_documents": num_documents, "num_ranges": len(ranges)}

    def write_token_data(name, chunks):
        b = stream.tell()
        stream.write(TokenDataReaderConfig.header)
        for c in chunks:
            stream.write(c.tobytes())
        stream.write(np.array(sizes, dtype=np.int64).tobytes())
        stream.write(TokenDataReaderConfig.footer)
        config[name] = {"type": "token_data", "begin": b, "end": stream.tell(), "num_documents": num_documents,
                        "num_tokens": sizes[-1], "shape": [], "data_type": "float32"}

    if flags[0]:
        write_ranges("loss_masking_spans", spans, span_counts)
    if flags[1]:
        write_ranges("chosen_spans", chosen, chosen_counts)
        write_ranges("rejected_spans", rejected, rejected_counts)
    if flags[2]:
        b = stream.tell()
        stream.write(PatchReaderConfig.header)
        all_patches = np.concatenate(patches) if patches else np.zeros((0, *patch_shape), dtype=np.uint8)
        stream.write(all_patches.tobytes())
        stream.write(np.concatenate(patch_pos).astype(np.int32).tobytes())
        stream.write(np.concatenate(patch_coord).astype(np.int32).tobytes())
        stream.write(np.array(patch_counts, dtype=np.int32).tobytes())
        stream.write(PatchReaderConfig.footer)
        config["image_patches"] = {"type": "patch", "begin": b, "end": stream.tell(), "num_documents": num_documents,
                                   "num_patches": patch_counts[-1], "num_patch_groups": 0, "patch_shape": list(patch_shape),
                                   "data_type": DataType.from_numpy(all_patches.dtype).value}
    if flags[3]:
        write_token_data("advantages", advantages)
        write_token_data("old_log_probabilities", old_log_probs)
    stream.write(LanguageModelReaderConfig.footer)
    config["end"] = stream.tell()
    return config
