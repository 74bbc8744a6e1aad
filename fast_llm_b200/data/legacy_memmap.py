"""Reader for the Megatron-LM style pair of files `<prefix>.bin` (all documents' tokens back to back) and `<prefix>.idx`
(sizes and byte offsets), in its three index versions: 1 plain, 2 with loss-masking spans, 3 with one chosen / rejected
preference span per document.  Older datasets are still in this format; new ones use the single-file format of
`fast_llm_b200.data.memmap`.  Both files are memory mapped, nothing is read until a document is asked for.
Parity: `fast_llm/data/dataset/gpt/legacy_memmap.py:26-230` (file format: the 9-byte magic `MMIDIDX\\0\\0`, a u64 version, flag
bytes, a dtype code, two u64 counts, then int32 sizes, int64 pointers and the span tables; spans are stored with inclusive ends).
"""

import pathlib
import struct

import numpy as np
import torch

from fast_llm_b200.data.document import LanguageModelDocument

INDEX_MAGIC = b"MMIDIDX\x00\x00"
DTYPE_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}


class LegacyMemmapDataset:
    def __init__(self, name: str, prefix: pathlib.Path | str):
        self._open(name, pathlib.Path(prefix))

    def _open(self, name: str, prefix: pathlib.Path) -> None:
        self._name, self._prefix = name, prefix
        index_path, data_path = prefix.with_suffix(".idx"), prefix.with_suffix(".bin")
        header = index_path.open("rb").read(64)
        if header[:9] != INDEX_MAGIC:
            raise ValueError(f"{index_path} is not a Megatron-style index file")
        (version,) = struct.unpack_from("<Q", header, 9)
        if version not in (1, 2, 3):
            raise ValueError(f"{index_path}: unsupported index version {version}")
        at = 17
        self._has_spans = bool(header[at]) if version >= 2 else False
        at += version >= 2
        self._has_preference = bool(header[at]) if version >= 3 else False
        at += version >= 3
        self._dtype = np.dtype(DTYPE_CODES[header[at]])
        documents, _ = struct.unpack_from("<QQ", header, at + 1)
        at += 17
        self._index = np.memmap(index_path, mode="r")
        if not 0 <= documents <= self._index.size:
            raise ValueError(f"{index_path}: implausible document count {documents} for a file of {self._index.size} bytes")
        self._sizes = np.frombuffer(self._index, dtype=np.int32, count=documents, offset=at)
        at += self._sizes.nbytes
        self._pointers = np.frombuffer(self._index, dtype=np.int64, count=documents, offset=at)
        at += self._pointers.nbytes
        self._span_counts = self._span_begin = self._spans = None
        if self._has_spans:
            self._span_counts = np.frombuffer(self._index, dtype=np.int32, count=documents, offset=at)
            if (self._span_counts < 0).any():
                raise ValueError(f"{index_path}: negative span count")
            at += self._span_counts.nbytes
            self._span_begin = np.concatenate([[0], np.cumsum(self._span_counts, dtype=np.int64)])
            total = int(self._span_begin[-1])
            if at + total * 8 > self._index.size:
                raise ValueError(f"{index_path}: span table runs past the end of the file")
            self._spans = np.frombuffer(self._index, dtype=np.int32, count=total * 2, offset=at).reshape(-1, 2)
            at += total * 8
        self._chosen = self._rejected = None
        if self._has_preference:
            if at + documents * 16 > self._index.size:
                raise ValueError(f"{index_path}: preference spans run past the end of the file")
            self._chosen = np.frombuffer(self._index, dtype=np.int32, count=documents * 2, offset=at).reshape(-1, 2)
            self._rejected = np.frombuffer(self._index, dtype=np.int32, count=documents * 2, offset=at + documents * 8).reshape(-1, 2)
        self._data = np.memmap(data_path, mode="r")
        self._num_tokens = self._data.size // self._dtype.itemsize

    def __getstate__(self):
        return self._name, self._prefix

    def __setstate__(self, state):
        self._open(*state)

    @property
    def name(self) -> str:
        return self._name

    def __len__(self) -> int:
        return len(self._sizes)

    @property
    def num_tokens(self) -> int:
        return self._num_tokens

    def get_document_sizes(self) -> np.ndarray:
        return np.asarray(self._sizes)

    def get_document_size(self, index: int) -> int:
        return int(self._sizes[index])

    def get_document(self, index: int, begin: int = 0, end: int | None = None) -> LanguageModelDocument:
        size = int(self._sizes[index])
        end = size if end is None else end
        assert 0 <= begin <= end <= size, (begin, end, size)
        tokens = np.frombuffer(self._data, dtype=self._dtype, count=end - begin, offset=int(self._pointers[index]) + begin * self._dtype.itemsize)
        document = LanguageModelDocument(tokens=torch.from_numpy(tokens.astype(np.int64)))
        if self._has_spans:
            lo, hi = int(self._span_begin[index]), int(self._span_begin[index + 1])
            document.loss_masking_spans = [(int(b), int(last) + 1) for b, last in self._spans[lo:hi]]  # stored with inclusive ends
        if self._has_preference:
            document.chosen_span = (int(self._chosen[index][0]), int(self._chosen[index][1]) + 1)
            document.rejected_span = (int(self._rejected[index][0]), int(self._rejected[index][1]) + 1)
        if begin or end != size:
            whole = document
            document = LanguageModelDocument(tokens=whole.tokens, loss_masking_spans=whole.loss_masking_spans, chosen_span=whole.chosen_span,
                                             rejected_span=whole.rejected_span)
            # spans are relative to the whole document: crop them with the token window (tokens are already cropped)
            cropped = LanguageModelDocument(tokens=torch.empty(size), loss_masking_spans=whole.loss_masking_spans, chosen_span=whole.chosen_span,
                                            rejected_span=whole.rejected_span).crop(begin, end)
            document = LanguageModelDocument(tokens=whole.tokens, loss_masking_spans=cropped.loss_masking_spans, chosen_span=cropped.chosen_span,
                                             rejected_span=cropped.rejected_span)
        return document

    @staticmethod
    def write_dataset(prefix: pathlib.Path | str, documents: list[LanguageModelDocument], dtype=np.uint16) -> None:
        """Write documents in this format (index version 1, 2 or 3 depending on what the documents carry); used to produce
        fixtures and to hand datasets to tools that still expect the pair of files."""
        prefix = pathlib.Path(prefix)
        has_spans = any(d.loss_masking_spans for d in documents)
        has_preference = any(d.chosen_span is not None for d in documents)
        version = 3 if has_preference else (2 if has_spans else 1)
        dtype = np.dtype(dtype)
        code = next(c for c, t in DTYPE_CODES.items() if np.dtype(t) == dtype)
        sizes = np.array([len(d) for d in documents], dtype=np.int32)
        pointers = np.concatenate([[0], np.cumsum(sizes[:-1].astype(np.int64) * dtype.itemsize)]).astype(np.int64) if len(documents) else np.zeros(0, np.int64)
        with prefix.with_suffix(".bin").open("wb") as f:
            for d in documents:
                f.write(d.tokens.numpy().astype(dtype).tobytes())
        with prefix.with_suffix(".idx").open("wb") as f:
            f.write(INDEX_MAGIC + struct.pack("<Q", version))
            if version >= 2:
                f.write(struct.pack("<B", int(has_spans)))
            if version >= 3:
                f.write(struct.pack("<B", int(has_preference)))
            f.write(struct.pack("<B", code) + struct.pack("<QQ", len(documents), len(documents) + 1))
            f.write(sizes.tobytes() + pointers.tobytes())
            if has_spans:
                counts = np.array([len(d.loss_masking_spans or []) for d in documents], dtype=np.int32)
                f.write(counts.tobytes())
                for d in documents:
                    for b, e in d.loss_masking_spans or []:
                        f.write(np.array([b, e - 1], dtype=np.int32).tobytes())
            if has_preference:
                for field in ("chosen_span", "rejected_span"):
                    for d in documents:
                        b, e = getattr(d, field) or (0, 1)
                        f.write(np.array([b, e - 1], dtype=np.int32).tobytes())
