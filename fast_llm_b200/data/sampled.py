"""Deterministic, resumable sampling of fixed-length token samples from an indexed dataset.

Documents are visited epoch after epoch in a seeded shuffled order and laid end to end into one token stream; sample
`i` covers tokens `[i * micro_batch_size, (i + 1) * micro_batch_size + predicted_tokens)` of that stream, so consecutive
samples overlap by the label token(s).  With `truncate_documents` documents are cut at sample boundaries (and the part of a
document inside a sample is split into pieces of at most `maximum_document_length`); without it documents stay whole: one that does not fit the rest of a
sample starts the next one and the gap is padding (native helper `flb_build_padded_token_cumsum`), over-long documents
are dropped.  Only a sub-sampled token cumsum is stored (every `token_cumsum_rate` documents), so the index stays small
for billions of documents; the index is cached as `.npy` next to a `.yaml` description of what produced it.
Parity: `fast_llm/data/dataset/sampled.py:66-433`.
"""

import ctypes
import logging
import math
import pathlib

import numpy as np
import yaml

from fast_llm_b200.data.config import SamplingConfig, ShufflingType
from fast_llm_b200.data.document import LanguageModelDocument
from fast_llm_b200.ops import _lib

logger = logging.getLogger(__name__)


def _host_lib():
    if not _lib.HOST_LIB_PATH.exists():
        return None
    lib = ctypes.CDLL(str(_lib.HOST_LIB_PATH))
    lib.flb_build_padded_token_cumsum.restype = ctypes.c_int64
    lib.flb_build_padded_token_cumsum.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64,
                                                  ctypes.c_void_p, ctypes.c_void_p]
    lib.flb_build_sample_idx.restype = ctypes.c_int32
    lib.flb_build_sample_idx.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p]
    return lib


def build_padded_token_cumsum_python(sizes: np.ndarray, sample_size: int, rate: int, offset: int = 0) -> tuple[np.ndarray, int]:
    """Plain restatement of the native helper (test oracle and fallback)."""
    cumsum, out = offset, []
    for i, size in enumerate(sizes.tolist()):
        if i % rate == 0:
            out.append(cumsum)
        if size > sample_size:
            continue
        used = cumsum % sample_size
        if used + size > sample_size:
            cumsum += sample_size - used
        cumsum += size
    if len(sizes) % rate == 0:
        out.append(cumsum)
    return np.array(out, dtype=np.int64), cumsum


def build_padded_token_cumsum(sizes: np.ndarray, sample_size: int, rate: int, offset: int = 0) -> tuple[np.ndarray, int]:
    lib = _host_lib()
    if lib is None:
        return build_padded_token_cumsum_python(sizes, sample_size, rate, offset)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    out = np.empty(len(sizes) // rate + 2, dtype=np.int64)
    total = ctypes.c_int64(0)
    n = lib.flb_build_padded_token_cumsum(sizes.ctypes.data, len(sizes), sample_size, rate, offset, out.ctypes.data, ctypes.byref(total))
    return out[:n].copy(), total.value


def build_sample_idx_python(sizes: np.ndarray, doc_idx: np.ndarray, seq_length: int, num_samples: int) -> np.ndarray:
    out = np.zeros((num_samples + 1, 2), dtype=np.int32)
    pos, doc_offset = 0, 0
    for s in range(1, num_samples + 1):
        remaining = seq_length + 1
        while remaining != 0:
            if pos >= len(doc_idx):
                raise ValueError("doc_idx holds too few tokens")
            doc_length = int(sizes[doc_idx[pos]]) - doc_offset
            remaining -= doc_length
            if remaining <= 0:
                doc_offset += remaining + doc_length - 1
                remaining = 0
            else:
                pos += 1
                doc_offset = 0
        out[s] = (pos, doc_offset)
    return out


def build_sample_idx(sizes: np.ndarray, doc_idx: np.ndarray, seq_length: int, num_samples: int) -> np.ndarray:
    lib = _host_lib()
    if lib is None:
        return build_sample_idx_python(sizes, doc_idx, seq_length, num_samples)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    out = np.zeros((num_samples + 1, 2), dtype=np.int32)
    status = lib.flb_build_sample_idx(sizes.ctypes.data, len(sizes), doc_idx.ctypes.data, len(doc_idx), seq_length, num_samples, out.ctypes.data)
    if status == -1:
        raise ValueError("doc_idx holds too few tokens")
    if status == -2:
        raise IndexError("document index out of range")
    return out


class SampledIndexedDataset:
    def __init__(self, dataset, sampling: SamplingConfig, num_samples: int, seed: int):
        self._dataset = dataset
        self._config = sampling
        self._num_samples = num_samples
        self._seed = seed
        self._truncate = sampling.truncate_documents is not False
        self._sample_tokens = sampling.micro_batch_size  # stream advance per sample
        self._sample_size = sampling.sample_size
        self._max_doc = sampling.sampling_maximum_document_length
        self._rate = sampling.token_cumsum_rate
        self._build()

    @property
    def name(self) -> str:
        return self._dataset.name

    def __len__(self) -> int:
        return self._num_samples

    # ------------------------------------------------------------------------------------------------
    def _cache_paths(self):
        d = self._config.cache_directory
        if d is None:
            return None
        d = pathlib.Path(d)
        tag = f"{self._config.dataset_name}_ns_{self._num_samples}_sl_{self._sample_tokens}_s_{self._seed}"
        return d / f"{tag}_index.npz", d / f"{tag}.yaml"

    def _description(self) -> dict:
        return {
            "dataset": {"name": self._dataset.name, "documents": len(self._dataset), "tokens": int(self._dataset.num_tokens)},
            "num_samples": self._num_samples, "micro_batch_size": self._sample_tokens, "predicted_tokens": self._config.predicted_tokens,
            "seed": self._seed, "shuffle": self._config.shuffle.value, "truncate_documents": self._truncate,
            "maximum_document_length": self._max_doc, "token_cumsum_rate": self._rate,
        }

    def _build(self) -> None:
        paths = self._cache_paths()
        description = self._description()
        if paths is not None and paths[0].exists() and paths[1].exists():
            if yaml.safe_load(paths[1].read_text()) == description:
                data = np.load(paths[0])
                self._doc_order, self._chunk_begin, self._chunk_size, self._cumsum = (data[k] for k in ("order", "begin", "size", "cumsum"))
                return
            logger.warning(f"Sampling cache {paths[1]} does not match the configuration; rebuilding")
        sizes = np.asarray(self._dataset.get_document_sizes(), dtype=np.int64)
        # --- units: whole documents.  When truncating, the stream is the plain concatenation of the documents; the part of a
        # document that falls into a sample is cut into pieces of at most `max_doc` tokens when the sample is assembled,
        # counted from where that part starts (`fast_llm/data/dataset/sampled.py:397-415`), so with the default limit (one
        # sample) a document is never split inside a sample.
        if self._truncate:
            unit_doc, unit_begin, unit_size = np.arange(len(sizes)), np.zeros(len(sizes), dtype=np.int64), sizes
            keep = sizes > 0
        else:
            unit_doc, unit_begin, unit_size = np.arange(len(sizes)), np.zeros(len(sizes), dtype=np.int64), sizes
            keep = sizes <= min(self._max_doc, self._sample_size)
            if (~keep).any():
                logger.warning(f"{int((~keep).sum())}/{len(sizes)} documents of {self._dataset.name} are longer than "
                               f"{min(self._max_doc, self._sample_size)} tokens and will be ignored")
        unit_doc, unit_begin, unit_size = unit_doc[keep], unit_begin[keep], unit_size[keep]
        tokens_per_epoch = int(unit_size.sum())
        if tokens_per_epoch == 0:
            raise RuntimeError(f"Dataset {self._dataset.name} has no usable documents")
        needed = self._num_samples * self._sample_tokens + self._config.predicted_tokens
        slack = 1.0 if self._truncate else 1.3  # padding wastes part of every sample
        epochs = max(math.ceil(needed * slack / tokens_per_epoch), 1) + (0 if self._truncate else 1)
        order = self._shuffled_order(len(unit_doc), epochs)
        self._doc_order = unit_doc[order].astype(np.int64)
        self._chunk_begin = unit_begin[order].astype(np.int64)
        self._chunk_size = unit_size[order].astype(np.int32)
        if self._truncate:
            self._cumsum = np.concatenate([[0], np.cumsum(self._chunk_size, dtype=np.int64)])[:: self._rate].copy()
        else:
            self._cumsum, total = build_padded_token_cumsum(self._chunk_size, self._sample_size, self._rate, 0)
            if total < self._num_samples * self._sample_size:
                raise RuntimeError("not enough documents for the requested number of padded samples")
        if paths is not None:
            paths[0].parent.mkdir(parents=True, exist_ok=True)
            np.savez(paths[0], order=self._doc_order, begin=self._chunk_begin, size=self._chunk_size, cumsum=self._cumsum)
            paths[1].write_text(yaml.safe_dump(description))

    def _shuffled_order(self, units: int, epochs: int) -> np.ndarray:
        shuffle = self._config.shuffle
        rng = np.random.RandomState(self._seed % 2**32)
        if shuffle == ShufflingType.disabled:
            return np.tile(np.arange(units), epochs)
        if shuffle == ShufflingType.full:
            return rng.permutation(np.tile(np.arange(units), epochs))
        parts = []
        for e in range(epochs):
            if shuffle == ShufflingType.skip_first_epoch and e == 0:
                parts.append(np.arange(units))
            else:
                parts.append(np.random.RandomState((self._seed + 7919 * (e + 1)) % 2**32).permutation(units))
        return np.concatenate(parts)

    # ------------------------------------------------------------------------------------------------
    def _unit_starts_from(self, anchor: int, count: int) -> np.ndarray:
        """Stream position of the first token of units anchor*rate ... (exact, rebuilt from the sparse cumsum)."""
        first = anchor * self._rate
        sizes = self._chunk_size[first : first + count].astype(np.int64)
        if self._truncate:
            return self._cumsum[anchor] + np.concatenate([[0], np.cumsum(sizes)[:-1]])
        starts, cumsum = np.empty(len(sizes), dtype=np.int64), int(self._cumsum[anchor])
        for i, size in enumerate(sizes.tolist()):
            if size <= self._sample_size:
                used = cumsum % self._sample_size
                if used + size > self._sample_size:
                    cumsum += self._sample_size - used
            starts[i] = cumsum
            if size <= self._sample_size:
                cumsum += size
        return starts

    def __getitem__(self, index: int) -> list[LanguageModelDocument]:
        if not 0 <= index < self._num_samples:
            raise IndexError(index)
        if self._truncate:
            begin, end = index * self._sample_tokens, index * self._sample_tokens + self._sample_size
        else:
            begin, end = index * self._sample_size, (index + 1) * self._sample_size
        anchor = max(int(np.searchsorted(self._cumsum, begin, side="right")) - 1, 0)
        documents = []
        position = anchor * self._rate
        while True:
            starts = self._unit_starts_from(anchor, 4 * self._rate + 64)
            done = False
            for j, start in enumerate(starts.tolist()):
                unit = position + j
                if unit >= len(self._chunk_size):
                    done = True
                    break
                size = int(self._chunk_size[unit])
                if not self._truncate and size > self._sample_size:
                    continue
                if start >= end:
                    done = True
                    break
                lo, hi = max(begin - start, 0), min(end - start, size)
                if hi > lo:
                    base = int(self._chunk_begin[unit])
                    step = self._max_doc if self._truncate else hi - lo
                    for piece in range(lo, hi, step):
                        documents.append(self._dataset.get_document(int(self._doc_order[unit]), base + piece, base + min(piece + step, hi)))
            if done:
                break
            anchor += 4 + 64 // self._rate
            position = anchor * self._rate
            if anchor >= len(self._cumsum):
                break
        return documents
