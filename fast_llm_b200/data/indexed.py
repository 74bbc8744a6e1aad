"""Indexed (random-access by document) dataset combinators: slices and concatenations
(parity: `fast_llm/data/dataset/indexed.py`)."""

import numpy as np


class DatasetSlice:
    def __init__(self, name: str, dataset, begin: int, end: int):
        assert 0 <= begin <= end <= len(dataset), (begin, end, len(dataset))
        self._name, self._dataset, self._begin, self._end = name, dataset, begin, end

    @property
    def name(self):
        return self._name

    def __len__(self):
        return self._end - self._begin

    @property
    def num_tokens(self) -> int:
        return int(self.get_document_sizes().sum())

    def get_document_sizes(self):
        return self._dataset.get_document_sizes()[self._begin : self._end]

    def get_document_size(self, index: int) -> int:
        return self._dataset.get_document_size(index + self._begin)

    def get_document(self, index: int, begin: int = 0, end: int | None = None):
        return self._dataset.get_document(index + self._begin, begin, end)


class ConcatenatedDataset:
    def __init__(self, name: str, datasets: list):
        self._name, self._datasets = name, datasets
        self._offsets = np.concatenate([[0], np.cumsum([len(d) for d in datasets])])

    @property
    def name(self):
        return self._name

    def __len__(self):
        return int(self._offsets[-1])

    @property
    def num_tokens(self) -> int:
        return sum(d.num_tokens for d in self._datasets)

    def get_document_sizes(self):
        return np.concatenate([d.get_document_sizes() for d in self._datasets])

    def _locate(self, index: int):
        which = int(np.searchsorted(self._offsets, index, side="right")) - 1
        return self._datasets[which], index - int(self._offsets[which])

    def get_document_size(self, index: int) -> int:
        dataset, local = self._locate(index)
        return dataset.get_document_size(local)

    def get_document(self, index: int, begin: int = 0, end: int | None = None):
        dataset, local = self._locate(index)
        return dataset.get_document(local, begin, end)
