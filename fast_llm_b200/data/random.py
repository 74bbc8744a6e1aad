"""Synthetic dataset: uniform-random token ids, one document per sample, seeded per index
(parity: `fast_llm/data/dataset/gpt/random.py:10-40`)."""

import time

import numpy as np
import torch

from fast_llm_b200.data.document import LanguageModelDocument


class GPTRandomSampledDataset:
    def __init__(self, sampling, name: str, num_samples: int, seed: int):
        self._name = name
        self._seed = seed
        self._sampling = sampling
        self._num_samples = num_samples
        self._vocab_size = sampling.vocab_size or 32000

    def __len__(self) -> int:
        return self._num_samples

    def __getitem__(self, index: int) -> list[LanguageModelDocument]:
        rng = np.random.RandomState((self._seed + 48576439 + 74593 * index) % 2**32)
        tokens = rng.randint(0, self._vocab_size, size=(self._sampling.sample_size,))
        return [LanguageModelDocument(tokens=torch.from_numpy(tokens))]

    @property
    def name(self) -> str:
        return self._name


class SlowDataset:
    """Wraps a dataset and sleeps on every access (exercises the slow-sample warning)."""

    def __init__(self, dataset, sleep: float):
        self._dataset, self._sleep = dataset, sleep

    def __len__(self):
        return len(self._dataset)

    def __getitem__(self, index):
        time.sleep(self._sleep)
        return self._dataset[index]

    @property
    def name(self):
        return self._dataset.name
