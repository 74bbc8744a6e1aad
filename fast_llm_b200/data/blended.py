"""Deterministic blending of sampled datasets (Megatron-compatible): sample i comes from the dataset whose share of
samples so far lags its weight the most (parity: `fast_llm/data/dataset/blended.py:13-85`)."""

import numpy as np


class BlendedDataset:
    def __init__(self, name: str, datasets: list, weights: list[float], num_samples: int):
        self._name, self._datasets, self._num_samples = name, datasets, num_samples
        w = np.asarray(weights, dtype=np.float64)
        self._weights = w / w.sum()
        self._dataset_index, self._sample_index = self._build(num_samples)

    def _build(self, n: int):
        """Greedy error minimisation: at step i pick argmax_d (w_d * (i + 1) - count_d)."""
        counts = np.zeros(len(self._weights), dtype=np.int64)
        which = np.empty(n, dtype=np.int16)
        within = np.empty(n, dtype=np.int64)
        for i in range(n):
            d = int(np.argmax(self._weights * (i + 1) - counts))
            which[i], within[i] = d, counts[d]
            counts[d] += 1
        for d, dataset in enumerate(self._datasets):
            assert counts[d] <= len(dataset), f"dataset {d} has {len(dataset)} samples, blending needs {counts[d]}"
        return which, within

    @property
    def name(self):
        return self._name

    def __len__(self):
        return self._num_samples

    def __getitem__(self, index: int):
        return self._datasets[int(self._dataset_index[index])][int(self._sample_index[index])]
