"""Synthetic dataset: uniform-random token ids, one document per sample, seeded per index
(parity: `fast_llm/data/dataset/gpt/random.py:10-40`)."""

import time

import numpy as np
import torch

from fast_llm_b200.data.document import LanguageModelDocument


class GPTRandomSampledDataset:
    def __init__(self, sampling, name: str, num_samples: int, seed: int, images_per_sample: int = 0,
                 image_patch_grid: tuple[int, int] = (2, 2), image_patch_shape: tuple[int, int, int] = (3, 16, 16)):
        self._images, self._grid, self._patch_shape = images_per_sample, image_patch_grid, image_patch_shape
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
        document = LanguageModelDocument(tokens=torch.from_numpy(tokens))
        if self._images:
            # every image occupies rows * columns consecutive token positions, images spread evenly over the sample
            rows, columns = self._grid
            per_image = rows * columns
            stride = len(tokens) // self._images
            assert stride >= per_image, "sample too short for the requested synthetic images"
            positions = torch.cat([torch.arange(per_image) + i * stride for i in range(self._images)])
            coordinates = torch.stack(torch.meshgrid(torch.arange(rows), torch.arange(columns), indexing="ij"), -1).reshape(-1, 2).repeat(self._images, 1)
            pixels = rng.randint(0, 256, size=(len(positions), *self._patch_shape)).astype(np.uint8)
            document.image_patches = torch.from_numpy(pixels)
            document.image_patch_positions = positions
            document.image_patch_coordinates = coordinates
        return [document]

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
