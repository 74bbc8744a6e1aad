"""A sampled dataset that watches the dataset it wraps: how long each sample takes to load (a warning above a limit) and
which sample failed (logged with its index and the dataset's name before the exception travels on).
Parity: `fast_llm/data/dataset/monitor.py:17-58`."""

import logging
import time

logger = logging.getLogger(__name__)


class DatasetMonitor:
    def __init__(self, dataset, data_sample_warn_time_ms: float):
        self._dataset = dataset
        self._warn_ms = data_sample_warn_time_ms
        self.slow_samples = 0  # samples that took longer than the limit since construction

    def __len__(self) -> int:
        return len(self._dataset)

    def __getitem__(self, index: int):
        start = time.perf_counter()
        try:
            sample = self._dataset[index]
        except Exception:
            logger.error(f"Failed to get sample {index} from dataset {self.name}")
            raise
        elapsed = (time.perf_counter() - start) * 1e3
        if elapsed > self._warn_ms:
            self.slow_samples += 1
            logger.warning(f"Sample {index} from dataset {self.name} took {elapsed:,.2f} ms to load")
        return sample

    @property
    def name(self) -> str:
        return getattr(self._dataset, "name", type(self._dataset).__name__)

    @property
    def requires_broadcast(self) -> bool:
        return getattr(self._dataset, "requires_broadcast", False)

    def __getattr__(self, item):
        return getattr(self._dataset, item)
