"""The data object of a trainer: samples datasets once, then serves per-rank iterators of model inputs.

Each batch-data-parallel rank reads different samples (`index = consumed + step * bdp + rank`); ranks that differ only
in tensor / pipeline / sequence-data coordinates read the same sample and slice it.  A background thread pool
prefetches and preprocesses samples into pinned host memory, so the training loop only issues asynchronous
host-to-device copies.  Parity: `fast_llm/data/data/gpt/data.py:25-141`, `fast_llm/data/data/data_loader.py:9-72`.
"""

import concurrent.futures
import logging
import pathlib
import time
import typing

import torch

from fast_llm_b200.data.config import GPTDataConfig, SamplingConfig
from fast_llm_b200.data.document import LanguageModelBatch, LanguageModelInput
from fast_llm_b200.parallel.topology import DistributedConfig

logger = logging.getLogger(__name__)


class GPTData:
    def __init__(self, config: GPTDataConfig, distributed_config: DistributedConfig):
        config.validate()
        self._config = config
        self._distributed_config = distributed_config
        self._datasets = {}
        self._sampling = {}
        self._preprocessing = {}
        self._is_setup = False
        self._cache_directory = None
        self._distributed = None

    @property
    def config(self):
        return self._config

    def setup(self, cache_directory: pathlib.Path | None = None, distributed=None) -> None:
        """`distributed`: the process groups of the run; needed by datasets that only one rank of a model replica may read
        (a stream): that rank reads and the documents are broadcast to the ranks that share its batch."""
        self._cache_directory = cache_directory
        self._distributed = distributed
        self._is_setup = True

    def sample_dataset(self, dataset_name: str, preprocessing: dict, num_samples: int) -> None:
        """`preprocessing`: the model's requirements (phase, predicted_tokens, vocab_size, micro_batch_splits, ...)."""
        assert self._is_setup
        if dataset_name not in self._config.datasets:
            raise KeyError(f"No dataset configured under `data.datasets.{dataset_name}` (have: {list(self._config.datasets)})")
        c = self._config
        sampling = SamplingConfig(
            gpu=c.gpu, shuffle=c.shuffle, micro_batch_size=c.micro_batch_size, maximum_document_length=c.maximum_document_length,
            truncate_documents=c.truncate_documents, predicted_tokens=preprocessing.get("predicted_tokens", 1),
            cache_directory=None if self._cache_directory is None else pathlib.Path(self._cache_directory) / dataset_name,
            dataset_name=dataset_name, world_size=self._distributed_config.world_size, rank=self._distributed_config.rank,
            seed=c.seed, num_samples=num_samples, vocab_size=preprocessing.get("vocab_size"),
            use_loss_masking_spans=preprocessing.get("use_loss_masking_spans", True),
            use_preference_spans=preprocessing.get("use_preference_spans", False),
            use_grpo_data=preprocessing.get("use_grpo_data", False), use_images=preprocessing.get("use_images", False),
        ).validate()
        t0 = time.perf_counter()
        from fast_llm_b200.data.monitor import DatasetMonitor

        self._datasets[dataset_name] = DatasetMonitor(c.datasets[dataset_name].build_and_sample(sampling, num_samples, c.seed),
                                                      c.data_sample_warn_time_ms)
        self._sampling[dataset_name] = sampling
        self._preprocessing[dataset_name] = dict(preprocessing)
        if self._distributed_config.rank == 0:
            logger.info(f"Sampled dataset {dataset_name}: {num_samples} samples of {sampling.sample_size} tokens "
                        f"in {time.perf_counter() - t0:.2f}s")

    def _load(self, dataset_name: str, index: int, pin: bool) -> list[LanguageModelInput]:
        t0 = time.perf_counter()
        sampling = self._sampling[dataset_name]
        pre = self._preprocessing[dataset_name]
        dataset = self._datasets[dataset_name]
        group = self._shared_batch_group(dataset)
        if group is None:
            documents = dataset[index % max(len(dataset), 1)]
        else:
            # tensor / pipeline / sequence-data ranks of one replica work on the same batch: the first of them reads it
            from fast_llm_b200.parallel.collectives import broadcast_object

            documents = broadcast_object(dataset[index % max(len(dataset), 1)] if group.rank() == 0 else None, group, 0)
        batch = LanguageModelBatch.from_documents(documents, sampling.sample_size, sampling.use_loss_masking_spans)
        dc = self._distributed_config
        inputs = batch.get_model_inputs(
            micro_batch_size=sampling.micro_batch_size, predicted_tokens=sampling.predicted_tokens,
            micro_batch_splits=pre.get("micro_batch_splits", 1), sequence_data_parallel=dc.sequence_data_parallel,
            sequence_data_rank=dc.sequence_data_rank, pin=pin)
        return inputs

    def _shared_batch_group(self, dataset):
        """The group to broadcast documents over, for datasets that must be read once per batch (`requires_broadcast`)."""
        if not getattr(dataset, "requires_broadcast", False) or self._distributed is None:
            return None
        group = getattr(self._distributed, "model_and_sequence_data_group", None)
        return group if group is not None and group.size() > 1 else None

    def get_iterator(self, dataset_name: str, *, consumed_samples: int, num_workers: int = 2, prefetch_factor: int | None = None,
                     timeout: float = 60, preprocess: bool = True, pin_memory: bool | None = None) -> typing.Iterator[list[LanguageModelInput]]:
        """Yields, forever, the model inputs of this rank's next micro-batch."""
        dc = self._distributed_config
        pin = (dc.use_cuda and torch.cuda.is_available()) if pin_memory is None else pin_memory
        stride, offset = dc.batch_data_parallel, dc.batch_data_rank
        depth = max(num_workers * (prefetch_factor or 2), 1)
        if self._shared_batch_group(self._datasets[dataset_name]) is not None:
            num_workers = 0  # the broadcast is a collective: it runs in the calling thread, in step with the other ranks

        def generator():
            index = consumed_samples + offset
            if num_workers == 0:
                while True:
                    yield self._load(dataset_name, index, pin)
                    index += stride
            with concurrent.futures.ThreadPoolExecutor(max_workers=num_workers, thread_name_prefix="data") as pool:
                queue = []
                try:
                    while True:
                        while len(queue) < depth:
                            queue.append(pool.submit(self._load, dataset_name, index, pin))
                            index += stride
                        yield queue.pop(0).result(timeout=timeout)
                finally:
                    for f in queue:
                        f.cancel()

        return generator()
