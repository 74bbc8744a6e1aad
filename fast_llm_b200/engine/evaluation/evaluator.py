"""Evaluators run at intervals during training or stand-alone (`fast-llm evaluate`).

`LossEvaluator` measures the losses on a named validation dataset for a fixed number of batches
(parity: `fast_llm/engine/evaluation/evaluator.py:73-165`)."""

import logging
import time

from fast_llm_b200.engine.schedule.schedule import Schedule
from fast_llm_b200.parallel.topology import PhaseType
from fast_llm_b200.utils.metrics import format_metrics

logger = logging.getLogger(__name__)


class Evaluator:
    def __init__(self, name: str, config):
        self._name = name
        self._config = config
        self._is_setup = False

    def setup(self, trainer, distributed, run) -> None:
        self._trainer, self._distributed, self._run = trainer, distributed, run
        self._is_setup = True

    def run(self, completed_steps: int, force: bool = False) -> dict | None:
        raise NotImplementedError


class LossEvaluator(Evaluator):
    def setup(self, trainer, distributed, run) -> None:
        super().setup(trainer, distributed, run)
        self._enabled = bool(self._config.iterations) and (self._config.enabled() or True)
        self._iterator = None
        self._evaluation_count = 0
        if not self._enabled:
            return
        config = trainer._config
        self._schedule = Schedule(trainer.multi_stage, config.schedule, config.model.distributed, PhaseType.validation)
        self._dataset_name = self._config.dataset_name or self._name
        train_iters = config.training.train_iters
        runs = (self._config.get_count(train_iters) + 1) if self._config.enabled() else 1
        self._samples = self._config.iterations * self._schedule.samples_per_batch
        preprocessing = trainer._get_preprocessing(PhaseType.validation)
        trainer._data.sample_dataset(self._dataset_name, preprocessing, runs * self._samples)

    def run(self, completed_steps: int, force: bool = False) -> dict | None:
        if not self._enabled or not (force or self._config.enabled(completed_steps)):
            return None
        trainer = self._trainer
        if self._iterator is None:
            self._iterator = trainer._data.get_iterator(self._dataset_name, consumed_samples=self._evaluation_count * self._samples,
                                                        num_workers=trainer._config.training.num_workers)
        t0 = time.perf_counter()
        totals: dict[str, float] = {}
        for i in range(self._config.iterations):
            losses, _, _ = trainer.runner.run_step(self._iterator, self._schedule, iteration=completed_steps * 1000 + i)
            for k, v in losses.items():
                totals[k] = totals.get(k, 0.0) + v
        self._evaluation_count += 1
        elapsed = time.perf_counter() - t0
        metrics = {k: v / self._config.iterations for k, v in totals.items()}
        metrics.update(iteration=completed_steps, train_iters=trainer._config.training.train_iters,
                       step_time_ms=elapsed * 1e3 / self._config.iterations)
        if self._distributed.config.rank == 0:
            logger.info(format_metrics(metrics, trainer.runner._loss_definitions.values(), PhaseType.validation, self._name))
        return {f"validation.{self._name}": metrics}
