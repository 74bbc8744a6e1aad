"""The training loop: setup (model, optimizer, data, schedules, evaluators), resume, iterate, log, evaluate,
checkpoint, export, stop cleanly on signals.  Parity: `fast_llm/engine/training/trainer.py:45-472`.
"""

import logging
import math
import pathlib
import shutil
import time
import typing

import torch

from fast_llm_b200.data.data import GPTData
from fast_llm_b200.engine.multi_stage.config import StageMode
from fast_llm_b200.engine.optimizer.optimizer import Optimizer
from fast_llm_b200.engine.schedule.runner import ScheduleRunner
from fast_llm_b200.engine.schedule.schedule import Schedule
from fast_llm_b200.engine.training.config import TrainerConfig
from fast_llm_b200.parallel.collectives import allreduce_scalar, broadcast_scalar, safe_barrier
from fast_llm_b200.parallel.topology import PhaseType
from fast_llm_b200.utils import Interrupter, get_and_reset_memory_usage_mib
from fast_llm_b200.utils.device_errors import check_device_errors, register_kernel_library_sources
from fast_llm_b200.utils.metrics import format_metrics

logger = logging.getLogger(__name__)


class Trainer:
    config_class: typing.ClassVar[type[TrainerConfig]] = TrainerConfig

    def __init__(self, config: TrainerConfig):
        config.validate()
        self._config = config
        self._is_setup = False
        self._data = self._get_data()
        model_class = type(config.model).get_model_class()
        self._multi_stage = model_class(config.model, optimizer_state_names=config.optimizer.state_names)
        self._reference_models = {}
        for name, ref_config in config.reference_models.items():
            from fast_llm_b200.engine.inference.runner import InferenceRunner

            ref_model = type(ref_config.model).get_model_class()(ref_config.model)
            self._reference_models[name] = (ref_config, InferenceRunner(ref_model))
        self._runner = ScheduleRunner(config=config.schedule, multi_stage=self._multi_stage, distributed_config=config.model.distributed)
        self._completed_steps = 0
        self._documents_seen = 0
        self._callbacks = {}
        self._evaluators = {}

    def _get_data(self):
        return GPTData(self._config.data, self._config.model.distributed)

    @property
    def multi_stage(self):
        return self._multi_stage

    @property
    def optimizer(self):
        return self._optimizer

    @property
    def runner(self):
        return self._runner

    @property
    def completed_steps(self) -> int:
        return self._completed_steps

    # ------------------------------------------------------------------------------------------------
    def setup(self, distributed, run) -> None:
        assert not self._is_setup
        self._is_setup = True
        self._distributed = distributed
        self._run = run
        config = self._config
        self._multi_stage.setup(distributed, mode=StageMode.training)
        for name, (ref_config, runner) in self._reference_models.items():
            runner.setup(distributed, ref_config)
            self._multi_stage.base_model.add_reference_model(name, runner)
        self._optimizer = Optimizer(config.optimizer, self._multi_stage.get_param_groups(), self._multi_stage.get_grad_norm_slices(),
                                    distributed, compute_dtype=config.model.distributed.compute_dtype.torch,
                                    weight_arena=self._multi_stage.weight_arena, grad_norm_partials=self._multi_stage.grad_norm_partials)
        self._runner.setup(distributed, self._optimizer)
        self._runner.set_run(run)
        cache_dir = None if run.experiment_directory is None else run.experiment_directory / "dataset_cache"
        self._data.setup(cache_dir, distributed)
        self._schedules = {PhaseType.training: Schedule(self._multi_stage, config.schedule, config.model.distributed, PhaseType.training)}
        self._samples_per_batch = self._schedules[PhaseType.training].samples_per_batch
        preprocessing = self._get_preprocessing(PhaseType.training)
        if config.training.train_iters > 0:
            self._data.sample_dataset("training", preprocessing, config.training.train_iters * self._samples_per_batch)
        for name, evaluator_config in config.training.evaluators.items():
            evaluator = evaluator_config.get_evaluator(name)
            evaluator.setup(self, distributed, run)
            self._evaluators[name] = evaluator
        for name, callback_config in config.callbacks.items():
            self._callbacks[name] = callback_config.get_callback(self._multi_stage)
        if distributed.device.type == "cuda":
            register_kernel_library_sources()
        safe_barrier(distributed.world_group, "data_preparation", config.training.timeout)

    def _check_device_errors(self) -> None:
        """Every rank raises if a bounded device-side wait (peer barrier, TMA / tensor-core pipeline) ran out on any rank
        since the last call.  Called where the host synchronises anyway; nothing is written to disk past a failure."""
        check_device_errors(self._distributed.world_group, self._distributed.device)

    def _get_preprocessing(self, phase: PhaseType) -> dict:
        pre = self._multi_stage.base_model.get_preprocessing_config(phase)
        pre["micro_batch_splits"] = self._config.schedule.micro_batch_splits
        return pre

    # ------------------------------------------------------------------------------------------------
    def run(self) -> None:
        assert self._is_setup
        from fast_llm_b200.engine.training.wandb import Wandb

        self._wandb = Wandb(self._config.training.wandb, self._run, self._config, module=getattr(self, "_wandb_module", None))
        with self._wandb, self._config.profiling.get_profiler(distributed_config=self._config.model.distributed, start_step=self._completed_steps, run=self._run) as profiler:
            self._run_training(profiler)

    def _run_training(self, profiler) -> None:
        self._prepare_training_state()
        if self._config.training.train_iters > 0 and self._completed_steps < self._config.training.train_iters:
            for callback in self._callbacks.values():
                callback.run_begin(self._completed_steps)
            done, metrics = self._train(profiler)
            for callback in self._callbacks.values():
                callback.train_end(self._completed_steps)
        else:
            done, metrics = True, {}
        if done and self._evaluators and not self._config.training.train_iters:
            for evaluator in self._evaluators.values():
                result = evaluator.run(self._completed_steps, force=True) or {}
                metrics.update(result)
                if result and getattr(self, "_wandb", None) is not None:
                    self._wandb.log_metrics(self._completed_steps, result)
        self._final_metrics = metrics

    def _train(self, profiler) -> tuple[bool, dict]:
        config = self._config.training
        distributed_config = self._config.model.distributed
        schedule = self._schedules[PhaseType.training]
        iterator = self._data.get_iterator(
            "training", consumed_samples=self._completed_steps * self._samples_per_batch, num_workers=config.num_workers,
            prefetch_factor=config.prefetch_factor, timeout=config.timeout or 60)
        advanced_iters, skipped_iters, nan_iters = 0, 0, 0
        total_losses: dict[str, float] = {}
        metrics: dict = {}
        done = False
        stop = False
        has_gpu = self._distributed.device.type == "cuda"
        batch_tokens = self._samples_per_batch * self._config.data.micro_batch_size
        logger.info("Starting training") if distributed_config.rank == 0 else None
        start_time = last_time = time.perf_counter()
        start_iteration = last_iteration = self._completed_steps
        if has_gpu:
            torch.cuda.synchronize()
        with Interrupter(True) as interrupter:
            while not done:
                is_logging = config.logs.enabled(self._completed_steps + 1)
                reduced_losses, update_successful, step_metrics = self._runner.run_step(
                    iterator, schedule, iteration=self._completed_steps + 1, return_metrics=is_logging)
                if update_successful:
                    advanced_iters += 1
                    for name, value in reduced_losses.items():
                        total_losses[name] = total_losses.get(name, 0.0) + value
                else:
                    skipped_iters += 1
                    nan_iters += not all(math.isfinite(v) for v in reduced_losses.values())
                self._completed_steps += 1
                for callback in self._callbacks.values():
                    extra = callback.step_end(self._completed_steps, reduced_losses, update_successful, step_metrics,
                                              self._completed_steps * self._samples_per_batch)
                    if extra and step_metrics is not None:
                        step_metrics.update(extra)
                if is_logging:
                    if has_gpu:
                        torch.cuda.synchronize()
                    self._check_device_errors()
                    now = time.perf_counter()
                    step_time = (now - last_time) / max(self._completed_steps - last_iteration, 1)
                    remaining = config.train_iters - self._completed_steps
                    train_metrics = {
                        "train_iters": config.train_iters, "batch_size": self._samples_per_batch, "iteration": self._completed_steps,
                        **{name: value / max(advanced_iters, 1) for name, value in total_losses.items()},
                        "consumed_samples": self._completed_steps * self._samples_per_batch,
                        "consumed_tokens": self._completed_steps * batch_tokens,
                        "step_time_ms": step_time * 1e3,
                        "step_time_average_ms": (now - start_time) * 1e3 / max(self._completed_steps - start_iteration, 1),
                        "remaining_time": remaining * step_time,
                        "completion_time": time.time() + remaining * step_time,
                        "percent_done": 100 * self._completed_steps / max(config.train_iters, 1),
                        "skipped_iters": skipped_iters, "nan_iters": nan_iters,
                        "tokens_per_sec_per_gpu": batch_tokens / distributed_config.world_size / step_time,
                        **schedule.get_compute_metrics(step_time, self._sample_kwargs()),
                        **{k: (v.item() if torch.is_tensor(v) else v) for k, v in (step_metrics or {}).items()},
                        **get_and_reset_memory_usage_mib(),
                    }
                    metrics["training"] = train_metrics
                    if distributed_config.rank == 0:
                        logger.info(format_metrics(train_metrics, self._runner._loss_definitions.values(), PhaseType.training))
                    self._wandb_log(train_metrics)
                    last_time, last_iteration = now, self._completed_steps
                    advanced_iters, skipped_iters, nan_iters = 0, 0, 0
                    total_losses = {}
                profiler.step()
                done = self._completed_steps >= config.train_iters
                if done:
                    self._check_device_errors()
                for name, evaluator in self._evaluators.items():
                    self._runner.wait_for_optimizer()
                    result = evaluator.run(self._completed_steps, force=done)
                    if result:
                        metrics.update(result)
                        wandb = getattr(self, "_wandb", None)
                        if wandb is not None:  # evaluation results travel with the step they were measured at
                            wandb.log_metrics(self._completed_steps, result)
                if config.export.enabled(None if done else self._completed_steps):
                    self._save_checkpoint(config.export, metrics)
                if interrupter.enabled:
                    stop = bool(allreduce_scalar(int(interrupter.interrupted), torch.int32, self._distributed.world_group, device=self._distributed.device))
                stop = stop or config.shutdown.enabled(self._completed_steps)
                if config.checkpoint.enabled(None if (done or stop) and config.checkpoint.enabled() else self._completed_steps):
                    self._save_checkpoint(config.checkpoint, metrics)
                if stop:
                    break
        return done, metrics

    def _sample_kwargs(self) -> dict:
        from fast_llm_b200.layers.kwargs import BlockKwargs

        tokens = self._config.data.micro_batch_size
        return {BlockKwargs.num_tokens: tokens // self._config.schedule.micro_batch_splits, BlockKwargs.max_seqlen_k: tokens}

    def _wandb_log(self, metrics: dict) -> None:
        wandb = getattr(self, "_wandb", None)
        if wandb is not None:
            wandb.log_metrics(self._completed_steps, {"train": metrics})

    # ------------------------------------------------------------------------------------------------
    def _prepare_training_state(self) -> None:
        last = self._get_last_checkpoint()
        if last is None:
            pretrained = self._config.pretrained
            if pretrained.path is not None and pretrained.model_weights:
                logger.info(f"Loading pretrained weights from {pretrained.path}")
                self._multi_stage.load_checkpoint(pretrained)
            else:
                self._multi_stage.initialize_weights()
            self._optimizer.reset_state()
        else:
            logger.info(f"Resuming from checkpoint {last}")
            self._load_checkpoint(self._config.training.checkpoint, last)
        for name, (ref_config, runner) in self._reference_models.items():
            runner.load(ref_config)

    def _checkpoint_base(self, config) -> pathlib.Path:
        return config.get_save_directory(self._run.experiment_directory)

    def _save_checkpoint(self, config, metrics: dict | None, iteration: int | None = None) -> None:
        iteration = self._completed_steps if iteration is None else iteration
        self._runner.wait_for_optimizer()
        self._check_device_errors()
        directory = self._checkpoint_base(config) / str(iteration)
        if self._run.is_main_rank:
            directory.mkdir(parents=True, exist_ok=True)
        safe_barrier(self._distributed.world_group, f"{config.save_name} {iteration} enter", device=self._distributed.device)
        extra = {"optimizer": self._optimizer.save(), "completed_steps": self._completed_steps, "documents_seen": self._documents_seen,
                 "metrics": _plain(metrics or {})}
        self._multi_stage.save_checkpoint(config.get_save_config(directory, timeout=self._config.training.timeout), extra)
        safe_barrier(self._distributed.world_group, f"{config.save_name} {iteration} exit", timeout=self._config.training.timeout, device=self._distributed.device)
        if self._run.is_main_rank:
            (directory / "ok").touch()
            existing = sorted(int(p.name) for p in self._checkpoint_base(config).iterdir() if p.name.isdigit() and (p / "ok").exists())
            for old in config.to_delete(existing):
                shutil.rmtree(self._checkpoint_base(config) / str(old), ignore_errors=True)
        logger.info(f"Saved {config.save_name} at iteration {iteration} to {directory}") if self._run.is_main_rank else None

    def _load_checkpoint(self, config, iteration: int) -> None:
        directory = self._checkpoint_base(config) / str(iteration)
        metadata = self._multi_stage.load_checkpoint(config.get_load_config(directory, timeout=self._config.training.timeout))
        metadata = metadata or {}
        self._optimizer.load(metadata.get("optimizer", {}))
        self._completed_steps = metadata.get("completed_steps", iteration)
        self._documents_seen = metadata.get("documents_seen", 0)

    def _get_last_checkpoint(self) -> int | None:
        if self._run.experiment_directory is None:
            return None
        base = self._checkpoint_base(self._config.training.checkpoint)
        last = -1
        if self._run.is_main_rank and base.is_dir():
            done = [int(p.name) for p in base.iterdir() if p.name.isdigit() and (p / "ok").exists()]
            last = max(done) if done else -1
        last = int(broadcast_scalar(last, torch.int64, self._distributed.world_group, device=self._distributed.device))
        return None if last < 0 else last


def _plain(obj):
    if isinstance(obj, dict):
        return {str(k): _plain(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_plain(v) for v in obj]
    if torch.is_tensor(obj):
        return obj.item() if obj.numel() == 1 else obj.tolist()
    if isinstance(obj, (int, float, str, bool)) or obj is None:
        return obj
    return str(obj)
