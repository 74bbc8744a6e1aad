"""Experiment directory, per-rank logging and run bookkeeping.

`experiment_dir/{config.yaml, config_verbose.yaml, runs/<n>/{logs/logs_rank_NN.txt, artifacts/<rank>/...},
checkpoint/, export/, dataset_cache/}`.  Parity: `fast_llm/engine/config_utils/run.py:21-273`,
`fast_llm/engine/config_utils/logging.py:14-98`, `fast_llm/engine/config_utils/interval.py`.
"""

import logging
import os
import pathlib
import sys
import typing

import yaml

from fast_llm_b200.config import Config, Field, FieldHint, FieldVerboseLevel, check_field, config_class, skip_valid_if_none
from fast_llm_b200.config.runnable import RunnableConfig
from fast_llm_b200.utils import Assert
from fast_llm_b200.utils.tensor_logs import TensorLogs

logger = logging.getLogger(__name__)


@config_class()
class IntervalConfig(Config):
    interval: int | None = Field(default=None, desc="Act every this many iterations (None / 0: never).", hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.gt, 0)))
    offset: int = Field(default=0, desc="Offset of the first action.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))

    def _validate(self):
        if self.interval:
            self.offset = self.offset % self.interval
        super()._validate()

    def enabled(self, iteration: int | None = None) -> bool:
        return bool(self.interval) and (iteration is None or (iteration - self.offset) % self.interval == 0)

    def is_sub_interval(self, other: "IntervalConfig") -> bool:
        if not self.enabled():
            return True
        return other.enabled() and self.interval % other.interval == 0 and (other.offset % other.interval) == (self.offset % other.interval)

    def assert_sub_interval(self, other: "IntervalConfig") -> None:
        assert self.is_sub_interval(other), f"{self} is not a sub-interval of {other}"

    def get_count(self, iteration: int) -> int:
        return (iteration - self.offset) // self.interval + 1 if self.enabled() and iteration >= self.offset else 0


@config_class()
class TensorLogsConfig(Config):
    save: bool = Field(default=False, desc="Store tensor logs as run artifacts.", hint=FieldHint.logging)
    show: bool = Field(default=True, desc="Print tensor logs.", hint=FieldHint.logging)
    max_elements: int = Field(default=8, desc="Sampled entries shown per tensor.", hint=FieldHint.logging, valid=check_field(Assert.gt, 0))
    full_tensors: bool = Field(default=False, desc="Store whole tensors (parity tests).")


@config_class()
class RunConfig(Config):
    tensor_logs: TensorLogsConfig = Field(desc="Tensor logging.", hint=FieldHint.logging)
    structured_logs: bool = Field(default=True, desc="Prefix log lines with time and rank.", hint=FieldHint.logging)
    experiment_dir: pathlib.Path | None = Field(default=None, desc="Where everything the run writes goes.", hint=FieldHint.core)
    enable_all_loggers: bool = Field(default=False, hint=FieldHint.logging)
    log_timestamps: bool = Field(default=True, hint=FieldHint.logging)
    experiment_name: str | None = Field(default=None, desc="Name for W&B (default: the experiment directory's name).", hint=FieldHint.feature)
    torch_dynamo_enable: bool = Field(default=True, desc="Accepted for compatibility; no tracing compiler is on the hot path.", hint=FieldHint.expert)
    enable_triton_kernels: bool = Field(default=True, desc="Accepted for compatibility; kernels are native CUDA.", hint=FieldHint.expert)
    triton_linear_kernels: bool = Field(default=False, desc="Accepted for compatibility.", hint=FieldHint.performance)
    model_debug_level: int = Field(default=0, desc="Debug verbosity of all models.", hint=FieldHint.logging, valid=check_field(Assert.geq, 0))

    def _validate(self):
        if self.experiment_dir is None:
            assert not self.tensor_logs.save if isinstance(self.tensor_logs, TensorLogsConfig) else True
        super()._validate()


@config_class()
class ExperimentConfig(RunnableConfig):
    run: RunConfig = Field(desc="Run-wide settings.", hint=FieldHint.core)

    def configure_logging(self) -> None:
        configure_logging(rank=int(os.environ.get("RANK", 0)), world_size=int(os.environ.get("WORLD_SIZE", 1)))

    def get_run(self, distributed) -> "Run":
        return Run(config=self, distributed=distributed)


def configure_logging(*, log_timestamps: bool = True, enable_all_loggers: bool = False, rank: int = 0, world_size: int = 1,
                      directory: pathlib.Path | str | None = None) -> None:
    rank_str = str(rank).zfill(len(str(max(world_size - 1, 0))))
    fmt = f"{'%(asctime)s ' if log_timestamps else ''}{f'[Rank {rank_str}] ' if world_size > 1 else ''}%(message)s"
    root = logging.getLogger()
    for handler in list(root.handlers):
        root.removeHandler(handler)
    handlers: list[logging.Handler] = [logging.StreamHandler(sys.stdout)]
    if directory is not None:
        pathlib.Path(directory).mkdir(parents=True, exist_ok=True)
        handlers.append(logging.FileHandler(pathlib.Path(directory) / f"logs_rank_{rank_str}.txt"))
    for handler in handlers:
        handler.setFormatter(logging.Formatter(fmt))
        root.addHandler(handler)
    root.setLevel(logging.INFO)
    if not enable_all_loggers:
        for name in logging.root.manager.loggerDict:
            if not name.startswith(("fast_llm_b200", "__main__")):
                logging.getLogger(name).setLevel(logging.WARNING)


class Run:
    """Created once per process; owns the run index, directories and artifact files."""

    def __init__(self, *, config: ExperimentConfig, distributed):
        from fast_llm_b200.parallel.collectives import broadcast_scalar

        self._config = config.run
        self._distributed = distributed
        dc = distributed.config
        self._rank = dc.rank
        self._is_main_rank = dc.rank == 0
        self._is_model_parallel_main_rank = dc.data_rank == 0
        self._is_pipeline_parallel_main_rank = dc.data_rank == 0 and dc.tensor_rank == 0
        self.index = None
        self._experiment_directory = self._config.experiment_dir
        self._artifact_dir = None
        if self._experiment_directory is not None:
            exp = pathlib.Path(self._experiment_directory)
            if self._is_main_rank:
                (exp / "runs").mkdir(parents=True, exist_ok=True)
                existing = [int(p.name) for p in (exp / "runs").iterdir() if p.name.isdigit()]
                run = max(existing) + 1 if existing else 0
            else:
                run = 0
            self.index = int(broadcast_scalar(run, torch_int64(), distributed.world_group))
            run_dir = exp / "runs" / str(self.index)
            self._artifact_dir = run_dir / "artifacts" / str(self._rank)
            log_dir = run_dir / "logs"
            if self._is_main_rank:
                (run_dir / "artifacts").mkdir(parents=True, exist_ok=True)
                log_dir.mkdir(parents=True, exist_ok=True)
                (exp / "config.yaml").write_text(yaml.safe_dump(config.to_dict(FieldVerboseLevel.explicit), sort_keys=False))
                (exp / "config_verbose.yaml").write_text(yaml.safe_dump(config.to_dict(FieldVerboseLevel.performance), sort_keys=False))
            from fast_llm_b200.parallel.collectives import safe_barrier

            safe_barrier(distributed.world_group, "run_setup")
            configure_logging(log_timestamps=self._config.log_timestamps, enable_all_loggers=self._config.enable_all_loggers,
                              rank=dc.rank, world_size=dc.world_size, directory=log_dir)
        else:
            configure_logging(log_timestamps=self._config.log_timestamps, enable_all_loggers=self._config.enable_all_loggers,
                              rank=dc.rank, world_size=dc.world_size)
        self._tensor_log_index = 0

    @property
    def is_main_rank(self) -> bool:
        return self._is_main_rank

    @property
    def experiment_directory(self) -> pathlib.Path | None:
        return None if self._experiment_directory is None else pathlib.Path(self._experiment_directory)

    @property
    def experiment_name(self) -> str:
        if self._config.experiment_name:
            return self._config.experiment_name
        return "default" if self._experiment_directory is None else pathlib.Path(self._experiment_directory).name

    def open_artifact(self, name: str, mode: str = "w", verbose: bool = True):
        if self._artifact_dir is None:
            return open(os.devnull, mode)
        self._artifact_dir.mkdir(parents=True, exist_ok=True)
        path = self._artifact_dir / name
        if verbose:
            logger.info(f"Saving artifact to {path}")
        return path.open(mode)

    def save_logged_tensors(self, iteration: int | str) -> None:
        import torch

        logs = TensorLogs.get()
        if logs and self._config.tensor_logs.save and self._artifact_dir is not None:
            self._artifact_dir.mkdir(parents=True, exist_ok=True)
            torch.save(logs, self._artifact_dir / f"tensor_logs_{iteration}.pt")
        TensorLogs.clear()

    def __enter__(self):
        tl = self._config.tensor_logs
        TensorLogs.reset(save=tl.save, show=tl.show, max_elements=tl.max_elements, full_tensors=tl.full_tensors)
        return self

    def __exit__(self, exc_type, exc, tb):
        TensorLogs.enabled = False
        if exc is not None:
            logger.error(f"Run failed with {exc_type.__name__}: {exc}")


def torch_int64():
    import torch

    return torch.int64


def log_main_rank(*message, log_fn=logger.info):
    if int(os.environ.get("RANK", 0)) == 0:
        log_fn(" ".join(map(str, message)))


def log_pipeline_parallel_main_rank(*message, log_fn=logger.info, distributed_config=None):
    if distributed_config is None or (distributed_config.data_rank == 0 and distributed_config.tensor_rank == 0):
        log_fn(" ".join(map(str, message)))
