"""The `fast-llm train` config tree (parity: `fast_llm/engine/training/config.py:40-370`)."""

import typing

from fast_llm_b200.config import Config, Field, FieldHint, FieldUpdate, check_field, config_class, skip_valid_if_none
from fast_llm_b200.config.runnable import RunnableConfig
from fast_llm_b200.data.config import DataConfig, RedisConfig
from fast_llm_b200.engine.checkpoint.config import (
    CheckpointLoadConfig,
    CheckpointSaveConfig,
    CheckpointStateSaveConfigBase,
    DistributedCheckpointFormat,
)
from fast_llm_b200.engine.multi_stage.config import PretrainedFastLLMModelConfig
from fast_llm_b200.engine.optimizer.config import OptimizerConfig
from fast_llm_b200.engine.run import ExperimentConfig, IntervalConfig
from fast_llm_b200.engine.schedule.config import ScheduleConfig
from fast_llm_b200.parallel.topology import DistributedBackend
from fast_llm_b200.utils import Assert
from fast_llm_b200.utils.profile import ProfilingConfig


@config_class()
class WandbAlertConfig(IntervalConfig):
    status_updates: bool | None = Field(default=None, desc="Send start / stop / crash alerts.", hint=FieldHint.feature)

    def _validate(self):
        if self.status_updates is None:
            self.status_updates = self.enabled()
        super()._validate()


@config_class()
class MetricsLogsConfig(IntervalConfig):
    interval = FieldUpdate(default=100)


@config_class()
class WandbConfig(Config):
    alert: WandbAlertConfig = Field(desc="Alerts.", hint=FieldHint.core)
    group_name: str = Field(default="default", hint=FieldHint.feature)
    project_name: str = Field(default="fast_llm", hint=FieldHint.feature)
    entity_name: str | None = Field(default=None, desc="W&B entity; None disables W&B.", hint=FieldHint.feature)


@config_class(registry=True)
class EvaluatorConfig(IntervalConfig):
    _abstract: typing.ClassVar[bool] = True

    @classmethod
    def _get_default_subclass(cls):
        return LossEvaluatorConfig if cls is EvaluatorConfig else cls

    def get_evaluator(self, name, eval_config, batch_config, data_load_num_proc, train_iters=None):
        raise NotImplementedError


@config_class(dynamic_type={EvaluatorConfig: "loss"})
class LossEvaluatorConfig(EvaluatorConfig):
    _abstract: typing.ClassVar[bool] = False
    iterations: int | None = Field(default=None, desc="Validation batches per evaluation (None disables).", hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.gt, 0)))
    dataset_name: str | None = Field(default=None, desc="Dataset to evaluate on (default: the evaluator's name).")

    def get_evaluator(self, name, *args, **kwargs):
        from fast_llm_b200.engine.evaluation.evaluator import LossEvaluator

        return LossEvaluator(name, self, *args, **kwargs)


@config_class()
class TrainingCheckpointBaseConfig(IntervalConfig):
    _abstract = True
    save_name: typing.ClassVar[str] = "save"
    keep: int | None = Field(default=None, desc="Keep only the newest this many.", hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.gt, 0)))
    keep_every: int | None = Field(default=None, desc="Additionally keep every this-many-th.", hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.gt, 0)))

    def get_save_directory(self, experiment_directory):
        import pathlib

        return pathlib.Path(experiment_directory) / self.save_name

    def to_delete(self, iterations: list[int]) -> list[int]:
        if not self.keep:
            return []
        candidates = sorted(iterations)[: -self.keep]
        if self.keep_every:
            candidates = [i for i in candidates if (i // self.interval) % self.keep_every != 0]
        return candidates


@config_class()
class TrainingCheckpointConfig(TrainingCheckpointBaseConfig):
    _abstract = False
    save_name: typing.ClassVar[str] = "checkpoint"
    keep = FieldUpdate(default=5)

    def get_save_config(self, path, timeout: float | None):
        return CheckpointSaveConfig(path=path, format=DistributedCheckpointFormat, model_weights=True, optimizer_state=True, timeout=timeout)

    def get_load_config(self, path, timeout: float | None):
        return CheckpointLoadConfig(path=path, format=DistributedCheckpointFormat, model_weights=True, optimizer_state=True, timeout=timeout)


@config_class()
class TrainingExportConfig(TrainingCheckpointBaseConfig, CheckpointStateSaveConfigBase):
    _abstract = False
    save_name: typing.ClassVar[str] = "export"

    def get_save_directory(self, experiment_directory):
        import pathlib

        return pathlib.Path(experiment_directory) / self.save_name / self.format.name

    def get_save_config(self, path, timeout: float | None):
        return CheckpointSaveConfig(path=path, format=self.format, model_weights=self.model_weights, optimizer_state=self.optimizer_state,
                                    parameters_per_file=self.parameters_per_file, data_type=self.data_type, timeout=timeout)


@config_class()
class ShutdownConfig(IntervalConfig):
    """Stop (after checkpointing) at these iterations: for pre-emptible jobs."""


@config_class()
class TrainingConfig(Config):
    evaluators: dict[str, EvaluatorConfig] = Field(default_factory=dict, desc="Named evaluators.", hint=FieldHint.core)
    logs: MetricsLogsConfig = Field(desc="Metric logging interval.", hint=FieldHint.core)
    checkpoint: TrainingCheckpointConfig = Field(desc="Resumable checkpoints.", hint=FieldHint.core)
    export: TrainingExportConfig = Field(desc="Exported (converted) checkpoints.", hint=FieldHint.core)
    shutdown: ShutdownConfig = Field(desc="Planned shutdown points.", hint=FieldHint.core)
    wandb: WandbConfig = Field(desc="Weights & Biases.", hint=FieldHint.core)
    train_iters: int = Field(default=0, desc="Total training iterations.", hint=FieldHint.core, valid=check_field(Assert.geq, 0))
    num_workers: int = Field(default=2, desc="Data loading workers.", hint=FieldHint.optional, valid=check_field(Assert.geq, 0))
    prefetch_factor: int | None = Field(default=None, desc="Samples prefetched per worker.", hint=FieldHint.performance, valid=skip_valid_if_none(check_field(Assert.gt, 0)))
    timeout: float | None = Field(default=3600, desc="Timeout of slow collective sections (checkpoints, data preparation).", hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.gt, 0)))

    def _validate(self):
        super()._validate()
        self.shutdown.assert_sub_interval(self.checkpoint)


@config_class(registry=True)
class TrainerCallbackConfig(Config):
    def get_callback(self, model):
        raise NotImplementedError


@config_class()
class WeightsBroadcastConfig(Config):
    host: str = Field(default="localhost", hint=FieldHint.feature)
    port: int = Field(default=23456, hint=FieldHint.feature)
    external_world_size: int = Field(default=1, desc="Number of external (inference) processes in the broadcast group.", hint=FieldHint.feature)
    backend: DistributedBackend = Field(default=DistributedBackend.nccl, hint=FieldHint.feature)


@config_class(dynamic_type={TrainerCallbackConfig: "streaming"})
class StreamingTrainerCallbackConfig(TrainerCallbackConfig, RedisConfig):
    """After every update, announce the step on a Redis stream and broadcast the exported weights to inference workers."""

    broadcast: WeightsBroadcastConfig = Field(desc="Weights broadcast group.", hint=FieldHint.core)
    export: CheckpointStateSaveConfigBase = Field(desc="Format the weights are exported in.", hint=FieldHint.core)

    def get_callback(self, model):
        from fast_llm_b200.engine.training.streaming import StreamingTrainerCallback

        return StreamingTrainerCallback(self, model)


@config_class(registry=True, dynamic_type={RunnableConfig: "train"})
class TrainerConfig(PretrainedFastLLMModelConfig, ExperimentConfig):
    _abstract = True
    training: TrainingConfig = Field(desc="Training loop.", hint=FieldHint.core)
    schedule: ScheduleConfig = Field(desc="Micro-batch schedule.", hint=FieldHint.core)
    data: DataConfig = Field(desc="Data.", hint=FieldHint.core)
    profiling: ProfilingConfig = Field(desc="Profiler.", hint=FieldHint.logging)
    optimizer: OptimizerConfig = Field(desc="Optimizer.", hint=FieldHint.core)
    reference_models: dict[str, PretrainedFastLLMModelConfig] = Field(default_factory=dict, desc="Frozen models used by distillation / preference losses.", hint=FieldHint.feature)
    callbacks: dict[str, TrainerCallbackConfig] = Field(default_factory=dict, desc="Callbacks run around training events.", hint=FieldHint.feature)

    def _validate(self):
        self.training.validate()
        self.training.export.setup(type(self.model))
        for reference in self.reference_models.values():
            reference.validate()
        super()._validate()
        if self.run.experiment_dir is None:
            assert not self.training.checkpoint.enabled(), "checkpointing needs run.experiment_dir"

    def _setup(self):
        super()._setup()

    def _get_runnable(self):
        from fast_llm_b200.parallel.distributed import Distributed

        distributed = Distributed(self.model.distributed)
        run = self.get_run(distributed)
        trainer = self.get_trainer_class()(config=self)

        def runnable():
            with run:
                trainer.setup(distributed, run)
                trainer.run()
            distributed.shutdown()

        return runnable

    @classmethod
    def get_trainer_class(cls):
        raise NotImplementedError
