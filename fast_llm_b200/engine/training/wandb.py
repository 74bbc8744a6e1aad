"""Weights & Biases wrapper: active only on the main rank and only when an entity is configured.

Parity: `fast_llm/engine/training/wandb.py` (init with the experiment config, `log_metrics`, `alert`, status alerts on
start / finish / crash).
"""

import logging

logger = logging.getLogger(__name__)


class Wandb:
    def __init__(self, config, run, experiment_config, module=None):
        self._config, self._run = config, run
        self._is_wandb_main_rank = run.is_main_rank and config.entity_name is not None
        self._wandb = None
        if self._is_wandb_main_rank:
            if module is None:
                import wandb as module
            self._wandb = module
            settings = {}
            try:
                settings = {"settings": module.Settings(init_timeout=300)}
            except Exception:
                pass
            directory = getattr(run, "experiment_directory", None)
            experiment_name = getattr(getattr(run, "_config", None), "experiment_name", None) or (directory.name if directory else "experiment")
            self._wandb.init(name=experiment_name, project=config.project_name, group=config.group_name, entity=config.entity_name,
                             config=experiment_config.to_dict() if hasattr(experiment_config, "to_dict") else experiment_config,
                             dir=str(run.experiment_directory) if getattr(run, "experiment_directory", None) else None, **settings)

    def log_metrics(self, completed_steps: int, metrics: dict, commit: bool = True) -> None:
        if self._wandb is not None:
            self._wandb.log(_flatten(metrics), step=completed_steps, commit=commit)

    def alert(self, title: str, text: str, level: str = "INFO", wait: float = 0.001) -> None:
        if self._wandb is not None:
            self._wandb.alert(title=f"[{self._config.project_name}/{self._config.group_name}] {title}", text=text, level=level, wait_duration=wait)

    def __enter__(self):
        if self._config.alert.status_updates:
            self.alert("Run started!", "", "ERROR")  # the highest level guarantees delivery with default filters
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        if self._config.alert.status_updates:
            if exc_type is None:
                self.alert("Run finished", "", "ERROR")
            else:
                self.alert("Run crashed!", f"{exc_type.__name__}: {exc_val}", "ERROR")
        if self._wandb is not None and hasattr(self._wandb, "finish"):
            self._wandb.finish(exit_code=0 if exc_type is None else 1)
        return False


def _flatten(metrics: dict, prefix: str = "") -> dict:
    out = {}
    for key, value in metrics.items():
        name = f"{prefix}{key}"
        if isinstance(value, dict):
            out.update(_flatten(value, name + "/"))
        else:
            out[name] = value
    return out
