"""Learning-rate schedules: warm-up then constant / linear / power / cosine decay, or an explicit list of stages
(parity: `fast_llm/engine/optimizer/learning_rate.py:12-136`)."""

import math

from fast_llm_b200.engine.optimizer.config import LearningRateScheduleConfig


class LRStage:
    def __init__(self, style: str, begin_step: int, end_step: int | None, begin_lr: float, end_lr: float, power: float = 1.0):
        self.style, self.begin_step, self.end_step = style, begin_step, end_step
        self.begin_lr, self.end_lr, self.power = begin_lr, end_lr, power

    def __call__(self, step: int) -> float:
        if self.style == "constant" or self.end_step is None or self.end_step <= self.begin_step:
            return self.begin_lr
        x = min(max((step - self.begin_step) / (self.end_step - self.begin_step), 0.0), 1.0)
        if self.style == "linear":
            c = 1 - x
        elif self.style == "power":
            c = (1 - x) ** self.power
        elif self.style == "cosine":
            c = 0.5 * (1 + math.cos(math.pi * x))
        else:
            raise ValueError(f"Unknown decay style {self.style}")
        return self.end_lr + c * (self.begin_lr - self.end_lr)


class LearningRateSchedule:
    def __init__(self, stages: list[LRStage]):
        self._stages = stages
        for a, b in zip(stages[:-1], stages[1:]):
            assert a.end_step == b.begin_step, "schedule stages must be contiguous"

    def __call__(self, step: int) -> float:
        for stage in self._stages:
            if stage.end_step is None or step < stage.end_step:
                return stage(step)
        return self._stages[-1](step)


def create_schedule_from_config(config: LearningRateScheduleConfig) -> LearningRateSchedule:
    stages = []
    if config.schedule is not None:
        for spec in config.schedule.split(";"):
            parts = spec.split(",")
            style, begin, end = parts[0], int(parts[1]), (None if parts[2] in ("", "None") else int(parts[2]))
            begin_lr, end_lr = float(parts[3]), float(parts[4]) if len(parts) > 4 else float(parts[3])
            power = float(parts[5]) if len(parts) > 5 else 1.0
            stages.append(LRStage(style, begin, end, begin_lr, end_lr, power))
        return LearningRateSchedule(stages)
    begin = 0
    if config.warmup_iterations > 0:
        # linear ramp from 0 to base: "linear" interpolates begin_lr -> end_lr as 1-x, so swap the roles
        stages.append(LRStage("linear", 0, config.warmup_iterations, 0.0, config.base))
        stages[-1] = _Warmup(config.warmup_iterations, config.base)
        begin = config.warmup_iterations
    if config.decay_style == "constant" or config.decay_iterations is None:
        stages.append(LRStage("constant", begin, None, config.base, config.base))
    else:
        end = config.decay_iterations
        stages.append(LRStage(config.decay_style, begin, end, config.base, config.minimum, config.decay_power))
        stages.append(LRStage("constant", end, None, config.minimum, config.minimum))
    return LearningRateSchedule(stages)


class _Warmup(LRStage):
    def __init__(self, steps: int, base: float):
        super().__init__("linear", 0, steps, 0.0, base)

    def __call__(self, step: int) -> float:
        return self.end_lr * min(max(step / self.end_step, 0.0), 1.0)
