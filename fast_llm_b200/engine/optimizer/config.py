"""Optimizer, learning-rate schedule and gradient scaler configuration (parity: `fast_llm/engine/optimizer/config.py`)."""

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class, skip_valid_if_none
from fast_llm_b200.utils import Assert


class LearningRateStageType:
    constant = "constant"
    linear = "linear"
    power = "power"
    cosine = "cosine"


@config_class()
class LearningRateScheduleConfig(Config):
    base: float = Field(default=0.0001, desc="Base learning rate.", hint=FieldHint.core)
    decay_style: str = Field(default="constant", desc="constant, linear, power or cosine.", hint=FieldHint.feature)
    decay_iterations: int | None = Field(default=None, desc="Length of the decay.", hint=FieldHint.feature)
    decay_power: float = Field(default=1.0, desc="Exponent for power decay.", hint=FieldHint.feature)
    warmup_iterations: int = Field(default=0, desc="Linear warm-up length.", hint=FieldHint.feature)
    minimum: float = Field(default=0.0, desc="Learning rate at the end of the decay.", hint=FieldHint.feature)
    schedule: str | None = Field(default=None, desc="Multi-stage schedule: 'style,begin_it,end_it,begin_lr,end_lr[,power];...'.", hint=FieldHint.wip)


@config_class()
class GradientScalerConfig(Config):
    constant: float | None = Field(default=None, desc="Constant loss scale (default: dynamic for fp16, none otherwise).", hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.geq, 0)))
    initial: float = Field(default=2**16, desc="Initial dynamic scale.", hint=FieldHint.feature, valid=check_field(Assert.gt, 0))
    minimum: float = Field(default=1.0, desc="Smallest dynamic scale.", hint=FieldHint.feature, valid=check_field(Assert.gt, 0))
    window: int = Field(default=1000, desc="Clean iterations before the scale doubles.", hint=FieldHint.feature, valid=check_field(Assert.gt, 0))
    hysteresis: int = Field(default=2, desc="Overflowing iterations before the scale halves.", hint=FieldHint.feature, valid=check_field(Assert.gt, 0))


@config_class()
class OptimizerConfig(Config):
    learning_rate: LearningRateScheduleConfig = Field(desc="Learning-rate schedule.", hint=FieldHint.core)
    gradient_scaler: GradientScalerConfig = Field(desc="Loss scaling.", hint=FieldHint.feature)
    weight_decay: float = Field(default=0.01, desc="Decoupled weight decay.", hint=FieldHint.core, valid=check_field(Assert.geq, 0))
    beta_1: float = Field(default=0.9, hint=FieldHint.optional, valid=check_field(Assert.in_range_incl, 0, 1))
    beta_2: float = Field(default=0.999, hint=FieldHint.optional, valid=check_field(Assert.in_range_incl, 0, 1))
    epsilon: float = Field(default=1e-8, hint=FieldHint.optional, valid=check_field(Assert.gt, 0))
    gradient_norm_clipping: float = Field(default=1.0, desc="Clip the global gradient norm to this value.", hint=FieldHint.feature, valid=check_field(Assert.gt, 0))
    default_learning_rate_scale: float = Field(default=1.0, desc="Multiplier for parameters without their own lr_scale.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))

    @property
    def state_names(self) -> tuple[str, ...]:
        return ("exp_avgs", "exp_avgs_sq")
