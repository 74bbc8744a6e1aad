"""Per-parameter configuration: initialisation, learning-rate scale, weight decay, optional parameters.

Parity: `fast_llm/engine/config_utils/parameter.py:14-110`.
"""

import math

from fast_llm_b200.config import Config, Field, FieldHint, config_class
from fast_llm_b200.engine.initialization import InitializationConfig, Initializer
from fast_llm_b200.tensor import ParameterMeta, TensorDim


def combine_lr_scales(*lr_scales: "float | None | tuple[float | None, ...]"):
    """Multiply learning-rate scales; tuples (per-chunk scales) broadcast against scalars. None means 1."""
    tuple_length = None
    for s in lr_scales:
        if isinstance(s, tuple):
            if tuple_length is None:
                tuple_length = len(s)
            else:
                assert len(s) == tuple_length
    if tuple_length is None:
        vals = [s for s in lr_scales if s is not None]
        return math.prod(vals) if vals else None
    out = []
    for i in range(tuple_length):
        vals = [(s[i] if isinstance(s, tuple) else s) for s in lr_scales]
        vals = [v for v in vals if v is not None]
        out.append(math.prod(vals) if vals else None)
    return tuple(out)


@config_class()
class ModuleConfig(Config):
    """Base of every config that describes part of a model."""

    _abstract = True


@config_class()
class ParameterConfig(ModuleConfig):
    _abstract = False
    initialization: InitializationConfig = Field(desc="Initialisation (default: the layer's own).", hint=FieldHint.feature)
    lr_scale: float | None = Field(default=None, desc="Learning-rate multiplier for this parameter.", hint=FieldHint.feature)
    weight_decay: float | bool | None = Field(default=None, desc="Override whether weight decay applies.", hint=FieldHint.feature)

    def get_parameter(self, dims: tuple[TensorDim, ...], *, default_initialization: Initializer, lr_scale=None,
                      weight_decay: bool = True, default_enabled: bool = True, peft=None,
                      allow_sequence_tensor_parallel: bool = True) -> ParameterMeta | None:
        init = default_initialization if self.initialization.is_default else self.initialization.get_initializer()
        wd = weight_decay if self.weight_decay is None else bool(self.weight_decay)
        meta = ParameterMeta(dims, init_method=init, lr_scale=combine_lr_scales(lr_scale, self.lr_scale), weight_decay=wd,
                             allow_sequence_tensor_parallel=allow_sequence_tensor_parallel)
        if peft is not None:
            meta = peft.apply_weight(meta)
        return meta


@config_class()
class OptionalParameterConfig(ParameterConfig):
    enabled: bool | None = Field(default=None, desc="Force the parameter on or off (default: decided by the layer).", hint=FieldHint.feature)

    def get_parameter(self, dims, *, default_initialization, lr_scale=None, weight_decay=True, default_enabled=False,
                      peft=None, allow_sequence_tensor_parallel=True):
        enabled = default_enabled if self.enabled is None else self.enabled
        if not enabled:
            return None
        return super().get_parameter(dims, default_initialization=default_initialization, lr_scale=lr_scale,
                                     weight_decay=weight_decay, peft=peft,
                                     allow_sequence_tensor_parallel=allow_sequence_tensor_parallel)
