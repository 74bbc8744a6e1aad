"""Parameter initialisation: callables `(meta, tensor, generator) -> None` and their config classes.

Parity: `fast_llm/engine/config_utils/initialization.py:24-172` (registry `fill` / `normal` / `uniform`, default =
"use the layer's own default").
"""

import typing

import torch

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class
from fast_llm_b200.utils import Assert


class Initialization:
    def get_initializer(self) -> "Initializer":
        raise NotImplementedError

    @property
    def is_default(self) -> bool:
        return False


Initializer = typing.Callable[[typing.Any, torch.Tensor, torch.Generator], None]


def init_fill_(value: float) -> Initializer:
    def init_(meta, tensor, generator):
        tensor.fill_(value)

    return init_


init_zeros_ = init_fill_(0.0)
init_ones_ = init_fill_(1.0)


def init_normal_(mean: float = 0.0, std: float = 1.0, min_val: float | None = None, max_val: float | None = None) -> Initializer:
    def init_(meta, tensor, generator):
        tensor.normal_(mean, std, generator=generator)
        if min_val is not None or max_val is not None:
            tensor.clamp_(min=min_val, max=max_val)

    return init_


def init_uniform_centered_(scale: float, mean: float = 0.0) -> Initializer:
    def init_(meta, tensor, generator):
        tensor.uniform_(mean - scale, mean + scale, generator=generator)

    return init_


def init_kaiming_(d_in: int) -> Initializer:
    return init_normal_(0.0, d_in**-0.5)


@config_class(registry=True)
class InitializationConfig(Config, Initialization):
    _abstract = True

    @classmethod
    def _get_default_subclass(cls):
        return DefaultInitializationConfig if cls is InitializationConfig else cls


@config_class()
class DefaultInitializationConfig(InitializationConfig):
    """Keep the default initialisation of the layer that owns the parameter."""

    _abstract = False

    @property
    def is_default(self) -> bool:
        return True

    def get_initializer(self):
        raise NotImplementedError("default initialisation is resolved by the owning layer")


@config_class(dynamic_type={InitializationConfig: "fill"})
class FillInitializationConfig(InitializationConfig):
    _abstract = False
    value: float = Field(default=1, desc="Constant value.", hint=FieldHint.optional, valid=check_field(Assert.geq, 0))

    def get_initializer(self):
        return init_fill_(self.value)


@config_class(dynamic_type={InitializationConfig: "normal"})
class NormalInitializationConfig(InitializationConfig):
    _abstract = False
    std: float = Field(default=1, desc="Standard deviation.", hint=FieldHint.optional, valid=check_field(Assert.geq, 0))
    mean: float = Field(default=0, desc="Mean.", hint=FieldHint.optional)
    min: float | None = Field(default=None, desc="Lower clamp.", hint=FieldHint.optional)
    max: float | None = Field(default=None, desc="Upper clamp.", hint=FieldHint.optional)

    def get_initializer(self):
        return init_normal_(self.mean, self.std, self.min, self.max)


@config_class(dynamic_type={InitializationConfig: "uniform"})
class UniformInitializationConfig(InitializationConfig):
    _abstract = False
    scale: float = Field(default=None, desc="Half-width of the interval.", hint=FieldHint.core, valid=check_field(Assert.geq, 0))
    mean: float = Field(default=0.0, desc="Centre of the interval.", hint=FieldHint.optional)

    def get_initializer(self):
        return init_uniform_centered_(self.scale, self.mean)
