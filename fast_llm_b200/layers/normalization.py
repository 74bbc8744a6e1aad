"""Normalization configs and layers: none, layer_norm, rms_norm, fixed_rms_norm (no weight), gated_rms_norm.

Parity: `fast_llm/layers/common/normalization/config.py:65-176`, `normalization.py:171-340`.  All variants run on the one
fused kernel family of `fast_llm_b200.ops.normalization`; `implementation` is accepted for schema compatibility.
"""

import enum

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import LayerBase
from fast_llm_b200.engine.initialization import init_ones_, init_zeros_
from fast_llm_b200.engine.parameter import ModuleConfig, ParameterConfig, combine_lr_scales
from fast_llm_b200.ops.activation import ActivationType, activation_reference
from fast_llm_b200.ops.normalization import add_norm, norm
from fast_llm_b200.tensor import TensorDim
from fast_llm_b200.utils import Assert


class NormalizationImplementation(str, enum.Enum):
    auto = "auto"
    torch = "torch"
    fused = "fused"
    fast = "fast"
    triton = "triton"


@config_class(registry=True)
class NormalizationConfig(ModuleConfig):
    lr_scale: float | None = Field(default=None, desc="Learning-rate multiplier of the layer.", hint=FieldHint.feature)

    @classmethod
    def _get_default_subclass(cls):
        return LayerNormalizationConfig if cls is NormalizationConfig else cls

    def get_layer(self, hidden_dim: TensorDim, *, lr_scale=None, peft=None, distributed_config=None) -> "Normalization":
        raise NotImplementedError


@config_class(dynamic_type={NormalizationConfig: "none"})
class NoNormalizationConfig(NormalizationConfig):
    _abstract = False

    def get_layer(self, hidden_dim, *, lr_scale=None, peft=None, distributed_config=None):
        return NoNormalization(self, hidden_dim, distributed_config=distributed_config)


@config_class()
class LayerNormalizationBaseConfig(NormalizationConfig):
    weight: ParameterConfig = Field(desc="Scale parameter.", hint=FieldHint.architecture)
    epsilon: float = Field(default=1e-5, desc="Regularizer for the division.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    zero_centered: bool = Field(default=False, desc="Store weight - 1 so weight decay pulls the scale towards 1.", hint=FieldHint.architecture)
    implementation: NormalizationImplementation = Field(default=NormalizationImplementation.auto, desc="Kept for schema compatibility; one fused kernel serves all.", hint=FieldHint.performance)


@config_class(dynamic_type={NormalizationConfig: "layer_norm"})
class LayerNormalizationConfig(LayerNormalizationBaseConfig):
    _abstract = False
    bias: ParameterConfig = Field(desc="Shift parameter.", hint=FieldHint.architecture)

    def get_layer(self, hidden_dim, *, lr_scale=None, peft=None, distributed_config=None):
        return LayerNormalization(self, hidden_dim, lr_scale=lr_scale, peft=peft, distributed_config=distributed_config)


@config_class(dynamic_type={NormalizationConfig: "rms_norm"})
class RMSNormalizationConfig(LayerNormalizationBaseConfig):
    _abstract = False

    def get_layer(self, hidden_dim, *, lr_scale=None, peft=None, distributed_config=None):
        return RMSNormalization(self, hidden_dim, lr_scale=lr_scale, peft=peft, distributed_config=distributed_config)


@config_class(dynamic_type={NormalizationConfig: "fixed_rms_norm"})
class FixedRMSNormConfig(NormalizationConfig):
    _abstract = False
    epsilon: float = Field(default=1e-5, desc="Regularizer for the division.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))

    def get_layer(self, hidden_dim, *, lr_scale=None, peft=None, distributed_config=None):
        return FixedRMSNormalization(self, hidden_dim, distributed_config=distributed_config)


@config_class(dynamic_type={NormalizationConfig: "gated_rms_norm"})
class GatedRMSNormalizationConfig(RMSNormalizationConfig):
    _abstract = False
    activation: ActivationType = Field(default=ActivationType.silu, desc="Activation applied to the gate.", hint=FieldHint.core)

    def get_layer(self, hidden_dim, *, lr_scale=None, peft=None, distributed_config=None):
        return GatedRMSNormalization(self, hidden_dim, lr_scale=lr_scale, peft=peft, distributed_config=distributed_config)


class Normalization(LayerBase):
    is_rms = False
    has_weight = False

    def __init__(self, config, hidden_dim: TensorDim, *, lr_scale=None, peft=None, distributed_config=None):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self._hidden_dim = hidden_dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_add(self, x: torch.Tensor, delta: torch.Tensor):
        """(x + delta, norm(x + delta))"""
        res = x + delta
        return res, self.forward(res)

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)


class NoNormalization(Normalization):
    def forward(self, x):
        return x


class LayerNormalization(Normalization):
    has_weight = True

    def __init__(self, config, hidden_dim, *, lr_scale=None, peft=None, distributed_config=None):
        super().__init__(config, hidden_dim, lr_scale=lr_scale, peft=peft, distributed_config=distributed_config)
        self.weight = config.weight.get_parameter((hidden_dim,), default_initialization=init_zeros_ if config.zero_centered else init_ones_,
                                                  lr_scale=self._lr_scale, weight_decay=False, peft=peft)
        self.bias = config.bias.get_parameter((hidden_dim,), default_initialization=init_zeros_, lr_scale=self._lr_scale,
                                              weight_decay=False, peft=peft)

    def forward(self, x):
        return norm(x, self.weight, self.bias, self._config.epsilon, self._config.zero_centered, True)

    def forward_add(self, x, delta):
        return add_norm(x, delta, self.weight, self.bias, self._config.epsilon, self._config.zero_centered, True)


class RMSNormalization(Normalization):
    is_rms = True
    has_weight = True

    def __init__(self, config, hidden_dim, *, lr_scale=None, peft=None, distributed_config=None):
        super().__init__(config, hidden_dim, lr_scale=lr_scale, peft=peft, distributed_config=distributed_config)
        self.weight = config.weight.get_parameter((hidden_dim,), default_initialization=init_zeros_ if config.zero_centered else init_ones_,
                                                  lr_scale=self._lr_scale, weight_decay=False, peft=peft)

    def forward(self, x):
        return norm(x, self.weight, None, self._config.epsilon, self._config.zero_centered, False)

    def forward_add(self, x, delta):
        return add_norm(x, delta, self.weight, None, self._config.epsilon, self._config.zero_centered, False)


class FixedRMSNormalization(Normalization):
    is_rms = True

    def forward(self, x):
        return norm(x, None, None, self._config.epsilon, False, False)

    def forward_add(self, x, delta):
        return add_norm(x, delta, None, None, self._config.epsilon, False, False)


class GatedRMSNormalization(RMSNormalization):
    """rms_norm(x) * weight * act(gate)"""

    def forward(self, x, gate=None):
        y = super().forward(x)
        if gate is None:
            return y
        return (y.float() * activation_reference(gate.float(), self._config.activation)).to(x.dtype)
