"""Linear layer configs and modules (plain / column-parallel / row-parallel) and the causal depthwise convolution.

Parity: `fast_llm/layers/common/linear/config.py:48-237`, `linear.py:67-168`, `convolution.py:15-68`.
"""

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import LayerBase
from fast_llm_b200.engine.initialization import Initializer, init_uniform_centered_, init_zeros_
from fast_llm_b200.engine.parameter import ModuleConfig, OptionalParameterConfig, ParameterConfig, combine_lr_scales
from fast_llm_b200.ops.activation import ActivationType, activation_reference
from fast_llm_b200.ops.linear import linear
from fast_llm_b200.tensor import ParameterMeta, TensorDim, scalar_dim
from fast_llm_b200.utils import Assert


@config_class()
class LinearBaseConfig(ModuleConfig):
    weight: ParameterConfig = Field(desc="Weight parameter.", hint=FieldHint.architecture)
    lr_scale: float | None = Field(default=None, desc="Learning-rate multiplier of the layer.", hint=FieldHint.feature)


@config_class()
class AffineLinearBaseConfig(LinearBaseConfig):
    bias: OptionalParameterConfig = Field(desc="Bias parameter (enabled by the owning layer unless overridden).", hint=FieldHint.architecture)


@config_class()
class LinearConfig(LinearBaseConfig):
    _abstract = False
    apply_peft: bool | None = Field(default=None, desc="Wrap with the model's PEFT method (default decided by the owning layer).", hint=FieldHint.feature)

    def get_layer(self, in_dim: TensorDim, out_dim: TensorDim, *, default_weight_initialization: Initializer,
                  default_bias_initialization: Initializer = init_zeros_, default_add_bias: bool = False,
                  default_apply_peft: bool = False, sequence_parallel: bool = False, transposed_weight: bool = False,
                  lr_scale=None, peft=None, distributed_config=None) -> "LinearBase":
        lr_scale = combine_lr_scales(lr_scale, self.lr_scale)
        weight = self.weight.get_parameter(
            (in_dim, out_dim) if transposed_weight else (out_dim, in_dim),
            default_initialization=default_weight_initialization, lr_scale=lr_scale)
        bias_config = getattr(self, "bias", None)
        bias = None
        if bias_config is not None:
            bias = bias_config.get_parameter((out_dim,), default_initialization=default_bias_initialization,
                                             lr_scale=lr_scale, weight_decay=False, default_enabled=default_add_bias)
        if in_dim.is_parallel:
            assert not out_dim.is_parallel
            cls = InputParallelLinear
        elif out_dim.is_parallel:
            cls = OutputParallelLinear
        else:
            assert not sequence_parallel or True
            cls = Linear
        layer = cls(weight, bias, in_dim=in_dim, out_dim=out_dim, transposed_weight=transposed_weight,
                    sequence_parallel=sequence_parallel, distributed_config=distributed_config)
        apply_peft = default_apply_peft if self.apply_peft is None else self.apply_peft
        if peft is not None:
            layer = peft.apply_linear(layer, apply_peft)
        return layer


@config_class()
class AffineLinearConfig(AffineLinearBaseConfig, LinearConfig):
    _abstract = False


class LinearBase(LayerBase):
    mode = "none"

    def __init__(self, weight: ParameterMeta, bias: ParameterMeta | None, *, in_dim, out_dim, transposed_weight=False,
                 sequence_parallel=False, distributed_config=None):
        super().__init__(None, distributed_config)
        self.weight = weight
        if bias is not None:
            self.bias = bias
        self._has_bias = bias is not None
        self._in_dim, self._out_dim = in_dim, out_dim
        self._transposed_weight = transposed_weight
        self._sequence_parallel = sequence_parallel
        self._group = None
        self._forward_hook = None  # set by PEFT wrappers

    def setup(self, distributed):
        super().setup(distributed)
        dim = self._in_dim if self._in_dim.is_parallel else self._out_dim
        self._group = dim.parallel_group if dim.is_parallel else None

    @property
    def transposed_weight(self) -> bool:
        return self._transposed_weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = linear(x, self.weight, self.bias if self._has_bias else None, transposed_weight=self._transposed_weight,
                   mode=self.mode, group=self._group, sequence_parallel=self._sequence_parallel and self._group is not None)
        if self._forward_hook is not None:
            y = self._forward_hook(x, y)
        return y

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def get_compute_usage(self, input_meta, kwargs=None, config=None) -> int:
        tokens = input_meta if isinstance(input_meta, int) else input_meta.numel() // self._in_dim.global_size
        return 2 * tokens * self._in_dim.global_size * self._out_dim.global_size


class Linear(LinearBase):
    mode = "none"


class OutputParallelLinear(LinearBase):
    """Column parallel: output features split over the tensor group."""

    mode = "output"


class InputParallelLinear(LinearBase):
    """Row parallel: input features split over the tensor group, output reduced."""

    mode = "input"


@config_class()
class CausalConv1dConfig(AffineLinearBaseConfig):
    _abstract = False
    kernel_size: int = Field(default=4, desc="Convolution kernel size.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    activation: ActivationType | None = Field(default=None, desc="Activation fused after the convolution (default decided by the owner).", hint=FieldHint.architecture)

    def get_layer(self, in_dim: TensorDim, *, default_weight_initialization=None, default_bias_initialization=None,
                  default_add_bias: bool = True, default_activation: ActivationType = ActivationType.identity,
                  lr_scale=None, peft=None, distributed_config=None) -> "CausalConv1d":
        lr_scale = combine_lr_scales(lr_scale, self.lr_scale)
        bound = (in_dim.global_size * self.kernel_size) ** -0.5 if False else self.kernel_size**-0.5
        weight = self.weight.get_parameter(
            (in_dim, scalar_dim, TensorDim("convolution_kernel", self.kernel_size)),
            default_initialization=default_weight_initialization or init_uniform_centered_(bound), lr_scale=lr_scale)
        bias = self.bias.get_parameter((in_dim,), default_initialization=default_bias_initialization or init_uniform_centered_(bound),
                                       lr_scale=lr_scale, weight_decay=False, default_enabled=default_add_bias)
        return CausalConv1d(weight, bias, activation=default_activation if self.activation is None else self.activation,
                            distributed_config=distributed_config)


class CausalConv1d(LayerBase):
    """Depthwise causal 1-d convolution over packed documents ([channels, tokens] layout handled internally)."""

    def __init__(self, weight, bias, *, activation: ActivationType, distributed_config=None):
        super().__init__(None, distributed_config)
        self.weight = weight
        if bias is not None:
            self.bias = bias
        self._has_bias = bias is not None
        self._activation = activation

    def forward(self, x: torch.Tensor, document_index: torch.Tensor | None = None) -> torch.Tensor:
        """x: [tokens, channels]. Tokens of different documents (document_index) do not see each other."""
        from fast_llm_b200.ops.ssm import causal_conv1d

        weight = self.weight  # [channels, 1, k]
        return causal_conv1d(x, weight.reshape(weight.shape[0], weight.shape[-1]), self.bias if self._has_bias else None, document_index, self._activation)

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)
