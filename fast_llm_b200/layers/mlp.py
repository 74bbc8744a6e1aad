"""Dense MLP (gated or not).  MoE variants live in `fast_llm_b200.layers.moe`.

Parameters: `layer_1.weight [(2 if gated)*ffn, hidden]` (gate rows then up rows; each half split separately under TP),
`layer_2.weight [ffn, hidden]` (transposed).  Parity: `fast_llm/layers/decoder/mlp/config.py:35-90`, `mlp.py:19-155`.
"""

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import LayerBase
from fast_llm_b200.engine.initialization import init_normal_
from fast_llm_b200.engine.parameter import combine_lr_scales
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.layers.linear import AffineLinearConfig
from fast_llm_b200.layers.mixer import MLPBaseConfig
from fast_llm_b200.ops.activation import ActivationType
from fast_llm_b200.ops.mlp import MLPRecomputeLevel, mlp
from fast_llm_b200.parallel.topology import DistributedDimNames
from fast_llm_b200.tensor import ConcatenatedTensorDim, TensorDim
from fast_llm_b200.utils import Assert


@config_class(dynamic_type={MLPBaseConfig: "mlp"})
class MLPConfig(MLPBaseConfig):
    _abstract = False
    layer_1: AffineLinearConfig = Field(desc="First (up / gate+up) projection.", hint=FieldHint.architecture)
    layer_2: AffineLinearConfig = Field(desc="Second (down) projection.", hint=FieldHint.architecture)
    intermediate_size: int = Field(default=4096, desc="Hidden size of the MLP.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    add_linear_biases: bool = Field(default=True, desc="Default for the biases of both projections.", hint=FieldHint.architecture)
    gated: bool = Field(default=False, desc="Gated (GLU-style) MLP.", hint=FieldHint.architecture)
    activation: ActivationType = Field(default=None, desc="Activation (default: silu if gated else gelu).", hint=FieldHint.architecture)
    recompute_level: MLPRecomputeLevel = Field(default=MLPRecomputeLevel.none, desc="What to recompute in backward instead of storing.", hint=FieldHint.performance)

    def _validate(self):
        if self.activation is None:
            self.activation = ActivationType.silu if self.gated else ActivationType.gelu
        super()._validate()

    @property
    def layer_class(self):
        return MLP


class MLP(LayerBase):
    def __init__(self, config: MLPConfig, distributed_config, *, hidden_dim: TensorDim, lr_scale=None, peft=None,
                 return_bias: bool = False, experts_dim: TensorDim | None = None, output_dim: TensorDim | None = None):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self._hidden_dim = hidden_dim
        self._output_dim = output_dim or hidden_dim  # an adapter maps to another width
        self._sequence_parallel = distributed_config.sequence_tensor_parallel
        tp_dim = distributed_config.get_distributed_dim(DistributedDimNames.tensor)
        ffn_dim = TensorDim("intermediate", config.intermediate_size, tp_dim)
        l1_dim = ConcatenatedTensorDim("gate_and_up", (ffn_dim, ffn_dim)) if config.gated else ffn_dim
        self._ffn_dim = ffn_dim
        self._build(config, distributed_config, hidden_dim, l1_dim, ffn_dim, peft)
        # optional norms of this branch alone (a hybrid MoE gives its dense and routed branches their own)
        if config.pre_norm is not None:
            self.pre_norm = config.pre_norm.get_layer(hidden_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        if config.post_norm is not None:
            self.post_norm = config.post_norm.get_layer(self._output_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)

    def _build(self, config, distributed_config, hidden_dim, l1_dim, ffn_dim, peft):
        common = dict(default_add_bias=config.add_linear_biases, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        self.layer_1 = config.layer_1.get_layer(hidden_dim, l1_dim, default_weight_initialization=init_normal_(0.0, hidden_dim.global_size**-0.5),
                                                sequence_parallel=self._sequence_parallel, **common)
        self.layer_2 = config.layer_2.get_layer(ffn_dim, getattr(self, "_output_dim", hidden_dim), default_weight_initialization=init_normal_(0.0, hidden_dim.global_size**-0.5),
                                                sequence_parallel=self._sequence_parallel, transposed_weight=True, **common)

    def forward(self, x: torch.Tensor, kwargs: dict | None = None, losses=None, metrics=None) -> torch.Tensor:
        c = self._config
        if c.pre_norm is not None:
            x = self.pre_norm(x)
        out = self._forward(x, kwargs, losses, metrics)
        if c.post_norm is not None:
            out = self.post_norm(out)
        return out

    def _forward(self, x: torch.Tensor, kwargs: dict | None = None, losses=None, metrics=None) -> torch.Tensor:
        c = self._config
        l1, l2 = self.layer_1, self.layer_2
        if l1._forward_hook is not None or l2._forward_hook is not None:
            # PEFT-wrapped projections: fall back to the composable path
            from fast_llm_b200.ops.activation import mlp_activation

            return l2(mlp_activation(l1(x), c.gated, c.activation))
        # Recomputing the activation output is free here (the backward kernel emits it while computing the gradient).
        recompute = c.recompute_level if c.recompute_level != MLPRecomputeLevel.none else MLPRecomputeLevel.activation
        return mlp(x, l1.weight, l1.bias if l1._has_bias else None, l2.weight, l2.bias if l2._has_bias else None,
                   gated=c.gated, activation=c.activation, group=l1._group, sequence_parallel=self._sequence_parallel,
                   recompute_level=recompute)

    def get_compute_usage(self, input_meta, kwargs, config=None) -> int:
        c = self._config
        tokens = kwargs[BlockKwargs.num_tokens]
        return 2 * tokens * self._hidden_dim.global_size * c.intermediate_size * (3 if c.gated else 2)

    def get_recompute_usage(self, kwargs) -> int:
        c = self._config
        if not c.recompute_level.recompute_layer_1:
            return 0
        return 2 * kwargs[BlockKwargs.num_tokens] * self._hidden_dim.global_size * c.intermediate_size * (2 if c.gated else 1)
