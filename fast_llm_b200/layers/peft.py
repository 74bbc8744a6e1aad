"""Parameter-efficient fine-tuning: `none` or LoRA (parity: `fast_llm/layers/common/peft/config.py:14-99`, `lora.py:11-89`).

LoRA wraps a linear layer with two low-rank projections `y += (alpha/rank) * B(A(dropout(x)))`; with `freeze_others`
every other parameter stops requiring gradients.
"""

import torch

from fast_llm_b200.config import Config, Field, FieldHint, config_class
from fast_llm_b200.engine.base_model import LayerBase
from fast_llm_b200.engine.initialization import init_normal_, init_zeros_
from fast_llm_b200.tensor import ParameterMeta, TensorDim


@config_class(registry=True)
class PeftConfig(Config):
    _abstract = True

    @classmethod
    def _get_default_subclass(cls):
        return NoPeftConfig if cls is PeftConfig else cls

    def apply_linear(self, layer, enabled: bool):
        return self.apply_other(layer)

    def apply_other(self, layer):
        for _, meta in layer.named_parameter_metas():
            self.apply_weight(meta)
        return layer

    def apply_weight(self, meta: ParameterMeta) -> ParameterMeta:
        return meta


@config_class(dynamic_type={PeftConfig: "none"})
class NoPeftConfig(PeftConfig):
    _abstract = False

    def apply_linear(self, layer, enabled):
        return layer

    def apply_other(self, layer):
        return layer


@config_class(dynamic_type={PeftConfig: "lora"})
class LoRAConfig(PeftConfig):
    _abstract = False
    rank: int = Field(default=8, desc="Rank of the update.", hint=FieldHint.stability)
    alpha: float = Field(default=8.0, desc="Scale numerator (update is alpha/rank * BA).", hint=FieldHint.stability)
    dropout: float = Field(default=0.0, desc="Dropout on the LoRA input.", hint=FieldHint.stability)
    freeze_others: bool = Field(default=True, desc="Freeze every non-LoRA parameter.")

    def apply_weight(self, meta):
        if self.freeze_others:
            meta.requires_grad = False
        return meta

    def apply_linear(self, layer, enabled: bool):
        if self.freeze_others:
            for _, meta in layer.named_parameter_metas():
                meta.requires_grad = False
        if not enabled:
            return layer
        assert not layer._in_dim.is_parallel and not layer._out_dim.is_parallel, "LoRA on tensor-parallel layers is not supported"
        return LoRALinear(layer, self)


class LoRALinear(LayerBase):
    """A linear layer plus a trainable low-rank update; exposes the wrapped layer's interface."""

    def __init__(self, layer, config: LoRAConfig):
        super().__init__(config, layer._distributed_config)
        self.base = layer
        rank_dim = TensorDim("lora_rank", config.rank)
        self.lora_a_weight = ParameterMeta((rank_dim, layer._in_dim), init_method=init_normal_(0.0, layer._in_dim.global_size**-0.5), weight_decay=True)
        self.lora_b_weight = ParameterMeta((layer._out_dim, rank_dim), init_method=init_zeros_, weight_decay=True)
        self._has_bias = layer._has_bias
        self._in_dim, self._out_dim = layer._in_dim, layer._out_dim
        self._forward_hook = self._hook
        self._group = None

    @property
    def mode(self):
        return self.base.mode

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def _hook(self, x, y):
        return y

    def forward(self, x):
        y = self.base.forward(x)
        h = x
        if self._config.dropout > 0 and torch.is_grad_enabled():
            h = torch.dropout(h, self._config.dropout, True)
        from fast_llm_b200.ops.linear import linear

        update = linear(linear(h, self.lora_a_weight), self.lora_b_weight)
        return y + update * (self._config.alpha / self._config.rank)

    def __call__(self, x):
        return self.forward(x)

    def get_compute_usage(self, input_meta, kwargs=None, config=None):
        return self.base.get_compute_usage(input_meta, kwargs, config)
