"""Registry bases shared by decoder sub-layers: block, mixer and MLP configs.

Parity: `fast_llm/layers/block/config.py:63-120`, `fast_llm/layers/decoder/config.py:60-131`.
"""

from fast_llm_b200.config import Field, FieldHint, config_class
from fast_llm_b200.engine.parameter import ModuleConfig
from fast_llm_b200.layers.normalization import NormalizationConfig


@config_class(registry=True)
class BlockConfig(ModuleConfig):
    """Base of everything that can be a layer of a model."""

    _abstract = True
    lr_scale: float | None = Field(default=None, desc="Learning-rate multiplier of every parameter below.", hint=FieldHint.feature)

    @classmethod
    def _get_default_subclass(cls):
        if cls is BlockConfig:
            from fast_llm_b200.layers.block import DecoderBlockConfig

            return DecoderBlockConfig
        return cls


@config_class()
class BlockWithBiasConfig(BlockConfig):
    """A sub-layer that may hand its output bias to the caller for fusion with the residual add."""

    def get_layer(self, distributed_config, hidden_dim, *, lr_scale=None, peft=None, return_bias: bool = False, **kwargs):
        return self.layer_class(self, distributed_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft, return_bias=return_bias, **kwargs)


@config_class(registry=True)
class MLPBaseConfig(BlockWithBiasConfig):
    _abstract = True
    pre_norm: NormalizationConfig | None = Field(default=None, desc="Extra normalization before the MLP.", hint=FieldHint.architecture)
    post_norm: NormalizationConfig | None = Field(default=None, desc="Extra normalization after the MLP.", hint=FieldHint.architecture)

    @classmethod
    def _get_default_subclass(cls):
        if cls is MLPBaseConfig:
            from fast_llm_b200.layers.mlp import MLPConfig

            return MLPConfig
        return cls


@config_class(registry=True)
class MixerConfig(BlockWithBiasConfig):
    """Base of token mixers (attention, SSMs, stochastic mixer)."""

    @classmethod
    def _get_default_subclass(cls):
        if cls is MixerConfig:
            from fast_llm_b200.layers.attention import AttentionConfig

            return AttentionConfig
        return cls
