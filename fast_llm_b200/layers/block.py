"""Decoder block and block sequences.

`DecoderBlock`: pre-norm -> mixer -> residual -> pre-norm -> MLP -> residual, with optional post-norms, dropout,
learnable output scale and activation distillation (`fast_llm/layers/decoder/block.py:66-267`).  The residual add after
the mixer is fused with the second pre-norm in one kernel.  `FixedBlockSequence` repeats one block config;
`PatternBlockSequence` interleaves named block configs (hybrid models) (`fast_llm/layers/block/sequence.py:17-120`).
"""

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import Layer, LayerBase, LossDef
from fast_llm_b200.engine.initialization import init_ones_
from fast_llm_b200.engine.parameter import OptionalParameterConfig, combine_lr_scales
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.layers.mixer import BlockConfig, MixerConfig, MLPBaseConfig
from fast_llm_b200.layers.normalization import NormalizationConfig
from fast_llm_b200.tensor import TensorDim, scalar_dim
from fast_llm_b200.utils import Assert


@config_class(dynamic_type={BlockConfig: "decoder"})
class DecoderBlockConfig(BlockConfig):
    _abstract = False
    mixer: MixerConfig = Field(desc="Token mixer (attention, SSM, ...).", hint=FieldHint.architecture)
    mlp: MLPBaseConfig = Field(desc="Channel mixer.", hint=FieldHint.architecture)
    normalization: NormalizationConfig = Field(desc="Default for both pre-norms.", hint=FieldHint.architecture)
    pre_mixer_normalization: NormalizationConfig | None = Field(default=None, hint=FieldHint.architecture)
    pre_mlp_normalization: NormalizationConfig | None = Field(default=None, hint=FieldHint.architecture)
    post_mixer_normalization: NormalizationConfig | None = Field(default=None, hint=FieldHint.architecture)
    post_mlp_normalization: NormalizationConfig | None = Field(default=None, hint=FieldHint.architecture)
    output_scale: OptionalParameterConfig = Field(desc="Learnable scalar applied to the block output.", hint=FieldHint.architecture)
    dropout: float = Field(default=0.0, desc="Dropout after mixer and MLP.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))
    distillation_model: str | None = Field(default=None, desc="Reference model whose activations this block imitates.", hint=FieldHint.feature)
    distillation_loss_weight: float = Field(default=1.0, hint=FieldHint.feature, valid=check_field(Assert.geq, 0))

    def get_layer(self, distributed_config, hidden_dim: TensorDim, *, lr_scale=None, peft=None, return_input: bool = False):
        return DecoderBlock(self, distributed_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft, return_input=return_input)

    def get_layers(self, distributed_config, hidden_dim, *, lr_scale=None, peft=None):
        return [self.get_layer(distributed_config, hidden_dim, lr_scale=lr_scale, peft=peft)]


class DecoderBlock(Layer):
    def __init__(self, config: DecoderBlockConfig, distributed_config, *, hidden_dim: TensorDim, lr_scale=None, peft=None,
                 return_input: bool = False):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self._hidden_dim = hidden_dim
        self._return_input = return_input
        norm = lambda c: (c or config.normalization).get_layer(hidden_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        self.norm_1 = norm(config.pre_mixer_normalization)
        self.norm_2 = norm(config.pre_mlp_normalization)
        self.mixer = config.mixer.get_layer(distributed_config, hidden_dim, lr_scale=self._lr_scale, peft=peft)
        self.mlp = config.mlp.get_layer(distributed_config, hidden_dim, lr_scale=self._lr_scale, peft=peft)
        if config.post_mixer_normalization is not None:
            self.post_mixer_norm = config.post_mixer_normalization.get_layer(hidden_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        if config.post_mlp_normalization is not None:
            self.post_mlp_norm = config.post_mlp_normalization.get_layer(hidden_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        scale = config.output_scale.get_parameter((scalar_dim,), default_initialization=init_ones_, lr_scale=self._lr_scale, weight_decay=False, default_enabled=False)
        if scale is not None:
            self.output_scale = scale
        self._has_output_scale = scale is not None

    def _dropout(self, x, kwargs):
        p = self._config.dropout
        if p > 0 and kwargs.get("training", True):
            from fast_llm_b200.parallel.collectives import set_generator

            gen = self._distributed.tp_generator if self._distributed_config.sequence_tensor_parallel else self._distributed.pp_generator
            with set_generator(gen):
                return torch.dropout(x, p, True)
        return x

    def forward(self, input_: torch.Tensor, kwargs: dict, losses: dict | None = None, metrics: dict | None = None) -> torch.Tensor:
        if self._return_input and input_.dim() == 3 and input_.shape[0] == 2:
            input_ = input_[1]  # stacked (input, output) from the previous block of a multi-token-prediction chain
        c = self._config
        hidden = self.norm_1(input_)
        mixed = self.mixer.forward(hidden, kwargs, losses, metrics)
        if c.distillation_model is not None and losses is not None:
            mixed = self._activation_distillation(mixed, kwargs, losses)
        if c.post_mixer_normalization is not None:
            mixed = self.post_mixer_norm(mixed)
        mixed = self._dropout(mixed, kwargs)
        residual, hidden = self.norm_2.forward_add(input_, mixed)
        out = self.mlp.forward(hidden, kwargs, losses, metrics)
        if c.post_mlp_normalization is not None:
            out = self.post_mlp_norm(out)
        out = self._dropout(out, kwargs)
        if self._has_output_scale:
            out = out * self.output_scale
        out = residual + out
        hs = kwargs.get(BlockKwargs.output_hidden_states)
        if hs and self.module_name in hs:
            kwargs[BlockKwargs.hidden_states][self.module_name] = out.detach()
        if self._return_input:
            return torch.stack((input_, out), dim=0)
        return out

    def _activation_distillation(self, mixed, kwargs, losses):
        teacher = kwargs.get(f"{self._config.distillation_model}_hidden_states", {}).get(self.module_name + ".mixer")
        if teacher is None:
            return mixed
        loss = (mixed.float() - teacher.float()).pow(2).sum(-1).sqrt().mean() * self._config.distillation_loss_weight
        from fast_llm_b200.ops.aux_loss import attach_auxiliary_loss

        mixed_with_loss = attach_auxiliary_loss(mixed, loss, kwargs.get(BlockKwargs.grad_output, 1.0))
        losses.setdefault("activation_distillation_loss", []).append(loss.detach())
        return mixed_with_loss

    def get_loss_definitions(self, count: int = 1):
        out = super().get_loss_definitions(count)
        if self._config.distillation_model is not None:
            out.append(LossDef("activation_distillation_loss", "activation distillation loss", count))
        return out


@config_class(registry=True)
class BlockSequenceConfig(BlockConfig):
    @classmethod
    def _get_default_subclass(cls):
        return FixedBlockSequenceConfig if cls is BlockSequenceConfig else cls

    def get_layers(self, distributed_config, hidden_dim, *, lr_scale=None, peft=None, return_last_layer_input: bool = False) -> list[Layer]:
        raise NotImplementedError

    def block_configs(self) -> list[BlockConfig]:
        raise NotImplementedError


@config_class(dynamic_type={BlockSequenceConfig: "fixed"})
class FixedBlockSequenceConfig(BlockSequenceConfig):
    _abstract = False
    block: BlockConfig = Field(desc="Config of every block.", hint=FieldHint.architecture)
    num_blocks: int = Field(default=12, desc="Number of blocks.", hint=FieldHint.architecture, valid=check_field(Assert.geq, 0))

    def block_configs(self):
        return [self.block] * self.num_blocks

    def get_layers(self, distributed_config, hidden_dim, *, lr_scale=None, peft=None, return_last_layer_input: bool = False):
        lr = combine_lr_scales(lr_scale, self.lr_scale)
        return [
            self.block.get_layer(distributed_config, hidden_dim, lr_scale=lr, peft=peft,
                                 return_input=return_last_layer_input and i == self.num_blocks - 1)
            for i in range(self.num_blocks)
        ]


@config_class(dynamic_type={BlockSequenceConfig: "pattern"})
class PatternBlockSequenceConfig(BlockSequenceConfig):
    _abstract = False
    blocks: dict[str, BlockConfig] = Field(default_factory=dict, desc="Named block configs.", hint=FieldHint.architecture)
    pattern: list[str] = Field(default=None, desc="Order of block names, repeated to fill num_blocks.", hint=FieldHint.architecture)
    num_blocks: int = Field(default=12, desc="Number of blocks.", hint=FieldHint.architecture, valid=check_field(Assert.geq, 0))

    def _validate(self):
        if not self.blocks:
            raise ValueError("No block configuration provided")
        if self.pattern is None:
            self.pattern = list(self.blocks)
        super()._validate()
        for name in self.pattern:
            Assert.incl(name, self.blocks)

    @property
    def expanded_pattern(self) -> list[str]:
        return [self.pattern[i % len(self.pattern)] for i in range(self.num_blocks)]

    def block_configs(self):
        return [self.blocks[n] for n in self.expanded_pattern]

    def get_layers(self, distributed_config, hidden_dim, *, lr_scale=None, peft=None, return_last_layer_input: bool = False):
        lr = combine_lr_scales(lr_scale, self.lr_scale)
        names = self.expanded_pattern
        return [
            self.blocks[name].get_layer(distributed_config, hidden_dim, lr_scale=lr, peft=peft,
                                        return_input=return_last_layer_input and i == len(names) - 1)
            for i, name in enumerate(names)
        ]
