"""State-space and linear-attention token mixers: Mamba, gated DeltaNet, Kimi delta attention.

Parameter names and shapes follow the reference so checkpoints map one to one; the recurrences are this package's
chunked scans (`fast_llm_b200/ops/ssm.py`) over packed documents.  Heads / channel groups are split over the tensor group
through the dimensions handed to the linear layers (column-parallel in, row-parallel out).
Parity: `fast_llm/layers/ssm/config.py:21-349`, `mamba.py:35-257`, `gdn.py:212-420`, `kda.py:206-437`.
"""

import math

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import LayerBase
from fast_llm_b200.engine.initialization import InitializationConfig, init_normal_, init_ones_, init_uniform_centered_
from fast_llm_b200.engine.parameter import ParameterConfig, combine_lr_scales
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.layers.linear import AffineLinearConfig, CausalConv1dConfig
from fast_llm_b200.layers.mixer import MixerConfig
from fast_llm_b200.layers.normalization import GatedRMSNormalizationConfig
from fast_llm_b200.ops.activation import ActivationType
from fast_llm_b200.ops.linear import linear
from fast_llm_b200.ops.ssm import chunk_delta_rule, gdn_log_decay, kda_gate, selective_scan
from fast_llm_b200.parallel.topology import DistributedDimNames
from fast_llm_b200.tensor import CompositeTensorDim, ConcatenatedTensorDim, TensorDim
from fast_llm_b200.utils import Assert, div


# ----------------------------------------------------------------------------------------------------------------------
# initialisers
# ----------------------------------------------------------------------------------------------------------------------
def init_dt_bias_(min_step_size: float = 0.001, max_step_size: float = 0.1, floor: float = 1e-4):
    """Bias b such that softplus(b) is log-uniform in [min_step_size, max_step_size]."""

    def init_(meta, tensor, generator):
        tensor.uniform_(math.log(min_step_size), math.log(max_step_size), generator=generator).exp_().clamp_min_(floor)
        tensor.add_(torch.log(-torch.expm1(-tensor)))  # inverse softplus

    return init_


def init_a_log_(state_size: int, d_inner: int):
    """A_log[d, n] = log(n + 1): the S4D-real initialisation, identical on every channel."""

    def init_(meta, tensor, generator):
        Assert.eq(tensor.numel() % state_size, 0)
        values = torch.log(torch.arange(1, state_size + 1, dtype=torch.float32, device=tensor.device))
        tensor.copy_(values.expand(tensor.numel() // state_size, state_size).reshape(tensor.shape))

    return init_


def init_log_uniform_(low: float, high: float):
    def init_(meta, tensor, generator):
        tensor.uniform_(low, high, generator=generator).log_()

    return init_


@config_class(dynamic_type={InitializationConfig: "mamba_dt_bias"})
class MambaDTBiasInitializationConfig(InitializationConfig):
    _abstract = False
    min_step_size: float = Field(default=0.001, desc="Smallest discretisation step.", hint=FieldHint.core, valid=check_field(Assert.gt, 0))
    max_step_size: float = Field(default=0.1, desc="Largest discretisation step.", hint=FieldHint.core, valid=check_field(Assert.gt, 0))
    floor: float = Field(default=1e-4, desc="Lower clamp of the sampled step.", hint=FieldHint.core, valid=check_field(Assert.gt, 0))

    def _validate(self):
        super()._validate()
        Assert.geq(self.max_step_size, self.min_step_size)

    def get_initializer(self):
        return init_dt_bias_(self.min_step_size, self.max_step_size, self.floor)


@config_class(dynamic_type={InitializationConfig: "mamba_a"})
class MambaAInitializationConfig(InitializationConfig):
    _abstract = False
    state_size: int = Field(desc="State size (repeated here for the initialiser).", hint=FieldHint.core, valid=check_field(Assert.gt, 0))
    d_inner: int = Field(desc="Inner size (repeated here for the initialiser).", hint=FieldHint.core, valid=check_field(Assert.gt, 0))

    def get_initializer(self):
        return init_a_log_(self.state_size, self.d_inner)


# ----------------------------------------------------------------------------------------------------------------------
# Mamba
# ----------------------------------------------------------------------------------------------------------------------
@config_class(dynamic_type={MixerConfig: "mamba"})
class MambaConfig(MixerConfig):
    _abstract = False
    z_layer: AffineLinearConfig = Field(desc="Fused input projection (z, x, B, C).", hint=FieldHint.architecture)
    x_layer: AffineLinearConfig = Field(desc="Kept for schema compatibility (part of the fused projection).", hint=FieldHint.architecture)
    b_layer: AffineLinearConfig = Field(desc="Kept for schema compatibility.", hint=FieldHint.architecture)
    c_layer: AffineLinearConfig = Field(desc="Kept for schema compatibility.", hint=FieldHint.architecture)
    convolution_layer: CausalConv1dConfig = Field(desc="Depthwise causal convolution on x.", hint=FieldHint.architecture)
    d_weight: ParameterConfig = Field(desc='The D "skip" weight.', hint=FieldHint.architecture)
    output_layer: AffineLinearConfig = Field(desc="Output projection.", hint=FieldHint.architecture)
    dt_layer: AffineLinearConfig = Field(desc="Step-size up-projection (dt_rank -> inner).", hint=FieldHint.architecture)
    a_log_weight: ParameterConfig = Field(desc="log(-A).", hint=FieldHint.architecture)
    dt_input_layer: AffineLinearConfig = Field(desc="Step-size down-projection (hidden -> dt_rank).", hint=FieldHint.architecture)
    state_size: int = Field(default=16, desc="State size per channel.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    d_inner: int = Field(default=2048, desc="Inner (channel) size.", hint=FieldHint.core)
    d_xb: int = Field(default=1024, desc="Size of the x and B projections (grouped heads).", hint=FieldHint.architecture)
    dt_rank: int = Field(default=64, desc="Rank of the step-size projection.", hint=FieldHint.architecture)
    add_linear_biases: bool = Field(default=True, desc="Default for the linear biases.", hint=FieldHint.architecture)
    repeat_kv_before_conv: bool = Field(default=True, desc="Expand x to all heads before (True) or after the convolution.", hint=FieldHint.architecture)
    cross_document_attention: bool = Field(default=True, desc="Let the state run across document boundaries.", hint=FieldHint.feature)

    @property
    def layer_class(self):
        return Mamba


class _SSMBase(LayerBase):
    def __init__(self, config, distributed_config, *, hidden_dim, lr_scale=None, peft=None, return_bias: bool = False):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self._hidden_dim = hidden_dim
        self._tp_dim = distributed_config.get_distributed_dim(DistributedDimNames.tensor)
        self._sequence_parallel = distributed_config.sequence_tensor_parallel
        self._return_bias = return_bias

    def _linear_kwargs(self, distributed_config, peft, add_bias: bool):
        return dict(default_add_bias=add_bias, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)

    @staticmethod
    def _documents(kwargs, enabled: bool = True):
        return (kwargs.get(BlockKwargs.cu_seqlens_q), kwargs.get(BlockKwargs.document_index)) if enabled else (None, None)


class Mamba(_SSMBase):
    def __init__(self, config: MambaConfig, distributed_config, *, hidden_dim, lr_scale=None, peft=None, return_bias=False):
        super().__init__(config, distributed_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft, return_bias=return_bias)
        c = config
        heads = div(c.d_inner, c.state_size)
        head_groups = div(c.d_xb, c.state_size)
        state_dim = TensorDim("state", c.state_size)
        groups_dim = TensorDim("head_groups", head_groups, self._tp_dim)
        group_heads_dim = TensorDim("group_heads", div(heads, head_groups))
        inner_dim = CompositeTensorDim("inner", (groups_dim, group_heads_dim, state_dim))
        xb_dim = CompositeTensorDim("xb", (groups_dim, state_dim))
        dt_rank_dim = TensorDim("dt_rank", c.dt_rank)
        projection_dim = ConcatenatedTensorDim("inner_projection", (inner_dim, xb_dim, xb_dim, inner_dim))
        self._local_groups = groups_dim.size
        self._group_heads = group_heads_dim.size
        self._local_heads = self._local_groups * self._group_heads
        self._local_inner, self._local_xb = inner_dim.size, xb_dim.size
        kw = self._linear_kwargs(distributed_config, peft, c.add_linear_biases)
        hidden = hidden_dim.global_size
        self.convolution = c.convolution_layer.get_layer(inner_dim if c.repeat_kv_before_conv else xb_dim, default_add_bias=c.add_linear_biases,
                                                         default_activation=ActivationType.silu, lr_scale=self._lr_scale, peft=peft,
                                                         distributed_config=distributed_config)
        self.in_proj = c.z_layer.get_layer(hidden_dim, projection_dim, default_weight_initialization=init_normal_(0.0, (2 / hidden) ** 0.5),
                                           sequence_parallel=self._sequence_parallel, **kw)
        self.dt_in_proj = c.dt_input_layer.get_layer(hidden_dim, dt_rank_dim, default_weight_initialization=init_normal_(0.0, (2 / hidden) ** 0.5),
                                                     sequence_parallel=self._sequence_parallel, **kw)
        self.dt_proj = c.dt_layer.get_layer(dt_rank_dim, inner_dim, default_weight_initialization=init_uniform_centered_(c.dt_rank**-0.5),
                                            default_bias_initialization=init_dt_bias_(), **kw)
        self.A_log = c.a_log_weight.get_parameter((inner_dim, state_dim), default_initialization=init_a_log_(c.state_size, c.d_inner),
                                                  weight_decay=False, lr_scale=self._lr_scale, peft=peft)
        self.D = c.d_weight.get_parameter((inner_dim,), default_initialization=init_ones_, weight_decay=False, lr_scale=self._lr_scale, peft=peft)
        self.out_proj = c.output_layer.get_layer(inner_dim, hidden_dim, default_weight_initialization=init_normal_(0.0, (2 / c.d_inner) ** 0.5),
                                                 sequence_parallel=self._sequence_parallel, **kw)

    def forward(self, x: torch.Tensor, kwargs: dict, losses=None, metrics=None) -> torch.Tensor:
        c = self._config
        n = c.state_size
        projected = self.in_proj(x)
        dt_low = self.dt_in_proj(x)
        if self._sequence_parallel and self._tp_dim.size > 1 and dt_low.shape[0] != projected.shape[0]:
            from fast_llm_b200.parallel.ops import gather_op

            dt_low = gather_op(dt_low, self._tp_dim.group, 0)
        # the step bias is applied inside the scan (softplus(dt + bias)), not by the projection
        dt = linear(dt_low, self.dt_proj.weight, None, mode=self.dt_proj.mode, group=self.dt_proj._group)
        z, xs, b, cs = torch.split(projected, [self._local_inner, self._local_xb, self._local_xb, self._local_inner], dim=-1)
        cu, doc_index = self._documents(kwargs, not c.cross_document_attention)
        tokens = xs.shape[0]

        def expand(t):  # [tokens, groups * n] -> [tokens, heads * n]
            return t.reshape(tokens, self._local_groups, 1, n).expand(-1, -1, self._group_heads, -1).reshape(tokens, self._local_inner)

        if c.repeat_kv_before_conv:
            xs = self.convolution(expand(xs), doc_index)
        else:
            xs = expand(self.convolution(xs, doc_index))
        # one state vector B per head group, one C per head; a head's `state_size` channels share them
        y = selective_scan(
            xs, dt, -torch.exp(self.A_log.float()), b.reshape(tokens, self._local_groups, n), cs.reshape(tokens, self._local_heads, n),
            self.D.float(), z, self.dt_proj.bias.float() if getattr(self.dt_proj, "_has_bias", False) else None, cu)
        return self.out_proj(y)

    def get_compute_usage(self, input_meta, kwargs=None, config=None) -> int:
        tokens = input_meta if isinstance(input_meta, int) else input_meta.shape[0]
        c = self._config
        dense = 2 * tokens * self._hidden_dim.global_size * (2 * c.d_inner + 2 * c.d_xb + c.dt_rank) + 2 * tokens * c.dt_rank * c.d_inner
        dense += 2 * tokens * c.d_inner * self._hidden_dim.global_size
        return dense + 9 * tokens * c.d_inner * c.state_size


# ----------------------------------------------------------------------------------------------------------------------
# Gated DeltaNet
# ----------------------------------------------------------------------------------------------------------------------
@config_class(dynamic_type={MixerConfig: "gdn"})
class GatedDeltaNetConfig(MixerConfig):
    _abstract = False
    normalization: GatedRMSNormalizationConfig = Field(desc="Gated RMS norm on the recurrence output.", hint=FieldHint.architecture)
    qkv_projection_layer: AffineLinearConfig = Field(desc="Projection to query, key, value and gate z.", hint=FieldHint.architecture)
    ba_projection_layer: AffineLinearConfig = Field(desc="Projection to beta and the decay pre-activation.", hint=FieldHint.architecture)
    convolution_layer: CausalConv1dConfig = Field(desc="Depthwise convolution over the concatenated q, k, v.", hint=FieldHint.architecture)
    output_layer: AffineLinearConfig = Field(desc="Output projection.", hint=FieldHint.architecture)
    dt_bias_weight: ParameterConfig = Field(desc="Time-step bias.", hint=FieldHint.architecture)
    a_log_weight: ParameterConfig = Field(desc="Log decay rates.", hint=FieldHint.architecture)
    value_heads: int = Field(default=16, desc="Value heads.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    key_heads: int = Field(default=8, desc="Key heads.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    key_head_dim: int = Field(default=64, desc="Key head size.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    value_head_dim: int = Field(default=64, desc="Value head size.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))

    def _validate(self):
        super()._validate()
        Assert.multiple(self.value_heads, self.key_heads)

    @property
    def layer_class(self):
        return GatedDeltaNet


class GatedDeltaNet(_SSMBase):
    """Projection layout `[Q all heads | K all heads | V all heads | Z all heads]` (`gdn.py:212-222`)."""

    def __init__(self, config: GatedDeltaNetConfig, distributed_config, *, hidden_dim, lr_scale=None, peft=None, return_bias=False):
        super().__init__(config, distributed_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft, return_bias=return_bias)
        c = config
        value_heads_dim = TensorDim("gdn_value_heads", c.value_heads, self._tp_dim if c.value_heads > 1 else None)
        key_heads_dim = TensorDim("gdn_key_heads", c.key_heads, self._tp_dim if c.key_heads > 1 else None)
        value_head_dim = TensorDim("gdn_value_head_dim", c.value_head_dim)
        key_head_dim = TensorDim("gdn_key_head_dim", c.key_head_dim)
        self._value_heads, self._key_heads = value_heads_dim.size, key_heads_dim.size
        self._heads_per_key = div(self._value_heads, self._key_heads)
        query_dim = CompositeTensorDim("gdn_query", (key_heads_dim, key_head_dim))
        key_dim = CompositeTensorDim("gdn_key", (key_heads_dim, key_head_dim))
        value_dim = CompositeTensorDim("gdn_value", (value_heads_dim, value_head_dim))
        z_dim = CompositeTensorDim("gdn_z", (value_heads_dim, value_head_dim))
        qkvz_dim = ConcatenatedTensorDim("gdn_qkvz", (query_dim, key_dim, value_dim, z_dim))
        ba_dim = ConcatenatedTensorDim("gdn_ba", (CompositeTensorDim("gdn_beta", (value_heads_dim,)), CompositeTensorDim("gdn_alpha", (value_heads_dim,))))
        qkv_dim = ConcatenatedTensorDim("gdn_qkv", (query_dim, key_dim, value_dim))
        init = init_normal_(0.0, hidden_dim.global_size**-0.5)
        kw = self._linear_kwargs(distributed_config, peft, False)
        self.in_proj_qkvz = c.qkv_projection_layer.get_layer(hidden_dim, qkvz_dim, default_weight_initialization=init, sequence_parallel=self._sequence_parallel, **kw)
        self.in_proj_ba = c.ba_projection_layer.get_layer(hidden_dim, ba_dim, default_weight_initialization=init, sequence_parallel=self._sequence_parallel, **kw)
        self.convolution = c.convolution_layer.get_layer(qkv_dim, default_add_bias=False, default_activation=ActivationType.silu,
                                                         lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        self.out_proj = c.output_layer.get_layer(value_dim, hidden_dim, default_weight_initialization=init, sequence_parallel=self._sequence_parallel, **kw)
        self.dt_bias = c.dt_bias_weight.get_parameter((value_heads_dim,), default_initialization=init_ones_, weight_decay=False, lr_scale=self._lr_scale, peft=peft)
        self.A_log = c.a_log_weight.get_parameter((value_heads_dim,), default_initialization=init_log_uniform_(1e-6, 16.0), weight_decay=False,
                                                  lr_scale=self._lr_scale, peft=peft)
        self.norm = c.normalization.get_layer(value_head_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)

    def forward(self, x: torch.Tensor, kwargs: dict, losses=None, metrics=None) -> torch.Tensor:
        c = self._config
        qkvz = self.in_proj_qkvz(x)
        ba = self.in_proj_ba(x)
        tokens = qkvz.shape[0]
        key_size, value_size = self._key_heads * c.key_head_dim, self._value_heads * c.value_head_dim
        qkv, z = torch.split(qkvz, [2 * key_size + value_size, value_size], dim=-1)
        cu, doc_index = self._documents(kwargs)
        qkv = self.convolution(qkv, doc_index)
        q, k, v = torch.split(qkv, [key_size, key_size, value_size], dim=-1)
        q = q.reshape(tokens, self._key_heads, c.key_head_dim)
        k = k.reshape(tokens, self._key_heads, c.key_head_dim)
        v = v.reshape(tokens, self._value_heads, c.value_head_dim)
        if self._heads_per_key > 1:
            q = q.repeat_interleave(self._heads_per_key, dim=1)
            k = k.repeat_interleave(self._heads_per_key, dim=1)
        beta, alpha = torch.split(ba, [self._value_heads, self._value_heads], dim=-1)
        out = chunk_delta_rule(q, k, v, gdn_log_decay(alpha, self.A_log, self.dt_bias), beta.float().sigmoid(), cu, normalize_qk=True)
        out = self.norm(out.to(x.dtype), z.reshape(tokens, self._value_heads, c.value_head_dim))
        return self.out_proj(out.reshape(tokens, value_size))

    def get_compute_usage(self, input_meta, kwargs=None, config=None) -> int:
        tokens = input_meta if isinstance(input_meta, int) else input_meta.shape[0]
        c = self._config
        width = 2 * c.key_heads * c.key_head_dim + 2 * c.value_heads * c.value_head_dim + 2 * c.value_heads
        dense = 2 * tokens * self._hidden_dim.global_size * (width + c.value_heads * c.value_head_dim)
        return dense + 6 * tokens * c.value_heads * c.key_head_dim * c.value_head_dim


# ----------------------------------------------------------------------------------------------------------------------
# Kimi delta attention
# ----------------------------------------------------------------------------------------------------------------------
@config_class(dynamic_type={MixerConfig: "kda"})
class KimiDeltaAttentionConfig(MixerConfig):
    _abstract = False
    normalization: GatedRMSNormalizationConfig = Field(desc="Gated normalization of the output.", hint=FieldHint.architecture)
    q_projection_layer: AffineLinearConfig = Field(desc="Query projection.", hint=FieldHint.architecture)
    k_projection_layer: AffineLinearConfig = Field(desc="Key projection.", hint=FieldHint.architecture)
    v_projection_layer: AffineLinearConfig = Field(desc="Value projection.", hint=FieldHint.architecture)
    f_a_projection_layer: AffineLinearConfig = Field(desc="Decay gate, low-rank down projection.", hint=FieldHint.architecture)
    f_b_projection_layer: AffineLinearConfig = Field(desc="Decay gate, up projection.", hint=FieldHint.architecture)
    g_a_projection_layer: AffineLinearConfig = Field(desc="Output gate, low-rank down projection.", hint=FieldHint.architecture)
    g_b_projection_layer: AffineLinearConfig = Field(desc="Output gate, up projection.", hint=FieldHint.architecture)
    beta_projection_layer: AffineLinearConfig = Field(desc="Write-strength projection.", hint=FieldHint.architecture)
    output_projection_layer: AffineLinearConfig = Field(desc="Output projection.", hint=FieldHint.architecture)
    convolution_layer: CausalConv1dConfig = Field(desc="Depthwise convolution applied to q, k and v separately.", hint=FieldHint.architecture)
    dt_bias_weight: ParameterConfig = Field(desc="Decay gate bias.", hint=FieldHint.architecture)
    a_log_weight: ParameterConfig = Field(desc="Log decay rates.", hint=FieldHint.architecture)
    heads: int = Field(default=16, desc="Heads.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    head_dim: int = Field(default=64, desc="Head size.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))

    @property
    def layer_class(self):
        return KimiDeltaAttention


class KimiDeltaAttention(_SSMBase):
    def __init__(self, config: KimiDeltaAttentionConfig, distributed_config, *, hidden_dim, lr_scale=None, peft=None, return_bias=False):
        super().__init__(config, distributed_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft, return_bias=return_bias)
        c = config
        heads_dim = TensorDim("kda_heads", c.heads, self._tp_dim if c.heads > 1 else None)
        head_dim = TensorDim("kda_head_dim", c.head_dim)
        projection_dim = CompositeTensorDim("kda_projection", (heads_dim, head_dim))
        self._heads = heads_dim.size
        init = init_normal_(0.0, hidden_dim.global_size**-0.5)
        kw = self._linear_kwargs(distributed_config, peft, False)
        sp = dict(sequence_parallel=self._sequence_parallel)
        self.q_proj = c.q_projection_layer.get_layer(hidden_dim, projection_dim, default_weight_initialization=init, **sp, **kw)
        self.k_proj = c.k_projection_layer.get_layer(hidden_dim, projection_dim, default_weight_initialization=init, **sp, **kw)
        self.v_proj = c.v_projection_layer.get_layer(hidden_dim, projection_dim, default_weight_initialization=init, **sp, **kw)
        conv = dict(default_add_bias=False, default_activation=ActivationType.silu, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        self.q_conv = c.convolution_layer.get_layer(projection_dim, **conv)
        self.k_conv = c.convolution_layer.get_layer(projection_dim, **conv)
        self.v_conv = c.convolution_layer.get_layer(projection_dim, **conv)
        self.f_a_proj = c.f_a_projection_layer.get_layer(hidden_dim, head_dim, default_weight_initialization=init, **sp, **kw)
        self.f_b_proj = c.f_b_projection_layer.get_layer(head_dim, projection_dim, default_weight_initialization=init, **kw)
        self.g_a_proj = c.g_a_projection_layer.get_layer(hidden_dim, head_dim, default_weight_initialization=init, **sp, **kw)
        self.g_b_proj = c.g_b_projection_layer.get_layer(head_dim, projection_dim, default_weight_initialization=init, **kw)
        self.beta_proj = c.beta_projection_layer.get_layer(hidden_dim, heads_dim, default_weight_initialization=init, **sp, **kw)
        self.o_proj = c.output_projection_layer.get_layer(projection_dim, hidden_dim, default_weight_initialization=init, **sp, **kw)
        self.dt_bias = c.dt_bias_weight.get_parameter((projection_dim,), default_initialization=init_ones_, weight_decay=False, lr_scale=self._lr_scale, peft=peft)
        self.A_log = c.a_log_weight.get_parameter((heads_dim,), default_initialization=init_log_uniform_(1.0, 16.0), weight_decay=False,
                                                  lr_scale=self._lr_scale, peft=peft)
        self.norm = c.normalization.get_layer(head_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)

    def _low_rank(self, x, down, up):
        low = down(x)
        if self._sequence_parallel and self._tp_dim.size > 1:
            from fast_llm_b200.parallel.ops import gather_op

            low = gather_op(low, self._tp_dim.group, 0)
        return up(low)

    def forward(self, x: torch.Tensor, kwargs: dict, losses=None, metrics=None) -> torch.Tensor:
        c = self._config
        cu, doc_index = self._documents(kwargs)
        shape = (-1, self._heads, c.head_dim)
        q = self.q_conv(self.q_proj(x), doc_index).reshape(shape)
        k = self.k_conv(self.k_proj(x), doc_index).reshape(shape)
        v = self.v_conv(self.v_proj(x), doc_index).reshape(shape)
        g = kda_gate(self._low_rank(x, self.f_a_proj, self.f_b_proj).reshape(shape), self.A_log, self.dt_bias)
        beta = self.beta_proj(x).float().sigmoid()
        out = chunk_delta_rule(q, k, v, g, beta, cu, normalize_qk=True).to(x.dtype)
        gate = self._low_rank(x, self.g_a_proj, self.g_b_proj).reshape(shape)
        out = self.norm(out, gate)
        return self.o_proj(out.reshape(out.shape[0], self._heads * c.head_dim))

    def get_compute_usage(self, input_meta, kwargs=None, config=None) -> int:
        tokens = input_meta if isinstance(input_meta, int) else input_meta.shape[0]
        c = self._config
        width = c.heads * c.head_dim
        dense = 2 * tokens * self._hidden_dim.global_size * (4 * width + 2 * c.head_dim + c.heads) + 4 * tokens * c.head_dim * width
        return dense + 6 * tokens * c.heads * c.head_dim * c.head_dim
