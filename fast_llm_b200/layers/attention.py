"""Multi-head / grouped-query attention mixer.

Parameters follow the reference layout so checkpoints map one to one: `query.weight [heads*head_size, hidden]`,
`key_value.weight [2*head_groups*head_size, hidden]` (key rows then value rows), `dense.weight [hidden,
heads*head_size]` (`fast_llm/layers/attention/attention.py:104-207`).  When the query and key_value weights are
neighbours in the stage's flat buffer (they are, by the stage's parameter ordering) the two projections run as ONE
GEMM over the joint view, so a sequence-parallel input is gathered once instead of twice; rotary runs in place on the
packed result; attention consumes the packed tensor; backward mirrors this with one packed gradient.
"""

import enum

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class, skip_valid_if_none
from fast_llm_b200.engine.base_model import LayerBase
from fast_llm_b200.engine.initialization import init_normal_, init_zeros_
from fast_llm_b200.engine.parameter import combine_lr_scales
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.layers.linear import AffineLinearConfig
from fast_llm_b200.layers.mixer import MixerConfig
from fast_llm_b200.layers.normalization import NormalizationConfig
from fast_llm_b200.layers.rotary import RotaryConfig
from fast_llm_b200.ops.attention import attention, packed_attention
from fast_llm_b200.ops.linear import linear
from fast_llm_b200.parallel.ops import gather_op, reduce_scatter_op
from fast_llm_b200.parallel.topology import DistributedDimNames
from fast_llm_b200.tensor import CompositeTensorDim, ConcatenatedTensorDim, TensorDim
from fast_llm_b200.utils import Assert, div


class AttentionImplementation(str, enum.Enum):
    auto = "auto"
    flash = "flash"
    sdpa_nested = "sdpa_nested"
    sdpa_dense = "sdpa_dense"
    backup = "backup"


@config_class(dynamic_type={MixerConfig: "attention"})
class AttentionConfig(MixerConfig):
    _abstract = False
    query_layer: AffineLinearConfig = Field(desc="Query projection.", hint=FieldHint.architecture)
    key_layer: AffineLinearConfig = Field(desc="Key projection.", hint=FieldHint.architecture)
    value_layer: AffineLinearConfig = Field(desc="Value projection.", hint=FieldHint.architecture)
    dense_layer: AffineLinearConfig = Field(desc="Output projection.", hint=FieldHint.architecture)
    rotary: RotaryConfig = Field(desc="Rotary embedding.", hint=FieldHint.architecture)
    heads: int = Field(default=8, desc="Number of query heads.", hint=FieldHint.architecture)
    head_groups: int = Field(default=1, desc="Number of key/value heads (1 = MQA, heads = MHA).", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    head_size: int = Field(default=128, desc="Size of one head.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    add_linear_biases: bool = Field(default=True, desc="Default for the biases of the four projections.", hint=FieldHint.architecture)
    causal: bool = Field(default=True, desc="Causal masking.", hint=FieldHint.architecture)
    dropout: float = Field(default=0.0, desc="Attention dropout.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))
    use_flash_attention: bool = Field(default=True, desc="Kept for schema compatibility.", hint=FieldHint.optional)
    window_size: int | None = Field(default=None, desc="Sliding-window size.", hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.geq, 0)))
    softmax_scale_power: float = Field(default=0.5, desc="Scores are scaled by head_size ** -power.", hint=FieldHint.architecture, valid=skip_valid_if_none(check_field(Assert.geq, 0)))
    implementation: AttentionImplementation = Field(default=AttentionImplementation.auto, desc="Kernel choice; the packed varlen path serves all.", hint=FieldHint.feature)
    query_norm: NormalizationConfig | None = Field(default=None, desc="Per-head normalization of queries.", hint=FieldHint.architecture)
    key_norm: NormalizationConfig | None = Field(default=None, desc="Per-head normalization of keys.", hint=FieldHint.architecture)
    value_norm: NormalizationConfig | None = Field(default=None, desc="Per-head normalization of values.", hint=FieldHint.architecture)
    shared_key_value: bool = Field(default=False, desc="Use the key projection as values too.", hint=FieldHint.architecture)

    def _validate(self):
        super()._validate()
        Assert.multiple(self.heads, self.head_groups)

    @property
    def layer_class(self):
        return Attention


class Attention(LayerBase):
    def __init__(self, config: AttentionConfig, distributed_config, *, hidden_dim: TensorDim, lr_scale=None, peft=None,
                 return_bias: bool = False):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self._hidden_dim = hidden_dim
        tp_dim = distributed_config.get_distributed_dim(DistributedDimNames.tensor)
        self._sequence_parallel = distributed_config.sequence_tensor_parallel
        self._sdp_dim = distributed_config.get_distributed_dim(DistributedDimNames.sequence_data)
        c = config
        # Head groups are split over the tensor group when there is more than one; with MQA the heads inside the
        # single group are split and the key/value projection is replicated.
        group_parallel = c.head_groups > 1
        if group_parallel:
            Assert.multiple(c.head_groups, tp_dim.size)
        else:
            Assert.multiple(c.heads, tp_dim.size)
        self._local_head_groups = div(c.head_groups, tp_dim.size) if group_parallel else 1
        self._local_heads = div(c.heads, tp_dim.size)
        head_size_dim = TensorDim("head_size", c.head_size)
        groups_dim = TensorDim("head_groups", c.head_groups, tp_dim if group_parallel else None)
        heads_dim = TensorDim("heads", c.heads, tp_dim)
        query_dim = CompositeTensorDim("query", (heads_dim, head_size_dim))
        key_dim = CompositeTensorDim("key", (groups_dim, head_size_dim))
        kv_parts = (key_dim,) if c.shared_key_value else (key_dim, CompositeTensorDim("value", (groups_dim, head_size_dim)))
        key_value_dim = ConcatenatedTensorDim("key_value", kv_parts)
        dense_dim = CompositeTensorDim("dense", (heads_dim, head_size_dim))
        self._softmax_scale = c.head_size ** (-c.softmax_scale_power)
        init = init_normal_(0.0, hidden_dim.global_size**-0.5)
        common = dict(default_add_bias=c.add_linear_biases, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        self.query = c.query_layer.get_layer(hidden_dim, query_dim, default_weight_initialization=init, default_apply_peft=True,
                                             sequence_parallel=self._sequence_parallel, **common)
        # key and value share one fused projection; `key_layer` configures it (value_layer must match, as in the reference)
        self.key_value = c.key_layer.get_layer(hidden_dim, key_value_dim, default_weight_initialization=init,
                                               sequence_parallel=self._sequence_parallel, **common)
        self.dense = c.dense_layer.get_layer(dense_dim, hidden_dim, default_weight_initialization=init_normal_(0.0, hidden_dim.global_size**-0.5),
                                             sequence_parallel=self._sequence_parallel, **common)
        self._rotary = c.rotary.get_layer(c.head_size)
        for name in ("query_norm", "key_norm", "value_norm"):
            norm_config = getattr(c, name)
            if norm_config is not None:
                setattr(self, name, norm_config.get_layer(head_size_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config))
        self._has_head_norms = any(getattr(c, n) is not None for n in ("query_norm", "key_norm", "value_norm"))
        self._return_bias = return_bias

    def preprocess(self, kwargs: dict) -> None:
        self._rotary.preprocess(kwargs)

    def _fused_weight(self):
        """Joint [q + kv, hidden] view when query and key_value weights (and their gradient buffers) are contiguous."""
        q, kv = self.query.weight, self.key_value.weight
        if getattr(self.query, "_forward_hook", None) or getattr(self.key_value, "_forward_hook", None):
            return None
        if not (torch.is_tensor(q) and torch.is_tensor(kv)) or q.dtype != kv.dtype or not q.is_contiguous():
            return None
        cached = self.__dict__.get("_fused_cache")
        if cached is not None and cached[0] == (q.data_ptr(), kv.data_ptr()):
            return cached[1]
        fused = None
        if q.data_ptr() + q.numel() * q.element_size() == kv.data_ptr() and q.untyped_storage().data_ptr() == kv.untyped_storage().data_ptr():
            rows = q.shape[0] + kv.shape[0]
            fused = torch.as_strided(q.detach(), (rows, q.shape[1]), (q.shape[1], 1))
            fused.requires_grad_(q.requires_grad)
            gq, gkv = getattr(q, "grad_buffer", None), getattr(kv, "grad_buffer", None)
            if gq is not None and gkv is not None and gq.data_ptr() + gq.numel() * gq.element_size() == gkv.data_ptr():
                fused.grad_buffer = torch.as_strided(gq, (rows, q.shape[1]), (q.shape[1], 1))
                fused._sources = (q, kv)
            elif gq is not None or gkv is not None or q.requires_grad:
                fused = None
        object.__setattr__(self, "_fused_cache", ((q.data_ptr(), kv.data_ptr()), fused))
        return fused

    def _project_qkv(self, x: torch.Tensor) -> torch.Tensor:
        has_bias = self.query._has_bias or self.key_value._has_bias
        fused = None if has_bias else self._fused_weight()
        if fused is not None:
            return linear(x, fused, None, mode=self.query.mode, group=self.query._group,
                          sequence_parallel=self._sequence_parallel and self.query._group is not None)
        return torch.cat([self.query(x), self.key_value(x)], dim=-1)

    def forward(self, x: torch.Tensor, kwargs: dict, losses=None, metrics=None) -> torch.Tensor:
        """x: [tokens(/tp with sequence parallelism), hidden] -> same shape."""
        c = self._config
        heads, groups, d = self._local_heads, self._local_head_groups, c.head_size
        qkv = self._project_qkv(x)
        if c.shared_key_value:
            qkv = torch.cat([qkv, qkv[:, heads * d :]], dim=-1)
        if self._has_head_norms:
            qkv = self._apply_head_norms(qkv, heads, groups, d)
        qkv = self._rotary.forward(qkv, heads + groups, kwargs)
        cu_q = kwargs[BlockKwargs.cu_seqlens_q]
        cu_k = kwargs.get(BlockKwargs.cu_seqlens_k, cu_q)
        max_q = kwargs[BlockKwargs.max_seqlen_q]
        max_k = kwargs.get(BlockKwargs.max_seqlen_k, max_q)
        past = kwargs.get(BlockKwargs.past_key_values)
        presents = kwargs.get(BlockKwargs.presents)
        simple = self._sdp_dim.size == 1 and past is None and presents is None
        if simple:
            out = packed_attention(qkv, cu_q, max_q, heads, groups, d, causal=c.causal, window_size=c.window_size,
                                   scale=self._softmax_scale, dropout_p=c.dropout if kwargs.get("training", True) else 0.0)
        else:
            t = qkv.shape[0]
            q = qkv[:, : heads * d].reshape(t, heads, d)
            kv = qkv[:, heads * d :]
            if self._sdp_dim.size > 1:
                # Sequence-data parallelism: every rank needs the keys/values of the whole sequence.
                kv = _GatherKV.apply(kv.contiguous(), self._sdp_dim.group)
            if past is not None and len(past) > 0:
                previous, rows = past.pop(0), kwargs.get(BlockKwargs.key_value_rows, 1)
                if rows > 1:  # a batch of sequences, each continuing its own cached prefix
                    kv = torch.cat([previous.view(rows, -1, kv.shape[-1]), kv.view(rows, -1, kv.shape[-1])], dim=1).reshape(-1, kv.shape[-1])
                else:
                    kv = torch.cat([previous, kv], dim=0)
            if presents is not None:
                presents.append(kv)
            tk = kv.shape[0]
            k = kv[:, : groups * d].reshape(tk, groups, d)
            v = kv[:, groups * d :].reshape(tk, groups, d)
            out = attention(q, k, v, cu_q, cu_k, max_q, max_k, causal=c.causal, window_size=c.window_size,
                            scale=self._softmax_scale, dropout_p=c.dropout if kwargs.get("training", True) else 0.0)
            out = out.reshape(t, heads * d)
        return self.dense(out)

    def _apply_head_norms(self, qkv, heads, groups, d):
        t = qkv.shape[0]
        q = qkv[:, : heads * d].reshape(t, heads, d)
        k = qkv[:, heads * d : (heads + groups) * d].reshape(t, groups, d)
        v = qkv[:, (heads + groups) * d :].reshape(t, groups, d)
        if self._config.query_norm is not None:
            q = self.query_norm(q)
        if self._config.key_norm is not None:
            k = self.key_norm(k)
        if self._config.value_norm is not None:
            v = self.value_norm(v)
        return torch.cat([q.reshape(t, -1), k.reshape(t, -1), v.reshape(t, -1)], dim=-1)

    def get_compute_usage(self, input_meta, kwargs, config=None) -> int:
        c = self._config
        tokens = kwargs[BlockKwargs.num_tokens]
        hidden = self._hidden_dim.global_size
        proj = 2 * tokens * hidden * (c.heads + 2 * c.head_groups) * c.head_size + 2 * tokens * hidden * c.heads * c.head_size
        # attention core: each query sees on average half its document (causal), capped by the window
        avg_k = kwargs.get("average_attended_keys", kwargs.get(BlockKwargs.max_seqlen_k, tokens) / (2 if c.causal else 1))
        if c.window_size is not None:
            avg_k = min(avg_k, c.window_size)
        core = 4 * tokens * avg_k * c.heads * c.head_size
        return int(proj + core)


class _GatherKV(torch.autograd.Function):
    """All-gather keys/values over the sequence-data group; backward reduce-scatters their gradient."""

    @staticmethod
    def forward(ctx, kv, group):
        from fast_llm_b200.parallel import fused_sdp

        ctx.group = group
        fused = fused_sdp.get(group)
        ctx.fused = fused if fused is not None and fused.usable(kv) else None
        if ctx.fused is not None:
            return ctx.fused.gather(kv)  # peers' slices pulled over NVLink by a copy kernel
        return gather_op(kv, group, 0)

    @staticmethod
    def backward(ctx, grad):
        if ctx.fused is not None:
            return ctx.fused.reduce_scatter(grad.contiguous()), None  # staged in the owners' buffers, summed in rank order
        return reduce_scatter_op(grad.contiguous(), ctx.group, dim=0), None
