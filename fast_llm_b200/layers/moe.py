"""Dropless mixture-of-experts MLP.

router (fp32) -> top-k -> softmax over the selected logits -> tokens sorted by expert (no capacity limit, nothing is
dropped) -> per-expert gated MLP on contiguous row ranges -> score-weighted scatter-add back to token order.
Auxiliary load-balancing loss, router z-loss, jitter, shared experts (always selected, score 1) and sinkhorn routing
follow `fast_llm/layers/decoder/mlp/mixture_of_experts.py:38-403`.  Parameters keep the reference layout:
`router.weight [experts, hidden]`, `layer_1.weight [experts * (2) * ffn, hidden]`, `layer_2.weight [experts * ffn, hidden]`.
The token permutation is built on the device without host synchronisation except for the per-expert row counts, which
size the grouped GEMM launches.
"""

import enum

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import LayerBase, LossDef
from fast_llm_b200.engine.initialization import init_normal_
from fast_llm_b200.engine.parameter import OptionalParameterConfig
from fast_llm_b200.layers.kwargs import BlockKwargs
from fast_llm_b200.layers.linear import LinearConfig
from fast_llm_b200.layers.mixer import MLPBaseConfig
from fast_llm_b200.layers.mlp import MLP, MLPConfig
from fast_llm_b200.layers.normalization import NormalizationConfig
from fast_llm_b200.ops.aux_loss import attach_auxiliary_loss
from fast_llm_b200.ops.mlp import MLPRecomputeLevel, mlp
from fast_llm_b200.parallel.topology import DistributedDimNames
from fast_llm_b200.tensor import CompositeTensorDim, ConcatenatedTensorDim, TensorDim
from fast_llm_b200.utils import Assert


class RoutingType(str, enum.Enum):
    topk = "aux_loss"
    sinkhorn = "sinkhorn"

    @classmethod
    def _missing_(cls, value):
        return {"topk": cls.topk, "top_k": cls.topk}.get(value)


class MoEImplementation(str, enum.Enum):
    auto = "auto"
    dropless = "dropless"
    looped = "looped"


@config_class(dynamic_type={MLPBaseConfig: "moe"})
class MoEMLPConfig(MLPConfig):
    router: LinearConfig = Field(desc="Router projection.", hint=FieldHint.architecture)
    router_normalization: NormalizationConfig | None = Field(default=None, desc="Normalization of the router input.", hint=FieldHint.architecture)
    router_scale: OptionalParameterConfig = Field(desc="Learnable per-channel scale of the router input.", hint=FieldHint.architecture)
    router_input_scale: float = Field(default=1.0, desc="Constant multiplier of the router input.", hint=FieldHint.architecture)
    router_per_expert_scale: OptionalParameterConfig = Field(desc="Learnable per-expert scale of the routing scores.", hint=FieldHint.architecture)
    experts: int = Field(default=2, desc="Number of experts.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 1))
    shared_experts: int = Field(default=0, desc="Experts applied to every token (counted in `experts`).", hint=FieldHint.architecture, valid=check_field(Assert.geq, 0))
    experts_per_token: int = Field(default=1, desc="Experts active per token, shared ones included.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    routing: RoutingType = Field(default=RoutingType.topk, desc="topk (with auxiliary loss) or sinkhorn.", hint=FieldHint.architecture)
    auxiliary_loss_coefficient: float = Field(default=0.01, desc="Weight of the load-balancing loss.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))
    z_loss_coefficient: float = Field(default=0.0, desc="Weight of the router z-loss.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))
    jitter_eps: float = Field(default=0.0, desc="Multiplicative noise on the router input during training.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))
    implementation: MoEImplementation = Field(default=MoEImplementation.auto, desc="dropless (sorted, grouped) or looped (masked dense per expert).", hint=FieldHint.expert)
    dropless_dynamic_shape: bool = Field(default=False, desc="Kept for schema compatibility (shapes are always exact here).", hint=FieldHint.expert)

    def _validate(self):
        super()._validate()
        Assert.leq(self.shared_experts, self.experts)
        Assert.in_range(self.experts_per_token, max(self.shared_experts, 1), self.experts + 1)

    @property
    def unshared_experts(self) -> int:
        return self.experts - self.shared_experts

    @property
    def routed_experts_per_token(self) -> int:
        return self.experts_per_token - self.shared_experts

    @property
    def layer_class(self):
        return MixtureOfExpertMLP


@config_class(dynamic_type={MLPBaseConfig: "hybrid_moe"})
class HybridMoEMLPConfig(MLPBaseConfig):
    """A dense MLP and a routed MoE applied to the same input; outputs are summed."""

    _abstract = False
    dense: MLPConfig = Field(desc="Dense branch.", hint=FieldHint.architecture)
    routed: MoEMLPConfig = Field(desc="Routed branch.", hint=FieldHint.architecture)

    @property
    def layer_class(self):
        return HybridMoEMLP


class MixtureOfExpertMLP(MLP):
    def __init__(self, config: MoEMLPConfig, distributed_config, *, hidden_dim: TensorDim, lr_scale=None, peft=None, return_bias=False):
        object.__setattr__(self, "_experts_dim", TensorDim("experts", config.experts))  # needed by _build, before base init
        super().__init__(config, distributed_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft, return_bias=return_bias)
        c = config
        self.router = c.router.get_layer(hidden_dim, TensorDim("router_experts", c.unshared_experts),
                                         default_weight_initialization=init_normal_(0.0, hidden_dim.global_size**-0.5),
                                         lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        if c.router_normalization is not None:
            self.router_norm = c.router_normalization.get_layer(hidden_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        from fast_llm_b200.engine.initialization import init_ones_

        scale = c.router_scale.get_parameter((hidden_dim,), default_initialization=init_ones_, lr_scale=self._lr_scale, weight_decay=False, default_enabled=False)
        if scale is not None:
            self.router_scale = scale
        self._has_router_scale = scale is not None
        per_expert = c.router_per_expert_scale.get_parameter((TensorDim("router_experts", c.unshared_experts),), default_initialization=init_ones_,
                                                            lr_scale=self._lr_scale, weight_decay=False, default_enabled=False)
        if per_expert is not None:
            self.router_per_expert_scale = per_expert
        self._has_per_expert_scale = per_expert is not None

    def _build(self, config, distributed_config, hidden_dim, l1_dim, ffn_dim, peft):
        # stacked expert weights: a leading `experts` factor on the output (layer 1) / input (layer 2) dimension
        experts = self._experts_dim
        l1 = CompositeTensorDim("moe_layer_1", (experts, l1_dim))
        l2 = CompositeTensorDim("moe_layer_2", (experts, ffn_dim))
        common = dict(default_add_bias=config.add_linear_biases, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        init = init_normal_(0.0, hidden_dim.global_size**-0.5)
        self.layer_1 = config.layer_1.get_layer(hidden_dim, l1, default_weight_initialization=init, sequence_parallel=self._sequence_parallel, **common)
        self.layer_2 = config.layer_2.get_layer(l2, hidden_dim, default_weight_initialization=init, sequence_parallel=self._sequence_parallel,
                                                transposed_weight=True, **common)
        assert not self.layer_1._has_bias and not self.layer_2._has_bias, "expert biases are not supported"

    def get_loss_definitions(self, count: int = 1):
        out = []
        if self._config.routing == RoutingType.topk and self._config.auxiliary_loss_coefficient > 0:
            out.append(LossDef("load_balancing_loss", "load balancing loss", count))
        if self._config.z_loss_coefficient > 0:
            out.append(LossDef("router_z_loss", "router z loss", count))
        return out

    # ------------------------------------------------------------------------------------------------
    def _route(self, x: torch.Tensor, kwargs: dict, losses: dict | None):
        """Returns (scores [T, k], expert indices [T, k], x possibly carrying auxiliary-loss gradients)."""
        c = self._config
        training = kwargs.get("training", True) and torch.is_grad_enabled()
        h = x
        if c.router_normalization is not None:
            h = self.router_norm(h)
        if c.router_input_scale != 1.0:
            h = h * c.router_input_scale
        if self._has_router_scale:
            h = h * self.router_scale
        if c.jitter_eps > 0 and training:
            noise = torch.empty_like(h).uniform_(1.0 - c.jitter_eps, 1.0 + c.jitter_eps, generator=self._distributed.tp_generator if self._distributed else None)
            h = h * noise
        logits = self.router(h.float() if h.dtype == torch.float32 or not h.is_cuda else h).float()
        grad_scale = kwargs.get(BlockKwargs.grad_output, 1.0)
        k = c.routed_experts_per_token
        from fast_llm_b200.ops.moe_routing import native_routing_available, route_topk

        if c.routing == RoutingType.topk and native_routing_available(logits, k):
            # scores, experts, both auxiliary losses and (in backward) the logit gradient of all of them in two kernels
            aux_weight = grad_scale * c.auxiliary_loss_coefficient if (training and c.auxiliary_loss_coefficient > 0) else 0.0
            z_weight = grad_scale * c.z_loss_coefficient if (training and c.z_loss_coefficient > 0) else 0.0
            scores, top_experts, aux, z = route_topk(logits, k, aux_weight, z_weight)
            if losses is not None:
                if c.z_loss_coefficient > 0:
                    losses.setdefault("router_z_loss", []).append(z)
                if c.auxiliary_loss_coefficient > 0:
                    losses.setdefault("load_balancing_loss", []).append(aux)
        else:
            if c.z_loss_coefficient > 0:
                z = torch.logsumexp(logits, dim=-1).pow(2).mean()
                if losses is not None:
                    losses.setdefault("router_z_loss", []).append(z.detach())
                if training:
                    logits = attach_auxiliary_loss(logits, z, grad_scale * c.z_loss_coefficient)
            if c.routing == RoutingType.sinkhorn:
                scores, top_experts = self._sinkhorn_routing(logits, k, training)
            else:
                top_logits, top_experts = torch.topk(logits, k=k, dim=-1)
                scores = torch.softmax(top_logits, dim=-1, dtype=torch.float32)
                if c.auxiliary_loss_coefficient > 0 and (training or losses is not None):
                    probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
                    mask = torch.zeros_like(probs).scatter_(1, top_experts, 1.0)
                    aux = c.unshared_experts * (mask.mean(0) * probs.mean(0)).sum()
                    if losses is not None:
                        losses.setdefault("load_balancing_loss", []).append(aux.detach())
                    if training:
                        scores = attach_auxiliary_loss(scores, aux, grad_scale * c.auxiliary_loss_coefficient)
        top_experts = top_experts.long() if (self._has_per_expert_scale or c.shared_experts > 0) else top_experts
        if self._has_per_expert_scale:
            scores = scores * self.router_per_expert_scale.float()[top_experts]
        if c.shared_experts > 0:
            # shared experts come first in the stacked weights; routed expert ids shift up
            t = scores.shape[0]
            shared_ids = torch.arange(c.shared_experts, device=x.device).expand(t, -1)
            top_experts = torch.cat([shared_ids, top_experts + c.shared_experts], dim=1)
            scores = torch.cat([scores.new_ones(t, c.shared_experts), scores], dim=1)
        return scores, top_experts

    @staticmethod
    def _sinkhorn(cost: torch.Tensor, tolerance: float = 1e-4, max_iterations: int = 100) -> torch.Tensor:
        cost = torch.exp(cost)
        d0 = torch.ones(cost.shape[0], device=cost.device, dtype=cost.dtype)
        d1 = torch.ones(cost.shape[1], device=cost.device, dtype=cost.dtype)
        eps, error, d1_old, it = 1e-8, 1e9, d1, 0
        while error > tolerance and it < max_iterations:
            d0 = (1 / d0.numel()) / (torch.sum(d1 * cost, 1) + eps)
            d1 = (1 / d1.numel()) / (torch.sum(d0.unsqueeze(1) * cost, 0) + eps)
            error = torch.mean(torch.abs(d1_old - d1)).item()
            d1_old = d1
            it += 1
        return d1 * cost * d0.unsqueeze(1)

    def _sinkhorn_routing(self, logits, k, training):
        if training:
            with torch.no_grad():
                _, top_experts = torch.topk(self._sinkhorn(logits.detach().float()), k=k, dim=-1)
            scores = torch.gather(torch.sigmoid(logits) if k == 1 else torch.softmax(logits, -1, dtype=torch.float32), 1, top_experts)
            return scores, top_experts
        probs = torch.sigmoid(logits) if k == 1 else torch.softmax(logits, -1, dtype=torch.float32)
        return torch.topk(probs, k=k, dim=-1)

    # ------------------------------------------------------------------------------------------------
    def _expert_weights(self):
        """Per-expert views of the stacked weights (and of their gradient buffers)."""
        c = self._config
        e = c.experts
        w1, w2 = self.layer_1.weight, self.layer_2.weight
        out = []
        for w in (w1, w2):
            gb = getattr(w, "grad_buffer", None)
            if gb is not None and getattr(w, "param_grad_is_zero", False) and torch.is_grad_enabled():
                # experts accumulate independently into slices of one buffer: start it from zero once
                gb.zero_()
                w.param_grad_is_zero = False
            views = list(w.view(e, w.shape[0] // e, w.shape[1]).unbind(0))
            if gb is not None:
                for view, g in zip(views, gb.view(e, w.shape[0] // e, w.shape[1]).unbind(0)):
                    view.grad_buffer = g
                    view.param_grad_is_zero = False
            out.append(views)
        return out

    def _forward(self, x: torch.Tensor, kwargs: dict | None = None, losses=None, metrics=None) -> torch.Tensor:
        kwargs = kwargs or {}
        c = self._config
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        group = self.layer_1._group
        sp = self._sequence_parallel and group is not None
        if sp:
            # routing needs every token: gather once, run the experts on all tokens, keep this rank's slice at the end
            from fast_llm_b200.parallel.ops import gather, split

            x2 = gather(x2, group, 0, reduce_grads=True)
        scores, top_experts = self._route(x2, kwargs, losses)
        from fast_llm_b200.ops.grouped_gemm import grouped_available

        if (c.implementation != MoEImplementation.looped and group is None and grouped_available(x2, c.intermediate_size, c.gated)
                and not self.layer_1._has_bias and self.layer_1._forward_hook is None and self.layer_2._forward_hook is None
                and torch.is_tensor(self.layer_1.weight) and self.layer_1.weight.is_contiguous()):
            out = self._forward_grouped(x2, scores, top_experts)
            return out.view(*shape[:-1], out.shape[-1])
        w1s, w2s = self._expert_weights()
        if c.implementation == MoEImplementation.looped:
            out = self._forward_looped(x2, scores, top_experts, w1s, w2s, group)
        else:
            out = self._forward_dropless(x2, scores, top_experts, w1s, w2s, group)
        if sp:
            out = split(out, group, 0)
        return out.view(*shape[:-1], out.shape[-1]) if out.shape[0] == x.reshape(-1, shape[-1]).shape[0] else out

    def _expert_mlp(self, rows, w1, w2, group):
        c = self._config
        recompute = c.recompute_level if c.recompute_level != MLPRecomputeLevel.none else MLPRecomputeLevel.activation
        # tensor-parallel experts: partial sums are all-reduced inside (sequence parallelism is handled by the caller)
        return mlp(rows, w1, None, w2, None, gated=c.gated, activation=c.activation, group=group, sequence_parallel=False, recompute_level=recompute)

    def _forward_grouped(self, x2, scores, top_experts):
        """All experts in one launch per product: rows sorted by expert and padded to whole tiles on the device (no host
        synchronisation), six grouped GEMMs on the tcgen05 kernel (`ops/grouped_gemm.py`)."""
        from fast_llm_b200.ops.grouped_gemm import TILE_ROWS, combine, dispatch, grouped_mlp
        from fast_llm_b200.ops.moe_routing import expert_rows_native

        c = self._config
        rows, row_begin, padded_rows = expert_rows_native(top_experts, c.experts, TILE_ROWS)
        xs = dispatch(x2, rows, padded_rows)
        ys = grouped_mlp(xs, row_begin, self.layer_1.weight, self.layer_2.weight, c.experts, c.gated, c.activation)
        return combine(ys, rows, scores)

    def _forward_dropless(self, x2, scores, top_experts, w1s, w2s, group):
        c = self._config
        top_experts = top_experts.long()
        t, k = top_experts.shape
        flat = top_experts.reshape(-1)
        order = torch.argsort(flat, stable=True)
        token_index = torch.div(order, k, rounding_mode="floor")
        counts = torch.bincount(flat, minlength=c.experts).tolist()  # sizes the per-expert launches
        xs = x2.index_select(0, token_index)
        sorted_scores = scores.reshape(-1).index_select(0, order)
        outs, begin = [], 0
        for e, n in enumerate(counts):
            rows = xs[begin : begin + n]
            outs.append(self._expert_mlp(rows, w1s[e], w2s[e], group) if n > 0 else rows.new_zeros(0, x2.shape[1]))
            begin += n
        ys = torch.cat(outs, 0)
        weighted = ys.float() * sorted_scores[:, None]
        out = torch.zeros(t, x2.shape[1], dtype=torch.float32, device=x2.device).index_add(0, token_index, weighted)
        return out.to(x2.dtype)

    def _forward_looped(self, x2, scores, top_experts, w1s, w2s, group):
        top_experts = top_experts.long()
        out = torch.zeros(x2.shape, dtype=torch.float32, device=x2.device)
        for e in range(self._config.experts):
            weight = (scores * (top_experts == e)).sum(-1)
            selected = torch.nonzero(weight, as_tuple=True)[0]
            if selected.numel() == 0:
                continue
            y = self._expert_mlp(x2.index_select(0, selected), w1s[e], w2s[e], group)
            out = out.index_add(0, selected, y.float() * weight[selected][:, None])
        return out.to(x2.dtype)

    def get_compute_usage(self, input_meta, kwargs, config=None) -> int:
        c = self._config
        tokens = kwargs[BlockKwargs.num_tokens]
        hidden = self._hidden_dim.global_size
        experts = 2 * tokens * c.experts_per_token * hidden * c.intermediate_size * (3 if c.gated else 2)
        return experts + 2 * tokens * hidden * c.unshared_experts


class HybridMoEMLP(LayerBase):
    def __init__(self, config: HybridMoEMLPConfig, distributed_config, *, hidden_dim, lr_scale=None, peft=None, return_bias=False):
        super().__init__(config, distributed_config, lr_scale=lr_scale, peft=peft)
        self.dense = config.dense.get_layer(distributed_config, hidden_dim, lr_scale=lr_scale, peft=peft)
        self.routed = config.routed.get_layer(distributed_config, hidden_dim, lr_scale=lr_scale, peft=peft)
        if config.pre_norm is not None:
            self.pre_norm = config.pre_norm.get_layer(hidden_dim, lr_scale=lr_scale, peft=peft, distributed_config=distributed_config)
        if config.post_norm is not None:
            self.post_norm = config.post_norm.get_layer(hidden_dim, lr_scale=lr_scale, peft=peft, distributed_config=distributed_config)

    def forward(self, x, kwargs=None, losses=None, metrics=None):
        if self._config.pre_norm is not None:
            x = self.pre_norm(x)
        out = self.dense.forward(x, kwargs, losses, metrics) + self.routed.forward(x, kwargs, losses, metrics)
        if self._config.post_norm is not None:
            out = self.post_norm(out)
        return out
