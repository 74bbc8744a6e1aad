"""Language-model head losses: label (cross-entropy / KL from labels), z_loss, distillation, dpo, grpo, gspo.

Every loss maps one chunk of logits to (scalar value, gradient wrt the logits).  Cross-entropy from labels, optionally
with a z-loss riding on the same softmax, runs on the fused kernels of `fast_llm_b200.ops.cross_entropy`
(vocabulary-parallel aware); the others are written with PyTorch ops and differentiated by autograd on the chunk.
Parity: `fast_llm/layers/language_model/loss/*.py`, `fast_llm/functional/entropy_loss.py`,
`fast_llm/functional/triton/{entropy_loss,z_loss,grpo_loss,gspo_loss,monolithic_loss}.py`.
"""

import enum

import torch

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import LossDef
from fast_llm_b200.layers.kwargs import LanguageModelKwargs
from fast_llm_b200.ops.cross_entropy import cross_entropy_forward_backward
from fast_llm_b200.parallel.collectives import all_reduce
from fast_llm_b200.parallel.ops import split_op
from fast_llm_b200.utils import Assert


class EntropyLossType(str, enum.Enum):
    cross_entropy = "cross_entropy"
    forward_kl = "forward_kl"
    reverse_kl = "reverse_kl"


class PolicyMetricsLevel(str, enum.Enum):
    auto = "auto"
    none = "none"
    basic = "basic"
    full = "full"


@config_class(registry=True)
class LanguageModelLossConfig(Config):
    _abstract = True
    weight: float = Field(default=1.0, desc="Weight of this loss in the total.", hint=FieldHint.core, valid=check_field(Assert.geq, 0.0))
    logits_scale_factor: float = Field(default=1.0, desc="Extra multiplier of the logits for this loss.", hint=FieldHint.feature, valid=check_field(Assert.gt, 0.0))

    @classmethod
    def _get_default_subclass(cls):
        return LanguageModelLabelEntropyLossConfig if cls is LanguageModelLossConfig else cls

    def get_layer(self, distributed_config, *, name: str, prediction_distance: int = 1, vocab_parallel: bool = False, weight: float | None = None):
        return self.loss_class(self, distributed_config, name=name, prediction_distance=prediction_distance,
                               vocab_parallel=vocab_parallel, weight=self.weight if weight is None else weight)


@config_class()
class CombinableLossConfig(LanguageModelLossConfig):
    _abstract = True
    use_triton: bool | None = Field(default=None, desc="Kept for schema compatibility (the fused CUDA kernels are always used on GPU).", hint=FieldHint.expert)


@config_class(dynamic_type={LanguageModelLossConfig: "label"})
class LanguageModelLabelEntropyLossConfig(CombinableLossConfig):
    _abstract = False
    loss_type: EntropyLossType = Field(default=EntropyLossType.cross_entropy, desc="cross_entropy, forward_kl or reverse_kl (identical for one-hot targets up to a constant).", hint=FieldHint.core)

    @property
    def loss_class(self):
        return LabelEntropyLoss


@config_class(dynamic_type={LanguageModelLossConfig: "distillation"})
class LanguageModelDistillationLossConfig(CombinableLossConfig):
    _abstract = False
    loss_type: EntropyLossType = Field(default=EntropyLossType.cross_entropy, hint=FieldHint.core)
    reference_model: str = Field(default="teacher", desc="Name of the reference model providing target logits.", hint=FieldHint.feature)
    temperature: float = Field(default=1.0, hint=FieldHint.optional, valid=check_field(Assert.gt, 0.0))

    @property
    def loss_class(self):
        return DistillationLoss


@config_class(dynamic_type={LanguageModelLossConfig: "dpo"})
class LanguageModelDPOLossConfig(LanguageModelLossConfig):
    _abstract = False
    beta: float = Field(default=1.0, hint=FieldHint.core, valid=check_field(Assert.gt, 0.0))
    reference_model: str = Field(default="reference", desc="Name of the frozen reference policy.", hint=FieldHint.feature)

    @property
    def loss_class(self):
        return DPOLoss


@config_class(dynamic_type={LanguageModelLossConfig: "z_loss"})
class LanguageModelZLossConfig(CombinableLossConfig):
    _abstract = False

    @property
    def loss_class(self):
        return ZLoss


@config_class()
class LanguageModelPolicyGradientLossConfig(LanguageModelLossConfig):
    _abstract = True
    epsilon_low: float = Field(default=0.2, desc="Lower clip of the probability ratio.")
    epsilon_high: float = Field(default=0.2, desc="Upper clip of the probability ratio.")
    metrics: PolicyMetricsLevel = Field(default=PolicyMetricsLevel.auto, desc="Extra policy metrics to log.", hint=FieldHint.feature)


@config_class(dynamic_type={LanguageModelLossConfig: "grpo"})
class LanguageModelGRPOLossConfig(LanguageModelPolicyGradientLossConfig, CombinableLossConfig):
    _abstract = False

    @property
    def loss_class(self):
        return GRPOLoss


@config_class(dynamic_type={LanguageModelLossConfig: "gspo"})
class LanguageModelGSPOLossConfig(LanguageModelPolicyGradientLossConfig, CombinableLossConfig):
    _abstract = False

    @property
    def loss_class(self):
        return GSPOLoss


@config_class()
class MonolithicLossConfig(LanguageModelLossConfig):
    """Several label-based losses evaluated over one shared softmax."""

    _abstract = False
    losses: dict[str, LanguageModelLossConfig] = Field(default_factory=dict, hint=FieldHint.core)
    use_triton: bool | None = Field(default=None, hint=FieldHint.expert)

    @property
    def loss_class(self):
        return MonolithicLoss


# ---------------------------------------------------------------------------------------------------------------------
class LanguageModelLoss:
    needs_reference = False

    def __init__(self, config, distributed_config, *, name: str, prediction_distance: int, vocab_parallel: bool, weight: float):
        self._config = config
        self._distributed_config = distributed_config
        self.name = name
        self.weight = weight
        self._prediction_distance = prediction_distance
        self._vocab_parallel = vocab_parallel
        self._sequence_parallel = distributed_config.sequence_tensor_parallel and not vocab_parallel
        self._group = None
        self._tp_group = None
        self._sdp_group = None
        self._vocab_begin = 0

    def setup(self, distributed, logits_group, vocab_begin: int) -> None:
        self._group = logits_group
        self._tp_group = distributed.tensor_group
        self._sdp_group = distributed.sequence_data_group
        self._vocab_begin = vocab_begin

    def get_loss_definitions(self, count: int = 1) -> list[LossDef]:
        return [LossDef(self.name, self.name.replace("_", " "), count)]

    def get_preprocessing_config(self, phase) -> dict:
        return {}

    # ---- helpers
    def _token_slice(self, tensor, rows, split_index, num_splits):
        """Rows of a per-token tensor matching this chunk of logits (sequence-parallel shard, then split chunk)."""
        if self._sequence_parallel and self._tp_group is not None:
            tensor = split_op(tensor, self._tp_group, 0)
        if num_splits > 1:
            tensor = tensor.chunk(num_splits, dim=0)[split_index]
        Assert.eq(tensor.shape[0], rows)
        return tensor

    def _labels(self, kwargs, rows, split_index, num_splits):
        key = LanguageModelKwargs.labels if self._prediction_distance == 1 else f"{LanguageModelKwargs.labels}_{self._prediction_distance}"
        return self._token_slice(kwargs[key], rows, split_index, num_splits)

    def _inverse_label_count(self, kwargs) -> torch.Tensor:
        """1 / (number of valid labels in the whole micro-batch, over all ranks that share it), kept on the device."""
        key = f"_inverse_label_count_{self._prediction_distance}"
        if key not in kwargs:
            lkey = LanguageModelKwargs.labels if self._prediction_distance == 1 else f"{LanguageModelKwargs.labels}_{self._prediction_distance}"
            count = (kwargs[lkey] >= 0).sum().float().reshape(1)
            kwargs[key] = 1.0 / count.clamp(min=1.0)
        return kwargs[key]

    def _finalize(self, per_token_sum: torch.Tensor) -> torch.Tensor:
        """Sum partial per-token sums over the ranks that share one micro-batch (sequence-parallel token shards,
        sequence-data-parallel token slices)."""
        if self._sequence_parallel and self._tp_group is not None:
            per_token_sum = per_token_sum.clone()
            all_reduce(per_token_sum, group=self._tp_group)
        if self._sdp_group is not None:
            per_token_sum = per_token_sum.clone()
            all_reduce(per_token_sum, group=self._sdp_group)
        return per_token_sum

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        raise NotImplementedError

    def _autograd(self, fn, logits, grad_output, accumulate_into):
        """Evaluate a PyTorch-written loss and its logits gradient."""
        if grad_output is None:
            with torch.no_grad():
                return fn(logits.float()), accumulate_into
        with torch.enable_grad():
            x = logits.detach().float().requires_grad_()
            value = fn(x)
        (g,) = torch.autograd.grad(value, x, torch.as_tensor(grad_output * self.weight, dtype=value.dtype, device=value.device))
        g = g.to(logits.dtype)
        if accumulate_into is not None:
            g = accumulate_into.add_(g)
        return value.detach(), g


class LabelEntropyLoss(LanguageModelLoss):
    z_coefficient = 0.0

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        rows = logits.shape[0]
        labels = self._labels(kwargs, rows, split_index, num_splits)
        inv = self._inverse_label_count(kwargs)
        scale = logits_scale * self._config.logits_scale_factor
        grad_scale = None if grad_output is None else inv * float(grad_output * self.weight)
        in_place = accumulate_into is None and kwargs.get("_single_loss", True)
        loss_tok, z_tok, grad = cross_entropy_forward_backward(
            logits, labels, grad_scale, scale, self.z_coefficient, self._group, self._vocab_begin, in_place=in_place)
        if grad is not None and accumulate_into is not None:
            grad = accumulate_into.add_(grad)
        value = self._finalize(loss_tok.sum().reshape(1) * inv).reshape(())
        self._z_value = self._finalize(z_tok.sum().reshape(1) * inv).reshape(()) if self.z_coefficient else None
        return value, grad


class ZLoss(LanguageModelLoss):
    """mean over tokens of logsumexp(logits)^2"""

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        rows = logits.shape[0]
        labels = self._labels(kwargs, rows, split_index, num_splits)
        inv = self._inverse_label_count(kwargs)
        scale = logits_scale * self._config.logits_scale_factor

        def fn(x):
            x = x * scale
            if self._group is not None:
                m = x.max(-1).values.detach()
                all_reduce(m, op=torch.distributed.ReduceOp.MAX, group=self._group)
                se = torch.exp(x - m[:, None]).sum(-1)
                se = _AllReduceSum.apply(se, self._group)
                lse = m + se.log()
            else:
                lse = torch.logsumexp(x, -1)
            return ((lse * lse) * (labels >= 0)).sum() * inv.reshape(())

        value, grad = self._autograd(fn, logits, grad_output, accumulate_into)
        return self._finalize(value.reshape(1)).reshape(()), grad


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad, None


def _log_softmax(x, group):
    if group is None:
        return torch.log_softmax(x, -1)
    m = x.max(-1).values.detach()
    all_reduce(m, op=torch.distributed.ReduceOp.MAX, group=group)
    se = _AllReduceSum.apply(torch.exp(x - m[:, None]).sum(-1), group)
    return x - m[:, None] - se.log()[:, None]


class DistillationLoss(LanguageModelLoss):
    needs_reference = True

    def get_preprocessing_config(self, phase):
        return {"reference_models": {self._config.reference_model}}

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        rows = logits.shape[0]
        teacher = kwargs[f"{self._config.reference_model}_logits"]
        teacher = self._token_slice(teacher, rows, split_index, num_splits).float()
        if self._group is not None:
            size = logits.shape[-1]
            teacher = teacher[:, self._vocab_begin : self._vocab_begin + size] if teacher.shape[-1] != size else teacher
        mask = kwargs.get(LanguageModelKwargs.loss_mask)
        mask = torch.ones(rows, device=logits.device) if mask is None else self._token_slice(mask, rows, split_index, num_splits).float()
        count = mask.sum().clamp(min=1.0) * (num_splits if False else 1)
        temp = self._config.temperature
        scale = logits_scale * self._config.logits_scale_factor / temp
        kind = self._config.loss_type

        def fn(x):
            student_lp = _log_softmax(x * scale, self._group)
            teacher_lp = _log_softmax(teacher / temp, self._group)
            if kind == EntropyLossType.reverse_kl:
                per = (student_lp.exp() * (student_lp - teacher_lp)).sum(-1)
            elif kind == EntropyLossType.forward_kl:
                per = (teacher_lp.exp() * (teacher_lp - student_lp)).sum(-1)
            else:
                per = -(teacher_lp.exp() * student_lp).sum(-1)
            if self._group is not None:
                per = _AllReduceSum.apply(per, self._group)
            return (per * mask).sum() / count

        value, grad = self._autograd(fn, logits, grad_output, accumulate_into)
        return self._finalize(value.reshape(1)).reshape(()), grad


def _gather_label_log_probs(x, labels, group, vocab_begin):
    """log p(label) for every token (0 for ignored labels)."""
    lp = _log_softmax(x, group)
    lab = labels - vocab_begin
    ok = (lab >= 0) & (lab < x.shape[-1]) & (labels >= 0)
    picked = lp.gather(-1, lab.clamp(0, x.shape[-1] - 1)[:, None])[:, 0] * ok
    if group is not None:
        picked = _AllReduceSum.apply(picked, group)
    return picked


class DPOLoss(LanguageModelLoss):
    """-log sigmoid(beta * ((pi_chosen - pi_rejected) - (ref_chosen - ref_rejected))) over preference spans."""

    needs_reference = True

    def get_preprocessing_config(self, phase):
        return {"use_preference_spans": True, "reference_models": {self._config.reference_model}}

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        Assert.eq(num_splits, 1)
        rows = logits.shape[0]
        labels = self._labels(kwargs, rows, 0, 1)
        chosen = kwargs[LanguageModelKwargs.chosen_spans]
        rejected = kwargs[LanguageModelKwargs.rejected_spans]
        ref_logits = kwargs[f"{self._config.reference_model}_logits"].float()
        scale = logits_scale * self._config.logits_scale_factor

        def span_sum(per_token, spans):
            return torch.stack([per_token[b:e].sum() for b, e in spans]) if len(spans) else per_token.new_zeros(0)

        def fn(x):
            lp = _gather_label_log_probs(x * scale, labels, self._group, self._vocab_begin)
            with torch.no_grad():
                ref_lp = _gather_label_log_probs(ref_logits * scale, labels, None, 0)
            pi = span_sum(lp, chosen) - span_sum(lp, rejected)
            ref = span_sum(ref_lp, chosen) - span_sum(ref_lp, rejected)
            return -torch.nn.functional.logsigmoid(self._config.beta * (pi - ref)).mean()

        return self._autograd(fn, logits, grad_output, accumulate_into)


class GRPOLoss(LanguageModelLoss):
    """Clipped policy-gradient surrogate per token: -min(r A, clip(r, 1-eps_low, 1+eps_high) A), r = pi / pi_old."""

    def get_preprocessing_config(self, phase):
        return {"use_grpo_data": True}

    def _ratio_terms(self, x, kwargs, rows, split_index, num_splits, scale):
        labels = self._labels(kwargs, rows, split_index, num_splits)
        adv = self._token_slice(kwargs[LanguageModelKwargs.advantages], rows, split_index, num_splits).float()
        old = self._token_slice(kwargs[LanguageModelKwargs.old_log_probabilities], rows, split_index, num_splits).float()
        lp = _gather_label_log_probs(x * scale, labels, self._group, self._vocab_begin)
        return labels, adv, old, lp

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        rows = logits.shape[0]
        inv = self._inverse_label_count(kwargs).reshape(())
        scale = logits_scale * self._config.logits_scale_factor
        c = self._config

        def fn(x):
            labels, adv, old, lp = self._ratio_terms(x, kwargs, rows, split_index, num_splits, scale)
            ratio = torch.exp(lp - old)
            clipped = ratio.clamp(1 - c.epsilon_low, 1 + c.epsilon_high)
            per = -torch.minimum(ratio * adv, clipped * adv) * (labels >= 0)
            return per.sum() * inv

        value, grad = self._autograd(fn, logits, grad_output, accumulate_into)
        return self._finalize(value.reshape(1)).reshape(()), grad


class GSPOLoss(GRPOLoss):
    """Sequence-level ratio: the geometric mean of token ratios of each document replaces the per-token ratio."""

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        Assert.eq(num_splits, 1)
        rows = logits.shape[0]
        inv = self._inverse_label_count(kwargs).reshape(())
        scale = logits_scale * self._config.logits_scale_factor
        c = self._config
        doc = self._token_slice(kwargs[LanguageModelKwargs.document_index], rows, 0, 1).long()

        def fn(x):
            labels, adv, old, lp = self._ratio_terms(x, kwargs, rows, 0, 1, scale)
            valid = (labels >= 0).float()
            n_docs = int(doc.max().item()) + 1 if doc.numel() else 0
            num = torch.zeros(n_docs, device=x.device).index_add(0, doc, (lp - old) * valid)
            den = torch.zeros(n_docs, device=x.device).index_add(0, doc, valid).clamp(min=1.0)
            seq_ratio = torch.exp(num / den)[doc]
            clipped = seq_ratio.clamp(1 - c.epsilon_low, 1 + c.epsilon_high)
            per = -torch.minimum(seq_ratio * adv, clipped * adv) * valid
            return per.sum() * inv

        value, grad = self._autograd(fn, logits, grad_output, accumulate_into)
        return self._finalize(value.reshape(1)).reshape(()), grad


class MonolithicLoss(LanguageModelLoss):
    """Label cross-entropy and z-loss share one softmax pass on the fused kernel; other members run after it."""

    def __init__(self, config, distributed_config, *, name, prediction_distance, vocab_parallel, weight):
        super().__init__(config, distributed_config, name=name, prediction_distance=prediction_distance, vocab_parallel=vocab_parallel, weight=weight)
        self._members = [
            lc.get_layer(distributed_config, name=n, prediction_distance=prediction_distance, vocab_parallel=vocab_parallel)
            for n, lc in config.losses.items()
        ]

    def setup(self, distributed, logits_group, vocab_begin):
        super().setup(distributed, logits_group, vocab_begin)
        for m in self._members:
            m.setup(distributed, logits_group, vocab_begin)

    def get_loss_definitions(self, count=1):
        return [LossDef(self.name, self.name.replace("_", " "), count)] + [d for m in self._members for d in m.get_loss_definitions(count)]

    def get_preprocessing_config(self, phase):
        out = {}
        for m in self._members:
            out.update(m.get_preprocessing_config(phase))
        return out

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        label = next((m for m in self._members if type(m) is LabelEntropyLoss), None)
        z = next((m for m in self._members if type(m) is ZLoss), None)
        others = [m for m in self._members if m is not label and (m is not z or label is None)]
        total, grad = None, accumulate_into
        sub_grad_output = None if grad_output is None else grad_output * self.weight
        for m in others:
            value, grad = m.forward_backward(logits, kwargs, sub_grad_output, split_index, num_splits, logits_scale, accumulate_into=grad)
            total = value * m.weight if total is None else total + value * m.weight
        if label is not None:
            label.z_coefficient = (z.weight / label.weight) if (z is not None and label.weight > 0) else 0.0
            kwargs["_single_loss"] = grad is None
            value, grad = label.forward_backward(logits, kwargs, sub_grad_output, split_index, num_splits, logits_scale, accumulate_into=grad)
            kwargs.pop("_single_loss", None)
            total = value * label.weight if total is None else total + value * label.weight
            if z is not None and label._z_value is not None:
                total = total + label._z_value * z.weight
        return total, grad
