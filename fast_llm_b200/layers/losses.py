"""Language-model head losses: label (cross-entropy / KL from labels), z_loss, distillation, dpo, grpo, gspo.

Every loss maps one chunk of logits to (scalar value, gradient wrt the logits).  The losses that see the logits only
through the softmax normaliser and the label's logit (label cross-entropy / KL, z-loss, GRPO, GSPO, DPO) are functions of
two per-token vectors; `MonolithicLoss` sums the coefficients of its members and writes their joint gradient in ONE pass
over the logits (`fast_llm_b200.ops.losses`, `csrc/loss.cu`).  Distillation (cross-entropy / forward KL / reverse KL
against teacher logits) has its own statistics and gradient kernels.  No loss makes an fp32 copy of the logits or runs
autograd over them; everything is vocabulary-parallel aware.
Parity: `fast_llm/layers/language_model/loss/*.py`, `fast_llm/functional/entropy_loss.py`,
`fast_llm/functional/triton/{entropy_loss,z_loss,grpo_loss,gspo_loss,monolithic_loss}.py`.
"""

import enum
import math

import torch

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class
from fast_llm_b200.engine.base_model import LossDef
from fast_llm_b200.layers.kwargs import LanguageModelKwargs
from fast_llm_b200.ops.losses import (SoftmaxStatistics, distribution_loss_forward_backward, label_coefficients, softmax_coeff_grad,
                                      softmax_statistics)
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

    def _scale(self, logits_scale: float) -> float:
        return logits_scale * self._config.logits_scale_factor

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        raise NotImplementedError


class LabelBasedLoss(LanguageModelLoss):
    """A loss that sees the logits only through `lse` and the label's logit (both `[tokens]` fp32 vectors).

    Subclasses implement `per_token_value(lse, target, labels, kwargs, rows, split_index, num_splits) -> scalar` (already
    normalised, differentiable wrt lse and target).  Several such losses share one statistics pass and one gradient pass when
    grouped in a `MonolithicLoss`; alone, each still needs just those two passes."""

    shares_softmax = True

    def per_token_value(self, lse, target, labels, kwargs, rows, split_index, num_splits) -> torch.Tensor:
        raise NotImplementedError

    def coefficients(self, stats: SoftmaxStatistics, labels, kwargs, rows, split_index, num_splits, grad_output):
        """(value, a, b): the loss value on this chunk and its derivatives wrt lse / target, times `grad_output * weight`."""
        weight = None if grad_output is None else float(grad_output) * self.weight
        return label_coefficients(lambda lse, target: self.per_token_value(lse, target, labels, kwargs, rows, split_index, num_splits),
                                  stats, weight)

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        rows = logits.shape[0]
        labels = self._labels(kwargs, rows, split_index, num_splits)
        stats = softmax_statistics(logits, labels, self._scale(logits_scale), self._group, self._vocab_begin)
        value, a, b = self.coefficients(stats, labels, kwargs, rows, split_index, num_splits, grad_output)
        grad = accumulate_into
        if a is not None:
            grad = softmax_coeff_grad(logits, labels, stats, a, b, accumulate_into=accumulate_into,
                                      in_place=accumulate_into is None and kwargs.get("_single_loss", True))
        return self._finalize(value.reshape(1)).reshape(()), grad


class LabelEntropyLoss(LabelBasedLoss):
    """Cross-entropy against labels.  Forward KL against a one-hot target equals it; reverse KL against a one-hot target
    (smoothed by 1e-10 inside the logarithm, as `fast_llm/functional/entropy_loss.py:56-80` does) is
    sum_j p_j (log p_j - log(onehot_j + 1e-10)), which needs the entropy of p and is evaluated on the logits directly."""

    def per_token_value(self, lse, target, labels, kwargs, rows, split_index, num_splits):
        inv = self._inverse_label_count(kwargs).reshape(())
        return ((lse - target) * (labels >= 0)).sum() * inv

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        if self._config.loss_type != EntropyLossType.reverse_kl:
            return super().forward_backward(logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into)
        rows = logits.shape[0]
        labels = self._labels(kwargs, rows, split_index, num_splits)
        inv = self._inverse_label_count(kwargs).reshape(())
        valid = labels >= 0
        lab = labels - self._vocab_begin
        in_shard = valid & (lab >= 0) & (lab < logits.shape[-1])
        # teacher "logits" of the smoothed one-hot target: log(1 + 1e-10) at the label, log(1e-10) elsewhere
        teacher = torch.full_like(logits, math.log(1e-10), dtype=torch.float32)
        teacher[in_shard, lab[in_shard]] = math.log1p(1e-10)
        g = None if grad_output is None else inv * float(grad_output * self.weight)
        loss, grad = distribution_loss_forward_backward(
            logits, teacher, valid.float(), g, "reverse_kl", logits_scale=self._scale(logits_scale), group=self._group,
            accumulate_into=accumulate_into, normalize_teacher=False)
        return self._finalize((loss.sum() * inv).reshape(1)).reshape(()), (grad if grad is not None else accumulate_into)


class ZLoss(LabelBasedLoss):
    """mean over valid tokens of logsumexp(logits)^2"""

    def per_token_value(self, lse, target, labels, kwargs, rows, split_index, num_splits):
        inv = self._inverse_label_count(kwargs).reshape(())
        return ((lse * lse) * (labels >= 0)).sum() * inv


class DistillationLoss(LanguageModelLoss):
    needs_reference = True

    def get_preprocessing_config(self, phase):
        return {"reference_models": {self._config.reference_model}}

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        rows = logits.shape[0]
        teacher = kwargs[f"{self._config.reference_model}_logits"]
        teacher = self._token_slice(teacher, rows, split_index, num_splits)
        size = logits.shape[-1]
        if self._group is not None and teacher.shape[-1] != size:
            teacher = teacher[:, self._vocab_begin : self._vocab_begin + size]
        mask = kwargs.get(LanguageModelKwargs.loss_mask)
        mask = None if mask is None else self._token_slice(mask, rows, split_index, num_splits).float()
        count = torch.tensor(float(rows), device=logits.device) if mask is None else mask.sum().clamp(min=1.0)
        # the temperature softens the teacher only (`fast_llm/functional/entropy_loss.py:42-44`, `triton/entropy_loss.py:890`)
        temperature = self._config.temperature
        scale = self._scale(logits_scale)
        g = None if grad_output is None else float(grad_output * self.weight) / count
        loss, grad = distribution_loss_forward_backward(
            logits, teacher, mask, g, self._config.loss_type.value, logits_scale=scale, teacher_scale=scale / temperature,
            group=self._group, accumulate_into=accumulate_into, in_place=accumulate_into is None and kwargs.get("_single_loss", True))
        value = loss.sum() / count
        return self._finalize(value.reshape(1)).reshape(()), (grad if grad is not None else accumulate_into)


def _label_log_probs(lse, target, labels):
    """log p(label) per token, 0 where the label is ignored."""
    return (target - lse) * (labels >= 0)


def _span_sums(per_token: torch.Tensor, spans) -> torch.Tensor:
    if not len(spans):
        return per_token.new_zeros(0)
    return torch.stack([per_token[b:e].sum() for b, e in spans])


class DPOLoss(LabelBasedLoss):
    """-log sigmoid(beta * ((pi_chosen - pi_rejected) - (ref_chosen - ref_rejected))), log-probabilities summed over the
    chosen / rejected spans."""

    needs_reference = True

    def get_preprocessing_config(self, phase):
        return {"use_preference_spans": True, "reference_models": {self._config.reference_model}}

    def per_token_value(self, lse, target, labels, kwargs, rows, split_index, num_splits):
        Assert.eq(num_splits, 1)
        chosen = kwargs[LanguageModelKwargs.chosen_spans]
        rejected = kwargs[LanguageModelKwargs.rejected_spans]
        log_probs = _label_log_probs(lse, target, labels)
        ref_key = f"_{self._config.reference_model}_label_log_probs_{self._prediction_distance}"
        if ref_key not in kwargs:
            ref_logits = kwargs[f"{self._config.reference_model}_logits"]
            ref_labels = labels
            ref_group, ref_begin = (self._group, self._vocab_begin) if ref_logits.shape[-1] == kwargs["_logits_columns"] else (None, 0)
            with torch.no_grad():
                ref_stats = softmax_statistics(ref_logits, ref_labels, kwargs["_logits_scale"], ref_group, ref_begin)
                kwargs[ref_key] = _label_log_probs(ref_stats.lse, ref_stats.target, ref_labels)
        ref_log_probs = kwargs[ref_key]
        # one log-ratio over all spans of the micro-batch, as `fast_llm/layers/language_model/loss/dpo.py:53-79`
        pi = _span_sums(log_probs, chosen).sum() - _span_sums(log_probs, rejected).sum()
        ref = _span_sums(ref_log_probs, chosen).sum() - _span_sums(ref_log_probs, rejected).sum()
        return -torch.nn.functional.logsigmoid(self._config.beta * (pi - ref))

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        kwargs["_logits_columns"] = logits.shape[-1]
        kwargs["_logits_scale"] = self._scale(logits_scale)
        value, grad = super().forward_backward(logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into)
        return value, grad

    def _finalize(self, per_token_sum):
        return per_token_sum  # spans are whole on every rank that holds the logits


class GRPOLoss(LabelBasedLoss):
    """Clipped policy-gradient surrogate per token: -min(r A, clip(r, 1-eps_low, 1+eps_high) A), r = pi / pi_old."""

    def get_preprocessing_config(self, phase):
        return {"use_grpo_data": True}

    def _inputs(self, kwargs, rows, split_index, num_splits):
        adv = self._token_slice(kwargs[LanguageModelKwargs.advantages], rows, split_index, num_splits).float()
        old = self._token_slice(kwargs[LanguageModelKwargs.old_log_probabilities], rows, split_index, num_splits).float()
        return adv, old

    def _surrogate(self, ratio, adv):
        c = self._config
        return -torch.minimum(ratio * adv, ratio.clamp(1 - c.epsilon_low, 1 + c.epsilon_high) * adv)

    def per_token_value(self, lse, target, labels, kwargs, rows, split_index, num_splits):
        adv, old = self._inputs(kwargs, rows, split_index, num_splits)
        inv = self._inverse_label_count(kwargs).reshape(())
        valid = labels >= 0
        ratio = torch.exp((_label_log_probs(lse, target, labels) - old) * valid)
        return (self._surrogate(ratio, adv) * valid).sum() * inv


class _SumOverRanks(torch.autograd.Function):
    """Sum a small tensor over a process group; the gradient passes through unchanged (every rank differentiates the global
    sum with respect to its own contribution)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class GSPOLoss(GRPOLoss):
    """Sequence-level clipping: per document d the ratio is the geometric mean of its token ratios,
    R_d = exp(mean_t log(pi_t / pi_old_t)), the advantage A_d the mean of its token advantages, and the loss
    sum_d N_d * -min(R_d A_d, clip(R_d) A_d) over the labelled-token counts N_d, divided by the batch's label count
    (`fast_llm/layers/language_model/loss/policy_gradient.py:1179-1250`).  Documents split over sequence-parallel or
    sequence-data-parallel ranks are aggregated across them; a document must not be split over micro-sequences."""

    def per_token_value(self, lse, target, labels, kwargs, rows, split_index, num_splits):
        Assert.eq(num_splits, 1)
        adv, old = self._inputs(kwargs, rows, 0, 1)
        inv = self._inverse_label_count(kwargs).reshape(())
        doc = self._token_slice(kwargs[LanguageModelKwargs.document_index], rows, 0, 1).long()
        valid = (labels >= 0).float()
        segments = kwargs.get("_num_documents")
        if segments is None:
            full = kwargs[LanguageModelKwargs.document_index]
            segments = kwargs["_num_documents"] = int(full.max().item()) + 1 if full.numel() else 0
        log_ratio = (_label_log_probs(lse, target, labels) - old) * valid
        sums = torch.zeros(3, segments, device=lse.device).index_add(1, doc, torch.stack([log_ratio, valid, adv * valid]))
        local_count = sums[1].detach()
        if self._sequence_parallel and self._tp_group is not None:
            sums = _SumOverRanks.apply(sums, self._tp_group)
        if self._sdp_group is not None:
            sums = _SumOverRanks.apply(sums, self._sdp_group)
        count = sums[1].clamp(min=1.0)
        ratio, advantage = torch.exp(sums[0] / count), sums[2] / count
        per_document = self._surrogate(ratio, advantage)
        # the gradient of the job-wide loss wrt this rank's tokens needs the whole document's weight; the value reported
        # by this rank counts its own tokens only (the ranks' values are summed afterwards)
        for_gradient = (per_document * sums[1].detach()).sum() * inv
        reported = (per_document.detach() * local_count).sum() * inv
        return for_gradient + (reported - for_gradient).detach()


class MonolithicLoss(LanguageModelLoss):
    """Several losses over one shared softmax: the label-based members (cross-entropy, z-loss, GRPO, GSPO, DPO) share one
    statistics pass, their per-token coefficients are added up and ONE pass writes the gradient of their weighted sum.
    Members of another family (distillation) run their own two passes and accumulate into the same gradient."""

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
        return [d for m in self._members for d in m.get_loss_definitions(count)]

    def get_preprocessing_config(self, phase):
        out = {}
        for m in self._members:
            for key, value in m.get_preprocessing_config(phase).items():
                out[key] = (out[key] | value) if isinstance(value, set) and key in out else value
        return out

    def forward_backward(self, logits, kwargs, grad_output, split_index, num_splits, logits_scale, accumulate_into=None):
        rows = logits.shape[0]
        sub_grad_output = None if grad_output is None else grad_output * self.weight
        shared = [m for m in self._members if isinstance(m, LabelBasedLoss) and not
                  (isinstance(m, LabelEntropyLoss) and m._config.loss_type == EntropyLossType.reverse_kl)]
        # members sharing the softmax must agree on the scale of the logits: group them by it
        by_scale: dict[float, list] = {}
        for m in shared:
            by_scale.setdefault(m._scale(logits_scale), []).append(m)
        others = [m for m in self._members if m not in shared]
        total, grad = None, accumulate_into
        passes = len(others) + len(by_scale)
        kwargs["_logits_columns"] = logits.shape[-1]
        for m in others:
            kwargs["_single_loss"] = False
            value, grad = m.forward_backward(logits, kwargs, sub_grad_output, split_index, num_splits, logits_scale, accumulate_into=grad)
            if grad is None and sub_grad_output is not None and passes > 1:
                pass
            total = value * m.weight if total is None else total + value * m.weight
            self._record(kwargs, m, value)
        remaining = len(by_scale)
        for scale, members in by_scale.items():
            remaining -= 1
            labels = self._labels(kwargs, rows, split_index, num_splits)
            stats = softmax_statistics(logits, labels, scale, self._group, self._vocab_begin)
            kwargs["_logits_scale"] = scale
            a_sum = b_sum = None
            for m in members:
                value, a, b = m.coefficients(stats, labels, kwargs, rows, split_index, num_splits, sub_grad_output)
                value = m._finalize(value.reshape(1)).reshape(())
                total = value * m.weight if total is None else total + value * m.weight
                self._record(kwargs, m, value)
                if a is not None:
                    a_sum = a if a_sum is None else a_sum + a
                    b_sum = b if b_sum is None else b_sum + b
            if a_sum is not None:
                # the last pass may overwrite the logits when nothing has been accumulated before it
                in_place = grad is None and remaining == 0 and kwargs.get("_single_loss", True) is not False
                if grad is None and not in_place:
                    grad = softmax_coeff_grad(logits, labels, stats, a_sum, b_sum, in_place=False)
                else:
                    grad = softmax_coeff_grad(logits, labels, stats, a_sum, b_sum, accumulate_into=grad, in_place=in_place)
        kwargs.pop("_single_loss", None)
        return total, grad

    @staticmethod
    def _record(kwargs, member, value):
        sink = kwargs.get("_member_losses")
        if sink is not None:
            sink.setdefault(member.name, []).append(value.detach())
