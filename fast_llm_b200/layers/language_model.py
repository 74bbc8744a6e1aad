"""Language-model embeddings, head (+ losses) and the top-level language-model config.

Parity: `fast_llm/layers/language_model/config.py:40-330`, `embedding.py:19-181`, `head.py:42-303`.
The head computes the logits, the loss AND the gradients of its inputs inside `forward` (the `[tokens, vocab]` logits
are overwritten by their gradient and never leave the head); the stage's backward then only carries the stashed
input gradient further.
"""

import enum

import torch

from fast_llm_b200.config import Field, FieldHint, check_field, config_class, skip_valid_if_none
from fast_llm_b200.engine.base_model import Layer, LossDef
from fast_llm_b200.engine.initialization import init_normal_
from fast_llm_b200.engine.parameter import OptionalParameterConfig, ParameterConfig, combine_lr_scales
from fast_llm_b200.layers.block import BlockSequenceConfig
from fast_llm_b200.layers.kwargs import LanguageModelKwargs
from fast_llm_b200.layers.losses import LanguageModelLossConfig, LanguageModelLabelEntropyLossConfig
from fast_llm_b200.layers.mixer import BlockConfig
from fast_llm_b200.layers.normalization import NormalizationConfig
from fast_llm_b200.ops.gemm import matmul_nn, matmul_nt
from fast_llm_b200.ops.linear import weight_grad
from fast_llm_b200.ops.pointwise import embedding
from fast_llm_b200.parallel import fused_tp
from fast_llm_b200.parallel.ops import gather, gather_op, reduce_forward, reduce_op, reduce_scatter_op, split_op
from fast_llm_b200.parallel.topology import DistributedDimNames
from fast_llm_b200.tensor import TensorDim
from fast_llm_b200.utils import Assert, div


class LossImplementation(str, enum.Enum):
    """`per_loss` runs every loss on its own; the other values group the losses that share the softmax (the reference's
    `compiled` / `triton` choose between its two fused implementations, here both mean the CUDA kernels)."""

    auto = "auto"
    per_loss = "per_loss"
    compiled = "compiled"
    triton = "triton"


@config_class()
class LanguageModelEmbeddingsConfig(BlockConfig):
    _abstract = False
    word_embeddings: ParameterConfig = Field(desc="Token embedding table.", hint=FieldHint.architecture)
    position_embeddings: OptionalParameterConfig = Field(desc="Learned absolute position embeddings (off by default).", hint=FieldHint.architecture)
    vocab_size: int = Field(default=49152, desc="Vocabulary size.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    num_position_embeddings: int = Field(default=2048, desc="Number of absolute positions.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    dropout: float = Field(default=0.0, desc="Dropout after the embedding.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))
    full_precision_residual: bool = Field(default=False, desc="Keep the residual stream in the optimization dtype.", hint=FieldHint.stability)
    vocab_parallel: bool = Field(default=True, desc="Split the vocabulary over the tensor group.", hint=FieldHint.performance)
    embedding_scale: float = Field(default=1.0, desc="Multiplier of the token embeddings.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))

    def get_layer(self, distributed_config, hidden_dim, *, lr_scale=None, peft=None):
        return LanguageModelEmbedding(self, distributed_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft)


@config_class()
class LanguageModelHeadConfig(BlockConfig):
    _abstract = False
    normalization: NormalizationConfig = Field(desc="Final normalization.", hint=FieldHint.architecture)
    losses: dict[str, LanguageModelLossConfig] = Field(default_factory=dict, desc="Named losses (default: cross-entropy from labels).", hint=FieldHint.core)
    loss_implementation: LossImplementation = Field(default=LossImplementation.auto, desc="`per_loss`: one pass pair per loss; otherwise losses sharing the softmax are fused into one pass pair.", hint=FieldHint.expert)
    output_weight: ParameterConfig = Field(desc="Output projection (unless tied to the embeddings).", hint=FieldHint.architecture)
    cross_entropy_splits: int = Field(default=1, desc="Process the logits in this many token chunks to bound memory.", hint=FieldHint.feature, valid=skip_valid_if_none(check_field(Assert.gt, 0)))
    logits_scale_factor: float = Field(default=1.0, desc="Multiplier of the logits.", hint=FieldHint.feature, valid=check_field(Assert.geq, 0))
    final_logit_softcap: float | None = Field(default=None, desc="Soft cap: cap * tanh(logits / cap).", hint=FieldHint.architecture, valid=skip_valid_if_none(check_field(Assert.gt, 0)))
    prediction_heads: int = Field(default=1, desc="Number of multi-token-prediction heads.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))
    prediction_loss_coefficient: list[float] | None = Field(default=None, desc="Loss weight of each prediction head.", hint=FieldHint.feature)

    def _validate(self):
        super()._validate()
        if self.prediction_loss_coefficient is not None:
            Assert.eq(len(self.prediction_loss_coefficient), self.prediction_heads)

    def get_layer(self, distributed_config, embeddings_config, hidden_dim, *, lr_scale=None, peft=None, prediction_distance: int = 1,
                  loss_coefficient: float = 1.0):
        return LanguageModelHead(self, distributed_config, embeddings_config, hidden_dim=hidden_dim, lr_scale=lr_scale, peft=peft,
                                 prediction_distance=prediction_distance, loss_coefficient=loss_coefficient)


@config_class()
class LanguageModelConfig(BlockConfig):
    decoder: BlockSequenceConfig = Field(desc="The decoder blocks.", hint=FieldHint.architecture)
    embeddings: LanguageModelEmbeddingsConfig = Field(desc="Input embeddings.", hint=FieldHint.architecture)
    head: LanguageModelHeadConfig = Field(desc="Output head and losses.", hint=FieldHint.architecture)
    tied_embedding_weight: bool = Field(default=False, desc="Use the embedding table as output projection.", hint=FieldHint.architecture)
    hidden_size: int = Field(default=1024, desc="Model width.", hint=FieldHint.architecture, valid=check_field(Assert.gt, 0))


class LanguageModelEmbedding(Layer):
    layer_count = 1000.0  # always a stage of its own, as in the reference (`embedding.py:27`)

    def __init__(self, config: LanguageModelEmbeddingsConfig, distributed_config, *, hidden_dim, lr_scale=None, peft=None):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self._hidden_dim = hidden_dim
        tp_dim = distributed_config.get_distributed_dim(DistributedDimNames.tensor)
        self._tp_dim = tp_dim
        self._sequence_parallel = distributed_config.sequence_tensor_parallel
        self._vocab_parallel = config.vocab_parallel and tp_dim.size > 1
        self._residual_dtype = (distributed_config.optimization_dtype if config.full_precision_residual else distributed_config.compute_dtype).torch
        vocab_dim = TensorDim("vocab", config.vocab_size, tp_dim if self._vocab_parallel else None)
        if self._vocab_parallel:
            self._vocab_begin = tp_dim.rank * vocab_dim.size
            self._vocab_end = self._vocab_begin + vocab_dim.size
        else:
            self._vocab_begin, self._vocab_end = 0, config.vocab_size
        self.word_embeddings_weight = config.word_embeddings.get_parameter(
            (vocab_dim, hidden_dim), default_initialization=init_normal_(0.0, hidden_dim.global_size**-0.5), lr_scale=self._lr_scale, peft=peft)
        pos = config.position_embeddings.get_parameter(
            (TensorDim("position_embeddings", config.num_position_embeddings), hidden_dim),
            default_initialization=init_normal_(0.0, hidden_dim.global_size**-0.5), lr_scale=self._lr_scale,
            allow_sequence_tensor_parallel=not config.vocab_parallel, peft=peft)
        if pos is not None:
            self.position_embeddings_weight = pos
        self._has_position_embeddings = pos is not None

    def forward(self, input_, kwargs, losses=None, metrics=None):
        """input_: token ids [tokens] (full micro-sequence); output [tokens(/tp under SP), hidden]."""
        c = self._config
        group = self._tp_dim.group if self._tp_dim.size > 1 else None
        ids = kwargs.get(LanguageModelKwargs.token_ids, input_)
        if torch.is_floating_point(ids):
            ids = input_
        # negative ids (image placeholders, padding) embed to zero; always checked when encoder outputs are merged in, so that
        # a patch's embedding replaces its placeholder instead of being added to some token's embedding
        mask_inputs = kwargs.get(LanguageModelKwargs.mask_inputs, False) or kwargs.get(LanguageModelKwargs.embedding_map) is not None
        if mask_inputs:
            token_mask = ids >= 0
            ids = ids * token_mask
        if self._vocab_parallel:
            out = embedding(ids, self.word_embeddings_weight, self._vocab_begin, self._vocab_end, c.embedding_scale)
            if self._has_position_embeddings:
                pos_ids = kwargs[LanguageModelKwargs.position_ids]
                # add the (replicated) position embedding once: on the first tensor rank
                if self._tp_dim.rank == 0:
                    out = out + torch.nn.functional.embedding(pos_ids.long(), self.position_embeddings_weight)
            out = _reduce_embedding(out, group, self._sequence_parallel)
        else:
            if self._sequence_parallel and group is not None:
                ids = split_op(ids, group, 0)
            out = embedding(ids, self.word_embeddings_weight, 0, c.vocab_size, c.embedding_scale)
            if self._has_position_embeddings:
                pos_ids = kwargs[LanguageModelKwargs.position_ids]
                if self._sequence_parallel and group is not None:
                    pos_ids = split_op(pos_ids, group, 0)
                out = out + torch.nn.functional.embedding(pos_ids.long(), self.position_embeddings_weight)
        if mask_inputs:
            m = token_mask if out.shape[0] == token_mask.shape[0] else split_op(token_mask, group, 0)
            out = out * m.unsqueeze(-1)
        emb_map = kwargs.get(LanguageModelKwargs.embedding_map)
        if emb_map is not None:
            # multimodal: add encoder outputs (input_) at the mapped token positions
            src_index, dst_index = emb_map
            features = input_
            if self._sequence_parallel and group is not None:
                # every rank holds a share of the encoder outputs and a share of the tokens: gather the former (their
                # gradients are summed back to the owners) and keep the pairs whose token lies in this rank's range
                features = gather(features, group, 0, reduce_grads=True)
                dst_index = dst_index - self._tp_dim.rank * out.shape[0]
                local = (dst_index >= 0) & (dst_index < out.shape[0])
                src_index, dst_index = src_index[local], dst_index[local]
            out = out.index_add(0, dst_index, features[src_index].to(out.dtype))
        if c.dropout > 0 and kwargs.get("training", True):
            from fast_llm_b200.parallel.collectives import set_generator

            with set_generator(self._distributed.tp_generator if self._sequence_parallel else self._distributed.pp_generator):
                out = torch.dropout(out, c.dropout, True)
        return out.to(self._residual_dtype)

    def get_compute_usage(self, input_meta, kwargs, config=None):
        return 0


class _ReduceEmbedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sequence_parallel):
        ctx.group, ctx.sp = group, sequence_parallel
        return reduce_scatter_op(x, group, dim=0) if sequence_parallel else reduce_op(x.clone(), group)

    @staticmethod
    def backward(ctx, grad):
        return (gather_op(grad.contiguous(), ctx.group, 0) if ctx.sp else grad), None, None


def _reduce_embedding(x, group, sequence_parallel):
    return x if group is None else _ReduceEmbedding.apply(x, group, sequence_parallel)


class _HeadLoss(torch.autograd.Function):
    """logits = x W^T -> losses -> d logits -> (dx, dW), all in forward; backward hands dx on."""

    @staticmethod
    def forward(ctx, x, weight, head, kwargs, losses_out, split_index, num_splits, gathered=False):
        x2 = x.detach()
        group = head._logits_group
        logits = None
        if gathered:
            x_full = x2  # the caller gathered the token shards (and reduce-scatters the gradient)
        elif head._sequence_parallel_logits_gather and group is not None:
            x_full = None
            fused = fused_tp.usable(group, True, x2, weight)
            if fused is not None and fused.single_launch and fused.fits(x2.shape[0] * group.size(), x2.shape[1]):
                # the token shards arrive inside the logits GEMM (peers push, the GEMM waits per row block)
                logits, x_full = fused.all_gather_matmul(x2, weight, False, return_gathered=True)
            else:
                x_full = gather_op(x2, group, 0)
        else:
            x_full = x2
        if logits is None:
            logits = matmul_nt(x_full, weight)
        c = head._config
        scale = c.logits_scale_factor
        softcap_state = None
        if c.final_logit_softcap is not None:
            lf = logits.float() * (scale / c.final_logit_softcap)
            th = torch.tanh(lf)
            softcap_state = th
            logits = (th * c.final_logit_softcap).to(logits.dtype)
            scale = 1.0
        total, grad_logits = head._loss_forward_backward(logits, kwargs, losses_out, split_index, num_splits, scale)
        dx = None
        if grad_logits is not None:
            if softcap_state is not None:
                grad_logits = (grad_logits.float() * (1 - softcap_state * softcap_state) * c.logits_scale_factor).to(grad_logits.dtype)
            fused = fused_tp.usable(group, True, grad_logits, weight) if (head._sequence_parallel_logits_gather and not gathered) else None
            use_fused = fused is not None and fused.fits(grad_logits.shape[0], weight.shape[1])
            if use_fused:
                # partial input gradients leave for their owners from the GEMM's epilogue
                dx = fused.matmul_reduce_scatter(grad_logits, weight, True)
            else:
                dx = matmul_nn(grad_logits, weight)
            if group is not None and not gathered and not use_fused:
                if head._sequence_parallel_logits_gather:
                    dx = reduce_scatter_op(dx, group, dim=0)
                elif head._vocab_parallel:
                    dx = reduce_op(dx, group)
            weight_grad(grad_logits, x_full, weight, transposed_weight=False)
        ctx.save_for_backward(dx)
        return total

    @staticmethod
    def backward(ctx, grad_loss):
        (dx,) = ctx.saved_tensors
        return dx, None, None, None, None, None, None, None


class LanguageModelHead(Layer):
    def __init__(self, config: LanguageModelHeadConfig, distributed_config, embeddings_config, *, hidden_dim, lr_scale=None,
                 peft=None, prediction_distance: int = 1, loss_coefficient: float = 1.0):
        super().__init__(config, distributed_config, lr_scale=combine_lr_scales(lr_scale, config.lr_scale), peft=peft)
        self._hidden_dim = hidden_dim
        self._prediction_distance = prediction_distance
        self._loss_coefficient = loss_coefficient
        tp_dim = distributed_config.get_distributed_dim(DistributedDimNames.tensor)
        self._tp_dim = tp_dim
        self._vocab_parallel = embeddings_config.vocab_parallel and tp_dim.size > 1
        self._sequence_parallel = distributed_config.sequence_tensor_parallel
        # vocab-parallel logits need every token on every rank; sequence-parallel logits keep token shards
        self._sequence_parallel_logits_gather = self._sequence_parallel and self._vocab_parallel
        self._vocab_size = embeddings_config.vocab_size
        vocab_dim = TensorDim("vocab", embeddings_config.vocab_size, tp_dim if self._vocab_parallel else None)
        self._vocab_begin = tp_dim.rank * vocab_dim.size if self._vocab_parallel else 0
        self.final_norm = config.normalization.get_layer(hidden_dim, lr_scale=self._lr_scale, peft=peft, distributed_config=distributed_config)
        self.output_weights = config.output_weight.get_parameter(
            (vocab_dim, hidden_dim), default_initialization=init_normal_(0.0, hidden_dim.global_size**-0.5), lr_scale=self._lr_scale, peft=peft)
        loss_configs = self._effective_losses(config)
        suffix = "" if prediction_distance == 1 else f"_{prediction_distance}"
        self._losses = [
            lc.get_layer(distributed_config, name=name + suffix, prediction_distance=prediction_distance, vocab_parallel=self._vocab_parallel,
                         weight=lc.weight * loss_coefficient)
            for name, lc in loss_configs.items()
        ]
        self._logits_group = None

    @staticmethod
    def _effective_losses(config) -> dict:
        """The losses the head runs.  Losses that share the softmax over the vocabulary are grouped, by logits scale, into
        one `MonolithicLoss` each, so that a group costs one statistics pass and one gradient pass over the logits however
        many members it has (`loss_implementation: per_loss` keeps them apart).  Grouping rule and the reserved names
        `monolithic` / `monolithic_<i>`: `fast_llm/layers/language_model/config.py:203-237`."""
        from fast_llm_b200.layers.losses import CombinableLossConfig, MonolithicLossConfig

        losses = dict(config.losses) or {"lm_loss": LanguageModelLabelEntropyLossConfig()}
        for name in losses:
            assert not (name == "monolithic" or (name.startswith("monolithic_") and name.removeprefix("monolithic_").isdigit())), \
                f"loss name {name!r} is reserved"
        combinable = {n: c for n, c in losses.items() if isinstance(c, CombinableLossConfig)}
        if config.loss_implementation == LossImplementation.per_loss or len(combinable) < 2:
            return losses
        groups: dict[float, dict] = {}
        slots = []
        for name, loss in losses.items():
            if name in combinable:
                if loss.logits_scale_factor not in groups:
                    groups[loss.logits_scale_factor] = {}
                    slots.append(loss.logits_scale_factor)
                groups[loss.logits_scale_factor][name] = loss
            else:
                slots.append((name, loss))
        effective, index = {}, 0
        for slot in slots:
            if isinstance(slot, tuple):
                effective[slot[0]] = slot[1]
            elif len(groups[slot]) == 1:
                effective.update(groups[slot])
            else:
                group = MonolithicLossConfig(losses=groups[slot])
                group.validate()
                effective[f"monolithic_{index}" if len(groups) > 1 else "monolithic"] = group
                index += 1
        return effective

    def setup(self, distributed):
        super().setup(distributed)
        self._logits_group = self._tp_dim.group if (self._vocab_parallel and self._tp_dim.size > 1) else None
        for loss in self._losses:
            loss.setup(distributed, self._logits_group, self._vocab_begin)

    def get_loss_definitions(self, count: int = 1):
        out = []
        for loss in self._losses:
            out += loss.get_loss_definitions(count)
        return out

    def get_preprocessing_config(self, phase):
        out = {}
        for loss in self._losses:
            out.update(loss.get_preprocessing_config(phase))
        return out

    def forward(self, input_, kwargs, losses=None, metrics=None):
        if input_.dim() == 3 and input_.shape[0] == 2:
            # multi-token prediction: (shared trunk output, this head's block output)
            input_ = input_[1]
        hidden = self.final_norm(input_)
        if kwargs.get("return_logits", False) or LanguageModelKwargs.labels not in kwargs and not any(l.needs_reference for l in self._losses):
            return self._logits_only(hidden, kwargs)
        splits = self._config.cross_entropy_splits or 1
        loss_dict = losses if losses is not None else {}
        if splits == 1:
            total = _HeadLoss.apply(hidden, self.output_weights, self, kwargs, loss_dict, 0, 1)
        else:
            total = None
            # Vocab-parallel logits of token shards: gather the (small) hidden states once, so that chunk i holds the same
            # contiguous tokens as chunk i of the labels; the gather's backward reduce-scatters the summed chunk gradients.
            gathered = self._sequence_parallel_logits_gather and self._logits_group is not None
            if gathered:
                from fast_llm_b200.parallel.ops import gather

                hidden = gather(hidden, self._logits_group, 0, reduce_grads=True)
            for i, chunk in enumerate(hidden.chunk(splits, dim=0)):
                part = _HeadLoss.apply(chunk, self.output_weights, self, kwargs, loss_dict, i, splits, gathered)
                total = part if total is None else total + part
        return total

    def _logits_only(self, hidden, kwargs):
        group = self._logits_group
        x = gather_op(hidden, group, 0) if (self._sequence_parallel_logits_gather and group is not None) else hidden
        logits = matmul_nt(x.detach(), self.output_weights.detach()).float() * self._config.logits_scale_factor
        if self._config.final_logit_softcap is not None:
            cap = self._config.final_logit_softcap
            logits = torch.tanh(logits / cap) * cap
        if group is not None:
            logits = gather_op(logits, group, dim=1)
        kwargs["logits"] = logits
        return logits

    def _loss_forward_backward(self, logits, kwargs, losses_out, split_index, num_splits, logits_scale):
        """Run every configured loss on one chunk of logits; returns (weighted total, grad wrt logits or None)."""
        training = kwargs.get("training", True)
        grad_output = kwargs.get(LanguageModelKwargs.grad_output, 1.0) if training else None
        total, grad = None, None
        kwargs["_single_loss"] = len(self._losses) == 1
        for loss in self._losses:
            members = kwargs["_member_losses"] = {}
            value, g = loss.forward_backward(logits, kwargs, grad_output, split_index, num_splits, logits_scale,
                                             accumulate_into=grad)
            kwargs.pop("_member_losses", None)
            if g is not None:
                grad = g
            # a group reports its members under their own names, a plain loss reports itself
            for name, entries in (members.items() if members else [(loss.name, [value.detach()])]):
                for entry in entries:
                    losses_out.setdefault(name, []).append(entry) if num_splits == 1 else _accumulate_split(losses_out, name, entry, split_index)
            weighted = value * loss.weight
            total = weighted if total is None else total + weighted
        if len(self._losses) > 1:
            _accumulate_split(losses_out, "lm_head_loss" + ("" if self._prediction_distance == 1 else f"_{self._prediction_distance}"), total.detach(), split_index) if num_splits > 1 else losses_out.setdefault(
                "lm_head_loss" + ("" if self._prediction_distance == 1 else f"_{self._prediction_distance}"), []).append(total.detach())
        return total, grad

    def get_compute_usage(self, input_meta, kwargs, config=None):
        tokens = kwargs[LanguageModelKwargs.num_tokens]
        return 2 * tokens * self._hidden_dim.global_size * self._vocab_size


def _accumulate_split(losses_out: dict, name: str, value: torch.Tensor, split_index: int) -> None:
    entries = losses_out.setdefault(name, [])
    if split_index == 0:
        entries.append(value)
    else:
        entries[-1] = entries[-1] + value
