"""A stage: consecutive layers that share weight/gradient buffers and run as one forward / backward unit.

Parity: `fast_llm/engine/multi_stage/stage_base.py:22-363`, `stage.py:32-270`.
"""

import logging

import torch

from fast_llm_b200.engine.base_model import Layer
from fast_llm_b200.engine.multi_stage.config import StageConfig, StageMode
from fast_llm_b200.engine.multi_stage.fsdp import FSDP
from fast_llm_b200.parallel.topology import DistributedConfig
from fast_llm_b200.tensor import ParameterMeta
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


def reorder_parameter_metas(metas: list[ParameterMeta]) -> list[ParameterMeta]:
    """Stable sort that groups (no-decay | decay) and, inside each, tensor-parallel and sequence-parallel parameters,
    so optimizer groups and the sequence-parallel gradient all-reduce each cover one contiguous slice."""

    def key(i):
        wd = bool(metas[i].param_weight_decay)
        return (wd, wd == metas[i].is_tensor_parallel, wd != metas[i].sequence_tensor_parallel)

    return [metas[i] for i in sorted(range(len(metas)), key=key)]


class Stage:
    def __init__(self, *, config: StageConfig, layers: list[Layer], distributed_config: DistributedConfig, index: int,
                 begin: int, end: int, tied_duplicates: set[str] = frozenset()):
        self._config = config
        self._layers = layers
        self._distributed_config = distributed_config
        self._index = index
        self._begin, self._end = begin, end
        self._is_setup = False
        self._mode = StageMode.off_device
        trainable, frozen, duplicates = [], [], []
        for layer in layers:
            for name, meta in layer.named_parameter_metas():
                if meta.tensor_name in tied_duplicates:
                    duplicates.append(meta)
                elif meta.requires_grad:
                    trainable.append(meta)
                else:
                    frozen.append(meta)
        self._duplicate_metas = duplicates
        self._fsdps: list[FSDP] = []
        if trainable:
            self._fsdps.append(FSDP(f"stage_{index}", reorder_parameter_metas(trainable), distributed_config,
                                    full_precision_gradient_buffer=config.full_precision_gradients, full_precision_shards=True))
        if frozen:
            self._fsdps.append(FSDP(f"stage_{index}_frozen", reorder_parameter_metas(frozen), distributed_config,
                                    full_precision_gradient_buffer=False,
                                    full_precision_shards=config.store_frozen_weights_in_optimization_precision))
        self._weight_buffer_index = None
        self._grad_buffer_index = None
        self._weights_valid = False
        self._buffer_registry = None

    @property
    def index(self) -> int:
        return self._index

    @property
    def layers(self) -> list[Layer]:
        return self._layers

    @property
    def fsdps(self) -> list[FSDP]:
        return self._fsdps

    @property
    def mode(self):
        return self._mode

    @property
    def parameter_count(self) -> int:
        return sum(f.parameter_count for f in self._fsdps)

    @property
    def parameter_names(self) -> list[str]:
        return [n for f in self._fsdps for n in f.parameter_names]

    def get_parameter_meta(self, name: str) -> ParameterMeta:
        for f in self._fsdps:
            if name in f:
                return f.get_parameter_meta(name)
        raise KeyError(name)

    def setup(self, *, distributed, mode: StageMode, weight_shards, grad_shards, weight_buffers, grad_buffers,
              buffer_registry: dict | None = None, weight_buffer_index=None, grad_buffer_index=None) -> None:
        assert not self._is_setup
        self._is_setup = True
        self._mode = mode
        self._distributed = distributed
        self._buffer_registry = buffer_registry if buffer_registry is not None else {}
        self._weight_buffer_index = weight_buffer_index
        self._grad_buffer_index = grad_buffer_index
        for layer in self._layers:
            if not layer._is_setup:
                layer.setup(distributed)
        for i, fsdp in enumerate(self._fsdps):
            fsdp.setup(mode, weight_shards[i], grad_shards[i], weight_buffers[i], grad_buffers[i],
                       fsdp_group=distributed.data_group, tensor_group=distributed.tensor_group)

    # ---- weights
    def initialize_weights(self) -> None:
        for fsdp in self._fsdps:
            fsdp.initialize_weights(self._distributed)
        self.invalidate_buffer()

    def restore_parameters(self) -> None:
        """Make the weight buffer hold this stage's current weights (no-op when already valid)."""
        if not self._mode.support_forward:
            return
        key = ("weight", self._weight_buffer_index)
        if self._weights_valid and self._buffer_registry.get(key, self._index) == self._index:
            return
        for fsdp in self._fsdps:
            fsdp.restore_parameters()
        self._weights_valid = True
        self._buffer_registry[key] = self._index

    def invalidate_buffer(self) -> None:
        self._weights_valid = False

    @property
    def weight_buffer_index(self):
        """Identity of the weight buffer this stage computes from (shared round-robin between stages under ZeRO-3)."""
        return self._weight_buffer_index

    @property
    def grad_buffer_index(self):
        return self._grad_buffer_index

    @property
    def is_restored(self) -> bool:
        return self._weights_valid and self._buffer_registry.get(("weight", self._weight_buffer_index), self._index) == self._index

    # ---- gradients
    def reset_gradients(self) -> None:
        for fsdp in self._fsdps:
            fsdp.reset_gradients()

    def reduce_gradients(self, accumulate: bool = False, allow_no_grad: bool = False) -> None:
        for fsdp in self._fsdps:
            fsdp.reduce_gradients(accumulate, allow_no_grad)

    # ---- compute
    def forward(self, input_, kwargs: dict, losses: dict | None = None, metrics: dict | None = None):
        """Returns (detached output, context for `backward`)."""
        assert self._mode.support_forward
        assert self.is_restored, f"Stage {self._index}: weights not restored"
        training = self._mode.support_backward and kwargs.get("training", True)
        if training and torch.is_tensor(input_) and input_.is_floating_point():
            input_ = input_.detach().requires_grad_()
        with torch.set_grad_enabled(training):
            output = input_
            for layer in self._layers:
                output = layer.forward(output, kwargs, losses, metrics)
                name = getattr(layer, "module_name", type(layer).__name__)
                if (self._config.debug_layer_outputs or self._config.debug_layer_gradients) and torch.is_tensor(output):
                    self._log_layer(output, name, kwargs, training)
                if self._config.debug_tensor_parallel:
                    self._check_replicated(output, name, training)
                if self._config.debug_activation_memory:
                    self._log_activation_memory(name)
        return (output.detach() if torch.is_tensor(output) else output), (input_, output)

    def _log_layer(self, output: torch.Tensor, name: str, kwargs: dict, training: bool) -> None:
        """`debug_layer_outputs` / `debug_layer_gradients`: one record per layer output (and per gradient reaching it), with
        the micro-batch and micro-sequence in the name.  Block outputs are replicated over the tensor group, or sharded by
        tokens over it with sequence parallelism; with `debug_global_tensors` the whole tensor is logged once, so the records
        of different layouts line up (parity: `fast_llm/engine/multi_stage/stage.py:216-232,249-263`)."""
        from fast_llm_b200.utils.tensor_logs import log_distributed_grad, log_distributed_tensor

        if (count := kwargs.get("num_micro_batches", 1)) > 1:
            name = f"{name}, mb={kwargs.get('micro_batch', 0)}/{count}"
        if (count := kwargs.get("micro_batch_splits", 1)) > 1:
            name = f"{name}, ms={kwargs.get('micro_batch_split', 0)}/{count}"
        group = getattr(self._distributed, "tensor_group", None)
        sharded = group is not None and self._distributed.config.sequence_tensor_parallel and output.dim() == 2 and output.is_floating_point()
        layout = dict(shard_group=group if sharded else None, shard_dim=0, duplicate_groups=() if sharded else (group,),
                      global_=self._config.debug_global_tensors)
        if self._config.debug_layer_outputs:
            log_distributed_tensor(f"{name} fw", output, level=self._config.debug_layer_outputs, **layout)
        if self._config.debug_layer_gradients and training and output.requires_grad:
            log_distributed_grad(f"{name} bw", output, level=self._config.debug_layer_gradients, **layout)

    def _check_replicated(self, output, name: str, training: bool) -> None:
        """`debug_tensor_parallel`: a layer output that every rank of the tensor group holds in full (no sequence
        parallelism) must be bit-identical on all of them, and so must its gradient (parity:
        `fast_llm/engine/multi_stage/stage.py:209-215,239-248`).  A mismatch is logged, training goes on."""
        from fast_llm_b200.parallel.collectives import check_parallel_match

        group = getattr(self._distributed, "tensor_group", None)
        if group is None or self._distributed.config.sequence_tensor_parallel or not torch.is_tensor(output) or not output.is_floating_point():
            return
        check_parallel_match(output.detach(), group, f"layer {name} fw")
        if training and output.requires_grad:
            output.register_hook(lambda grad: check_parallel_match(grad, group, f"layer {name} bw") and None)

    def _log_activation_memory(self, name: str) -> None:
        """`debug_activation_memory`: allocator state after every layer of the forward pass, on the first rank of each pipeline
        stage group (parity: `fast_llm/engine/multi_stage/stage.py:233-234`)."""
        config = self._distributed.config
        if config.data_rank or config.tensor_rank:
            return
        if torch.cuda.is_available() and self._distributed.device.type == "cuda":
            mib = 2**20
            logger.info(f"layer {name} fw: allocated {torch.cuda.memory_allocated() / mib:,.2f} MiB | max allocated "
                        f"{torch.cuda.max_memory_allocated() / mib:,.2f} MiB | reserved {torch.cuda.memory_reserved() / mib:,.2f} MiB")
        else:
            import resource

            logger.info(f"layer {name} fw: host peak resident set {resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1024:,.2f} MiB")

    def backward(self, output_grad, context) -> torch.Tensor | None:
        assert self._mode.support_backward
        input_, output = context
        if output.requires_grad:
            output.backward(output_grad)
        if torch.is_tensor(input_) and input_.is_floating_point() and input_.requires_grad:
            grad = input_.grad
            input_.grad = None
            return grad
        return None

    def get_param_groups(self, optimizer_state_shards: dict[str, list[torch.Tensor]]):
        """One optimizer group per contiguous run of parameters with equal (weight_decay, lr_scale), as shard slices."""
        groups = []
        for i, fsdp in enumerate(self._fsdps):
            if not fsdp.requires_grad:
                continue
            current = None
            for name in fsdp.parameter_names:
                meta = fsdp.get_parameter_meta(name)
                begin, end = fsdp.parameter_range_in_shard(name)
                if end <= begin:
                    continue
                lr_scales = meta.lr_scale
                chunks = len(lr_scales)
                # per-chunk lr scales split the parameter evenly along its flattened form
                piece = meta.numel() // chunks
                pbegin = fsdp.get_parameter_begin_in_buffer(name) - fsdp._fsdp_dim.rank * fsdp.shard_size
                for c, lr_scale in enumerate(lr_scales):
                    cb = min(max(pbegin + c * piece, 0), fsdp.shard_size)
                    ce = min(max(pbegin + (c + 1) * piece if c < chunks - 1 else pbegin + meta.numel(), 0), fsdp.shard_size)
                    if ce <= cb:
                        continue
                    key = (bool(meta.param_weight_decay), lr_scale)  # None: the optimizer's default_learning_rate_scale applies
                    if current is not None and current["key"] == key and current["end"] == cb:
                        current["end"] = ce
                        current["names"].append(name)
                    else:
                        current = {"key": key, "begin": cb, "end": ce, "fsdp": i, "names": [name]}
                        groups.append(current)
        out = []
        for g in groups:
            sl = slice(g["begin"], g["end"])
            out.append({
                "name": f"stage_{self._index}_{g['names'][0]}..{g['names'][-1]}",
                "stage": self._index,
                "weight_decay": g["key"][0],
                "lr_scale": g["key"][1],
                "params": self._fsdps[g["fsdp"]].weight_shard[sl],
                "grads": self._fsdps[g["fsdp"]].grad_shard[sl],
                "buffer": self._fsdps[g["fsdp"]]._weight_buffer_local_shard[sl] if self._mode.support_forward else None,
                **{k: v[g["fsdp"]][sl] for k, v in optimizer_state_shards.items()},
            })
        return out

    def get_grad_norm_slices(self) -> list[torch.Tensor]:
        """Gradient shard slices that count towards the global norm on this rank (replicated parameters are counted
        by tensor rank 0 only)."""
        out = []
        tensor_rank = self._distributed_config.tensor_rank
        for fsdp in self._fsdps:
            if not fsdp.requires_grad:
                continue
            begin = end = None
            for name in fsdp.parameter_names:
                meta = fsdp.get_parameter_meta(name)
                b, e = fsdp.parameter_range_in_shard(name)
                counted = meta.is_tensor_parallel or tensor_rank == 0
                if counted and e > b:
                    if end == b:
                        end = e
                    else:
                        if begin is not None and end > begin:
                            out.append(fsdp.grad_shard[begin:end])
                        begin, end = b, e
            if begin is not None and end > begin:
                out.append(fsdp.grad_shard[begin:end])
        return out
