"""Flat, padded, data-parallel-sharded storage of one stage's parameters (the ZeRO substrate).

Every stage packs its parameters, in a fixed order, into one flat buffer padded to `data_parallel * 32` elements:

    weight shard   [shard_size]        optimization dtype (fp32)  - this data rank's 1/dp slice: master weights
    optimizer state shards (same shape), gradient shard (same shape)
    weight buffer  [shard_size * dp]   compute dtype              - the full stage, rebuilt by all-gather
    grad buffer    [shard_size * dp]   fp32 or compute dtype      - backward accumulates here; reduce-scattered

Parameters are views of the weight buffer carrying a `grad_buffer` view.  The element layout (parameter order,
padding rule, shard boundaries) equals `fast_llm/engine/multi_stage/fsdp.py:23-444`, so `rank_*.safetensors` files are
interchangeable with the reference.  With one data rank and fp32 gradients the gradient shard *is* the gradient
buffer (no copy).
"""

import math
import typing

import torch

from fast_llm_b200.engine.multi_stage.config import SHARD_PAD_TO_MULTIPLE, StageMode
from fast_llm_b200.parallel.collectives import all_gather_into_tensor, all_reduce, reduce_scatter_tensor
from fast_llm_b200.parallel.topology import DistributedConfig, DistributedDimNames
from fast_llm_b200.tensor import ParameterMeta
from fast_llm_b200.utils import Assert, padded_cumsum


class FSDP:
    def __init__(self, name: str, parameter_metas: list[ParameterMeta], distributed_config: DistributedConfig,
                 full_precision_gradient_buffer: bool = False, full_precision_shards: bool = True,
                 is_tied_weight_copy: bool = False):
        self._name = name
        self._parameter_metas = {meta.tensor_name: meta for meta in parameter_metas}
        Assert.eq(len(self._parameter_metas), len(parameter_metas))
        self._distributed_config = distributed_config
        self._fsdp_dim = distributed_config.get_distributed_dim(DistributedDimNames.data)
        self._is_tied_weight_copy = is_tied_weight_copy
        self._requires_grad = any(meta.requires_grad for meta in parameter_metas)

        sizes = [meta.numel() for meta in parameter_metas]
        self._parameter_count = sum(sizes)
        offsets = padded_cumsum(sizes).tolist()
        self._parameter_begins_in_buffer = {m.tensor_name: o for m, o in zip(parameter_metas, offsets[:-1])}
        self._parameter_ends_in_buffer = {m.tensor_name: o for m, o in zip(parameter_metas, offsets[1:])}

        dp = self._fsdp_dim.size
        self._global_pad = -self._parameter_count % (dp * SHARD_PAD_TO_MULTIPLE)
        self._shard_size = (self._parameter_count + self._global_pad) // dp
        # padding normally sits in the last shard but may spill into earlier ones
        self._shard_pad = min(max(self._global_pad - self._shard_size * (dp - self._fsdp_dim.rank - 1), 0), self._shard_size)

        self._shard_dtype = (distributed_config.optimization_dtype if full_precision_shards else distributed_config.compute_dtype).torch
        self._weight_buffer_dtype = distributed_config.compute_dtype.torch
        self._grad_buffer_dtype = (distributed_config.optimization_dtype if full_precision_gradient_buffer else distributed_config.compute_dtype).torch
        self._grad_shard_size = self._shard_size if self._requires_grad else 0
        self._buffer_size = self._shard_size * dp
        self._grad_buffer_size = self._buffer_size if self._requires_grad else 0

        # contiguous range of parameters replicated over the tensor group but fed sequence-parallel activations
        sp = [m for m in parameter_metas if m.sequence_tensor_parallel and m.requires_grad] if distributed_config.sequence_tensor_parallel else []
        if sp:
            self._sp_begin = self._parameter_begins_in_buffer[sp[0].tensor_name]
            self._sp_end = self._parameter_ends_in_buffer[sp[-1].tensor_name]
            Assert.eq(self._sp_end - self._sp_begin, sum(m.numel() for m in sp), msg="sequence-parallel parameters must be contiguous")
        else:
            self._sp_begin = self._sp_end = 0
        self._mode = StageMode.off_device
        self._is_setup = False
        self._grad_shard_is_buffer = False
        self._weight_arena = self._grad_arena = None

    # ---- layout queries
    @property
    def name(self):
        return self._name

    @property
    def parameter_names(self) -> list[str]:
        return list(self._parameter_metas)

    @property
    def parameter_count(self) -> int:
        return self._parameter_count

    @property
    def shard_size(self) -> int:
        return self._shard_size

    @property
    def grad_shard_size(self) -> int:
        return self._grad_shard_size

    @property
    def buffer_size(self) -> int:
        return self._buffer_size

    @property
    def grad_buffer_size(self) -> int:
        return self._grad_buffer_size

    @property
    def shard_dtype(self):
        return self._shard_dtype

    @property
    def weight_buffer_dtype(self):
        return self._weight_buffer_dtype

    @property
    def grad_buffer_dtype(self):
        return self._grad_buffer_dtype

    @property
    def requires_grad(self) -> bool:
        return self._requires_grad

    @property
    def is_tied_weight_copy(self) -> bool:
        return self._is_tied_weight_copy

    @property
    def mode(self):
        return self._mode

    def __contains__(self, name: str) -> bool:
        return name in self._parameter_metas

    def get_parameter_meta(self, name: str) -> ParameterMeta:
        return self._parameter_metas[name]

    def get_parameter_begin_in_buffer(self, name: str) -> int:
        return self._parameter_begins_in_buffer[name]

    def get_parameter_end_in_buffer(self, name: str) -> int:
        return self._parameter_ends_in_buffer[name]

    def parameter_range_in_shard(self, name: str, rank: int | None = None) -> tuple[int, int]:
        """[begin, end) of the parameter's elements inside data rank `rank`'s shard (clipped; may be empty)."""
        rank = self._fsdp_dim.rank if rank is None else rank
        shard_begin = rank * self._shard_size
        begin = min(max(self._parameter_begins_in_buffer[name] - shard_begin, 0), self._shard_size)
        end = min(max(self._parameter_ends_in_buffer[name] - shard_begin, 0), self._shard_size)
        return begin, end

    def set_symmetric_arenas(self, weight_arena, grad_arena) -> None:
        """Buffers live in NVLink symmetric memory: reductions and weight updates use the fused peer-memory kernels."""
        self._weight_arena, self._grad_arena = weight_arena, grad_arena

    # ---- memory binding
    def setup(self, mode: StageMode, weight_shard: torch.Tensor | None, grad_shard: torch.Tensor | None,
              weight_buffer: torch.Tensor | None, grad_buffer: torch.Tensor | None, fsdp_group=None, tensor_group=None) -> None:
        assert not self._is_setup
        self._is_setup = True
        self._mode = mode
        self._fsdp_group = fsdp_group
        self._tensor_group = tensor_group
        self._weight_shard = weight_shard
        self._grad_shard = grad_shard
        self._weight_buffer = weight_buffer
        self._grad_buffer = grad_buffer
        if weight_shard is not None:
            Assert.eq(weight_shard.numel(), self._shard_size)
        if mode.support_forward:
            Assert.eq(weight_buffer.numel(), self._buffer_size)
            rank = self._fsdp_dim.rank
            self._weight_buffer_local_shard = weight_buffer[rank * self._shard_size : (rank + 1) * self._shard_size]
        if mode.support_backward and self._requires_grad:
            Assert.eq(grad_buffer.numel(), self._grad_buffer_size)
            rank = self._fsdp_dim.rank
            self._grad_buffer_local_shard = grad_buffer[rank * self._shard_size : (rank + 1) * self._shard_size]
            self._grad_shard_is_buffer = grad_shard is not None and grad_shard.data_ptr() == self._grad_buffer_local_shard.data_ptr()
        if mode.support_forward:
            for name, meta in self._parameter_metas.items():
                begin, end = self._parameter_begins_in_buffer[name], self._parameter_ends_in_buffer[name]
                param = weight_buffer[begin:end].view(meta.shape)
                if mode.support_backward and meta.requires_grad:
                    param.requires_grad_(True)
                    param.grad_buffer = grad_buffer[begin:end].view(meta.shape)
                    param.param_grad_is_zero = False
                    if meta.auto_grad_accumulation:
                        param.register_post_accumulate_grad_hook(_move_grad_to_buffer)
                meta.tensor = param

    @property
    def weight_shard(self):
        return self._weight_shard

    @property
    def grad_shard(self):
        return self._grad_shard

    @property
    def weight_buffer(self):
        return self._weight_buffer

    @property
    def grad_buffer(self):
        return self._grad_buffer

    def get_parameter_buffer(self, name: str) -> torch.Tensor:
        return self._parameter_metas[name].tensor

    def split_buffer(self, buffer: torch.Tensor) -> dict[str, torch.Tensor]:
        return {
            name: buffer[self._parameter_begins_in_buffer[name] : self._parameter_ends_in_buffer[name]].view(meta.shape)
            for name, meta in self._parameter_metas.items()
        }

    def split_shard(self, shard: torch.Tensor) -> dict[str, torch.Tensor]:
        """Flat pieces of every parameter that live in this rank's shard."""
        out = {}
        for name in self._parameter_metas:
            begin, end = self.parameter_range_in_shard(name)
            out[name] = shard[begin:end]
        return out

    # ---- weights
    def initialize_weights(self, distributed, log_fn=None) -> None:
        """Fill this rank's weight shard from each parameter's initialiser (identical on all data ranks)."""
        assert self._weight_shard is not None
        for name, meta in self._parameter_metas.items():
            begin, end = self.parameter_range_in_shard(name)
            full = torch.empty(meta.shape, dtype=torch.float32, device=self._weight_shard.device)
            meta.init_parameter(full, distributed)
            if end > begin:
                offset = self._fsdp_dim.rank * self._shard_size + begin - self._parameter_begins_in_buffer[name]
                self._weight_shard[begin:end].copy_(full.view(-1)[offset : offset + end - begin])
        if self._shard_pad > 0:
            self._weight_shard[self._shard_size - self._shard_pad :].zero_()

    def restore_parameters(self) -> None:
        """Rebuild the compute-dtype weight buffer from the fp32 shards (copy own slice, all-gather the rest)."""
        assert self._mode.support_forward
        # A shared buffer is re-filled between a stage's forward and backward with the very same values; keep the
        # version counter so tensors saved for backward (views of this buffer) stay valid for autograd.
        with torch.autograd._unsafe_preserve_version_counter(self._weight_buffer):
            self._weight_buffer_local_shard.copy_(self._weight_shard)
            if self._fsdp_dim.size > 1:
                all_gather_into_tensor(self._weight_buffer, self._weight_buffer_local_shard, group=self._fsdp_group)

    # ---- gradients
    def reset_gradients(self) -> None:
        if not (self._mode.support_backward and self._requires_grad):
            return
        for meta in self._parameter_metas.values():
            if meta.tensor is not None and meta.requires_grad:
                meta.tensor.param_grad_is_zero = True

    def reduce_gradients(self, accumulate: bool = False, allow_no_grad: bool = False) -> None:
        """Average the gradient buffer over the data group into the gradient shard (add to it if `accumulate`)."""
        if not (self._mode.support_backward and self._requires_grad):
            return
        for name, meta in self._parameter_metas.items():
            param = meta.tensor
            if meta.requires_grad and param.param_grad_is_zero:
                if not (allow_no_grad or meta.allow_no_grad):
                    raise RuntimeError(f"Parameter {name} got no gradient in this step")
                param.grad_buffer.zero_()
                param.param_grad_is_zero = False
        if self._sp_end > self._sp_begin and self._tensor_group is not None:
            all_reduce(self._grad_buffer[self._sp_begin : self._sp_end], group=self._tensor_group)
        if self._fsdp_dim.size > 1 and getattr(self, "_grad_arena", None) is not None:
            # Fused path: after a bounded barrier (every rank finished this stage's backward) each rank sums its slice of
            # all ranks' gradient buffers straight out of peer memory into its fp32 gradient shard.
            from fast_llm_b200.parallel.symmetric import rs_reduce

            self._grad_arena.barrier(0)
            # the kernel also leaves the per-block sums of squares of the reduced shard: the gradient norm needs no pass of
            # its own (`norm_partials` is a view into one buffer of all stages, finished by a single launch)
            rs_reduce(self._grad_arena, self._grad_buffer, self._grad_shard, self._shard_size, 1.0 / self._fsdp_dim.size,
                      accumulate, getattr(self, "norm_partials", None))
            return
        if self._fsdp_dim.size > 1:
            reduce_scatter_tensor(self._grad_buffer_local_shard, self._grad_buffer, op=torch.distributed.ReduceOp.AVG, group=self._fsdp_group)
        if self._grad_shard_is_buffer:
            assert not accumulate or self._fsdp_dim.size == 1
            return
        if accumulate:
            self._grad_shard.add_(self._grad_buffer_local_shard)
        else:
            self._grad_shard.copy_(self._grad_buffer_local_shard)

    # ---- (de)serialisation helpers
    def export_shard(self, shard: torch.Tensor) -> typing.Iterator[tuple[str, torch.Tensor]]:
        """Yield (parameter name, full local-shape tensor) reconstructed from every data rank's shard."""
        if self._fsdp_dim.size > 1:
            full = shard.new_empty(self._buffer_size)
            all_gather_into_tensor(full, shard.contiguous(), group=self._fsdp_group)
        else:
            full = shard
        for name, tensor in self.split_buffer(full).items():
            yield name, tensor

    def import_state_tensor(self, name: str, shard: torch.Tensor, tensor: torch.Tensor) -> int:
        """Copy the part of local-shape `tensor` that falls in this rank's shard; returns the number of elements set."""
        Assert.eq(tuple(tensor.shape), self._parameter_metas[name].shape)
        begin, end = self.parameter_range_in_shard(name)
        if end > begin:
            offset = self._fsdp_dim.rank * self._shard_size + begin - self._parameter_begins_in_buffer[name]
            shard[begin:end].copy_(tensor.reshape(-1)[offset : offset + end - begin])
        return end - begin

    def reset_shard_pad(self, shard: torch.Tensor) -> int:
        if self._shard_pad > 0:
            shard[self._shard_size - self._shard_pad :].zero_()
        return self._shard_pad

    def copy_shard_overlaps(self, loaded_fsdp: "FSDP", shards: dict[str, torch.Tensor], loaded_shards: dict[str, torch.Tensor],
                            loaded_rank_in_data: int | None = None, skip_replicated: bool = False) -> dict[str, int]:
        """Copy into `shards` whatever part of each of our parameters is present in `loaded_shards`, the shards of
        one rank of a model saved under another layout (`loaded_fsdp` describes that rank).  Handles different
        data-parallel sizes (different shard boundaries) and different tensor-parallel splits (via index maps).
        `skip_replicated`: the loaded rank is not the first of its tensor group, so its copies of the parameters that are not
        split over that group repeat what the first rank holds and are left out (each element is then loaded exactly once).
        Returns elements copied per parameter, for load verification."""
        counter: dict[str, int] = {}
        device = next(iter(shards.values())).device if shards else "cpu"
        for name, meta in self._parameter_metas.items():
            if name not in loaded_fsdp:
                continue
            loaded_meta = loaded_fsdp.get_parameter_meta(name)
            if skip_replicated and not loaded_meta.is_tensor_parallel:
                continue
            begin, end = self.parameter_range_in_shard(name)
            lbegin, lend = loaded_fsdp.parameter_range_in_shard(name)
            if end <= begin or lend <= lbegin:
                continue
            # element ids (position in the GLOBAL parameter) of the pieces held by us and by the loaded rank
            ours = _global_indices(meta, self._fsdp_dim.rank * self._shard_size + begin - self._parameter_begins_in_buffer[name], end - begin, device)
            theirs = _global_indices(loaded_meta, loaded_fsdp._fsdp_dim.rank * loaded_fsdp._shard_size + lbegin - loaded_fsdp._parameter_begins_in_buffer[name], lend - lbegin, device)
            # both index lists are sorted only when neither side is tensor-parallel; use a generic match
            global_numel = meta.global_numel()
            lookup = torch.full((global_numel,), -1, dtype=torch.int64, device=device)
            lookup[theirs] = torch.arange(theirs.numel(), device=device)
            src = lookup[ours]
            hit = src >= 0
            n = int(hit.sum().item())
            if n:
                dst_pos = torch.nonzero(hit, as_tuple=True)[0] + begin
                src_pos = src[hit] + lbegin
                for shard_name, shard in shards.items():
                    if shard_name in loaded_shards:
                        shard[dst_pos] = loaded_shards[shard_name][src_pos].to(shard.dtype)
            counter[name] = n
        return counter


def _global_indices(meta: ParameterMeta, local_offset: int, count: int, device) -> torch.Tensor:
    """Positions in the flattened GLOBAL parameter of `count` consecutive elements of the flattened LOCAL parameter."""
    if not meta.is_tensor_parallel:
        return torch.arange(local_offset, local_offset + count, device=device)
    index = torch.arange(meta.global_numel(), device=device).view(meta.global_shape)
    local = meta.global_to_local(index).reshape(-1)
    return local[local_offset : local_offset + count]


def _move_grad_to_buffer(param: torch.Tensor) -> None:
    """Post-accumulate hook: gradients produced by autograd are folded into the flat gradient buffer."""
    from fast_llm_b200.ops.param_grad import accumulate_param_grad

    if param.grad is not None:
        accumulate_param_grad(param, param.grad)
        param.grad = None
