"""Named tensor dimensions and parameter descriptions.

`TensorDim` knows whether a dimension is split over a process group, and converts tensors between their local (per
rank) and global forms.  Products (`CompositeTensorDim`, e.g. heads x head_size) and sums (`ConcatenatedTensorDim`,
e.g. gate rows followed by up rows) of dimensions shard each factor / term separately, so fused weights shard the way
their parts would.  `ParameterMeta` describes one parameter before any memory exists: shape, initialisation,
weight-decay / learning-rate-scale flags; the stage later binds it to views of the flat weight and gradient buffers.

Parity: `fast_llm/engine/config_utils/tensor_dim.py:16-231`, `fast_llm/tensor.py:52-355` (this implementation keeps
metas as plain objects rather than `torch.Tensor` subclasses on the meta device).
"""

import math
import typing

import torch

from fast_llm_b200.parallel.topology import DistributedDim
from fast_llm_b200.utils import Assert, div


class TensorDim:
    def __init__(self, name: str, global_size: int, parallel_dim: DistributedDim | None = None):
        self._name = name
        self._global_size = global_size
        self._parallel_dim = parallel_dim if parallel_dim is not None and parallel_dim.size > 1 else None
        self._size = global_size if self._parallel_dim is None else div(global_size, self._parallel_dim.size)

    def __repr__(self):
        return f"{type(self).__name__}({self._name}, size={self._size}, global_size={self._global_size}, parallel={self.parallel_dim is not None})"

    def __eq__(self, other):
        return isinstance(other, TensorDim) and self._name == other._name and self._size == other._size and self._global_size == other._global_size

    __hash__ = object.__hash__

    @property
    def name(self) -> str:
        return self._name

    @property
    def size(self) -> int:
        return self._size

    @property
    def global_size(self) -> int:
        return self._global_size

    @property
    def is_parallel(self) -> bool:
        return self._parallel_dim is not None

    @property
    def parallel_dim(self) -> DistributedDim | None:
        return self._parallel_dim

    @property
    def parallel_group(self):
        return None if self._parallel_dim is None else self._parallel_dim.group

    def replace_parallel_dim(self, distributed_dim: DistributedDim) -> "TensorDim":
        assert self.is_parallel
        return TensorDim(self._name, self._global_size, distributed_dim)

    # --- conversions along tensor axis `dim`
    def local_to_global(self, tensor: torch.Tensor, dim: int = 0) -> torch.Tensor:
        """All-gather the shards of `tensor` along `dim` (needs the process group)."""
        if not self.is_parallel:
            return tensor
        from fast_llm_b200.parallel.ops import gather_op

        return gather_op(tensor, self.parallel_group, dim)

    def local_to_global_partial(self, tensor: torch.Tensor, dim: int = 0, fill_value: float = -1) -> torch.Tensor:
        """Global-shaped tensor holding this rank's shard and `fill_value` elsewhere (no communication)."""
        if not self.is_parallel:
            return tensor
        shape = list(tensor.shape)
        shape[dim] = self._global_size
        out = tensor.new_full(shape, fill_value)
        rank = self._parallel_dim.rank
        out.narrow(dim, rank * self._size, self._size).copy_(tensor)
        return out

    def global_to_local(self, tensor: torch.Tensor, dim: int = 0, rank: int | None = None) -> torch.Tensor:
        if not self.is_parallel:
            return tensor
        rank = self._parallel_dim.rank if rank is None else rank
        return tensor.narrow(dim, rank * self._size, self._size)


class CompositeTensorDim(TensorDim):
    """Product of dimensions (row-major); at most one factor may be parallel."""

    def __init__(self, name: str, dims: typing.Sequence[TensorDim]):
        parallel = [(i, d) for i, d in enumerate(dims) if d.is_parallel]
        Assert.leq(len(parallel), 1)
        self._dims = tuple(dims)
        self._parallel_index = parallel[0][0] if parallel else None
        super().__init__(name, math.prod(d.global_size for d in dims), parallel[0][1].parallel_dim if parallel else None)
        Assert.eq(self._size, math.prod(d.size for d in dims))

    @property
    def dims(self):
        return self._dims

    def replace_parallel_dim(self, distributed_dim):
        return CompositeTensorDim(self._name, [d.replace_parallel_dim(distributed_dim) if d.is_parallel else d for d in self._dims])

    def _split(self, tensor, dim, use_global):
        sizes = [d.global_size if use_global else d.size for d in self._dims]
        return tensor.reshape(*tensor.shape[:dim], *sizes, *tensor.shape[dim + 1 :])

    def local_to_global(self, tensor, dim=0):
        if not self.is_parallel:
            return tensor
        t = self._split(tensor, dim, False)
        t = self._dims[self._parallel_index].local_to_global(t, dim + self._parallel_index)
        return t.reshape(*tensor.shape[:dim], self._global_size, *tensor.shape[dim + 1 :])

    def local_to_global_partial(self, tensor, dim=0, fill_value=-1):
        if not self.is_parallel:
            return tensor
        t = self._split(tensor, dim, False)
        t = self._dims[self._parallel_index].local_to_global_partial(t, dim + self._parallel_index, fill_value)
        return t.reshape(*tensor.shape[:dim], self._global_size, *tensor.shape[dim + 1 :])

    def global_to_local(self, tensor, dim=0, rank=None):
        if not self.is_parallel:
            return tensor
        t = self._split(tensor, dim, True)
        t = self._dims[self._parallel_index].global_to_local(t, dim + self._parallel_index, rank)
        return t.reshape(*tensor.shape[:dim], self._size, *tensor.shape[dim + 1 :])


class ConcatenatedTensorDim(TensorDim):
    """Concatenation of dimensions that are all parallel over the same group, or all not parallel."""

    def __init__(self, name: str, dims: typing.Sequence[TensorDim]):
        parallel_dim = dims[0].parallel_dim
        for d in dims[1:]:
            Assert.eq(d.parallel_dim is None, parallel_dim is None)
        self._dims = tuple(dims)
        super().__init__(name, sum(d.global_size for d in dims), parallel_dim)
        Assert.eq(self._size, sum(d.size for d in dims))

    @property
    def dims(self):
        return self._dims

    def replace_parallel_dim(self, distributed_dim):
        return ConcatenatedTensorDim(self._name, [d.replace_parallel_dim(distributed_dim) for d in self._dims])

    def local_to_global(self, tensor, dim=0):
        if not self.is_parallel:
            return tensor
        parts = tensor.split([d.size for d in self._dims], dim)
        return torch.cat([d.local_to_global(p, dim) for d, p in zip(self._dims, parts)], dim)

    def local_to_global_partial(self, tensor, dim=0, fill_value=-1):
        if not self.is_parallel:
            return tensor
        parts = tensor.split([d.size for d in self._dims], dim)
        return torch.cat([d.local_to_global_partial(p, dim, fill_value) for d, p in zip(self._dims, parts)], dim)

    def global_to_local(self, tensor, dim=0, rank=None):
        if not self.is_parallel:
            return tensor
        parts = tensor.split([d.global_size for d in self._dims], dim)
        return torch.cat([d.global_to_local(p, dim, rank) for d, p in zip(self._dims, parts)], dim)


scalar_dim = TensorDim("scalar", 1)


class ParameterMeta:
    """Description of one parameter; `tensor` is set when a stage (or `Layer.materialize`) binds memory to it."""

    def __init__(self, dims: typing.Sequence[TensorDim], *, name: str = "", init_method: "typing.Callable | None" = None,
                 weight_decay: bool = True, lr_scale: float | None | tuple = None, requires_grad: bool = True,
                 allow_sequence_tensor_parallel: bool = True, allow_no_grad: bool = False,
                 auto_grad_accumulation: bool = True):
        self.dims = tuple(dims)
        self.tensor_name = name
        self.param_init_method = init_method
        self.param_weight_decay = weight_decay
        self._lr_scale = lr_scale if isinstance(lr_scale, tuple) else (lr_scale,)
        self.requires_grad = requires_grad and any(s != 0 for s in self._lr_scale)
        # Replicated over the tensor group but fed sequence-parallel activations: its gradient needs a tensor-group sum.
        self.sequence_tensor_parallel = allow_sequence_tensor_parallel and not self.is_tensor_parallel
        self.allow_no_grad = allow_no_grad
        self.auto_grad_accumulation = auto_grad_accumulation
        self.tensor: torch.Tensor | None = None

    def __repr__(self):
        return f"ParameterMeta({self.tensor_name}, shape={self.shape}, global_shape={self.global_shape})"

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(d.size for d in self.dims)

    @property
    def global_shape(self) -> tuple[int, ...]:
        return tuple(d.global_size for d in self.dims)

    def numel(self) -> int:
        return math.prod(self.shape)

    def global_numel(self) -> int:
        return math.prod(self.global_shape)

    @property
    def is_tensor_parallel(self) -> bool:
        return any(d.is_parallel for d in self.dims)

    @property
    def lr_scale(self) -> tuple:
        return self._lr_scale

    def local_to_global(self, tensor: torch.Tensor) -> torch.Tensor:
        Assert.eq(tuple(tensor.shape), self.shape)
        for i, d in enumerate(self.dims):
            tensor = d.local_to_global(tensor, i)
        return tensor

    def local_to_global_partial(self, tensor: torch.Tensor, fill_value: float = -1) -> torch.Tensor:
        for i, d in enumerate(self.dims):
            tensor = d.local_to_global_partial(tensor, i, fill_value)
        return tensor

    def global_to_local(self, tensor: torch.Tensor, rank: int | None = None) -> torch.Tensor:
        Assert.eq(tuple(tensor.shape), self.global_shape)
        for i, d in enumerate(self.dims):
            tensor = d.global_to_local(tensor, i, rank)
        return tensor

    def init_parameter(self, tensor: torch.Tensor, distributed, reproducible: bool | None = None) -> None:
        """Fill `tensor` (local shape).  With reproducible init, draw the global tensor and keep this rank's slice."""
        assert self.param_init_method is not None, f"No init method for {self.tensor_name}"
        override = getattr(self, "init_override", None)
        if override is not None:  # e.g. the Megatron-compatible initialisation order
            return override(tensor, distributed)
        reproducible = distributed.config.reproducible_init if reproducible is None else reproducible
        generator = distributed.tp_init_generator if self.is_tensor_parallel and not reproducible else distributed.pp_init_generator
        if reproducible:
            # One private stream per parameter, keyed by its name: the values do not depend on which other
            # parameters this rank initialises (pipeline / stage splits) nor on how the parameter is sharded.
            import zlib

            seed = (distributed.config.seed + distributed.config.pp_gen_init_seed_shift + zlib.crc32(self.tensor_name.encode())) % 2**63
            generator = torch.Generator(device=generator.device).manual_seed(seed)
        if reproducible and self.is_tensor_parallel:
            full = torch.empty(self.global_shape, dtype=torch.float32, device=generator.device)
            self.param_init_method(self, full, generator)
            tensor.copy_(self.global_to_local(full))
        else:
            tmp = torch.empty(self.shape, dtype=torch.float32, device=generator.device)
            self.param_init_method(self, tmp, generator)
            tensor.copy_(tmp)
