"""Parallel layout of a job: which global ranks form the tensor / pipeline / data / ... groups.

The world is a mixed-radix mesh whose fastest-varying axis is `tensor`, followed by either
(sequence_data, batch_data, pipeline) or, with `pipeline_first`, (pipeline, sequence_data, batch_data).  Every named
group is the set of ranks obtained by varying a subset of axes while the others stay at this rank's coordinates.
The resulting rank assignments are identical to `fast_llm/engine/distributed/config.py:296-395`
(tensor_rank = rank % tp, and so on), so checkpoints and launch scripts are interchangeable.
"""

import dataclasses
import enum
import os
import typing

from fast_llm_b200.config import Config, Field, FieldHint, check_field, config_class
from fast_llm_b200.utils import Assert, div
from fast_llm_b200.utils.data_type import DataType

_BIG_PRIMES = (
    317767863445754100075399033823, 811026271858507938190098775099, 500460795349110443334056239993,
    631112027069964424381239824623, 705275193289568515128435800471, 557334919521627299485226546649,
    302512698914367389283822541603, 524349078566919481839996533519, 777213299180617990335487093979,
    566651603736003330313203603679, 727191698855007974519213398423, 612345874987293461243865328471,
)
MAX_SEED = 2**64


class PhaseType(str, enum.Enum):
    training = "training"
    validation = "validation"
    inference = "inference"

    @property
    def is_training(self) -> bool:
        return self == PhaseType.training


class DistributedBackend(str, enum.Enum):
    nccl = "nccl"
    gloo = "gloo"


class DistributedDimNames:
    world = "world"
    tensor = "tensor"
    data = "data"
    pipeline = "pipeline"
    sequence_data = "sequence_data"
    batch_data = "batch_data"
    tensor_and_sequence_data = "tensor_and_sequence_data"
    tensor_and_data = "tensor_and_data"
    model_and_sequence_data = "model_and_sequence_data"


@dataclasses.dataclass
class DistributedDim:
    """Name, size, this rank's index and the global ranks of one process group (the group itself is bound later)."""

    name: str
    size: int
    rank: int
    global_ranks: tuple[int, ...]
    _group: typing.Any = dataclasses.field(default=None, repr=False, compare=False)
    _is_setup: bool = dataclasses.field(default=False, repr=False, compare=False)

    def __getstate__(self):
        state = self.__dict__.copy()
        state["_group"] = None
        state["_is_setup"] = False
        return state

    @property
    def group(self):
        assert self._is_setup, f"Process group {self.name} is not set up"
        return self._group

    def setup(self, group) -> None:
        assert not self._is_setup
        Assert.eq(group is None, self.size == 1)
        self._group = group
        self._is_setup = True


@dataclasses.dataclass(frozen=True)
class _Axis:
    name: str
    size: int
    stride: int


def mesh_axes(tensor: int, pipeline: int, sequence_data: int, batch_data: int, pipeline_first: bool) -> dict[str, _Axis]:
    order = [("tensor", tensor)]
    if pipeline_first:
        order += [("pipeline", pipeline), ("sequence_data", sequence_data), ("batch_data", batch_data)]
    else:
        order += [("sequence_data", sequence_data), ("batch_data", batch_data), ("pipeline", pipeline)]
    axes, stride = {}, 1
    for name, size in order:
        axes[name] = _Axis(name, size, stride)
        stride *= size
    return axes


def group_for(name: str, rank: int, axes: typing.Sequence[_Axis]) -> DistributedDim:
    """Ranks reached from `rank` by varying `axes` (listed fastest-first), and this rank's index among them."""
    base = rank
    index, span = 0, 1
    for axis in axes:
        coord = rank // axis.stride % axis.size
        base -= coord * axis.stride
        index += coord * span
        span *= axis.size
    ranks = [base]
    for axis in axes:
        ranks = [r + c * axis.stride for c in range(axis.size) for r in ranks]
    return DistributedDim(name=name, size=span, rank=index, global_ranks=tuple(ranks))


@config_class()
class DistributedConfig(Config):
    """Parallel layout and global numerics of a run (same keys as the reference's `model.distributed`)."""

    tensor_parallel: int = Field(default=1, desc="Tensor parallelism group size.", hint=FieldHint.performance, valid=check_field(Assert.gt, 0))
    pipeline_parallel: int = Field(default=1, desc="Pipeline parallelism group size.", hint=FieldHint.performance, valid=check_field(Assert.gt, 0))
    sequence_tensor_parallel: bool = Field(default=False, desc="Split activations between layers along tokens over the tensor group.", hint=FieldHint.performance)
    sequence_data_parallel: int = Field(default=1, desc="Split each sequence over this many data ranks.", hint=FieldHint.performance, valid=check_field(Assert.gt, 0))
    world_size: int = Field(default=None, desc="Number of processes (default: WORLD_SIZE).", hint=FieldHint.expert, valid=check_field(Assert.gt, 0))
    rank: int = Field(default=None, desc="Rank of this process (default: RANK).", hint=FieldHint.expert, valid=check_field(Assert.geq, 0))
    local_world_size: int = Field(default=None, desc="Processes per node (default: LOCAL_WORLD_SIZE).", hint=FieldHint.expert, valid=check_field(Assert.gt, 0))
    pipeline_first: bool = Field(default=False, desc="Place pipeline neighbours before data-parallel neighbours in the rank order.", hint=FieldHint.expert)
    backend: DistributedBackend = Field(default=DistributedBackend.nccl, desc="Collective backend.", hint=FieldHint.expert)
    timeout: float = Field(default=60, desc="Timeout of distributed operations (s).", hint=FieldHint.optional, valid=check_field(Assert.gt, 0))
    use_cuda: bool = Field(default=True, desc="Run on GPU.", hint=FieldHint.expert)
    force_cpu_initialization: bool = Field(default=False, desc="Generate initial weights on the CPU for bitwise reproducibility across devices.", hint=FieldHint.expert)
    seed: int = Field(default=1234, desc="Base seed.", hint=FieldHint.optional)
    compute_dtype: DataType = Field(default=DataType.float32, desc="Activation / compute dtype.", hint=FieldHint.core)
    optimization_dtype: DataType = Field(default=DataType.float32, desc="Dtype of master weights and optimizer state.", hint=FieldHint.expert)
    dp_seed_shift: int = Field(default=_BIG_PRIMES[0], hint=FieldHint.optional)
    pp_seed_shift: int = Field(default=_BIG_PRIMES[1], hint=FieldHint.optional)
    pp_gen_seed_shift: int = Field(default=_BIG_PRIMES[2], hint=FieldHint.optional)
    pp_gen_init_seed_shift: int = Field(default=_BIG_PRIMES[3], hint=FieldHint.optional)
    tp_seed_shift: int = Field(default=_BIG_PRIMES[4], hint=FieldHint.optional)
    tp_gen_seed_shift: int = Field(default=_BIG_PRIMES[5], hint=FieldHint.optional)
    tp_gen_init_seed_shift: int = Field(default=_BIG_PRIMES[6], hint=FieldHint.optional)
    sample_seed_shift: int = Field(default=_BIG_PRIMES[7], hint=FieldHint.optional)
    train_seed_shift: int = Field(default=_BIG_PRIMES[8], hint=FieldHint.optional)
    valid_seed_shift: int = Field(default=_BIG_PRIMES[9], hint=FieldHint.optional)
    inference_seed_shift: int = Field(default=_BIG_PRIMES[10], hint=FieldHint.optional)
    reproducible_init: bool = Field(default=False, desc="Initialise every parameter from its global shape so weights do not depend on the layout.", hint=FieldHint.testing)
    reference_config: "DistributedConfig|None" = Field(default=None, init=False, desc="Config of the model this one shares its Distributed with.", hint=FieldHint.derived)

    def _validate(self) -> None:
        if self.world_size is None:
            self.world_size = int(os.environ.get("WORLD_SIZE", 1))
        if self.rank is None:
            self.rank = int(os.environ.get("RANK", 0))
        if self.local_world_size is None:
            self.local_world_size = int(os.environ.get("LOCAL_WORLD_SIZE", self.world_size))
        if self.tensor_parallel == 1 and self.sequence_tensor_parallel:
            self.sequence_tensor_parallel = False
        super()._validate()
        Assert.multiple(self.world_size, self.tensor_parallel * self.pipeline_parallel)
        Assert.multiple(self.data_parallel, self.sequence_data_parallel)
        Assert.multiple(self.local_world_size, self.tensor_parallel)
        Assert.in_range(self.rank, 0, self.world_size)

    # ---- derived sizes and coordinates
    @property
    def model_parallel(self) -> int:
        return self.tensor_parallel * self.pipeline_parallel

    @property
    def data_parallel(self) -> int:
        return div(self.world_size, self.model_parallel)

    @property
    def batch_data_parallel(self) -> int:
        return div(self.data_parallel, self.sequence_data_parallel)

    @property
    def num_nodes(self) -> int:
        return div(self.world_size, self.local_world_size)

    @property
    def local_rank(self) -> int:
        return self.rank % self.local_world_size

    def _axes(self) -> dict[str, _Axis]:
        return mesh_axes(self.tensor_parallel, self.pipeline_parallel, self.sequence_data_parallel,
                         self.batch_data_parallel, self.pipeline_first)

    def _coord(self, axis: str) -> int:
        a = self._axes()[axis]
        return self.rank // a.stride % a.size

    @property
    def tensor_rank(self) -> int:
        return self._coord("tensor")

    @property
    def pipeline_rank(self) -> int:
        return self._coord("pipeline")

    @property
    def sequence_data_rank(self) -> int:
        return self._coord("sequence_data")

    @property
    def batch_data_rank(self) -> int:
        return self._coord("batch_data")

    @property
    def data_rank(self) -> int:
        return self.batch_data_rank * self.sequence_data_parallel + self.sequence_data_rank

    def dims_for_rank(self, rank: int) -> dict[str, DistributedDim]:
        ax = self._axes()
        n = DistributedDimNames
        world = _Axis("world", self.world_size, 1)
        spec = {
            n.world: [world],
            n.data: [ax["sequence_data"], ax["batch_data"]],
            n.pipeline: [ax["pipeline"]],
            n.tensor: [ax["tensor"]],
            n.sequence_data: [ax["sequence_data"]],
            n.batch_data: [ax["batch_data"]],
            n.tensor_and_sequence_data: [ax["tensor"], ax["sequence_data"]],
            n.tensor_and_data: [ax["tensor"], ax["sequence_data"], ax["batch_data"]],
            n.model_and_sequence_data: sorted([ax["tensor"], ax["pipeline"], ax["sequence_data"]], key=lambda a: a.stride),
        }
        return {name: group_for(name, rank, axes) for name, axes in spec.items()}

    @property
    def distributed_dims(self) -> dict[str, DistributedDim]:
        if self.reference_config is not None:
            return self.reference_config.distributed_dims
        cache = self.__dict__.get("_dims_cache")
        if cache is None:
            cache = self.dims_for_rank(self.rank)
            object.__setattr__(self, "_dims_cache", cache)
        return cache

    def get_distributed_dim(self, name: str) -> DistributedDim:
        return self.distributed_dims[name]

    def all_group_rank_sets(self) -> list[tuple[int, ...]]:
        """Every distinct multi-rank group of every rank, in one order shared by all ranks (for collective creation)."""
        seen, out = set(), []
        for rank in range(self.world_size):
            for dim in self.dims_for_rank(rank).values():
                if dim.size > 1 and dim.global_ranks not in seen:
                    seen.add(dim.global_ranks)
                    out.append(dim.global_ranks)
        return out

    def log_first_rank(self, *message, log_fn=None):
        import logging

        if self.rank == 0:
            (log_fn or logging.getLogger(__name__).info)(" ".join(map(str, message)))
