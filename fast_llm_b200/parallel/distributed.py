"""Process groups, seeds and random generators of one training process.

One process drives one GPU.  `torch.distributed` (NCCL on GPUs, Gloo on CPU) provides the control plane and the plain
collectives; groups are created once per distinct rank set and shared between the named dimensions that resolve to the
same ranks.  Parity: `fast_llm/engine/distributed/distributed.py:23-271` (ProcessGroupPool + Distributed); here groups
come from `torch.distributed.new_group`, which also makes them usable as symmetric-memory groups for the fused kernels.
"""

import datetime
import logging
import os

import torch
import torch.distributed

from fast_llm_b200.parallel.topology import (
    MAX_SEED,
    DistributedBackend,
    DistributedConfig,
    DistributedDim,
    DistributedDimNames,
    PhaseType,
)

logger = logging.getLogger(__name__)


class ProcessGroupPool:
    """Creates (and caches) one process group per distinct tuple of global ranks."""

    def __init__(self, config: DistributedConfig, use_cuda: bool | None = None):
        self.world_size = config.world_size
        self.rank = config.rank
        self.use_cuda = (config.use_cuda and torch.cuda.is_available()) if use_cuda is None else use_cuda
        self.backend = DistributedBackend.nccl if self.use_cuda and config.backend == DistributedBackend.nccl else DistributedBackend.gloo
        self.timeout = datetime.timedelta(seconds=config.timeout)
        self._groups: dict[tuple[int, ...], torch.distributed.ProcessGroup] = {}
        self._owns_default_group = False
        if self.use_cuda:
            local_rank = int(os.environ.get("LOCAL_RANK", config.local_rank))
            self.device = torch.device("cuda", local_rank % max(torch.cuda.device_count(), 1))
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        if self.world_size > 1 and not torch.distributed.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            kwargs = {"device_id": self.device} if self.use_cuda else {}
            torch.distributed.init_process_group(
                backend=self.backend.value, rank=self.rank, world_size=self.world_size, timeout=self.timeout, **kwargs
            )
            self._owns_default_group = True
        if self.world_size > 1:
            assert torch.distributed.get_world_size() == self.world_size
            assert torch.distributed.get_rank() == self.rank
            # Every rank creates every group, in the same order (new_group is collective over the world).
            for ranks in config.all_group_rank_sets():
                if len(ranks) == self.world_size:
                    group = torch.distributed.group.WORLD
                else:
                    group = torch.distributed.new_group(list(ranks), timeout=self.timeout, backend=self.backend.value)
                if self.rank in ranks:
                    self._groups[tuple(ranks)] = group

    def get_process_group(self, global_ranks: tuple[int, ...] | range, group_rank: int | None = None):
        ranks = tuple(global_ranks)
        if len(ranks) == 1:
            return None
        return self._groups[ranks]

    def shutdown(self) -> None:
        self._groups.clear()
        if self._owns_default_group and torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()
            self._owns_default_group = False


class Distributed:
    """Owns the named process groups and the seeded generators of this rank."""

    def __init__(self, config: DistributedConfig, use_cpu: bool = False, pool: ProcessGroupPool | None = None):
        config.validate()
        self._config = config
        self._use_cpu = use_cpu or not (config.use_cuda and torch.cuda.is_available())
        self._pool = pool or ProcessGroupPool(config, use_cuda=not self._use_cpu)
        self._owns_pool = pool is None
        self.device = self._pool.device
        dims = config.distributed_dims
        for dim in dims.values():
            if not dim._is_setup:
                dim.setup(self._pool.get_process_group(dim.global_ranks))
        n = DistributedDimNames
        self.world_group = dims[n.world].group
        self.data_group = dims[n.data].group
        self.pipeline_group = dims[n.pipeline].group
        self.tensor_group = dims[n.tensor].group
        self.sequence_data_group = dims[n.sequence_data].group
        self.batch_data_group = dims[n.batch_data].group
        self.tensor_and_sequence_data_group = dims[n.tensor_and_sequence_data].group
        self.tensor_and_data_group = dims[n.tensor_and_data].group
        self.model_and_sequence_data_group = dims[n.model_and_sequence_data].group

        self._config.log_first_rank(f"Setting random seeds (base {config.seed})")
        dp_shift = config.dp_seed_shift * config.data_rank
        pp_shift = config.pp_seed_shift * config.pipeline_rank
        tp_shift = config.tp_seed_shift * config.tensor_rank
        pp_base = config.seed + dp_shift + pp_shift
        tp_base = pp_base + tp_shift
        self._pp_seed = (pp_base + config.pp_gen_seed_shift) % MAX_SEED
        self._tp_seed = (tp_base + config.tp_gen_seed_shift) % MAX_SEED
        pp_init = (config.seed + pp_shift * (0 if config.reproducible_init else 1) + config.pp_gen_init_seed_shift) % MAX_SEED
        tp_init = (config.seed + (pp_shift + tp_shift) * (0 if config.reproducible_init else 1) + config.tp_gen_init_seed_shift) % MAX_SEED
        gen_device = "cpu" if config.force_cpu_initialization else self.device
        self.default_cpu_generator = torch.random.default_generator
        self.pp_generator = torch.Generator(device=self.device).manual_seed(self._pp_seed)
        self.tp_generator = torch.Generator(device=self.device).manual_seed(self._tp_seed)
        self.pp_init_generator = torch.Generator(device=gen_device).manual_seed(pp_init)
        self.tp_init_generator = torch.Generator(device=gen_device).manual_seed(tp_init)
        self._phase_seeds_shifts = {
            PhaseType.training: config.train_seed_shift,
            PhaseType.validation: config.valid_seed_shift,
            PhaseType.inference: config.inference_seed_shift,
        }

    @property
    def config(self) -> DistributedConfig:
        return self._config

    def check_config(self, config: DistributedConfig) -> None:
        if config.reference_config is None:
            assert config is self._config or config.to_dict() == self._config.to_dict()
        else:
            assert config.reference_config is self._config

    def set_step(self, step: int, phase: PhaseType) -> None:
        """Reseed the per-step generators so dropout etc. depend only on (seed, step, phase, rank coordinates)."""
        shift = step * self._config.sample_seed_shift + self._phase_seeds_shifts[phase]
        self.pp_generator.manual_seed((self._pp_seed + shift) % MAX_SEED)
        self.tp_generator.manual_seed((self._tp_seed + shift) % MAX_SEED)

    def shutdown(self) -> None:
        if self._owns_pool:
            self._pool.shutdown()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.shutdown()
