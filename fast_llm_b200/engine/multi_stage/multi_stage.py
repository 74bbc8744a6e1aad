"""A model split into stages with ZeRO-sharded state carved from a few flat tensors.

Stage `i` lives on pipeline rank `i % pipeline_parallel`.  Each named state shard (weights, Adam moments, gradients)
is ONE flat tensor per rank: the concatenation, in stage order, of every local stage's shard - exactly what a
`rank_r.safetensors` of the distributed checkpoint format stores.  Weight and gradient buffers are separate flat
tensors; with ZeRO-2/3 a small number of buffers is shared round-robin between stages.
Parity: `fast_llm/engine/multi_stage/multi_stage.py:25-633`.
"""

import logging
import typing

import torch

from fast_llm_b200.engine.base_model import BaseModel
from fast_llm_b200.engine.multi_stage.config import FastLLMModelConfig, StageMode
from fast_llm_b200.engine.multi_stage.stage import Stage
from fast_llm_b200.parallel.distributed import Distributed
from fast_llm_b200.parallel.topology import DistributedDimNames
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


class ShardName:
    weights = "weights"
    grads = "grads"


class MultiStageModel:
    config_class: typing.ClassVar[type[FastLLMModelConfig]] = FastLLMModelConfig
    base_model_class: typing.ClassVar[type[BaseModel]] = BaseModel

    def __init__(self, config: FastLLMModelConfig, *, optimizer_state_names: tuple[str, ...] = (), verbose: bool = True,
                 stage_filter: set | None = None):
        config.validate()
        self._config = config
        self._base_model = config.base_model.get_base_model(config.distributed)
        self._training = None
        self._verbose = verbose
        self._state_shard_names = (ShardName.weights, *optimizer_state_names)
        self._is_setup = False
        self._stage_filter = stage_filter

        layers = self._base_model.get_layers()
        self._layers = layers
        splits = self._split_into_stages([layer.layer_count for layer in layers], config.multi_stage.layers_per_stage)
        self._num_stages = len(splits) - 1
        pp = config.distributed.pipeline_parallel
        Assert.geq(self._num_stages, pp)

        # tied parameters: the first meta owns the storage; later metas on the same pipeline rank alias it
        self._tied_parameters = self._base_model.get_tied_parameters()
        meta_stage = {}
        for s in range(self._num_stages):
            for layer in layers[splits[s] : splits[s + 1]]:
                for _, meta in layer.named_parameter_metas():
                    meta_stage[id(meta)] = s
        self._tied_duplicates: dict[str, tuple] = {}
        # Copies on ANOTHER pipeline rank keep storage of their own: they receive the owner's values after
        # initialisation / loading, and both sides add each other's gradient before their data-parallel reduction, so the
        # copies stay identical (`fast_llm/engine/multi_stage/multi_stage.py` tied groups, `runner.py:243`).
        self._tied_remote: list[tuple] = []
        duplicate_names = set()
        for name, metas in self._tied_parameters.items():
            owner = metas[0]
            owner_rank = meta_stage[id(owner)] % pp
            holders = {owner_rank: owner}
            for dup in metas[1:]:
                dup_rank = meta_stage[id(dup)] % pp
                if dup_rank in holders:
                    local_owner = holders[dup_rank]
                    duplicate_names.add(dup.tensor_name)
                    self._tied_duplicates[dup.tensor_name] = (local_owner, dup, meta_stage[id(local_owner)], meta_stage[id(dup)])
                else:
                    holders[dup_rank] = dup
                    self._tied_remote.append((owner, dup, meta_stage[id(owner)], meta_stage[id(dup)]))

        self._stages = [
            Stage(config=config.multi_stage, layers=layers[splits[s] : splits[s + 1]], distributed_config=config.distributed,
                  index=s, begin=splits[s], end=splits[s + 1], tied_duplicates=duplicate_names)
            for s in range(self._num_stages)
        ]
        self._stages_on_device = {s: stage for s, stage in enumerate(self._stages)
                                  if s % pp == config.distributed.pipeline_rank and (stage_filter is None or s in stage_filter)}
        self._stage_pipeline_ranks = {s: s % pp for s in range(self._num_stages)}
        self._parameter_stages = {name: s for s, stage in enumerate(self._stages) for name in stage.parameter_names}

    @staticmethod
    def _split_into_stages(layer_counts: list[float], layers_per_stage: float) -> list[int]:
        """Greedy split: close a stage once it holds `layers_per_stage` worth of layers."""
        splits = [0]
        acc = 0.0
        for i, count in enumerate(layer_counts):
            if acc > 0 and acc + count > layers_per_stage + 1e-6:
                splits.append(i)
                acc = 0.0
            acc += count
            if acc >= layers_per_stage - 1e-6:
                splits.append(i + 1)
                acc = 0.0
        if splits[-1] != len(layer_counts):
            splits.append(len(layer_counts))
        return sorted(set(splits))

    # ---- properties
    @property
    def config(self):
        return self._config

    @property
    def base_model(self):
        return self._base_model

    @property
    def stages(self) -> list[Stage]:
        return self._stages

    @property
    def stages_on_device(self) -> dict[int, Stage]:
        return self._stages_on_device

    @property
    def distributed(self) -> Distributed:
        return self._distributed

    @property
    def state_shard_names(self) -> tuple[str, ...]:
        return self._state_shard_names

    @property
    def is_setup(self):
        return self._is_setup

    def get_shard_names(self, shard_config) -> tuple[str, ...]:
        if shard_config.optimizer_state:
            return self._state_shard_names if shard_config.model_weights else self._state_shard_names[1:]
        return (ShardName.weights,) if shard_config.model_weights else ()

    def get_parameter_stage(self, name: str) -> Stage:
        return self._stages[self._parameter_stages[name]]

    @property
    def parameter_names(self) -> list[str]:
        return list(self._parameter_stages)

    def is_parameter_on_device(self, name: str) -> bool:
        return self._parameter_stages[name] in self._stages_on_device

    # ---- memory
    def setup(self, distributed: Distributed | None = None, mode: StageMode = StageMode.training, allocator=None) -> None:
        assert not self._is_setup
        self._is_setup = True
        self._mode = mode
        self._distributed = distributed or Distributed(self._config.distributed)
        self._base_model._distributed = self._distributed
        self._training = mode.support_training
        device = self._distributed.device
        allocator = allocator or (lambda n, dtype, name: torch.empty(n, dtype=dtype, device=device))
        ms = self._config.multi_stage
        dist_config = self._config.distributed
        local = list(self._stages_on_device.items())

        if not mode.on_device:
            return
        # ---- shards: one flat tensor per name, stage after stage, fsdp after fsdp
        entries = [(s, i, fsdp) for s, stage in local for i, fsdp in enumerate(stage.fsdps)]
        dtypes = {fsdp.shard_dtype for _, _, fsdp in entries} or {dist_config.optimization_dtype.torch}
        shard_dtype = dist_config.optimization_dtype.torch if len(dtypes) > 1 else next(iter(dtypes))
        total = sum(fsdp.shard_size for _, _, fsdp in entries)
        self._shards = {name: allocator(total, shard_dtype, f"{name}_shard") for name in self._state_shard_names}
        for t in self._shards.values():
            t.zero_()
        num_weight_buffers = min(ms.num_weight_buffers or len(local), max(len(local), 1))
        num_grad_buffers = min(ms.num_grad_buffers or len(local), max(len(local), 1))
        dp1_alias = (mode.support_backward and dist_config.data_parallel == 1 and num_grad_buffers == len(local)
                     and all(fsdp.grad_buffer_dtype == shard_dtype for _, _, fsdp in entries if fsdp.requires_grad))
        grad_total = sum(fsdp.grad_shard_size for _, _, fsdp in entries)
        self._grad_shard_is_buffer = dp1_alias
        if mode.support_backward and not dp1_alias:
            self._shards[ShardName.grads] = allocator(grad_total, shard_dtype, "grads_shard")

        # ---- buffers (in NVLink symmetric memory when the fused ZeRO kernels will use them)
        from fast_llm_b200.parallel.symmetric import SymmetricArena, symmetric_memory_available

        self._weight_arena = self._grad_arena = None
        use_symmetric = (
            ms.fused_collectives and mode.support_backward and dist_config.data_parallel > 1
            and dist_config.compute_dtype.torch == torch.bfloat16 and num_weight_buffers == len(local)
            and num_grad_buffers == len(local) and symmetric_memory_available(self._distributed.data_group, device)
        )

        # tensor-parallel GEMMs fused with their all-gather / reduce-scatter (sequence-parallel layout)
        if (ms.fused_collectives and dist_config.tensor_parallel > 1 and dist_config.sequence_tensor_parallel
                and dist_config.compute_dtype.torch == torch.bfloat16 and symmetric_memory_available(self._distributed.tensor_group, device)):
            from fast_llm_b200.parallel import fused_tp

            fused_tp.enable_lazy(self._distributed.tensor_group, device)

        # vocabulary-parallel loss statistics exchanged by the loss kernels themselves
        if ms.fused_collectives and dist_config.tensor_parallel > 1 and symmetric_memory_available(self._distributed.tensor_group, device):
            from fast_llm_b200.parallel import fused_ce

            fused_ce.enable(self._distributed.tensor_group, device)

        # sequence-data parallelism: key / value exchange through symmetric memory
        if (ms.fused_collectives and dist_config.sequence_data_parallel > 1 and dist_config.compute_dtype.torch == torch.bfloat16
                and symmetric_memory_available(self._distributed.sequence_data_group, device)):
            from fast_llm_b200.parallel import fused_sdp

            fused_sdp.enable(self._distributed.sequence_data_group, device)

        def carve(sizes_bytes: list[int], what: str):
            aligned = [(n + 255) // 256 * 256 for n in sizes_bytes]
            arena = SymmetricArena(sum(aligned), self._distributed.data_group, device)
            out, off = [], 0
            for n, a in zip(sizes_bytes, aligned):
                out.append(arena.buffer[off : off + n])
                off += a
            return arena, out

        if mode.support_forward:
            sizes = [0] * num_weight_buffers
            for k, (s, stage) in enumerate(local):
                sizes[k % num_weight_buffers] = max(sizes[k % num_weight_buffers], sum(f.buffer_size for f in stage.fsdps))
            wdtype = dist_config.compute_dtype.torch
            if use_symmetric:
                self._weight_arena, raw = carve([n * wdtype.itemsize for n in sizes], "weights")
                self._weight_buffers = [b.view(wdtype) for b in raw]
            else:
                self._weight_buffers = [allocator(n, wdtype, f"weight_buffer_{i}") for i, n in enumerate(sizes)]
        if mode.support_backward:
            sizes = [0] * num_grad_buffers
            for k, (s, stage) in enumerate(local):
                nbytes = sum(f.grad_buffer_size * f.grad_buffer_dtype.itemsize for f in stage.fsdps)
                sizes[k % num_grad_buffers] = max(sizes[k % num_grad_buffers], nbytes)
            if use_symmetric:
                self._grad_arena, self._grad_buffers = carve(sizes, "grads")
            else:
                self._grad_buffers = [allocator(n, torch.uint8, f"grad_buffer_{i}") for i, n in enumerate(sizes)]
            for b in self._grad_buffers:
                b.zero_()
        self._buffer_registry = {}

        shard_offset, grad_offset = 0, 0
        self._stage_shard_ranges = {}
        for k, (s, stage) in enumerate(local):
            weight_shards, grad_shards, wbufs, gbufs = [], [], [], []
            wb_off, gb_off = 0, 0
            wi, gi = k % num_weight_buffers, k % num_grad_buffers
            for i, fsdp in enumerate(stage.fsdps):
                sl = slice(shard_offset, shard_offset + fsdp.shard_size)
                self._stage_shard_ranges[(s, i)] = sl
                weight_shards.append(self._shards[ShardName.weights][sl])
                shard_offset += fsdp.shard_size
                wbuf = gbuf = gshard = None
                if mode.support_forward:
                    wbuf = self._weight_buffers[wi][wb_off : wb_off + fsdp.buffer_size]
                    wb_off += fsdp.buffer_size
                if mode.support_backward and fsdp.requires_grad:
                    nbytes = fsdp.grad_buffer_size * fsdp.grad_buffer_dtype.itemsize
                    gbuf = self._grad_buffers[gi][gb_off : gb_off + nbytes].view(fsdp.grad_buffer_dtype)
                    gb_off += nbytes
                    if dp1_alias:
                        gshard = gbuf
                    else:
                        gshard = self._shards[ShardName.grads][grad_offset : grad_offset + fsdp.grad_shard_size]
                    grad_offset += fsdp.grad_shard_size
                wbufs.append(wbuf)
                gbufs.append(gbuf)
                grad_shards.append(gshard)
            for fsdp in stage.fsdps:
                fsdp.set_symmetric_arenas(self._weight_arena, self._grad_arena)
            stage.setup(distributed=self._distributed, mode=mode, weight_shards=weight_shards, grad_shards=grad_shards,
                        weight_buffers=wbufs, grad_buffers=gbufs, buffer_registry=self._buffer_registry,
                        weight_buffer_index=wi if num_weight_buffers < len(local) else ("own", s),
                        grad_buffer_index=gi if num_grad_buffers < len(local) else ("own", s))
        self._num_weight_buffers, self._num_grad_buffers = num_weight_buffers, num_grad_buffers
        # The fused gradient reduction leaves per-block sums of squares of every reduced shard: when each of them counts in
        # full towards this rank's share of the global norm, one launch over this buffer replaces a norm pass per stage.
        self._grad_norm_partials = None
        if mode.support_backward and self._grad_arena is not None:
            from fast_llm_b200.ops import _lib

            fsdps = [f for _, stage in local for f in stage.fsdps if f.requires_grad]
            tensor_rank = dist_config.tensor_rank
            counted_in_full = all(f.get_parameter_meta(n).is_tensor_parallel or tensor_rank == 0 for f in fsdps for n in f.parameter_names)
            if fsdps and counted_in_full:
                blocks = _lib.get_lib().flb_rs_reduce_blocks()
                self._grad_norm_partials = torch.zeros(len(fsdps) * blocks, dtype=torch.float32, device=device)
                for i, f in enumerate(fsdps):
                    f.norm_partials = self._grad_norm_partials[i * blocks : (i + 1) * blocks]
        # tied duplicates alias their owner's tensors
        if mode.support_forward:
            for owner, dup, _, _ in self._tied_duplicates.values():
                dup.tensor = owner.tensor
        for layer in self._layers:
            if not layer._is_setup:
                layer.setup(self._distributed)
        if self._verbose and dist_config.rank == 0:
            n_params = sum(stage.parameter_count for stage in self._stages)
            logger.info(f"Model: {self._num_stages} stages, {n_params:,} parameters (per tensor rank), "
                        f"{len(local)} stages on this rank, shard {total:,} elements, "
                        f"{num_weight_buffers} weight / {num_grad_buffers} grad buffers, mode {mode.value}")

    @property
    def weight_arena(self):
        """Symmetric-memory arena holding every weight buffer (None when the fused ZeRO path is off)."""
        return getattr(self, "_weight_arena", None)

    @property
    def grad_arena(self):
        return getattr(self, "_grad_arena", None)

    @property
    def shards(self) -> dict[str, torch.Tensor]:
        return self._shards

    @property
    def grad_shard_is_buffer(self) -> bool:
        return self._grad_shard_is_buffer

    def get_shard(self, name: str) -> torch.Tensor:
        return self._shards[name]

    def get_stage_shards(self, shard_name: str, stage_index: int) -> list[torch.Tensor]:
        stage = self._stages[stage_index]
        return [self._shards[shard_name][self._stage_shard_ranges[(stage_index, i)]] for i in range(len(stage.fsdps))]

    def get_param_groups(self) -> list[dict]:
        groups = []
        for s, stage in self._stages_on_device.items():
            state = {name: self.get_stage_shards(name, s) for name in self._state_shard_names[1:]}
            groups += stage.get_param_groups(state)
        return groups

    @property
    def grad_norm_partials(self) -> "torch.Tensor | None":
        """Per-block sums of squares of all reduced gradient shards of this rank (written by the fused reduction), or None
        when the norm has to be computed from `get_grad_norm_slices`."""
        return getattr(self, "_grad_norm_partials", None)

    def get_grad_norm_slices(self) -> list[torch.Tensor]:
        return [sl for stage in self._stages_on_device.values() for sl in stage.get_grad_norm_slices()]

    def initialize_weights(self) -> None:
        for stage in self._stages_on_device.values():
            stage.initialize_weights()
        self.synchronize_tied_weights()

    # ---- tied parameters held by two pipeline ranks
    @property
    def tied_remote_stages(self) -> set[int]:
        """Stages on this rank whose gradient reduction must wait for the exchange with the other holder."""
        pp_rank, pp = self._config.distributed.pipeline_rank, self._config.distributed.pipeline_parallel
        return {s for _, _, a, b in self._tied_remote for s in (a, b) if s % pp == pp_rank and s in self._stages_on_device}

    def _pipeline_peer(self, stage_index: int) -> int:
        """Rank, inside the pipeline group, of the holder of `stage_index`."""
        return stage_index % self._config.distributed.pipeline_parallel

    def _export_parameter(self, name: str, shard_name: str = "weights") -> torch.Tensor:
        s = self._parameter_stages[name]
        stage = self._stages_on_device[s]
        for i, fsdp in enumerate(stage.fsdps):
            if name in fsdp.parameter_names:
                shard = self._shards[shard_name][self._stage_shard_ranges[(s, i)]]
                for got, tensor in fsdp.export_shard(shard):
                    if got == name:
                        return fsdp.get_parameter_meta(name).local_to_global(tensor)
        raise KeyError(name)

    def synchronize_tied_weights(self) -> None:
        """Send the owner's weights to the copies on other pipeline ranks (after initialisation or loading)."""
        from fast_llm_b200.parallel.collectives import recv, send

        pp_rank, pp = self._config.distributed.pipeline_rank, self._config.distributed.pipeline_parallel
        group = self._distributed.pipeline_group
        for owner, dup, owner_stage, dup_stage in self._tied_remote:
            if owner_stage % pp == pp_rank and owner_stage in self._stages_on_device:
                value = self._export_parameter(owner.tensor_name).float().contiguous()
                send(value, self._pipeline_peer(dup_stage), group)
            elif dup_stage % pp == pp_rank and dup_stage in self._stages_on_device:
                value = torch.empty(dup.global_shape, dtype=torch.float32, device=self._distributed.device)
                recv(value, self._pipeline_peer(owner_stage), group)
                self.import_state_tensor(dup.tensor_name, "weights", value)
                self._stages_on_device[dup_stage].invalidate_buffer()

    def exchange_tied_gradients(self) -> None:
        """Both holders of a tied parameter end up with the sum of their gradient buffers (before the data reduction)."""
        from fast_llm_b200.parallel.collectives import recv, send

        pp_rank, pp = self._config.distributed.pipeline_rank, self._config.distributed.pipeline_parallel
        group = self._distributed.pipeline_group
        for owner, dup, owner_stage, dup_stage in self._tied_remote:
            mine, other_stage = (owner, dup_stage) if owner_stage % pp == pp_rank else (dup, owner_stage)
            if not ((owner_stage % pp == pp_rank and owner_stage in self._stages_on_device) or (dup_stage % pp == pp_rank and dup_stage in self._stages_on_device)):
                continue
            param = mine.tensor
            grad = param.grad_buffer
            if getattr(param, "param_grad_is_zero", False):
                grad.zero_()
                param.param_grad_is_zero = False
            peer = self._pipeline_peer(other_stage)
            theirs = torch.empty_like(grad)
            local = grad.contiguous()
            # the lower pipeline rank sends first: a fixed order avoids both sides blocking in a send
            if pp_rank < other_stage % pp:
                send(local, peer, group)
                recv(theirs, peer, group)
            else:
                recv(theirs, peer, group)
                send(local, peer, group)
            grad.add_(theirs)

    def invalidate_buffers(self) -> None:
        for stage in self._stages_on_device.values():
            stage.invalidate_buffer()

    def train(self, mode: bool = True):
        self._training = mode
        return self

    # ---- state tensors (checkpoint import / export)
    def get_state_tensor_iterator(self, shard_names: tuple[str, ...], data_type=None):
        """Yield (parameter name, shard name, GLOBAL tensor) for every parameter on this pipeline rank."""
        for shard_name in shard_names:
            for s, stage in self._stages_on_device.items():
                for i, fsdp in enumerate(stage.fsdps):
                    shard = self._shards[shard_name][self._stage_shard_ranges[(s, i)]]
                    for name, tensor in fsdp.export_shard(shard):
                        meta = fsdp.get_parameter_meta(name)
                        tensor = meta.local_to_global(tensor)
                        if data_type is not None:
                            tensor = tensor.to(data_type)
                        yield name, shard_name, tensor

    def import_state_tensor(self, parameter_name: str, shard_name: str, tensor: torch.Tensor) -> int:
        """Load a GLOBAL tensor into this rank's shard; returns the number of elements written."""
        s = self._parameter_stages[parameter_name]
        if s not in self._stages_on_device:
            return 0
        stage = self._stages[s]
        for i, fsdp in enumerate(stage.fsdps):
            if parameter_name in fsdp:
                meta = fsdp.get_parameter_meta(parameter_name)
                local = meta.global_to_local(tensor.to(self._shards[shard_name].device))
                shard = self._shards[shard_name][self._stage_shard_ranges[(s, i)]]
                return fsdp.import_state_tensor(parameter_name, shard, local)
        raise KeyError(parameter_name)

    def iter_fsdps(self):
        for s, stage in self._stages_on_device.items():
            for i, fsdp in enumerate(stage.fsdps):
                yield s, i, fsdp, self._stage_shard_ranges[(s, i)]
