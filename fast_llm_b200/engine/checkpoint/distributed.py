"""The resumable `distributed` checkpoint format: `metadata.yaml` plus one `rank_{r}.safetensors` per process holding
that rank's flat shards (`weights_shard`, `exp_avgs_shard`, `exp_avgs_sq_shard`).

Loading into the layout that saved it is a straight copy.  Loading into ANY other layout (different data / tensor /
pipeline parallelism, ZeRO stage, stage split) goes rank file by rank file: a memory-less replica of the saved model is
built for each saved rank, and the overlap of every parameter's saved piece with this rank's piece is copied.
Parity: `fast_llm/engine/checkpoint/distributed.py:28-134`.
"""

import logging
import pathlib

import safetensors.torch
import torch
import yaml

from fast_llm_b200.engine.checkpoint.config import (
    CheckpointHandler,
    CheckpointLoadConfig,
    CheckpointLoadMetadataConfig,
    CheckpointSaveConfig,
    CheckpointSaveMetadataConfig,
    DistributedCheckpointFormat,
)
from fast_llm_b200.engine.checkpoint.safe_load import SafeLoad
from fast_llm_b200.engine.multi_stage.config import CheckpointMetadata, StageMode
from fast_llm_b200.parallel.collectives import broadcast_scalar
from fast_llm_b200.utils import Assert

logger = logging.getLogger(__name__)


class DistributedCheckpointHandler(CheckpointHandler):
    format = DistributedCheckpointFormat

    @classmethod
    def save_metadata(cls, config: CheckpointSaveMetadataConfig, metadata: CheckpointMetadata) -> None:
        config.path.mkdir(parents=True, exist_ok=True)
        (config.path / "metadata.yaml").write_text(yaml.safe_dump(_serialize_metadata(metadata), sort_keys=False))

    @classmethod
    def _load_metadata(cls, config: CheckpointLoadMetadataConfig) -> CheckpointMetadata:
        data = yaml.safe_load((pathlib.Path(config.path) / "metadata.yaml").read_text())
        return CheckpointMetadata.from_dict(data).validate()

    def save(self, config: CheckpointSaveConfig, metadata: CheckpointMetadata) -> None:
        dc = self._model.config.distributed
        if dc.rank == 0:
            self.save_metadata(config, metadata)
        pathlib.Path(config.path).mkdir(parents=True, exist_ok=True)
        tensors = {f"{name}_shard": self._model.get_shard(name).detach().cpu().contiguous() for name in metadata.shards}
        safetensors.torch.save_file(tensors, str(pathlib.Path(config.path) / f"rank_{dc.rank}.safetensors"), metadata={"format": "pt"})

    def load(self, config: CheckpointLoadConfig) -> dict | None:
        loaded_metadata = self._model.config.load_metadata(config.to_copy({"load_config": "fast_llm"}))
        shard_names = self.get_shard_names(config)
        for name in shard_names:
            Assert.incl(name, loaded_metadata.shards)
        loaded_config = loaded_metadata.config
        model = self._model
        dc = model.config.distributed
        same_layout = (
            _layout_dict(loaded_config.distributed) == _layout_dict(dc)
            and _stage_dict(loaded_config.multi_stage) == _stage_dict(model.config.multi_stage)
            and not _architecture_differs(loaded_config.base_model, model.config.base_model)
        )
        same_layout = bool(broadcast_scalar(int(same_layout), torch.int64, model.distributed.world_group, device=model.distributed.device))
        path = pathlib.Path(config.path)
        if same_layout:
            logger.info("Checkpoint layout matches: loading shards directly") if dc.rank == 0 else None
            with safetensors.safe_open(str(path / f"rank_{dc.rank}.safetensors"), framework="pt", device="cpu") as f:
                for name in shard_names:
                    saved = f.get_tensor(f"{name}_shard")
                    shard = model.get_shard(name)
                    Assert.eq(saved.numel(), shard.numel())
                    shard.copy_(saved)
        else:
            logger.info("Checkpoint layout differs: loading by shard overlap") if dc.rank == 0 else None
            loaded_config.base_model.compare_architecture(model.config.base_model, logger.warning)
            with SafeLoad(model, shard_names=shard_names, timeout=config.timeout) as context:
                saved_world = loaded_config.distributed.world_size
                for saved_rank in range(saved_world):
                    replica_config = loaded_config.to_copy({("distributed", "rank"): saved_rank, ("distributed", "world_size"): saved_world,
                                                            ("distributed", "local_world_size"): saved_world})
                    replica = type(model)(replica_config, optimizer_state_names=tuple(n for n in shard_names if n != "weights"), verbose=False)
                    replica_ranges = _replica_shard_ranges(replica)
                    file = path / f"rank_{saved_rank}.safetensors"
                    # only open files that can contain parameters we hold
                    local_names = {n for _, _, fsdp, _ in model.iter_fsdps() for n in fsdp.parameter_names}
                    if not any(n in fsdp for _, fsdp, _ in replica_ranges for n in local_names):
                        continue
                    with safetensors.safe_open(str(file), framework="pt", device="cpu") as f:
                        saved = {name: f.get_tensor(f"{name}_shard").to(model.distributed.device) for name in shard_names}
                    for _, _, fsdp, sl in model.iter_fsdps():
                        shards = {name: model.get_shard(name)[sl] for name in shard_names}
                        for _, loaded_fsdp, lsl in replica_ranges:
                            loaded_shards = {name: saved[name][lsl] for name in shard_names}
                            counts = fsdp.copy_shard_overlaps(loaded_fsdp, shards, loaded_shards,
                                                              skip_replicated=replica_config.distributed.tensor_rank != 0)
                            for pname, count in counts.items():
                                context.mark_as_loaded(count * len(shard_names), (pname, "all"))
        return loaded_metadata.metadata


def _replica_shard_ranges(replica):
    """(stage index, fsdp, slice of the rank's flat shard) for a model that was never given memory."""
    out, offset = [], 0
    for s, stage in replica.stages_on_device.items():
        for fsdp in stage.fsdps:
            out.append((s, fsdp, slice(offset, offset + fsdp.shard_size)))
            offset += fsdp.shard_size
    return out


def _layout_dict(dc) -> dict:
    return {k: getattr(dc, k) for k in ("world_size", "rank", "tensor_parallel", "pipeline_parallel", "sequence_data_parallel", "pipeline_first")} | {
        "sequence_tensor_parallel": dc.sequence_tensor_parallel}


def _stage_dict(ms) -> dict:
    return {"layers_per_stage": ms.layers_per_stage}


def _architecture_differs(a, b) -> bool:
    from fast_llm_b200.engine.base_model import architecture_dict

    return architecture_dict(a) != architecture_dict(b)


def _serialize_metadata(metadata: CheckpointMetadata) -> dict:
    from fast_llm_b200.config import FieldVerboseLevel

    out = metadata.to_dict(FieldVerboseLevel.explicit)
    out["fast_llm_version"] = str(metadata.fast_llm_version)
    out["model"] = metadata.model.model_name if isinstance(metadata.model, type) else metadata.model
    out["format"] = metadata.format.name if isinstance(metadata.format, type) else metadata.format
    out["config"] = metadata.config.to_dict(FieldVerboseLevel.explicit)
    # the layout that wrote the shards must be recoverable without the environment of the writer
    dist = out["config"].setdefault("distributed", {})
    dist["world_size"] = metadata.config.distributed.world_size
    # (the reference validates this section in the reading process, where a missing `local_world_size` defaults to that
    # process's environment and must still be a multiple of the writer's tensor-parallel size)
    dist["local_world_size"] = metadata.config.distributed.local_world_size
    dist.pop("rank", None)
    out["shards"] = list(metadata.shards)
    out["metadata"] = metadata.metadata
    out.pop("type", None)
    return out
