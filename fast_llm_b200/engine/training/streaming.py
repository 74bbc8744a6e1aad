"""Trainer callback for online RL: after every successful update, announce the step on a Redis stream and broadcast the
exported weights to external inference workers over a dedicated process group (trainer rank 0 + the workers).

Protocol per step (rank 0): `xadd` {"type": "weights_ready", "step", "documents_seen"}; then for every exported tensor a
metadata object `(shard, name, shape, dtype)` followed by the tensor, and `None` to close.  All trainer ranks walk the
export iterator (it contains collectives); only rank 0 talks to the workers.  `train_end` posts "training_finished".
Parity: `fast_llm/engine/training/streaming.py:24-140`, `fast_llm/engine/training/config.py` (StreamingTrainerCallbackConfig).
"""

import json
import logging
import time

import torch

logger = logging.getLogger(__name__)

REDIS_TRAINING_STREAM = "fast_llm_events"
REDIS_TRAINING_FIELD = "event"


class TrainerCallback:
    def run_begin(self, step: int) -> None:
        pass

    def step_end(self, step: int, reduced_losses: dict, update_successful: bool, train_metrics: dict | None, documents_seen: int = 0):
        return None

    def train_end(self, step: int) -> None:
        pass


class StreamingTrainerCallback(TrainerCallback):
    def __init__(self, config, model, client=None, process_group=None):
        self._config, self._model = config, model
        self._do_broadcast = model.config.distributed.rank == 0
        self._client = client
        self._process_group = process_group
        self._weight_sync_time_ms = None
        if self._do_broadcast:
            if self._client is None:
                self._client = config.get_client()
            if self._process_group is None and config.broadcast.external_world_size > 0:
                self._process_group = self._create_group()

    def _create_group(self):
        """A process group of its own (trainer rank 0 + the external workers, ranks 1..n), built straight on a TCP store so
        it neither needs nor disturbs the trainer's default group."""
        import datetime

        broadcast = self._config.broadcast
        world_size = broadcast.external_world_size + 1
        timeout = datetime.timedelta(seconds=self._config.timeout)
        store = torch.distributed.TCPStore(broadcast.host, broadcast.port, world_size, is_master=True, timeout=timeout, wait_for_workers=True)
        self._store = store
        if broadcast.backend.value == "nccl" and self._model.distributed.device.type == "cuda":
            return torch.distributed.ProcessGroupNCCL(store, 0, world_size, torch.distributed.ProcessGroupNCCL.Options())
        return torch.distributed.ProcessGroupGloo(store, 0, world_size, timeout)

    def run_begin(self, step: int) -> None:
        # workers start from the trainer's weights, whatever checkpoint it resumed from
        self._broadcast_weights(step, 0)

    def step_end(self, step, reduced_losses, update_successful, train_metrics, documents_seen: int = 0):
        if update_successful:
            self._broadcast_weights(step, documents_seen)
        return None if self._weight_sync_time_ms is None else {"weight_sync_time_ms": self._weight_sync_time_ms}

    def train_end(self, step: int) -> None:
        if self._do_broadcast:
            self._client.xadd(REDIS_TRAINING_STREAM, {REDIS_TRAINING_FIELD: json.dumps({"type": "training_finished"})})
        self._clear()

    def _clear(self) -> None:
        self._process_group = None
        self.__dict__.pop("_store", None)

    def _send_tensor(self, tensor: torch.Tensor) -> None:
        if self._process_group is not None:
            options = torch.distributed.BroadcastOptions()
            options.rootRank, options.rootTensor = 0, 0
            self._process_group.broadcast([tensor], options).wait()

    def _send_object(self, obj) -> None:
        """Length-prefixed pickle, the same framing `broadcast_object_list` uses."""
        if self._process_group is None:
            return
        import pickle

        device = self._model.distributed.device if self._model.distributed.device.type == "cuda" and "NCCL" in type(self._process_group).__name__ else "cpu"
        payload = torch.frombuffer(bytearray(pickle.dumps(obj)), dtype=torch.uint8).to(device)
        self._send_tensor(torch.tensor([payload.numel()], dtype=torch.int64, device=device))
        self._send_tensor(payload)

    def _broadcast_weights(self, step: int, documents_seen: int) -> None:
        if self._do_broadcast:
            self._client.xadd(REDIS_TRAINING_STREAM, {REDIS_TRAINING_FIELD: json.dumps(
                {"type": "weights_ready", "step": step, "documents_seen": documents_seen})})
        start = time.perf_counter()
        for shard_name, tensor_name, tensor in self._model.iter_exported_tensors(self._config.export):
            if self._do_broadcast:
                self._send_object((shard_name, tensor_name, tuple(tensor.shape), tensor.dtype))
                self._send_tensor(tensor.contiguous())
                self._on_tensor(shard_name, tensor_name, tensor)
        if self._do_broadcast:
            self._send_object(None)
            if self._model.distributed.device.type == "cuda":
                torch.cuda.synchronize()
            self._weight_sync_time_ms = (time.perf_counter() - start) * 1000

    def _on_tensor(self, shard_name: str, tensor_name: str, tensor: torch.Tensor) -> None:
        """Hook for tests and in-process consumers."""


def receive_object(process_group, device="cpu"):
    """Worker side of `_send_object` (rank > 0 of the broadcast group)."""
    import pickle

    options = torch.distributed.BroadcastOptions()
    options.rootRank, options.rootTensor = 0, 0
    size = torch.zeros(1, dtype=torch.int64, device=device)
    process_group.broadcast([size], options).wait()
    payload = torch.empty(int(size.item()), dtype=torch.uint8, device=device)
    process_group.broadcast([payload], options).wait()
    return pickle.loads(payload.cpu().numpy().tobytes())


def receive_weights(process_group, device="cpu"):
    """Worker side of one weight broadcast: yields (shard, name, tensor) until the closing `None`."""
    options = torch.distributed.BroadcastOptions()
    options.rootRank, options.rootTensor = 0, 0
    while True:
        header = receive_object(process_group, device)
        if header is None:
            return
        shard_name, tensor_name, shape, dtype = header
        tensor = torch.empty(shape, dtype=dtype, device=device)
        process_group.broadcast([tensor], options).wait()
        yield shard_name, tensor_name, tensor
