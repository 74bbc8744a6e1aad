"""Online-RL plumbing without a Redis server: stream documents in, announce and ship weights out; W&B wrapper."""

import json
import threading

import torch

from tests.common import build_trainer, tiny_trainer_config


class FakeRedis:
    """The few Redis stream calls the framework uses, in memory."""

    def __init__(self):
        self.streams: dict[str, list] = {}
        self.cursor: dict[str, int] = {}
        self.groups = set()

    def xadd(self, stream, fields):
        self.streams.setdefault(stream, []).append(({k: v for k, v in fields.items()}))
        return f"{len(self.streams[stream])}-0".encode()

    def xgroup_create(self, name, groupname, id="0", mkstream=False):
        if (name, groupname) in self.groups:
            raise RuntimeError("BUSYGROUP Consumer Group name already exists")
        self.groups.add((name, groupname))
        self.streams.setdefault(name, [])

    def xreadgroup(self, groupname, consumername, streams, count=1, block=0, noack=False):
        out = []
        for stream in streams:
            position = self.cursor.get(stream, 0)
            entries = self.streams.get(stream, [])[position : position + count]
            self.cursor[stream] = position + len(entries)
            if entries:
                out.append((stream.encode(), [(f"{position + i}-0".encode(), {k.encode(): v for k, v in e.items()}) for i, e in enumerate(entries)]))
        return out


def test_streaming_dataset_packs_documents_in_arrival_order():
    from fast_llm_b200.data.config import SamplingConfig, StreamingDatasetConfig
    from fast_llm_b200.data.streaming import REDIS_DATA_STREAM, RedisStreamingDataset, decode_document, encode_document

    client = FakeRedis()
    lengths = [5, 7, 4, 9, 3, 10]
    for i, n in enumerate(lengths):
        client.xadd(REDIS_DATA_STREAM, encode_document(list(range(i * 100, i * 100 + n)), old_log_probabilities=[-0.5] * n, advantage=float(i),
                                                       loss_masking_spans=[(0, 2)]))
    round_trip = decode_document({k.encode(): v for k, v in client.streams[REDIS_DATA_STREAM][1].items()})
    assert round_trip.tokens.tolist() == list(range(100, 107)) and round_trip.loss_masking_spans == [(0, 2)]
    assert round_trip.advantages.tolist() == [1.0] * 7 and round_trip.old_log_probabilities.tolist() == [-0.5] * 7
    sampling = SamplingConfig.from_dict({"micro_batch_size": 15, "predicted_tokens": 1, "num_samples": 2})
    dataset = RedisStreamingDataset(StreamingDatasetConfig.from_dict({"timeout": 0.1}), sampling, client=client)
    first, second = dataset[0], dataset[1]
    assert [len(d) for d in first] == [5, 7, 4]  # 16 tokens: exactly full
    assert [len(d) for d in second] == [9, 3]  # the 10-token document opens the third sample
    try:
        dataset[0]
        raise AssertionError("going back in a stream must fail")
    except IndexError:
        pass


def _shared_stream_rank(rank, world_size):
    """Two tensor-parallel ranks share every batch: only the first reads the stream (the other rank's client is empty and would
    time out), the documents reach the second by broadcast."""
    from fast_llm_b200.data.config import GPTDataConfig, SamplingConfig, StreamingDatasetConfig
    from fast_llm_b200.data.data import GPTData
    from fast_llm_b200.data.monitor import DatasetMonitor
    from fast_llm_b200.data.streaming import REDIS_DATA_STREAM, RedisStreamingDataset, encode_document
    from fast_llm_b200.parallel.distributed import Distributed
    from fast_llm_b200.parallel.topology import DistributedConfig

    config = DistributedConfig.from_dict({"world_size": world_size, "rank": rank, "local_world_size": world_size, "tensor_parallel": 2,
                                          "backend": "gloo", "use_cuda": False})
    config.validate()
    distributed = Distributed(config)
    client = FakeRedis()
    if rank == 0:
        for i, n in enumerate([5, 7, 4, 9, 3, 10, 6]):
            client.xadd(REDIS_DATA_STREAM, encode_document(list(range(i * 100, i * 100 + n))))
    data = GPTData(GPTDataConfig.from_dict({"datasets": {"training": {"type": "streaming", "timeout": 0.2}}, "micro_batch_size": 15}), config)
    data.setup(None, distributed)
    sampling = SamplingConfig.from_dict({"micro_batch_size": 15, "predicted_tokens": 1, "num_samples": 2}).validate()
    data._datasets["training"] = DatasetMonitor(RedisStreamingDataset(StreamingDatasetConfig.from_dict({"timeout": 0.2}), sampling, client=client), 1e9)
    data._sampling["training"], data._preprocessing["training"] = sampling, {}
    iterator = data.get_iterator("training", consumed_samples=0, num_workers=2, pin_memory=False)
    tokens = [next(iterator)[0].tokens.tolist() for _ in range(2)]
    distributed.shutdown()
    return tokens


def test_a_stream_is_read_once_per_model_replica():
    from tests.distributed_utils import run_distributed

    first, second = run_distributed(_shared_stream_rank, 2)
    assert first == second and len(first[0]) == 15
    assert first[0][:5] == [0, 1, 2, 3, 4] and first[1][:9] == list(range(300, 309))


def _receive(port, received):
    import datetime

    from fast_llm_b200.engine.training.streaming import receive_weights

    store = torch.distributed.TCPStore("127.0.0.1", port, 2, is_master=False, timeout=datetime.timedelta(seconds=60))
    group = torch.distributed.ProcessGroupGloo(store, 1, 2, datetime.timedelta(seconds=60))
    for _ in range(2):  # the initial broadcast and the one after the training step
        received.append({name: tensor.clone() for _, name, tensor in receive_weights(group)})


def test_streaming_callback_announces_and_broadcasts_weights():
    import socket

    from fast_llm_b200.engine.training.streaming import REDIS_TRAINING_FIELD, REDIS_TRAINING_STREAM, StreamingTrainerCallback

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    config = tiny_trainer_config({("callbacks", "stream"): {"type": "streaming", "broadcast": {"host": "127.0.0.1", "port": port, "backend": "gloo"},
                                                            "export": {"format": "llama"}}})
    received: list[dict] = []
    worker = threading.Thread(target=_receive, args=(port, received), daemon=True)
    worker.start()
    client = FakeRedis()
    import fast_llm_b200.engine.training.config as training_config

    original = training_config.StreamingTrainerCallbackConfig.get_callback
    training_config.StreamingTrainerCallbackConfig.get_callback = lambda self, model: StreamingTrainerCallback(self, model, client=client)
    try:
        trainer, _ = build_trainer(config)
        callback = trainer._callbacks["stream"]
        callback.run_begin(0)
        from tests.common import train_steps

        train_steps(trainer, 1)
        metrics = callback.step_end(1, {}, True, None, 128)
        callback.train_end(1)
    finally:
        training_config.StreamingTrainerCallbackConfig.get_callback = original
    worker.join(timeout=60)
    assert not worker.is_alive() and len(received) == 2
    events = [json.loads(e[REDIS_TRAINING_FIELD]) for e in client.streams[REDIS_TRAINING_STREAM]]
    assert [e["type"] for e in events] == ["weights_ready", "weights_ready", "training_finished"]
    assert events[1] == {"type": "weights_ready", "step": 1, "documents_seen": 128}
    assert "model.layers.0.self_attn.q_proj.weight" in received[0] and "lm_head.weight" in received[0]
    # the second broadcast carries the updated weights
    assert not torch.equal(received[0]["model.layers.0.mlp.down_proj.weight"], received[1]["model.layers.0.mlp.down_proj.weight"])
    assert metrics["weight_sync_time_ms"] > 0


class FakeWandbModule:
    def __init__(self):
        self.calls = []

    def Settings(self, **kwargs):
        return kwargs

    def init(self, **kwargs):
        self.calls.append(("init", kwargs["project"], kwargs["entity"]))

    def log(self, metrics, step, commit):
        self.calls.append(("log", step, metrics))

    def alert(self, **kwargs):
        self.calls.append(("alert", kwargs["title"]))

    def finish(self, exit_code=0):
        self.calls.append(("finish", exit_code))


def test_wandb_wrapper_logs_on_main_rank_only():
    from fast_llm_b200.engine.training.config import WandbConfig
    from fast_llm_b200.engine.training.wandb import Wandb

    class Run:
        is_main_rank = True
        experiment_directory = None

    module = FakeWandbModule()
    config = WandbConfig.from_dict({"entity_name": "team", "project_name": "p", "alert": {"interval": 1}})
    config.validate()
    with Wandb(config, Run(), {"a": 1}, module=module) as wandb:
        wandb.log_metrics(3, {"train": {"loss": 1.5}})
    kinds = [c[0] for c in module.calls]
    assert kinds == ["init", "alert", "log", "alert", "finish"]
    assert module.calls[2] == ("log", 3, {"train/loss": 1.5})
    silent = FakeWandbModule()
    Run.is_main_rank = False
    with Wandb(config, Run(), {}, module=silent) as wandb:
        wandb.log_metrics(1, {"x": 1})
    assert silent.calls == []
