"""Failure detection and recovery, with every failure made on the host (no GPU is faulted, trapped or hung):
a bounded device wait that nothing satisfies, a rank that leaves between steps, a truncated checkpoint file, a data
loader that raises, SIGTERM during training.  Parity of intent: `fast_llm/engine/training/trainer.py:325-331`,
`fast_llm/utils.py:362-390`, `fast_llm/data/data/data_loader.py:63-72`."""

import os
import signal
import threading
import time

import pytest
import torch

from tests.common import build_trainer, tiny_trainer_config, train_steps
from tests.distributed_utils import run_distributed


# ---------------------------------------------------------------------------------------------------------------------
# error words -> trainer
def test_registered_failure_raises_once():
    from fast_llm_b200.utils import device_errors

    state = {"word": 101}

    def read():
        word, state["word"] = state["word"], 0
        return f"fake barrier timed out waiting for rank {word - 100}" if word else None

    device_errors.register_error_source("fake", read)
    try:
        with pytest.raises(device_errors.DeviceWaitError, match="rank 1"):
            device_errors.check_device_errors()
        device_errors.check_device_errors()  # the source cleared itself
    finally:
        device_errors.unregister_error_source("fake")


def test_trainer_raises_on_device_wait_failure(tmp_path):
    """A failed wait reported during step 2 stops training at the next logging point, before the checkpoint."""
    from fast_llm_b200.utils import device_errors

    config = tiny_trainer_config({("run", "experiment_dir"): str(tmp_path), ("training", "train_iters"): 4,
                                  ("training", "checkpoint", "interval"): 2, ("training", "logs", "interval"): 2})
    config.validate()
    from fast_llm_b200.parallel.distributed import Distributed

    distributed = Distributed(config.model.distributed)
    run = config.get_run(distributed)
    trainer = config.get_trainer_class()(config=config)
    calls = {"n": 0}

    def read():
        calls["n"] += 1
        return "injected: barrier timed out waiting for rank 1"

    try:
        with run:
            trainer.setup(distributed, run)
            device_errors.register_error_source("injected", read)
            with pytest.raises(device_errors.DeviceWaitError, match="injected"):
                trainer.run()
    finally:
        device_errors.unregister_error_source("injected")
    assert calls["n"] == 1
    assert trainer.completed_steps == 2
    assert not (tmp_path / "checkpoint" / "2" / "ok").exists()


def _rank_with_failure(rank, world_size):
    from fast_llm_b200.utils import device_errors

    torch.distributed.init_process_group("gloo", rank=rank, world_size=world_size)
    if rank == 1:
        device_errors.register_error_source("fake", lambda: "barrier timed out waiting for rank 0")
    try:
        device_errors.check_device_errors(torch.distributed.group.WORLD, torch.device("cpu"))
    except device_errors.DeviceWaitError as e:
        return str(e)
    return None


def test_failure_on_one_rank_raises_on_all():
    results = run_distributed(_rank_with_failure, 2)
    assert "reported by another rank" in results[0]
    assert "waiting for rank 0" in results[1]


# ---------------------------------------------------------------------------------------------------------------------
# a rank that leaves between steps
def _leaving_rank(rank, world_size):
    import datetime

    updates = {("model", "distributed", "world_size"): world_size, ("model", "distributed", "rank"): rank,
               ("model", "distributed", "local_world_size"): world_size, ("model", "distributed", "backend"): "gloo",
               ("model", "distributed", "timeout"): 5.0, ("schedule", "depth_first_micro_batches"): 1}
    trainer, distributed = build_trainer(tiny_trainer_config(updates))
    losses = train_steps(trainer, 1)
    if rank == 1:
        # leaves between steps: none of its collectives is in flight
        return "left", losses
    t0 = time.perf_counter()
    try:
        train_steps(trainer, 1, start=1)
    except Exception as e:  # noqa: BLE001 - the backend's error type varies
        return "error", (type(e).__name__, time.perf_counter() - t0)
    return "no error", None


def test_rank_leaving_between_steps_ends_the_others_with_an_error():
    results = run_distributed(_leaving_rank, 2, timeout=120)
    assert results[1][0] == "left"
    status, detail = results[0]
    assert status == "error", "the surviving rank must fail its next collective instead of waiting for ever"
    assert detail[1] < 60


# ---------------------------------------------------------------------------------------------------------------------
# truncated checkpoint file
def test_truncated_checkpoint_file_is_reported(tmp_path):
    config = tiny_trainer_config({("run", "experiment_dir"): str(tmp_path), ("training", "train_iters"): 2,
                                  ("training", "checkpoint", "interval"): 2})
    config.validate()
    from fast_llm_b200.parallel.distributed import Distributed

    distributed = Distributed(config.model.distributed)
    run = config.get_run(distributed)
    trainer = config.get_trainer_class()(config=config)
    with run:
        trainer.setup(distributed, run)
        trainer.run()
    path = tmp_path / "checkpoint" / "2" / "rank_0.safetensors"
    assert path.exists() and (tmp_path / "checkpoint" / "2" / "ok").exists()
    data = path.read_bytes()
    path.write_bytes(data[: len(data) // 2])
    config2 = tiny_trainer_config({("run", "experiment_dir"): str(tmp_path), ("training", "train_iters"): 4,
                                   ("training", "checkpoint", "interval"): 2})
    config2.validate()
    run2 = config2.get_run(distributed)
    trainer2 = config2.get_trainer_class()(config=config2)
    with run2:
        trainer2.setup(distributed, run2)
        with pytest.raises(Exception) as info:
            trainer2.run()
    assert "rank_0.safetensors" in str(info.value) or "safetensors" in type(info.value).__name__.lower() or "incomplete" in str(info.value).lower()
    assert trainer2.completed_steps == 0, "a corrupt checkpoint must not be half-loaded and trained on"


# ---------------------------------------------------------------------------------------------------------------------
# data loader that raises
class _DatasetError(RuntimeError):
    pass


@pytest.mark.parametrize("num_workers", [0, 2])
def test_data_loader_exception_reaches_the_training_loop(num_workers):
    config = tiny_trainer_config({("training", "train_iters"): 8, ("training", "num_workers"): num_workers})
    trainer, _ = build_trainer(config)
    data = trainer._data
    inner = data._load
    served = {"n": 0}

    def failing_load(name, index, pin):
        if index >= 3:
            raise _DatasetError(f"sample {index} is unreadable")
        served["n"] += 1
        return inner(name, index, pin)

    data._load = failing_load
    t0 = time.perf_counter()
    with pytest.raises(_DatasetError, match="sample 3"):
        train_steps(trainer, 8)
    assert time.perf_counter() - t0 < 60


# ---------------------------------------------------------------------------------------------------------------------
# SIGTERM -> checkpoint
def test_sigterm_saves_a_checkpoint_and_stops(tmp_path):
    config = tiny_trainer_config({("run", "experiment_dir"): str(tmp_path), ("training", "train_iters"): 100000,
                                  ("training", "checkpoint", "interval"): 50000, ("training", "logs", "interval"): 1000})
    config.validate()
    from fast_llm_b200.parallel.distributed import Distributed

    distributed = Distributed(config.model.distributed)
    run = config.get_run(distributed)
    trainer = config.get_trainer_class()(config=config)
    pid = os.getpid()

    def send():
        while trainer.completed_steps < 3:
            time.sleep(0.01)
        os.kill(pid, signal.SIGTERM)

    thread = threading.Thread(target=send, daemon=True)
    with run:
        trainer.setup(distributed, run)
        thread.start()
        trainer.run()
    thread.join(timeout=5)
    steps = trainer.completed_steps
    assert 3 <= steps < 100000
    assert (tmp_path / "checkpoint" / str(steps) / "ok").exists()
    # and the run resumes from there
    trainer2 = config.get_trainer_class()(config=config)
    run2 = config.get_run(distributed)
    with run2:
        trainer2.setup(distributed, run2)
        trainer2._prepare_training_state()
    assert trainer2.completed_steps == steps


# ---------------------------------------------------------------------------------------------------------------------
# the device side: a wait that nothing satisfies returns an error status (the context stays usable)
@pytest.mark.gpu
def test_barrier_wait_runs_out_and_reports_the_missing_peer():
    import ctypes

    from fast_llm_b200.ops import _lib
    from fast_llm_b200.parallel import symmetric

    lib = _lib.get_lib()
    device = torch.device("cuda", 0)
    # a group of two whose second member never arrives: both pads are local buffers and nothing writes the flag of "rank 1"
    pad_bytes = lib.flb_symm_signal_pad_bytes(8)
    pads = [torch.zeros(pad_bytes, dtype=torch.uint8, device=device) for _ in range(2)]
    pad_ptrs = (ctypes.c_void_p * 2)(*[p.data_ptr() for p in pads])
    err = torch.zeros(1, dtype=torch.int32, device=device)
    old = symmetric.set_barrier_limit_seconds(0.002)
    try:
        t0 = time.perf_counter()
        _lib.check(lib.flb_symm_barrier(pad_ptrs, 0, 2, 0, 1, err.data_ptr(), _lib.stream_ptr()), "flb_symm_barrier")
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        symmetric.set_barrier_limit_seconds(old)
    assert err.item() == 101, "error word = 100 + the rank that did not arrive"
    assert elapsed < 2.0
    # kernels that follow a failed barrier leave memory untouched
    shard = 1024
    grads = torch.ones(2 * shard, dtype=torch.float32, device=device)
    out = torch.full((shard,), 7.0, dtype=torch.float32, device=device)
    ptrs = (ctypes.c_void_p * 2)(grads.data_ptr(), grads.data_ptr())
    _lib.check(lib.flb_rs_reduce(ptrs, 0, 0, 2, shard, 0.5, out.data_ptr(), 0, None, err.data_ptr(), _lib.stream_ptr()), "flb_rs_reduce")
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)
    err.zero_()
    _lib.check(lib.flb_rs_reduce(ptrs, 0, 0, 2, shard, 0.5, out.data_ptr(), 0, None, err.data_ptr(), _lib.stream_ptr()), "flb_rs_reduce")
    torch.cuda.synchronize()
    assert torch.all(out == 1.0)
    # the context is still usable
    assert torch.ones(4, device=device).sum().item() == 4
